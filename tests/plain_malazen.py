"""The Malazen architecture restated from its equations: float64, no paging, no slots, no kernels, one function
per mechanism.  It shares no code with the engine; the tests hold the engine against it.

Notation: ``x`` the stream ``[T, D]``, weights ``[out, in]`` applied as ``W v``, positions from 0.  Functions that
carry something from one portion of a sequence to the next take and return it (``state``), so the tests can also
cut a sequence and hand it over.  ``w`` is the dictionary of a model's tensors by name (float64).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
#: None, or a type to which every matrix product's input and result, what is cached and what is activated are
#: rounded: that run is the model of what rounding alone does to the logits.
ROUND = [None]


def _r(v):
    return v if ROUND[0] is None else v.to(ROUND[0]).to(F64)


def group_norm(v, weight, eps, groups):
    """The row is cut into ``groups`` equal consecutive parts; each is divided by its own sqrt(mean(part^2) + eps);
    the whole is multiplied by ``weight``."""
    t, d = v.shape
    parts = v.reshape(t, groups, d // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(t, d) * weight


def linear(v, w, name):
    """``W v`` plus the bias ``<name>.b`` if the model has one."""
    y = _r(v) @ w[name].T
    return _r(y + w[name + ".b"] if name + ".b" in w else y)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1.0) / every) + 1.0)


def biased_attention(h, w, name, m, positions=None):
    """Grouped-query attention over every earlier position without rotation: the query grows with its position,
    and a score loses ``r1_h * ln(1 + r2_h * distance)``."""
    t = h.shape[0]
    nh, d = m["heads"], m["dim"]
    nkv, vd, scale = m.get("kv_heads") or nh, m.get("vdim") or d, m.get("scale") or d ** -0.5
    pos = torch.arange(t) if positions is None else positions
    q = linear(h, w, name + ".q").reshape(t, nh, d)
    if m.get("q_temp"):
        q = q * query_temperature(pos, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    k = linear(h, w, name + ".k").reshape(t, nkv, d)
    v = linear(h, w, name + ".v").reshape(t, nkv, vd)
    dist = (pos[:, None] - pos[None, :]).to(F64)
    seen = dist >= 0
    out = torch.zeros((t, nh, vd), dtype=F64)
    for head in range(nh):
        kv = head // (nh // nkv)
        s = (q[:, head] @ k[:, kv].T) * scale
        s = s - w[name + ".r1"][head] * torch.log(1.0 + w[name + ".r2"][head] * dist.clamp(min=0.0))
        s = s.masked_fill(~seen, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, kv]
    return linear(out.reshape(t, nh * vd), w, name + ".o")


def channel_decay(h, w, name, m):
    """alpha = sigmoid(z)^(1 / tau), z = W_a2 (W_a1 h) + b: one number per head and key channel."""
    z = linear(h, w, name + ".a1") @ w[name + ".a2"].T + w[name + ".a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"])


def gated_linear_attention(h, w, name, m, eps, state=None):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T and o_t = S_t^T q_t per head, token by token; every head's o divided
    by its root mean square and multiplied by ``.norm``; heads side by side times silu(W_g h); W_o.
    Returns (result, the state after the last token)."""
    t = h.shape[0]
    nh, d = m["heads"], m["dim"]
    vd = m.get("vdim") or d
    q = linear(h, w, name + ".q").reshape(t, nh, d) * d ** -0.5
    k = linear(h, w, name + ".k").reshape(t, nh, d)
    v = linear(h, w, name + ".v").reshape(t, nh, vd)
    alpha = channel_decay(h, w, name, m).reshape(t, nh, d)
    s = torch.zeros((nh, d, vd), dtype=F64) if state is None else state.clone()
    o = torch.zeros((t, nh, vd), dtype=F64)
    for i in range(t):
        s = alpha[i][:, :, None] * s + k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hdv,hd->hv", s, q[i])
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * w[name + ".norm"]
    g = linear(h, w, name + ".g")
    return linear(o.reshape(t, nh * vd) * g * torch.sigmoid(g), w, name + ".o"), s


def parallel_mixer(h, w, name, m, eps, state=None):
    left = biased_attention(h, w, name + ".left", m["left"])
    right, state = gated_linear_attention(h, w, name + ".right", m["right"], eps, state)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right, state


def rotary_frequencies(rot):
    """(f_i for i < dims/2, the factor on cos and sin), stretched where the scaling says so."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    where = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_pairs(x, positions, rot):
    """x ``[T, ..., dims]``: neighbours (2i, 2i+1) turn by position * f_i."""
    f, mag = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [f.shape[0]]
    c, s = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
    a, b = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2], out[..., 1::2] = a * c - b * s, b * c + a * s
    return out


def latent_attention(h, w, name, m, eps, positions=None):
    """Keys and values of every head from one normed latent per token; one rotated key part for all heads; a
    window; a sink in the softmax's denominator."""
    t = h.shape[0]
    nh, d, rd, vd, r = m["heads"], m["dim"], m.get("rot_dim") or 0, m["vdim"], m["kv_rank"]
    scale = m.get("scale") or (d + rd) ** -0.5
    pos = torch.arange(t) if positions is None else positions
    q = linear(h, w, name + ".q").reshape(t, nh, d + rd)
    q_plain, q_rot = q[..., :d], (rotate_pairs(q[..., d:], pos, m["rot"]) if rd else q[..., d:])
    down = linear(h, w, name + ".dkv")
    c = down[:, :r]
    c = _r(c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * w[name + ".dkv.norm"])
    k_rot = _r(rotate_pairs(down[:, r:], pos, m["rot"])) if rd else down[:, r:]
    k_plain = linear(c, w, name + ".uk").reshape(t, nh, d)
    v = linear(c, w, name + ".uv").reshape(t, nh, vd)
    dist = pos[:, None] - pos[None, :]
    seen = (dist >= 0) & (dist < m["mask"]["size"]) if m.get("mask") else dist >= 0
    out = torch.zeros((t, nh, vd), dtype=F64)
    for head in range(nh):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * scale
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, w[name + ".sink"][head])
        e = torch.exp(s - top)
        out[:, head] = (e / (e.sum(-1, keepdim=True) + torch.exp(w[name + ".sink"][head] - top))) @ v[:, head]
    return linear(out.reshape(t, nh * vd), w, name + ".o")


def clamped_glu(h, w, name, limit):
    g = linear(h, w, name + ".gate").clamp(max=limit)
    u = linear(h, w, name + ".up").clamp(-limit, limit)
    return linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), w, name + ".down")


def schedule(cfg):
    """[(layer, pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["times"] <= 1 or loop["stop"] <= loop["start"]:
        return [(i, 0) for i in range(n)]
    runs = [(i, 0) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, 0) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, collect=None):
    """Logits ``[T, vocab]`` of a whole sequence.  ``collect`` (a list) takes the stream after every layer run."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups") or 1
    x0 = w["embed"][torch.as_tensor(tokens)]
    x = x0.clone()
    loop = cfg.get("loop")
    for layer, t in schedule(cfg):
        if loop and t > 0 and layer == loop["start"]:
            x = x + x0
        spec, name = cfg["layers"][layer], f"l{layer}"
        h = group_norm(x, w[name + ".norm1"], eps, groups)
        if spec["type"] == "parallel":
            y, _ = parallel_mixer(h, w, name + ".mix", spec["mixer"], eps)
        elif spec["type"] == "latent_attention":
            y = latent_attention(h, w, name + ".mix", spec["mixer"], eps)
        else:
            raise ValueError(spec["type"])
        x = x + y
        if spec.get("mlp"):
            x = x + clamped_glu(group_norm(x, w[name + ".norm2"], eps, groups), w, name + ".mlp", spec["mlp"]["limit"])
        if collect is not None:
            collect.append(x.clone())
    return _r(group_norm(x, w["final.norm"], eps, groups)) @ w["embed"].T
