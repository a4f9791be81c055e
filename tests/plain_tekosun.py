"""A plain, slow restatement of the Tekosun architecture in float64 torch on the CPU: one function per mechanism,
token by token where the design is a recurrence, no cache, no batching.  It shares no code with the engine; the
tests compare the engine's parts and whole models with it.  ``w`` maps tensor names to float64 tensors; ``m`` is a
mixer's entry of config.json with absent keys filled in by :func:`fill_attention`."""
from __future__ import annotations

import math

import torch

F = torch.float64
ROUND = [None]      # a type whose rounding every matrix product's input and result take (a model of a 16-bit engine's error), or None


def lin(x, weight):
    """weight [out, in] applied to the rows of x; with ROUND set, x and the result are rounded to that type."""
    if ROUND[0] is None:
        return x @ weight.T
    return (x.to(ROUND[0]).to(F) @ weight.T).to(ROUND[0]).to(F)


def rnd(x):
    """What a 16-bit engine keeps in its cache or hands from one kernel to the next, rounded likewise."""
    return x if ROUND[0] is None else x.to(ROUND[0]).to(F)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 40.0, x, torch.log1p(torch.exp(torch.clamp(x, max=40.0))))


# ------------------------------------------------------------------ the state-space mixer
def causal_conv(u, weight, bias, tail=None):
    """u [T, C]; weight [C, taps], its last column the current token's; zeros (or ``tail``, the taps - 1 inputs
    before u) ahead.  Returns (y [T, C], the new tail)."""
    taps = weight.shape[1]
    before = torch.zeros(taps - 1, u.shape[1], dtype=F) if tail is None else tail
    full = torch.cat([before, u])
    y = torch.stack([sum(full[t + j] * weight[:, j] for j in range(taps)) for t in range(u.shape[0])]) + bias
    return y, full[full.shape[0] - (taps - 1):]


def ssm_scan(x, b, c, dt, a_log, d_skip, state=None):
    """x [T, H, P], b and c [T, G, N], dt [T, H] (already positive).  Returns (y [T, H, P], state [H, N, P])."""
    t_len, heads, p = x.shape
    groups, n = b.shape[1], b.shape[2]
    s = torch.zeros(heads, n, p, dtype=F) if state is None else state.clone()
    ys = torch.zeros(t_len, heads, p, dtype=F)
    for t in range(t_len):
        for h in range(heads):
            g = h // (heads // groups)
            s[h] = math.exp(-math.exp(float(a_log[h])) * float(dt[t, h])) * s[h] + dt[t, h] * torch.outer(b[t, g], x[t, h])
            ys[t, h] = s[h].T @ c[t, g] + d_skip[h] * x[t, h]
    return ys, s


def mamba2(hid, w, p, m, eps, carry=None):
    """carry = (conv tail, state) of the tokens before ``hid`` or None.  Returns (out [T, width], carry)."""
    t_len = hid.shape[0]
    heads, pdim, n, groups = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner = heads * pdim
    proj = lin(hid, w[p + ".in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
    y, tail = causal_conv(xbc, w[p + ".conv"], w[p + ".conv.b"], carry[0] if carry else None)
    y = rnd(silu(y))
    x = y[:, :inner].reshape(t_len, heads, pdim)
    b = y[:, inner:inner + groups * n].reshape(t_len, groups, n)
    c = y[:, inner + groups * n:].reshape(t_len, groups, n)
    dt = softplus(dt + w[p + ".dt_bias"])
    ys, state = ssm_scan(x, b, c, dt, w[p + ".A_log"], w[p + ".D"], carry[1] if carry else None)
    gated = ys.reshape(t_len, inner) * silu(z)
    parts = m.get("norm_groups", 1)
    normed = unit_rms(gated.reshape(t_len, parts, inner // parts), eps).reshape(t_len, inner) * w[p + ".norm"]
    return lin(normed, w[p + ".o"]), (tail, state)


# ------------------------------------------------------------------ the generalized delta rule
def delta_scan(r, k, v, decay, rate, state=None):
    """r, k, decay, rate [T, H, D], v [T, H, E].  Returns (o [T, H, E], state [H, D, E])."""
    t_len, heads, d = k.shape
    s = torch.zeros(heads, d, v.shape[2], dtype=F) if state is None else state.clone()
    out = torch.zeros(t_len, heads, v.shape[2], dtype=F)
    for t in range(t_len):
        for h in range(heads):
            u = k[t, h] / torch.sqrt((k[t, h] ** 2).sum() + 1e-6)
            old = s[h]
            s[h] = decay[t, h][:, None] * old - torch.outer(rate[t, h] * u, u @ old) + torch.outer(k[t, h], v[t, h])
            out[t, h] = s[h].T @ r[t, h]
    return out, s


def general_delta(hid, w, p, m, eps, carry=None):
    t_len, heads, d = hid.shape[0], m["heads"], m["dim"]
    split = lambda y: y.reshape(t_len, heads, d)
    r, k, v = (split(lin(hid, w[f"{p}.{x}"])) for x in ("r", "k", "v"))
    inner = lin(torch.tanh(lin(hid, w[p + ".w1"])), w[p + ".w2"]) + w[p + ".w0"]
    decay = split(torch.exp(-math.exp(-0.5) * torch.sigmoid(inner)))
    rate = split(torch.sigmoid(lin(hid, w[p + ".a"]) + w[p + ".a.b"]))
    o, state = delta_scan(r, k, v, decay, rate, carry)
    o = unit_rms(o, eps).reshape(t_len, heads * d) * w[p + ".norm"] * torch.sigmoid(lin(hid, w[p + ".g"]))
    return lin(o, w[p + ".o"]), state


# ------------------------------------------------------------------ attention
def fill_attention(m):
    m = dict(m)
    m.setdefault("kv_heads", m["heads"])
    m.setdefault("vdim", m["dim"])
    m.setdefault("scale", m["dim"] ** -0.5)
    return m


def frequencies(rot):
    dims = rot["dims"]
    out = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        sc = rot.get("scaling")
        if sc:
            length = 2.0 * math.pi / f
            if length > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif length >= sc["original"] / sc["high"]:
                s = (sc["original"] / length - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims of every head rotate, dimension i paired with i + dims / 2."""
    if not rot or not rot.get("dims"):
        return x
    half = rot["dims"] // 2
    ang = positions.to(F)[:, None] * frequencies(rot)[None]
    cs, sn = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * cs - b * sn, b * cs + a * sn, x[..., 2 * half:]], -1)


def visible(n_q, first_q, window):
    """[n_q, first_q + n_q] booleans: which keys each query (at positions first_q ...) sees."""
    i = torch.arange(first_q, first_q + n_q)[:, None]
    j = torch.arange(first_q + n_q)[None]
    see = j <= i
    if window:
        see = see & (i - j < window)
    return see


def attention(hid, w, p, m, eps, shared, mode):
    """Whole sequences only (no carry).  ``mode`` None, "first" or "blend"; ``shared`` carries the first layer's values."""
    m = fill_attention(m)
    t_len, heads, kvh, d, vd = hid.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(lin(hid, w[p + ".q"]), w[p + ".q.norm"], eps).reshape(t_len, heads, d)
    k = rms_norm(lin(hid, w[p + ".k"]), w[p + ".k.norm"], eps).reshape(t_len, kvh, d)
    pos = torch.arange(t_len)
    q, k = rnd(rotate(q, pos, m.get("rot"))), rnd(rotate(k, pos, m.get("rot")))
    v = unit_rms(lin(hid, w[p + ".v"]).reshape(t_len, kvh, vd), eps)
    if mode == "first":
        shared["v_first"] = v
    elif mode == "blend":
        lam = w[p + ".vmix"]
        v = (1.0 - lam) * v + lam * shared["v_first"]
    v = rnd(v)
    see = visible(t_len, 0, (m.get("mask") or {}).get("size"))
    out = torch.zeros(t_len, heads, vd, dtype=F)
    for h in range(heads):
        g = h // (heads // kvh)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~see, float("-inf"))
        out[:, h] = rnd(torch.softmax(s, -1)) @ v[:, g]
    return lin(out.reshape(t_len, heads * vd), w[p + ".o"])


# ------------------------------------------------------------------ the feed-forward
def route(logits, top, scale):
    """(ids, weights): the ``top`` largest softmax scores over all experts (lowest index first among equals), the
    chosen scores divided by their sum, times ``scale``."""
    s = torch.softmax(logits, -1)
    ids = torch.argsort(-s, dim=-1, stable=True)[:, :top]
    val = torch.gather(s, 1, ids)
    return ids, val / (val.sum(-1, keepdim=True) + 1e-20) * scale


def relu2_mlp(x, up, down):
    return lin(torch.relu(lin(x, up)) ** 2, down)


def moe(hid, w, p, f):
    r = f["router"]
    ids, wts = route(hid @ w[p + ".router"].T, r["top"], r.get("scale", 1.0))
    out = torch.zeros_like(hid)
    for t in range(hid.shape[0]):
        for j in range(r["top"]):
            e = int(ids[t, j])
            out[t] += wts[t, j] * relu2_mlp(hid[t:t + 1], w[f"{p}.e{e}.up"], w[f"{p}.e{e}.down"])[0]
    if f.get("shared"):
        out = out + relu2_mlp(hid, w[p + ".shared.up"], w[p + ".shared.down"])
    return out


# ------------------------------------------------------------------ the model
def forward(cfg, w, tokens, streams=None):
    """float64 logits [T, vocab] for one whole sequence; ``streams`` (a list) receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens))] * (cfg.get("embedding") or {}).get("scale", 1.0)
    shared, mixing = {}, False
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix", layer["mixer"]
        if layer["type"] == "mamba2":
            y, _ = mamba2(x, w, p, m, eps)
        elif layer["type"] == "general_delta":
            y, _ = general_delta(x, w, p, m, eps)
        else:
            mode = None
            if m.get("v_mix"):
                mode, mixing = ("blend" if mixing else "first"), True
            y = attention(x, w, p, m, eps, shared, mode)
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp"):
            x = x + rms_norm(moe(x, w, f"l{i}.mlp", layer["mlp"]), w[f"l{i}.norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return lin(rms_norm(x, w["final.norm"], eps), w["head"])
