"""The Malazen architecture against its plain restatement (plain_malazen.py): every mechanism alone through its part
and kernels, then whole models of three tiny configurations that differ in every size, option and order of layers,
stepped whole, token by token, in portions down to two tokens, in mixed batches over a pool so small that pages and
state slots are used again, through bin/trace_run and through Engine.generate.  Weights are random; where random
weights would hide a fault the tests set keys and queries by hand so that one score stands out (a key hundreds of
tokens back under the distance's toll, the keys just inside and just outside a window, at page borders, the first
token), slow the decays so that a state lost far back would show, and move the sink until it takes half the weight."""
from __future__ import annotations

import copy
import math
import random

import numpy as np
import pytest
import torch

import plain_malazen as plain
from helpers import ML, TraceProcess, make_malazen_folder, malazen_tensors, random_tokens

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
PTOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
# Whole models.  float32: the largest difference as a fraction of the largest logit (5e-5, or three times what rounding
# the matrix products to float32 causes if that is more).  bfloat16: a position's root-mean-square error over the
# vocabulary as a fraction of the logits' root mean square, against three times what rounding alone causes there: the
# plain model run again with every matrix product's input and result and what is cached rounded to bfloat16.
MTOL = {torch.float32: 5e-5}
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}
gpu = pytest.mark.gpu


def _rel(got, want):
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def _row_err(got, want):
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return float(d.pow(2).mean(-1).sqrt().max() / (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt())


def _plain_logits(cfg, w, toks, dtype):
    """(the plain logits, the limit for an engine of ``dtype`` against them)."""
    want = plain.forward(cfg, w, toks)
    single = dtype in (torch.float32, "float32")
    plain.ROUND[0] = torch.float32 if single else torch.bfloat16
    try:
        rounded = plain.forward(cfg, w, toks)
    finally:
        plain.ROUND[0] = None
    return want, max(MTOL[torch.float32], 3.0 * _rel(rounded, want)) if single else 3.0 * _row_err(rounded, want)


def _model_err(got, want, dtype):
    return _rel(got, want) if dtype in (torch.float32, "float32") else _row_err(got, want)


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def _dense(y):
    from inferflux_b200.parts.base import PartialSums, ScaledSum
    if isinstance(y, ScaledSum):
        return sum(_dense(v) * f for v, f in y.terms)
    return y.tensor.sum(0) if isinstance(y, PartialSums) else y.float()


# ------------------------------------------------------------------ CPU: configuration, spec, cache plan, the plain code
def test_config_is_read_from_its_own_keys():
    from inferflux_b200.config import ConfigError, MalazenConfig, build_spec, load_config
    cfg = load_config(copy.deepcopy(ML["A"]))
    assert isinstance(cfg, MalazenConfig) and cfg.width == 64 and cfg.vocab_size == 300 and cfg.norm_eps == 1e-5
    assert cfg.norm_groups == 4 and [l.type for l in cfg.layers] == ["parallel", "latent_attention", "parallel"]
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (0, 2, 3)
    a = cfg.layers[0].mixer
    assert a["left"] == dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, q_temp=dict(coef=0.7, every=8))
    assert a["right"] == dict(heads=3, dim=12, vdim=20, tau=4.0) and (a["left_scale"], a["right_scale"]) == (0.8, 1.3)
    b = cfg.layers[1].mixer
    assert (b["heads"], b["dim"], b["rot_dim"], b["vdim"], b["kv_rank"], b["window"], b["scale"]) == (3, 8, 12, 20, 24, 20, 0.4)
    assert b["rot"]["scaling"] == dict(factor=4.0, original=64.0, fast=16.0, slow=2.0)
    assert cfg.layers[0].mlp == dict(kind="dense", ff=96, limit=2.0) and cfg.layers[2].mlp is None
    bare = load_config(copy.deepcopy(ML["B"]))                             # absent keys: their defaults
    assert bare.norm_groups == 1 and bare.loop_times == 0
    l, r = bare.layers[1].mixer["left"], bare.layers[3].mixer["right"]
    assert (l["kv_heads"], l["scale"]) == (3, 10 ** -0.5) and r["vdim"] == 10 and bare.layers[3].mixer["left"]["q_temp"] is None
    assert (bare.layers[1].mixer["left_scale"], bare.layers[1].mixer["right_scale"]) == (1.0, 1.0)
    c = bare.layers[2].mixer
    assert (c["rot_dim"], c["window"], c["rot"], c["scale"]) == (0, 0, None, 6 ** -0.5)
    assert load_config(cfg.to_dict()) == cfg and load_config(bare.to_dict()) == bare
    spec = build_spec(cfg)
    assert sorted(spec.positions) == ["rot0"] and [l.arrangement for l in spec.layers] == ["prenorm"] * 3 + ["junction"]
    assert [l.parts["mixer"].kind for l in spec.layers[:3]] == ["side_by_side", "latent_attention", "side_by_side"]
    assert [(r.layer, r.params.get("pass")) for r in spec.schedule] == [(0, 0), (1, 0), (3, 1), (0, 1), (1, 1), (3, 2), (0, 2), (1, 2), (2, None)]
    assert "feed_forward" not in spec.layers[2].parts and spec.lm_head.params["tied_to"] == "embed"
    once = build_spec(load_config(dict(copy.deepcopy(ML["A"]), loop=dict(start=1, stop=3, times=1))))
    assert [r.layer for r in once.schedule] == [0, 1, 2] and len(once.layers) == 3      # a loop that runs once is no loop
    for breaker, text in [(lambda d: d["layers"][0].update(type="serial"), "type"), (lambda d: d.pop("width"), "width"),
                          (lambda d: d["layers"][0]["mixer"]["left"].pop("dim"), "dim"),
                          (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
                          (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
                          (lambda d: d["layers"][0]["mixer"]["right"].update(tau=0.0), "tau"),
                          (lambda d: d["norm"].update(groups=5), "groups"), (lambda d: d["norm"].pop("eps"), "eps"),
                          (lambda d: d["loop"].update(stop=4), "loop"), (lambda d: d["layers"][0]["mlp"].pop("limit"), "limit"),
                          (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "kind")]:
        bad = copy.deepcopy(ML["A"])
        breaker(bad)
        with pytest.raises(ConfigError, match=text):
            load_config(bad)


def test_cache_and_state_plan():
    from inferflux_b200.config import build_spec, load_config
    from inferflux_b200.engine import Model
    model = Model(build_spec(load_config(copy.deepcopy(ML["A"]))), torch.float32, "cpu")
    specs = {w.name: w for w in model.weight_specs()}
    names = {n: tuple(w.shape) for n, w in specs.items() if w.kind != "ignored"}
    assert names["embed"] == (300, 64) and "head" not in names and names["final.norm"] == (64,)
    assert names["l0.mix.left.q"] == (64, 64) and names["l0.mix.left.k"] == (32, 64) and names["l0.mix.left.v"] == (48, 64)
    assert names["l0.mix.left.q.b"] == (64,) and names["l0.mix.left.o.b"] == (64,) and names["l0.mix.left.r1"] == (4,)
    assert names["l0.mix.left.o"] == (64, 96) and "l0.mix.left.g" not in names and "l0.mix.left.out" not in names
    assert names["l0.mix.right.q"] == (36, 64) and names["l0.mix.right.v"] == (60, 64) and names["l0.mix.right.norm"] == (20,)
    assert names["l0.mix.right.a1"] == (-1, 64) and names["l0.mix.right.a2"] == (36, -1) and names["l0.mix.right.a2.b"] == (36,)
    assert specs["l0.mix.right.a1"].fits((7, 64)) and not specs["l0.mix.right.a1"].fits((7, 65))     # the stored size stands
    assert names["l1.mix.q"] == (3 * 20, 64) and names["l1.mix.dkv"] == (36, 64) and names["l1.mix.dkv.norm"] == (24,)
    assert names["l1.mix.uk"] == (24, 24) and names["l1.mix.uv"] == (60, 24) and names["l1.mix.sink"] == (3,)
    assert names["l0.mlp.gate.b"] == (96,) and names["l0.mlp.down.b"] == (64,) and "l2.norm2" not in names
    needs = [[(s.name, s.heads, s.width) for s in n.streams] + [n.window] for n in model.kv_needs]
    assert needs == [[("k", 2, 16), ("v", 2, 24), None], [("latent", 1, 36), 20], [("k", 1, 32), ("v", 1, 32), None]]
    assert model.runs_per_group == [3, 3, 1]                                     # every pass of the loop has a cache of its own
    states = [{s.name: tuple(s.shape) for s in per_run} for per_run in model.state_needs]
    gla = {"gla": (3, 12, 20)}
    assert states == [gla, {}, {}, gla, {}, {}, gla, {}, {"gla": (1, 16, 8)}]
    b = Model(build_spec(load_config(copy.deepcopy(ML["B"]))), torch.float32, "cpu")
    assert [(n.streams[0].width, n.window) for n in b.kv_needs] == [(15, 7), (10, None), (13, None), (6, None)]


def test_plain_carry_over_and_closed_forms():
    """The plain implementation's own consistency: a sequence cut in two with the state handed over, the recurrence
    as a sum over earlier tokens, the temperature's steps, the toll at distance 0, the norm in one group, the window."""
    cfg = ML["A"]
    _, t = malazen_tensors(cfg, 3)
    w = {k: v.double() for k, v in t.items()}
    m, eps = cfg["layers"][0]["mixer"]["right"], cfg["norm"]["eps"]
    h = _rand((11, 64), 1).double()
    whole, s = plain.gated_linear_attention(h, w, "l0.mix.right", m, eps)
    a1, s1 = plain.gated_linear_attention(h[:4], w, "l0.mix.right", m, eps)
    a2, s2 = plain.gated_linear_attention(h[4:], w, "l0.mix.right", m, eps, s1)
    assert torch.allclose(torch.cat([a1, a2]), whole) and torch.allclose(s2, s)
    q = (h @ w["l0.mix.right.q"].T).reshape(11, 3, 12) * 12 ** -0.5
    k, v = (h @ w["l0.mix.right.k"].T).reshape(11, 3, 12), (h @ w["l0.mix.right.v"].T).reshape(11, 3, 20)
    alpha = plain.channel_decay(h, w, "l0.mix.right", m).reshape(11, 3, 12)
    assert float(alpha.min()) > 0.0 and float(alpha.max()) < 1.0
    z = (h @ w["l0.mix.right.a1"].T) @ w["l0.mix.right.a2"].T + w["l0.mix.right.a2.b"]
    assert torch.allclose(alpha.reshape(11, 36), torch.sigmoid(z) ** 0.25)
    direct = sum(((q[10, 1] * alpha[j + 1:, 1].prod(0)) @ k[j, 1]) * v[j, 1] for j in range(11))     # head 1 at the last token
    assert torch.allclose(s[1].T @ q[10, 1], direct)
    temp = plain.query_temperature(torch.tensor([0, 6, 7, 8, 15, 16, 23]), 0.7, 8)
    assert torch.allclose(temp, 1.0 + 0.7 * torch.log(torch.tensor([1.0, 1.0, 2.0, 2.0, 3.0, 3.0, 4.0], dtype=torch.float64)))
    x = _rand((5, 24), 2).double()
    one = plain.group_norm(x, torch.ones(24, dtype=torch.float64), 1e-6, 1)
    assert torch.allclose(one, x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6))
    three = plain.group_norm(x, torch.ones(24, dtype=torch.float64), 1e-6, 3)
    assert torch.allclose(three[:, 8:16], x[:, 8:16] / torch.sqrt((x[:, 8:16] ** 2).mean(-1, keepdim=True) + 1e-6))
    # a single token sees itself alone (distance 0 costs nothing) and shares its weight with the sink
    lm = cfg["layers"][1]["mixer"]
    y = plain.latent_attention(h[:1], w, "l1.mix", lm, eps)
    down = h[:1] @ w["l1.mix.dkv"].T
    c = down[:, :24] / torch.sqrt((down[:, :24] ** 2).mean(-1, keepdim=True) + eps) * w["l1.mix.dkv.norm"]
    qq = (h[:1] @ w["l1.mix.q"].T).reshape(1, 3, 20)
    heads = []
    for hd in range(3):                                      # position 0 rotates by nothing but the factor on cos
        mag = 0.1 * math.log(4.0) + 1.0
        sc = (qq[0, hd, :8] @ (w["l1.mix.uk"].reshape(3, 8, 24)[hd] @ c[0]) + mag * mag * (qq[0, hd, 8:] @ down[0, 24:])) * 0.4
        p = torch.exp(sc) / (torch.exp(sc) + torch.exp(w["l1.mix.sink"][hd]))
        heads.append(p * (w["l1.mix.uv"].reshape(3, 20, 24)[hd] @ c[0]))
    assert torch.allclose(y[0], torch.cat(heads) @ w["l1.mix.o"].T)
    assert plain.schedule(cfg) == [(0, 0), (1, 0), (0, 1), (1, 1), (0, 2), (1, 2), (2, 0)]


# ------------------------------------------------------------------ GPU: the mechanisms alone
def _runner_for(cfg, dtype, seed, tokens=512, tensors=None, **kw):
    from inferflux_b200.config import EngineConfig
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine import Model, StepRunner
    config, made = malazen_tensors(cfg, seed, **kw)
    tensors = tensors or made
    model = Model(build_spec(config), dtype, DEV)
    plain_w = {k: v.double() for k, v in tensors.items()}
    model.load({k: (v.to(dtype) if v.dim() > 1 else v.float()).to(DEV) for k, v in tensors.items()})
    runner = StepRunner(model, EngineConfig(dtype=NAME[dtype], kv_cache_tokens=tokens, max_seqs=4))
    return model, runner, plain_w


def _mixer_in_portions(model, runner, layer, x, portions, dtype, branch=None):
    """Call one layer's mixer (or one of its two branches) alone on rows cut into portions of one request."""
    from inferflux_b200.engine import StepEntry
    info, block = model.runs[layer], model.blocks[layer]
    mixer = block.mixer if branch is None else block.mixer.mixers[branch]
    outs, pos = [], 0
    for n in portions:
        ctx = runner.build_context([StepEntry("r", [1] * n, [])])
        for name, part in model.positions.items():
            ctx.position_tables[name] = part.prepare(ctx)
        position = ctx.position_tables.get(block.position_name) if block.position_name else None
        outs.append(_dense(mixer.forward(x[pos:pos + n].to(dtype).to(DEV).contiguous(), ctx, info, position)))
        runner.kv.advance("r", n)
        pos += n
    runner.end("r")
    return torch.cat(outs)


def _one_layer(name, layer, **changes):
    cfg = dict(ML[name], layers=[copy.deepcopy(ML[name]["layers"][layer])], loop=None)
    cfg["layers"][0]["mixer"].update(changes)
    return cfg


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,groups", [(50, 1), (50, 5), (64, 4), (1000, 8), (96, 24)])
def test_group_norm_with_a_weighted_sum(dtype, hidden, groups):
    """The norm in groups alone, with a tensor, with partial sums, with two branches and a factor each (the sum goes
    into the float32 stream), and on picked rows, which leave the stream as it is."""
    from inferflux_b200.parts.base import PartialSums, ScaledSum
    from inferflux_b200.parts.norm import GroupRMSNorm
    eps, tol = 3e-6, (2e-6 if dtype == torch.float32 else 5e-3)
    part = GroupRMSNorm(dict(weight_name="n", hidden=hidden, eps=eps, groups=groups), "", dtype, DEV)
    wt = (1 + _rand((hidden,), 3, 0.2))
    part.load({"n": wt.to(DEV)})
    res, a, b = _rand((7, hidden), 1, 3.0), _rand((3, 7, hidden), 2), _rand((7, hidden), 4)
    stream = res.clone().to(DEV)
    assert _rel(part.forward(stream, None), plain.group_norm(res.double(), wt.double(), eps, groups)) < tol
    assert torch.equal(stream.cpu(), res)
    want = res.double() + 0.7 * a.double().sum(0) + 1.9 * b.double()
    got = part.forward(stream, ScaledSum([(PartialSums(a.to(DEV)), 0.7), (b.to(DEV), 1.9)]))
    assert _rel(stream, want) < 1e-6 and _rel(got, plain.group_norm(want, wt.double(), eps, groups)) < tol
    stream2 = res.clone().to(DEV)
    got = part.forward(stream2, PartialSums(a.to(DEV)))
    assert _rel(got, plain.group_norm(res.double() + a.double().sum(0), wt.double(), eps, groups)) < tol
    rows = torch.tensor([6, 0, 6], dtype=torch.int32, device=DEV)
    before = stream2.clone()
    picked = part.forward(stream2, None, rows=rows)
    assert torch.equal(stream2, before) and _rel(picked, plain.group_norm(before.cpu().double()[[6, 0, 6]], wt.double(), eps, groups)) < tol
    if groups == 1:                                          # one group is the plain norm
        from inferflux_b200.parts.norm import RMSNorm
        ref = RMSNorm(dict(weight_name="n", hidden=hidden, eps=eps), "", dtype, DEV)
        ref.load({"n": wt.to(DEV)})
        assert _rel(part.forward(stream2, None), ref.forward(stream2, None)) < tol


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,ff,limit,rows", [(64, 96, 2.0, 3), (50, 35, 0.7, 70), (128, 160, 1.5, 300), (50, 45, 30.0, 1)])
def test_clamped_feed_forward_alone(dtype, hidden, ff, limit, rows):
    """Inputs large enough that both clamps bite (and, at a limit of 30, never), few rows and many."""
    from inferflux_b200.parts.feed_forward import ClampedGLU
    params = dict(name="mlp", hidden=hidden, intermediate=ff, limit=limit)
    part = ClampedGLU(params, "l0", dtype, DEV)
    w = {s.name: _rand(s.shape, 50 + i, 0.3).to(torch.bfloat16).float() for i, s in enumerate(ClampedGLU.weight_specs(params, "l0"))}
    part.load({k: (v.to(dtype) if v.dim() > 1 else v).to(DEV) for k, v in w.items()})
    x = _rand((rows, hidden), 51, 2.0).to(dtype)
    w64 = {k: v.double() for k, v in w.items()}
    want = plain.clamped_glu(x.double(), w64, "l0.mlp", limit)
    g = x.double() @ w64["l0.mlp.gate"].T + w64["l0.mlp.gate.b"]
    assert (limit > 10) or (float((g > limit).double().mean()) > 0.02 and float((g < -limit).double().mean()) > 0.02)
    assert _rel(_dense(part.forward(x.to(DEV), None)), want) < PTOL[dtype]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 2), ("B", 1), ("B", 3), ("C", 1)])
def test_biased_attention_alone(dtype, name, layer):
    """The left branch: portions that start and end inside pages, single tokens across page borders and across the
    temperature's steps; grouped and ungrouped heads, with and without temperature; then the pages again."""
    cfg = _one_layer(name, layer)
    model, runner, w = _runner_for(cfg, dtype, 30 + layer, tokens=512)
    portions = [21, 1, 2, 1, 1, 10, 45, 1, 1, 2, 16, 1, 40]
    x = _rand((sum(portions), cfg["width"]), 31).to(dtype)
    want = plain.biased_attention(x.double(), w, "l0.mix.left", cfg["layers"][0]["mixer"]["left"])
    got = _mixer_in_portions(model, runner, 0, x, portions, dtype, branch=0)
    assert _rel(got, want) < PTOL[dtype]
    again = _mixer_in_portions(model, runner, 0, x[:9], [2, 7], dtype, branch=0)
    assert _rel(again, want[:9]) < PTOL[dtype]
    runner.kv.check()


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,vdim,width", [(16, 12, 64), (64, 64, 160), (128, 128, 320)])
def test_a_key_far_back_under_the_toll(dtype, dim, vdim, width):
    """400 tokens, pages of 16.  Head 0's query is the token's first ``dim`` numbers and the key the next ``dim``.  Each
    of the last eight tokens gets a query that matches the key of one chosen earlier token and no other: the very
    first token, a page's last and first token, the token just before, itself, tokens hundreds back.  The match
    outweighs the distance's toll, so that token takes the weight; altering it changes the plain result.  The toll
    and the temperature are on: with the toll's sign turned the far keys would win by much more, which the second
    comparison shows.  The first two of the eight queries come inside a portion, the others as single tokens."""
    n = 400
    left = dict(heads=2, kv_heads=1, dim=dim, vdim=vdim, scale=1.0, q_temp=dict(coef=0.3, every=64))
    cfg = dict(ML["A"], width=width, loop=None, layers=[dict(type="parallel", mixer=dict(left=left, right=dict(heads=1, dim=4, vdim=4, tau=2.0)), mlp=None)])
    _, tensors = malazen_tensors(cfg, 21)
    eye = torch.eye(dim)
    tensors["l0.mix.left.q"] = torch.cat([torch.cat([eye, torch.zeros(dim, width - dim)], 1), _rand((dim, width), 22, 0.05)]).to(torch.bfloat16)
    tensors["l0.mix.left.k"] = torch.cat([torch.zeros(dim, dim), eye, torch.zeros(dim, width - 2 * dim)], 1).to(torch.bfloat16)
    for leaf in ("q.b", "k.b"):
        tensors[f"l0.mix.left.{leaf}"] = torch.zeros_like(tensors[f"l0.mix.left.{leaf}"])
    tensors["l0.mix.left.r1"] = torch.tensor([1.5, 0.5]).to(torch.bfloat16)
    tensors["l0.mix.left.r2"] = torch.tensor([0.75, 2.0]).to(torch.bfloat16)
    model, runner, w = _runner_for(cfg, dtype, 21, tensors=tensors)
    x = _rand((n, width), 23, 0.3).to(torch.bfloat16).float()
    x[:, :2 * dim] *= 0.1                                        # quiet queries and keys, but for the chosen pairs
    first_q = n - 8
    targets = [0, 15, 16, first_q + 2, first_q + 4, 7, 200, 383]
    for q, t in zip(range(first_q, n), targets):
        u = torch.zeros(dim)
        u[(q - first_q) % dim] = 1.0                             # a direction of its own for every pair
        x[t, dim:2 * dim] += 5.0 * u                             # added: one token may be the target of two queries
        x[q, :dim] = 5.0 * u
    m = cfg["layers"][0]["mixer"]["left"]
    want = plain.biased_attention(x.double(), w, "l0.mix.left", m)
    for q, t in zip(range(first_q, n), targets):                 # the plain result does rest on these single keys
        other = x.clone()
        other[t, dim:2 * dim] = 0.03
        moved = plain.biased_attention(other.double(), w, "l0.mix.left", m)[q]
        assert _rel(moved, want[q]) > 0.2, (q, t)
    got = _mixer_in_portions(model, runner, 0, x, [150, 200, 44] + [1] * 6, dtype, branch=0)
    assert _rel(got, want) < PTOL[dtype]
    w_free = dict(w)
    w_free["l0.mix.left.r1"] = torch.zeros(2, dtype=torch.float64)
    assert _rel(plain.biased_attention(x.double(), w_free, "l0.mix.left", m), want) > 0.05       # the toll does show
    flat = dict(m, q_temp=None)
    assert _rel(plain.biased_attention(x.double(), w, "l0.mix.left", flat), want) > 0.01         # and so does the temperature


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 2), ("B", 1), ("B", 3), ("C", 1)])
def test_gated_linear_attention_alone(dtype, name, layer):
    """The right branch: portions longer than the kernel's staging, portions of one and two tokens, single tokens;
    heads of 6 to 64 rows with values narrower and wider than a block's columns; a decay projection whose inner
    size the tensors give; then the slot again, which the next request finds zeroed."""
    cfg = _one_layer(name, layer)
    model, runner, w = _runner_for(cfg, dtype, 40 + layer, tokens=512)
    assert model.blocks[0].mixer.mixers[1].rank == 16
    portions = [150, 1, 1, 2, 64, 7, 1, 33, 16, 17]
    x = _rand((sum(portions), cfg["width"]), 41).to(dtype)
    m, eps = cfg["layers"][0]["mixer"]["right"], cfg["norm"]["eps"]
    want, _ = plain.gated_linear_attention(x.double(), w, "l0.mix.right", m, eps)
    got = _mixer_in_portions(model, runner, 0, x, portions, dtype, branch=1)
    assert _rel(got, want) < PTOL[dtype]
    again = _mixer_in_portions(model, runner, 0, x[:10], [10], dtype, branch=1)
    assert _rel(again, want[:10]) < PTOL[dtype]


@gpu
def test_gated_linear_state_far_back_shows():
    """Decays close to one (a large bias under a large tau): what the first token wrote into the state still carries
    the result 300 tokens on, in a prompt and in decoding, so a state that a portion's start, a slot or a step lost
    would show; and decays close to zero, where only the token itself is left."""
    cfg = _one_layer("A", 0)
    m, eps = cfg["layers"][0]["mixer"]["right"], cfg["norm"]["eps"]
    for bias in (9.0, -40.0):
        _, tensors = malazen_tensors(cfg, 5)
        tensors["l0.mix.right.a2.b"] = torch.full((36,), bias).to(torch.bfloat16)
        tensors["l0.mix.right.a2"] = tensors["l0.mix.right.a2"] * 0
        model, runner, w = _runner_for(cfg, torch.float32, 5, tensors=tensors)
        x = _rand((300, 64), 6).to(torch.bfloat16).float()
        x[1:] *= 0.05
        want, _ = plain.gated_linear_attention(x.double(), w, "l0.mix.right", m, eps)
        lost, _ = plain.gated_linear_attention(x.double()[1:], w, "l0.mix.right", m, eps)
        assert (_rel(lost[-1], want[-1]) > 0.05) == (bias > 0)                      # the plain result rests on token 0, or not at all
        got = _mixer_in_portions(model, runner, 0, x, [1, 2, 200, 90] + [1] * 7, torch.float32, branch=1)
        assert _rel(got, want) < PTOL[torch.float32]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 1), ("B", 0), ("B", 2), ("C", 0), ("C", 2)])
def test_latent_attention_alone(dtype, name, layer):
    """Portions that start and end inside pages and windows, single tokens across page borders and past the window;
    a rotated part longer and shorter than the plain one and none, stretched frequencies, a window shorter than a
    page and none, a latent that is no multiple of 8; then the pages again."""
    cfg = _one_layer(name, layer)
    model, runner, w = _runner_for(cfg, dtype, 30 + layer, tokens=512)
    portions = [21, 1, 2, 1, 1, 10, 45, 1, 1, 2, 16, 1, 40]
    x = _rand((sum(portions), cfg["width"]), 31).to(dtype)
    want = plain.latent_attention(x.double(), w, "l0.mix", cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    got = _mixer_in_portions(model, runner, 0, x, portions, dtype)
    assert _rel(got, want) < PTOL[dtype]
    again = _mixer_in_portions(model, runner, 0, x[:9], [2, 7], dtype)
    assert _rel(again, want[:9]) < PTOL[dtype]
    runner.kv.check()


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 700])
def test_latent_attention_over_a_long_context(dtype, window):
    """900 tokens without a window or with one of 700: single tokens whose keys the tensor-core kernel cuts into parts
    that a second kernel merges, the sink counted once."""
    cfg = _one_layer("C", 2)
    cfg["layers"][0]["mixer"].pop("mask")
    if window:
        cfg["layers"][0]["mixer"]["mask"] = dict(size=window)
    model, runner, w = _runner_for(cfg, dtype, 33, tokens=1024)
    portions = [600, 1, 1, 290, 1, 1, 2, 1, 1, 1, 1]
    x = _rand((sum(portions), cfg["width"]), 34).to(dtype)
    want = plain.latent_attention(x.double(), w, "l0.mix", cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    got = _mixer_in_portions(model, runner, 0, x, portions, dtype)
    assert _rel(got, want) < PTOL[dtype]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank,rot,width", [(16, 12, 64), (56, 8, 160)])
def test_latent_window_edges_and_sink_with_one_score_that_stands_out(dtype, rank, rot, width):
    """210 tokens, a window of 40, pages of 16.  Head 0's rotated query part is read off the token's first ``rot``
    numbers and the shared rotated key part off the next ``rot``, with a rotation base so large that nothing turns;
    the plain parts are quiet.  Each of the last eight tokens gets a query that matches the key part of one chosen
    earlier token and no other: the last one inside its window, the first one outside, a page's last and first token
    inside the window, the token just before, the very first token (long gone), one far outside, and itself.  A
    visible target takes the weight it does not leave to the sink; a window or a page's edge that is off by one
    changes the result entirely.  Head 0's sink is set so high that it takes about half of every weight, head 1's so
    low that it takes none: a sink left out, counted twice or scaled would show."""
    n, wn = 210, 40
    mixer = dict(heads=2, dim=8, rot_dim=rot, vdim=12, kv_rank=rank, mask=dict(size=wn), rot=dict(dims=rot, base=1e30), scale=1.0)
    cfg = dict(ML["A"], width=width, loop=None, layers=[dict(type="latent_attention", mixer=mixer, mlp=None)])
    _, tensors = malazen_tensors(cfg, 21)
    eye = torch.eye(rot)
    q = _rand((2 * (8 + rot), width), 22, 0.02)
    q[8:8 + rot] = torch.cat([eye, torch.zeros(rot, width - rot)], 1)                                  # head 0's rotated part
    tensors["l0.mix.q"] = q.to(torch.bfloat16)
    dkv = _rand((rank + rot, width), 24, 0.5)
    dkv[rank:] = torch.cat([torch.zeros(rot, rot), eye, torch.zeros(rot, width - 2 * rot)], 1)
    tensors["l0.mix.dkv"] = dkv.to(torch.bfloat16)
    tensors["l0.mix.sink"] = torch.tensor([9.0, -30.0]).to(torch.bfloat16)                             # 3 * 3 = the match's score
    model, runner, w = _runner_for(cfg, dtype, 21, tensors=tensors)
    x = _rand((n, width), 23, 0.3).to(torch.bfloat16).float()
    x[:, :2 * rot] *= 0.1
    first_q = n - 8
    targets = [p - off if off is not None else t for p, (off, t) in zip(range(first_q, n), [
        (wn - 1, None), (wn, None), (None, 191), (None, 192), (1, None), (None, 0), (100, None), (0, None)])]
    for qi, t in zip(range(first_q, n), targets):
        u = torch.zeros(rot)
        u[2 + (qi - first_q) % (rot - 2)] = 1.0                  # not the first pair: its frequency is 1 whatever the base
        x[t, rot:2 * rot] += 3.0 * u
        x[qi, :rot] = 3.0 * u
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    want = plain.latent_attention(x.double(), w, "l0.mix", m, eps)
    seen = [True, False, True, True, True, False, False, True]
    for qi, t, vis in zip(range(first_q, n), targets, seen):      # the plain result does rest on exactly the visible ones
        other = x.clone()
        other[t, rot:2 * rot] = 0.03
        moved = plain.latent_attention(other.double(), w, "l0.mix", m, eps)[qi]
        assert (_rel(moved, want[qi]) > 0.1) == vis, (qi, t)
    got = _mixer_in_portions(model, runner, 0, x, [150, 54] + [1] * 6, dtype)
    assert _rel(got, want) < PTOL[dtype]
    wider = dict(m, mask=dict(size=wn + 1))                       # the first invisible target, made visible, would show
    assert _rel(plain.latent_attention(x.double(), w, "l0.mix", wider, eps)[first_q + 1], want[first_q + 1]) > 0.1
    for sink in ([-30.0, -30.0], [9.0 + math.log(2.0), -30.0]):  # no sink, or one counted twice, would show
        w2 = dict(w)
        w2["l0.mix.sink"] = torch.tensor(sink, dtype=torch.float64)
        assert _rel(plain.latent_attention(x.double(), w2, "l0.mix", m, eps)[first_q], want[first_q]) > 0.1


@gpu
def test_rotation_of_neighbouring_pairs_with_stretched_frequencies():
    from inferflux_b200.parts.position import RotaryHalf
    rot = dict(dims=12, base=3000.0, scaling=dict(factor=6.0, original=40, fast=8.0, slow=1.5))
    part = RotaryHalf(dict(rotary_dim=12, theta=3000.0, scaling=rot["scaling"]), "", torch.float32, DEV)
    f, mag = plain.rotary_frequencies(rot)
    assert _rel(part.inv_freq, f) < 1e-12 and abs(part.magnitude - mag) < 1e-12
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 123456], dtype=torch.int32, device=DEV)

    class Ctx:
        n_tokens, positions, device = 7, pos, DEV
    cos, sin = part.prepare(Ctx)
    ang = pos.cpu().double()[:, None] * f[None, :]
    assert _rel(cos, torch.cos(ang) * mag) < 2e-6 and _rel(sin, torch.sin(ang) * mag) < 2e-6


# ------------------------------------------------------------------ GPU: whole models through the step function
def _logits_in_steps(runner, rid, toks, sizes):
    from inferflux_b200.engine import StepEntry
    outs, pos, k = [], 0, 0
    while pos < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - pos)
        outs.append(runner.step([StepEntry(rid, toks[pos:pos + n], list(range(n)))]).clone())
        pos, k = pos + n, k + 1
    runner.end(rid)
    return torch.cat(outs)


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_model_whole_one_by_one_and_in_portions(dtype, name):
    """The logits at every position for three ways of cutting the same prompt."""
    cfg = ML[name]
    model, runner, w = _runner_for(cfg, dtype, ord(name), tokens=1024)
    toks = random_tokens(cfg["vocab"], 150, 31)
    want, limit = _plain_logits(cfg, w, toks, dtype)
    whole = _logits_in_steps(runner, "w", toks, [150])
    assert _model_err(whole, want, dtype) < limit
    ones = _logits_in_steps(runner, "o", toks[:90], [1])              # the captured decode graph after three steps
    assert runner.graph_replays > 0 and _model_err(ones, want[:90], dtype) < limit
    cut = _logits_in_steps(runner, "c", toks, [2, 3, 17, 1, 16, 5, 32, 2, 15, 64, 2])
    assert _model_err(cut, want, dtype) < limit
    if dtype == torch.float32:
        assert _rel(cut, whole) < 1e-5 and _rel(ones, whole[:90]) < 1e-5
    runner.kv.check(), runner.slots.check()


@gpu
def test_stream_after_every_layer():
    from inferflux_b200.engine import StepEntry
    from inferflux_b200.parts.base import ScaledSum
    cfg = ML["A"]
    model, runner, w = _runner_for(cfg, torch.float32, 9)
    toks = random_tokens(cfg["vocab"], 60, 4)
    want = []
    plain.forward(cfg, w, toks, want)
    seen = []
    for block in model.blocks:
        if not hasattr(block, "mixer"):
            continue                                                  # the junction ahead of a pass is no layer

        def watched(residual, delta, ctx, run, inner=block.forward):
            out = inner(residual, delta, ctx, run)
            seen.append(residual.clone() + (_dense(out) if out is not None else 0.0))
            return out
        block.forward = watched
    runner.step([StepEntry("s", toks, [0])])
    assert len(seen) == len(want) == 7 and all(_rel(g, x) < 2e-5 for g, x in zip(seen, want))


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_batches_of_unequal_requests_and_reused_slots(dtype, name):
    """Four requests of unequal length, portions beside single tokens, against each alone; then four more in
    the slots and pages the first ones gave back."""
    from inferflux_b200.engine import StepEntry
    cfg = ML[name]
    model, runner, w = _runner_for(cfg, dtype, 41, tokens=4 * 128)
    rng = random.Random(3)
    for round_ in range(2):
        lens = [97, 5, 64, 33] if round_ == 0 else [31, 120, 2, 70]
        reqs = {f"r{round_}{i}": random_tokens(cfg["vocab"], n, 500 + 100 * round_ + 10 * i) for i, n in enumerate(lens)}
        want = {r: _plain_logits(cfg, w, t, dtype) for r, t in reqs.items()}
        alone = {}
        for r, t in reqs.items():                                  # each alone, its whole prompt in one step
            alone[r] = runner.step([StepEntry("alone", t, list(range(len(t))))]).clone()
            runner.end("alone")
        at, got = {r: 0 for r in reqs}, {r: [] for r in reqs}
        while any(at[r] < len(reqs[r]) for r in reqs):
            entries = []
            for r, t in reqs.items():
                left = len(t) - at[r]
                if left == 0 or (rng.random() < 0.2 and len(entries)):
                    continue
                n = 1 if left <= 6 else min(left - 6, rng.choice([1, 2, 3, 16, 29]))
                entries.append(StepEntry(r, t[at[r]:at[r] + n], list(range(n))))
            logits = runner.step(entries)
            row = 0
            for e in entries:
                got[e.rid].append(logits[row:row + len(e.tokens)].clone())
                row += len(e.tokens)
                at[e.rid] += len(e.tokens)
        for r in reqs:
            rows = torch.cat(got[r])
            ref, limit = want[r]
            assert _model_err(rows, ref, dtype) < limit, r
            assert _model_err(rows, alone[r], dtype) < (1e-5 if dtype == torch.float32 else limit), r
            runner.end(r)
        runner.kv.check(), runner.slots.check()
    assert all(p.reuses > 0 for p in runner.kv.pools)


@gpu
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_past_the_window(name):
    """300 tokens at once, then 200 one by one through the captured graph: the windows (7 and 20 tokens) pass over
    decoded tokens many times, pages behind them go back to the pool and come again, the states go on, the
    temperature steps up."""
    cfg = ML[name]
    model, runner, w = _runner_for(cfg, torch.float32, 51, tokens=512)
    toks = random_tokens(cfg["vocab"], 500, 52)
    want = plain.forward(cfg, w, toks)
    got = _logits_in_steps(runner, "d", toks, [300] + [1] * 200)
    assert runner.graph_replays >= 190 and _rel(got, want) < 5e-5
    windowed = [p for p, need in zip(runner.kv.pools, model.kv_needs) if need.window]
    assert windowed and all(p.reuses > 0 for p in windowed)


# ------------------------------------------------------------------ GPU: bin/trace_run and Engine.generate
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_trace_replay_mixed_with_page_and_slot_reuse(name, dtype):
    """The command-line replay: the config.json picks the architecture; four state slots, a pool of the four
    longest requests; every request twice, so pages and slots turn over."""
    from helpers import load_plain_folder as load_plain
    cfg = ML[name]
    folder = make_malazen_folder(cfg, seed=60 + ord(name))
    pcfg, w = load_plain(folder)
    lengths = [70, 33, 5, 130, 64, 97, 1]
    requests = [random_tokens(cfg["vocab"], n, 1000 + 50 * i) for i, n in enumerate(lengths)]
    refs, limits = zip(*(_plain_logits(pcfg, w, r, dtype) for r in requests))
    pool = sum((n + 63) // 64 * 64 for n in sorted(lengths)[-4:])
    proc = TraceProcess(folder, dtype, pool)
    rng = random.Random(7)
    waiting = [(f"m{j}_{i}", i) for j, i in enumerate(list(range(len(requests))) * 2)]
    live, worst = {}, 0.0
    while waiting or live:
        while waiting and len(live) < 4:
            rid, i = waiting.pop(0)
            live[rid] = [i, 0]
        entries, ends, checks = [], [], []
        for rid, (i, pos) in list(live.items()):
            toks = requests[i]
            if rng.random() < 0.15 and len(live) > 1:
                continue
            left = len(toks) - pos
            n = 1 if left <= 20 else min(left - 20, rng.choice([2, 3, 7, 16, 29, 48]))
            want = list(range(n)) if n <= 3 else sorted(rng.sample(range(n), 3))
            entries.append(dict(id=rid, tokens=toks[pos:pos + n], want=want))
            checks.append((i, pos, want))
            live[rid][1] = pos + n
            if pos + n == len(toks):
                ends.append(rid)
                del live[rid]
        if not entries:
            continue
        got = proc.step(entries, end=ends)
        row = 0
        for i, pos, want in checks:
            for p in want:
                g = torch.tensor(got[row:row + 1].astype(np.float64))
                if dtype == "float32":
                    err = float((g[0] - refs[i][pos + p]).abs().max() / refs[i].abs().max())
                else:                                                  # the row's error on the whole request's scale
                    d = g[0] - refs[i][pos + p]
                    err = float((d - d.mean()).pow(2).mean().sqrt() / (refs[i] - refs[i].mean(-1, keepdim=True)).pow(2).mean().sqrt())
                worst = max(worst, err / limits[i])
                row += 1
    stats = proc.stats()
    assert proc.close() == 0
    assert worst < 1.0, worst
    assert all(u > 0 for u in stats["page_reuses"]) and stats["pages_free"] == stats["pages_total"]


@gpu
def test_greedy_generation_through_the_engine():
    """Engine.from_pretrained picks the architecture by config.json; the scheduler cuts prompts into portions of
    16 and batches them with decoding requests; float32 greedy continuations equal the plain ones."""
    from helpers import load_plain_folder as load_plain
    from inferflux_b200 import Engine, SamplingParams
    cfg = ML["A"]
    folder = make_malazen_folder(cfg, seed=71)
    pcfg, w = load_plain(folder)
    prompts = [random_tokens(cfg["vocab"], n, 80 + n) for n in (5, 41, 17, 70, 3)]

    def plain_greedy(p, n):
        seq = list(p)
        for _ in range(n):
            seq.append(int(plain.forward(pcfg, w, seq)[-1].argmax()))
        return seq[len(p):]

    want = [plain_greedy(p, 12) for p in prompts]
    eng = Engine.from_pretrained(folder, dtype="float32", kv_cache_tokens=512, max_seqs=4, chunked_prefill_tokens=16)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    assert [g.tokens for g in got] == want
