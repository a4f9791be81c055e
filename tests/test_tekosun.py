"""The Tekosun architecture against its plain restatement (plain_tekosun.py): every mechanism alone through its part
and kernels, then whole models of three tiny configurations that differ in every size, option and order of layers,
stepped whole, token by token, in portions down to two tokens, in mixed batches over a pool so small that pages and
state slots are used again, through bin/trace_run and through Engine.generate.  Weights are random; one test sets
keys and queries by hand so that one score stands out just inside and just outside the window, at page borders and
at the first token; the recurrences get slow decays so that a state lost far back would show."""
from __future__ import annotations

import copy
import math
import random

import numpy as np
import pytest
import torch

import plain_tekosun as plain
from helpers import TK, TraceProcess, make_tekosun_folder, random_tokens, tekosun_tensors

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
PTOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
# Whole models.  float32: the largest difference as a fraction of the largest logit (5e-5, or three times what rounding
# the matrix products to float32 causes if that is more).  bfloat16: a position's
# root-mean-square error over the vocabulary as a fraction of the logits' root mean square, against three times what
# rounding alone causes there: the plain model run again with every matrix product's input and result rounded to
# bfloat16 (every sublayer's result is normed before it joins the stream, so a sublayer's rounding reaches the logits
# undamped, and how much that is differs from one configuration and prompt to the next).
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


def _steady_tokens(cfg, w, n, seed):
    """Random tokens for a request, the seed moved on until rounding alone does little to its logits: a prompt can
    meet a cancellation (a state-space head whose step size times B . C all but equals minus its skip weight leaves
    a norm group of nearly nothing, which the group's norm then blows up), and no engine's rounding is judged there."""
    while True:
        toks = random_tokens(cfg["vocab"], n, seed)
        if _plain_logits(_for_dtype(cfg, torch.bfloat16), w, toks, torch.bfloat16)[1] < 0.3:
            return toks
        seed += 1


def _model_err(got, want, dtype):
    return _rel(got, want) if dtype in (torch.float32, "float32") else _row_err(got, want)


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def _dense(y):
    from inferflux_b200.parts.base import PartialSums
    return y.tensor.sum(0) if isinstance(y, PartialSums) else y.float()


def _for_dtype(cfg, dtype):
    """Which experts a token takes is a discrete choice: in bfloat16 the stream differs from the plain one by
    roundings that can turn a close call the other way, and the logits then differ entirely.  So bfloat16 whole
    models take every expert (the weights still vary with the token, the sort and the tiles are the same); the
    choice itself is tested in bfloat16 on the part alone, close calls left out, and in whole models in float32."""
    if dtype in (torch.float32, "float32"):
        return cfg
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer["mlp"]:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return cfg


# ------------------------------------------------------------------ CPU: configuration, spec, cache plan, the plain code
def test_config_is_read_from_its_own_keys():
    from inferflux_b200.config import ConfigError, TekosunConfig, build_spec, load_config
    cfg = load_config(copy.deepcopy(TK["A"]))
    assert isinstance(cfg, TekosunConfig) and cfg.width == 64 and cfg.vocab_size == 300 and cfg.norm_eps == 1e-5
    assert cfg.embedding_scale == 3.0 and [l.type for l in cfg.layers] == ["attention", "mamba2", "general_delta", "attention"]
    a = cfg.layers[0].mixer
    assert (a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["window"], a["v_mix"]) == (4, 2, 16, 24, 20, True)
    assert a["rot"]["scaling"] == dict(factor=4.0, low=1.0, high=8.0, original=64.0)
    assert cfg.layers[1].mixer == dict(heads=3, vdim=12, state=8, groups=1, conv=4, norm_groups=1) and cfg.layers[1].mlp is None
    assert cfg.layers[2].mlp == dict(kind="moe", ff=32, experts=4, top=1, scale=0.5, shared_ff=None)
    assert cfg.layers[0].mlp["shared_ff"] == 24
    bare = load_config(copy.deepcopy(TK["B"]))
    b = bare.layers[1].mixer                                                # absent keys: their defaults
    assert (b["kv_heads"], b["vdim"], b["window"], b["v_mix"], b["rot"]["dims"]) == (3, 10, None, False, 0)
    assert bare.embedding_scale == 1.0 and bare.layers[0].mlp["scale"] == 1.0 and bare.layers[4].mixer["groups"] == 1
    assert load_config(cfg.to_dict()) == cfg and load_config(bare.to_dict()) == bare
    spec = build_spec(cfg)
    assert sorted(spec.positions) == ["rot0", "rot1"] and [l.arrangement for l in spec.layers] == ["post_norm"] * 4
    assert [l.parts["mixer"].kind for l in spec.layers] == ["window_attention", "mamba2", "general_delta", "window_attention"]
    assert [l.parts["mixer"].params.get("v_mix") for l in spec.layers] == ["first", None, None, "blend"]
    assert "feed_forward" not in spec.layers[1].parts and spec.layers[0].parts["feed_forward"].params["shared"] == 24
    c = build_spec(load_config(copy.deepcopy(TK["C"])))
    assert [l.parts["mixer"].params.get("v_mix") for l in c.layers] == [None, "first", None, "blend", "blend"]
    assert len(c.positions) == 2                                            # the first and the last attention share a table
    for breaker, text in [(lambda d: d["layers"][0].update(type="serial"), "type"), (lambda d: d.pop("width"), "width"),
                          (lambda d: d["layers"][0]["mixer"].pop("dim"), "dim"),
                          (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
                          (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
                          (lambda d: d["layers"][3]["mixer"].update(vdim=16), "v_mix"),
                          (lambda d: d["layers"][1]["mixer"].update(groups=2), "groups"),
                          (lambda d: d["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
                          (lambda d: d["layers"][2]["mlp"]["router"].update(top=6), "top"),
                          (lambda d: d["norm"].pop("eps"), "eps"), (lambda d: d["layers"][0]["mlp"].update(kind="glu"), "kind")]:
        bad = copy.deepcopy(TK["A"])
        breaker(bad)
        with pytest.raises(ConfigError, match=text):
            load_config(bad)


def test_cache_and_state_plan():
    from inferflux_b200.config import build_spec, load_config
    from inferflux_b200.engine import Model
    model = Model(build_spec(load_config(copy.deepcopy(TK["A"]))), torch.float32, "cpu")
    specs = {w.name: w for w in model.weight_specs()}
    names = {n: tuple(w.shape) for n, w in specs.items()}
    assert names["embed"] == (300, 64) and names["head"] == (300, 64) and names["final.norm"] == (64,)
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.v"] == (48, 64)
    assert names["l0.mix.q.norm"] == (64,) and names["l0.mix.k.norm"] == (32,) and names["l0.mix.vmix"] == ()
    assert names["l0.mix.o"] == (64, 96) and "l0.mix.g" not in names and "l0.mix.q.conv" not in names
    assert names["l1.mix.in"] == (2 * 36 + 2 * 8 + 3, 64) and names["l1.mix.conv"] == (36 + 16, 4) and names["l1.mix.D"] == (3,)
    assert names["l2.mix.w1"] == (-1, 64) and names["l2.mix.w2"] == (24, -1) and names["l2.mix.a.b"] == (24,)
    assert specs["l2.mix.w1"].fits((7, 64)) and not specs["l2.mix.w1"].fits((7, 65))       # the stored size stands
    assert names["l0.mlp.router"] == (5, 64) and "l0.mlp.router.b" not in names and "l0.mlp.e0.gate" not in names
    assert names["l0.mlp.e4.up"] == (40, 64) and names["l0.mlp.shared.down"] == (64, 24) and "l2.mlp.shared.up" not in names
    assert "l1.norm2" not in names and names["l1.norm1"] == (64,)
    needs = [(n.streams[0].width, n.streams[1].width, n.window) for n in model.kv_needs]
    assert needs == [(16, 24, 20), (32, 24, 33)]
    states = [{s.name: tuple(s.shape) for s in per_run} for per_run in model.state_needs]
    assert states == [{}, {"ssm": (3, 12, 8), "ssm_conv_tail": (3, 52)}, {"delta": (2, 12, 12)}, {}]
    one_tap = Model(build_spec(load_config(copy.deepcopy(TK["B"]))), torch.float32, "cpu")
    assert [s.name for s in one_tap.state_needs[4]] == ["ssm"]                     # one tap reaches no token back
    c = Model(build_spec(load_config(copy.deepcopy(TK["C"]))), torch.float32, "cpu")
    assert c.runs_per_group == [2, 1]                                              # equal needs share a cache group


def test_plain_carry_over_routing_and_bands():
    """The plain implementation's own consistency: sequences cut in two with tail and state handed over, the
    recurrences as sums over earlier tokens, the router, the frequency bands."""
    u, w, b = _rand((11, 6), 1).double(), _rand((6, 4), 2).double(), _rand((6,), 3).double()
    whole, _ = plain.causal_conv(u, w, b)
    a1, tail = plain.causal_conv(u[:2], w, b)
    a2, tail = plain.causal_conv(u[2:3], w, b, tail)
    a3, _ = plain.causal_conv(u[3:], w, b, tail)
    assert torch.allclose(torch.cat([a1, a2, a3]), whole)
    assert torch.allclose(whole[0], b + w[:, 3] * u[0]) and torch.allclose(whole[1], b + w[:, 3] * u[1] + w[:, 2] * u[0])
    x, bb, cc = _rand((9, 4, 5), 4).double(), _rand((9, 2, 3), 5).double(), _rand((9, 2, 3), 6).double()
    dt, a_log, d = _rand((9, 4), 7).double().abs(), _rand((4,), 8).double(), _rand((4,), 9).double()
    y, s = plain.ssm_scan(x, bb, cc, dt, a_log, d)
    y1, s1 = plain.ssm_scan(x[:4], bb[:4], cc[:4], dt[:4], a_log, d)
    y2, s2 = plain.ssm_scan(x[4:], bb[4:], cc[4:], dt[4:], a_log, d, s1)
    assert torch.allclose(torch.cat([y1, y2]), y) and torch.allclose(s2, s)
    h, g = 3, 1                                                             # head 3 reads group 1; as a sum over earlier tokens
    direct = d[h] * x[8, h] + sum(math.exp(-math.exp(float(a_log[h])) * float(dt[j + 1:, h].sum())) * dt[j, h] * (cc[8, g] @ bb[j, g]) * x[j, h]
                                  for j in range(9))
    assert torch.allclose(y[8, h], direct)
    r, k, v = _rand((7, 2, 4), 10).double(), _rand((7, 2, 4), 11).double(), _rand((7, 2, 4), 12).double()
    dec, rate = torch.rand(7, 2, 4, dtype=torch.float64), torch.rand(7, 2, 4, dtype=torch.float64)
    o, s = plain.delta_scan(r, k, v, dec, rate)
    o1, s1 = plain.delta_scan(r[:3], k[:3], v[:3], dec[:3], rate[:3])
    o2, s2 = plain.delta_scan(r[3:], k[3:], v[3:], dec[3:], rate[3:], s1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(s2, s)
    assert torch.allclose(o[0, 1], (r[0, 1] @ k[0, 1]) * v[0, 1])          # the first token finds an empty state
    # no removal and no decay: plain linear attention
    o_lin, _ = plain.delta_scan(r, k, v, torch.ones_like(dec), torch.zeros_like(rate))
    assert torch.allclose(o_lin[6, 0], sum((r[6, 0] @ k[j, 0]) * v[j, 0] for j in range(7)))
    ids, wts = plain.route(torch.tensor([[1.0, 3.0, 3.0, -1.0]], dtype=torch.float64), 2, 2.25)
    assert ids.tolist() == [[1, 2]] and torch.allclose(wts, torch.tensor([[1.125, 1.125]], dtype=torch.float64))
    ids, wts = plain.route(torch.tensor([[0.0, math.log(3.0)]], dtype=torch.float64), 1, 1.0)
    assert ids.tolist() == [[1]] and torch.allclose(wts, torch.ones(1, 1, dtype=torch.float64))   # one choice: its score over itself
    see = plain.visible(3, 10, 4)
    assert see[0].nonzero().flatten().tolist() == [7, 8, 9, 10] and see[2].nonzero().flatten().tolist() == [9, 10, 11, 12]
    f = plain.frequencies(dict(dims=8, base=10000.0, scaling=dict(factor=4.0, low=1.0, high=8.0, original=64)))
    # wavelengths 6.3, 63, 628, 6283 against the bands' edges 8 and 64: kept, in between, stretched, stretched
    assert abs(float(f[0]) - 1.0) < 1e-12 and abs(float(f[2]) - 1e-2 / 4) < 1e-15 and abs(float(f[3]) - 1e-3 / 4) < 1e-15
    s = (64 / (2 * math.pi / 0.1) - 1.0) / 7.0
    assert abs(float(f[1]) - ((1 - s) * 0.1 / 4 + s * 0.1)) < 1e-15


# ------------------------------------------------------------------ GPU: the mechanisms alone
def _runner_for(cfg, dtype, seed, tokens=512, tensors=None, **kw):
    from inferflux_b200.config import EngineConfig
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine import Model, StepRunner
    config, made = tekosun_tensors(cfg, seed, **kw)
    tensors = tensors or made
    model = Model(build_spec(config), dtype, DEV)
    plain_w = {k: v.double() for k, v in tensors.items()}
    model.load({k: (v.to(dtype) if v.dim() > 1 else v.float()).to(DEV) for k, v in tensors.items()})
    runner = StepRunner(model, EngineConfig(dtype=NAME[dtype], kv_cache_tokens=tokens, max_seqs=4))
    return model, runner, plain_w


def _mixer_in_portions(model, runner, layer, x, portions, dtype, v_first=None):
    """Call one layer's mixer alone on rows cut into portions of one request (``v_first``: the values an earlier
    layer would have kept for the step, by row)."""
    from inferflux_b200.engine import StepEntry
    info, block = model.runs[layer], model.blocks[layer]
    outs, pos = [], 0
    for n in portions:
        ctx = runner.build_context([StepEntry("r", [1] * n, [])])
        for name, part in model.positions.items():
            ctx.position_tables[name] = part.prepare(ctx)
        position = ctx.position_tables.get(block.position_name) if block.position_name else None
        if v_first is not None:
            ctx.scratch["v_first"] = v_first[pos:pos + n].float().contiguous().to(DEV)
        outs.append(_dense(block.mixer.forward(x[pos:pos + n].to(dtype).to(DEV).contiguous(), ctx, info, position)))
        runner.kv.advance("r", n)
        pos += n
    runner.end("r")
    return torch.cat(outs)


def _one_layer(name, layer, **mixer_changes):
    cfg = dict(TK[name], layers=[copy.deepcopy(TK[name]["layers"][layer])])
    cfg["layers"][0]["mixer"].update(mixer_changes)
    return cfg


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [50, 64, 1000])
def test_stream_read_behind_a_normed_sum(dtype, hidden):
    """A block without norms ahead: the pending result is normed, added to the float32 stream, and the sublayer
    reads the stream itself (rounded into the engine's type; a float32 engine reads it in place)."""
    from inferflux_b200.parts.base import NormedDelta, PartialSums
    from inferflux_b200.parts.block import PostNormBlock
    eps = 3e-6

    class Ctx:
        pass
    Ctx.dtype = dtype
    res, a = _rand((7, hidden), 1, 3.0).to(DEV), _rand((3, 7, hidden), 2).to(DEV)
    w = (1 + _rand((hidden,), 3, 0.2))
    want = res.cpu().double() + plain.rms_norm(a.cpu().double().sum(0), w.double(), eps)
    x = PostNormBlock._read(res, NormedDelta(PartialSums(a), w.to(DEV), eps), Ctx)
    assert x.dtype == dtype and _rel(res, want) < 1e-6 and _rel(x, want) < (1e-6 if dtype == torch.float32 else 4e-3)
    if dtype == torch.float32:
        assert x.data_ptr() == res.data_ptr()
    first = PostNormBlock._read(res, None, Ctx)                                     # the first layer: nothing is pending
    assert _rel(first, want) < (1e-6 if dtype == torch.float32 else 4e-3) and _rel(res, want) < 1e-6


@gpu
def test_embedding_scale_and_banded_rotation():
    from inferflux_b200.kernels import ops
    from inferflux_b200.parts.embedding import TokenEmbedding
    from inferflux_b200.parts.position import RotaryHalf
    for dtype in DTYPES:
        part = TokenEmbedding(dict(vocab=11, hidden=24, weight_name="embed", scale=7.25), "", dtype, DEV)
        table = _rand((11, 24), 1).to(torch.bfloat16)
        part.load({"embed": table.to(dtype).to(DEV)})
        ids = torch.tensor([3, 0, 10, 3], dtype=torch.int32, device=DEV)
        assert _rel(part.forward(ids), table.double()[[3, 0, 10, 3]] * 7.25) < 1e-6
    rot = dict(dims=12, base=3000.0, scaling=dict(factor=6.0, low=1.5, high=5.0, original=40))
    part = RotaryHalf(dict(rotary_dim=12, theta=3000.0, scaling=rot["scaling"]), "", torch.float32, DEV)
    assert _rel(part.inv_freq, plain.frequencies(rot)) < 1e-12
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 123456], dtype=torch.int32, device=DEV)

    class Ctx:
        n_tokens, positions, device = 7, pos, DEV
    cos, sin = part.prepare(Ctx)
    x = _rand((7, 3 * 20), 4).to(DEV)
    want = plain.rotate(x.cpu().double().reshape(7, 3, 20), pos.cpu(), rot).reshape(7, 60)
    ops.rotate_heads(x, 0, 3, 20, cos, sin, ops.ROT_HALF)
    assert _rel(x, want) < 2e-6


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 1), ("B", 2), ("B", 4), ("C", 0)])
def test_state_space_mixer_alone(dtype, name, layer):
    """Portions that start and end inside the convolution's reach (one and two tokens against up to four taps), a
    long portion, single tokens; two groups, a state of more rows than a thread holds, one tap; then the slot
    again, which the next request finds zeroed."""
    cfg = _one_layer(name, layer)
    model, runner, w = _runner_for(cfg, dtype, 30 + layer, tokens=512)
    portions = [21, 1, 2, 1, 1, 10, 150, 1, 1, 2, 16, 1, 40]
    x = _rand((sum(portions), cfg["width"]), 31).to(dtype)
    want, _ = plain.mamba2(x.double(), w, "l0.mix", cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    got = _mixer_in_portions(model, runner, 0, x, portions, dtype)
    assert _rel(got, want) < PTOL[dtype]
    again = _mixer_in_portions(model, runner, 0, x[:9], [2, 7], dtype)
    assert _rel(again, want[:9]) < PTOL[dtype]


@gpu
def test_state_space_state_far_back_shows():
    """A decay close to one: what the first token wrote into the state still carries the result 300 tokens on, in a
    prompt and in decoding, so a state that a portion's start, a slot or a step lost would show."""
    cfg = _one_layer("A", 1)
    _, tensors = tekosun_tensors(cfg, 5)
    tensors["l0.mix.A_log"] = torch.full((3,), -9.0).to(torch.bfloat16)
    model, runner, w = _runner_for(cfg, torch.float32, 5, tensors=tensors)
    x = _rand((300, 64), 6).to(torch.bfloat16).float()
    x[1:] *= 0.05
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    want, _ = plain.mamba2(x.double(), w, "l0.mix", m, eps)
    lost, _ = plain.mamba2(x.double()[1:], w, "l0.mix", m, eps)
    assert _rel(lost[-1], want[-1]) > 0.05                                          # the plain result does rest on token 0
    got = _mixer_in_portions(model, runner, 0, x, [1, 2, 200, 90] + [1] * 7, torch.float32)
    assert _rel(got, want) < PTOL[torch.float32]


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("A", 2), ("B", 0), ("C", 2)])
def test_delta_rule_mixer_alone(dtype, name, layer):
    """Portions and single tokens, heads of 10, 12 and 64, a decay projection whose inner size the tensors give (16
    by default, 5 by configuration); then the slot again."""
    cfg = _one_layer(name, layer)
    model, runner, w = _runner_for(cfg, dtype, 40 + layer, tokens=512)
    assert model.blocks[0].mixer.rank == (5 if name == "B" else 16)
    portions = [150, 1, 1, 2, 64, 7, 1, 33]
    x = _rand((sum(portions), cfg["width"]), 41).to(dtype)
    want, _ = plain.general_delta(x.double(), w, "l0.mix", cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    got = _mixer_in_portions(model, runner, 0, x, portions, dtype)
    assert _rel(got, want) < PTOL[dtype]
    again = _mixer_in_portions(model, runner, 0, x[:10], [10], dtype)
    assert _rel(again, want[:10]) < PTOL[dtype]


@gpu
def test_delta_rule_removal_and_decay_show():
    """With the raw decays and removal rates pushed far up or down the rule becomes plain linear attention (decay 1,
    nothing removed) or forgets (the smallest decay, everything along the key removed): the engine follows both, and
    the first token's key still carries the last result in the first case."""
    cfg = _one_layer("A", 2)
    for w0, ab in ((-30.0, -30.0), (30.0, 30.0)):
        _, tensors = tekosun_tensors(cfg, 7)
        tensors["l0.mix.w0"] = torch.full((24,), w0).to(torch.bfloat16)
        tensors["l0.mix.a.b"] = torch.full((24,), ab).to(torch.bfloat16)
        model, runner, w = _runner_for(cfg, torch.float32, 7, tensors=tensors)
        x = _rand((120, 64), 8).to(torch.bfloat16).float()
        m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
        want, _ = plain.general_delta(x.double(), w, "l0.mix", m, eps)
        got = _mixer_in_portions(model, runner, 0, x, [1, 2, 70, 40] + [1] * 7, torch.float32)
        assert _rel(got, want) < PTOL[torch.float32]
        if w0 < 0:
            r, k, v = (plain_heads(x.double() @ w[f"l0.mix.{n}"].T, 2, 12) for n in ("r", "k", "v"))
            lin = torch.stack([sum((r[119, h] @ k[j, h]) * v[j, h] for j in range(120)) for h in range(2)])
            gate = torch.sigmoid(x.double()[119] @ w["l0.mix.g"].T)
            direct = (plain.unit_rms(lin, eps).reshape(24) * w["l0.mix.norm"] * gate) @ w["l0.mix.o"].T
            assert _rel(want[119], direct) < 1e-6


def plain_heads(y, heads, dim):
    return y.reshape(y.shape[0], heads, dim)


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,vdim,width", [(16, 12, 64), (64, 64, 160)])
def test_attention_edges_with_one_score_that_stands_out(dtype, dim, vdim, width):
    """210 tokens, a window of 40, pages of 16.  Head 0's query is the token's first ``dim`` numbers and the key the
    next ``dim``, nothing rotates; every key carries one large constant in a channel that no query reads, so that the
    norm over the key projection leaves quiet keys quiet.  Each of the last eight tokens gets a query that matches
    the key of one chosen earlier token and no other: the last one inside its window, the first one outside, a page's
    last and first token inside the window, the token just before, the very first token (long gone), one far outside,
    and itself.  A visible target takes the whole weight; a window or a page's edge that is off by one changes the
    result entirely.  The first two of the eight queries come inside a portion, the others as single tokens."""
    n, wn = 210, 40
    mixer = dict(heads=2, kv_heads=1, dim=dim, vdim=vdim, mask=dict(size=wn), scale=1.0)
    cfg = dict(TK["A"], width=width, layers=[dict(type="attention", mixer=mixer, mlp=None)])
    _, tensors = tekosun_tensors(cfg, 21)
    eye = torch.eye(dim)
    tensors["l0.mix.q"] = torch.cat([torch.cat([eye, torch.zeros(dim, width - dim)], 1), _rand((dim, width), 22, 0.05)]).to(torch.bfloat16)
    tensors["l0.mix.k"] = torch.cat([torch.zeros(dim, dim), eye, torch.zeros(dim, width - 2 * dim)], 1).to(torch.bfloat16)
    tensors["l0.mix.q.norm"] = torch.ones(2 * dim).to(torch.bfloat16)
    tensors["l0.mix.k.norm"] = torch.ones(dim).to(torch.bfloat16)
    model, runner, w = _runner_for(cfg, dtype, 21, tensors=tensors)
    x = _rand((n, width), 23, 0.3).to(torch.bfloat16).float()
    x[:, :2 * dim] *= 0.1                                        # quiet queries and keys, but for the chosen pairs
    x[:, 2 * dim - 1] = 4.0                                      # the keys' constant; queries never point there
    x[:, dim - 1] = 0.0
    first_q = n - 8
    targets = [p - off if off is not None else t for p, (off, t) in zip(range(first_q, n), [
        (wn - 1, None), (wn, None), (None, 191), (None, 192), (1, None), (None, 0), (100, None), (0, None)])]
    for q, t in zip(range(first_q, n), targets):
        u = torch.zeros(dim)
        u[(q - first_q) % (dim - 1)] = 1.0                       # a direction of its own for every pair
        x[t, dim:2 * dim - 1] += 4.0 * u[:dim - 1]               # added: one token may be the target of two queries
        x[q, :dim] = 4.0 * u
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    want = plain.attention(x.double(), w, "l0.mix", m, eps, {}, None)
    seen = [True, False, True, True, True, False, False, True]
    for q, t, vis in zip(range(first_q, n), targets, seen):      # the plain result does rest on these single keys
        other = x.clone()
        other[t, dim:2 * dim - 1] = 0.03
        moved = plain.attention(other.double(), w, "l0.mix", m, eps, {}, None)[q]
        assert (_rel(moved, want[q]) > 0.2) == vis, (q, t)
    got = _mixer_in_portions(model, runner, 0, x, [150, 54] + [1] * 6, dtype)
    assert _rel(got, want) < PTOL[dtype]
    wider = dict(m, mask=dict(size=wn + 1))                      # the first invisible target, made visible, would show
    shown = plain.attention(x.double(), w, "l0.mix", wider, eps, {}, None)
    assert _rel(shown[first_q + 1], want[first_q + 1]) > 0.2


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer,mode", [("A", 0, "first"), ("A", 3, "blend"), ("B", 1, None), ("B", 3, None),
                                             ("C", 1, "first"), ("C", 3, "blend"), ("C", 4, "blend")])
def test_attention_mixer_alone(dtype, name, layer, mode):
    """Portions that start and end inside pages, single tokens across page borders and past the window; with and
    without window, rotation, grouped heads and value mixing (the kept values given by hand); a window shorter than
    a page; then the slot and the pages again."""
    cfg = _one_layer(name, layer)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    if mode == "blend":                                          # alone, the layer would be the first: give it one ahead
        cfg["layers"].insert(0, copy.deepcopy(cfg["layers"][0]))
    model, runner, w = _runner_for(cfg, dtype, 30 + layer, tokens=512)
    at = len(cfg["layers"]) - 1
    assert model.blocks[at].mixer.v_mix == mode
    portions = [21, 1, 2, 1, 1, 10, 45, 1, 1, 2, 16, 1, 40]
    x = _rand((sum(portions), cfg["width"]), 31).to(dtype)
    kvw = plain.fill_attention(m)["kv_heads"] * plain.fill_attention(m)["vdim"]
    v_first = _rand((sum(portions), kvw), 32)
    shared = {"v_first": v_first.double().reshape(x.shape[0], -1, plain.fill_attention(m)["vdim"])}
    want = plain.attention(x.double(), w, f"l{at}.mix", m, eps, shared, mode)
    got = _mixer_in_portions(model, runner, at, x, portions, dtype, v_first if mode == "blend" else None)
    assert _rel(got, want) < PTOL[dtype]
    again = _mixer_in_portions(model, runner, at, x[:9], [2, 7], dtype, v_first if mode == "blend" else None)
    assert _rel(again, want[:9]) < PTOL[dtype]
    runner.kv.check()


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,ff,experts,top,shared,scale,rows", [
    (64, 40, 5, 2, 24, 1.7, 3), (64, 40, 5, 2, None, 2.25, 300), (50, 35, 3, 3, 9, 1.0, 70), (50, 18, 3, 1, None, 3.0, 5),
    (128, 48, 12, 3, 64, 2.0, 1), (96, 200, 40, 8, 120, 0.5, 130),
    (128, 48, 12, 3, 64, 2.0, 400)])                                    # bfloat16, 1,200 pairs: the tcgen05 tiles
def test_squared_relu_experts_alone(dtype, hidden, ff, experts, top, shared, scale, rows):
    """Few rows (short tiles) and many (tiles of 64 and of 256), one expert a token and every expert, with and without
    the shared expert; the weights are softmax scores over all experts, renormed over the chosen and scaled.  Rows
    whose choice rests on a close call are left out of the comparison."""
    from inferflux_b200.parts.feed_forward import RoutedExperts
    params = dict(name="mlp", hidden=hidden, intermediate=ff, experts=experts, top=top, activation="relu2", route="all",
                  scale=scale, router_bias=False, shared=shared)
    part = RoutedExperts(params, "l0", dtype, DEV)
    w = {s.name: (_rand(s.shape, 50 + i, 0.5 if "router" in s.name else 0.15)).to(torch.bfloat16).float()
         for i, s in enumerate(RoutedExperts.weight_specs(params, "l0"))}
    assert ("l0.mlp.shared.up" in w) == bool(shared) and "l0.mlp.router.b" not in w and "l0.mlp.e0.gate" not in w
    part.load({k: v.to(dtype).to(DEV) for k, v in w.items()})
    x = _rand((rows, hidden), 51).to(dtype)
    w64 = {k: v.double() for k, v in w.items()}
    mlp = dict(router=dict(experts=experts, top=top, scale=scale), **({"shared": dict(ff=shared)} if shared else {}))
    want = plain.moe(x.double(), w64, "l0.mlp", mlp)
    srt = torch.sort(x.double() @ w64["l0.mlp.router"].T, dim=-1, descending=True).values
    clear = torch.ones(rows, dtype=torch.bool) if top == experts else (srt[:, top - 1] - srt[:, top]) > 0.05
    got = _dense(part.forward(x.to(DEV), None)).cpu()
    assert clear.sum() >= rows * 0.7 and _rel(got[clear], want[clear]) < PTOL[dtype]


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
    cfg = _for_dtype(TK[name], dtype)
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
    from inferflux_b200.parts.base import NormedDelta
    from inferflux_b200.parts.norm import normed_sum
    cfg = TK["A"]
    model, runner, w = _runner_for(cfg, torch.float32, 9)
    toks = random_tokens(cfg["vocab"], 60, 4)
    want = []
    plain.forward(cfg, w, toks, want)
    seen = []
    for block in model.blocks:
        def watched(residual, delta, ctx, run, inner=block.forward):
            out = inner(residual, delta, ctx, run)
            stream = residual.clone()
            if isinstance(out, NormedDelta):
                normed_sum(stream, out, None, None)
            seen.append(stream)
            return out
        block.forward = watched
    runner.step([StepEntry("s", toks, [0])])
    assert len(seen) == len(want) and all(_rel(g, x) < 2e-5 for g, x in zip(seen, want))


@gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_batches_of_unequal_requests_and_reused_slots(dtype, name):
    """Four requests of unequal length, portions beside single tokens, against each alone; then four more in
    the slots and pages the first ones gave back."""
    from inferflux_b200.engine import StepEntry
    cfg = _for_dtype(TK[name], dtype)
    model, runner, w = _runner_for(cfg, dtype, 41, tokens=4 * 128)
    rng = random.Random(3)
    for round_ in range(2):
        lens = [97, 5, 64, 33] if round_ == 0 else [31, 120, 2, 70]
        reqs = {f"r{round_}{i}": _steady_tokens(cfg, w, n, 500 + 100 * round_ + 10 * i) for i, n in enumerate(lens)}
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
    """300 tokens at once, then 200 one by one through the captured graph: the windows (7 to 33 tokens) pass over
    decoded tokens many times, pages behind them go back to the pool and come again, the states go on."""
    cfg = TK[name]
    model, runner, w = _runner_for(cfg, torch.float32, 51, tokens=512)
    toks = random_tokens(cfg["vocab"], 500, 52)
    want = plain.forward(cfg, w, toks)
    got = _logits_in_steps(runner, "d", toks, [300] + [1] * 200)
    assert runner.graph_replays >= 190 and _rel(got, want) < 5e-5
    assert runner.kv.pools[-1].reuses > 0


# ------------------------------------------------------------------ GPU: bin/trace_run and Engine.generate
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_trace_replay_mixed_with_page_and_slot_reuse(name, dtype):
    """The command-line replay: the config.json picks the architecture; four state slots, a pool of the four
    longest requests; every request twice, so pages and slots turn over."""
    from helpers import load_plain_folder as load_plain
    cfg = _for_dtype(TK[name], dtype)
    folder = make_tekosun_folder(cfg, seed=60 + ord(name))
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
    cfg = TK["A"]
    folder = make_tekosun_folder(cfg, seed=71)
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
