"""Shared test helpers: the tiny configurations, model folders in temporary
directories, a driver for bin/trace_run, tolerances."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=512,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256,
              use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=96, num_hidden_layers=3,
              num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=1000,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512,
              use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
# head_dim * heads != hidden, 5 query heads per kv head, an odd vocabulary
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=80, num_hidden_layers=2,
              num_attention_heads=10, num_key_value_heads=2, head_dim=48, intermediate_size=136, vocab_size=777,
              rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=384,
              use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
# head_dim 64: the size the tensor-core attention kernels take; 3 query heads per kv head, a window
TINY_D = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=120, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=200, vocab_size=600,
              rope_theta=200000.0, rms_norm_eps=2e-6, tie_word_embeddings=True, max_position_embeddings=400,
              use_sliding_window=True, sliding_window=70, max_window_layers=1, hidden_act="silu",
              torch_dtype="bfloat16")
# B's sizes with a window of 40 keys on all layers but the first: two cache groups, pages given back behind the window
TINY_E = dict(TINY_B, use_sliding_window=True, sliding_window=40, max_window_layers=1)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}

# Largest |engine - plain| allowed, as a fraction of the largest |plain logit|.
# float32: a few hundred float32 roundings; bfloat16: 8-bit mantissas through every layer.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def make_model_folder(cfg: dict, seed: int, folder: Optional[str] = None, sharpen: float = 6.0,
                      vector_dtype=None) -> str:
    """Write a random model folder.  ``sharpen`` multiplies the q and k
    projection weights so that attention is peaked: with N(0, 0.02) weights it
    is nearly uniform and one wrong key among many would hide below the
    bfloat16 tolerance."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine.model import Model
    from inferflux_b200.weights.random_init import random_tensors
    from inferflux_b200.weights.safetensors_io import write_safetensors
    folder = folder or tempfile.mkdtemp(prefix="ifx_model_")
    config = Qwen2Config.from_dict(cfg)
    config.save(folder)
    specs = Model(build_spec(config), torch.float32, "cpu").weight_specs()
    tensors = random_tensors(specs, seed, torch.bfloat16, vector_dtype, "cpu")
    if sharpen != 1.0:
        for name in tensors:
            if name.endswith(("q_proj.weight", "k_proj.weight")):
                tensors[name] = (tensors[name].float() * sharpen).to(tensors[name].dtype)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class TraceProcess:
    """A running bin/trace_run: send steps, wait for ``done``, read logits."""

    def __init__(self, model_dir: Optional[str], dtype: str, max_tokens: int, extra: Sequence[str] = ()):
        self.out = tempfile.mkdtemp(prefix="ifx_trace_")
        self.step_no = 0
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), *(["--model", model_dir] if model_dir else []),
               "--dtype", dtype, "--out", self.out, "--max-tokens", str(max_tokens), *extra]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

    def step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        """entries: dicts with id, tokens, want.  Returns [wanted, vocab] or None."""
        n = self.step_no
        self.step_no += 1
        self.proc.stdin.write(json.dumps({"step": n, "entries": list(entries), "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {n}":
            rc = self.proc.poll()
            raise RuntimeError(f"trace_run answered {line!r} to step {n} (exit code {rc})")
        wanted = sum(len(e.get("want", [])) for e in entries)
        if not wanted:
            return None
        arr = np.fromfile(os.path.join(self.out, f"{n}.f32"), dtype="<f4")
        return arr.reshape(wanted, -1)

    def stats(self) -> dict:
        """The counters of the cache pools and of the step function."""
        self.proc.stdin.write(json.dumps({"stats": True}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if not line.startswith("stats "):
            raise RuntimeError(f"trace_run answered {line!r} to a request for its counters")
        return json.loads(line[len("stats "):])

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        return rc


def rel_err(got, ref) -> float:
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


# ------------------------------------------------------------------ Kunonex
def _kx_attn(heads, dim, vdim, kv_rank, q_rank, scale, ff=None):
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale),
                mlp=dict(kind="dense", ff=ff) if ff else None)


def _kx_gru(width, ff=None):
    return dict(type="mingru", mixer=dict(width=width), mlp=dict(kind="dense", ff=ff) if ff else None)


# Tiny Kunonex configurations that differ in every size and option: dim != vdim, q_rank != heads * dim, ranks
# that are no multiple of 32, one head, a layer without feed-forward, a loop over a recurrent layer (every pass
# has a state of its own), a loop that starts at layer 0, a loop that runs once, no loop, other constants.
KX_A = dict(architecture="Kunonex", width=64, vocab=300, norm=dict(eps=1e-5), logit_scale=0.25,
            layers=[_kx_attn(3, 24, 16, 40, 56, 0.31, ff=96), _kx_gru(64, ff=80), _kx_attn(1, 32, 48, 24, 20, 0.2),
                    _kx_gru(48, ff=72)],
            loop=dict(start=1, stop=3, times=2))
KX_B = dict(architecture="Kunonex", width=96, vocab=411, norm=dict(eps=3e-6), logit_scale=1.5,
            layers=[_kx_gru(200, ff=136), _kx_attn(5, 16, 8, 72, 32, 0.5, ff=100), _kx_attn(2, 40, 40, 96, 104, 0.11, ff=64)],
            loop=dict(start=0, stop=2, times=3))
KX_C = dict(architecture="Kunonex", width=40, vocab=97, norm=dict(eps=1e-6), logit_scale=1.0,
            layers=[_kx_attn(2, 8, 12, 16, 16, 0.7, ff=64), _kx_gru(24), _kx_attn(4, 12, 4, 33, 28, 0.4, ff=48)], loop=None)
KX_D = dict(KX_C, loop=dict(start=2, stop=3, times=1), logit_scale=2.0)
# heads of 128: in bfloat16 prompt portions are attended per head by the tcgen05 prompt kernel, single tokens over the latents
KX_E = dict(architecture="Kunonex", width=128, vocab=200, norm=dict(eps=1e-6), logit_scale=0.7,
            layers=[_kx_attn(2, 128, 128, 48, 64, 0.09, ff=160), _kx_gru(128, ff=96), _kx_attn(3, 128, 128, 64, 40, 0.09)],
            loop=dict(start=0, stop=1, times=2))
# sizes that are no multiple of 4 or 8 anywhere: the kernels' plain (not vectorised) paths and the library products
KX_F = dict(architecture="Kunonex", width=50, vocab=77, norm=dict(eps=2e-6), logit_scale=0.9,
            layers=[_kx_gru(30, ff=45), _kx_attn(2, 10, 6, 12, 14, 0.3, ff=35), _kx_attn(3, 6, 10, 9, 11, 0.4)],
            loop=dict(start=1, stop=2, times=2))
KX = {"A": KX_A, "B": KX_B, "C": KX_C, "D": KX_D, "E": KX_E, "F": KX_F}


def kunonex_tensors(cfg: dict, seed: int, sharpen: float = 6.0, lively: float = 12.0):
    """Random tensors (bfloat16 matrices) for a Kunonex configuration.  ``sharpen`` multiplies the query
    up-projections so that attention is peaked on single keys, wherever they lie (with N(0, 0.02) weights it is
    nearly uniform and a lost key among hundreds would hide below the bfloat16 tolerance); ``lively`` multiplies
    the recurrence's gate projections so that its gates leave the middle and its state matters."""
    from inferflux_b200.config import load_config
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine.model import Model
    from inferflux_b200.weights.random_init import random_tensors
    config = load_config(dict(cfg))
    specs = Model(build_spec(config), torch.float32, "cpu").weight_specs()
    tensors = random_tensors(specs, seed, torch.bfloat16, None, "cpu")
    for name in tensors:
        f = sharpen if name.endswith((".mix.uq", ".mix.uk")) else lively if name.endswith((".mix.z", ".mix.x", ".mix.g")) else 1.0
        if name.endswith((".mix.uv", ".mix.o", ".mlp.down", ".mlp.up", ".mix.dq", ".mix.dkv")):
            f = 4.0
        if f != 1.0:
            tensors[name] = (tensors[name].float() * f).to(tensors[name].dtype)
    return config, tensors


def make_kunonex_folder(cfg: dict, seed: int, folder: Optional[str] = None, **kw) -> str:
    from inferflux_b200.weights.safetensors_io import write_safetensors
    folder = folder or tempfile.mkdtemp(prefix="ifx_kx_")
    config, tensors = kunonex_tensors(cfg, seed, **kw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def load_kunonex_plain(folder: str):
    """(config dict, tensors in float64) of a model folder, for the plain implementation."""
    from inferflux_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    sf = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return cfg, {n: sf.tensor(n).double() for n in sf.names()}


# ------------------------------------------------------------------ Pemorax
def _px_left(heads, kv_heads, dim, vdim, conv=None, mask=None, rot=None, scale=None, softcap=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim)
    for k, v in (("conv", conv), ("mask", mask), ("rot", rot), ("scale", scale), ("softcap", softcap)):
        if v is not None:
            m[k] = v
    return m


def _px_right(heads, dim, vdim, decay, rot=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=decay)
    if rot is not None:
        m["rot"] = rot
    return m


def _px_layer(left, right, mlp):
    return dict(type="parallel", mixer=dict(left=left, right=right), mlp=mlp)


_YARN = dict(factor=4.0, original=64, fast=16.0, slow=2.0)
_MOE = lambda ff, experts, top: dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))
# Tiny Pemorax configurations that differ in every size and option.  A: dim != vdim on both sides, part of a head
# rotates, scaled frequencies, a window of 20 that keeps 3, four taps, a decay of 1, experts 2 of 5, a layer
# without feed-forward whose attention has no convolution, no window, no rotation and no cap.
PX_A = dict(architecture="Pemorax", width=64, vocab=300, norm=dict(eps=1e-5), layers=[
    _px_layer(_px_left(4, 2, 16, 24, conv=4, mask=dict(size=20, keep_first=3), rot=dict(dims=8, base=10000.0, scaling=_YARN),
                       scale=0.3, softcap=8.0),
              _px_right(3, 12, 20, [0.9, 0.97, 1.0], rot=dict(dims=12, base=5000.0)), dict(kind="dense", ff=96)),
    _px_layer(_px_left(2, 2, 32, 32, conv=2, mask=dict(size=33, keep_first=0), rot=dict(dims=32, base=300.0)),
              _px_right(1, 16, 8, [0.95], rot=dict(dims=4, base=100.0)), _MOE(40, 5, 2)),
    _px_layer(_px_left(3, 1, 8, 4), _px_right(2, 8, 8, [0.5, 0.99]), None)])
# B: sizes that are no multiple of 4 or 8 anywhere, a window shorter than a page, every expert chosen, one expert of
# three, convolutions of eight taps and of one
PX_B = dict(architecture="Pemorax", width=50, vocab=77, norm=dict(eps=3e-6), layers=[
    _px_layer(_px_left(3, 3, 10, 6, conv=3, mask=dict(size=7, keep_first=1), rot=dict(dims=6, base=50.0), softcap=3.0),
              _px_right(2, 6, 10, [0.8, 0.999], rot=dict(dims=6, base=1000.0)), _MOE(35, 3, 3)),
    _px_layer(_px_left(5, 1, 6, 10, conv=8, mask=dict(size=40, keep_first=18), rot=dict(dims=2, base=20.0)),
              _px_right(5, 10, 6, [0.7, 0.9, 0.95, 0.99, 0.995], rot=dict(dims=10, base=7.0)), _MOE(18, 3, 1)),
    _px_layer(_px_left(1, 1, 14, 14, conv=1, mask=dict(size=64, keep_first=64)), _px_right(1, 14, 2, [0.96]), dict(kind="dense", ff=45))])
# C: heads of 64 and of 128 (the sizes tensor-core kernels take), windows longer than several pages, many experts
PX_C = dict(architecture="Pemorax", width=128, vocab=200, norm=dict(eps=1e-6), layers=[
    _px_layer(_px_left(4, 2, 64, 64, conv=4, mask=dict(size=70, keep_first=5), rot=dict(dims=64, base=200000.0, scaling=_YARN),
                       softcap=30.0),
              _px_right(2, 64, 64, [0.97, 0.999], rot=dict(dims=64, base=7e5)), _MOE(48, 12, 3)),
    _px_layer(_px_left(2, 1, 128, 128, conv=2, mask=dict(size=100, keep_first=17), rot=dict(dims=64, base=10000.0), softcap=20.0),
              _px_right(1, 128, 128, [0.99], rot=dict(dims=32, base=1e4)), dict(kind="dense", ff=160))])
PX = {"A": PX_A, "B": PX_B, "C": PX_C}


def pemorax_tensors(cfg: dict, seed: int, sharpen: float = 8.0):
    """Random tensors (bfloat16 matrices) for a Pemorax configuration.  ``sharpen`` multiplies the attention's
    query and key projections so that the softmax is peaked on single keys wherever they lie (with N(0, 0.02)
    weights it is nearly uniform, and a lost key among hundreds or a missing sink would hide below the bfloat16
    tolerance); the other projections are enlarged so that every branch carries weight in the sums."""
    from inferflux_b200.config import load_config
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine.model import Model
    from inferflux_b200.weights.random_init import random_tensors
    config = load_config(json.loads(json.dumps(cfg)))
    specs = Model(build_spec(config), torch.float32, "cpu").weight_specs()
    tensors = random_tensors(specs, seed, torch.bfloat16, None, "cpu")
    for name in tensors:
        f = 1.0
        if name.endswith((".left.q", ".left.k")):
            f = sharpen
        elif name.endswith((".right.q", ".right.k", ".right.v", ".left.v", ".g", ".o", ".up", ".down", ".gate")):
            f = 4.0
        elif name == "embed":
            f = 20.0
        if f != 1.0:
            tensors[name] = (tensors[name].float() * f).to(tensors[name].dtype)
    return config, tensors


def make_pemorax_folder(cfg: dict, seed: int, folder: Optional[str] = None, **kw) -> str:
    from inferflux_b200.weights.safetensors_io import write_safetensors
    folder = folder or tempfile.mkdtemp(prefix="ifx_px_")
    config, tensors = pemorax_tensors(cfg, seed, **kw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


load_plain_folder = load_kunonex_plain        # (config dict, float64 tensors) of any model folder


# ------------------------------------------------------------------ Tekosun
_BANDS = dict(factor=4.0, low=1.0, high=8.0, original=64)
_TK_MOE = lambda ff, experts, top, scale=None, shared=None: dict(
    kind="moe", expert=dict(ff=ff), router={k: v for k, v in (("experts", experts), ("top", top), ("scale", scale)) if v is not None},
    **({"shared": dict(ff=shared)} if shared else {}))
# Tiny Tekosun configurations that differ in every size, option and order of layers.  A: attention first (it keeps its
# values for the later one, whose heads and key size differ), part of a head rotates by banded frequencies, windows of
# 20 and 33, a layer without feed-forward, one state-space group, a shared expert here and none there.
TK_A = dict(architecture="Tekosun", width=64, vocab=300, norm=dict(eps=1e-5), embedding=dict(scale=3.0), layers=[
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.6, v_mix=True, mask=dict(size=20),
                                      rot=dict(dims=8, base=10000.0, scaling=_BANDS)), mlp=_TK_MOE(40, 5, 2, 1.7, 24)),
    dict(type="mamba2", mixer=dict(heads=3, vdim=12, state=8, groups=1, conv=4, norm_groups=1), mlp=None),
    dict(type="general_delta", mixer=dict(heads=2, dim=12), mlp=_TK_MOE(32, 4, 1, 0.5)),
    dict(type="attention", mixer=dict(heads=2, kv_heads=2, dim=32, vdim=24, scale=0.4, v_mix=True, mask=dict(size=33),
                                      rot=dict(dims=32, base=300.0)), mlp=_TK_MOE(40, 5, 2, 2.25, 56))])
# B: sizes that are no multiple of 4 or 8 anywhere, two state-space groups and two norm groups, two taps, an attention
# without window, rotation, value mixing or key/value head count, a window shorter than a page, every expert chosen,
# no embedding scale, a decay projection of five
TK_B = dict(architecture="Tekosun", width=50, vocab=77, norm=dict(eps=3e-6), layers=[
    dict(type="general_delta", mixer=dict(heads=3, dim=10, decay_rank=5), mlp=_TK_MOE(35, 3, 3, shared=9)),
    dict(type="attention", mixer=dict(heads=3, dim=10, scale=0.9), mlp=None),
    dict(type="mamba2", mixer=dict(heads=4, vdim=5, state=6, groups=2, conv=2, norm_groups=2), mlp=_TK_MOE(18, 3, 1, 3.0)),
    dict(type="attention", mixer=dict(heads=5, kv_heads=1, dim=6, vdim=10, scale=1.2, mask=dict(size=7), rot=dict(dims=2, base=20.0)),
         mlp=_TK_MOE(18, 3, 2, shared=30)),
    dict(type="mamba2", mixer=dict(heads=2, vdim=7, state=3, conv=1), mlp=None)])
# C: heads of 64 (the sizes tensor-core kernels take), a state of 64 and of more rows than a thread holds, a window
# longer than several pages, many experts, three attention layers of which two blend, four norm groups
TK_C = dict(architecture="Tekosun", width=128, vocab=200, norm=dict(eps=1e-6), embedding=dict(scale=11.0), layers=[
    dict(type="mamba2", mixer=dict(heads=4, vdim=32, state=64, groups=2, conv=4, norm_groups=4), mlp=_TK_MOE(48, 12, 3, 2.0, 64)),
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.25, v_mix=True, mask=dict(size=70),
                                      rot=dict(dims=64, base=200000.0, scaling=_BANDS)), mlp=_TK_MOE(48, 12, 3, 2.0, 64)),
    dict(type="general_delta", mixer=dict(heads=2, dim=64), mlp=None),
    dict(type="attention", mixer=dict(heads=2, kv_heads=2, dim=32, vdim=64, scale=0.3, v_mix=True, rot=dict(dims=16, base=1e4)),
         mlp=_TK_MOE(24, 6, 2, 1.0)),
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.25, v_mix=True, mask=dict(size=70),
                                      rot=dict(dims=64, base=200000.0, scaling=_BANDS)), mlp=None)])
TK = {"A": TK_A, "B": TK_B, "C": TK_C}


def tekosun_tensors(cfg: dict, seed: int, sharpen: float = 1.0):
    """Random tensors (bfloat16 matrices) for a Tekosun configuration.  Queries and keys are normed, so how peaked the
    softmax is lies with the configuration's ``scale``; ``sharpen`` multiplies the query norm's weight on top.  The
    projections that feed the recurrences are enlarged so that states carry weight, and the state-space decays are
    slowed (``A_log`` lowered) so that a state lost many tokens back would show."""
    from inferflux_b200.config import load_config
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine.model import Model
    from inferflux_b200.weights.random_init import random_tensors
    config = load_config(json.loads(json.dumps(cfg)))
    specs = Model(build_spec(config), torch.float32, "cpu").weight_specs()
    tensors = random_tensors(specs, seed, torch.bfloat16, None, "cpu")
    for name in tensors:
        f, add = 1.0, 0.0
        if name.endswith(".q.norm"):
            f = sharpen
        elif name.endswith((".mix.in", ".mix.r", ".mix.k", ".mix.v", ".mix.a", ".mix.g", ".mix.w1", ".up", ".down", ".mix.o")):
            f = 5.0
        elif name.endswith(".A_log"):
            add = -2.0
        elif name == "embed":
            f = 20.0
        if f != 1.0 or add:
            tensors[name] = (tensors[name].float() * f + add).to(tensors[name].dtype)
    return config, tensors


def make_tekosun_folder(cfg: dict, seed: int, folder: Optional[str] = None, **kw) -> str:
    from inferflux_b200.weights.safetensors_io import write_safetensors
    folder = folder or tempfile.mkdtemp(prefix="ifx_tk_")
    config, tensors = tekosun_tensors(cfg, seed, **kw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


# ------------------------------------------------------------------ Malazen
def _ml_left(heads, dim, kv_heads=None, vdim=None, scale=None, q_temp=None):
    m = dict(heads=heads, dim=dim)
    for k, v in (("kv_heads", kv_heads), ("vdim", vdim), ("scale", scale), ("q_temp", q_temp)):
        if v is not None:
            m[k] = v
    return m


def _ml_parallel(left, right, mlp=None, left_scale=None, right_scale=None):
    mixer = dict(left=left, right=right)
    if left_scale is not None:
        mixer.update(left_scale=left_scale, right_scale=right_scale)
    return dict(type="parallel", mixer=mixer, mlp=mlp)


def _ml_latent(heads, dim, vdim, kv_rank, rot_dim=None, mask=None, rot=None, scale=None, mlp=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank)
    for k, v in (("rot_dim", rot_dim), ("mask", mask), ("rot", rot), ("scale", scale)):
        if v is not None:
            m[k] = v
    return dict(type="latent_attention", mixer=m, mlp=mlp)


_ML_FF = lambda ff, limit: dict(kind="dense", ff=ff, limit=limit)
# Tiny Malazen configurations that differ in every size, option and order of layers.  A: four norm groups; key, value
# and decay sizes all different; a rotated part longer than the plain one with stretched frequencies; a window of 20; a
# loop from layer 0 that runs three times; a layer without feed-forward.
ML_A = dict(architecture="Malazen", width=64, vocab=300, norm=dict(eps=1e-5, groups=4), layers=[
    _ml_parallel(_ml_left(4, 16, kv_heads=2, vdim=24, scale=0.3, q_temp=dict(coef=0.7, every=8)), dict(heads=3, dim=12, vdim=20, tau=4.0),
                 _ML_FF(96, 2.0), 0.8, 1.3),
    _ml_latent(3, 8, 20, 24, rot_dim=12, mask=dict(size=20), rot=dict(dims=12, base=1000.0, scaling=_YARN), scale=0.4, mlp=_ML_FF(72, 1.0)),
    _ml_parallel(_ml_left(2, 32, kv_heads=1, scale=0.2, q_temp=dict(coef=0.25, every=30)), dict(heads=1, dim=16, vdim=8, tau=9.0), None, 1.5, 0.5)],
    loop=dict(start=0, stop=2, times=3))
# B: sizes that are no multiple of 4 or 8 anywhere, one norm group, a window shorter than a page, a latent layer without
# rotated part and without window, a temperature that steps at every token and none at all, as many key/value heads
# as heads, factors left out, no loop
ML_B = dict(architecture="Malazen", width=50, vocab=77, norm=dict(eps=3e-6), layers=[
    _ml_latent(2, 10, 7, 9, rot_dim=6, mask=dict(size=7), rot=dict(dims=6, base=50.0), scale=0.9, mlp=_ML_FF(35, 0.7)),
    _ml_parallel(_ml_left(3, 10, vdim=6, q_temp=dict(coef=1.5, every=1)), dict(heads=2, dim=6, vdim=10, tau=1.0), _ML_FF(45, 3.0)),
    _ml_latent(5, 6, 10, 13, mlp=None),
    _ml_parallel(_ml_left(5, 6, kv_heads=1, vdim=10, scale=0.5), dict(heads=5, dim=10, tau=30.0), _ML_FF(18, 1.2), 1.0, 2.0)])
# C: heads of 64 (the size tensor-core kernels take), a latent row of 64, windows longer than several pages, eight norm
# groups, a loop over a single layer, a loop that ends with the last layer
ML_C = dict(architecture="Malazen", width=128, vocab=200, norm=dict(eps=1e-6, groups=8), layers=[
    _ml_latent(4, 32, 32, 48, rot_dim=16, mask=dict(size=70), rot=dict(dims=16, base=200000.0, scaling=_YARN), scale=0.15, mlp=_ML_FF(160, 1.5)),
    _ml_parallel(_ml_left(4, 64, kv_heads=2, vdim=64, scale=0.125, q_temp=dict(coef=0.5, every=16)), dict(heads=2, dim=64, vdim=64, tau=12.0),
                 _ML_FF(96, 2.5), 1.1, 0.7),
    _ml_latent(2, 64, 64, 120, rot_dim=8, mask=dict(size=100), rot=dict(dims=8, base=1e4), scale=0.1, mlp=_ML_FF(64, 1.0))],
    loop=dict(start=2, stop=3, times=2))
ML = {"A": ML_A, "B": ML_B, "C": ML_C}


def malazen_tensors(cfg: dict, seed: int, sharpen: float = 8.0):
    """Random tensors (bfloat16 matrices) for a Malazen configuration.  ``sharpen`` multiplies the attentions' query
    and key projections so that the softmax is peaked on single keys wherever they lie (with N(0, 0.02) weights it is
    nearly uniform, and a lost key among hundreds or a missing sink would hide below the bfloat16 tolerance); the
    other projections are enlarged so that every branch carries weight in the sums, and the decays' biases are raised
    so that a state lost many tokens back would show."""
    from inferflux_b200.config import load_config
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine.model import Model
    from inferflux_b200.weights.random_init import random_tensors
    config = load_config(json.loads(json.dumps(cfg)))
    specs = Model(build_spec(config), torch.float32, "cpu").weight_specs()
    tensors = random_tensors(specs, seed, torch.bfloat16, None, "cpu")
    for name in tensors:
        f, add = 1.0, 0.0
        if name.endswith((".left.q", ".left.k", ".mix.q", ".mix.uk", ".mix.dkv")):
            f = sharpen
        elif name.endswith((".right.q", ".right.k", ".right.v", ".left.v", ".g", ".o", ".up", ".down", ".gate", ".uv", ".a1")):
            f = 4.0
        elif name.endswith(".a2.b"):
            add = 2.0
        elif name == "embed":
            f = 20.0
        if f != 1.0 or add:
            tensors[name] = (tensors[name].float() * f + add).to(tensors[name].dtype)
    return config, tensors


def make_malazen_folder(cfg: dict, seed: int, folder: Optional[str] = None, **kw) -> str:
    from inferflux_b200.weights.safetensors_io import write_safetensors
    folder = folder or tempfile.mkdtemp(prefix="ifx_ml_")
    config, tensors = malazen_tensors(cfg, seed, **kw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder
