"""``window_attention``: grouped-query attention with the options of newer
decoder designs, each a parameter:

  q, k, v (and a gate g) = one stacked projection of the normed input, float32 sums
  ``conv`` taps          a short causal convolution over time on every channel of q, k and v, straight after
                         the projection: y_t = sum_j w[:, j] u_(t - taps + 1 + j), with u = 0 ahead of the first token
  ``qk_norm``            all of a token's query columns (heads side by side) are divided by their common root
                         mean square and multiplied by a weight of that size; the key columns likewise; ahead
                         of the rotation
  ``v_norm``             every value head is divided by its own root mean square (no weight); cached so
  ``v_mix``              ``first``: this layer's (normed) values are kept for the step's later layers;
                         ``blend``: v <- (1 - lambda) v + lambda v_first with the kept values of the same token
                         and lambda a stored number; the blended values are what is cached
  rotation               of the first ``rot_dims`` dimensions of every query and key head by the layer's
                         position table, pairs ``interleaved`` (2i, 2i+1) or in ``half``s (i, i + rot_dims/2)
  scores                 s = (q . k) * scale, then ``softcap`` * tanh(s / softcap) if given
  visibility             key j for the query at p: j <= p and (p - j < window or j < keep_first); no window
                         = all earlier keys.  Kept tokens keep their own positions.
  ``sink``               one more term of score 0 and no value in the denominator:
                         p_j = exp(s_j) / (1 + sum exp(s_j))
  ``gate``               the heads' results times sigmoid(g), element by element, ahead of the output projection
  ``bias``               q, k, v and the output projection have a bias each, added in the projection
  ``q_temp``             {coef, every}: the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
  ``distance_toll``      the score of key j for the query at p loses r1_h * ln(1 + r2_h * (p - j)), with two stored
                         numbers per head (after the cap, if there is one)

Keys are ``dim`` wide, values ``vdim``.  Keys (rotated) and values live in the paged cache; the last
``taps - 1`` projected rows of a sequence live in its state slot, so a prompt may be cut anywhere.  Scores,
softmax and the gate are float32 in either engine type.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import KVNeed, Part, RunInfo, StateNeed
from .linear import Linear

QUERY_TILE = 16     # tokens per query tile of the plain attention kernel
CHUNK_TILE = 64     # tokens per query tile of the tensor-core kernel for prompt portions
PORTION_MIN = 8     # an entry with fewer new tokens than this is run token by token by the kernel for single tokens


@dataclass
class QueryTiles:
    """How the attention kernels see the step, and the entry of every row: int32 device tensors.  ``single_*``: one
    (entry, place in the entry) per token of the entries with fewer than PORTION_MIN new tokens (decoded tokens
    among them); ``dec_entry``: the entries that bring exactly one token, and ``short_*``: the tokens of the other
    entries below PORTION_MIN (the two together are ``single_*`` again, for mixers whose single tokens take the split
    tensor-core kernel); ``tile_*`` and ``chunk_*``: the other entries cut into tiles of QUERY_TILE and of CHUNK_TILE
    tokens."""

    single_entry: torch.Tensor
    single_q0: torch.Tensor
    n_single: int
    tile_entry: torch.Tensor
    tile_q0: torch.Tensor
    n_tiles: int
    chunk_entry: torch.Tensor
    chunk_q0: torch.Tensor
    n_chunk: int
    row_entry: torch.Tensor
    dec_entry: torch.Tensor = None
    n_dec: int = 0
    short_entry: torch.Tensor = None
    short_q0: torch.Tensor = None
    n_short: int = 0


def describe_query_tiles(layout, put) -> QueryTiles:
    single_entry, single_q0, tile_entry, tile_q0, chunk_entry, chunk_q0 = [], [], [], [], [], []
    dec_entry, short_entry, short_q0 = [], [], []
    for i in range(layout.n_entries):
        n = int(layout.q_len[i])
        if n < PORTION_MIN:
            for q0 in range(n):
                single_entry.append(i), single_q0.append(q0)
                if n > 1:
                    short_entry.append(i), short_q0.append(q0)
            if n == 1:
                dec_entry.append(i)
            continue
        for q0 in range(0, n, QUERY_TILE):
            tile_entry.append(i), tile_q0.append(q0)
        for q0 in range(0, n, CHUNK_TILE):
            chunk_entry.append(i), chunk_q0.append(q0)
    rows = np.repeat(np.arange(layout.n_entries), layout.q_len[:layout.n_entries])
    return QueryTiles(put(single_entry), put(single_q0), len(single_entry), put(tile_entry), put(tile_q0), len(tile_entry),
                      put(chunk_entry), put(chunk_q0), len(chunk_entry), put(rows), put(dec_entry), len(dec_entry),
                      put(short_entry), put(short_q0), len(short_entry))


class WindowAttention(Part):
    """params: ``hidden``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps, 0 = none), ``rot_dims``,
    ``rot_layout`` (``interleaved`` or ``half``), ``scale`` (None = ``dim^-1/2``), ``softcap`` (None = none),
    ``window`` (None = all keys), ``keep_first``, ``sink``, ``gate``, ``qk_norm``, ``v_norm``, ``v_mix`` (None,
    ``first`` or ``blend``), ``eps`` (of these norms), ``bias``, ``q_temp``, ``distance_toll``, ``name``.  Tensors
    ``<prefix>.<name>.{q,k,v,g,o}``, ``<prefix>.<name>.{q,k,v,o}.b``, ``<prefix>.<name>.{r1,r2}`` ``[heads]``,
    ``<prefix>.<name>.{q,k,v}.conv`` ``[channels, taps]``, ``<prefix>.<name>.{q,k}.norm`` and ``<prefix>.<name>.vmix``
    (one number; stored but unused in the ``first`` layer).
    State: ``conv_tail`` float32 ``[taps - 1, channels of q, k and v]``.
    Position: a pair ``(cos, sin)`` of float32 ``[N, rot_dims / 2]`` tensors."""

    family = "mixer"
    describe_key = "query_tiles"
    #: Switch for tests and measurements: prompt portions of a bfloat16 engine on the tensor-core kernel.
    TENSOR_CORES = True

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden = int(p["hidden"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.taps = int(p.get("conv") or 0)
        self.rot_dims = int(p.get("rot_dims") or 0)
        self.layout = ops.ROT_INTERLEAVED if p.get("rot_layout", "half") == "interleaved" else ops.ROT_HALF
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dim)
        self.softcap = float(p.get("softcap") or 0.0)
        self.window = int(p.get("window") or 0)
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.sink, self.gate = bool(p.get("sink")), bool(p.get("gate"))
        self.qk_norm, self.v_norm, self.v_mix = bool(p.get("qk_norm")), bool(p.get("v_norm")), p.get("v_mix") or None
        self.eps = float(p.get("eps") or 0.0)
        self.bias = bool(p.get("bias"))
        qt = p.get("q_temp") or None
        self.q_temp = (float(qt["coef"]), int(qt["every"])) if qt else None
        if self.q_temp and self.q_temp[1] < 1:
            raise ValueError("window_attention: q_temp.every must be at least 1")
        self.distance_toll = bool(p.get("distance_toll"))
        self.toll = None
        if self.v_mix not in (None, "first", "blend"):
            raise ValueError(f"v_mix {self.v_mix!r} is not one of None, 'first', 'blend'")
        self.normed = self.qk_norm or self.v_norm or self.v_mix is not None
        if self.normed and self.taps:
            raise ValueError("window_attention: the short convolution and the norms of q, k, v are not built together")
        if self.normed and self.eps <= 0.0:
            raise ValueError("window_attention: norms of q, k or v need a positive eps")
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} is not a multiple of kv_heads {self.kv_heads}")
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"rot_dims {self.rot_dims} must be even and at most dim {self.dim}")
        if not (1 <= self.dim <= 256 and 1 <= self.vdim <= 256):
            raise ValueError("dim and vdim must be within 1..256")
        if self.taps > 16:
            raise ValueError("a convolution of more than 16 taps is not built")
        self.qkvg: Linear = None
        self.conv_w: Optional[torch.Tensor] = None
        self.q_norm_w = self.k_norm_w = self.mix_lambda = None
        self.o: Linear = None

    @classmethod
    def _channels(cls, p) -> int:
        return (int(p["heads"]) + int(p["kv_heads"])) * int(p["dim"]) + int(p["kv_heads"]) * int(p["vdim"])

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, nh, nkv, d, vd = (int(params[k]) for k in ("hidden", "heads", "kv_heads", "dim", "vdim"))
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        rows = {"q": nh * d, "k": nkv * d, "v": nkv * vd}
        specs = [WeightSpec(n(x), (r, h), MATRIX) for x, r in rows.items()]
        taps = int(params.get("conv") or 0)
        if taps >= 1:                       # one tap is a weight per channel and no reach back in time
            specs += [WeightSpec(n(f"{x}.conv"), (r, taps), VECTOR, std=0.5) for x, r in rows.items()]
        if params.get("gate"):
            specs.append(WeightSpec(n("g"), (nh * vd, h), MATRIX))
        if params.get("qk_norm"):
            specs += [WeightSpec(n("q.norm"), (nh * d,), VECTOR, init="one_plus_normal"),
                      WeightSpec(n("k.norm"), (nkv * d,), VECTOR, init="one_plus_normal")]
        if params.get("v_mix"):
            specs.append(WeightSpec(n("vmix"), (), VECTOR, std=0.3))
        specs.append(WeightSpec(n("o"), (h, nh * vd), MATRIX))
        if params.get("bias"):
            specs += [WeightSpec(n(f"{x}.b"), (r,), VECTOR) for x, r in rows.items()] + [WeightSpec(n("o.b"), (h,), VECTOR)]
        if params.get("distance_toll"):
            specs += [WeightSpec(n("r1"), (nh,), VECTOR, init="abs_normal", std=0.5),
                      WeightSpec(n("r2"), (nh,), VECTOR, init="abs_normal", std=0.5)]
        return specs

    @classmethod
    def kv_need(cls, params: Dict[str, Any]) -> Optional[KVNeed]:
        window = int(params.get("window") or 0) or None
        return KVNeed.keys_and_values(int(params["kv_heads"]), int(params["dim"]), window,
                                      value_dim=int(params["vdim"]), keep_first=int(params.get("keep_first") or 0))

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        taps = int(params.get("conv") or 0)
        return [StateNeed("conv_tail", (taps - 1, cls._channels(params)), torch.float32)] if taps > 1 else []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        names = ["q", "k", "v"] + (["g"] if self.gate else [])
        mats = [tensors.pop(n(x)) for x in names]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        bias = None
        if self.bias:
            bias = torch.cat([tensors.pop(n(f"{x}.b")).float() for x in ("q", "k", "v")]
                             + ([torch.zeros(mats[3].shape[0], device=mats[3].device)] if self.gate else []))
        self.qkvg = Linear(torch.cat(mats, dim=0), bias)
        del mats
        if self.distance_toll:
            self.toll = tuple(tensors.pop(n(x)).to(torch.float32).contiguous() for x in ("r1", "r2"))
        if self.taps >= 1:
            self.conv_w = torch.cat([tensors.pop(n(f"{x}.conv")).float() for x in ("q", "k", "v")]).contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors.pop(n("q.norm")).to(torch.float32).contiguous()
            self.k_norm_w = tensors.pop(n("k.norm")).to(torch.float32).contiguous()
        if self.v_mix:
            self.mix_lambda = tensors.pop(n("vmix")).to(torch.float32).reshape(1).contiguous()
        self.o = Linear(tensors.pop(n("o")), tensors.pop(n("o.b")) if self.bias else None)

    def describe_step(self, layout, put) -> QueryTiles:
        return describe_query_tiles(layout, put)

    @property
    def inner_width(self) -> int:
        return self.heads * self.vdim

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position, out: torch.Tensor = None) -> torch.Tensor:
        """The gated heads ``[N, heads * vdim]`` that the output projection takes."""
        n = x.shape[0]
        step: QueryTiles = ctx.extras[self.describe_key]
        if self.rot_dims:
            if not (isinstance(position, (tuple, list)) and len(position) == 2 and 2 * position[0].shape[1] == self.rot_dims):
                raise TypeError("window_attention takes its position as a pair (cos, sin) of [N, rot_dims / 2] float32 "
                                "tensors; the layer's position encoding gave something else")
            cos, sin = position
        else:
            cos = sin = torch.empty((n, 0), dtype=torch.float32, device=x.device)
        g = run.kv_group
        views, page_stride = ctx.kv.stream_views(g, run.kv_index)
        k_layer, v_layer = views["k"], views["v"]
        proj = self.qkvg.forward(x, out_dtype=torch.float32)            # float32 sums: they go on into the convolution and the rotation
        q = torch.empty((n, self.heads * self.dim), dtype=x.dtype, device=x.device)
        if self.normed:
            mode, v_first = ops.MIX_NONE, None
            if self.v_mix == "first":
                mode = ops.MIX_STORE
                v_first = ctx.scratch["v_first"] = torch.empty((n, self.kv_heads * self.vdim), dtype=torch.float32, device=x.device)
            elif self.v_mix == "blend":
                mode, v_first = ops.MIX_BLEND, ctx.scratch.get("v_first")
                if v_first is None or tuple(v_first.shape) != (n, self.kv_heads * self.vdim):
                    raise RuntimeError("window_attention: v_mix 'blend' needs an earlier layer of the step with v_mix 'first' "
                                       "and the same kv_heads and vdim")
            ops.qkv_norm_rope_write(proj, self.q_norm_w, self.k_norm_w, self.eps, cos, sin, self.layout, self.heads,
                                    self.kv_heads, self.dim, self.vdim, self.v_norm, mode, self.mix_lambda, v_first, q,
                                    ctx.slot_maps[g], k_layer, v_layer, page_stride, ctx.page_size)
        else:
            ops.conv_rope_kv_write(proj, self.conv_w, self.taps, run.states["conv_tail"] if self.taps > 1 else None,
                                   step.row_entry, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot, ctx.n_entries, cos, sin,
                                   self.layout, self.heads, self.kv_heads, self.dim, self.vdim, q, ctx.slot_maps[g],
                                   k_layer, v_layer, page_stride, ctx.page_size)
        if out is None:
            out = torch.empty((n, self.heads * self.vdim), dtype=x.dtype, device=x.device)
        gate = proj[:, self._channels(self.params):] if self.gate else None
        common = (ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start, self.heads, self.kv_heads, self.dim, self.scale,
                  self.window)
        rest = (self.vdim, self.softcap, self.keep_first, self.sink, gate)
        more = dict(q_temp=self.q_temp, distance_toll=self.toll)
        pages = (k_layer, v_layer, page_stride, ctx.page_size, ctx.block_tables[g])
        fast = (self.TENSOR_CORES and x.dtype == torch.bfloat16 and self.dim == self.vdim and out.is_contiguous()
                and self.dim in ops.FAST_ATTENTION_HEAD_DIMS)
        singles = (step.single_entry, step.single_q0, step.n_single)
        if fast and step.n_dec and not (self.softcap or self.keep_first or self.sink or self.gate):
            # entries of one token: the split tensor-core kernel, which reads a key once for all the heads that share it
            max_keys = min(ctx.max_ctx_len, self.window) if self.window else ctx.max_ctx_len
            n_splits = ops.attn_decode_splits(step.n_dec, self.heads, self.kv_heads, self.dim, max_keys)
            part_o = part_ml = None
            if n_splits > 1:
                part_o = torch.empty(step.n_dec * self.heads * n_splits * self.dim, dtype=torch.float32, device=x.device)
                part_ml = torch.empty(step.n_dec * self.heads * n_splits * 2, dtype=torch.float32, device=x.device)
            ops.attn_decode_bf16(q, q.stride(0), out, *pages, step.dec_entry, step.n_dec, ctx.entry_q_start, ctx.entry_q_len,
                                 ctx.entry_ctx_start, part_o, part_ml, self.heads, self.kv_heads, self.dim, self.scale,
                                 self.window, n_splits, **more)
            singles = (step.short_entry, step.short_q0, step.n_short)
        if singles[2]:          # decoded tokens and the shortest portions: a block a token and head
            ops.attn_paged_options(q, q.stride(0), out, *pages, *singles, *common, *rest, single_tokens=True, **more)
        if step.n_chunk and fast:
            ops.attn_prefill_options_bf16(q, q.stride(0), out, *pages, step.chunk_entry, step.chunk_q0, step.n_chunk, *common,
                                          self.softcap, self.keep_first, self.sink, gate, **more)      # portions on tensor cores
        elif step.n_tiles:
            ops.attn_paged_options(q, q.stride(0), out, *pages, step.tile_entry, step.tile_q0, step.n_tiles, *common, *rest, **more)
        return out

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position):
        return self.o.forward(self.inner(x, ctx, run, position), allow_partials=True, f32_sums=True, out_dtype=torch.float32)


register_part("mixer", "window_attention", WindowAttention)
