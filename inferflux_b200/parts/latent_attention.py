"""``latent_attention``: causal attention whose keys and values follow from one
cached latent vector per token, without positions.

    c_q = unit_rms(W_dq x) * w_q            q_h = (W_uq c_q)_h                 per head h, ``dim`` wide
    c   = unit_rms(W_dkv x) * w_kv          k_h = (W_uk c)_h,  v_h = (W_uv c)_h   (``dim`` and ``vdim`` wide)
    p_h(i, .) = softmax_j<=i( (q_h(i) . k_h(j)) * scale )
    o_h(i) = sigmoid(W_g x_i)_h * sum_j p_h(i, j) v_h(j)          y = W_o [o_1 .. o_H]

Only ``c`` is cached (one stream of ``kv_rank`` elements a token).  Keys and
values are never formed: the key projection is moved to the query,
``q_h . (Uk_h c) = (Uk_h^T q_h) . c``, and the value projection behind the
sum, ``sum_j p_j (Uv_h c_j) = Uv_h (sum_j p_j c_j)``, so the attention kernel
works on latents alone and all heads of a token read the same cached rows.
The three projections of x are stacked at load into one product whose sums
stay float32; both unit-rms norms, the cache write and the gates' sigmoid are
one kernel; scores, softmax and the weighted sums are float32.

Options, each a parameter: ``q_rank`` 0 = the queries are one projection of x (``q``) without a latent of their
own; ``gate`` false = no output gates; ``rot_dim`` > 0 = every query head has ``rot_dim`` more columns behind its
``dim`` plain ones, the down projection ``dkv`` has ``rot_dim`` more rows behind the latent's (not normed), and
both are rotated by the layer's position table in neighbouring pairs ``(2i, 2i + 1)``: one rotated key part per
token, shared by all heads, so that

    score_h(i, j) = (q_plain_h(i) . (Uk_h c_j) + q_rot_h(i) . k_rot(j)) * scale;

the cached row is then ``[c | k_rot]``, ``kv_rank + rot_dim`` wide, the kernel's query ``[Uk_h^T q_plain_h | q_rot_h]``,
and the value still the latent alone.  ``window`` > 0 = key j is visible to position p iff ``0 <= p - j < window``
(pages behind the window go back to the pool); ``sink`` = a stored number per head whose exponential joins the
softmax's denominator, without a key or a value.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import CacheStream, KVNeed, Part, RunInfo
from .linear import Linear

QUERY_TILE = 16     # tokens per query tile of the latent attention kernel
PROMPT_PAGE = 64    # tokens per page of the keys and values that a prompt step forms for its own use


@dataclass
class LatentStep:
    """The step's query tiles: int32 device tensors.  For the float32 kernel
    tiles of QUERY_TILE tokens; for the tensor-core kernel tiles of ``bm``
    (token, head) rows, which depend on the number of heads."""

    tile_entry: torch.Tensor
    tile_q0: torch.Tensor
    n_tiles: int
    bm: int
    row_tile_entry: torch.Tensor
    row_tile_row0: torch.Tensor
    n_row_tiles: int
    prompt: Optional["PromptStep"] = None     # set when the step's portions go through keys and values per head


@dataclass
class PromptStep:
    """Prompt portions attended per head (see :meth:`LatentAttention._prompt_by_heads`):
    which cached latents to expand, where the expanded keys and values of each
    entry lie, and the query tiles of the tensor-core prompt kernel."""

    g_entry: torch.Tensor                     # [G] entry of every latent to expand (each entry's context, padded to whole pages)
    g_pos: torch.Tensor                       # [G] its position
    n_gather: int
    block_tables: torch.Tensor                # [R, B] pages of the expanded keys and values, -1 for entries without a portion
    tile_entry: torch.Tensor
    tile_q0: torch.Tensor
    n_tiles: int
    tile_rows: int
    max_keys: int
    row_entry: torch.Tensor                   # [N] the entry of every row of the step


class LatentAttention(Part):
    """params: ``hidden``, ``heads``, ``dim`` (of queries and keys), ``vdim``,
    ``kv_rank``, ``q_rank``, ``scale``, ``eps`` (of the two unit-rms norms),
    ``gate`` (default true), ``rot_dim``, ``window``, ``sink`` (defaults 0, 0, false),
    ``name`` (tensors ``<prefix>.<name>.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}``; with
    ``q_rank`` 0 ``q`` instead of ``dq``, ``dq.norm`` and ``uq``; ``sink`` ``[heads]``).
    Position (with ``rot_dim``): a pair ``(cos, sin)`` of float32 ``[N, rot_dim / 2]`` tensors."""

    family = "mixer"
    #: Switch for tests and measurements: the tensor-core kernel over the latents where the sizes allow it.
    TENSOR_CORES = True

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.kv_rank, self.q_rank = int(p["kv_rank"]), int(p.get("q_rank") or 0)
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.gated = bool(p.get("gate", True))
        self.rot_dim, self.window, self.has_sink = int(p.get("rot_dim") or 0), int(p.get("window") or 0), bool(p.get("sink"))
        self.width = self.kv_rank + self.rot_dim        # of a cached row and of the kernel's queries
        self.plain = self.q_rank > 0 and self.gated and not (self.rot_dim or self.window or self.has_sink)
        if self.rot_dim % 2:
            raise ValueError(f"latent_attention: rot_dim {self.rot_dim} must be even")
        if self.rot_dim and self.q_rank:
            raise ValueError("latent_attention: a rotated part and a query latent are not built together")
        if not self.q_rank and self.gated:
            raise ValueError("latent_attention: output gates without a query latent are not built")
        self.sink: torch.Tensor = None
        # layers of the same sizes share a step's description
        self.describe_key = f"latent_attention/{self.heads}/{self.dim}/{self.vdim}/{self.kv_rank}/{self.plain}"
        self.ukv: Linear = None             # [uk; uv] stacked, for steps that form keys and values
        if not 1 <= self.kv_rank <= 1024:
            raise ValueError(f"kv_rank {self.kv_rank} is outside 1..1024")
        self.down: Linear = None            # [dq; dkv; g]
        self.uq: Linear = None
        self.uk_t: torch.Tensor = None      # [heads, kv_rank, dim]: a head's key projection, transposed
        self.uv: torch.Tensor = None        # [heads, vdim, kv_rank]
        self.o: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, nh, d, vd, r = (int(params[k]) for k in ("hidden", "heads", "dim", "vdim", "kv_rank"))
        qr, rot = int(params.get("q_rank") or 0), int(params.get("rot_dim") or 0)
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        if not qr:
            return ([WeightSpec(n("q"), (nh * (d + rot), h), MATRIX), WeightSpec(n("dkv"), (r + rot, h), MATRIX),
                     WeightSpec(n("dkv.norm"), (r,), VECTOR, init="one_plus_normal"), WeightSpec(n("uk"), (nh * d, r), MATRIX),
                     WeightSpec(n("uv"), (nh * vd, r), MATRIX), WeightSpec(n("o"), (h, nh * vd), MATRIX)]
                    + ([WeightSpec(n("sink"), (nh,), VECTOR, std=1.0)] if params.get("sink") else []))
        return [WeightSpec(n("dq"), (qr, h), MATRIX), WeightSpec(n("dq.norm"), (qr,), VECTOR, init="one_plus_normal"),
                WeightSpec(n("uq"), (nh * d, qr), MATRIX),
                WeightSpec(n("dkv"), (r, h), MATRIX), WeightSpec(n("dkv.norm"), (r,), VECTOR, init="one_plus_normal"),
                WeightSpec(n("uk"), (nh * d, r), MATRIX), WeightSpec(n("uv"), (nh * vd, r), MATRIX),
                WeightSpec(n("g"), (nh, h), MATRIX), WeightSpec(n("o"), (h, nh * vd), MATRIX)]

    @classmethod
    def kv_need(cls, params: Dict[str, Any]) -> Optional[KVNeed]:
        return KVNeed((CacheStream("latent", 1, int(params["kv_rank"]) + int(params.get("rot_dim") or 0)),),
                      int(params.get("window") or 0) or None)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        if not self.q_rank:
            mats = [tensors.pop(n(x)) for x in ("q", "dkv")]
            if len({m.dtype for m in mats}) > 1:
                mats = [m.float() for m in mats]
            self.down = Linear(torch.cat(mats, dim=0))
            del mats
            self.wkv = tensors.pop(n("dkv.norm")).to(torch.float32).contiguous()
            uk = tensors.pop(n("uk"))
            self.uk_t = uk.view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
            self.uv = tensors.pop(n("uv")).view(self.heads, self.vdim, self.kv_rank).contiguous()
            if self.has_sink:
                self.sink = tensors.pop(n("sink")).to(torch.float32).contiguous()
            self.o = Linear(tensors.pop(n("o")))
            return
        mats = [tensors.pop(n(x)) for x in ("dq", "dkv", "g")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.down = Linear(torch.cat(mats, dim=0))
        del mats
        self.wq = tensors.pop(n("dq.norm")).to(torch.float32).contiguous()
        self.wkv = tensors.pop(n("dkv.norm")).to(torch.float32).contiguous()
        self.uq = Linear(tensors.pop(n("uq")))
        self.uk_t = tensors[n("uk")].view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        uk, uv = tensors[n("uk")], tensors.pop(n("uv"))
        if self._prompt_by_heads(uk.dtype):
            self.ukv = Linear(torch.cat([uk, uv], dim=0))
        del tensors[n("uk")]
        self.uv = uv.view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.o = Linear(tensors.pop(n("o")))

    def _prompt_by_heads(self, weight_dtype=None) -> bool:
        """Whether prompt portions are attended per head: bfloat16 and heads
        of the size the tcgen05 prompt kernel takes.  A portion's queries then
        meet keys and values ``k_h = Uk_h c``, ``v_h = Uv_h c`` that the step
        forms from the cached latents of the portion's whole context (one
        product over the gathered latents), which costs ``dim + vdim`` instead
        of ``2 kv_rank`` multiplications per query, key and head.  Single
        tokens stay with the latents, which all their heads share."""
        dtype = weight_dtype if weight_dtype is not None else self.dtype
        return (self.plain and dtype == torch.bfloat16 and self.dtype == torch.bfloat16 and torch.device(self.device).type == "cuda"
                and self.dim == self.vdim == ops.UMMA_ATTENTION_HEAD_DIM and self.kv_rank % 8 == 0)

    def describe_step(self, layout, put) -> LatentStep:
        r = layout.n_entries
        q_len = [int(n) for n in layout.q_len[:r]]
        tile_entry, tile_q0 = [], []
        for i in range(r):
            for q0 in range(0, q_len[i], QUERY_TILE):
                tile_entry.append(i), tile_q0.append(q0)
        prompt = None
        portions = [i for i in range(r) if q_len[i] > 1]
        if portions and self.ukv is not None:
            g_entry, g_pos, tabs, at = [], [], [[] for _ in range(r)], 0
            for i in portions:
                total = int(layout.ctx_start[i]) + q_len[i]
                pages = (total + PROMPT_PAGE - 1) // PROMPT_PAGE
                g_entry += [i] * (pages * PROMPT_PAGE)
                g_pos += list(range(total)) + [0] * (pages * PROMPT_PAGE - total)      # padding repeats position 0; it is never visible
                tabs[i] = list(range(at, at + pages))
                at += pages
            width = max(len(t) for t in tabs)
            table = [t + [-1] * (width - len(t)) for t in tabs]
            full = ops.UMMA_ATTENTION_TILE
            blocks = sum((q_len[i] + full - 1) // full for i in portions) * self.heads
            rows = full // 2 if 2 * blocks <= ops.sm_count(self.device) else full
            p_entry, p_q0 = [], []
            for i in portions:
                for q0 in range(0, q_len[i], rows):
                    p_entry.append(i), p_q0.append(q0)
            prompt = PromptStep(put(g_entry), put(g_pos), len(g_entry), put([v for t in table for v in t]).view(r, width),
                                put(p_entry), put(p_q0), len(p_entry), rows,
                                max(int(layout.ctx_start[i]) + q_len[i] for i in portions),
                                put([i for i in range(r) for _ in range(q_len[i])]))
        # tiles of (token, head) rows over the latents: every entry, or only the single tokens beside such portions
        rows = [(0 if prompt is not None and n > 1 else n * self.heads) for n in q_len]
        bm = next((t for t in ops.LATENT_MMA_TILES if max(rows) <= t), ops.LATENT_MMA_TILES[-1])
        row_entry, row0 = [], []
        for i, n in enumerate(rows):
            for r0 in range(0, n, bm):
                row_entry.append(i), row0.append(r0)
        return LatentStep(put(tile_entry), put(tile_q0), len(tile_entry), bm, put(row_entry), put(row0), len(row_entry), prompt)

    def _per_head(self, x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x ``[N, heads, a]`` (a view), w ``[heads, b, a]`` -> float32 ``[N, heads, b]``
        (a view, or ``out`` if given): head h's vectors times ``w[h]^T``."""
        n, width_out = x.shape[0], w.shape[1]
        if w.dtype == torch.float32:
            if out is None:
                out = torch.empty((n, self.heads, width_out), dtype=torch.float32, device=x.device)
            for h in range(self.heads):
                ops.gemm_f32(x[:, h], w[h], None, out[:, h])
            return out
        # bfloat16 weights: one batched library product over the heads, float32 sums
        y = torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32).transpose(0, 1)
        return y if out is None else out.copy_(y)

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position=None, out: torch.Tensor = None) -> torch.Tensor:
        """The gated heads ``[N, heads * vdim]`` that the output projection takes;
        writes this step's latents into the run's cache and attends over it."""
        n = x.shape[0]
        step: LatentStep = ctx.extras[self.describe_key]
        g = run.kv_group
        views, page_stride = ctx.kv.stream_views(g, run.kv_index)
        cache = views["latent"]
        if not self.plain:
            return self._inner_options(x, ctx, position, out, step, g, cache, page_stride)
        p = self.down.forward(x, out_dtype=torch.float32)
        cq = torch.empty((n, self.q_rank), dtype=x.dtype, device=x.device)
        gate = torch.empty((n, self.heads), dtype=torch.float32, device=x.device)
        ops.latent_prep(p, self.wq, self.wkv, self.eps, self.q_rank, self.kv_rank, self.heads, cq, cache, page_stride,
                        ctx.page_size, ctx.slot_maps[g], gate)
        q = self.uq.forward(cq, out_dtype=x.dtype).view(n, self.heads, self.dim)
        if out is None:
            out = torch.empty((n, self.heads * self.vdim), dtype=x.dtype, device=x.device)
        prompt = step.prompt
        if prompt is not None:
            self._attend_portions(q, gate, out, ctx, prompt, cache, page_stride, g)
            if not step.n_row_tiles:
                return out
        q_lat = self._per_head(q, self.uk_t)                                   # float32 [N, heads, kv_rank]
        alloc = torch.zeros if prompt is not None else torch.empty             # rows of portions stay unwritten, and finite
        o_lat = alloc((self.heads, n, self.kv_rank), dtype=x.dtype, device=x.device).transpose(0, 1)
        if ops.attn_latent_mma_ok(self.kv_rank, cache):
            splits = ops.attn_latent_mma_splits(step.n_row_tiles, step.bm, self.kv_rank, ctx.max_ctx_len)
            ops.attn_latent_mma(q_lat, o_lat, cache, page_stride, ctx.page_size, ctx.block_tables[g], step.row_tile_entry,
                                step.row_tile_row0, step.n_row_tiles, step.bm, ctx.entry_q_start, ctx.entry_q_len,
                                ctx.entry_ctx_start, self.scale, splits)
        else:
            ops.attn_latent_paged(q_lat, o_lat, cache, page_stride, ctx.page_size, ctx.block_tables[g], step.tile_entry,
                                  step.tile_q0, step.n_tiles, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start,
                                  self.scale)
        heads = self._per_head(o_lat, self.uv)                                 # float32 [N, heads, vdim]
        if prompt is not None:                                                 # only the single tokens' rows
            return ops.gate_heads(heads, gate, out, prompt.row_entry, ctx.entry_q_len, prompt_rows=False)
        return ops.gate_heads(heads, gate, out)

    def _inner_options(self, x, ctx, position, out, step: LatentStep, g, cache, page_stride) -> torch.Tensor:
        """The mixer with its options (a direct query projection, a rotated part, a window, a sink; no gates):
        the kernel's queries are ``[Uk_h^T q_plain_h | q_rot_h]`` against cached rows ``[c | k_rot]``."""
        n, nh, r, rot = x.shape[0], self.heads, self.kv_rank, self.rot_dim
        if rot:
            if not (isinstance(position, (tuple, list)) and len(position) == 2 and 2 * position[0].shape[1] == rot):
                raise TypeError("latent_attention takes its position as a pair (cos, sin) of [N, rot_dim / 2] float32 tensors; "
                                "the layer's position encoding gave something else")
            cos, sin = position
        else:
            cos = sin = torch.empty((n, 0), dtype=torch.float32, device=x.device)
        p = self.down.forward(x, out_dtype=torch.float32)                      # [q heads | latent | rotating key part]
        q_plain = torch.empty((n, nh * self.dim), dtype=x.dtype, device=x.device)
        q_rows = torch.empty((n, nh, self.width), dtype=torch.float32, device=x.device)
        ops.latent_rope_prep(p, self.wkv, self.eps, nh, self.dim, rot, r, cos, sin, q_plain, q_rows, cache, page_stride,
                             ctx.page_size, ctx.slot_maps[g])
        self._per_head(q_plain.view(n, nh, self.dim), self.uk_t, out=q_rows[:, :, :r])
        o_lat = torch.empty((nh, n, r), dtype=x.dtype, device=x.device).transpose(0, 1)
        if self.TENSOR_CORES and r % 8 == 0 and ops.attn_latent_mma_ok(self.width, cache):
            keys = min(ctx.max_ctx_len, self.window + step.bm) if self.window else ctx.max_ctx_len     # what a tile can see
            splits = ops.attn_latent_mma_splits(step.n_row_tiles, step.bm, self.width, keys)
            ops.attn_latent_mma(q_rows, o_lat, cache, page_stride, ctx.page_size, ctx.block_tables[g], step.row_tile_entry,
                                step.row_tile_row0, step.n_row_tiles, step.bm, ctx.entry_q_start, ctx.entry_q_len,
                                ctx.entry_ctx_start, self.scale, splits, window=self.window, sink=self.sink)
        else:
            ops.attn_latent_paged(q_rows, o_lat, cache, page_stride, ctx.page_size, ctx.block_tables[g], step.tile_entry,
                                  step.tile_q0, step.n_tiles, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start,
                                  self.scale, window=self.window, sink=self.sink)
        heads = self._per_head(o_lat, self.uv)                                 # float32 [N, heads, vdim]
        if out is None:
            out = torch.empty((n, nh * self.vdim), dtype=x.dtype, device=x.device)
        return ops.gate_heads(heads, None, out)

    def _attend_portions(self, q, gate, out, ctx, prompt: "PromptStep", cache, page_stride, g) -> None:
        """The step's prompt portions per head: expand the cached latents of
        their contexts into keys and values, laid out in pages of their own,
        and run the tensor-core prompt kernel over them; gated rows into out."""
        n, h, d = q.shape[0], self.heads, self.dim
        lat = torch.empty((prompt.n_gather, self.kv_rank), dtype=cache.dtype, device=q.device)
        ops.gather_latents(cache, page_stride, ctx.page_size, ctx.block_tables[g], prompt.g_entry, prompt.g_pos, lat)
        kv = self.ukv.forward(lat, out_dtype=cache.dtype)                      # [G, (k | v) x heads x d]
        pages = prompt.n_gather // PROMPT_PAGE
        pool = kv.view(pages, PROMPT_PAGE, 2, h, d).permute(0, 2, 3, 1, 4).contiguous()     # [page][k|v][head][slot][d]
        attn = torch.empty((n, h * d), dtype=q.dtype, device=q.device)
        splits = ops.attn_prefill_umma_splits(prompt.n_tiles, h, prompt.max_keys)
        ops.attn_prefill_umma(q.view(n, h * d), h * d, attn, pool[0, 0], pool[0, 1], pool.stride(0), PROMPT_PAGE,
                              prompt.block_tables, prompt.tile_entry, prompt.tile_q0, prompt.n_tiles, ctx.entry_q_start,
                              ctx.entry_q_len, ctx.entry_ctx_start, h, h, d, self.scale, 0, splits,
                              tile_rows=prompt.tile_rows)
        ops.gate_heads(attn.view(n, h, d), gate, out, prompt.row_entry, ctx.entry_q_len, prompt_rows=True)

    @property
    def inner_width(self) -> int:
        return self.heads * self.vdim

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position) -> torch.Tensor:
        return self.o.forward(self.inner(x, ctx, run, position), out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttention)
