"""``gated_linear_attention``: linear attention whose state shrinks by a decay of its own per key channel and token,

    S_t = diag(alpha_t) S_{t-1} + k_t v_t^T        S: [dim x vdim] per head, float32, zero at the start of a sequence
    o_t = S_t^T (q_t * q_scale)
    alpha_t = sigmoid(W_a2 (W_a1 h_t) + b_a)^(1 / tau)       heads x dim numbers in (0, 1)

the decay coming from a projection through a narrow middle (its size is the stored ``a1``'s).  Each head's o is
divided by its root mean square and multiplied by a weight ``vdim`` long that all heads share, the heads side by
side are multiplied by silu(W_g h) and projected.  q, k, v, g and the narrow a1 are one stacked projection whose
sums stay float32; the second decay projection runs in float32 on those sums (its matrix is small), and decays,
state, outputs and the norm are float32 in either engine type.  The state lives in the request's state slot, so a
prompt may be cut anywhere; a portion longer than a segment is cut into segments that run side by side (the
recurrence is linear in S).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import Part, RunInfo, StateNeed
from .linear import Linear


@dataclass
class GlaStep:
    """The step cut into segments for the scan kernels: int32 device tensors; ``n_segments`` 0 = every entry fits
    one segment and is walked from its slot."""

    seg_entry: torch.Tensor
    seg_t0: torch.Tensor
    entry_first_seg: torch.Tensor
    n_segments: int


class GatedLinearAttention(Part):
    """params: ``hidden``, ``heads``, ``dim``, ``vdim``, ``tau``, ``q_scale`` (None = ``dim^-1/2``), ``decay_rank``
    (0 = whatever the stored ``a1`` has), ``eps`` (of the per-head norm), ``name`` (tensors
    ``<prefix>.<name>.{q,k,v,g,o,a1,a2,a2.b,norm}``).  State: ``gla`` float32 ``[heads, dim, vdim]``."""

    family = "mixer"
    describe_key = "gla_segments"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.tau, self.eps = float(p["tau"]), float(p["eps"])
        self.q_scale = float(p["q_scale"]) if p.get("q_scale") is not None else float(self.dim) ** -0.5
        if not 1 <= self.dim <= 256:
            raise ValueError("gated_linear_attention: dim must be within 1..256")
        if self.tau <= 0.0:
            raise ValueError("gated_linear_attention: tau must be positive")
        self.rank = 0
        self.stacked: Linear = None         # [q; k; v; g; a1]
        self.a2: Linear = None
        self.o: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, nh, d, vd = (int(params[k]) for k in ("hidden", "heads", "dim", "vdim"))
        rank = int(params.get("decay_rank") or 0) or -1
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("q"), (nh * d, h), MATRIX), WeightSpec(n("k"), (nh * d, h), MATRIX),
                WeightSpec(n("v"), (nh * vd, h), MATRIX), WeightSpec(n("g"), (nh * vd, h), MATRIX),
                WeightSpec(n("o"), (h, nh * vd), MATRIX), WeightSpec(n("norm"), (vd,), VECTOR, init="one_plus_normal"),
                WeightSpec(n("a1"), (rank, h), MATRIX), WeightSpec(n("a2"), (nh * d, rank), MATRIX, std=0.5),
                WeightSpec(n("a2.b"), (nh * d,), VECTOR, std=1.0)]

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        return [StateNeed("gla", (int(params["heads"]), int(params["dim"]), int(params["vdim"])), torch.float32)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        mats = [tensors.pop(n(x)) for x in ("q", "k", "v", "g", "a1")]
        a2 = tensors.pop(n("a2"))
        self.rank = mats[-1].shape[0]
        if a2.shape[1] != self.rank:
            raise ValueError(f"{n('a2')} takes {a2.shape[1]} inputs but {n('a1')} gives {self.rank}")
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.stacked = Linear(torch.cat(mats, dim=0))
        del mats
        self.a2 = Linear(a2.float())            # widened exactly: the product runs on the float32 sums of a1
        self.a2_bias = tensors.pop(n("a2.b")).to(torch.float32).contiguous()
        self.norm_w = tensors.pop(n("norm")).to(torch.float32).repeat(self.heads).contiguous()
        self.o = Linear(tensors.pop(n("o")))

    def describe_step(self, layout, put) -> GlaStep:
        seg = ops.gla_segment() if torch.device(self.device).type == "cuda" else 64
        if all(int(layout.q_len[i]) <= seg for i in range(layout.n_entries)):
            return GlaStep(put([]), put([]), put([]), 0)
        seg_entry, seg_t0, first = [], [], []
        for i in range(layout.n_entries):
            first.append(len(seg_entry))
            for t0 in range(0, int(layout.q_len[i]), seg):
                seg_entry.append(i), seg_t0.append(t0)
        return GlaStep(put(seg_entry), put(seg_t0), put(first), len(seg_entry))

    @property
    def inner_width(self) -> int:
        return self.heads * self.vdim

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position=None, out: torch.Tensor = None) -> torch.Tensor:
        """The normed, gated heads ``[N, heads * vdim]`` that the output projection takes."""
        n, dev, hd, hv = x.shape[0], x.device, self.heads * self.dim, self.heads * self.vdim
        proj = self.stacked.forward(x, out_dtype=torch.float32)               # [q | k | v | g | a1]
        z = self.a2.forward(proj[:, 2 * hd + 2 * hv:], out_dtype=torch.float32)
        o = torch.empty((n, hv), dtype=torch.float32, device=dev)
        step: GlaStep = ctx.extras[self.describe_key]
        ops.gla_scan(proj, 0, hd, 2 * hd, z, self.a2_bias, self.tau, self.q_scale, run.states["gla"], ctx.entry_q_start,
                     ctx.entry_q_len, ctx.entry_slot, ctx.n_entries, o, self.heads, self.dim, self.vdim, step.seg_entry,
                     step.seg_t0, step.entry_first_seg, step.n_segments)
        if out is None:
            out = torch.empty((n, hv), dtype=x.dtype, device=dev)
        return ops.head_norm_gate(o, proj[:, 2 * hd + hv:2 * hd + 2 * hv], self.norm_w, out, self.heads, self.vdim, self.eps,
                                  ops.GATE_SILU)

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position):
        return self.o.forward(self.inner(x, ctx, run), allow_partials=True, f32_sums=True, out_dtype=torch.float32)


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
