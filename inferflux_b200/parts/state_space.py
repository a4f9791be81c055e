"""``mamba2``: a selective state-space mixer (the scalar-decay form in which the recurrence equals a masked
attention, "state-space duality").  With ``inner = heads * vdim``, ``N = state`` and ``G = groups``, one projection of
the input gives ``[z: inner | x: inner | B: G N | C: G N | dt: heads]``;

    (x, B, C) <- silu(conv(x, B, C) + b)       a causal convolution over time on every channel, zeros ahead of a sequence
    dt        <- softplus(dt + dt_bias)         no clamp
    S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T         S: [N x vdim] per head, float32, zero at the start
    y_t = S_t^T C_t + D_h x_t                   head h reads B and C of group h // (heads / G)
    out = W_o ( N_groups(y * silu(z)) * w )     the gate ahead of the norm; N over ``norm_groups`` equal parts of the row

The projection's sums stay float32, and so do the convolution, the step sizes, the decays, the state and the norm in
either engine type.  The state and the last ``taps - 1`` inputs of the convolution live in the request's state
slot, so a prompt may be cut anywhere and a decoded token is the same kernels with one token.
"""
from __future__ import annotations

from typing import Any, Dict, List

import numpy as np
import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import Part, RunInfo, StateNeed
from .linear import Linear


def describe_row_entries(layout, put) -> torch.Tensor:
    """The entry of every row of the step, int32 on the device (for kernels that run a block a row)."""
    return put(np.repeat(np.arange(layout.n_entries), layout.q_len[:layout.n_entries]))


class Mamba2(Part):
    """params: ``hidden``, ``heads``, ``vdim``, ``state``, ``groups``, ``conv`` (taps), ``norm_groups``, ``eps``,
    ``name`` (tensors ``<prefix>.<name>.{in,conv,conv.b,dt_bias,A_log,D,norm,o}``).
    State: ``ssm`` float32 ``[heads, vdim, state]``, ``ssm_conv_tail`` float32 ``[taps - 1, channels of x, B and C]``."""

    family = "mixer"
    describe_key = "row_entries"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden, self.heads, self.vdim = int(p["hidden"]), int(p["heads"]), int(p["vdim"])
        self.state, self.groups = int(p["state"]), int(p.get("groups") or 1)
        self.taps, self.norm_groups = int(p["conv"]), int(p.get("norm_groups") or 1)
        self.eps = float(p["eps"])
        if self.heads % self.groups:
            raise ValueError(f"mamba2: heads {self.heads} is not a multiple of groups {self.groups}")
        if (self.heads * self.vdim) % self.norm_groups:
            raise ValueError("mamba2: heads * vdim is not a multiple of norm_groups")
        if not 1 <= self.taps <= 16 or not 1 <= self.state <= 512:
            raise ValueError("mamba2: conv must be within 1..16 taps and state within 1..512")
        self.n_inner = self.heads * self.vdim
        self.channels = self.n_inner + 2 * self.groups * self.state
        self.in_proj: Linear = None
        self.o: Linear = None

    @classmethod
    def _sizes(cls, p):
        inner = int(p["heads"]) * int(p["vdim"])
        channels = inner + 2 * int(p.get("groups") or 1) * int(p["state"])
        return inner, channels

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, heads, taps = int(params["hidden"]), int(params["heads"]), int(params["conv"])
        inner, channels = cls._sizes(params)
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("in"), (inner + channels + heads, h), MATRIX),
                WeightSpec(n("conv"), (channels, taps), VECTOR, std=0.5), WeightSpec(n("conv.b"), (channels,), VECTOR, std=0.1),
                WeightSpec(n("dt_bias"), (heads,), VECTOR, std=0.5), WeightSpec(n("A_log"), (heads,), VECTOR, std=0.5),
                WeightSpec(n("D"), (heads,), VECTOR, std=0.5),
                WeightSpec(n("norm"), (inner,), VECTOR, init="one_plus_normal"), WeightSpec(n("o"), (h, inner), MATRIX)]

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        _, channels = cls._sizes(params)
        taps = int(params["conv"])
        needs = [StateNeed("ssm", (int(params["heads"]), int(params["vdim"]), int(params["state"])), torch.float32)]
        if taps > 1:
            needs.append(StateNeed("ssm_conv_tail", (taps - 1, channels), torch.float32))
        return needs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        f32 = lambda leaf: tensors.pop(n(leaf)).to(torch.float32).contiguous()
        self.in_proj = Linear(tensors.pop(n("in")))
        self.conv_w, self.conv_b = f32("conv"), f32("conv.b")
        self.dt_bias, self.a_log, self.d_skip = f32("dt_bias"), f32("A_log"), f32("D")
        self.norm_w = f32("norm")
        self.o = Linear(tensors.pop(n("o")))

    def describe_step(self, layout, put) -> torch.Tensor:
        return describe_row_entries(layout, put)

    @property
    def inner_width(self) -> int:
        return self.n_inner

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position=None, out: torch.Tensor = None) -> torch.Tensor:
        """The gated, normed rows ``[N, heads * vdim]`` that the output projection takes."""
        n, dev = x.shape[0], x.device
        row_entry = ctx.extras[self.describe_key]
        proj = self.in_proj.forward(x, out_dtype=torch.float32)
        inner, gn = self.n_inner, self.groups * self.state
        xbc = torch.empty((n, self.channels), dtype=torch.float32, device=dev)
        ops.causal_conv(proj, inner, self.channels, self.conv_w, self.conv_b,
                        run.states["ssm_conv_tail"] if self.taps > 1 else None, row_entry, ctx.entry_q_start,
                        ctx.entry_q_len, ctx.entry_slot, ctx.n_entries, xbc, silu=True)
        y = torch.empty((n, inner), dtype=torch.float32, device=dev)
        ops.ssm_scan(xbc, 0, inner, inner + gn, proj[:, inner + self.channels:], self.dt_bias, self.a_log, self.d_skip,
                     run.states["ssm"], ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot, ctx.n_entries, y, self.heads,
                     self.groups, self.vdim, self.state)
        if out is None:
            out = torch.empty((n, inner), dtype=x.dtype, device=dev)
        return ops.gated_group_norm(y, proj[:, :inner], self.norm_w, out, self.norm_groups, self.eps)

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position):
        return self.o.forward(self.inner(x, ctx, run), allow_partials=True, f32_sums=True, out_dtype=torch.float32)


register_part("mixer", "mamba2", Mamba2)
