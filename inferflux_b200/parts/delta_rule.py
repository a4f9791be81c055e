"""``general_delta``: linear attention by the generalized delta rule.  Per head, with r, k, v of ``dim`` each
(``r = W_r h`` and so on), a decay and a removal rate per key channel,

    w_t = exp(-e^(-1/2) * sigmoid(W_w2 tanh(W_w1 h_t) + w0))        in (exp(-e^(-1/2)), 1)
    a_t = sigmoid(W_a h_t + a_b)
    u_t = k_t / sqrt(sum(k_t^2) + 1e-6)                              the head's unit key
    S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T   S: [dim x dim], float32, zero at the start;
                                                                      the decay and the removal both read S_{t-1}
    o_t = S_t^T r_t

every head's o is divided by its root mean square, the heads side by side are multiplied by a weight over all of them
and by sigmoid(W_g h), and projected.  r, k, v, the raw removal rates, the gate and the decay's inner projection are
one stacked product whose sums stay float32; the decay, the removal rate, the unit key, the state and the norm are
float32 in either engine type.  The inner size of the decay's two-step projection is the stored tensors' own.  The
state lives in the request's state slot.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import Part, RunInfo, StateNeed
from .linear import Linear

DECAY_SCALE = math.exp(-0.5)
KEY_EPS = 1e-6


class GeneralDelta(Part):
    """params: ``hidden``, ``heads``, ``dim``, ``decay_rank`` (0 = whatever the stored ``w1`` has), ``eps`` (of the
    per-head norm), ``decay_scale`` and ``key_eps`` (default ``e^(-1/2)`` and 1e-6), ``name`` (tensors
    ``<prefix>.<name>.{r,k,v,a,a.b,g,w1,w2,w0,norm,o}``).  State: ``delta`` float32 ``[heads, dim (value), dim (key)]``."""

    family = "mixer"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden, self.heads, self.dim = int(p["hidden"]), int(p["heads"]), int(p["dim"])
        self.eps = float(p["eps"])
        self.decay_scale = float(p.get("decay_scale", DECAY_SCALE))
        self.key_eps = float(p.get("key_eps", KEY_EPS))
        if not 1 <= self.dim <= 512:
            raise ValueError("general_delta: dim must be within 1..512")
        self.rank = 0
        self.stacked: Linear = None
        self.w2: Linear = None
        self.o: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, hd = int(params["hidden"]), int(params["heads"]) * int(params["dim"])
        rank = int(params.get("decay_rank") or 0) or -1
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return ([WeightSpec(n(x), (hd, h), MATRIX) for x in ("r", "k", "v", "a", "g")]
                + [WeightSpec(n("a.b"), (hd,), VECTOR, std=0.5), WeightSpec(n("w1"), (rank, h), MATRIX),
                   WeightSpec(n("w2"), (hd, rank), MATRIX, std=0.5), WeightSpec(n("w0"), (hd,), VECTOR, std=0.5),
                   WeightSpec(n("norm"), (hd,), VECTOR, init="one_plus_normal"), WeightSpec(n("o"), (h, hd), MATRIX)])

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        d = int(params["dim"])
        return [StateNeed("delta", (int(params["heads"]), d, d), torch.float32)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        f32 = lambda leaf: tensors.pop(n(leaf)).to(torch.float32).contiguous()
        mats = [tensors.pop(n(x)) for x in ("r", "k", "v", "a", "g", "w1")]
        w2 = tensors.pop(n("w2"))
        self.rank = mats[-1].shape[0]
        if w2.shape[1] != self.rank:
            raise ValueError(f"{n('w2')} takes {w2.shape[1]} inputs but {n('w1')} gives {self.rank}")
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.stacked = Linear(torch.cat(mats, dim=0))
        del mats
        self.w2 = Linear(w2)
        self.a_bias, self.w0, self.norm_w = f32("a.b"), f32("w0"), f32("norm")
        self.o = Linear(tensors.pop(n("o")))

    @property
    def inner_width(self) -> int:
        return self.heads * self.dim

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position=None, out: torch.Tensor = None) -> torch.Tensor:
        """The normed, gated heads ``[N, heads * dim]`` that the output projection takes."""
        n, dev, hd = x.shape[0], x.device, self.heads * self.dim
        proj = self.stacked.forward(x, out_dtype=torch.float32)               # [r | k | v | a | g | w1]
        t = torch.empty((n, self.rank), dtype=x.dtype, device=dev)
        ops.activation(proj[:, 5 * hd:], t, ops.ACT_TANH)
        w_raw = self.w2.forward(t, out_dtype=torch.float32)
        o = torch.empty((n, hd), dtype=torch.float32, device=dev)
        ops.delta_rule_scan(proj, 0, hd, 2 * hd, 3 * hd, w_raw, self.w0, self.a_bias, run.states["delta"],
                            ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot, ctx.n_entries, o, self.heads, self.dim,
                            self.dim, self.decay_scale, self.key_eps)
        if out is None:
            out = torch.empty((n, hd), dtype=x.dtype, device=dev)
        return ops.head_norm_gate(o, proj[:, 4 * hd:5 * hd], self.norm_w, out, self.heads, self.dim, self.eps, ops.GATE_SIGMOID)

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position):
        return self.o.forward(self.inner(x, ctx, run), allow_partials=True, f32_sums=True, out_dtype=torch.float32)


register_part("mixer", "general_delta", GeneralDelta)
