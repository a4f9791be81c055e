"""``side_by_side``: two mixers that read the same input.  ``combine`` says what becomes of their outputs:
``normed_mean`` (the default): half their sum, each first normed over the model's width with a weight of its own,

    y = (N(a(h)) * w_a + N(b(h)) * w_b) / 2,      N(v) = v / sqrt(mean(v^2) + eps);

``weighted``: their sum with one factor each, ``y = s_a a(h) + s_b b(h)`` (``scales``), without norms or weights.

The branches are registered mixers of any kind, built from their own parameters; at most one of them may keep
keys and values in pages (a run has one paged cache), both may keep state in the slot under different names.
Each branch names the position table it reads (an entry of the model's positions) or none.  The two norms and
the mean are not computed here: the result is handed on as a :class:`BranchMean` (or, weighted, as a
:class:`ScaledSum`), which the next norm's kernel computes while it adds.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from ..config.registry import part_class, register_part
from ..weights.loader import VECTOR, WeightSpec
from .base import BranchMean, KVNeed, Part, RunInfo, ScaledSum, StateNeed


class SideBySide(Part):
    """params: ``hidden``, ``eps``, ``name``, ``combine`` (``normed_mean`` or ``weighted``), ``scales`` (the two
    factors of ``weighted``), ``branches``: a list of two ``{"kind", "params", "position", "out"}`` (a registered
    mixer kind, its parameters, the name of its position table or None, and, for ``normed_mean``, the leaf name of
    the weight of the norm behind it, ``<prefix>.<name>.<out>``)."""

    family = "mixer"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.eps = int(params["hidden"]), float(params["eps"])
        self.combine = params.get("combine") or "normed_mean"
        if self.combine not in ("normed_mean", "weighted"):
            raise ValueError(f"side_by_side: combine {self.combine!r} is not one of 'normed_mean', 'weighted'")
        self.scales = [float(v) for v in (params.get("scales") or (1.0, 1.0))]
        self.branch_specs = list(params["branches"])
        if len(self.branch_specs) != 2:
            raise ValueError("side_by_side is built for two branches")
        self.mixers = [part_class("mixer", b["kind"])(b["params"], prefix, dtype, device) for b in self.branch_specs]
        self.out_weights: List[torch.Tensor] = []

    def subparts(self) -> list:
        return list(self.mixers)

    @classmethod
    def _out_name(cls, prefix, params, branch) -> str:
        return cls.full_name(prefix, params, branch["out"])

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        specs = []
        for b in params["branches"]:
            specs += part_class("mixer", b["kind"]).weight_specs(b["params"], prefix)
            if (params.get("combine") or "normed_mean") == "normed_mean":
                specs.append(WeightSpec(cls._out_name(prefix, params, b), (int(params["hidden"]),), VECTOR, init="one_plus_normal"))
        return specs

    @classmethod
    def kv_need(cls, params: Dict[str, Any]) -> Optional[KVNeed]:
        needs = [n for n in (part_class("mixer", b["kind"]).kv_need(b["params"]) for b in params["branches"]) if n is not None]
        if len(needs) > 1:
            raise ValueError("side_by_side: both branches ask for a paged cache; a run has one")
        return needs[0] if needs else None

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        out = []
        for b in params["branches"]:
            out += part_class("mixer", b["kind"]).state_needs(b["params"])
        return out

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for m in self.mixers:
            m.load(tensors)
        if self.combine == "weighted":
            self.out_weights = list(self.scales)
            return
        self.out_weights = [tensors.pop(self._out_name(self.prefix, self.params, b)).to(torch.float32).contiguous()
                            for b in self.branch_specs]

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position):
        outs = []
        for m, b, w in zip(self.mixers, self.branch_specs, self.out_weights):
            pos = ctx.position_tables.get(b["position"]) if b.get("position") else None
            outs.append((m.forward(x, ctx, run, pos), w))
        return ScaledSum(outs) if self.combine == "weighted" else BranchMean(outs, self.eps)


register_part("mixer", "side_by_side", SideBySide)
