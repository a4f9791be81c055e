"""Root-mean-square norm fused with the residual sum.

``residual += delta;  out = residual * rsqrt(mean(residual^2) + eps) * weight``
in float32 on the float32 residual stream, rounded once on output
(reference: runtime/backends/cuda/native/cuda_kernels.cu:469-501 norm,
:541-579 fused add + norm; call sites
runtime/backends/cuda/native/transformer_forward.cu:1413-1424,1744-1754).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import VECTOR, WeightSpec
from .base import BranchMean, NormedDelta, Part, PartialSums, ScaledSum


class RMSNorm(Part):
    """params: ``hidden``, ``eps``, and the weight's name: ``name`` (weight is ``<prefix>.<name>.weight``) or
    ``weight_name`` (the leaf itself, ``<prefix>.<weight_name>``).

    ``delta`` may also be a :class:`NormedDelta` (a sublayer's result that is normed before it joins the
    stream, itself possibly the mean of two normed branches): both norms and the sum are one kernel."""

    family = "norm"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def _weight_name(cls, prefix, params) -> str:
        if params.get("weight_name"):
            return ".".join(p for p in (prefix, params["weight_name"]) if p)
        return cls.full_name(prefix, params, "weight")

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        return [WeightSpec(cls._weight_name(prefix, params), (int(params["hidden"]),), VECTOR, init="one_plus_normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self._weight_name(self.prefix, self.params)].to(torch.float32).contiguous()

    def forward(self, residual: torch.Tensor, delta, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Adds ``delta`` (a tensor, a :class:`PartialSums` or None) into the
        float32 ``residual`` (unless ``rows`` picks rows, which leaves it
        untouched) and returns the normed rows in the engine's type."""
        n_partials = 1
        n_rows = rows.numel() if rows is not None else residual.shape[0]
        if out is None:
            out = torch.empty((n_rows, self.hidden), dtype=self.dtype, device=residual.device)
        if isinstance(delta, NormedDelta):
            return normed_sum(residual, delta, self.weight, out, rows)
        if isinstance(delta, PartialSums):
            delta, n_partials = delta.tensor, delta.count
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows, n_partials)


def _sums(v) -> torch.Tensor:
    """float32 sums as the chain kernel takes them: ``[N, H]`` or slices ``[P, N, H]``."""
    if isinstance(v, PartialSums):
        return v.tensor
    if v.dtype != torch.float32:
        raise TypeError("a normed delta is made of float32 sums; a part gave " + str(v.dtype))
    return v


def normed_sum(residual: torch.Tensor, delta: NormedDelta, w_next: Optional[torch.Tensor], out: Optional[torch.Tensor],
               rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``residual += N(value) * delta.weight`` and, with ``w_next``, ``out = N(residual) * w_next``, in one kernel;
    ``value`` may be the mean of two normed branches."""
    v = delta.value
    if isinstance(v, BranchMean):
        if len(v.branches) != 2:
            raise ValueError("the mean of normed branches is built for two branches")
        (a, wa), (b, wb) = v.branches
        return ops.norm_chain(residual, _sums(a), delta.eps, w_a=wa, b=_sums(b), w_b=wb, w_post=delta.weight,
                              w_next=w_next, out=out, rows=rows)
    return ops.norm_chain(residual, _sums(v), delta.eps, w_post=delta.weight, w_next=w_next, out=out, rows=rows)


class LayerNorm(Part):
    """Layer norm with a weight and no bias, fused with the residual sum:
    ``residual += delta;  out = (r - mean(r)) / sqrt(mean((r - mean(r))^2) + eps) * weight``
    in float32.  params: ``hidden``, ``eps``, and the weight's name: ``name``
    (weight is ``<prefix>.<name>.weight``) or ``weight_name`` (the leaf itself,
    ``<prefix>.<weight_name>``)."""

    family = "norm"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def _weight_name(cls, prefix, params) -> str:
        if params.get("weight_name"):
            return ".".join(p for p in (prefix, params["weight_name"]) if p)
        return cls.full_name(prefix, params, "weight")

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        return [WeightSpec(cls._weight_name(prefix, params), (int(params["hidden"]),), VECTOR, init="one_plus_normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self._weight_name(self.prefix, self.params)].to(torch.float32).contiguous()

    def forward(self, residual: torch.Tensor, delta, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, out32: Optional[torch.Tensor] = None) -> torch.Tensor:
        """As :meth:`RMSNorm.forward`; ``out32`` (float32 ``[rows, hidden]``)
        takes the normed rows unrounded as well."""
        n_partials = 1
        if isinstance(delta, PartialSums):
            delta, n_partials = delta.tensor, delta.count
        n_rows = rows.numel() if rows is not None else residual.shape[0]
        if out is None:
            out = torch.empty((n_rows, self.hidden), dtype=self.dtype, device=residual.device)
        return ops.add_layernorm(residual, delta, self.weight, self.eps, out, rows, n_partials, out32)


class GroupRMSNorm(RMSNorm):
    """RMS norm over ``groups`` equal consecutive parts of the row, each divided by its own root mean square, the whole
    multiplied by one weight of the row's length; fused with the sum into the stream like :class:`RMSNorm`.
    ``delta`` may also be a :class:`ScaledSum` of two branches: the weighted sum, the sum into the stream and the norm
    are one kernel.  params: those of ``rmsnorm`` and ``groups`` (default 1, which is the plain norm)."""

    family = "norm"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.groups = int(params.get("groups") or 1)
        if self.groups < 1 or self.hidden % self.groups:
            raise ValueError(f"group_rmsnorm: {self.groups} groups do not divide a row of {self.hidden}")

    def forward(self, residual: torch.Tensor, delta, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n_rows = rows.numel() if rows is not None else residual.shape[0]
        if out is None:
            out = torch.empty((n_rows, self.hidden), dtype=self.dtype, device=residual.device)
        if isinstance(delta, NormedDelta) or isinstance(delta, BranchMean):
            raise TypeError("group_rmsnorm takes a tensor, partial sums or a weighted sum of two branches")
        terms = delta.terms if isinstance(delta, ScaledSum) else ([(delta, 1.0)] if delta is not None else [])
        if len(terms) > 2:
            raise ValueError("a weighted sum is built for two branches")
        flat = [((v.tensor if isinstance(v, PartialSums) else v), float(f)) for v, f in terms] + [(None, 1.0)] * (2 - len(terms))
        (a, fa), (b, fb) = flat
        if rows is not None and (a is not None or b is not None):
            # picked rows leave the stream untouched: the pending sum goes in first
            ops.add_group_rmsnorm(residual, a, self.weight, self.eps, self.groups, None, None, fa, b, fb)
            a = b = None
        return ops.add_group_rmsnorm(residual, a, self.weight, self.eps, self.groups, out, rows, fa, b, fb)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "group_rmsnorm", GroupRMSNorm)
register_part("norm", "layernorm", LayerNorm)
