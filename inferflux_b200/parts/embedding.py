"""Token embedding and output head.

Embedding: ``residual[t, :] = float32(E[id_t, :])``, no scale (reference:
runtime/backends/cuda/native/cuda_kernels.cu:599-614).  Output head:
``logits = x W^T`` with ``W = lm_head.weight [V, H]`` or the embedding table
when the head is tied (reference falls back to the embedding when
``lm_head.weight`` is absent, runtime/backends/cuda/native/weight_map.cpp:33-37);
logits come out in float32 (the reference rounds them to 16 bits first,
transformer_forward.cu:2178-2189).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import IGNORED, MATRIX, VECTOR, WeightSpec
from .base import Part
from .linear import Linear


class TokenEmbedding(Part):
    """params: ``vocab``, ``hidden``, ``name`` (weight ``<name>.weight``) or ``weight_name`` (the table's full name),
    ``scale`` (default 1: the float32 row is multiplied by it)."""

    family = "embedding"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.scale = float(params.get("scale", 1.0))
        self.table: torch.Tensor = None

    @classmethod
    def _table_name(cls, prefix, params) -> str:
        return params.get("weight_name") or cls.full_name(prefix, params, "weight")

    @classmethod
    def weight_specs(cls, params, prefix) -> List[WeightSpec]:
        return [WeightSpec(cls._table_name(prefix, params), (int(params["vocab"]), int(params["hidden"])), MATRIX,
                           std=float(params.get("std", 0.02)))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self._table_name(self.prefix, self.params)].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        return ops.embed_gather(self.table, token_ids, out, self.scale)

    def forward_step(self, ctx) -> torch.Tensor:
        return self.forward(ctx.token_ids)


class SinusoidNormEmbedding(Part):
    """Token embedding plus a sinusoidal position vector, then a layer norm:

        x = E[id] + P(pos),  P[2i] = sin(pos * base^(-2i/hidden)),  P[2i+1] = cos(the same angle)
        out = (x - mean) / sqrt(var + eps) * w

    in one kernel (angles in float64, the rest float32).  params: ``vocab``,
    ``hidden``, ``eps``, ``base`` (default 10000), ``table`` and
    ``norm_weight`` (the full names of the two tensors)."""

    family = "embedding"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.eps, self.base = float(params["eps"]), float(params.get("base", 10000.0))
        self.table: torch.Tensor = None
        self.weight: torch.Tensor = None

    @classmethod
    def weight_specs(cls, params, prefix) -> List[WeightSpec]:
        v, h = int(params["vocab"]), int(params["hidden"])
        return [WeightSpec(params["table"], (v, h), MATRIX, std=float(params.get("std", 0.02))),
                WeightSpec(params["norm_weight"], (h,), VECTOR, init="one_plus_normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.params["table"]].contiguous()
        self.weight = tensors[self.params["norm_weight"]].to(torch.float32).contiguous()

    def forward_step(self, ctx) -> torch.Tensor:
        out = torch.empty((ctx.token_ids.numel(), self.hidden), dtype=torch.float32, device=ctx.token_ids.device)
        return ops.embed_sinusoid_layernorm(self.table, ctx.token_ids, ctx.positions, self.weight, self.eps, self.base, out)


class LinearHead(Part):
    """params: ``vocab``, ``hidden``, ``name``, ``tied_to`` (None, or the full
    name of the embedding table to use instead of a weight of its own),
    ``weight_name`` (the weight's full name where it is not ``<name>.weight``),
    ``scale`` (a factor on the float32 logits, default 1)."""

    family = "lm_head"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.scale = float(params.get("scale", 1.0) or 1.0)
        self.linear: Linear = None

    @classmethod
    def _own_name(cls, prefix, params) -> str:
        return params.get("weight_name") or cls.full_name(prefix, params, "weight")

    @classmethod
    def weight_specs(cls, params, prefix) -> List[WeightSpec]:
        shape = (int(params["vocab"]), int(params["hidden"]))
        name = cls._own_name(prefix, params)
        if params.get("tied_to"):
            return [WeightSpec(name, shape, IGNORED, optional=True)]
        return [WeightSpec(name, shape, MATRIX)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        src = self.params.get("tied_to") or self._own_name(self.prefix, self.params)
        self.linear = Linear(tensors[src])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [W, hidden] -> float32 logits [W, vocab]."""
        logits = self.linear.forward(x, out_dtype=torch.float32)
        return logits if self.scale == 1.0 else logits.mul_(self.scale)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "sinusoid_norm_embedding", SinusoidNormEmbedding)
register_part("lm_head", "linear_head", LinearHead)
