"""Parts that rewrite the stream between layers (family ``junction``).

``loop_entry``: where a pass over a stretch of layers begins, the stream is
renewed from itself and from the embedding output,

    x <- W_in [x ; x0] + step[t]          W_in [hidden, 2 hidden], step [passes, hidden]

``t`` being the number of the pass (the run's parameter ``pass``) and ``x0``
the stream as the embedding left it.  The half of the product that reads x0
is the same in every pass and is made once per step; the sum is float32.

``add_embedding``: ``x <- x + x0``, nothing else.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import Part, RunInfo
from .linear import Linear


class LoopEntry(Part):
    """params: ``hidden``, ``passes``, ``in_name``, ``step_name`` (full tensor names)."""

    family = "junction"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.passes = int(params["hidden"]), int(params["passes"])
        self.from_x: Linear = None
        self.from_x0: Linear = None
        self.step: torch.Tensor = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, t = int(params["hidden"]), int(params["passes"])
        return [WeightSpec(params["in_name"], (h, 2 * h), MATRIX, std=0.7 / h ** 0.5),
                WeightSpec(params["step_name"], (t, h), VECTOR)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.pop(self.params["in_name"])
        self.from_x = Linear(w[:, :self.hidden].contiguous())
        self.from_x0 = Linear(w[:, self.hidden:].contiguous())
        self.step = tensors.pop(self.params["step_name"]).to(torch.float32).contiguous()

    def _operand(self, t: torch.Tensor) -> torch.Tensor:
        if self.dtype == torch.float32:
            return t
        return ops.convert(t, torch.empty(t.shape, dtype=self.dtype, device=t.device))

    def forward(self, residual: torch.Tensor, ctx, run: RunInfo) -> None:
        key = ("loop_entry", id(self))
        base = ctx.scratch.get(key)
        if base is None:
            base = ctx.scratch[key] = self.from_x0.forward(self._operand(ctx.embedding_output), out_dtype=torch.float32)
        y = self.from_x.forward(self._operand(residual), out_dtype=torch.float32)
        ops.add_rows_vector(y, base, self.step[int(run.params["pass"])], residual)


class AddEmbedding(Part):
    """``x <- x + x0`` with ``x0`` the stream as the embedding left it: where a later pass over a stretch of layers
    begins, the tokens' embeddings join the stream again.  No weights; params: none."""

    family = "junction"

    def forward(self, residual: torch.Tensor, ctx, run: RunInfo) -> None:
        ops.add_into(residual, ctx.embedding_output, 1)


register_part("junction", "loop_entry", LoopEntry)
register_part("junction", "add_embedding", AddEmbedding)
