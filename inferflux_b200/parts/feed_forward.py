"""Feed-forward parts.

``swiglu``: ``down( silu(gate(x)) * up(x) )`` with ``silu(g) = g / (1 + exp(-g))``
in float32, no biases (reference:
runtime/backends/cuda/native/transformer_forward.cu:1877-1879,1912-1914 gate
and up, :1981-1983 activation, :2024-2026 down;
runtime/backends/cuda/native/cuda_kernels.cu:137-149).  The reference runs
gate and up as two products and the activation as a kernel of its own; here
their weights are stacked at load and in bfloat16 one kernel does the product
and the activation, so the ``[gate | up]`` intermediate never goes to memory:
the weight-streaming kernel for a few rows, the tcgen05 product for many.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import Part, PartialSums
from .linear import Linear


FUSED_PRODUCT_ROWS = 128   # above this many rows gate/up + activation run as one tcgen05 product (measured: 256 rows 63 us
                           # against 76 us for library product + activation kernel; at 64 rows the library is ahead)


class SwiGLU(Part):
    """params: ``hidden``, ``intermediate``, ``name`` (weights are
    ``<prefix>.<name>.{gate,up,down}_proj.weight``)."""

    family = "feed_forward"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.gate_up: Linear = None
        self.down: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("gate_proj.weight"), (i, h), MATRIX),
                WeightSpec(n("up_proj.weight"), (i, h), MATRIX),
                WeightSpec(n("down_proj.weight"), (h, i), MATRIX)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        gate, up = tensors.pop(n("gate_proj.weight")), tensors.pop(n("up_proj.weight"))
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.gate_up = Linear(torch.cat([gate, up], dim=0))
        del gate, up
        self.down = Linear(tensors.pop(n("down_proj.weight")))

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        w = self.gate_up.weight
        act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        fused = w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and self.hidden % 8 == 0
        if fused and x.shape[0] <= ops.GEMV_MAX_ROWS:         # (up to 16 rows the fused kernel beats library product + activation)
            ops.gemv_bf16(x, w, None, act, swiglu=True)       # product and activation in one kernel
        elif fused and x.is_contiguous() and x.shape[0] > FUSED_PRODUCT_ROWS:
            ops.gemm_umma(x, w, None, act, swiglu=True)       # many rows: tcgen05 product, activation in its epilogue
        else:
            ops.swiglu(self.gate_up.forward(x), act)
        return self.down.forward(act, out_dtype=x.dtype, allow_partials=True)


class PolyNormFF(Part):
    """``down( act( up(x) + b_up ) ) + b_down`` with the PolyNorm activation

        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,   N(v) = v / sqrt(mean(v^2) + eps) over a token's row,

    powers taken element by element; a, b, c, e are four numbers of the layer.
    The up projection leaves float32 sums; bias, the three mean squares and the
    activation are one kernel in float32.  params: ``hidden``, ``intermediate``,
    ``eps``, ``name`` (tensors ``<prefix>.<name>.{up,up.b,down,down.b,act}``)."""

    family = "feed_forward"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.eps = float(params["eps"])
        self.up: Linear = None
        self.up_bias: torch.Tensor = None
        self.down: Linear = None
        self.coeff: torch.Tensor = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("up"), (i, h), MATRIX), WeightSpec(n("up.b"), (i,), VECTOR),
                WeightSpec(n("down"), (h, i), MATRIX), WeightSpec(n("down.b"), (h,), VECTOR),
                WeightSpec(n("act"), (4,), VECTOR, std=0.5)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        self.up = Linear(tensors.pop(n("up")))
        self.up_bias = tensors.pop(n("up.b")).to(torch.float32).contiguous()
        self.down = Linear(tensors.pop(n("down")), tensors.pop(n("down.b")))
        self.coeff = tensors.pop(n("act")).to(torch.float32).contiguous()

    def inner(self, x: torch.Tensor, ctx, out: torch.Tensor = None) -> torch.Tensor:
        """The activated rows ``[N, intermediate]`` that the down projection takes."""
        z = self.up.forward(x, out_dtype=torch.float32)
        if out is None:
            out = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        return ops.polynorm(z, self.up_bias, self.coeff, self.eps, out)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return self.down.forward(self.inner(x, ctx), out_dtype=torch.float32)


class GeluMLP(Part):
    """``down( gelu(up(x)) )`` with the tanh form of gelu, ``0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``,
    and no biases.  The up projection leaves float32 sums; the activation rounds once into the engine's type.
    params: ``hidden``, ``intermediate``, ``name`` (tensors ``<prefix>.<name>.{up,down}``)."""

    family = "feed_forward"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.up: Linear = None
        self.down: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("up"), (i, h), MATRIX), WeightSpec(n("down"), (h, i), MATRIX)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        self.up, self.down = Linear(tensors.pop(n("up"))), Linear(tensors.pop(n("down")))

    def forward(self, x: torch.Tensor, ctx):
        z = self.up.forward(x, out_dtype=torch.float32, allow_partials=True, f32_sums=True)
        act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        ops.gelu_tanh(z.tensor if isinstance(z, PartialSums) else z, act)
        return self.down.forward(act, out_dtype=torch.float32, allow_partials=True, f32_sums=True)


class ClampedGLU(Part):
    """A gated feed-forward whose two inputs are clamped before they meet:

        g = min(W_gate x + b_gate, limit)          u = clamp(W_up x + b_up, -limit, limit)
        y = W_down ( g * sigmoid(alpha * g) * (u + shift) ) + b_down

    Gate and up are one stacked projection whose sums stay float32; biases, clamps and the activation are one
    kernel that rounds once into the engine's type.  params: ``hidden``, ``intermediate``, ``limit``, ``alpha``
    (default 1.702), ``shift`` (default 1), ``bias`` (default true), ``name`` (tensors
    ``<prefix>.<name>.{gate,up,down}`` and ``.{gate,up,down}.b``)."""

    family = "feed_forward"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.limit = float(params["limit"])
        self.alpha, self.shift = float(params.get("alpha", 1.702)), float(params.get("shift", 1.0))
        self.has_bias = bool(params.get("bias", True))
        self.gate_up: Linear = None
        self.gate_up_bias: torch.Tensor = None
        self.down: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        specs = [WeightSpec(n("gate"), (i, h), MATRIX), WeightSpec(n("up"), (i, h), MATRIX), WeightSpec(n("down"), (h, i), MATRIX)]
        if params.get("bias", True):
            specs += [WeightSpec(n("gate.b"), (i,), VECTOR), WeightSpec(n("up.b"), (i,), VECTOR), WeightSpec(n("down.b"), (h,), VECTOR)]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        gate, up = tensors.pop(n("gate")), tensors.pop(n("up"))
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.gate_up = Linear(torch.cat([gate, up], dim=0))
        del gate, up
        if self.has_bias:
            self.gate_up_bias = torch.cat([tensors.pop(n("gate.b")).float(), tensors.pop(n("up.b")).float()]).contiguous()
        self.down = Linear(tensors.pop(n("down")), tensors.pop(n("down.b")) if self.has_bias else None)

    def forward(self, x: torch.Tensor, ctx):
        z = self.gate_up.forward(x, out_dtype=torch.float32, allow_partials=True, f32_sums=True)
        act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        ops.glu_clamped(z.tensor if isinstance(z, PartialSums) else z, self.gate_up_bias, act, self.limit, self.alpha, self.shift)
        return self.down.forward(act, out_dtype=torch.float32, allow_partials=True, f32_sums=True)


class SquaredReluMLP(Part):
    """``down( relu(up(x))^2 )``, no biases.  The up projection leaves float32 sums; the activation rounds once into
    the engine's type.  params: ``hidden``, ``intermediate``, ``name`` (tensors ``<prefix>.<name>.{up,down}``)."""

    family = "feed_forward"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.up: Linear = None
        self.down: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("up"), (i, h), MATRIX), WeightSpec(n("down"), (h, i), MATRIX)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        self.up, self.down = Linear(tensors.pop(n("up"))), Linear(tensors.pop(n("down")))

    def forward(self, x: torch.Tensor, ctx):
        z = self.up.forward(x, out_dtype=torch.float32, allow_partials=True, f32_sums=True)
        act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        ops.activation(z.tensor if isinstance(z, PartialSums) else z, act, ops.ACT_RELU2)
        return self.down.forward(act, out_dtype=torch.float32, allow_partials=True, f32_sums=True)


class RoutedExperts(Part):
    """A mixture of experts: every token runs the ``top`` experts with the largest router logits and adds their
    results, weighted.

        z = W_router x (+ b)          float32 (x may be the engine type's rounding)
        ``route`` ``chosen``:  weights = softmax over the chosen logits alone
        ``route`` ``all``:     s = softmax(z) over every expert; weights = the chosen s over their sum (+ 1e-20)
        either times ``scale``
        expert e, ``activation`` ``swiglu``:  W_down_e ( silu(W_gate_e x) * (W_up_e x) )
                  ``activation`` ``relu2``:   W_down_e ( relu(W_up_e x)^2 )                      no biases
        ``shared`` (an intermediate size): one more expert of the ``relu2`` form that every token runs, added unweighted

    The experts' matrices are stacked at load; the (token, expert) pairs are sorted by expert on the device and
    run as tiles of one expert each, so nothing waits for the host and a step of single tokens is captured like
    any other.  params: ``hidden``, ``intermediate`` (of one expert), ``experts``, ``top``, ``activation``, ``route``,
    ``scale``, ``router_bias`` (default true), ``shared``, ``name`` (tensors ``<prefix>.<name>.router``, ``.router.b``,
    ``.e<i>.{gate,up,down}``, ``.shared.{up,down}``)."""

    family = "feed_forward"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.experts, self.top = int(params["experts"]), int(params["top"])
        if not 1 <= self.top <= min(self.experts, 64):
            raise ValueError(f"routed_experts: top {self.top} must be within 1..min(experts, 64)")
        self.activation = {"swiglu": ops.MOE_SWIGLU, "relu2": ops.MOE_RELU2}.get(params.get("activation", "swiglu"))
        self.over_all = {"chosen": False, "all": True}.get(params.get("route", "chosen"))
        if self.activation is None or self.over_all is None:
            raise ValueError("routed_experts: activation is 'swiglu' or 'relu2', route is 'chosen' or 'all'")
        self.scale = float(params.get("scale", 1.0))
        self.shared = self._shared(params, prefix, dtype, device)
        self.router: Linear = None
        self.gate_up: torch.Tensor = None
        self.down: torch.Tensor = None

    @classmethod
    def _shared(cls, params, prefix, dtype=None, device=None):
        """The shared expert as a part of its own (or its class and parameters, for the weight list)."""
        if not params.get("shared"):
            return None
        sp = dict(name=cls.full_name("", params, "shared"), hidden=int(params["hidden"]), intermediate=int(params["shared"]))
        return SquaredReluMLP(sp, prefix, dtype, device) if dtype is not None else sp

    def subparts(self) -> list:
        return [self.shared] if self.shared is not None else []

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, i, e = int(params["hidden"]), int(params["intermediate"]), int(params["experts"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        specs = [WeightSpec(n("router"), (e, h), MATRIX, std=0.5)]
        if params.get("router_bias", True):
            specs.append(WeightSpec(n("router.b"), (e,), VECTOR, std=0.5))
        mats = ("gate", "up") if params.get("activation", "swiglu") == "swiglu" else ("up",)
        for k in range(e):
            specs += [WeightSpec(n(f"e{k}.{x}"), (i, h), MATRIX) for x in mats] + [WeightSpec(n(f"e{k}.down"), (h, i), MATRIX)]
        sp = cls._shared(params, prefix)
        if sp is not None:
            specs += SquaredReluMLP.weight_specs(sp, prefix)
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        # The router's products are 32-bit whatever the engine: a bfloat16 weight times a bfloat16 input is exact
        # in float32, and the sums are float32 (the library's product or the weight-streaming kernel).
        self.router = Linear(tensors.pop(n("router")), tensors.pop(n("router.b")) if self.params.get("router_bias", True) else None)
        ups = ("gate", "up") if self.activation == ops.MOE_SWIGLU else ("up",)
        mats = [[tensors.pop(n(f"e{k}.{x}")) for x in (*ups, "down")] for k in range(self.experts)]
        kinds = {m.dtype for row in mats for m in row}
        cast = (lambda m: m.float()) if len(kinds) > 1 else (lambda m: m)
        self.gate_up = torch.stack([torch.cat([cast(m) for m in row[:-1]], dim=0) for row in mats]).contiguous()
        self.down = torch.stack([cast(row[-1]) for row in mats]).contiguous()
        if self.shared is not None:
            self.shared.load(tensors)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        logits = self.router.forward(x, out_dtype=torch.float32)
        chosen, weights = ops.moe_route(logits, self.top, self.over_all, self.scale)
        xe = x
        if x.dtype != self.gate_up.dtype:
            xe = ops.convert(x.contiguous(), torch.empty(x.shape, dtype=self.gate_up.dtype, device=x.device))
        out = ops.moe_experts(xe.contiguous(), self.gate_up, self.down, chosen, weights, self.activation)
        if self.shared is not None:
            y = self.shared.forward(x, ctx)
            y, parts = (y.tensor, y.count) if isinstance(y, PartialSums) else (y, 1)
            ops.add_into(out, y, parts)
        return out


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "gelu_mlp", GeluMLP)
register_part("feed_forward", "clamped_glu", ClampedGLU)
register_part("feed_forward", "routed_experts", RoutedExperts)
register_part("feed_forward", "relu2_mlp", SquaredReluMLP)
register_part("feed_forward", "polynorm", PolyNormFF)
