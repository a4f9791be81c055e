"""How a layer's parts are arranged.

``prenorm`` (the reference's only block,
runtime/backends/cuda/native/transformer_forward.cu:1400-2103):

    x  = norm_1(residual)          residual is the float32 stream
    residual += mixer(x)
    x2 = norm_2(residual)
    residual += feed_forward(x2)

The second sum is not done here: the block returns the feed-forward's output
as a pending delta, and the next block's first norm (or the final norm) adds
it in the same kernel that norms (the reference fuses the same pair,
transformer_forward.cu:2054-2077).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from .base import NormedDelta, PartialSums, RunInfo, ScaledSum
from .linear import Linear
from .norm import normed_sum


class PreNormBlock:
    """An arrangement declares its roles (role -> family of the part that fills
    it) and is built from the layer's parts by role; ``optional_roles`` may be
    left out of a layer."""

    family = "arrangement"
    roles = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}
    optional_roles = frozenset({"feed_forward", "feed_forward_norm"})       # a layer may have no feed-forward

    def __init__(self, parts: Dict[str, object], position_name: Optional[str]):
        self.mixer = parts["mixer"]
        self.mixer_norm = parts["mixer_norm"]
        self.feed_forward = parts.get("feed_forward")
        self.feed_forward_norm = parts.get("feed_forward_norm")
        if (self.feed_forward is None) != (self.feed_forward_norm is None):
            raise ValueError("a prenorm block has a feed-forward with the norm ahead of it or neither")
        self.position_name = position_name

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx, run: RunInfo) -> torch.Tensor:
        """residual float32 [N, H] (updated in place); delta = the previous
        block's pending output or None.  Returns this block's pending output."""
        x = self.mixer_norm.forward(residual, delta)
        position = ctx.position_tables.get(self.position_name) if self.position_name else None
        a = self.mixer.forward(x, ctx, run, position)
        if self.feed_forward is None:
            return a
        x2 = self.feed_forward_norm.forward(residual, a)
        return self.feed_forward.forward(x2, ctx)


register_part("arrangement", "prenorm", PreNormBlock)


class ParallelBlock:
    """One norm, both branches read it, one sum:

        h = norm(residual);   residual += mixer(shift(h)) + feed_forward(h)

    ``shift`` (optional) mixes what the mixer reads with the token before it;
    the feed-forward reads ``h`` as it is and may be left out of a layer.
    When mixer and feed-forward both offer ``inner`` (their rows before the
    output projection) and an output Linear (``o``, ``down``), the two output
    projections run as one product over the rows side by side,
    ``[inner_mixer | inner_ff] [W_o | W_down]^T + b_down``, whose float32 sums
    are the block's pending delta.  In a step of single tokens the residual
    sum, the norm, the shift and the update of the shift's state are one kernel.
    """

    family = "arrangement"
    roles = {"norm": "norm", "shift": "shift", "mixer": "mixer", "feed_forward": "feed_forward"}
    optional_roles = frozenset({"shift", "feed_forward"})
    #: Switches for tests and measurements: the two output projections as one product; sum, norm, shift and
    #: state update of a single-token step as one kernel.  Off, the block runs its parts one by one.
    JOINT_OUTPUT = True
    FUSED_SINGLE = True

    def __init__(self, parts: Dict[str, object], position_name: Optional[str]):
        self.norm = parts["norm"]
        self.shift = parts.get("shift")
        self.mixer = parts["mixer"]
        self.feed_forward = parts.get("feed_forward")
        self.position_name = position_name
        self._joint = None                    # Linear over [W_o | W_down], built at the first step

    def _joint_output(self):
        """The two output projections as one Linear, if the parts allow it."""
        if self._joint is None:
            self._joint = False
            if not self.JOINT_OUTPUT:
                return False
            m, f = self.mixer, self.feed_forward
            if (f is not None and hasattr(m, "inner") and hasattr(f, "inner") and getattr(m, "o", None) is not None
                    and getattr(f, "down", None) is not None and m.o.bias is None
                    and m.o.weight.dtype == f.down.weight.dtype):
                self._joint = Linear(torch.cat([m.o.weight, f.down.weight], dim=1), f.down.bias)
                self._widths = (m.o.in_features, f.down.in_features)
                m.o = f.down = None           # the joint matrix replaces them
        return self._joint

    def forward(self, residual: torch.Tensor, delta, ctx, run: RunInfo):
        n = residual.shape[0]
        position = ctx.position_tables.get(self.position_name) if self.position_name else None
        if self.shift is None:
            h = hs = self.norm.forward(residual, delta)
        elif self.FUSED_SINGLE and ctx.max_q_len == 1 and hasattr(self.norm, "weight") and hasattr(self.shift, "mu"):
            n_partials = 1
            if isinstance(delta, PartialSums):
                delta, n_partials = delta.tensor, delta.count
            h = torch.empty((n, residual.shape[1]), dtype=ctx.dtype, device=residual.device)
            hs = torch.empty_like(h)
            ops.add_layernorm_shift1(residual, delta, self.norm.weight, self.norm.eps, self.shift.mu,
                                     run.states["shift_prev"], ctx.entry_slot, h, hs, n_partials)
        elif ctx.dtype == torch.float32:
            h = self.norm.forward(residual, delta)
            hs = self.shift.forward(h, ctx, run)
        else:
            h32 = torch.empty((n, residual.shape[1]), dtype=torch.float32, device=residual.device)
            h = self.norm.forward(residual, delta, out32=h32)
            hs = self.shift.forward(h32, ctx, run)
        joint = self._joint_output()
        if joint:
            wm, wf = self._widths
            both = torch.empty((n, wm + wf), dtype=ctx.dtype, device=residual.device)
            self.mixer.inner(hs, ctx, run, position, out=both[:, :wm])
            self.feed_forward.inner(h, ctx, out=both[:, wm:])
            return joint.forward(both, out_dtype=torch.float32, allow_partials=True, f32_sums=True)
        a = self.mixer.forward(hs, ctx, run, position)
        if self.feed_forward is None:
            return a
        f = self.feed_forward.forward(h, ctx)
        dense = lambda y: y.tensor.sum(0) if isinstance(y, PartialSums) else y.float()
        return dense(a).add_(dense(f))


class JunctionBlock:
    """An arrangement that is no layer: the pending delta goes into the stream,
    then its one part (family ``junction``) rewrites the stream in place."""

    family = "arrangement"
    roles = {"junction": "junction"}
    optional_roles = frozenset()
    needs_embedding_output = True

    def __init__(self, parts: Dict[str, object], position_name: Optional[str]):
        self.junction = parts["junction"]

    def forward(self, residual: torch.Tensor, delta, ctx, run: RunInfo):
        if isinstance(delta, ScaledSum):
            for value, factor in delta.terms:
                t = value.tensor.sum(0) if isinstance(value, PartialSums) else value
                residual.add_(t, alpha=float(factor))
        elif delta is not None:
            n_partials = 1
            if isinstance(delta, PartialSums):
                delta, n_partials = delta.tensor, delta.count
            ops.add_into(residual, delta, n_partials)
        self.junction.forward(residual, ctx, run)
        return None


class PrePostNormBlock:
    """A norm ahead of and a norm behind every sublayer:

        residual += norm_1b(mixer(norm_1(residual)))
        residual += norm_2b(feed_forward(norm_2(residual)))         (a layer may have no feed-forward)

    A sublayer's result is not added here: it goes on as a :class:`NormedDelta` with the weight of the norm
    behind it, and the next norm ahead (this block's second, the next block's first, or the model's last) norms
    it, adds it to the stream and norms the stream in one kernel.  Norms of the kind ``rmsnorm`` take such a
    delta."""

    family = "arrangement"
    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    optional_roles = frozenset({"feed_forward_norm", "feed_forward", "feed_forward_post_norm"})

    def __init__(self, parts: Dict[str, object], position_name: Optional[str]):
        self.mixer_norm, self.mixer, self.mixer_post = parts["mixer_norm"], parts["mixer"], parts["mixer_post_norm"]
        self.ff_norm, self.ff, self.ff_post = (parts.get(r) for r in ("feed_forward_norm", "feed_forward",
                                                                      "feed_forward_post_norm"))
        if (self.ff is None) != (self.ff_norm is None) or (self.ff is None) != (self.ff_post is None):
            raise ValueError("a pre_post_norm block has a feed-forward with both of its norms or none of the three")
        self.position_name = position_name

    def forward(self, residual: torch.Tensor, delta, ctx, run: RunInfo):
        x = self.mixer_norm.forward(residual, delta)
        position = ctx.position_tables.get(self.position_name) if self.position_name else None
        a = NormedDelta(self.mixer.forward(x, ctx, run, position), self.mixer_post.weight, self.mixer_post.eps)
        if self.ff is None:
            return a
        x2 = self.ff_norm.forward(residual, a)
        return NormedDelta(self.ff.forward(x2, ctx), self.ff_post.weight, self.ff_post.eps)


class PostNormBlock:
    """A norm behind every sublayer and none ahead: the sublayers read the stream itself,

        residual += norm_1(mixer(residual))
        residual += norm_2(feed_forward(residual))                  (a layer may have no feed-forward)

    A sublayer's result is not added here: it goes on as a :class:`NormedDelta` with the weight of the norm
    behind it.  The next reader of the stream (this block's feed-forward, the next block's mixer, or the model's
    last norm) norms it and adds it to the float32 stream in one kernel, which also hands out the stream rounded
    into the engine's type for the sublayer's products (a float32 engine reads the stream in place)."""

    family = "arrangement"
    roles = {"mixer": "mixer", "mixer_post_norm": "norm", "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    optional_roles = frozenset({"feed_forward", "feed_forward_post_norm"})

    def __init__(self, parts: Dict[str, object], position_name: Optional[str]):
        self.mixer, self.mixer_post = parts["mixer"], parts["mixer_post_norm"]
        self.ff, self.ff_post = parts.get("feed_forward"), parts.get("feed_forward_post_norm")
        if (self.ff is None) != (self.ff_post is None):
            raise ValueError("a post_norm block has a feed-forward with the norm behind it or neither")
        self.position_name = position_name

    @staticmethod
    def _read(residual: torch.Tensor, delta, ctx) -> torch.Tensor:
        """Adds the pending delta into the stream and returns what a sublayer reads: the stream in the engine's type."""
        if ctx.dtype == torch.float32:
            if isinstance(delta, NormedDelta):
                normed_sum(residual, delta, None, None)
            elif delta is not None:
                d, n = (delta.tensor, delta.count) if isinstance(delta, PartialSums) else (delta, 1)
                ops.add_into(residual, d, n)
            return residual
        out = torch.empty(residual.shape, dtype=ctx.dtype, device=residual.device)
        if isinstance(delta, NormedDelta):
            return normed_sum(residual, delta, None, out)
        if delta is not None:
            d, n = (delta.tensor, delta.count) if isinstance(delta, PartialSums) else (delta, 1)
            ops.add_into(residual, d, n)
        return ops.convert(residual, out)

    def forward(self, residual: torch.Tensor, delta, ctx, run: RunInfo):
        x = self._read(residual, delta, ctx)
        position = ctx.position_tables.get(self.position_name) if self.position_name else None
        a = NormedDelta(self.mixer.forward(x, ctx, run, position), self.mixer_post.weight, self.mixer_post.eps)
        if self.ff is None:
            return a
        x2 = self._read(residual, a, ctx)
        return NormedDelta(self.ff.forward(x2, ctx), self.ff_post.weight, self.ff_post.eps)


register_part("arrangement", "pre_post_norm", PrePostNormBlock)
register_part("arrangement", "post_norm", PostNormBlock)
register_part("arrangement", "parallel", ParallelBlock)
register_part("arrangement", "junction", JunctionBlock)
