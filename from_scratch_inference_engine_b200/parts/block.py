"""Arrangements: how a layer's parts are wired around the residual stream."""

from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import LayerSpec
from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Part, build_part, register_part
from .norm import LayerNorm, NormedDelta, PendingSum, RMSNorm


@register_part("arrangement", "prenorm")
class PreNormBlock(Part):
    """x += mixer(norm(x)); x += feed_forward(norm(x))  (src/model/model.cpp:107-141).  A layer may
    have no feed-forward.

    The residual stream `x` is float32 and is updated in place.  A sublayer's output is
    not added at once: it is handed on as `delta` and added by the next norm kernel, which
    reads and writes x anyway.  forward returns the feed-forward's output as the new delta.
    """

    def __init__(self, prefix: str, layer: LayerSpec):
        self.prefix = prefix
        self.mixer_norm = build_part("norm", layer.mixer_norm, prefix + layer.mixer_norm_name)
        self.mixer = build_part("mixer", layer.mixer, prefix + layer.mixer_name)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:          # a layer may have no feed-forward
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm,
                                                prefix + layer.feed_forward_norm_name)
            self.feed_forward = build_part("feed_forward", layer.feed_forward,
                                           prefix + layer.feed_forward_name)
        # a checkpoint may still hold the norm of a feed-forward that the layer does not have
        self.unused: List[TensorSpec] = []
        if layer.feed_forward is None and layer.feed_forward_norm is not None:
            import dataclasses
            unused = build_part("norm", layer.feed_forward_norm, prefix + layer.feed_forward_norm_name)
            self.unused = [dataclasses.replace(spec, optional=True) for spec in unused.tensor_specs()]

    def parts(self):
        return [part for part in (self.mixer_norm, self.mixer, self.feed_forward_norm,
                                  self.feed_forward) if part is not None]

    @property
    def capturable(self) -> bool:
        return all(part.capturable for part in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        return [spec for part in self.parts() for spec in part.tensor_specs()] + self.unused

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(tensors, runtime)

    def forward(self, ctx, x: torch.Tensor, delta: Optional[torch.Tensor],
                cache: LayerCache) -> torch.Tensor:
        ctx.residual_copy = None      # this block changes x without keeping a copy of it up to date
        # the normed rows are read by the sublayer that follows and by nothing after it
        y = self._normed(self.mixer_norm, x, delta, "prenorm.mixer_in")
        mixed = self.mixer.forward(ctx, y, cache)     # a tensor, or what the norms add as a whole
        if self.feed_forward is None:
            return mixed
        y = self._normed(self.feed_forward_norm, x, mixed, "prenorm.feed_forward_in")
        return self.feed_forward.forward(ctx, y)

    @staticmethod
    def _normed(norm, x, delta, tag):
        """A norm of this package is told where its result may live; any other norm part has the
        plain interface forward(x, delta)."""
        if isinstance(norm, RMSNorm):
            return norm.forward(x, delta, tag=tag)
        return norm.forward(x, delta)


@register_part("arrangement", "outnorm")
class OutNormBlock(Part):
    """x += norm(mixer(x)); x += norm(feed_forward(x)): the norms sit on the sublayers' OUTPUTS
    and the sublayers read the residual stream itself.  A layer may have no feed-forward.

    The residual stream `x` is float32 and is updated in place by the kernel that norms a
    sublayer's output.  In bfloat16 that kernel also writes the new x in bfloat16, which is what
    the next sublayer's matrix product reads (`ctx.residual_copy`); in float32 the sublayers read
    x directly.  Nothing is left pending: forward returns None.
    """

    def __init__(self, prefix: str, layer: LayerSpec):
        self.prefix = prefix
        self.mixer_norm = build_part("norm", layer.mixer_norm, prefix + layer.mixer_norm_name)
        self.mixer = build_part("mixer", layer.mixer, prefix + layer.mixer_name)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm,
                                                prefix + layer.feed_forward_norm_name)
            self.feed_forward = build_part("feed_forward", layer.feed_forward,
                                           prefix + layer.feed_forward_name)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not isinstance(norm, LayerNorm):
                raise TypeError("the outnorm arrangement takes norms that can accumulate into the "
                                "residual stream (layernorm)")

    def parts(self):
        return [part for part in (self.mixer_norm, self.mixer, self.feed_forward_norm,
                                  self.feed_forward) if part is not None]

    @property
    def capturable(self) -> bool:
        return all(part.capturable for part in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(tensors, runtime)

    def _copy_buffer(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        rt = self.runtime
        if rt.dtype is torch.float32:
            return None
        return rt.buffer("outnorm.copy", x.shape[0], x.shape[1], rt.dtype)

    def forward(self, ctx, x: torch.Tensor, delta: Optional[torch.Tensor],
                cache: LayerCache) -> None:
        if delta is not None:
            raise ValueError("outnorm: the block before left a sublayer output pending")
        copy = self._copy_buffer(x)
        if copy is None:
            h = x
        else:
            h = getattr(ctx, "residual_copy", None)
            if h is None:                       # the first block of a model: nobody has cast x yet
                h = ops.cast_rows(x, copy)
        mixed = self.mixer.forward(ctx, h, cache)
        self.mixer_norm.accumulate(x, mixed, copy)
        if self.feed_forward is not None:
            out = self.feed_forward.forward(ctx, x if copy is None else copy)
            self.feed_forward_norm.accumulate(x, out, copy)
        ctx.residual_copy = copy
        return None


@register_part("arrangement", "sandwich")
class SandwichBlock(Part):
    """x += norm_b(mixer(norm_a(x))); x += norm_d(feed_forward(norm_c(x))): an RMS norm before AND
    after each sublayer.  A layer may have no feed-forward.

    The residual stream `x` is float32 and is updated in place.  A sublayer's output is not normed
    and added at once: it is handed on with its norm's gain (`NormedDelta`), and the kernel of the
    norm that runs next - the next sublayer's input norm, or the model's final norm - norms it,
    adds it to x and norms the sum in one pass over the row.
    """

    def __init__(self, prefix: str, layer: LayerSpec):
        self.prefix = prefix
        if layer.mixer_out_norm is None or \
                (layer.feed_forward is not None and layer.feed_forward_out_norm is None):
            raise ValueError("the sandwich arrangement needs a norm for every sublayer's output")
        self.mixer_norm = build_part("norm", layer.mixer_norm, prefix + layer.mixer_norm_name)
        self.mixer = build_part("mixer", layer.mixer, prefix + layer.mixer_name)
        self.mixer_out_norm = build_part("norm", layer.mixer_out_norm,
                                         prefix + layer.mixer_out_norm_name)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_out_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = build_part("norm", layer.feed_forward_norm,
                                                prefix + layer.feed_forward_norm_name)
            self.feed_forward = build_part("feed_forward", layer.feed_forward,
                                           prefix + layer.feed_forward_name)
            self.feed_forward_out_norm = build_part("norm", layer.feed_forward_out_norm,
                                                    prefix + layer.feed_forward_out_norm_name)
        for norm in (self.mixer_norm, self.mixer_out_norm, self.feed_forward_norm,
                     self.feed_forward_out_norm):
            if norm is not None and not isinstance(norm, RMSNorm):
                raise TypeError("the sandwich arrangement takes RMS norms")
        # a checkpoint may still hold the norms of a feed-forward that the layer does not have
        self.unused = []
        if layer.feed_forward is None:
            width = self.mixer_norm.width
            self.unused = [TensorSpec(prefix + name, (width,), role="vector", init="gain", optional=True)
                           for name in (layer.feed_forward_norm_name, layer.feed_forward_out_norm_name)]

    def parts(self):
        return [part for part in (self.mixer_norm, self.mixer, self.mixer_out_norm,
                                  self.feed_forward_norm, self.feed_forward,
                                  self.feed_forward_out_norm) if part is not None]

    @property
    def capturable(self) -> bool:
        return all(part.capturable for part in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        return [spec for part in self.parts() for spec in part.tensor_specs()] + self.unused

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(tensors, runtime)

    def forward(self, ctx, x: torch.Tensor, delta, cache: LayerCache) -> NormedDelta:
        ctx.residual_copy = None
        y = self.mixer_norm.forward(x, delta, tag="sandwich.mixer_in")
        mixed = self.mixer_out_norm.pending(self.mixer.forward(ctx, y, cache))
        if self.feed_forward is None:
            return mixed
        y = self.feed_forward_norm.forward(x, mixed, tag="sandwich.feed_forward_in")
        return self.feed_forward_out_norm.pending(self.feed_forward.forward(ctx, y))


@register_part("arrangement", "parallel")
class ParallelBlock(Part):
    """y = norm(x); x += mixer(y) + feed_forward(y): one norm, and both sublayers read its output.
    A layer may have no feed-forward.

    The residual stream `x` is float32 and is updated in place.  The two outputs are not added at
    once: they are handed on as a `PendingSum`, and the kernel of the norm that runs next (the next
    layer's, or the model's final norm on the wanted rows only) adds both to x in 32-bit and norms
    the sum in one pass over the row.
    """

    def __init__(self, prefix: str, layer: LayerSpec):
        self.prefix = prefix
        self.norm = build_part("norm", layer.mixer_norm, prefix + layer.mixer_norm_name)
        if not isinstance(self.norm, LayerNorm):
            raise TypeError("the parallel arrangement takes a norm that adds a pending sum (layernorm)")
        self.mixer = build_part("mixer", layer.mixer, prefix + layer.mixer_name)
        self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward = build_part("feed_forward", layer.feed_forward,
                                           prefix + layer.feed_forward_name)

    def parts(self):
        return [part for part in (self.norm, self.mixer, self.feed_forward) if part is not None]

    @property
    def capturable(self) -> bool:
        return all(part.capturable for part in self.parts())

    def tensor_specs(self) -> List[TensorSpec]:
        return [spec for part in self.parts() for spec in part.tensor_specs()]

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(tensors, runtime)

    def forward(self, ctx, x: torch.Tensor, delta, cache: LayerCache) -> PendingSum:
        ctx.residual_copy = None
        y = self.norm.forward(x, delta, write_x=True, tag="parallel.in")
        mixed = self.mixer.forward(ctx, y, cache)
        if self.feed_forward is None:
            return PendingSum((mixed,))
        return PendingSum((mixed, self.feed_forward.forward(ctx, y)))
