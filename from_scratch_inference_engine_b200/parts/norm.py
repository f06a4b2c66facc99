"""Norms: RMSNorm fused with the residual add that precedes it, and layer norm with a gain."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Union

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Part, register_part


@dataclass
class NormedDelta:
    """A sublayer's output that is still to be RMS-normed (gain, eps) and added to the residual
    stream: what an arrangement with norms on the sublayers' outputs hands to the norm that runs
    next, so that one kernel norms it, adds it and norms the sum."""

    delta: torch.Tensor
    gain: torch.Tensor          # float32 [width]
    eps: float


@dataclass
class PendingSum:
    """The outputs of sublayers that read the same norm, still to be added to the residual stream
    (x += d1 + d2): what an arrangement with one norm for both sublayers hands to the norm that
    runs next."""

    deltas: tuple


@dataclass
class ScaledSum:
    """The outputs of mixers that ran side by side on the same input, each with its weight, still
    to be added to the residual stream (x += a1 d1 + a2 d2): the norm that runs next adds them in
    32-bit, so the weighted sum is never rounded to the storage type."""

    deltas: tuple
    scales: tuple


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * gain over the last axis, statistics in 32-bit (reference:
    src/model/nn.cpp:45-72, 64-bit statistics there).  The gain is the stored tensor, or - with
    `one_plus`, a weight stored around zero - 1 + the stored tensor (summed in 32-bit at bind).

    forward adds `delta` into the float32 residual `x` first (one kernel, one pass over x).
    """

    capturable = True

    def __init__(self, prefix: str, width: int, eps: float, weight_name: str = "weight",
                 one_plus: bool = False):
        self.prefix, self.width, self.eps = prefix, int(width), float(eps)
        self.name = prefix + weight_name
        self.one_plus = bool(one_plus)
        self.gain: Optional[torch.Tensor] = None
        self._gain_f32: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), role="vector",
                           init="normal" if self.one_plus else "gain")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        self.gain = tensors[self.name].contiguous()
        if self.one_plus:
            self.gain = (self.gain.to(torch.float32) + 1.0).contiguous()
        self._gain_f32 = None

    @property
    def gain_f32(self) -> torch.Tensor:
        """The gain in 32-bit (what the kernels that norm on both sides of a sublayer read)."""
        if self._gain_f32 is None:
            self._gain_f32 = self.gain.to(torch.float32).contiguous()
        return self._gain_f32

    def forward(self, x: torch.Tensor, delta: Union[None, torch.Tensor, NormedDelta, ScaledSum],
                rows: Optional[torch.Tensor] = None, write_x: bool = True,
                tag: Optional[str] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """`tag`: where the result may live (`Runtime.buffer`); None asks for fresh memory.
        `delta` is added to x as it is, or - a `NormedDelta` - after its own RMS norm, or - a
        `ScaledSum` - as the weighted sum of its parts.  `out_dtype` float32 (nothing pending) gives
        the normed rows in 32-bit: a norm whose result is itself the residual stream."""
        count = x.shape[0] if rows is None else rows.numel()
        if out_dtype is torch.float32 and delta is None:
            out = self.runtime.buffer(tag, count, self.width, torch.float32)
            return ops.add_rmsnorm(x, None, self.gain_f32, self.eps, out, rows=rows, write_x=False)
        out = self.runtime.buffer(tag, count, self.width, self.runtime.dtype)
        if isinstance(delta, ScaledSum):
            return ops.scaled_sum_rmsnorm(x, delta.deltas, delta.scales, self.gain_f32, self.eps, out,
                                          rows=rows, write_x=write_x)
        if isinstance(delta, NormedDelta):
            return ops.norm_add_norm(x, delta.delta, delta.gain, delta.eps, self.gain_f32, self.eps,
                                     out, rows=rows, write_x=write_x)
        return ops.add_rmsnorm(x, delta, self.gain, self.eps, out, rows=rows, write_x=write_x)

    def pending(self, delta: torch.Tensor) -> NormedDelta:
        """`delta`, to be normed by this norm and added by whichever norm runs next."""
        return NormedDelta(delta, self.gain_f32, self.eps)


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * gain (+ bias) over the last axis,
    statistics in 32-bit.  The gain is `prefix + weight_name`; with `bias_name` there is a bias,
    the tensor `prefix + bias_name`.

    Two uses: `forward` norms rows of the float32 residual stream (an arrangement's input norm, a
    model's final norm), adding what is still pending first; `accumulate` norms a sublayer's
    output and adds it into the residual stream, for arrangements whose norms sit on the outputs
    of the sublayers.
    """

    capturable = True

    def __init__(self, prefix: str, width: int, eps: float, weight_name: str = "weight",
                 bias_name: Optional[str] = None):
        self.prefix, self.width, self.eps = prefix, int(width), float(eps)
        self.name = prefix + weight_name
        self.bias_name = None if bias_name is None else prefix + bias_name
        self.gain: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.name, (self.width,), role="vector", init="gain")]
        if self.bias_name is not None:
            specs.append(TensorSpec(self.bias_name, (self.width,), role="vector", init="normal"))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        self.gain = tensors[self.name].to(torch.float32).contiguous()
        if self.bias_name is not None:
            self.bias = tensors[self.bias_name].to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, delta: Union[None, torch.Tensor, PendingSum] = None,
                rows: Optional[torch.Tensor] = None, write_x: bool = False,
                tag: Optional[str] = None) -> torch.Tensor:
        """The normed rows of x (all, or those `rows` names) in the compute dtype.  What is
        pending (`delta`: one sublayer output, or a `PendingSum` of up to two) is added to x
        first, in 32-bit, and - with `write_x` - stays added."""
        count = x.shape[0] if rows is None else rows.numel()
        out = self.runtime.buffer(tag, count, self.width, self.runtime.dtype)
        if delta is None and self.bias is None:
            return ops.layernorm_rows(x, self.gain, self.eps, out, rows=rows)
        deltas = delta.deltas if isinstance(delta, PendingSum) else (delta,)
        return ops.sum_layernorm(x, deltas, self.gain, self.bias, self.eps, out, rows=rows,
                                 write_x=write_x)

    def accumulate(self, x: torch.Tensor, delta: torch.Tensor,
                   copy: Optional[torch.Tensor]) -> None:
        """x += LN(delta) * gain; `copy` (compute dtype) receives the new x when given."""
        if self.bias is not None:
            raise ValueError("LayerNorm.accumulate takes a norm without bias")
        ops.add_layernorm(x, delta, self.gain, self.eps, copy)
