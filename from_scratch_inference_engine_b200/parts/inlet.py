"""Inlets: what may run between two calls of a model's run order, on the residual stream."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Part, register_part
from .norm import PendingSum


@register_part("inlet", "concat_embedding")
class ConcatEmbeddingInlet(Part):
    """x <- W [x; x0]: the residual stream beside the embedding output of the same tokens, through
    one matrix [width, 2 width] whose first `width` columns meet x.  What the layer before left
    pending is added to x first (32-bit); the product's sums are 32-bit and so is the new x.  The
    tensor is `prefix + weight_name`."""

    capturable = True

    def __init__(self, prefix: str, hidden_size: int, weight_name: str = "weight"):
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.name = prefix + weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.hidden_size, 2 * self.hidden_size))]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.name].contiguous()
        runtime.prepare_weight(self.weight)

    def forward(self, ctx, x: torch.Tensor, delta, x0: torch.Tensor) -> torch.Tensor:
        rt = self.runtime
        deltas = delta.deltas if isinstance(delta, PendingSum) else (delta,)
        both = rt.buffer("inlet.both", x.shape[0], 2 * self.hidden_size, rt.dtype)
        ops.settle_concat(x, deltas, x0, both)
        return rt.linear_f32_out(both, self.weight, "inlet.out")
