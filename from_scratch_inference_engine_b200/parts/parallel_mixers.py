"""Two mixers side by side on the same input, their outputs added with a weight each."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheNeed
from ..config.spec import PartSpec
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, StateNeed, build_part, register_part
from .norm import ScaledSum


@register_part("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    """out = left_scale * left(y) + right_scale * right(y) for any two mixers `left` and `right`
    (their tensors below the prefixes `names["left"]` and `names["right"]`).

    At most one of the two may keep keys in the cache and at most one per-request state: the layer's
    cache entry and state slot go to the one that asks.  The weighted sum is not formed in the
    compute dtype: both outputs are handed on with their weights (`ScaledSum`) and the norm that
    runs next adds them to the 32-bit residual stream.
    """

    NAMES = {"left": "left.", "right": "right."}

    def __init__(self, prefix: str, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                 right_scale: float = 1.0, names: Optional[Dict[str, str]] = None):
        self.prefix = prefix
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.left = build_part("mixer", left, prefix + self.names["left"])
        self.right = build_part("mixer", right, prefix + self.names["right"])
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        needs = [m.cache_need() for m in (self.left, self.right)]
        states = [m.state_need() for m in (self.left, self.right)]
        if sum(n is not None for n in needs) > 1 or sum(s is not None for s in states) > 1:
            raise ValueError("parallel_mixers: only one of the two mixers may keep keys in the cache, "
                             "and only one per-request state")

    @property
    def capturable(self) -> bool:
        return bool(self.left.capturable and self.right.capturable)

    def tensor_specs(self) -> List[TensorSpec]:
        return self.left.tensor_specs() + self.right.tensor_specs()

    def cache_need(self) -> Optional[CacheNeed]:
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self) -> Optional[StateNeed]:
        return self.left.state_need() or self.right.state_need()

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        self.left.bind(tensors, runtime)
        self.right.bind(tensors, runtime)

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> ScaledSum:
        # each mixer finds in the layer's cache what it asked for and ignores the rest
        left = self.left.forward(ctx, y, cache)
        right = self.right.forward(ctx, y, cache)
        return ScaledSum((left, right), (self.left_scale, self.right_scale))
