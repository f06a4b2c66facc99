"""A feed-forward of routed experts beside an optional expert that every token uses."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Part, build_part, register_part


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    """`experts` gated feed-forwards down(act(gate y) * (up y)) without biases, of which a token
    uses `top`.  `gated`=False: the experts have no gate, down(act(up y)); "relu2" (the square of
    relu) is an activation for those.  `identity` > 0: the router has that many more outputs behind
    the experts', each an expert whose output is its input y itself (times its weight); they have
    no tensors, and they count as experts for the scores, the groups and the choice.

    Router: z = W_r y in 32-bit, s = sigmoid(z) (`scores` "softmax": softmax over the experts).
    The choice is made on s + correction (a stored vector, `correction`=False: none) and the
    weights on s without it.  The experts form `groups` equal groups of neighbours; a group's
    score is the sum of its two largest choice values (`group_score` "max": the largest), and only
    experts of the `keep` best groups can be chosen.  The `top` largest are taken; their weights are s / (their sum + 1e-20) * `scale`
    (`normalise`=False: s * scale).  The output is the weighted sum of the chosen experts' outputs,
    plus - with `shared` (any feed-forward part) - what that part gives for the token.

    All experts' matrices are stacked at bind ([experts, 2 ff, width] gate rows then up rows;
    [experts, width, ff]).  The router's logits are a product with a 32-bit result.  A step sorts
    its (token, choice) pairs by expert on the device and runs the two products over tiles of rows
    that share an expert, so it launches the same kernels whatever the router says: tiles of 64
    rows through the mma.sync / FFMA kernels, or - bfloat16 steps with at least `GROUPED_MIN_ROWS`
    rows per expert on average - the tokens' rows gathered into a layout in which every expert's
    rows start on a multiple of 256, and the grouped form of the tiled tcgen05 product (SwiGLU in
    its epilogue) over it.  `names` gives the tensor names below the prefix ("expert" takes the
    expert's index).
    """

    GROUPED_MIN_ROWS = 32       # average rows per expert from which the tcgen05 form is taken

    NAMES = {"expert": "e{index}.", "gate": "gate", "up": "up", "down": "down", "router": "router",
             "correction": "correction", "shared": "shared."}

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, experts: int, top: int,
                 groups: int = 1, keep: int = 1, scale: float = 1.0, scores: str = "sigmoid",
                 normalise: bool = True, correction: bool = True, activation: str = "silu",
                 shared: Optional[PartSpec] = None, names: Optional[Dict[str, str]] = None,
                 gated: bool = True, identity: int = 0, group_score: str = "top2"):
        if activation not in (ops.FUSED_GATES if gated else ops.GATE_KINDS):
            raise ValueError(f"unknown activation '{activation}' for experts "
                             f"{'with' if gated else 'without'} a gate")
        if group_score not in ("top2", "max"):
            raise ValueError("group_score must be 'top2' or 'max'")
        self.gated, self.identity, self.group_score = bool(gated), int(identity), group_score
        if self.identity < 0:
            raise ValueError("routed_experts: identity must not be negative")
        if scores not in ("sigmoid", "softmax"):
            raise ValueError("scores must be 'sigmoid' or 'softmax'")
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.intermediate_size, self.experts, self.top = int(intermediate_size), int(experts), int(top)
        self.groups, self.keep, self.scale = int(groups), int(keep), float(scale)
        self.scores, self.normalise, self.activation = scores, bool(normalise), activation
        self.routed = self.experts + self.identity        # outputs of the router
        if self.experts <= 0 or not 0 < self.top <= self.routed:
            raise ValueError("routed_experts: top must lie in 1..experts (+ identity)")
        if self.groups <= 0 or self.routed % self.groups or not 0 < self.keep <= self.groups:
            raise ValueError("routed_experts: experts (+ identity) must divide into `groups` groups, "
                             "keep in 1..groups")
        if self.top > self.keep * (self.routed // self.groups):
            raise ValueError("routed_experts: the kept groups hold fewer than `top` experts")
        self.has_correction = bool(correction)
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.shared = None if shared is None else build_part("feed_forward", shared,
                                                             prefix + self.names["shared"])
        self.w_router = self.correction = self.w_gate_up = self.w_down = None

    @property
    def capturable(self) -> bool:
        return self.shared is None or bool(self.shared.capturable)

    def _expert(self, index: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(index=index) + self.names[which]

    def tensor_specs(self) -> List[TensorSpec]:
        h, f = self.hidden_size, self.intermediate_size
        specs = []
        for e in range(self.experts):
            if self.gated:
                specs.append(TensorSpec(self._expert(e, "gate"), (f, h)))
            specs += [TensorSpec(self._expert(e, "up"), (f, h)), TensorSpec(self._expert(e, "down"), (h, f))]
        specs.append(TensorSpec(self.prefix + self.names["router"], (self.routed, h)))     # in the compute dtype
        if self.has_correction:
            specs.append(TensorSpec(self.prefix + self.names["correction"], (self.routed,), role="vector"))
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        if self.gated:
            self.w_gate_up = torch.stack([torch.cat([tensors[self._expert(e, "gate")],
                                                     tensors[self._expert(e, "up")]])
                                          for e in range(self.experts)]).contiguous()
        else:           # the same name for the first matrix of an expert without a gate
            self.w_gate_up = torch.stack([tensors[self._expert(e, "up")]
                                          for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")]
                                   for e in range(self.experts)]).contiguous()
        self.w_router = tensors[self.prefix + self.names["router"]].contiguous()
        self._grouped = None             # descriptors of the stacked matrices, made when first needed
        if self.has_correction:
            self.correction = tensors[self.prefix + self.names["correction"]].to(torch.float32).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors, runtime)

    def _grouped_weights(self):
        if self._grouped is None:
            first = (ops.GroupedTiledWeight(self.w_gate_up, True, self.activation) if self.gated else
                     ops.GroupedTiledWeight(self.w_gate_up, False, plain_activation=self.activation))
            self._grouped = (first, ops.GroupedTiledWeight(self.w_down, False))
        return self._grouped

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        rt = self.runtime
        tokens, top = y.shape[0], self.top
        pairs = tokens * top
        ids = rt.buffer("routed.ids", tokens, top, torch.int32)
        weights = rt.buffer("routed.weights", tokens, top, torch.float32)
        logits = rt.linear_f32_out(y, self.w_router, "routed.logits")
        ops.moe_route(None, None, self.correction, ids, weights, top, self.groups, self.keep,
                      self.scale, self.scores, self.normalise, logits=logits, group_score=self.group_score)
        # choices at or beyond `experts` are identity experts: no rows in the products, and the
        # weighted sum takes the token's own row for them
        identity = dict(ids=ids, experts=self.experts, y=y) if self.identity else {}
        shared = None if self.shared is None else self.shared.forward(ctx, y)
        out = rt.buffer("routed.out", tokens, self.hidden_size, y.dtype)
        grouped = (y.dtype is torch.bfloat16 and rt.products == "own"
                   and (self.gated or self.activation == "relu2")
                   and pairs >= self.GROUPED_MIN_ROWS * self.experts
                   and self.hidden_size % 8 == 0 and self.intermediate_size % 8 == 0
                   and y.stride(0) % 8 == 0 and y.data_ptr() % 16 == 0)
        if grouped:
            tile = ops.GEMM_TILES_ROWS
            rows = (pairs // tile + self.experts) * tile
            lists = ops.moe_align(ids, pairs, self.experts,
                                  rt.buffer("routed.lists", 1, ops.moe_lists_size(pairs, self.experts, tile, True),
                                            torch.int32).view(-1), tile, True)
            gate_up, down = self._grouped_weights()
            x_sorted = ops.moe_gather(y, lists, tile, top,
                                      rt.buffer("routed.x_sorted", rows, self.hidden_size, y.dtype))
            act = rt.buffer("routed.act", rows, self.intermediate_size, y.dtype)
            ops.gemm_tiles_grouped(gate_up, x_sorted, act, lists[2], lists[4], ctx.error, rt.sm_count)
            expert_out = rt.buffer("routed.expert_out", rows, self.hidden_size, y.dtype)
            ops.gemm_tiles_grouped(down, act, expert_out, lists[2], lists[4], ctx.error, rt.sm_count)
            return ops.moe_combine(expert_out, weights, shared, out, top, place=lists[5], **identity)
        lists = ops.moe_align(ids, pairs, self.experts,
                              rt.buffer("routed.lists", 1, ops.moe_lists_size(pairs, self.experts),
                                        torch.int32).view(-1))
        act = rt.buffer("routed.act", pairs, self.intermediate_size, y.dtype)
        ops.moe_product(y, self.w_gate_up, act, lists, pairs, top, self.gated, self.activation, first=True)
        expert_out = rt.buffer("routed.expert_out", pairs, self.hidden_size, y.dtype)
        ops.moe_product(act, self.w_down, expert_out, lists, pairs, top, False)
        return ops.moe_combine(expert_out, weights, shared, out, top, **identity)
