"""Dense gated feed-forward (SwiGLU, or another activation on the gate)."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import Part, register_part


@register_part("feed_forward", "gated_mlp")
@register_part("feed_forward", "swiglu")
class SwiGluMlp(Part):
    """down( act(gate(y)) * up(y) ) with act = SiLU unless `activation` names another
    ("gelu_tanh": g/2 * (1 + tanh(0.7978845608 * (g + 0.044715 g^3)))), without biases (reference: src/model/model.cpp:136-140,
    src/model/nn.cpp:74-88) or, with `bias`, with one on each of the three projections.  gate
    and up are one product over the stacked weight [2 * intermediate, hidden]: gate rows first,
    then up rows.  `names` gives the tensor names below the prefix: the three projections, and
    what is appended for a weight and for a bias."""

    capturable = True

    NAMES = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj", "weight": ".weight",
             "bias": ".bias"}

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, bias: bool = False,
                 names: Optional[Dict[str, str]] = None, activation: str = "silu"):
        if activation not in ops.FUSED_GATES:
            raise ValueError(f"unknown gate activation '{activation}' "
                             f"({', '.join(sorted(ops.FUSED_GATES))})")
        self.activation = activation
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.bias = bool(bias)
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def _name(self, which: str, kind: str) -> str:
        return self.prefix + self.names[which] + self.names[kind]

    def tensor_specs(self) -> List[TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        specs = [TensorSpec(self._name("gate", "weight"), (i, h)),
                 TensorSpec(self._name("up", "weight"), (i, h)),
                 TensorSpec(self._name("down", "weight"), (h, i))]
        if self.bias:
            specs += [TensorSpec(self._name("gate", "bias"), (i,), role="vector"),
                      TensorSpec(self._name("up", "bias"), (i,), role="vector"),
                      TensorSpec(self._name("down", "bias"), (h,), role="vector")]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        self.w_gate_up = torch.cat([tensors[self._name("gate", "weight")],
                                    tensors[self._name("up", "weight")]]).contiguous()
        self.w_down = tensors[self._name("down", "weight")].contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([tensors[self._name("gate", "bias")],
                                        tensors[self._name("up", "bias")]]).to(runtime.dtype).contiguous()
            self.b_down = tensors[self._name("down", "bias")].to(runtime.dtype).contiguous()
        # the fused SwiGLU products take no bias: with one, the stacked product adds it and a
        # kernel of its own applies the activation
        runtime.prepare_weight(self.w_gate_up, swiglu=not self.bias, activation=self.activation)
        runtime.prepare_weight(self.w_down)

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        rt = self.runtime
        # the activation and the result are dead when the next feed-forward of the model runs
        act = rt.linear_swiglu(y, self.w_gate_up, "swiglu.act", bias=self.b_gate_up,
                               activation=self.activation)
        return rt.linear(act, self.w_down, self.b_down, "swiglu.down")
