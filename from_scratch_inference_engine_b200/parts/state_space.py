"""A state-space mixer in its "state-space duality" form: a recurrence over a matrix per head whose
decay and step size depend on the token."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, StateNeed, register_part


@register_part("mixer", "state_space_duality")
class StateSpaceDuality(Mixer):
    """One product gives [z | x | B | C | dt] (inner = heads * vdim columns of z and of x,
    groups * state of B and of C, one dt per head).  x, B and C together pass a causal convolution
    over time per channel (`taps` taps, the last the current token's, a bias, zeros before the
    sequence starts) and SiLU.  dt <- softplus(dt + dt_bias).  Head h, which reads the B and C of
    group h // (heads / groups), keeps S [state, vdim]:

        S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T        y_t = S_t^T C_t + D_h x_t

    y (the heads side by side) is multiplied by silu(z), divided by its root mean square in
    `norm_groups` equal parts (`eps` inside the root), multiplied by a gain, and projected.

    Per request the slot holds S of every head and, behind them, the convolution's inputs of the
    last taps - 1 tokens; both are float32, zero when a request starts, and carried from step to
    step.  Step sizes, decays, the convolution's results, the recurrence, the gate and the norm
    are 32-bit in both compute dtypes.  Prompts of more than two chunks of 64 tokens run
    chunk-parallel through the same scan as decaying linear attention (`ops.lightning_scan` with a
    decay per token and head).  `names` gives the tensor names below the prefix.
    """

    capturable = True
    CHUNK_TOKENS = 64

    NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log",
             "skip": "D", "norm": "norm", "o": "o"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, vdim: int, state: int, groups: int,
                 taps: int, norm_groups: int, eps: float, names: Optional[Dict[str, str]] = None):
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.heads, self.vdim, self.state, self.groups = int(heads), int(vdim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps = int(taps), int(norm_groups), float(eps)
        if min(self.heads, self.vdim, self.state, self.groups, self.norm_groups) <= 0:
            raise ValueError("state_space_duality: heads, vdim, state, groups and norm_groups are positive")
        if self.heads % self.groups:
            raise ValueError("state_space_duality: heads must be a multiple of groups")
        self.inner = self.heads * self.vdim
        if self.inner % self.norm_groups:
            raise ValueError("state_space_duality: heads * vdim must divide into norm_groups equal parts")
        if self.taps < 1:
            raise ValueError("state_space_duality: the convolution has at least one tap")
        self.channels = self.inner + 2 * self.groups * self.state
        self.width = 2 * self.inner + 2 * self.groups * self.state + self.heads
        self.matrix_floats = self.heads * self.state * self.vdim
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.w_in = self.w_o = self.conv = self.conv_bias = None
        self.dt_bias = self.a_log = self.skip = self.gain = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, h, n = self.prefix, self.hidden_size, self.names
        return [TensorSpec(p + n["in"], (self.width, h)),
                TensorSpec(p + n["conv"], (self.channels, self.taps), role="vector", init="taps"),
                TensorSpec(p + n["conv_bias"], (self.channels,), role="vector", init="normal"),
                TensorSpec(p + n["dt_bias"], (self.heads,), role="vector", init="normal"),
                TensorSpec(p + n["a_log"], (self.heads,), role="vector", init="normal"),
                TensorSpec(p + n["skip"], (self.heads,), role="vector", init="gain"),
                TensorSpec(p + n["norm"], (self.inner,), role="vector", init="gain"),
                TensorSpec(p + n["o"], (h, self.inner))]

    def state_need(self) -> Optional[StateNeed]:
        floats = self.matrix_floats + (self.taps - 1) * self.channels
        return StateNeed((-(-floats // 8) * 8,), torch.float32)      # slots start on 32 bytes

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p, n = self.prefix, self.names
        if self.state > 256:
            raise ValueError(f"state_space_duality: {self.state} state rows per head, the scan holds 256")
        if self.taps > ops.ssd_max_taps():
            raise ValueError(f"state_space_duality: {self.taps} taps, the kernels hold {ops.ssd_max_taps()}")

        def vector(key):
            return tensors[p + n[key]].to(torch.float32).contiguous()
        self.w_in = tensors[p + n["in"]].contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        self.conv, self.conv_bias = vector("conv"), vector("conv_bias")
        self.conv_by_tap = self.conv.t().contiguous()          # [taps, channels]: eight channels' weights in a row
        self.dt_bias, self.a_log, self.skip, self.gain = (vector("dt_bias"), vector("a_log"),
                                                          vector("skip"), vector("norm"))
        runtime.prepare_weight(self.w_in)
        runtime.prepare_weight(self.w_o)

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = self.runtime
        tokens = y.shape[0]
        inner, gn = self.inner, self.groups * self.state
        proj = rt.linear(y, self.w_in, None, "state_space.in")
        # [ x | B | C ] after convolution and SiLU, then dt * x; and the decay of every token and head
        act = rt.buffer("state_space.act", tokens, self.channels + inner, torch.float32)
        decay = rt.buffer("state_space.decay", tokens, self.heads, torch.float32)
        items = (ctx.item_qstart, ctx.item_qlen, ctx.item_slots, ctx.num_items)
        ops.ssd_prep(proj, inner, inner + self.channels, *items, cache.state, self.matrix_floats,
                     self.conv, self.conv_bias, self.dt_bias, self.a_log, self.heads, self.vdim, act, decay,
                     conv_wt=self.conv_by_tap)
        ops.ssd_tails(proj, inner, self.channels, self.taps, *items, cache.state, self.matrix_floats)
        chunks = {}
        if int(ctx.h_qlen.max()) > 2 * self.CHUNK_TOKENS:
            tiles = ctx.attention_tiles(1, self.CHUNK_TOKENS)
            chunks = dict(seg_item=tiles.item, seg_row0=tiles.row0, num_segs=tiles.count,
                          seg_tokens=self.CHUNK_TOKENS,
                          chunk_states=ctx.scratch("state_space.chunk_states",
                                                   tiles.count * (self.matrix_floats + self.heads)))
        o = rt.buffer("state_space.o", tokens, inner, torch.float32)
        # q = C, k = B, v = dt * x; the heads of a group share its B and C
        ops.lightning_scan(act, inner + gn, inner, self.channels, ctx.item_qstart, ctx.item_qlen,
                           ctx.item_slots, ctx.num_items, cache.state, None, o, self.heads, self.state,
                           self.vdim, share=self.heads // self.groups, decay_tok=decay, **chunks)
        gated = rt.buffer("state_space.gated", tokens, inner, proj.dtype)
        ops.ssd_gate_norm(o, act, proj, 0, self.skip, self.gain, gated, self.vdim, self.norm_groups, self.eps)
        return rt.linear(gated, self.w_o, None, "state_space.out")
