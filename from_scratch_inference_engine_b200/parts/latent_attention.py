"""Attention over a cache of latent rows: per token one normed low-rank vector and a single rotated
key vector that every head uses."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheNeed
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, build_part, register_part
from .scaled_attention import attend


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """q = W_q y, per head [dim unrotated | rope rotated].  W_dkv y = [lat (rank) | kr (rope)]:
    c = rms_norm(lat) * gain is the latent, kr a single rotated key vector that every head uses.  Head h
    has keys [U_h c | kr] and values V_h c (W_uk = U, W_uv = V stacked head by head); scores
    (q . k) * scale over the keys j in (i - window, i] (all j <= i without a window); softmax;
    output projection on the concatenated heads.  Rotation by `position` over the first
    rotary_dim columns of a rope part, of the pairs that the position part names (2i with 2i + 1,
    or i with i + rotary_dim / 2).  rope_dim = 0: no rotated part, W_dkv y is the latent alone.
    `gate`: the concatenated heads are multiplied element by element by sigmoid(W_g y) before the
    output projection (W_g reads the same y as the other projections and rides in their product).

    Only [c | kr] is cached: one row per token, read by every head as key and as value.  Keys and
    values per head are never formed: (U_h^T q_h) . c = q_h . (U_h c), so the queries take U over
    before the attention, which then runs with `heads` query heads over ONE key/value head of
    width rank + rope whose values are the first rank columns of the same rows, and V_h is
    applied to each head's output over c afterwards.
    `names` gives the tensor names below the prefix.
    """

    capturable = True

    NAMES = {"q": "q", "dkv": "dkv", "norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o", "g": "g"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, dim: int, rope_dim: int,
                 vdim: int, rank: int, scale: float, eps: float, position: PartSpec,
                 window: int = 0, names: Optional[Dict[str, str]] = None, gate: bool = False):
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.heads, self.dim, self.rope_dim = int(heads), int(dim), int(rope_dim)
        self.vdim, self.rank = int(vdim), int(rank)
        self.scale, self.eps, self.window = float(scale), float(eps), int(window)
        self.q_head = self.dim + self.rope_dim
        self.row = self.rank + self.rope_dim             # what the cache keeps per token
        self.position = build_part("position", position, prefix)
        if self.position.rotary_dim > self.rope_dim:
            raise ValueError("the rotated size exceeds the rope part")
        pairing = getattr(self.position, "pairing", "interleaved")
        if self.position.rotary_dim and pairing not in ("interleaved", "half"):
            raise ValueError("latent_attention rotates interleaved pairs or pairs half a rotation apart")
        self.half_pairs = pairing == "half"
        self.gate = bool(gate)
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.gain = self.head_scale = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, h, n = self.prefix, self.hidden_size, self.names
        return [TensorSpec(p + n["q"], (self.heads * self.q_head, h)),
                TensorSpec(p + n["dkv"], (self.row, h)),
                TensorSpec(p + n["norm"], (self.rank,), role="vector", init="gain"),
                TensorSpec(p + n["uk"], (self.heads * self.dim, self.rank)),
                TensorSpec(p + n["uv"], (self.heads * self.vdim, self.rank)),
                TensorSpec(p + n["o"], (h, self.heads * self.vdim))] + \
            ([TensorSpec(p + n["g"], (self.heads * self.vdim, h))] if self.gate else []) + \
            self.position.tensor_specs()

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(1, self.row, self.window, 0, self.rank, values_in_keys=True)

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p, n = self.prefix, self.names
        stacked = [tensors[p + n["q"]], tensors[p + n["dkv"]]] + ([tensors[p + n["g"]]] if self.gate else [])
        self.w_in = torch.cat(stacked).contiguous()
        self.gain = tensors[p + n["norm"]].to(torch.float32).contiguous()
        # U_h^T [rank, dim] per head: the product that takes U over to the queries
        self.w_uk_t = tensors[p + n["uk"]].view(self.heads, self.dim, self.rank) \
            .transpose(1, 2).contiguous()
        self.w_uv = tensors[p + n["uv"]].view(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        self.head_scale = torch.full((self.heads,), self.scale, dtype=torch.float32,
                                     device=runtime.device)
        runtime.prepare_weight(self.w_in)
        runtime.prepare_weight(self.w_o)
        self.position.bind(tensors, runtime)

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = self.runtime
        tokens = y.shape[0]
        group = ctx.groups[cache.group]
        proj = rt.linear(y, self.w_in, None, "latent.in")
        qa = rt.buffer("latent.q", tokens, self.heads * self.row, proj.dtype)
        ops.latent_prep(proj, ctx.positions, self.position.table, group.slot_of, cache.k_pages,
                        cache.page_stride, group.page_size, self.gain, self.eps, qa, self.heads,
                        self.dim, self.rope_dim, self.rank, self.position.rotary_dim, ctx.error,
                        half_pairs=self.half_pairs)
        ops.head_product(proj, proj.stride(0), self.q_head, self.w_uk_t, qa, self.heads * self.row,
                         self.row, tokens)
        over_c = rt.buffer("latent.over_c", tokens, self.heads * self.rank, proj.dtype)
        attend(ctx, rt, qa, self.head_scale, group, cache, over_c, self.heads, 1, self.row, self.rank,
               True, self.window)
        out = rt.buffer("latent.out", tokens, self.heads * self.vdim, proj.dtype)
        ops.head_product(over_c, self.heads * self.rank, self.rank, self.w_uv, out,
                         self.heads * self.vdim, self.vdim, tokens)
        if self.gate:
            first = self.heads * self.q_head + self.row
            ops.sigmoid_gate(out, proj[:, first:first + self.heads * self.vdim])
        return rt.linear(out, self.w_o, None, "latent.o")
