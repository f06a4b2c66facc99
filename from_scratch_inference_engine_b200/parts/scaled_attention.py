"""Grouped-query attention with a scale per head, keys and values of different widths, and values
blended across layers."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheNeed
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, build_part, register_part

MAX_KEY_SPLITS = 64
# which form of the attention kernel `attend` asks for: "auto" (a tensor-core kernel where one takes
# the sizes), or "plain" to measure or test the 32-bit kernel in its place
FORM = "auto"


def key_splits(blocks: int, longest: int, sms: int, key_tile: int = 32) -> int:
    """Into how many key ranges to split every tile of a step whose tiles alone would not fill
    the GPU (two blocks per SM): ranges of at least four key tiles, 64 at most."""
    slots = 2 * sms
    if blocks >= slots or longest <= 4 * key_tile:
        return 1
    return max(1, min(-(-slots // blocks), longest // (4 * key_tile), MAX_KEY_SPLITS))


def attend(ctx, rt, q: torch.Tensor, head_scale: torch.Tensor, group, cache: LayerCache,
           out: torch.Tensor, heads: int, kv_heads: int, key_dim: int, value_dim: int,
           values_in_keys: bool, window: int, chunk: int = 0) -> torch.Tensor:
    """The step's tokens over the pages through `ops.scaled_attention`: tiles of query rows, key
    ranges split over blocks when the tiles are few."""
    tokens = q.shape[0]
    form = FORM
    value_ld = key_dim if values_in_keys else value_dim
    if form == "auto" and (q.stride(0) % 8 or cache.page_stride % 8 or value_ld % 8 or q.data_ptr() % 16
                           or cache.k_pages.data_ptr() % 16 or cache.v_pages.data_ptr() % 16
                           or (heads * value_dim) % 2):
        form = "plain"          # rows that do not start where the tensor-core kernels' 16-byte copies need them
    rows = ops.scaled_attention_rows(q.dtype, key_dim, value_dim, values_in_keys, form)
    tiles = ctx.attention_tiles(heads // kv_heads, rows)
    reach = min(window if window > 0 else chunk, chunk if chunk > 0 else window)   # 0: every key
    longest = ctx.max_context if reach <= 0 else min(ctx.max_context, reach + rows)
    nsplit = key_splits(tiles.count * kv_heads, longest, rt.sm_count,
                        key_tile=64 if q.dtype is torch.bfloat16 else 32)
    part_o = part_ml = None
    if nsplit > 1:
        part_o = ctx.scratch("scaled_attention.part_o", nsplit * tokens * heads * value_dim)
        part_ml = ctx.scratch("scaled_attention.part_ml", nsplit * tokens * heads * 2)
    return ops.scaled_attention(q, q.stride(0), head_scale, cache.k_pages, cache.v_pages,
                                cache.page_stride, group.page_size, key_dim, value_dim,
                                values_in_keys, group.block_tables, tiles.item, tiles.row0,
                                tiles.count, ctx.item_qstart, ctx.item_qlen, ctx.item_pos0,
                                ctx.item_slots, out, tokens, heads, kv_heads, window, ctx.error,
                                nsplit, part_o, part_ml, form=form, chunk=chunk)


@register_part("mixer", "scaled_gqa_attention")
class ScaledGqaAttention(Mixer):
    """q, k, v projections with biases (one product over the stacked weight); rotation of q and
    k by `position` (pairs i, i + rotary_dim / 2 over the first rotary_dim of a head); scores
    (q . k) * scale * temperature[head] over the keys j <= i (or the last `window` of them);
    softmax; head h reads key/value head h // (heads / kv_heads); output projection without bias.
    Keys are `dim` wide, values `vdim`.

    `value_mix`: "source" keeps this layer's values of the step's tokens for later layers;
    "mix" blends its own with them before they are cached, v <- (1 - m) v + m v_source, m being
    the layer's `mix` tensor (one number); "none" does neither.  The source's values of a token
    are needed only while that token runs, so they travel in the step context, not in the cache.

    `chunk` > 0: position i sees j <= i only where i // chunk == j // chunk, the chunks counted
    from position 0 of the sequence (beside, or instead of, the window).  `qk_norm`: every head of q
    and of k is divided by its root mean square (`eps` inside the root) times a stored gain of `dim`
    numbers that all heads share, in 32-bit, before the rotation.  `head_gate`: every head's output
    is multiplied by sigmoid(W_g y)[head], one number per head, before the output projection; W_g
    rides in the one product with q, k and v.
    `names` gives the tensor names below the prefix.
    """

    capturable = True

    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "bias": ".b", "temperature": "temp",
             "mix": "vmix", "norm": ".norm", "gate": "g"}

    def __init__(self, prefix: str, hidden_size: int, heads: int, kv_heads: int, dim: int,
                 vdim: int, scale: float, position: PartSpec, window: int = 0,
                 value_mix: str = "none", temperature: bool = True,
                 names: Optional[Dict[str, str]] = None, chunk: int = 0, qk_norm: bool = False,
                 eps: float = 0.0, head_gate: bool = False):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if value_mix not in ("none", "source", "mix"):
            raise ValueError("value_mix must be 'none', 'source' or 'mix'")
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.window, self.value_mix = float(scale), int(window), value_mix
        self.temperature = bool(temperature)
        self.chunk, self.qk_norm, self.eps, self.head_gate = int(chunk), bool(qk_norm), float(eps), bool(head_gate)
        if self.chunk < 0 or self.window < 0:
            raise ValueError("window and chunk must not be negative")
        if (self.qk_norm or self.head_gate) and value_mix != "none":
            raise ValueError("scaled_gqa_attention: blended values go with neither qk_norm nor head_gate")
        self.q_width, self.k_width = self.heads * self.dim, self.kv_heads * self.dim
        self.v_width = self.kv_heads * self.vdim
        self.position = build_part("position", position, prefix)
        if self.position.rotary_dim > self.dim:
            raise ValueError("the rotated size exceeds dim")
        if self.position.rotary_dim and getattr(self.position, "pairing", "half") != "half":
            raise ValueError("scaled_gqa_attention rotates pairs half a rotation apart")
        self.names = dict(self.NAMES)
        self.names.update(names or {})
        self.w_qkv = self.b_qkv = self.w_o = self.head_scale = self.mix = None
        self.q_gain = self.k_gain = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, h, n = self.prefix, self.hidden_size, self.names
        specs = []
        for which, width in (("q", self.q_width), ("k", self.k_width), ("v", self.v_width)):
            specs.append(TensorSpec(p + n[which], (width, h)))
            specs.append(TensorSpec(p + n[which] + n["bias"], (width,)))
        if self.value_mix != "none":        # the source has the tensor too, and does not use it
            specs.append(TensorSpec(p + n["mix"], (), role="vector", init="half"))
        if self.temperature:
            specs.append(TensorSpec(p + n["temperature"], (self.heads,), role="vector", init="gain"))
        if self.qk_norm:
            specs += [TensorSpec(p + n[which] + n["norm"], (self.dim,), role="vector", init="gain")
                      for which in ("q", "k")]
        if self.head_gate:
            specs.append(TensorSpec(p + n["gate"], (self.heads, h)))
        specs.append(TensorSpec(p + n["o"], (h, self.heads * self.vdim)))
        return specs + self.position.tensor_specs()

    def cache_need(self) -> Optional[CacheNeed]:
        # a query sees no key further back than its chunk is long: the pages behind that are
        # given back as those behind a window are
        reach = min(self.window if self.window > 0 else self.chunk,
                    self.chunk if self.chunk > 0 else self.window)
        return CacheNeed(self.kv_heads, self.dim, reach, 0,
                         0 if self.vdim == self.dim else self.vdim)

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p, n = self.prefix, self.names
        stacked = [tensors[p + n[k]] for k in "qkv"]
        biases = [tensors[p + n[k] + n["bias"]].to(runtime.dtype) for k in "qkv"]
        if self.head_gate:                  # the gate's rows behind q, k and v; it has no bias
            stacked.append(tensors[p + n["gate"]])
            biases.append(torch.zeros(self.heads, dtype=runtime.dtype, device=biases[0].device))
        rows = sum(w.shape[0] for w in stacked)
        if self.head_gate and rows % 8:     # rows of the product's result start on 16 bytes
            pad = 8 - rows % 8
            stacked.append(torch.zeros(pad, self.hidden_size, dtype=stacked[0].dtype, device=stacked[0].device))
            biases.append(torch.zeros(pad, dtype=runtime.dtype, device=biases[0].device))
        self.w_qkv = torch.cat(stacked).contiguous()
        self.b_qkv = torch.cat(biases).contiguous()
        if self.qk_norm:
            self.q_gain = tensors[p + n["q"] + n["norm"]].to(torch.float32).contiguous()
            self.k_gain = tensors[p + n["k"] + n["norm"]].to(torch.float32).contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        scale = torch.full((self.heads,), self.scale, dtype=torch.float32, device=runtime.device)
        if self.temperature:
            scale = scale * tensors[p + n["temperature"]].to(torch.float32)
        self.head_scale = scale.contiguous()
        if self.value_mix == "mix":
            self.mix = tensors[p + n["mix"]].to(torch.float32).reshape(1).contiguous()
        runtime.prepare_weight(self.w_qkv)
        runtime.prepare_weight(self.w_o)
        self.position.bind(tensors, runtime)

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = self.runtime
        tokens = y.shape[0]
        group = ctx.groups[cache.group]
        qkv = rt.linear(y, self.w_qkv, self.b_qkv, "scaled_attention.qkv")
        v_first, mode = None, 0
        if self.value_mix == "source":
            mode = 1
            v_first = ctx.shared["value_mix"] = rt.buffer("scaled_attention.v_source", tokens,
                                                          self.v_width, qkv.dtype)
        elif self.value_mix == "mix":
            mode = 2
            v_first = ctx.shared.get("value_mix")
            if v_first is None or v_first.shape != (tokens, self.v_width):
                raise ValueError("scaled_gqa_attention: no layer before this one has left values "
                                 "of this width to blend with")
        if self.qk_norm or self.head_gate:
            ops.norm_rotate_write(qkv, ctx.positions, self.position.table, group.slot_of, cache.k_pages,
                                  cache.v_pages, cache.page_stride, group.page_size, self.heads,
                                  self.kv_heads, self.dim, self.vdim, self.position.rotary_dim,
                                  self.q_gain, self.k_gain, self.eps, ctx.error)
        else:
            ops.rotate_mix_write(qkv, ctx.positions, self.position.table, group.slot_of, cache.k_pages,
                                 cache.v_pages, cache.page_stride, group.page_size, self.heads,
                                 self.kv_heads, self.dim, self.vdim, self.position.rotary_dim, mode,
                                 self.mix, v_first, ctx.error)
        out = rt.buffer("scaled_attention.out", tokens, self.heads * self.vdim, qkv.dtype)
        attend(ctx, rt, qkv, self.head_scale, group, cache, out, self.heads, self.kv_heads, self.dim,
               self.vdim, False, self.window, self.chunk)
        if self.head_gate:
            gate0 = self.q_width + self.k_width + self.v_width
            ops.head_gate(out, qkv[:, gate0:gate0 + self.heads], self.heads, self.vdim)
        return rt.linear(out, self.w_o, None, "scaled_attention.o")
