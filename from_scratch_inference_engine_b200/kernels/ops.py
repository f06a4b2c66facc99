"""Typed Python entry points of the hand-written CUDA kernels.

Each function checks what the kernel assumes (device, dtype, contiguity, sizes),
passes raw pointers and the current CUDA stream to the C entry point, and raises on
any non-zero return.  There is no other implementation behind these functions: on a
machine without the compiled library or without a GPU they raise.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from ..csrc import build

DTYPE_F32, DTYPE_BF16 = 0, 1
GATE_KINDS = {"silu": 0, "gelu_tanh": 1, "relu2": 2}   # activations of a feed-forward ("relu2": the square of relu)
FUSED_GATES = ("silu", "gelu_tanh")        # ... those that the matrix products' gated epilogues know


class KernelError(RuntimeError):
    pass


def _tag(dtype: torch.dtype) -> int:
    if dtype is torch.float32:
        return DTYPE_F32
    if dtype is torch.bfloat16:
        return DTYPE_BF16
    raise KernelError(f"kernels take float32 or bfloat16 storage, not {dtype}")


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    """The address for a pointer argument (ctypes takes an int or None for c_void_p)."""
    return None if tensor is None else tensor.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch (streams change under
    graph capture), so by the cheapest route torch offers."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(tensor: torch.Tensor, dtype, name: str, contiguous: bool = True) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must live on the GPU (the engine has no CPU path)")
    if dtype is not None and tensor.dtype is not dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if contiguous and not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


launches = 0      # kernel launches issued through this module (benchmarks read this)


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{what}: argument refused by the kernel launcher")
    if code == -2:
        raise KernelError(f"{what}: size not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


_core = None


def core():
    """The core kernel library, compiled at first use."""
    global _core
    if _core is None:
        lib = build.load_library("core")
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_embed_gather.argtypes = [p, p, p, i, i, i, f, i, p, p]
        lib.fsie_add_rmsnorm.argtypes = [p, p, p, i, p, p, i, i, f, i, i, p]
        lib.fsie_rope_kv_write.argtypes = [p, i, p, p, i, p, p, p, ll, i, i, i, i, i, i, i, i, p, p]
        lib.fsie_swiglu.argtypes = [p, p, ll, i, i, p]
        lib.fsie_place_tokens.argtypes = [p, p, p, p, i, p]
        lib.fsie_gemm_f32.argtypes = [p, p, p, p, i, i, i, i, i, i, i, p]
        lib.fsie_gemm_f32_rows_limit.argtypes = []
        lib.fsie_gemm_f32_rows_limit.restype = i
        lib.fsie_attn_generic.argtypes = [p, i, p, p, ll, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                          i, i, i, i, i, i, f, i, p]
        lib.fsie_attn_tiles.argtypes = [p, i, p, p, ll, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                        i, i, i, i, i, i, f, i, i, i, p]
        lib.fsie_attn_tiles.restype = i
        lib.fsie_attn_generic_rows.argtypes = []
        lib.fsie_attn_rows16_rows.argtypes = []
        lib.fsie_attn_rows16_rows.restype = i
        lib.fsie_attn_rows16_takes.argtypes = [i]
        lib.fsie_attn_rows16_takes.restype = i
        lib.fsie_argmax.argtypes = [p, i, i, p, p]
        lib.fsie_argmax_staged.argtypes = [p, i, i, p, p, i, p]
        lib.fsie_sample.argtypes = [p, i, i, p, p, p, p, p, p]
        for name in ("fsie_embed_gather", "fsie_add_rmsnorm", "fsie_rope_kv_write", "fsie_swiglu",
                     "fsie_gemm_f32", "fsie_attn_generic", "fsie_attn_generic_rows",
                     "fsie_argmax", "fsie_argmax_staged", "fsie_sample"):
            getattr(lib, name).restype = ctypes.c_int
        _core = lib
    return _core


# ------------------------------------------------------------------------- embedding
def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                 error: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[ids[t]] widened to float32 (times `scale`); an id outside the table sets
    error[0]."""
    _need(ids, torch.int32, "ids")
    _need(table, None, "table")
    _need(out, torch.float32, "out")
    _need(error, torch.int32, "error")
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out.shape[-1] != hidden or out.numel() < tokens * hidden:
        raise KernelError("embed_gather: out is too small")
    _check(core().fsie_embed_gather(_ptr(ids), _ptr(table), _ptr(out), tokens, hidden, vocab,
                                    float(scale), _tag(table.dtype), _ptr(error), _stream()), "embed_gather")
    return out


# ---------------------------------------------------------------------- add + RMSNorm
def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                write_x: bool = True) -> torch.Tensor:
    """x (float32 residual) += delta; out = rmsnorm(x) * gain in out's dtype.

    With `rows` (int32 indices) only those rows are normed, into out[0..len(rows)), and
    x is left untouched unless write_x.
    """
    _need(x, torch.float32, "x")
    _need(out, None, "out")
    hidden = x.shape[-1]
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[-1] != hidden:
            raise KernelError("add_rmsnorm: delta width differs from x")
    _need(gain, None, "gain")
    if gain.numel() != hidden:
        raise KernelError("add_rmsnorm: gain width differs from x")
    if gain.dtype not in (torch.float32, out.dtype):
        raise KernelError(f"add_rmsnorm: gain must be float32 or {out.dtype}")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        count = rows.numel()
    else:
        count = x.numel() // hidden
    if out.numel() < count * hidden:
        raise KernelError("add_rmsnorm: out is too small")
    _check(core().fsie_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(gain),
                                   int(gain.dtype is torch.float32), _ptr(out), _ptr(rows), count,
                                   hidden, float(eps), int(write_x), _tag(out.dtype), _stream()),
           "add_rmsnorm")
    return out


# ------------------------------------------------------- rotary + paged cache write
def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                  slot_of: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
                  v_pages: Optional[torch.Tensor], page_stride: int, page_size: int,
                  heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                  error: torch.Tensor) -> None:
    """Rotate q in place in the fused projection rows; rotate k and store k, v in their pages.

    k_pages / v_pages are views whose first element is page 0 of this cache entry;
    page p of it starts page_stride elements further per page.
    """
    _need(qkv, None, "qkv")
    _need(positions, torch.int32, "positions")
    _need(cos_sin, torch.float32, "cos_sin")
    tokens, ld = qkv.shape
    if ld < (heads + 2 * kv_heads) * head_dim:
        raise KernelError("rope_kv_write: projection rows are narrower than q, k and v")
    if rotary_dim > 0 and cos_sin.shape[-1] != rotary_dim:
        raise KernelError("rope_kv_write: cos/sin table width differs from rotary_dim")
    write = k_pages is not None
    if write:
        _need(slot_of, torch.int32, "slot_of")
        if k_pages.dtype is not qkv.dtype or v_pages.dtype is not qkv.dtype:
            raise KernelError("rope_kv_write: cache dtype differs from the projection dtype")
    _check(core().fsie_rope_kv_write(_ptr(qkv), ld, _ptr(positions), _ptr(cos_sin),
                                     cos_sin.shape[0], _ptr(slot_of), _ptr(k_pages), _ptr(v_pages),
                                     page_stride, page_size, tokens, heads, kv_heads, head_dim,
                                     rotary_dim, int(write), _tag(qkv.dtype), _ptr(error),
                                     _stream()), "rope_kv_write")


# ----------------------------------------------------------------------------- SwiGLU
def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i]."""
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    tokens, two_inter = gate_up.shape
    inter = two_inter // 2
    if two_inter != 2 * inter or out.numel() < tokens * inter:
        raise KernelError("swiglu: shapes do not fit")
    _check(core().fsie_swiglu(_ptr(gate_up), _ptr(out), tokens, inter, _tag(out.dtype), _stream()),
           "swiglu")
    return out


def place_tokens(ids: torch.Tensor, dst_and_row: torch.Tensor, chosen: torch.Tensor) -> None:
    """ids[dst[i]] = chosen[row[i]] for dst_and_row = [dst (n), row (n)], all int32 on the device."""
    for name, t in (("ids", ids), ("dst_and_row", dst_and_row), ("chosen", chosen)):
        _need(t, torch.int32, name)
    n = dst_and_row.numel() // 2
    _check(core().fsie_place_tokens(_ptr(ids), _ptr(dst_and_row), _ptr(dst_and_row[n:]),
                                    _ptr(chosen), n, _stream()), "place_tokens")


# --------------------------------------------------------------------- float32 product
GEMM_F32_KINDS = {"auto": 0, "rows": 1, "tiles": 2, "plain": 3}


def gemm_f32_rows_limit() -> int:
    """Rows of x up to which the float32 product takes its few-rows kernel."""
    return int(core().fsie_gemm_f32_rows_limit())


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
             out: Optional[torch.Tensor] = None, kind: str = "auto",
             rows_per_warp: int = 0) -> torch.Tensor:
    """out = x @ weight.T (+ bias), all float32, plain FFMA (no tensor-core mode).  `kind`
    names one of the three kernels (few rows, tiles, plain) instead of the choice by size;
    `rows_per_warp` (1, 2, 4) fixes how many rows of the weight a warp of the few-rows kernel
    owns instead of the choice by size."""
    _need(x, torch.float32, "x", contiguous=False)
    _need(weight, torch.float32, "weight")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("gemm_f32: x must be 2-D with unit inner stride")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError("gemm_f32: inner sizes differ")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _need(out, torch.float32, "out", contiguous=False)
    if out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError("gemm_f32: out must be [rows of x, rows of weight] with unit inner stride")
    _check(core().fsie_gemm_f32(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), m, n, k,
                                x.stride(0), out.stride(0), GEMM_F32_KINDS[kind], int(rows_per_warp),
                                _stream()),
           "gemm_f32")
    return out


# -------------------------------------------------------------------------- attention
def attention_rows_per_tile() -> int:
    return int(core().fsie_attn_generic_rows())


def attention_generic(q: torch.Tensor, q_ld: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      page_stride: int, page_size: int, block_tables: torch.Tensor,
                      tile_item: torch.Tensor, tile_row0: torch.Tensor, num_tiles: int,
                      item_qstart: torch.Tensor, item_qlen: torch.Tensor, item_pos0: torch.Tensor,
                      out: torch.Tensor, tokens: int, heads: int, kv_heads: int, head_dim: int,
                      window: int, scale: float, nsplit: int = 1,
                      part_o: Optional[torch.Tensor] = None,
                      part_ml: Optional[torch.Tensor] = None, rows16: bool = False,
                      merge: bool = True) -> torch.Tensor:
    """The 32-bit attention over tiles of up to 32 query rows (any storage, any head size up to
    256), or with `rows16` over tiles of up to 16 rows by the kernel for few rows (float storage,
    head sizes in steps of 4).  `merge=False` leaves the partial results of split key ranges
    unmerged: a step whose tiles go out in several launches merges with the last."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0)):
        _need(t, torch.int32, name)
    _need(q, None, "q", contiguous=False)
    _need(out, q.dtype, "out")
    if k_pages.dtype is not q.dtype or v_pages.dtype is not q.dtype:
        raise KernelError("attention: cache dtype differs from q")
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention: split scratch is too small")
    _check(core().fsie_attn_tiles(_ptr(q), q_ld, _ptr(k_pages), _ptr(v_pages), page_stride,
                                  page_size, _ptr(block_tables), block_tables.stride(0),
                                  _ptr(tile_item), _ptr(tile_row0), num_tiles,
                                  _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0),
                                  _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), tokens,
                                  heads, kv_heads, head_dim, window, nsplit, float(scale),
                                  _tag(q.dtype), int(rows16), int(merge), _stream()),
           "attention_generic")
    return out


def attention_rows16_fits(dtype: torch.dtype, head_dim: int, page_stride: int) -> bool:
    """Whether the 32-bit attention kernel for tiles of up to 16 rows takes this cache."""
    return (dtype is torch.float32 and page_stride % 4 == 0
            and bool(core().fsie_attn_rows16_takes(int(head_dim))))


def attention_rows16_rows() -> int:
    return int(core().fsie_attn_rows16_rows())


_attn_mma = {}


def attn_mma(head_dim: int):
    """The tensor-core attention library for one head size, compiled at first use."""
    if head_dim not in _attn_mma:
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise KernelError(f"tensor-core attention takes head sizes 16..256 in steps of 16, "
                              f"not {head_dim}")
        lib = build.load_library("attn_mma", (f"-DHEAD_DIM={head_dim}",))
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_attn_mma.argtypes = [i, p, i, p, p, ll, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                      i, i, i, i, i, i, f, p, i, p]
        lib.fsie_attn_mma.restype = i
        lib.fsie_attn_mma_rows.argtypes = [i]
        lib.fsie_attn_mma_rows.restype = i
        _attn_mma[head_dim] = lib
    return _attn_mma[head_dim]


ATTENTION_ROW_CLASSES = (16, 32, 64)      # rows per tile of row class 0, 1, 2


def attention_mma(row_class: int, q: torch.Tensor, q_ld: int, k_pages: torch.Tensor,
                  v_pages: torch.Tensor, page_stride: int, page_size: int,
                  block_tables: torch.Tensor, tile_item: torch.Tensor, tile_row0: torch.Tensor,
                  num_tiles: int, item_qstart: torch.Tensor, item_qlen: torch.Tensor,
                  item_pos0: torch.Tensor, out: torch.Tensor, tokens: int, heads: int,
                  kv_heads: int, head_dim: int, window: int, scale: float, nsplit: int = 1,
                  part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                  combine_tokens: Optional[torch.Tensor] = None, num_combine: int = 0
                  ) -> torch.Tensor:
    """bfloat16 attention of one row class (tiles of 16, 32 or 64 rows) on the tensor cores."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0)):
        _need(t, torch.int32, name)
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(out, torch.bfloat16, "out")
    if k_pages.dtype is not torch.bfloat16 or v_pages.dtype is not torch.bfloat16:
        raise KernelError("attention_mma: the cache must be bfloat16")
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention_mma: split scratch is too small")
        if combine_tokens is not None:
            _need(combine_tokens, torch.int32, "combine_tokens")
    _check(attn_mma(head_dim).fsie_attn_mma(
        row_class, _ptr(q), q_ld, _ptr(k_pages), _ptr(v_pages), page_stride, page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles,
        _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0), _ptr(out), out.stride(0),
        _ptr(part_o), _ptr(part_ml), tokens, heads, kv_heads, head_dim, window, nsplit,
        float(scale), _ptr(combine_tokens), num_combine, _stream()), "attention_mma")
    return out


_attn_tc = {}
ATTENTION_TC_PAGES = (8, 16, 32, 64, 128)
ATTENTION_TC_HEAD_DIMS = (64, 128)
ATTENTION_TC_ROWS = 256
ATTENTION_TC_DECODE_HEAD_DIMS = (128,)      # tiles of up to 16 rows: attention_tc_decode


def attn_tc(head_dim: int):
    """The tcgen05 attention library (prompt portions) for one head size (64 or 128)."""
    if head_dim not in _attn_tc:
        if head_dim not in ATTENTION_TC_HEAD_DIMS:
            raise KernelError(f"tcgen05 attention takes head sizes 64 and 128, not {head_dim}")
        lib = build.load_library("attn_tc", (f"-DHEAD_DIM={head_dim}",))
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_attn_tc_map_bytes.argtypes = []
        lib.fsie_attn_tc_pages_map.argtypes = [p, p, ll, i, i]
        lib.fsie_attn_tc.argtypes = [p, i, i, p, i, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                     i, i, i, i, i, i, f, p, i, p, p]
        lib.fsie_attn_tc_decode.argtypes = lib.fsie_attn_tc.argtypes
        lib.fsie_attn_tc_decode_rows.argtypes = []
        for name in ("fsie_attn_tc_map_bytes", "fsie_attn_tc_pages_map", "fsie_attn_tc",
                     "fsie_attn_tc_decode", "fsie_attn_tc_decode_rows"):
            getattr(lib, name).restype = i
        _attn_tc[head_dim] = lib
    return _attn_tc[head_dim]


class PagesMap:
    """TMA descriptor of one cache group's pages [pages, entries, 2, kv_heads, slots, head_dim]
    (boxes of one page x 64 columns, 128-byte swizzle), as the tcgen05 attention kernels read it."""

    def __init__(self, pages: torch.Tensor, kind: str = "tc"):
        _need(pages, torch.bfloat16, "pages")
        num_pages, entries, two, kv_heads, page_size, head_dim = pages.shape
        if two != 2:
            raise KernelError("pages must be [pages, entries, 2, kv_heads, slots, head_dim]")
        self.pages, self.entries, self.page_size, self.head_dim = pages, entries, page_size, head_dim
        rows = num_pages * entries * 2 * kv_heads * page_size
        if kind != "tc":
            raise KernelError(f"PagesMap: unknown kind '{kind}'")
        lib = attn_tc(head_dim)
        size, encode = lib.fsie_attn_tc_map_bytes(), lib.fsie_attn_tc_pages_map
        self.buffer = ctypes.create_string_buffer(size + 64)
        offset = (-ctypes.addressof(self.buffer)) % 64
        self.ptr = ctypes.c_void_p(ctypes.addressof(self.buffer) + offset)
        _check(encode(self.ptr, _ptr(pages), rows, head_dim, page_size), "attention pages map")


def attention_tc(pages_map: PagesMap, entry: int, q: torch.Tensor, q_ld: int,
                 block_tables: torch.Tensor, tile_item: torch.Tensor, tile_row0: torch.Tensor,
                 num_tiles: int, item_qstart: torch.Tensor, item_qlen: torch.Tensor,
                 item_pos0: torch.Tensor, out: torch.Tensor, tokens: int, heads: int,
                 kv_heads: int, window: int, scale: float, error: torch.Tensor, nsplit: int = 1,
                 part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                 combine_tokens: Optional[torch.Tensor] = None, num_combine: int = 0
                 ) -> torch.Tensor:
    """bfloat16 attention of prompt portions (tiles of 128 query rows) with tcgen05.mma."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0), ("error", error)):
        _need(t, torch.int32, name)
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(out, torch.bfloat16, "out")
    head_dim = pages_map.head_dim
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention_tc: split scratch is too small")
    _check(attn_tc(head_dim).fsie_attn_tc(
        pages_map.ptr, pages_map.entries, entry, _ptr(q), q_ld, pages_map.page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles,
        _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0), _ptr(out), out.stride(0),
        _ptr(part_o), _ptr(part_ml), tokens, heads, kv_heads, head_dim, window, nsplit,
        float(scale), _ptr(combine_tokens), num_combine, _ptr(error), _stream()), "attention_tc")
    return out


def attention_tc_decode(pages_map: PagesMap, entry: int, q: torch.Tensor, q_ld: int,
                        block_tables: torch.Tensor, tile_item: torch.Tensor,
                        tile_row0: torch.Tensor, num_tiles: int, item_qstart: torch.Tensor,
                        item_qlen: torch.Tensor, item_pos0: torch.Tensor, out: torch.Tensor,
                        tokens: int, heads: int, kv_heads: int, window: int, scale: float,
                        error: torch.Tensor, nsplit: int = 1,
                        part_o: Optional[torch.Tensor] = None,
                        part_ml: Optional[torch.Tensor] = None,
                        combine_tokens: Optional[torch.Tensor] = None, num_combine: int = 0
                        ) -> torch.Tensor:
    """bfloat16 attention of decoded tokens (tiles of up to 16 query rows, head size 128) with
    tcgen05.mma: the keys of a tile are the M side."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0), ("error", error)):
        _need(t, torch.int32, name)
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(out, torch.bfloat16, "out")
    head_dim = pages_map.head_dim
    if head_dim not in ATTENTION_TC_DECODE_HEAD_DIMS:
        raise KernelError(f"attention_tc_decode takes head size 128, not {head_dim}")
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention_tc_decode: split scratch is too small")
    _check(attn_tc(head_dim).fsie_attn_tc_decode(
        pages_map.ptr, pages_map.entries, entry, _ptr(q), q_ld, pages_map.page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles,
        _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0), _ptr(out), out.stride(0),
        _ptr(part_o), _ptr(part_ml), tokens, heads, kv_heads, head_dim, window, nsplit,
        float(scale), _ptr(combine_tokens), num_combine, _ptr(error), _stream()),
        "attention_tc_decode")
    return out


# ------------------------------------------------- tcgen05 product for few tokens
_gemm_decode = None


def gemm_decode_lib():
    global _gemm_decode
    if _gemm_decode is None:
        lib = build.load_library("gemm_decode")
        i, ll, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_tensor_map_bytes.argtypes = []
        lib.fsie_gemm_decode_weight_map.argtypes = [p, p, ll, ll, i]
        lib.fsie_gemm_decode.argtypes = [p, p, i, p, i, p, i, i, i, i, i, i, p, p]
        for name in ("fsie_tensor_map_bytes", "fsie_gemm_decode_weight_map", "fsie_gemm_decode"):
            getattr(lib, name).restype = i
        _gemm_decode = lib
    return _gemm_decode


GEMM_DECODE_MAX_TOKENS = 64


class DecodeWeight:
    """A bfloat16 weight [rows, K] prepared for `gemm_decode`: its TMA descriptor.
    For SwiGLU the weight holds the gate rows and then as many up rows."""

    def __init__(self, weight: torch.Tensor, swiglu: bool = False, activation: str = "silu"):
        _need(weight, torch.bfloat16, "weight")
        self.gate = 1 + GATE_KINDS[activation] if swiglu else 0     # what the kernel is told
        rows, k = weight.shape
        if k % 8:
            raise KernelError("gemm_decode: K must be a multiple of 8")
        if swiglu and rows % 2:
            raise KernelError("gemm_decode: a SwiGLU weight holds gate rows and as many up rows")
        lib = gemm_decode_lib()
        self.weight, self.swiglu, self.k = weight, swiglu, k
        self.n = rows // 2 if swiglu else rows
        self.map = ctypes.create_string_buffer(lib.fsie_tensor_map_bytes() + 64)
        offset = (-ctypes.addressof(self.map)) % 64
        self.map_ptr = ctypes.c_void_p(ctypes.addressof(self.map) + offset)
        _check(lib.fsie_gemm_decode_weight_map(self.map_ptr, _ptr(weight), rows, k,
                                               64 if swiglu else 128), "gemm_decode weight map")


def gemm_decode_splits(tiles: int, k: int, sm_count: int) -> int:
    """Blocks of a cluster that share the k range of one tile: enough to occupy the GPU."""
    splits = 1
    while splits < 8 and tiles * splits < sm_count and (k // 64) // (splits * 2) >= 4:
        splits *= 2
    return splits


def gemm_decode(weight: DecodeWeight, x: torch.Tensor, out: torch.Tensor,
                bias: Optional[torch.Tensor], error: torch.Tensor, splits: int = 1) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w.T (+ bias), or silu(x @ gate.T) * (x @ up.T); T <= 64; out is
    bfloat16 or float32."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, None, "out")
    tokens, k = x.shape
    if k != weight.k or x.stride(1) != 1 or tokens > GEMM_DECODE_MAX_TOKENS:
        raise KernelError("gemm_decode: x does not fit the weight (or more than 64 tokens)")
    if out.shape[0] < tokens or out.shape[1] != weight.n or out.dtype not in (torch.bfloat16,
                                                                            torch.float32):
        raise KernelError("gemm_decode: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
    _check(gemm_decode_lib().fsie_gemm_decode(
        weight.map_ptr, _ptr(x), x.stride(0), _ptr(out), out.stride(0), _ptr(bias), tokens,
        weight.n, k, weight.gate, int(out.dtype is torch.float32), splits, _ptr(error),
        _stream()), "gemm_decode")
    return out


_gemm_skinny = None
GEMM_SKINNY_MAX_TOKENS = 16


def gemm_skinny_fits(tokens: int, k: int) -> bool:
    """Whether `gemm_skinny` takes a product of `tokens` rows over `k`."""
    return 0 < tokens <= GEMM_SKINNY_MAX_TOKENS and k % 32 == 0


def gemm_skinny_lib():
    global _gemm_skinny
    if _gemm_skinny is None:
        lib = build.load_library("gemm_skinny")
        i, ll, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_gemm_skinny.argtypes = [p, p, ll, p, ll, p, i, i, i, i, p]
        lib.fsie_gemm_skinny.restype = i
        lib.fsie_gemm_skinny_qkv_rope.argtypes = [p, p, ll, p, ll, p, i, i, p, p, i, p, p, p, ll, i,
                                                  i, i, i, p, p]
        lib.fsie_gemm_skinny_qkv_rope.restype = i
        _gemm_skinny = lib
    return _gemm_skinny


def gemm_skinny_qkv_rope(weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor,
                         bias: Optional[torch.Tensor], positions: torch.Tensor,
                         cos_sin: torch.Tensor, slot_of: Optional[torch.Tensor],
                         k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                         page_stride: int, page_size: int, heads: int, kv_heads: int,
                         head_dim: int, error: torch.Tensor) -> torch.Tensor:
    """The q, k, v product of up to 16 tokens with the rotation of q and k and the cache write in
    its epilogue: rotated queries into out[:, :heads * head_dim] (bfloat16; the key and value
    columns of `out` are not written), rotated keys and the values into the pages (not when
    k_pages is None).  The whole head is rotated: cos_sin is [positions, head_dim]."""
    lib = gemm_skinny_lib()
    _need(weight, torch.bfloat16, "weight")
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(positions, torch.int32, "positions")
    _need(cos_sin, torch.float32, "cos_sin")
    _need(error, torch.int32, "error")
    tokens, k = x.shape
    n = (heads + 2 * kv_heads) * head_dim
    if weight.shape != (n, k) or x.stride(1) != 1 or not gemm_skinny_fits(tokens, k):
        raise KernelError("gemm_skinny_qkv_rope: x does not fit the weight, or the sizes are beyond the kernel")
    if head_dim % 16 or cos_sin.shape[-1] != head_dim:
        raise KernelError("gemm_skinny_qkv_rope: needs a head size in steps of 16, rotated as a whole")
    if out.shape[0] != tokens or out.shape[1] < heads * head_dim or out.stride(1) != 1:
        raise KernelError("gemm_skinny_qkv_rope: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
    if k_pages is not None:
        _need(slot_of, torch.int32, "slot_of")
        if k_pages.dtype is not torch.bfloat16 or v_pages.dtype is not torch.bfloat16:
            raise KernelError("gemm_skinny_qkv_rope: the cache must be bfloat16")
    _check(lib.fsie_gemm_skinny_qkv_rope(
        _ptr(weight), _ptr(x), x.stride(0), _ptr(out), out.stride(0), _ptr(bias), tokens, k,
        _ptr(positions), _ptr(cos_sin), cos_sin.shape[0], _ptr(slot_of), _ptr(k_pages),
        _ptr(v_pages), page_stride, page_size, heads, kv_heads, head_dim, _ptr(error), _stream()),
        "gemm_skinny_qkv_rope")
    return out


def gemm_skinny(weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor,
                bias: Optional[torch.Tensor]) -> torch.Tensor:
    """out[T, N] = x[T, K] @ weight.T (+ bias) for T <= 16: no pipeline to fill, every lane asks
    for its weights straight from global memory (for matrices so small that set-up would
    dominate).  out is bfloat16 or float32."""
    gemm_skinny_lib()
    _need(weight, torch.bfloat16, "weight")
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, None, "out", contiguous=False)
    tokens, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or x.stride(1) != 1 or not gemm_skinny_fits(tokens, k):
        raise KernelError("gemm_skinny: x does not fit the weight, or the sizes are beyond the kernel")
    if out.shape[0] != tokens or out.shape[1] != n or out.stride(1) != 1 or \
            out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_skinny: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
    _check(_gemm_skinny.fsie_gemm_skinny(_ptr(weight), _ptr(x), x.stride(0), _ptr(out), out.stride(0),
                                         _ptr(bias), tokens, n, k, int(out.dtype is torch.float32),
                                         _stream()), "gemm_skinny")
    return out


_gemm_tiles = None


def gemm_tiles_lib():
    global _gemm_tiles
    if _gemm_tiles is None:
        lib = build.load_library("gemm_tiles")
        i, ll, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_gemm_tiles_map_bytes.argtypes = []
        lib.fsie_gemm_tiles_weight_map.argtypes = [p, p, ll, ll]
        lib.fsie_gemm_tiles.argtypes = [p, p, ll, p, ll, p, i, i, i, i, i, i, p, ll, p, i, p, p]
        lib.fsie_gemm_tiles_workspace.argtypes = [i, i, i, i, i, ctypes.POINTER(ll), ctypes.POINTER(i)]
        lib.fsie_gemm_tiles_pairs.argtypes = []
        lib.fsie_gemm_tiles_grouped.argtypes = [p, p, ll, p, ll, i, i, i, i, i, p, p, i, p, p]
        for name in ("fsie_gemm_tiles_map_bytes", "fsie_gemm_tiles_weight_map", "fsie_gemm_tiles",
                     "fsie_gemm_tiles_pairs", "fsie_gemm_tiles_workspace", "fsie_gemm_tiles_grouped"):
            getattr(lib, name).restype = i
        pairs = lib.fsie_gemm_tiles_pairs()       # also sets the kernels up, outside any capture
        if pairs <= 0:
            raise KernelError(f"gemm_tiles: pairs of blocks cannot be launched here (code {pairs})")
        lib.pairs = pairs
        _gemm_tiles = lib
    return _gemm_tiles


def gemm_tiles_count(rows: int, n: int, swiglu: bool) -> int:
    """Output tiles of `gemm_tiles` for a product of `rows` tokens and `n` output features."""
    return -(-rows // 256) * -(-n // (128 if swiglu else 256))


class TiledWeight:
    """A bfloat16 weight [rows, K] prepared for `gemm_tiles`: its TMA descriptor (boxes of 128
    rows).  For SwiGLU the weight holds the gate rows and then as many up rows."""

    def __init__(self, weight: torch.Tensor, swiglu: bool = False, activation: str = "silu"):
        _need(weight, torch.bfloat16, "weight")
        self.gate = 1 + GATE_KINDS[activation] if swiglu else 0     # what the kernel is told
        rows, k = weight.shape
        if k % 8:
            raise KernelError("gemm_tiles: K must be a multiple of 8")
        if swiglu and rows % 2:
            raise KernelError("gemm_tiles: a SwiGLU weight holds gate rows and as many up rows")
        lib = gemm_tiles_lib()
        self.weight, self.swiglu, self.k = weight, swiglu, k
        self.n = rows // 2 if swiglu else rows
        self.map = ctypes.create_string_buffer(lib.fsie_gemm_tiles_map_bytes() + 64)
        offset = (-ctypes.addressof(self.map)) % 64
        self.map_ptr = ctypes.c_void_p(ctypes.addressof(self.map) + offset)
        _check(lib.fsie_gemm_tiles_weight_map(self.map_ptr, _ptr(weight), rows, k),
               "gemm_tiles weight map")


def gemm_tiles_workspace(rows: int, n: int, k: int, swiglu: bool, blocks: int) -> Tuple[int, int]:
    """(floats of workspace, ints of counters) with which `gemm_tiles` shares the tiles of a
    partial last round out among all pairs of blocks; (0, 0) where it has none to share."""
    floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
    code = gemm_tiles_lib().fsie_gemm_tiles_workspace(rows, n, k, int(swiglu), blocks,
                                                      ctypes.byref(floats), ctypes.byref(counters))
    if code != 0:
        raise KernelError(f"gemm_tiles_workspace failed with code {code}")
    return int(floats.value), int(counters.value)


def gemm_tiles(weight: TiledWeight, x: torch.Tensor, out: torch.Tensor,
               bias: Optional[torch.Tensor], error: torch.Tensor, blocks: int,
               workspace: Optional[torch.Tensor] = None,
               counters: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w.T (+ bias), or silu(x @ gate.T) * (x @ up.T), any M; out is
    bfloat16 (or float32 for the plain product).  `blocks`: size of the persistent grid.
    workspace (float32) and counters (int32, zero before the first call; every call leaves them
    zero) of the sizes `gemm_tiles_workspace` names let the kernel share out the tiles of a
    partial last round; without them every tile is summed by one pair of blocks."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, None, "out", contiguous=False)
    rows, k = x.shape
    if k != weight.k or x.stride(1) != 1 or x.stride(0) % 8:
        raise KernelError("gemm_tiles: x does not fit the weight (rows must start on 16 bytes)")
    if (out.shape[0] != rows or out.shape[1] != weight.n or out.stride(1) != 1
            or out.dtype not in (torch.bfloat16, torch.float32)
            or (weight.swiglu and out.dtype is torch.float32)):
        raise KernelError("gemm_tiles: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
        if weight.swiglu or bias.numel() != weight.n:
            raise KernelError("gemm_tiles: bias does not fit")
    if workspace is not None:
        _need(workspace, torch.float32, "workspace")
        _need(counters, torch.int32, "counters")
    _check(gemm_tiles_lib().fsie_gemm_tiles(
        weight.map_ptr, _ptr(x), x.stride(0), _ptr(out), out.stride(0), _ptr(bias), rows,
        weight.n, k, weight.gate, int(out.dtype is torch.float32), blocks,
        _ptr(workspace), workspace.numel() if workspace is not None else 0,
        _ptr(counters), counters.numel() if counters is not None else 0, _ptr(error),
        _stream()), "gemm_tiles")
    return out


GEMM_TILES_ROWS = 256     # rows of a tile of `gemm_tiles`: a group's rows start on a multiple of it


class GroupedTiledWeight:
    """Bfloat16 matrices [groups, rows, K] of equal shape prepared for `gemm_tiles_grouped`: one TMA
    descriptor over all of them.  For SwiGLU each matrix holds the gate rows and then as many up
    rows."""

    def __init__(self, weight: torch.Tensor, swiglu: bool = False, activation: str = "silu",
                 plain_activation: Optional[str] = None):
        _need(weight, torch.bfloat16, "weight")
        if swiglu and GATE_KINDS[activation] > 1:
            raise KernelError("gemm_tiles_grouped: the gate is SiLU or the tanh form of GELU")
        self.gate = 1 + GATE_KINDS[activation] if swiglu else 0
        if plain_activation is not None:       # no gate: the activation on the product itself
            if swiglu or plain_activation != "relu2":
                raise KernelError("gemm_tiles_grouped: without a gate the activation is 'relu2'")
            self.gate = 3
        groups, rows, k = weight.shape
        if k % 8 or (swiglu and rows % 2):
            raise KernelError("gemm_tiles_grouped: K must be a multiple of 8, a SwiGLU matrix hold "
                              "gate rows and as many up rows")
        lib = gemm_tiles_lib()
        self.weight, self.swiglu, self.k, self.groups, self.rows = weight, swiglu, k, groups, rows
        self.n = rows // 2 if swiglu else rows
        self.map = ctypes.create_string_buffer(lib.fsie_gemm_tiles_map_bytes() + 64)
        offset = (-ctypes.addressof(self.map)) % 64
        self.map_ptr = ctypes.c_void_p(ctypes.addressof(self.map) + offset)
        _check(lib.fsie_gemm_tiles_weight_map(self.map_ptr, _ptr(weight), groups * rows, k),
               "gemm_tiles_grouped weight map")


def gemm_tiles_grouped(weight: GroupedTiledWeight, x: torch.Tensor, out: torch.Tensor,
                       tile_group: torch.Tensor, tiles_used: torch.Tensor, error: torch.Tensor,
                       blocks: int) -> torch.Tensor:
    """Row tile m of x (256 rows, all of one group) times the matrix of group tile_group[m]:
    out[r] = x[r] @ w[g].T, or silu(x[r] @ gate[g].T) * (x[r] @ up[g].T).  x [M, K] and out [M, N]
    are bfloat16 with M a multiple of 256; only the first tiles_used[0] row tiles are computed (both
    lists are int32 on the device, written by a kernel earlier in the stream)."""
    _need(x, torch.bfloat16, "x")
    _need(out, torch.bfloat16, "out")
    _need(tile_group, torch.int32, "tile_group")
    _need(tiles_used, torch.int32, "tiles_used")
    rows, k = x.shape
    if k != weight.k or rows % GEMM_TILES_ROWS or out.shape[0] != rows or out.shape[1] != weight.n or \
            tile_group.numel() < rows // GEMM_TILES_ROWS:
        raise KernelError("gemm_tiles_grouped: shapes do not fit")
    _check(gemm_tiles_lib().fsie_gemm_tiles_grouped(
        weight.map_ptr, _ptr(x), x.stride(0), _ptr(out), out.stride(0), rows, weight.n, k, weight.gate,
        blocks, _ptr(tile_group), _ptr(tiles_used), weight.rows, _ptr(error), _stream()),
        "gemm_tiles_grouped")
    return out


# --------------------------------------------------------------------------- sampling
ARGMAX_PARTS = 64      # blocks per row of the two-stage argmax
_argmax_scratch: Dict[int, torch.Tensor] = {}


def argmax(logits: torch.Tensor, out: torch.Tensor,
           scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = index of the largest logit of row r, ties to the smallest index.  A wide row is
    reduced by ARGMAX_PARTS blocks and a second small kernel (in `scratch`, float32, at least
    2 * rows * ARGMAX_PARTS elements; the module keeps one per device when none is given -
    pass your own inside a stream capture); a narrow row by one block."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    rows, vocab = logits.shape
    if vocab >= 8192:
        need = 2 * rows * ARGMAX_PARTS
        if scratch is None:
            key = logits.device.index or 0
            scratch = _argmax_scratch.get(key)
            if scratch is None or scratch.numel() < need:
                scratch = _argmax_scratch[key] = torch.empty(max(need, 1 << 16), dtype=torch.float32,
                                                             device=logits.device)
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError("argmax: scratch is too small")
        # enough blocks to fill the GPU several times over, each with more than a few loads per thread
        parts = max(4, min(ARGMAX_PARTS, 2048 // rows))
        _check(core().fsie_argmax_staged(_ptr(logits), rows, vocab, _ptr(out), _ptr(scratch),
                                         parts, _stream()), "argmax")
        return out
    _check(core().fsie_argmax(_ptr(logits), rows, vocab, _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(top_k, torch.int32, "top_k")
    _need(top_p, torch.float32, "top_p")
    _need(uniform, torch.float32, "uniform")
    _need(out, torch.int32, "out")
    rows, vocab = logits.shape
    _check(core().fsie_sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k),
                              _ptr(top_p), _ptr(uniform), _ptr(out), _stream()), "sample")
    return out


# ------------------------------------------------------------- parts of hybrid decoders
_hybrid = None


_scan = None


def scan():
    """The library of recurrences over per-request state of the form S <- a S + k v^T, o = S^T q
    (decaying linear attention; a state-space mixer with its convolution, step sizes and gated
    norm), compiled at first use."""
    global _scan
    if _scan is None:
        lib = build.load_library("scan")
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_lightning_scan.argtypes = [p, i, i, i, i, p, p, p, i, p, p, p, i, i, i, p, p, i, i, p,
                                            i, p, ll, p]
        lib.fsie_silu_rows.argtypes = [p, i, i, p, i, i, p]
        lib.fsie_gated_rmsnorm.argtypes = [p, p, i, i, p, p, i, i, f, i, p]
        lib.fsie_ssd_max_taps.argtypes = []
        lib.fsie_ssd_prep.argtypes = [p, i, i, i, p, p, p, i, p, ll, ll, p, p, i, i, p, p, i, i, p, i, p,
                                      p, i, i, p]
        lib.fsie_ssd_tails.argtypes = [p, i, i, p, p, p, i, p, ll, ll, i, i, i, p]
        lib.fsie_ssd_gate_norm.argtypes = [p, p, i, p, i, i, p, p, p, i, i, i, i, f, i, p]
        for name in ("fsie_lightning_scan", "fsie_silu_rows", "fsie_gated_rmsnorm", "fsie_ssd_max_taps",
                     "fsie_ssd_prep", "fsie_ssd_tails", "fsie_ssd_gate_norm"):
            getattr(lib, name).restype = i
        _scan = lib
    return _scan


def hybrid():
    """The library of the hybrid decoders' parts (layer norm on a sublayer's output, windowed
    attention with mixed heads), compiled at first use."""
    global _hybrid
    if _hybrid is None:
        lib = build.load_library("hybrid")
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_add_layernorm.argtypes = [p, p, p, p, p, i, i, f, i, i, p]
        lib.fsie_cast_rows.argtypes = [p, p, ll, i, p]
        lib.fsie_conv_norm_rotate.argtypes = [p, i, i, i, p, p, p, p, p, i, p, p, p, i, i, p, p, p,
                                              ll, i, p, i, i, i, i, i, f, i, p, p]
        lib.fsie_conv_tails.argtypes = [p, i, p, p, p, i, p, i, i, i, p]
        lib.fsie_talking_attention_tile_tokens.argtypes = [i]
        lib.fsie_talking_attention_key_tile.argtypes = [i, i, i, i, i]
        lib.fsie_talking_attention.argtypes = [p, p, p, ll, i, p, i, p, p, i, p, p, p, p, p, p,
                                               i, i, i, i, i, i, i, i, f, i, p, p, i, p, p]
        lib.fsie_talking_attention_mma_takes.argtypes = [i, i, i, i]
        lib.fsie_talking_attention_mma.argtypes = [p, p, p, ll, i, p, i, p, p, i, p, p, p, p, p, p, p,
                                                   i, i, i, i, i, i, i, f, p, p]
        lib.fsie_talking_attention_mma_takes.restype = i
        lib.fsie_talking_attention_mma.restype = i
        for name in ("fsie_add_layernorm", "fsie_cast_rows", "fsie_conv_norm_rotate", "fsie_conv_tails",
                     "fsie_talking_attention_tile_tokens", "fsie_talking_attention_key_tile",
                     "fsie_talking_attention"):
            getattr(lib, name).restype = i
        _hybrid = lib
    return _hybrid


def layernorm_rows(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
                   rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = LN(x[rows[r]]) * gain in out's dtype; x is the float32 residual stream.
    LN(v) = (v - mean) / sqrt(mean((v - mean)^2) + eps)."""
    _need(x, torch.float32, "x")
    _need(gain, torch.float32, "gain")
    _need(out, None, "out")
    width = x.shape[-1]
    if gain.numel() != width:
        raise KernelError("layernorm_rows: gain width differs from x")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        count = rows.numel()
    else:
        count = x.numel() // width
    if out.numel() < count * width:
        raise KernelError("layernorm_rows: out is too small")
    _check(hybrid().fsie_add_layernorm(_ptr(x), _ptr(rows), _ptr(gain), None, _ptr(out), count,
                                       width, float(eps), 0, _tag(out.dtype), _stream()),
           "layernorm_rows")
    return out


def add_layernorm(x: torch.Tensor, delta: torch.Tensor, gain: torch.Tensor, eps: float,
                  copy: Optional[torch.Tensor]) -> None:
    """x (float32 residual) += LN(delta) * gain; `copy`, when given, gets the new x in delta's
    dtype (what the next matrix product reads)."""
    _need(x, torch.float32, "x")
    _need(delta, None, "delta")
    _need(gain, torch.float32, "gain")
    width = x.shape[-1]
    count = x.numel() // width
    if delta.shape[-1] != width or delta.numel() != x.numel() or gain.numel() != width:
        raise KernelError("add_layernorm: shapes do not fit")
    if copy is not None:
        _need(copy, delta.dtype, "copy")
        if copy.numel() < x.numel():
            raise KernelError("add_layernorm: copy is too small")
    _check(hybrid().fsie_add_layernorm(_ptr(delta), None, _ptr(gain), _ptr(x), _ptr(copy), count,
                                       width, float(eps), 1, _tag(delta.dtype), _stream()),
           "add_layernorm")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = x (float32) in out's dtype."""
    _need(x, torch.float32, "x")
    _need(out, None, "out")
    if out.numel() < x.numel():
        raise KernelError("cast_rows: out is too small")
    _check(hybrid().fsie_cast_rows(_ptr(x), _ptr(out), x.numel(), _tag(out.dtype), _stream()),
           "cast_rows")
    return out


def silu_rows(proj: torch.Tensor, width: int, act: torch.Tensor) -> torch.Tensor:
    """act[t, c] = silu(proj[t, c]) for the first `width` columns, as float32 [tokens, width]."""
    _need(proj, None, "proj")
    _need(act, torch.float32, "act")
    tokens, ld = proj.shape
    if width > ld or act.numel() < tokens * width:
        raise KernelError("silu_rows: shapes do not fit")
    _check(scan().fsie_silu_rows(_ptr(proj), ld, width, _ptr(act), tokens, _tag(proj.dtype),
                                   _stream()), "silu_rows")
    return act


def lightning_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int,
                   item_qstart: torch.Tensor, item_qlen: torch.Tensor, item_slots: torch.Tensor,
                   items: int, state: torch.Tensor, decay: torch.Tensor, out: torch.Tensor,
                   heads: int, dim: int, vdim: int, seg_item: Optional[torch.Tensor] = None,
                   seg_row0: Optional[torch.Tensor] = None, num_segs: int = 0, seg_tokens: int = 0,
                   chunk_states: Optional[torch.Tensor] = None, share: int = 1,
                   decay_tok: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per request and head, token by token: S = decay * S + k v^T, o = S^T q.  proj [tokens, ld]
    (float32) holds the ACTIVATED projections (`silu_rows`) at the given column offsets; state
    [slots, heads, dim, vdim] (float32; or [slots, n] with the heads' matrices in the first
    heads * dim * vdim floats of a slot) is read and left updated; out [tokens, heads * vdim]
    float32.  `decay_tok` (float32 [tokens, heads]) gives a decay per token and head in place of
    `decay`; `share` heads in a row read the same q and k columns (q and k then hold heads / share
    column groups of `dim`).

    With `seg_item` / `seg_row0` (int32, one entry per chunk of `seg_tokens` tokens, listed
    request by request) and `chunk_states` (float32, num_segs * heads * dim * vdim at least; with
    `decay_tok` num_segs * heads more) the
    chunks of long prompts run side by side: each sums its own tokens, the sums are chained into
    the state at every chunk's start, and each chunk runs again from there for its outputs."""
    _need(proj, torch.float32, "proj")
    _need(state, torch.float32, "state")
    if decay is not None:
        _need(decay, torch.float32, "decay")
    _need(out, torch.float32, "out")
    for name, t in (("item_qstart", item_qstart), ("item_qlen", item_qlen), ("item_slots", item_slots)):
        _need(t, torch.int32, name)
    tokens, ld = proj.shape
    if share <= 0 or heads % share:
        raise KernelError("lightning_scan: heads must be a multiple of share")
    if max(q_off, k_off) + heads // share * dim > ld or v_off + heads * vdim > ld:
        raise KernelError("lightning_scan: projection rows are narrower than q, k and v")
    if decay_tok is not None:
        _need(decay_tok, torch.float32, "decay_tok")
        if decay_tok.numel() < tokens * heads:
            raise KernelError("lightning_scan: decay_tok is too small")
    elif decay is None:
        raise KernelError("lightning_scan: a decay per head or per token and head is needed")
    state_stride = state.stride(0)
    if state_stride < heads * dim * vdim or (decay is not None and decay.numel() != heads):
        raise KernelError("lightning_scan: state or decay does not fit the heads")
    if out.numel() < tokens * heads * vdim:
        raise KernelError("lightning_scan: out is too small")
    if seg_item is not None:
        _need(seg_item, torch.int32, "seg_item")
        _need(seg_row0, torch.int32, "seg_row0")
        _need(chunk_states, torch.float32, "chunk_states")
        if chunk_states.numel() < num_segs * heads * (dim * vdim + (decay_tok is not None)):
            raise KernelError("lightning_scan: chunk_states is too small")
    _check(scan().fsie_lightning_scan(_ptr(proj), ld, q_off, k_off, v_off, _ptr(item_qstart),
                                      _ptr(item_qlen), _ptr(item_slots), items, _ptr(state),
                                      _ptr(decay), _ptr(out), heads, dim, vdim, _ptr(seg_item),
                                      _ptr(seg_row0), num_segs, seg_tokens, _ptr(chunk_states),
                                      int(share), _ptr(decay_tok), state_stride, _stream()),
           "lightning_scan")
    return out


def ssd_max_taps() -> int:
    return int(scan().fsie_ssd_max_taps())


def ssd_prep(proj: torch.Tensor, conv_off: int, dt_off: int, item_qstart: torch.Tensor,
             item_qlen: torch.Tensor, item_slots: torch.Tensor, items: int,
             state: Optional[torch.Tensor], tail_off: int, conv_w: torch.Tensor,
             conv_b: Optional[torch.Tensor], dt_bias: torch.Tensor, a_log: torch.Tensor, heads: int,
             vdim: int, act: torch.Tensor, decay: torch.Tensor,
             conv_wt: Optional[torch.Tensor] = None) -> None:
    """What a state-space mixer's scan reads, per token of proj [tokens, ld] (the stored projection
    with the convolution's input columns at conv_off and the step sizes at dt_off):
    act [tokens, channels + heads * vdim] float32 = [silu(causal convolution + bias) | dt * x] with x
    the first heads * vdim convolved columns, dt = softplus(dt + dt_bias), and decay [tokens, heads]
    = exp(-exp(a_log) * dt).  conv_w float32 [channels, taps], the last column the current token's;
    the inputs of the taps - 1 tokens before a step's first live in the request's slot of `state`
    [slots, n] (float32) from float tail_off on, oldest first (`ssd_tails` moves them on).  conv_wt:
    conv_w transposed ([taps, channels], contiguous), with which sizes in multiples of 8 take eight
    channels per thread."""
    _need(proj, None, "proj")
    _need(conv_w, torch.float32, "conv_w")
    _need(dt_bias, torch.float32, "dt_bias")
    _need(a_log, torch.float32, "a_log")
    _need(act, torch.float32, "act")
    _need(decay, torch.float32, "decay")
    tokens, ld = proj.shape
    channels, taps = conv_w.shape
    if conv_off + channels > ld or dt_off + heads > ld or act.shape[1] < channels + heads * vdim or \
            act.shape[0] < tokens or decay.numel() < tokens * heads or dt_bias.numel() != heads or \
            a_log.numel() != heads or (conv_b is not None and conv_b.numel() != channels):
        raise KernelError("ssd_prep: shapes do not fit")
    if conv_wt is not None:
        _need(conv_wt, torch.float32, "conv_wt")
        if tuple(conv_wt.shape) != (taps, channels):
            raise KernelError("ssd_prep: conv_wt is not conv_w transposed")
    stride = 0
    if taps > 1:
        _need(state, torch.float32, "state", contiguous=False)
        stride = state.stride(0)
        if tail_off + (taps - 1) * channels > stride:
            raise KernelError("ssd_prep: the state slots do not hold the convolution's inputs")
    _check(scan().fsie_ssd_prep(_ptr(proj), ld, conv_off, dt_off, _ptr(item_qstart), _ptr(item_qlen),
                                _ptr(item_slots), items, _ptr(state), stride, tail_off, _ptr(conv_w),
                                _ptr(conv_b), taps, channels, _ptr(dt_bias), _ptr(a_log), heads, vdim,
                                _ptr(act), act.stride(0), _ptr(decay), _ptr(conv_wt), tokens,
                                _tag(proj.dtype), _stream()), "ssd_prep")


def ssd_tails(proj: torch.Tensor, conv_off: int, channels: int, taps: int, item_qstart: torch.Tensor,
              item_qlen: torch.Tensor, item_slots: torch.Tensor, items: int, state: torch.Tensor,
              tail_off: int) -> None:
    """After `ssd_prep`: every request's slot receives the convolution inputs of the last taps - 1
    tokens of (what it held, then the step's tokens)."""
    if taps <= 1:
        return
    _need(proj, None, "proj")
    _need(state, torch.float32, "state", contiguous=False)
    _check(scan().fsie_ssd_tails(_ptr(proj), proj.shape[1], conv_off, _ptr(item_qstart), _ptr(item_qlen),
                                 _ptr(item_slots), items, _ptr(state), state.stride(0), tail_off, taps,
                                 channels, _tag(proj.dtype), _stream()), "ssd_tails")


def ssd_gate_norm(o: torch.Tensor, act: torch.Tensor, proj: torch.Tensor, z_off: int, skip: torch.Tensor,
                  gain: torch.Tensor, out: torch.Tensor, vdim: int, parts: int, eps: float) -> torch.Tensor:
    """out[t] = v / sqrt(mean over each of `parts` equal parts of v^2 + eps) * gain with
    v = (o[t] + skip[head] * x[t]) * silu(z[t]); o float32 [tokens, inner], x the first inner
    columns of act (float32), z = proj[t, z_off : z_off + inner] of the storage type."""
    _need(o, torch.float32, "o")
    _need(act, torch.float32, "act")
    _need(proj, None, "proj")
    _need(skip, torch.float32, "skip")
    _need(gain, torch.float32, "gain")
    _need(out, proj.dtype, "out")
    tokens, inner = o.shape
    if z_off + inner > proj.shape[1] or gain.numel() != inner or skip.numel() * vdim != inner or \
            out.numel() < tokens * inner or act.shape[1] < inner:
        raise KernelError("ssd_gate_norm: shapes do not fit")
    _check(scan().fsie_ssd_gate_norm(_ptr(o), _ptr(act), act.stride(0), _ptr(proj), proj.shape[1], z_off,
                                     _ptr(skip), _ptr(gain), _ptr(out), tokens, inner, vdim, int(parts),
                                     float(eps), _tag(proj.dtype), _stream()), "ssd_gate_norm")
    return out


def gated_rmsnorm(o: torch.Tensor, proj: torch.Tensor, g_off: int, gain: torch.Tensor, eps: float,
                  out: torch.Tensor) -> torch.Tensor:
    """out[t] = o[t] * rsqrt(mean(o[t]^2) + eps) * gain * sigmoid(proj[t, g_off:g_off + width])."""
    _need(o, torch.float32, "o")
    _need(proj, None, "proj")
    _need(gain, torch.float32, "gain")
    _need(out, proj.dtype, "out")
    tokens, width = o.shape
    if g_off + width > proj.shape[1] or gain.numel() != width or out.numel() < tokens * width:
        raise KernelError("gated_rmsnorm: shapes do not fit")
    _check(scan().fsie_gated_rmsnorm(_ptr(o), _ptr(proj), proj.shape[1], g_off, _ptr(gain),
                                       _ptr(out), tokens, width, float(eps), _tag(proj.dtype),
                                       _stream()), "gated_rmsnorm")
    return out


def conv_norm_rotate(proj: torch.Tensor, items: int, item_qstart: torch.Tensor,
                     item_pos0: torch.Tensor, item_slots: torch.Tensor,
                     tails: Optional[torch.Tensor], conv_w: torch.Tensor, taps: int,
                     q_gain: torch.Tensor, k_gain: Optional[torch.Tensor], cos_sin: torch.Tensor,
                     rot_dims: int, slot_of: Optional[torch.Tensor],
                     k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                     page_stride: int, page_size: int, q_out: torch.Tensor, heads: int,
                     kv_heads: int, dim: int, vdim: int, has_kv: bool, eps: float,
                     error: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time of the projected q | k | v rows (earlier rows of the step, or
    the request's tail of taps - 1 rows), RMS norm of the whole q and the whole k with gains,
    rotation of interleaved pairs, per-head RMS of v; q -> q_out (float32), k and v -> pages."""
    _need(proj, None, "proj")
    _need(conv_w, torch.float32, "conv_w")
    _need(q_gain, torch.float32, "q_gain")
    _need(cos_sin, torch.float32, "cos_sin")
    _need(q_out, torch.float32, "q_out")
    for name, t in (("item_qstart", item_qstart), ("item_pos0", item_pos0), ("item_slots", item_slots)):
        _need(t, torch.int32, name)
    tokens, ld = proj.shape
    width = heads * dim + (kv_heads * (dim + vdim) if has_kv else 0)
    if ld != width or conv_w.shape != (width, taps) or q_gain.numel() != heads * dim:
        raise KernelError("conv_norm_rotate: projection, taps or gains do not fit")
    if taps > 1:
        _need(tails, torch.float32, "tails")
        if tuple(tails.shape[1:]) != (taps - 1, width):
            raise KernelError("conv_norm_rotate: tails must be [slots, taps - 1, width]")
    if rot_dims > 0 and cos_sin.shape[-1] != rot_dims:
        raise KernelError("conv_norm_rotate: cos/sin table width differs from the rotated size")
    if has_kv:
        _need(k_gain, torch.float32, "k_gain")
        _need(slot_of, torch.int32, "slot_of")
        if k_pages.dtype is not proj.dtype or v_pages.dtype is not proj.dtype:
            raise KernelError("conv_norm_rotate: cache dtype differs from the projection dtype")
    if q_out.numel() < tokens * heads * dim:
        raise KernelError("conv_norm_rotate: q_out is too small")
    _check(hybrid().fsie_conv_norm_rotate(
        _ptr(proj), ld, tokens, items, _ptr(item_qstart), _ptr(item_pos0), _ptr(item_slots),
        _ptr(tails) if taps > 1 else None, _ptr(conv_w), taps, _ptr(q_gain), _ptr(k_gain),
        _ptr(cos_sin), cos_sin.shape[0], rot_dims, _ptr(slot_of) if has_kv else None,
        _ptr(k_pages) if has_kv else None, _ptr(v_pages) if has_kv else None, page_stride,
        page_size, _ptr(q_out), heads, kv_heads, dim, vdim, int(has_kv), float(eps),
        _tag(proj.dtype), _ptr(error), _stream()), "conv_norm_rotate")
    return q_out


def conv_tails(proj: torch.Tensor, item_qstart: torch.Tensor, item_qlen: torch.Tensor,
               item_slots: torch.Tensor, items: int, tails: torch.Tensor, taps: int) -> None:
    """Leave in every request's tail the projected rows of its last taps - 1 positions."""
    _need(proj, None, "proj")
    _need(tails, torch.float32, "tails")
    width = proj.shape[1]
    if tuple(tails.shape[1:]) != (taps - 1, width):
        raise KernelError("conv_tails: tails must be [slots, taps - 1, width]")
    _check(hybrid().fsie_conv_tails(_ptr(proj), width, _ptr(item_qstart), _ptr(item_qlen),
                                    _ptr(item_slots), items, _ptr(tails), taps, width,
                                    _tag(proj.dtype), _stream()), "conv_tails")


def talking_attention_tile_tokens(heads: int) -> int:
    """Consecutive tokens of one request that a block of the mixed-heads attention takes: 8, 4,
    2 or 1 as the heads grow (0: more heads than the kernel holds)."""
    return int(hybrid().fsie_talking_attention_tile_tokens(int(heads)))


def talking_attention_key_tile(heads: int, kv_heads: int, dim: int, vdim: int,
                               dtype: torch.dtype) -> int:
    """Keys that a block of the mixed-heads attention takes at a time (0: sizes do not fit)."""
    return int(hybrid().fsie_talking_attention_key_tile(heads, kv_heads, dim, vdim, _tag(dtype)))


def talking_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      page_stride: int, page_size: int, block_tables: torch.Tensor,
                      tile_item: torch.Tensor, tile_row0: torch.Tensor, num_tiles: int,
                      item_qstart: torch.Tensor, item_qlen: torch.Tensor, item_pos0: torch.Tensor,
                      item_slots: torch.Tensor, talk: torch.Tensor, out: torch.Tensor, heads: int,
                      kv_heads: int, dim: int, vdim: int, window: int, keep_first: int,
                      tile_tokens: int, scale: float, error: torch.Tensor, nsplit: int = 1,
                      part_stats: Optional[torch.Tensor] = None,
                      part_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax attention of q (float32 [tokens, heads * dim]) over the visible keys of the pages
    (j <= i and (window == 0 or i - j < window or j < keep_first)); the normalised weights of all
    heads are mixed by `talk` [heads, heads] before head h applies its own to the values of its
    key/value head.  out [tokens, heads * vdim] in the pages' dtype.  Tiles are `tile_tokens`
    consecutive tokens of a request (1, or what `talking_attention_tile_tokens` says); with
    nsplit > 1 every tile's keys are split over that many blocks (float32 scratch part_stats
    [tiles * nsplit * 128], part_out [nsplit * tokens * heads * vdim])."""
    _need(q, torch.float32, "q")
    _need(talk, torch.float32, "talk")
    _need(out, k_pages.dtype, "out")
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0), ("item_slots", item_slots)):
        _need(t, torch.int32, name)
    if v_pages.dtype is not k_pages.dtype:
        raise KernelError("talking_attention: keys and values differ in dtype")
    if talk.numel() != heads * heads:
        raise KernelError("talking_attention: the mixing matrix must be [heads, heads]")
    tokens = q.shape[0]
    if nsplit > 1:
        _need(part_stats, torch.float32, "part_stats")
        _need(part_out, torch.float32, "part_out")
        if part_stats.numel() < num_tiles * nsplit * 128 or \
                part_out.numel() < nsplit * tokens * heads * vdim:
            raise KernelError("talking_attention: split scratch is too small")
    _check(hybrid().fsie_talking_attention(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), page_stride, page_size, _ptr(block_tables),
        block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles, _ptr(item_qstart),
        _ptr(item_qlen), _ptr(item_pos0), _ptr(item_slots), _ptr(talk), _ptr(out), tokens, heads,
        kv_heads, dim, vdim, window, keep_first, tile_tokens, float(scale), nsplit,
        _ptr(part_stats), _ptr(part_out), _tag(k_pages.dtype), _ptr(error), _stream()),
        "talking_attention")
    return out


TALKING_MMA_TILE_TOKENS = 16


def talking_attention_mma_takes(heads: int, kv_heads: int, dim: int, vdim: int,
                                dtype: torch.dtype) -> bool:
    """Whether the tensor-core form of the mixed-heads attention takes these sizes."""
    return dtype is torch.bfloat16 and bool(
        hybrid().fsie_talking_attention_mma_takes(heads, kv_heads, dim, vdim))


def talking_attention_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                          page_stride: int, page_size: int, block_tables: torch.Tensor,
                          tile_item: torch.Tensor, tile_row0: torch.Tensor, num_tiles: int,
                          item_qstart: torch.Tensor, item_qlen: torch.Tensor,
                          item_pos0: torch.Tensor, item_slots: torch.Tensor, talk: torch.Tensor,
                          partial: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int,
                          dim: int, vdim: int, window: int, keep_first: int, scale: float,
                          error: torch.Tensor) -> torch.Tensor:
    """The mixed-heads attention of `talking_attention` for tiles of 16 consecutive tokens on the
    tensor cores (bfloat16 pages): every (query head, value head) pair as a one-walk attention
    into `partial` (float32, tokens * heads * kv_heads * vdim), then the mixing of the partial
    outputs by `talk` into out."""
    _need(q, torch.float32, "q")
    _need(talk, torch.float32, "talk")
    _need(partial, torch.float32, "partial")
    _need(out, torch.bfloat16, "out")
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0), ("item_slots", item_slots)):
        _need(t, torch.int32, name)
    if k_pages.dtype is not torch.bfloat16 or v_pages.dtype is not torch.bfloat16:
        raise KernelError("talking_attention_mma: the cache must be bfloat16")
    tokens = q.shape[0]
    if partial.numel() < tokens * heads * kv_heads * vdim or talk.numel() != heads * heads:
        raise KernelError("talking_attention_mma: scratch or mixing matrix does not fit")
    _check(hybrid().fsie_talking_attention_mma(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), page_stride, page_size, _ptr(block_tables),
        block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles, _ptr(item_qstart),
        _ptr(item_qlen), _ptr(item_pos0), _ptr(item_slots), _ptr(talk), _ptr(partial), _ptr(out),
        tokens, heads, kv_heads, dim, vdim, window, keep_first, float(scale), _ptr(error),
        _stream()), "talking_attention_mma")
    return out


# --------------------------------------------------- more parts: norms on both sides, minGRU,
# ------------------------------------------------- scaled attention, attention over latent rows
_mixers = None


def mixers():
    """The library of the sandwich norm, the gated activation, the minGRU recurrence, the
    attention with a scale per head and the steps of attention over a latent cache, compiled at
    first use."""
    global _mixers
    if _mixers is None:
        lib = build.load_library("mixers")
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_norm_add_norm.argtypes = [p, p, p, p, p, p, i, i, f, f, i, i, p]
        lib.fsie_gated_act.argtypes = [p, p, ll, i, i, i, p]
        lib.fsie_mingru_scan.argtypes = [p, i, i, p, p, p, i, p, p, i, i, p, p, p, p, i, p]
        lib.fsie_scaled_attention_rows.argtypes = []
        lib.fsie_scaled_attention_tile_rows.argtypes = [i, i, i, i, i]
        lib.fsie_scaled_attention_tile_rows.restype = i
        lib.fsie_scaled_attention.argtypes = [p, i, p, p, p, ll, i, i, i, i, p, i, p, p, i, p, p, p, p,
                                              p, i, p, p, i, i, i, i, i, i, i, i, p, p]
        lib.fsie_norm_rotate_write.argtypes = [p, i, p, p, i, p, p, p, ll, i, i, i, i, i, i, i, p, p, f,
                                               i, p, p]
        lib.fsie_head_gate.argtypes = [p, i, p, i, i, i, i, i, p]
        lib.fsie_scaled_sum_rmsnorm.argtypes = [p, p, f, p, f, p, p, p, i, i, f, i, i, p]
        lib.fsie_rotate_mix_write.argtypes = [p, i, p, p, i, p, p, p, ll, i, i, i, i, i, i, i, i, p, p,
                                              i, p, p]
        lib.fsie_latent_prep.argtypes = [p, i, p, p, i, p, p, ll, i, p, f, p, i, i, i, i, i, i, i, i, p, p]
        lib.fsie_head_product.argtypes = [p, ll, i, p, p, ll, i, i, i, i, i, i, p]
        for name in ("fsie_norm_add_norm", "fsie_gated_act", "fsie_mingru_scan",
                     "fsie_scaled_attention_rows", "fsie_scaled_attention", "fsie_rotate_mix_write",
                     "fsie_latent_prep", "fsie_head_product", "fsie_norm_rotate_write", "fsie_head_gate",
                     "fsie_scaled_sum_rmsnorm"):
            getattr(lib, name).restype = i
        _mixers = lib
    return _mixers


def norm_add_norm(x: torch.Tensor, delta: Optional[torch.Tensor], delta_gain: Optional[torch.Tensor],
                  delta_eps: float, gain: Optional[torch.Tensor], eps: float,
                  out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                  write_x: bool = True) -> Optional[torch.Tensor]:
    """x (float32 residual) += rms(delta) * delta_gain; out = rms(x) * gain in out's dtype, where
    rms(v) = v / sqrt(mean(v^2) + eps).  Without `delta` a plain norm of x, without `out` the
    sum alone.  With `rows` (int32 indices) only those rows, into out[0..len(rows)), and x is
    left untouched unless write_x."""
    _need(x, torch.float32, "x")
    hidden = x.shape[-1]
    dtype = out.dtype if out is not None else delta.dtype
    if delta is not None:
        _need(delta, dtype, "delta")
        _need(delta_gain, torch.float32, "delta_gain")
        if delta.shape[-1] != hidden or delta_gain.numel() != hidden:
            raise KernelError("norm_add_norm: delta or its gain is not as wide as x")
    if out is not None:
        _need(out, None, "out")
        _need(gain, torch.float32, "gain")
        if gain.numel() != hidden:
            raise KernelError("norm_add_norm: gain width differs from x")
    if delta is None and out is None:
        raise KernelError("norm_add_norm: nothing to do")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        count = rows.numel()
    else:
        count = x.numel() // hidden
    if out is not None and out.numel() < count * hidden:
        raise KernelError("norm_add_norm: out is too small")
    _check(mixers().fsie_norm_add_norm(_ptr(x), _ptr(delta), _ptr(delta_gain), _ptr(gain), _ptr(out),
                                       _ptr(rows), count, hidden, float(delta_eps), float(eps),
                                       int(write_x), _tag(dtype), _stream()), "norm_add_norm")
    return out


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, kind: str) -> torch.Tensor:
    """out[t, i] = f(gate_up[t, i]) * gate_up[t, inter + i] with f = SiLU or the tanh form of GELU."""
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    tokens, two_inter = gate_up.shape
    inter = two_inter // 2
    if two_inter != 2 * inter or out.numel() < tokens * inter:
        raise KernelError("gated_act: shapes do not fit")
    _check(mixers().fsie_gated_act(_ptr(gate_up), _ptr(out), tokens, inter, GATE_KINDS[kind],
                                   _tag(out.dtype), _stream()), "gated_act")
    return out


def mingru_scan(proj: torch.Tensor, width: int, item_qstart: torch.Tensor, item_qlen: torch.Tensor,
                item_slots: torch.Tensor, items: int, state: torch.Tensor, out: torch.Tensor,
                seg_item: Optional[torch.Tensor] = None, seg_row0: Optional[torch.Tensor] = None,
                num_segs: int = 0, seg_tokens: int = 0, seg_ab: Optional[torch.Tensor] = None,
                seg_start: Optional[torch.Tensor] = None) -> torch.Tensor:
    """proj [tokens, 3 width] = gate | candidate | output gate (biases added).  Per request and
    channel: z = sigmoid(gate); cand = u + 1/2 (u >= 0) or sigmoid(u); S = (1 - z) S + z cand from
    the state in the request's slot (float32 [slots, width], updated); out[t] = S_t * silu(output
    gate).  With segments (num_segs > 0) a request's tokens run chunk-parallel."""
    _need(proj, None, "proj")
    _need(state, torch.float32, "state")
    _need(out, proj.dtype, "out")
    tokens, ld = proj.shape
    if ld < 3 * width or out.numel() < tokens * width or state.shape[-1] != width:
        raise KernelError("mingru_scan: shapes do not fit")
    if num_segs:
        if seg_ab.numel() < 2 * num_segs * width or seg_start.numel() < num_segs * width:
            raise KernelError("mingru_scan: segment scratch is too small")
    _check(mixers().fsie_mingru_scan(_ptr(proj), ld, width, _ptr(item_qstart), _ptr(item_qlen),
                                     _ptr(item_slots), items, _ptr(seg_item), _ptr(seg_row0), num_segs,
                                     seg_tokens, _ptr(state), _ptr(seg_ab), _ptr(seg_start), _ptr(out),
                                     _tag(proj.dtype), _stream()), "mingru_scan")
    return out


SCALED_ATTENTION_FORMS = {"auto": 0, "plain": 1, "mma": 2, "mma_split": 3}


def scaled_attention_rows(dtype: torch.dtype = torch.float32, key_dim: int = 0, value_dim: int = 0,
                          values_in_keys: bool = False, form: str = "auto") -> int:
    """Query rows of one tile of `scaled_attention` for these sizes and this form of the kernel
    (64 where a warp of the tensor-core kernel owns 16 rows with all their value columns, else 32)."""
    if key_dim <= 0:
        return int(mixers().fsie_scaled_attention_rows())
    return int(mixers().fsie_scaled_attention_tile_rows(_tag(dtype), key_dim, value_dim,
                                                        int(values_in_keys), SCALED_ATTENTION_FORMS[form]))


def scaled_attention(q: torch.Tensor, q_ld: int, head_scale: torch.Tensor, k_pages: torch.Tensor,
                     v_pages: Optional[torch.Tensor], page_stride: int, page_size: int, key_dim: int,
                     value_dim: int, values_in_keys: bool, block_tables: torch.Tensor,
                     tile_item: torch.Tensor, tile_row0: torch.Tensor, tiles: int,
                     item_qstart: torch.Tensor, item_qlen: torch.Tensor, item_pos0: torch.Tensor,
                     item_slots: Optional[torch.Tensor], out: torch.Tensor, tokens: int, heads: int,
                     kv_heads: int, window: int, error: torch.Tensor, nsplit: int = 1,
                     part_o: Optional[torch.Tensor] = None,
                     part_ml: Optional[torch.Tensor] = None, form: str = "auto",
                     chunk: int = 0) -> torch.Tensor:
    """Causal (optionally windowed; `chunk` > 0: only over the keys j with j // chunk == i // chunk)
    softmax attention of q [tokens, heads x key_dim] over paged keys
    [kv_head][slot][key_dim] and values [kv_head][slot][value_dim] (or, values_in_keys, the first
    value_dim columns of the key rows), scores multiplied by head_scale[head]; scores, softmax and
    weights in 32-bit.  `form`: "auto" takes a tensor-core kernel where one fits (bfloat16, key
    sizes in steps of 16, value sizes 64 ... 512), "plain" the 32-bit kernel, "mma" insists on a
    tensor-core kernel, "mma_split" on the one whose warps split the value columns.  The tiles
    hold `scaled_attention_rows(dtype, key_dim, value_dim, values_in_keys, form)` rows."""
    _need(q, None, "q", contiguous=False)
    _need(head_scale, torch.float32, "head_scale")
    _need(out, q.dtype, "out")
    if k_pages.dtype is not q.dtype:
        raise KernelError("scaled_attention: cache dtype differs from q")
    if head_scale.numel() != heads or out.numel() < tokens * heads * value_dim:
        raise KernelError("scaled_attention: shapes do not fit")
    if nsplit > 1:
        if part_o.numel() < nsplit * tokens * heads * value_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("scaled_attention: scratch for the key splits is too small")
    _check(mixers().fsie_scaled_attention(
        _ptr(q), q_ld, _ptr(head_scale), _ptr(k_pages), _ptr(v_pages), page_stride, page_size, key_dim,
        value_dim, int(values_in_keys), _ptr(block_tables), block_tables.stride(0), _ptr(tile_item),
        _ptr(tile_row0), tiles, _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0), _ptr(item_slots),
        _ptr(out), heads * value_dim, _ptr(part_o), _ptr(part_ml), tokens, heads, kv_heads, window,
        int(chunk), nsplit, _tag(q.dtype), SCALED_ATTENTION_FORMS[form], _ptr(error), _stream()),
        "scaled_attention")
    return out


def rotate_mix_write(proj: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                     slot_of: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     page_stride: int, page_size: int, heads: int, kv_heads: int, dim: int, vdim: int,
                     rotary_dim: int, mix_mode: int, mix: Optional[torch.Tensor],
                     v_first: Optional[torch.Tensor], error: torch.Tensor) -> None:
    """proj [tokens, q | k | v]: rotate q in place and k into its page over the first rotary_dim of
    each head (pairs i, i + rotary_dim / 2); values into their page, blended with v_first
    (mix_mode 2: v <- (1 - mix) v + mix v_first) or copied to it first (mix_mode 1)."""
    _need(proj, None, "proj")
    _need(positions, torch.int32, "positions")
    _need(cos_sin, torch.float32, "cos_sin")
    _need(slot_of, torch.int32, "slot_of")
    tokens, ld = proj.shape
    if rotary_dim > 0 and cos_sin.shape[-1] != rotary_dim:
        raise KernelError("rotate_mix_write: cos/sin table width differs from rotary_dim")
    if k_pages.dtype is not proj.dtype or v_pages.dtype is not proj.dtype:
        raise KernelError("rotate_mix_write: cache dtype differs from the projection dtype")
    if mix_mode:
        _need(v_first, proj.dtype, "v_first")
        if v_first.numel() < tokens * kv_heads * vdim:
            raise KernelError("rotate_mix_write: v_first is too small")
    if mix_mode == 2:
        _need(mix, torch.float32, "mix")
    _check(mixers().fsie_rotate_mix_write(_ptr(proj), ld, _ptr(positions), _ptr(cos_sin),
                                          cos_sin.shape[0], _ptr(slot_of), _ptr(k_pages), _ptr(v_pages),
                                          page_stride, page_size, tokens, heads, kv_heads, dim, vdim,
                                          rotary_dim, mix_mode, _ptr(mix), _ptr(v_first),
                                          _tag(proj.dtype), _ptr(error), _stream()), "rotate_mix_write")


def norm_rotate_write(proj: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                      slot_of: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      page_stride: int, page_size: int, heads: int, kv_heads: int, dim: int, vdim: int,
                      rotary_dim: int, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
                      eps: float, error: torch.Tensor) -> None:
    """proj [tokens, q | k | v | ...]: every head of q (of k) divided by its root mean square (eps
    inside the root) times q_gain (k_gain) [dim] in 32-bit where that gain is given; then q rotated in
    place and k into its page over the first rotary_dim of each head (pairs i, i + rotary_dim / 2);
    values into their page."""
    _need(proj, None, "proj")
    _need(positions, torch.int32, "positions")
    _need(cos_sin, torch.float32, "cos_sin")
    _need(slot_of, torch.int32, "slot_of")
    tokens, ld = proj.shape
    if rotary_dim > 0 and cos_sin.shape[-1] != rotary_dim:
        raise KernelError("norm_rotate_write: cos/sin table width differs from rotary_dim")
    if k_pages.dtype is not proj.dtype or v_pages.dtype is not proj.dtype:
        raise KernelError("norm_rotate_write: cache dtype differs from the projection dtype")
    for name, gain in (("q_gain", q_gain), ("k_gain", k_gain)):
        if gain is not None:
            _need(gain, torch.float32, name)
            if gain.numel() != dim:
                raise KernelError(f"norm_rotate_write: {name} must hold one number per column of a head")
    _check(mixers().fsie_norm_rotate_write(_ptr(proj), ld, _ptr(positions), _ptr(cos_sin), cos_sin.shape[0],
                                           _ptr(slot_of), _ptr(k_pages), _ptr(v_pages), page_stride,
                                           page_size, tokens, heads, kv_heads, dim, vdim, rotary_dim,
                                           _ptr(q_gain), _ptr(k_gain), float(eps), _tag(proj.dtype),
                                           _ptr(error), _stream()), "norm_rotate_write")


def head_gate(out: torch.Tensor, gate: torch.Tensor, heads: int, vdim: int) -> torch.Tensor:
    """out[t, h, :] <- out[t, h, :] * sigmoid(gate[t, h]); out [tokens, heads * vdim], `gate`
    [tokens, heads] may be a view of columns of a wider tensor."""
    _need(out, None, "out", contiguous=False)
    _need(gate, out.dtype, "gate", contiguous=False)
    tokens = out.shape[0]
    if out.shape[1] != heads * vdim or gate.shape != (tokens, heads) or out.stride(1) != 1 or gate.stride(1) != 1:
        raise KernelError("head_gate: shapes do not fit")
    _check(mixers().fsie_head_gate(_ptr(out), out.stride(0), _ptr(gate), gate.stride(0), tokens, heads, vdim,
                                   _tag(out.dtype), _stream()), "head_gate")
    return out


def scaled_sum_rmsnorm(x: torch.Tensor, deltas, scales, gain: Optional[torch.Tensor], eps: float,
                       out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                       write_x: bool = True) -> Optional[torch.Tensor]:
    """x (float32 residual) += scales[0] * deltas[0] + scales[1] * deltas[1] (one or two pending
    outputs, in 32-bit); out = rmsnorm(x) * gain in out's dtype (gain float32).  With `rows` only
    those rows are worked on (out row r from x row rows[r]); x is left untouched unless write_x."""
    _need(x, torch.float32, "x")
    hidden = x.shape[-1]
    deltas, scales = tuple(deltas), tuple(float(v) for v in scales)
    if not 1 <= len(deltas) <= 2 or len(scales) != len(deltas):
        raise KernelError("scaled_sum_rmsnorm: one or two pending outputs, a scale for each")
    for d in deltas:
        _need(d, deltas[0].dtype, "delta")
        if d.shape[-1] != hidden or d.numel() != x.numel():
            raise KernelError("scaled_sum_rmsnorm: a pending output is not of x's shape")
    count = x.numel() // hidden
    if rows is not None:
        _need(rows, torch.int32, "rows")
        count = rows.numel()
    if out is not None:
        _need(out, deltas[0].dtype, "out")
        _need(gain, torch.float32, "gain")
        if out.numel() < count * hidden or gain.numel() != hidden:
            raise KernelError("scaled_sum_rmsnorm: out or gain does not fit")
    second = deltas[1] if len(deltas) > 1 else None
    _check(mixers().fsie_scaled_sum_rmsnorm(_ptr(x), _ptr(deltas[0]), scales[0], _ptr(second),
                                            scales[1] if second is not None else 0.0, _ptr(gain), _ptr(out),
                                            _ptr(rows), count, hidden, float(eps), int(write_x),
                                            _tag(deltas[0].dtype), _stream()), "scaled_sum_rmsnorm")
    return out


def latent_prep(proj: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                slot_of: torch.Tensor, pages: torch.Tensor, page_stride: int, page_size: int,
                gain: torch.Tensor, eps: float, qa: torch.Tensor, heads: int, dim: int, rope: int,
                rank: int, rotary_dim: int, error: torch.Tensor, half_pairs: bool = False) -> None:
    """proj [tokens, heads x (dim | rope) | rank | rope]: the RMS-normed latent (gain, eps) and the
    rotated shared key part into the token's cache row [rank | rope]; every head's rotated rope
    part of q into qa [tokens, heads, rank + rope] behind the rank columns.  Rotation of pairs
    (2i, 2i + 1) of the first rotary_dim columns of a rope part, or - `half_pairs` - of pairs
    (i, i + rotary_dim / 2)."""
    _need(proj, None, "proj")
    _need(positions, torch.int32, "positions")
    _need(cos_sin, torch.float32, "cos_sin")
    _need(slot_of, torch.int32, "slot_of")
    _need(gain, torch.float32, "gain")
    _need(qa, proj.dtype, "qa")
    tokens, ld = proj.shape
    if rotary_dim > 0 and cos_sin.shape[-1] != rotary_dim:
        raise KernelError("latent_prep: cos/sin table width differs from rotary_dim")
    if pages.dtype is not proj.dtype or gain.numel() != rank or \
            qa.numel() < tokens * heads * (rank + rope):
        raise KernelError("latent_prep: shapes or dtypes do not fit")
    _check(mixers().fsie_latent_prep(_ptr(proj), ld, _ptr(positions), _ptr(cos_sin), cos_sin.shape[0],
                                     _ptr(slot_of), _ptr(pages), page_stride, page_size, _ptr(gain),
                                     float(eps), _ptr(qa), tokens, heads, dim, rope, rank, rotary_dim,
                                     int(half_pairs), _tag(proj.dtype), _ptr(error), _stream()), "latent_prep")


def head_product(x: torch.Tensor, x_ld: int, x_head: int, weight: torch.Tensor, out: torch.Tensor,
                 out_ld: int, out_head: int, tokens: int) -> torch.Tensor:
    """out[t, h, :] = weight[h] @ x[t, h, :] for weight [heads, n, k]; head h of token t of x at
    t * x_ld + h * x_head, of out at t * out_ld + h * out_head.  32-bit sums."""
    _need(x, None, "x", contiguous=False)
    _need(weight, x.dtype, "weight")
    _need(out, x.dtype, "out", contiguous=False)
    heads, n, k = weight.shape
    _check(mixers().fsie_head_product(_ptr(x), x_ld, x_head, _ptr(weight), _ptr(out), out_ld, out_head,
                                      tokens, heads, n, k, _tag(x.dtype), _stream()), "head_product")
    return out


# ------------------------------------------------- one norm for two sublayers; routed experts
_routed = None


def routed():
    """The library of decoders whose sublayers share one norm and whose feed-forward is a set of
    routed experts (layer norm with gain and bias over a sum of pending outputs, the residual stream
    beside the embedding output, a cap on the logits, a sigmoid gate; router, sorting of the
    (token, expert) pairs, the experts' products, the weighted sum), compiled at first use."""
    global _routed
    if _routed is None:
        lib = build.load_library("routed")
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_sum_layernorm.argtypes = [p, p, p, p, p, p, p, i, i, f, i, i, p]
        lib.fsie_settle_concat.argtypes = [p, p, p, p, p, i, i, i, p]
        lib.fsie_logit_cap.argtypes = [p, ll, f, f, p]
        lib.fsie_sigmoid_gate.argtypes = [p, i, p, i, i, i, i, p]
        lib.fsie_moe_tile_rows.argtypes = []
        lib.fsie_moe_route.argtypes = [p, i, p, p, p, p, p, i, i, i, i, i, i, f, i, i, i, i, p]
        lib.fsie_moe_align.argtypes = [p, i, i, i, i, p, p, p, p, p, p, p]
        lib.fsie_moe_gather.argtypes = [p, ll, p, p, i, i, p, i, i, p]
        lib.fsie_moe_product.argtypes = [p, ll, p, p, ll, p, p, p, p, p, i, i, i, i, i, i, i, i, p]
        lib.fsie_moe_combine.argtypes = [p, p, p, p, p, i, i, i, p, i, p, ll, i, p]
        for name in ("fsie_sum_layernorm", "fsie_settle_concat", "fsie_logit_cap", "fsie_sigmoid_gate",
                     "fsie_moe_tile_rows", "fsie_moe_route", "fsie_moe_align", "fsie_moe_gather", "fsie_moe_product",
                     "fsie_moe_combine"):
            getattr(lib, name).restype = i
        _routed = lib
    return _routed


def sum_layernorm(x: torch.Tensor, deltas, gain: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                  eps: float, out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                  write_x: bool = True) -> Optional[torch.Tensor]:
    """x (float32 residual) += d1 + d2 for the up to two pending sublayer outputs in `deltas`;
    out = (x - mean) / sqrt(mean((x - mean)^2) + eps) * gain + bias in out's dtype.  Without `out`
    the sum alone.  With `rows` (int32 indices) only those rows, into out[0..len(rows)), and x is
    left untouched unless write_x."""
    _need(x, torch.float32, "x")
    width = x.shape[-1]
    deltas = [d for d in (deltas or ()) if d is not None]
    if len(deltas) > 2:
        raise KernelError("sum_layernorm: at most two pending outputs")
    dtype = out.dtype if out is not None else (deltas[0].dtype if deltas else None)
    if dtype is None:
        raise KernelError("sum_layernorm: nothing to do")
    for d in deltas:
        _need(d, dtype, "delta")
        if d.shape[-1] != width or d.numel() != x.numel():
            raise KernelError("sum_layernorm: a pending output is not of x's shape")
    if out is not None:
        _need(out, None, "out")
        _need(gain, torch.float32, "gain")
        if gain.numel() != width or (bias is not None and bias.numel() != width):
            raise KernelError("sum_layernorm: gain or bias width differs from x")
        if bias is not None:
            _need(bias, torch.float32, "bias")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        count = rows.numel()
    else:
        count = x.numel() // width
    if out is not None and out.numel() < count * width:
        raise KernelError("sum_layernorm: out is too small")
    d1 = deltas[0] if deltas else None
    d2 = deltas[1] if len(deltas) > 1 else None
    _check(routed().fsie_sum_layernorm(_ptr(x), _ptr(d1), _ptr(d2), _ptr(gain), _ptr(bias), _ptr(rows),
                                       _ptr(out), count, width, float(eps), int(write_x), _tag(dtype),
                                       _stream()), "sum_layernorm")
    return out


def settle_concat(x: torch.Tensor, deltas, x0: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = [x[t] + d1[t] + d2[t] | x0[t]] in out's dtype ([tokens, 2 width]); x and x0 are
    float32 and stay as they are."""
    _need(x, torch.float32, "x")
    _need(x0, torch.float32, "x0")
    _need(out, None, "out")
    tokens, width = x.shape
    deltas = [d for d in (deltas or ()) if d is not None]
    if len(deltas) > 2 or x0.shape != x.shape or out.numel() < 2 * x.numel():
        raise KernelError("settle_concat: shapes do not fit")
    for d in deltas:
        _need(d, out.dtype, "delta")
        if d.numel() != x.numel():
            raise KernelError("settle_concat: a pending output is not of x's shape")
    d1 = deltas[0] if deltas else None
    d2 = deltas[1] if len(deltas) > 1 else None
    _check(routed().fsie_settle_concat(_ptr(x), _ptr(d1), _ptr(d2), _ptr(x0), _ptr(out), tokens, width,
                                       _tag(out.dtype), _stream()), "settle_concat")
    return out


def logit_cap(logits: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """logits <- cap * tanh(logits * scale / cap) in place (cap = 0: logits * scale)."""
    _need(logits, torch.float32, "logits")
    _check(routed().fsie_logit_cap(_ptr(logits), logits.numel(), float(scale), float(cap), _stream()),
           "logit_cap")
    return logits


def sigmoid_gate(out: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """out[t, c] <- out[t, c] * sigmoid(gate[t, c]); `gate` may be a view of columns of a wider
    tensor."""
    _need(out, None, "out", contiguous=False)
    _need(gate, out.dtype, "gate", contiguous=False)
    tokens, width = out.shape
    if gate.shape != out.shape or out.stride(1) != 1 or gate.stride(1) != 1:
        raise KernelError("sigmoid_gate: shapes do not fit")
    _check(routed().fsie_sigmoid_gate(_ptr(out), out.stride(0), _ptr(gate), gate.stride(0), tokens, width,
                                      _tag(out.dtype), _stream()), "sigmoid_gate")
    return out


def moe_tile_rows() -> int:
    return routed().fsie_moe_tile_rows()


def moe_route(y: Optional[torch.Tensor], w_router: Optional[torch.Tensor], correction: Optional[torch.Tensor],
              ids: torch.Tensor, weights: torch.Tensor, top: int, groups: int, keep: int, scale: float,
              scores: str = "sigmoid", normalise: bool = True, logits: Optional[torch.Tensor] = None,
              group_score: str = "top2") -> None:
    """Per token: s = sigmoid (or softmax) of the router's logits in 32-bit; the `top` experts with the
    largest s + correction among the `keep` best of `groups` groups (a group's score: the sum of its
    two largest s + correction, or - `group_score` "max" - the largest); weights s / (their sum + 1e-20) * scale.  The logits are w_router y, summed here
    (w_router float32 [experts, width]) or - `logits`, float32 [tokens, experts] - by a product
    before this call.  ids int32, weights float32, both [tokens, top]."""
    _need(ids, torch.int32, "ids")
    _need(weights, torch.float32, "weights")
    if correction is not None:
        _need(correction, torch.float32, "correction")
    if scores not in ("sigmoid", "softmax"):
        raise KernelError("moe_route: scores must be 'sigmoid' or 'softmax'")
    if group_score not in ("top2", "max"):
        raise KernelError("moe_route: group_score must be 'top2' or 'max'")
    if logits is not None:
        _need(logits, torch.float32, "logits")
        tokens, experts = logits.shape
        y_ptr, y_ld, width, tag, w_ptr = None, 0, 0, DTYPE_F32, None
    else:
        _need(y, None, "y", contiguous=False)
        _need(w_router, torch.float32, "w_router")
        tokens, width = y.shape
        experts = w_router.shape[0]
        if w_router.shape[1] != width or y.stride(1) != 1:
            raise KernelError("moe_route: shapes do not fit")
        y_ptr, y_ld, tag, w_ptr = _ptr(y), y.stride(0), _tag(y.dtype), _ptr(w_router)
    if ids.numel() < tokens * top or weights.numel() < tokens * top or \
            (correction is not None and correction.numel() != experts):
        raise KernelError("moe_route: shapes do not fit")
    _check(routed().fsie_moe_route(y_ptr, y_ld, w_ptr, _ptr(logits), _ptr(correction), _ptr(ids),
                                   _ptr(weights), tokens, width, experts, int(top), int(groups), int(keep),
                                   float(scale), int(scores == "softmax"), int(normalise),
                                   int(group_score == "max"), tag, _stream()), "moe_route")


def moe_align(ids: torch.Tensor, pairs: int, experts: int, lists: torch.Tensor,
              tile: int = 0, padded: bool = False) -> Tuple[torch.Tensor, ...]:
    """Sort the (token, choice) pairs by expert.  `lists` is int32 working memory of at least
    `moe_lists_size(pairs, experts, tile, padded)` entries; returns its views (offsets [experts + 1],
    sorted, tile_expert, tile_row0, meta [1], place).  Compact layout: sorted [pairs] holds the pairs
    expert after expert, place is None.  `padded`: every expert's rows start on a multiple of `tile`,
    sorted [(pairs // tile + experts) * tile] holds -1 where no pair owns the row, place [pairs] is
    each pair's row."""
    _need(ids, torch.int32, "ids")
    _need(lists, torch.int32, "lists")
    tile = tile or moe_tile_rows()
    tiles = pairs // tile + experts
    if lists.numel() < moe_lists_size(pairs, experts, tile, padded) or ids.numel() < pairs:
        raise KernelError("moe_align: working memory is too small")
    cut = 0
    views = []
    for n in (experts + 1, tiles * tile if padded else pairs, tiles, tiles, 1, pairs if padded else 0):
        views.append(lists[cut:cut + n])
        cut += n
    offsets, order, tile_expert, tile_row0, meta, place = views
    _check(routed().fsie_moe_align(_ptr(ids), pairs, experts, tile, int(padded), _ptr(offsets), _ptr(order),
                                   _ptr(tile_expert), _ptr(tile_row0), _ptr(meta),
                                   _ptr(place) if padded else None, _stream()), "moe_align")
    return offsets, order, tile_expert, tile_row0, meta, (place if padded else None)


def moe_lists_size(pairs: int, experts: int, tile: int = 0, padded: bool = False) -> int:
    tile = tile or moe_tile_rows()
    tiles = pairs // tile + experts
    return experts + 1 + (tiles * tile + pairs if padded else pairs) + 2 * tiles + 1


def moe_gather(x: torch.Tensor, lists, tile: int, top: int, out: torch.Tensor) -> torch.Tensor:
    """out[r] = x[sorted[r] // top] for the rows of the used tiles of a padded layout (zeros where
    no pair owns the row); bfloat16, rows of 16-byte multiples."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, torch.bfloat16, "out")
    _, order, _, _, meta, _ = lists
    rows, k = out.shape
    if x.shape[1] != k or x.stride(1) != 1 or rows > order.numel():
        raise KernelError("moe_gather: shapes do not fit")
    _check(routed().fsie_moe_gather(_ptr(x), x.stride(0), _ptr(order), _ptr(meta), int(tile), int(top),
                                    _ptr(out), rows, k, _stream()), "moe_gather")
    return out


def moe_product(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, lists, pairs: int, top: int,
                gated: bool, activation: str = "silu", first: Optional[bool] = None) -> torch.Tensor:
    """The experts' products over the sorted pairs.  gated: weight [experts, 2 n, k] (gate rows, then up
    rows), x [tokens, k] read at pair // top, out [pairs, n] = f(gate) * up in sorted order.  Not gated:
    weight [experts, n, k], x [pairs, k] in sorted order, out [pairs, n] at each pair's own row - or,
    `first` (an expert without a gate: its first product), x [tokens, k] read at pair // top and
    out [pairs, n] = f(x w^T) in sorted order."""
    mode = 1 if gated else (2 if first else 0)
    _need(x, None, "x", contiguous=False)
    _need(weight, x.dtype, "weight")
    _need(out, x.dtype, "out")
    offsets, order, tile_expert, tile_row0, meta = lists[:5]
    experts, rows, k = weight.shape
    n = rows // 2 if gated else rows
    if x.shape[1] != k or x.stride(1) != 1 or out.shape[1] != n or out.shape[0] < pairs or \
            (gated and rows % 2):
        raise KernelError("moe_product: shapes do not fit")
    _check(routed().fsie_moe_product(_ptr(x), x.stride(0), _ptr(weight), _ptr(out), out.stride(0),
                                     _ptr(offsets), _ptr(order), _ptr(tile_expert), _ptr(tile_row0),
                                     _ptr(meta), pairs, experts, int(top), n, k, mode,
                                     GATE_KINDS[activation], _tag(x.dtype), _stream()), "moe_product")
    return out


def moe_combine(expert_out: torch.Tensor, weights: torch.Tensor, shared: Optional[torch.Tensor],
                out: torch.Tensor, top: int, place: Optional[torch.Tensor] = None,
                ids: Optional[torch.Tensor] = None, experts: int = 0,
                y: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * expert_out[t * top + j] (+ shared[t]), summed in 32-bit; with
    `place` (int32 [tokens * top]) pair p's row of expert_out is place[p].  With `ids` (int32
    [tokens, top]), `experts` and `y` [tokens, width]: a choice at or beyond `experts` names an
    identity expert, whose output is the token's row of y."""
    _need(expert_out, None, "expert_out")
    _need(weights, torch.float32, "weights")
    _need(out, expert_out.dtype, "out")
    tokens, width = out.shape
    if shared is not None:
        _need(shared, expert_out.dtype, "shared")
        if shared.shape != out.shape:
            raise KernelError("moe_combine: the shared expert's output is not of out's shape")
    if expert_out.numel() < tokens * top * width or weights.numel() < tokens * top:
        raise KernelError("moe_combine: shapes do not fit")
    if place is not None:
        _need(place, torch.int32, "place")
    y_ld = 0
    if ids is not None:
        _need(ids, torch.int32, "ids")
        _need(y, out.dtype, "y", contiguous=False)
        if ids.numel() < tokens * top or y.shape != out.shape or y.stride(1) != 1:
            raise KernelError("moe_combine: ids or y does not fit")
        y_ld = y.stride(0)
    _check(routed().fsie_moe_combine(_ptr(expert_out), _ptr(weights), _ptr(shared), _ptr(place), _ptr(out),
                                     tokens, width, int(top), _ptr(ids), int(experts), _ptr(y), y_ld,
                                     _tag(out.dtype), _stream()), "moe_combine")
    return out
