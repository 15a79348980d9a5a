"""Tensor-level wrappers of the kernel library.

Each function checks devices, dtypes, shapes and contiguity on the host, then launches
on the current CUDA stream.  torch is used for allocation and streams only; every
operation here runs a kernel of this library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as _lib
from .lib import KernelError, check

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not supported by the kernels (float32 or bfloat16)")


def _stream() -> int:
    """The current stream's handle (of the current device): the raw query, a hundred times cheaper than building a
    torch.cuda.Stream object for every launch."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need(t: torch.Tensor, what: str, dtype: Optional[torch.dtype] = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: expected a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t,:] = table[ids[t],:] * scale as fp32; ids outside the table give zero rows."""
    _need(ids, "embedding ids", torch.int32)
    _need(table, "embedding table")
    _need(out, "embedding out", torch.float32)
    n, (v, d) = ids.numel(), table.shape
    if out.shape != (n, d):
        raise KernelError(f"embedding: out is {tuple(out.shape)}, expected {(n, d)}")
    check(_lib.load().mm_embedding(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), out.data_ptr(), n, v, d,
                                   float(scale), _stream()), "embedding")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual (fp32) += delta, out = rmsnorm(residual) * weight.  With ``rows`` output row i comes
    from source row rows[i] and the residual is left untouched."""
    _need(residual, "rmsnorm residual", torch.float32)
    _need(weight, "rmsnorm weight")
    _need(out, "rmsnorm out")
    d = residual.shape[-1]
    n_out = out.shape[0]
    if weight.shape != (d,) or out.shape[-1] != d:
        raise KernelError("rmsnorm: width mismatch")
    if delta is not None:
        _need(delta, "rmsnorm delta", out.dtype)
        if delta.shape != residual.shape:
            raise KernelError("rmsnorm: delta and residual differ in shape")
    if rows is not None:
        _need(rows, "rmsnorm rows", torch.int32)
        if rows.numel() != n_out:
            raise KernelError("rmsnorm: rows and out differ in length")
    elif n_out != residual.shape[0]:
        raise KernelError("rmsnorm: out and residual differ in rows")
    check(_lib.load().mm_add_rmsnorm(residual.data_ptr(), _ptr(delta), _ptr(rows), weight.data_ptr(),
                                     dtype_code(weight.dtype), out.data_ptr(), dtype_code(out.dtype), n_out, d,
                                     float(eps), _stream()), "rmsnorm")
    return out


def add_residual(residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _need(residual, "add_residual residual", torch.float32)
    _need(delta, "add_residual delta")
    if delta.shape != residual.shape:
        raise KernelError("add_residual: shapes differ")
    check(_lib.load().mm_add_residual(residual.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype), residual.numel(),
                                      _stream()), "add_residual")
    return residual


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """out[n,f] = silu(gate) * up.  interleave 0: gate_up[n,f] and gate_up[n,F+f]; interleave 8: gate and
    up alternate in blocks of 8 columns."""
    _need(gate_up, "silu_mul input")
    _need(out, "silu_mul out", gate_up.dtype)
    n, two_f = gate_up.shape
    if two_f % 2 or out.shape != (n, two_f // 2):
        raise KernelError("silu_mul: shapes do not match [n,2F] -> [n,F]")
    check(_lib.load().mm_silu_mul(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), n, two_f // 2, interleave,
                                  _stream()), "silu_mul")
    return out


def qkv_rope_kvwrite(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                     k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], positions: torch.Tensor,
                     token_req: torch.Tensor, block_table: torch.Tensor, page_size: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, rotary_dim: int, theta: float, interleave: bool = False) -> None:
    """Adds the bias, rotates q and k by position, writes q to ``q_out`` and k, v into their pages.
    ``interleave``: the q and k columns of ``qkv`` and ``bias`` are in the order of :func:`interleave_halves`."""
    _need(qkv, "qkv")
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape != (n, width):
        raise KernelError(f"qkv: shape {tuple(qkv.shape)} is not [n, {width}]")
    _need(q_out, "q_out", qkv.dtype)
    if q_out.shape != (n, num_heads * head_dim):
        raise KernelError("q_out: wrong shape")
    if bias is not None:
        _need(bias, "qkv bias")
        if bias.shape != (width,):
            raise KernelError("qkv bias: wrong shape")
    if k_pages is not None:
        for name, pool in (("k_pages", k_pages), ("v_pages", v_pages)):
            _need(pool, name, qkv.dtype)
            if pool.dim() != 4 or pool.shape[1:] != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name}: shape {tuple(pool.shape)} is not [pages, {num_kv_heads}, {page_size}, {head_dim}]")
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if block_table.dim() != 2:
        raise KernelError("block_table: expected [requests, width]")
    check(_lib.load().mm_qkv_rope_kvwrite(
        qkv.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
        _ptr(k_pages), _ptr(v_pages), dtype_code(qkv.dtype), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, n, num_heads, num_kv_heads, head_dim, rotary_dim,
        float(theta), int(interleave), _stream()), "qkv_rope_kvwrite")


def qkv_rope_tables(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                    k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], table: torch.Tensor,
                    slots: Optional[torch.Tensor], page_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                    interleave: bool = False) -> None:
    """:func:`qkv_rope_kvwrite` for bfloat16 and a rotation of the whole head, with the step's tables: ``table``
    from :func:`rope_table`, ``slots`` from :func:`slot_mapping` (needed when there are pages to write)."""
    _need(qkv, "qkv", torch.bfloat16)
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape != (n, width):
        raise KernelError(f"qkv: shape {tuple(qkv.shape)} is not [n, {width}]")
    if head_dim % 16:
        raise KernelError(f"qkv_rope_tables: head size {head_dim} is not a multiple of 16")
    _need(q_out, "q_out", torch.bfloat16)
    if q_out.shape != (n, num_heads * head_dim):
        raise KernelError("q_out: wrong shape")
    if bias is not None:
        _need(bias, "qkv bias")
        if bias.shape != (width,):
            raise KernelError("qkv bias: wrong shape")
    _need(table, "rope table", torch.float32)
    if table.shape != (n, head_dim):
        raise KernelError(f"rope table: shape {tuple(table.shape)} is not [{n}, {head_dim}]")
    if k_pages is not None:
        for name, pool in (("k_pages", k_pages), ("v_pages", v_pages)):
            _need(pool, name, torch.bfloat16)
            if pool.dim() != 4 or pool.shape[1:] != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name}: shape {tuple(pool.shape)} is not [pages, {num_kv_heads}, {page_size}, {head_dim}]")
        if slots is None:
            raise KernelError("qkv_rope_tables: pages without slots")
        _need(slots, "slots", torch.int32)
        if slots.shape != (n,):
            raise KernelError("slots: wrong shape")
    check(_lib.load().mm_qkv_rope_tables(
        qkv.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
        _ptr(k_pages), _ptr(v_pages), table.data_ptr(), _ptr(slots), page_size, n, num_heads, num_kv_heads, head_dim,
        int(interleave), _stream()), "qkv_rope_tables")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(src, "gather src")
    _need(rows, "gather rows", torch.int32)
    _need(out, "gather out", src.dtype)
    check(_lib.load().mm_gather_rows(src.data_ptr(), rows.data_ptr(), out.data_ptr(), dtype_code(src.dtype),
                                     rows.numel(), src.shape[-1], _stream()), "gather_rows")
    return out


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                      positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor, page_size: int,
                      num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float) -> torch.Tensor:
    """Causal attention of every token over its request's pages (fp32 arithmetic, any head size)."""
    _need(q, "attention q")
    n = q.shape[0]
    _need(out, "attention out", q.dtype)
    _need(k_pages, "attention k_pages", q.dtype)
    _need(v_pages, "attention v_pages", q.dtype)
    if q.shape != (n, num_heads * head_dim) or out.shape != q.shape:
        raise KernelError("attention: q/out shape mismatch")
    if k_pages.shape[1:] != (num_kv_heads, page_size, head_dim) or v_pages.shape != k_pages.shape:
        raise KernelError("attention: page pool shape mismatch")
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    check(_lib.load().mm_attention_generic(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), dtype_code(q.dtype), positions.data_ptr(),
        token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, n, num_heads, num_kv_heads,
        head_dim, window, float(scale), _stream()), "attention_generic")
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) on the fp32 FMA units, k summed in ascending order."""
    _need(a, "gemm a")
    _need(w, "gemm w")
    _need(out, "gemm out")
    m, k = a.shape
    n = w.shape[0]
    if w.shape != (n, k) or out.shape != (m, n):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not match")
    if bias is not None:
        _need(bias, "gemm bias")
        if bias.shape != (n,):
            raise KernelError("gemm: bias shape mismatch")
    check(_lib.load().mm_gemm_simt(a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype), _ptr(bias),
                                   dtype_code(bias.dtype) if bias is not None else F32, out.data_ptr(),
                                   dtype_code(out.dtype), m, n, k, k, n, _stream()), "gemm_simt")
    return out


GEMV_MAX_ROWS = 8      # measured on B200 (7B shapes, 8 layers, whole decode step): from 9 rows on the tcgen05 product is ahead of the register-streaming kernel's two-tile variant (9 rows 1.15 vs 1.25 ms, 12 rows 1.20 vs 1.30 ms)


# Above the streaming kernel's rows and up to here the tcgen05 weight-streaming product (with the fused epilogues) is
# used.  Measured per layer on B200 (7B shapes, sum of the four products against library products + separate norm,
# rotary and activation kernels): 16 rows 94.6 vs 106.9 us, 64 rows 100.6 vs 109.8 us, 128 rows 119 vs 114 us.
SKINNY_MAX_ROWS = 64


def gemv_supported(m: int, n: int, k: int) -> bool:
    return 1 <= m <= GEMV_MAX_ROWS and n % 16 == 0 and k % 32 == 0 and k >= 256


def skinny_supported(m: int, n: int, k: int) -> bool:
    return GEMV_MAX_ROWS < m <= SKINNY_MAX_ROWS and n % 16 == 0 and k % 8 == 0 and k >= 64


def small_batch_supported(m: int, n: int, k: int) -> bool:
    """True if the products of a few rows (and their fused epilogues) take these sizes: the register-streaming
    kernel up to GEMV_MAX_ROWS rows, the tcgen05 one up to SKINNY_MAX_ROWS."""
    return gemv_supported(m, n, k) or skinny_supported(m, n, k)


def _skinny_pad(m: int) -> int:
    return 16 if m <= 16 else (32 if m <= 32 else (64 if m <= 64 else 128))


def _skinny_splits(n: int, k: int) -> int:
    """K splits (= cluster size) of the tcgen05 product: enough CTAs to fill the GPU when the weight has few
    128-row tiles, but no more clusters than are resident at once (256 CTAs in clusters of 8 on 148 SMs), at least
    6 blocks of 64 along K per CTA, and a power of two (other cluster sizes place badly)."""
    tiles, k_blocks = -(-n // 128), -(-k // 64)
    s = 1
    while s < 8 and tiles * s * 2 <= 256 and k_blocks // (s * 2) >= 6:
        s *= 2
    return s


@dataclass
class RowScale:
    """The deferred 1/rms of rows that were written as ``residual * norm_weight``: per 16-column tile of the
    producer, the partial sums of squares of each row ([tiles, 16] fp32).  A consuming matrix product multiplies
    row m of its result by ``1 / sqrt(sum_j ss[j, m] / dim + eps)``."""

    ss: torch.Tensor
    dim: int
    eps: float


def _gemv_layout(n: int, k: int):
    # 8 warps per CTA as row tiles x K splits: as many row tiles per CTA (8, 4, 2, 1) as still leave one and a half
    # CTAs per SM (measured: 1,728 tiles of 5,120 at 8 rows: 4 tiles per CTA 45.9 us, 2: 47.5, 8: 50.8, 1: 51.7;
    # 2,368 tiles of 3,584: 8: 44.6, 2: 49.4; 608 of 896: 2: 6.4, 1: 8.3; 320 tiles and fewer: 1).  The same rule as
    # the library's executor (csrc/exec/core.cu): the order of a sum depends on the split.
    tiles = n // 16
    rt = 8
    while rt > 1 and -(-tiles // rt) < 222:
        rt //= 2
    ks = 8 // rt
    while ks > k // 32:
        ks //= 2
        rt *= 2
    return rt, ks


def _scale_args(scale: Optional["RowScale"], m: int):
    """(pointer, tiles, dim, eps) for the register-streaming kernel: partial sums [tiles, 16]."""
    if scale is None:
        return None, 0, 0, 0.0
    _need(scale.ss, "row scale", torch.float32)
    if scale.ss.dim() != 2 or scale.ss.shape[1] != 16 or m > 16:
        raise KernelError("row scale: expected [tiles, 16] partial sums")
    return scale.ss.data_ptr(), scale.ss.shape[0], int(scale.dim), float(scale.eps)


def _skinny_scale_args(scale: Optional["RowScale"], m: int):
    """(pointer, tiles, dim, row stride, eps) for the tcgen05 product: partial sums [tiles, stride >= m]."""
    if scale is None:
        return None, 0, 0, 0, 0.0
    _need(scale.ss, "row scale", torch.float32)
    if scale.ss.dim() != 2 or scale.ss.shape[1] < m:
        raise KernelError("row scale: expected [tiles, >= rows] partial sums")
    return scale.ss.data_ptr(), scale.ss.shape[0], int(scale.dim), scale.ss.shape[1], float(scale.eps)


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
              swiglu: bool = False, scale: Optional[RowScale] = None) -> torch.Tensor:
    """x[M<=16, K] @ w[N, K]^T (+ bias) with the weight-streaming kernel.  ``swiglu``: w interleaves gate and
    up rows in blocks of 8 and the result is silu(gate) * up, [M, N/2].  ``scale``: rows of the product are
    multiplied by the deferred 1/rms before bias and activation."""
    _need(x, "gemv x", torch.bfloat16)
    _need(w, "gemv w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or not small_batch_supported(m, n, k):
        raise KernelError(f"gemv: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    if bias is not None:
        _need(bias, "gemv bias")
    out = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=x.device)
    if m > GEMV_MAX_ROWS:
        if out.shape[1] % 8:
            raise KernelError("gemv: the tcgen05 product needs output rows of a multiple of 8 columns")
        check(_lib.load().mm_gemm_skinny(w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                         out.data_ptr(), dtype_code(out_dtype), m, n, k, k, out.shape[1], _skinny_splits(n, k),
                                         int(swiglu), *_skinny_scale_args(scale, m), tcgen05_error_flag(x.device).data_ptr(),
                                         _stream()), "gemm_skinny")
        return out
    rt, ks = _gemv_layout(n, k)
    check(_lib.load().mm_gemv_bf16(w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                   out.data_ptr(), dtype_code(out_dtype), m, n, k, k, out.shape[1], rt, ks, int(swiglu),
                                   *_scale_args(scale, m), _stream()), "gemv_bf16")
    return out


def gemv_bf16_residual(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_weight: Optional[torch.Tensor],
                       eps: float = 0.0, scale: Optional[RowScale] = None):
    """residual[M, N] (fp32, in place) += x @ w^T.  With ``norm_weight`` returns (xw, RowScale): the rows of
    ``residual * norm_weight`` in bfloat16 and the partial sums for their 1/rms; else returns None."""
    _need(x, "gemv x", torch.bfloat16)
    _need(w, "gemv w", torch.bfloat16)
    _need(residual, "gemv residual", torch.float32)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or residual.shape != (m, n) or not small_batch_supported(m, n, k):
        raise KernelError(f"gemv residual: shapes x{tuple(x.shape)} w{tuple(w.shape)} residual{tuple(residual.shape)} are not supported")
    skinny = m > GEMV_MAX_ROWS
    xw = ss = None
    if norm_weight is not None:
        _need(norm_weight, "norm weight")
        if norm_weight.shape != (n,):
            raise KernelError("gemv residual: norm weight has the wrong length")
        xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        ss = torch.empty((n // 16, _skinny_pad(m) if skinny else 16), dtype=torch.float32, device=x.device)
    if skinny:
        check(_lib.load().mm_gemm_skinny_residual(
            w.data_ptr(), x.data_ptr(), residual.data_ptr(), _ptr(norm_weight),
            dtype_code(norm_weight.dtype) if norm_weight is not None else F32, _ptr(xw), _ptr(ss), ss.shape[1] if ss is not None else 0,
            m, n, k, k, _skinny_splits(n, k), *_skinny_scale_args(scale, m), tcgen05_error_flag(x.device).data_ptr(), _stream()),
            "gemm_skinny_residual")
        return None if norm_weight is None else (xw, RowScale(ss, n, float(eps)))
    rt, ks = _gemv_layout(n, k)
    check(_lib.load().mm_gemv_bf16_residual(w.data_ptr(), x.data_ptr(), residual.data_ptr(), _ptr(norm_weight),
                                            dtype_code(norm_weight.dtype) if norm_weight is not None else F32, _ptr(xw), _ptr(ss),
                                            m, n, k, k, rt, ks, *_scale_args(scale, m), _stream()), "gemv_bf16_residual")
    return None if norm_weight is None else (xw, RowScale(ss, n, float(eps)))


def interleave_halves(t: torch.Tensor, num_rot_heads: int, head_dim: int) -> torch.Tensor:
    """Row order the fused q/k/v product wants: within each of the first ``num_rot_heads`` heads (q and k), rows
    16b..16b+7 are elements 8b.. of the head's first half and rows 16b+8..16b+15 the same elements of the second
    half, so the thread that holds an element holds its rotation partner.  Other rows (v) keep their place."""
    hd, half = head_dim, head_dim // 2
    if hd % 16:
        raise KernelError("interleave_halves: the head size must be a multiple of 16")
    rot = num_rot_heads * hd
    head = t[:rot].reshape(num_rot_heads, 2, half // 8, 8, *t.shape[1:])     # [head, half, block, 8, ...]
    head = head.transpose(1, 2).reshape(rot, *t.shape[1:])                   # [head, block, half, 8, ...]
    return torch.cat([head, t[rot:]], dim=0).contiguous()


def rope_table(positions: torch.Tensor, dim: int, theta: float) -> torch.Tensor:
    """[n, dim] fp32: cos of the dim/2 rotation angles of every token's position, then their sin."""
    _need(positions, "positions", torch.int32)
    out = torch.empty((positions.numel(), dim), dtype=torch.float32, device=positions.device)
    check(_lib.load().mm_rope_table(positions.data_ptr(), out.data_ptr(), positions.numel(), dim, float(theta), _stream()), "rope_table")
    return out


def slot_mapping(positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor, page_size: int) -> torch.Tensor:
    """[n] int32: where each token's key and value go in a page pool (page * page_size + place in the page), -1: nowhere."""
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if block_table.dim() != 2:
        raise KernelError("block_table: expected [requests, width]")
    out = torch.empty(positions.numel(), dtype=torch.int32, device=positions.device)
    check(_lib.load().mm_slot_mapping(positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                      page_size, positions.numel(), out.data_ptr(), _stream()), "slot_mapping")
    return out


def gemv_bf16_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                       k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], table: torch.Tensor,
                       slots: Optional[torch.Tensor], page_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                       scale: Optional[RowScale] = None) -> None:
    """The q/k/v projection of up to 16 tokens with bias, rotary encoding and cache write in its epilogue.
    ``w`` and ``bias`` are in the order of :func:`interleave_halves`; q_out, k and v are in natural order.
    ``table``: :func:`rope_table` of the tokens for this head size; ``slots``: :func:`slot_mapping`."""
    _need(x, "gemv x", torch.bfloat16)
    _need(w, "gemv w", torch.bfloat16)
    m, k = x.shape
    n = (num_heads + 2 * num_kv_heads) * head_dim
    if w.shape != (n, k) or not small_batch_supported(m, n, k) or head_dim % 16:
        raise KernelError(f"gemv qkv: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    _need(q_out, "q_out", torch.bfloat16)
    if q_out.shape != (m, num_heads * head_dim):
        raise KernelError("q_out: wrong shape")
    if bias is not None:
        _need(bias, "qkv bias")
        if bias.shape != (n,):
            raise KernelError("qkv bias: wrong shape")
    _need(table, "rope table", torch.float32)
    if table.shape != (m, head_dim):
        raise KernelError("rope table: expected [tokens, head_dim]")
    if k_pages is not None:
        for name, pool in (("k_pages", k_pages), ("v_pages", v_pages)):
            _need(pool, name, torch.bfloat16)
            if pool.dim() != 4 or pool.shape[1:] != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name}: shape {tuple(pool.shape)} is not [pages, {num_kv_heads}, {page_size}, {head_dim}]")
        _need(slots, "slots", torch.int32)
        if slots.numel() != m:
            raise KernelError("slots: one per token")
    if m > GEMV_MAX_ROWS:
        check(_lib.load().mm_gemm_skinny_qkv_rope(
            w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
            _ptr(k_pages), _ptr(v_pages), table.data_ptr(), _ptr(slots) if k_pages is not None else None, page_size,
            num_heads, num_kv_heads, head_dim, m, k, k, _skinny_splits(n, k), *_skinny_scale_args(scale, m),
            tcgen05_error_flag(x.device).data_ptr(), _stream()), "gemm_skinny_qkv_rope")
        return
    rt, ks = _gemv_layout(n, k)
    check(_lib.load().mm_gemv_bf16_qkv_rope(
        w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
        _ptr(k_pages), _ptr(v_pages), table.data_ptr(), _ptr(slots) if k_pages is not None else None, page_size,
        num_heads, num_kv_heads, head_dim, m, k, k, rt, ks, *_scale_args(scale, m), _stream()), "gemv_bf16_qkv_rope")


_TC_ERR = {}
EPI_BF16, EPI_SWIGLU, EPI_F32 = 0, 1, 2
# Measured on B200 (7B shapes, gate/up product): from 256 rows on the fused product is level with or ahead of the
# library product + activation kernel (65 against 80 us at 256 rows, 197 against 217 at 1,024, 346 against 409 at 2,048);
# below, a 128-row tile leaves the tensor cores short of work and the library's smaller tiles win (58 against 71 us at 96).
TCGEN05_SWIGLU_MIN_ROWS = 256


def tcgen05_error_flag(device) -> torch.Tensor:
    """Device int that the tcgen05 kernels set to 1 when one of their bounded waits ran out."""
    key = str(device)
    if key not in _TC_ERR:
        _TC_ERR[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_ERR[key]


def check_tcgen05_errors(device) -> None:
    """Raises if a tcgen05 kernel gave up a wait since the last check (synchronises)."""
    flag = _TC_ERR.get(str(device))
    if flag is not None and int(flag.item()) != 0:
        flag.zero_()
        raise KernelError("a tcgen05 kernel gave up waiting on its pipeline; its output is not valid")


def gemm_tcgen05_supported(m: int, n: int, k: int) -> bool:
    return m >= 1 and k % 8 == 0 and n % 8 == 0 and k >= 64


# From this many rows on, the product runs on pairs of CTAs (cta_group::2, 256 x 256 tiles), unless the last pair's
# second CTA would have nothing but padding (384 rows cost as much as 512 there: 126 against 91 us).
TCGEN05_PAIR_MIN_ROWS = 256


def tcgen05_pair_suits(m: int) -> bool:
    return m >= TCGEN05_PAIR_MIN_ROWS and (m - 1) % 256 >= 128


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                 swiglu: bool = False, pair: Optional[bool] = None) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T (+ bias) on the tcgen05 tensor cores (TMA operands, TMEM accumulators).
    ``swiglu``: w interleaves gate and up rows in blocks of 8; returns silu(gate) * up, [M, N/2].
    ``pair``: the kernel of CTA pairs or the single-CTA one; None chooses by the number of rows."""
    _need(x, "gemm x", torch.bfloat16)
    _need(w, "gemm w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or not gemm_tcgen05_supported(m, n, k):
        raise KernelError(f"gemm_tcgen05: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    if swiglu:
        if n % 16 or bias is not None or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tcgen05: the SwiGLU epilogue needs N a multiple of 16, no bias, bf16 output")
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
        epi = EPI_SWIGLU
    else:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        epi = EPI_F32 if out_dtype == torch.float32 else EPI_BF16
    if bias is not None:
        _need(bias, "gemm bias")
    if pair is None:
        pair = tcgen05_pair_suits(m)
    fn = _lib.load().mm_gemm_tcgen05_pair if pair else _lib.load().mm_gemm_tcgen05
    check(fn(x.data_ptr(), w.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
             out.data_ptr(), epi, m, n, k, k, out.shape[1], tcgen05_error_flag(x.device).data_ptr(), _stream()), "gemm_tcgen05")
    return out


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "argmax logits", torch.float32)
    r, v = logits.shape
    if out is None:
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
    _need(out, "argmax out", torch.int32)
    if v > 16384:
        # wide rows: several blocks per row, then one to reduce them
        p = min(256, -(-v // 4096))
        part_val = torch.empty((r, p), dtype=torch.float32, device=logits.device)
        part_idx = torch.empty((r, p), dtype=torch.int32, device=logits.device)
        check(_lib.load().mm_argmax_rows_split(logits.data_ptr(), out.data_ptr(), part_val.data_ptr(), part_idx.data_ptr(),
                                               r, v, p, _stream()), "argmax_rows_split")
        return out
    check(_lib.load().mm_argmax_rows(logits.data_ptr(), out.data_ptr(), r, v, _stream()), "argmax_rows")
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                seeds: torch.Tensor, counters: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "sample logits", torch.float32)
    r, v = logits.shape
    _need(temperature, "temperature", torch.float32)
    _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32)
    _need(seeds, "seeds", torch.int64)
    _need(counters, "counters", torch.int64)
    for t in (temperature, top_k, top_p, seeds, counters):
        if t.numel() != r:
            raise KernelError("sample: per-row parameter length mismatch")
    if out is None:
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
    check(_lib.load().mm_sample_rows(logits.data_ptr(), out.data_ptr(), r, v, temperature.data_ptr(), top_k.data_ptr(),
                                     top_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(), _stream()), "sample_rows")
    return out


def apply_penalties(logits: torch.Tensor, recent: Optional[torch.Tensor], repetition: torch.Tensor,
                    frequency: torch.Tensor, presence: torch.Tensor, softcap: Optional[torch.Tensor]) -> torch.Tensor:
    _need(logits, "penalties logits", torch.float32)
    r, v = logits.shape
    w = 0
    if recent is not None:
        _need(recent, "recent tokens", torch.int32)
        w = recent.shape[1]
    for t in (repetition, frequency, presence):
        _need(t, "penalty parameter", torch.float32)
    if softcap is not None:
        _need(softcap, "softcap", torch.float32)
    check(_lib.load().mm_apply_penalties(logits.data_ptr(), r, v, _ptr(recent), w, repetition.data_ptr(),
                                         frequency.data_ptr(), presence.data_ptr(), _ptr(softcap), _stream()),
          "apply_penalties")
    return logits


def window_push(recent: torch.Tensor, widths: torch.Tensor, lengths: torch.Tensor, tokens: torch.Tensor) -> None:
    """recent int32 [R, W]: per row a ring of its last widths[r] tokens; writes tokens[r] at lengths[r] % widths[r]
    and adds one to lengths[r] (int64)."""
    _need(recent, "recent tokens", torch.int32)
    _need(widths, "window widths", torch.int32)
    _need(lengths, "sequence lengths", torch.int64)
    _need(tokens, "tokens", torch.int32)
    r, w = recent.shape
    if widths.numel() != r or lengths.numel() != r or tokens.numel() != r:
        raise KernelError("window_push: one width, length and token per row")
    check(_lib.load().mm_window_push(recent.data_ptr(), r, w, widths.data_ptr(), lengths.data_ptr(), tokens.data_ptr(), _stream()),
          "window_push")


def uniform_from(seed: int, counter: int) -> float:
    """The uniform number in [0,1) the device sampler draws for (seed, counter)."""
    return float(_lib.load().mm_uniform_from(seed & 0xFFFFFFFFFFFFFFFF, counter & 0xFFFFFFFFFFFFFFFF))
