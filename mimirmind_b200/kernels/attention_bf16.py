"""Launch plans for the tensor-core attention kernels (bfloat16, head size 64 or 128).

Per step the batch is sorted once, on the host, into *prefill tiles* (64 query tokens of one
request) for portions of at least ``PREFILL_MIN`` tokens and *decode items* (single tokens)
for the rest; every layer of the step reuses the plan.  The decode kernel cuts each token's
key range into splits by absolute position; the split length is chosen so that the grid
fills the GPU, and its partial results go through scratch memory that the plan owns.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as _lib
from .lib import check

PREFILL_MIN = 16       # shorter portions go token by token through the decode kernel
TILE_ROWS = 64         # query rows per CTA of the mma.sync prefill kernel
TILE_ROWS_TC = 128     # ... of the tcgen05 prefill kernel
USE_TCGEN05_PREFILL = True
USE_TMA_DECODE = True   # decode attention with a TMA producer warp (page sizes 8..64)
TMA_DECODE_STAGES = 3
TARGET_CTAS = 2 * 148  # decode CTAs wanted (measured: 2 per SM beat 1 and 4 at batch 8; batch 64 is best unsplit)
USE_CLUSTER_MERGE = True   # up to 8 splits per token: one thread-block cluster merges them through shared memory
CLUSTER_MAX_WANTED = 12    # ... preferred over more splits and a merge launch when up to this many were wanted
FIXED_SPLIT = None     # tests set a split length in keys to cut by absolute position instead

_declared = False


def _declare():
    global _declared
    if _declared:
        return
    P, I, F = c_void_p, c_int, c_float
    _lib.declare("mm_attention_prefill_bf16", [P, P, P, P, P, I, P, I, I, I, I, I, I, F, P])
    _lib.declare("mm_attention_prefill_tcgen05", [P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, F, P, P])
    _lib.declare("mm_attention_decode_tma_bf16", [P, P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, I, I, P, P])
    _lib.declare("mm_attention_decode_tma_max_clusters", [I, I, P])
    _lib.declare("mm_attention_decode_merge_bf16", [P, P, P, P, I, P, I, I, I, I, I, P])
    _lib.declare("mm_attention_decode_bf16", [P, P, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P])
    _declared = True


def supports(head_dim: int, num_heads: int, num_kv_heads: int) -> bool:
    return head_dim in (64, 128) and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16


@dataclass
class AttentionPlan:
    tiles: Optional[torch.Tensor]      # int32 [n_tiles, 4] or None
    n_tiles: int
    tile_rows: int                     # 64: mma.sync kernel, 128: tcgen05 kernel
    items: Optional[torch.Tensor]      # int32 [n_items]; None with n_items > 0 means "every token"
    n_items: int
    split_len: int
    max_splits: int
    part_o: Optional[torch.Tensor] = None
    part_ml: Optional[torch.Tensor] = None
    cluster: bool = False              # the splits of a token are one thread-block cluster that merges them itself


_cluster_capacity = {}


def cluster_capacity(head_dim: int, size: int) -> int:
    """Clusters of ``size`` decode CTAs that are resident on the current device at once (asked of the runtime)."""
    key = (torch.cuda.current_device(), head_dim, size)
    if key not in _cluster_capacity:
        _declare()
        n = c_int(0)
        check(_lib.load().mm_attention_decode_tma_max_clusters(head_dim, size, ctypes.byref(n)), "attention_decode_tma_max_clusters")
        _cluster_capacity[key] = n.value
    return _cluster_capacity[key]


def choose_split(n_items: int, num_kv_heads: int, max_kv_len: int, head_dim: int = 0, page_size: int = 0):
    """(split_len, max_splits, cluster) for the decode kernel.  split_len 0: every token's key range is cut evenly
    into at most max_splits pieces of whole 64-key tiles, so the grid is full whatever the lengths.  cluster: the
    splits of a token are one thread-block cluster and merge themselves."""
    if FIXED_SPLIT:
        return FIXED_SPLIT, max(1, -(-max_kv_len // FIXED_SPLIT)), False
    ctas = max(1, n_items * num_kv_heads)
    if ctas >= TARGET_CTAS // 2:
        return 0, 1, False       # one CTA per SM or more already: a split would only add the merge pass
    # never more CTAs than are resident at once (two per SM): a second, nearly empty wave costs a whole pass
    wanted = max(1, min(TARGET_CTAS // ctas, -(-max_kv_len // 64)))
    # Clusters of 2, 4 or 8 place well on the GPU (measured: 3 and 6 do not), and only as many as are resident at
    # once.  Worth a few splits less (12 -> 8 measured faster), not half of them (6 -> 4, 3 -> 2 measured slower).
    if USE_TMA_DECODE and USE_CLUSTER_MERGE and head_dim in (64, 128) and page_size in (8, 16, 32, 64) and wanted >= 2:
        size = 1 << (min(wanted, 8).bit_length() - 1)
        if (wanted >= 8 or 4 * size >= 3 * wanted) and wanted <= CLUSTER_MAX_WANTED and ctas <= cluster_capacity(head_dim, size):
            return 0, size, True
    return 0, wanted, False


def tcgen05_prefill_usable(head_dim: int, page_size: int) -> bool:
    return USE_TCGEN05_PREFILL and head_dim in (64, 128) and page_size in (8, 16, 32, 64, 128)


def make_plan(ctx, num_heads: int, num_kv_heads: int, head_dim: int) -> AttentionPlan:
    device = ctx.positions.device
    tiles, items = [], []
    tile_rows = TILE_ROWS_TC if tcgen05_prefill_usable(head_dim, ctx.page_size) else TILE_ROWS
    for r in range(ctx.n_requests):
        s, n, kv = ctx.q_start[r], ctx.q_len[r], ctx.kv_len[r]
        if n >= PREFILL_MIN:
            for off in range(0, n, tile_rows):
                tiles.append((r, s + off, min(tile_rows, n - off), kv - n + off))
        else:
            items.extend(range(s, s + n))
    tiles.sort(key=lambda tile: tile[3] + tile[2])   # by keys seen, ascending: the kernels start from the far end
    d_tiles = torch.tensor(tiles, dtype=torch.int32, device=device) if tiles else None
    if len(items) == ctx.n_tokens:
        d_items = None
    else:
        d_items = torch.tensor(items, dtype=torch.int32, device=device) if items else None
    split_len, max_splits, cluster = choose_split(len(items), num_kv_heads, ctx.max_kv_len, head_dim, ctx.page_size) if items else (0, 1, False)
    plan = AttentionPlan(d_tiles, len(tiles), tile_rows, d_items, len(items), split_len, max_splits, cluster=cluster)
    if items and max_splits > 1 and not plan.cluster:
        plan.part_o = torch.empty((len(items), num_heads, max_splits, head_dim), dtype=torch.float32, device=device)
        plan.part_ml = torch.empty((len(items), num_heads, max_splits, 2), dtype=torch.float32, device=device)
    return plan


def run(q, cache, out, ctx, num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float):
    _declare()
    key = ("attention_bf16", num_heads, num_kv_heads, head_dim)
    plan: AttentionPlan = ctx.plans.get(key)
    if plan is None:
        plan = make_plan(ctx, num_heads, num_kv_heads, head_dim)
        ctx.plans[key] = plan
    lib = _lib.load()
    from . import ops
    stream = ops._stream()
    table = cache.block_table
    if plan.n_tiles and plan.tile_rows == TILE_ROWS_TC:
        from . import ops
        check(lib.mm_attention_prefill_tcgen05(q.data_ptr(), cache.k_pages.data_ptr(), cache.v_pages.data_ptr(), out.data_ptr(),
                                               plan.tiles.data_ptr(), plan.n_tiles, table.data_ptr(), table.shape[1],
                                               cache.page_size, cache.k_pages.shape[0], q.shape[0], num_heads, num_kv_heads,
                                               head_dim, window, float(scale), ops.tcgen05_error_flag(q.device).data_ptr(), stream),
              "attention_prefill_tcgen05")
    elif plan.n_tiles:
        check(lib.mm_attention_prefill_bf16(q.data_ptr(), cache.k_pages.data_ptr(), cache.v_pages.data_ptr(),
                                            out.data_ptr(), plan.tiles.data_ptr(), plan.n_tiles, table.data_ptr(),
                                            table.shape[1], cache.page_size, num_heads, num_kv_heads, head_dim, window,
                                            float(scale), stream), "attention_prefill_bf16")
    if plan.n_items and USE_TMA_DECODE and cache.page_size in (8, 16, 32, 64):
        from . import ops
        po = plan.part_o.data_ptr() if plan.part_o is not None else None
        pm = plan.part_ml.data_ptr() if plan.part_ml is not None else None
        it = plan.items.data_ptr() if plan.items is not None else None
        check(lib.mm_attention_decode_tma_bf16(
            q.data_ptr(), cache.k_pages.data_ptr(), cache.v_pages.data_ptr(), out.data_ptr(), po, pm, it, plan.n_items,
            ctx.positions.data_ptr(), ctx.token_req.data_ptr(), table.data_ptr(), table.shape[1], cache.page_size,
            cache.k_pages.shape[0], num_heads, num_kv_heads, head_dim, window, float(scale), plan.split_len, plan.max_splits,
            TMA_DECODE_STAGES, int(plan.cluster), ops.tcgen05_error_flag(q.device).data_ptr(), stream), "attention_decode_tma_bf16")
        if plan.max_splits > 1 and not plan.cluster:
            check(lib.mm_attention_decode_merge_bf16(out.data_ptr(), po, pm, it, plan.n_items, ctx.positions.data_ptr(), num_heads,
                                                     head_dim, window, plan.split_len, plan.max_splits, stream),
                  "attention_decode_merge_bf16")
    elif plan.n_items:
        check(lib.mm_attention_decode_bf16(
            q.data_ptr(), cache.k_pages.data_ptr(), cache.v_pages.data_ptr(), out.data_ptr(),
            plan.part_o.data_ptr() if plan.part_o is not None else None,
            plan.part_ml.data_ptr() if plan.part_ml is not None else None,
            plan.items.data_ptr() if plan.items is not None else None, plan.n_items, ctx.positions.data_ptr(),
            ctx.token_req.data_ptr(), table.data_ptr(), table.shape[1], cache.page_size, num_heads, num_kv_heads,
            head_dim, window, float(scale), plan.split_len, plan.max_splits, stream), "attention_decode_bf16")
    return out
