// bfloat16 paged attention on the tensor cores (mma.sync m16n8k16, fp32 accumulate and
// fp32 softmax), head size 64 or 128:
//
//   * prefill: one CTA per (tile of 64 query tokens of one request, query head); keys and
//     values stream through shared memory in tiles of 64 keys gathered page by page with
//     cp.async, two stages deep; online softmax.
//   * decode: one CTA per (token, KV head, split of the key range).  The rows of the tile
//     are the query heads that share the KV head, so a key or value is read once for all of
//     them; the four warps take 16 keys each of every 64-key tile.  A split whose token
//     has no other split writes the output directly; otherwise it writes (max, sum,
//     unnormalised output) to scratch and a merge kernel combines the splits in order.
//
// Same formula as the fp32 kernel (reference src/compute/Attention.cpp:43-94): kv head
// (h*G)/H, a query at position a sees keys [max(0, a+1-W), a], s = (q.k)*scale.  The
// reference's counterparts are its flash prefill and split-key decode kernels
// (kernels/cuda/llm/attention_prefill_flash.cu:76-196; attention_paged_v2.cu:101-269,
// 324-418), which are fp32 SIMT.
#include "common.cuh"

#define KT 64            // keys per tile
#define ATT_THREADS 128  // 4 warps
#define DEC_STAGES 3     // K/V tiles in flight per CTA of the decode kernel

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gathers 64 key rows and the same 64 value rows of one KV head into shared memory
// [64][HD + 8] each.  The page of a row is looked up once for both.  Rows outside [lo, hi)
// are zero-filled so that masked probabilities multiply zeros.
template <int HD>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* dK, __nv_bfloat16* dV, const __nv_bfloat16* __restrict__ kpool,
                                             const __nv_bfloat16* __restrict__ vpool, const int32_t* __restrict__ table,
                                             int key0, int lo, int hi, int G, int g, int page_size, int page_shift) {
    constexpr int STRIDE = HD + 8;
    constexpr int CHUNKS = HD / 8;                     // 16-byte chunks per row
    constexpr int ROWS_PER_PASS = ATT_THREADS / CHUNKS;
    const int part = threadIdx.x % CHUNKS;
#pragma unroll
    for (int r = threadIdx.x / CHUNKS; r < KT; r += ROWS_PER_PASS) {
        const int key = key0 + r;
        __nv_bfloat16* dk = dK + r * STRIDE + part * 8;
        __nv_bfloat16* dv = dV + r * STRIDE + part * 8;
        if (key >= lo && key < hi) {
            const int pidx = page_shift >= 0 ? (key >> page_shift) : (key / page_size);
            const int slot = key - pidx * page_size;
            const size_t off = (((size_t)table[pidx] * G + g) * page_size + slot) * HD + part * 8;
            cp_async16(dk, kpool + off);
            cp_async16(dv, vpool + off);
        } else {
            *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
        }
    }
}

// How a token's key range [lo, hi) is cut into splits.  split_len > 0: by absolute position,
// split s covers [s*split_len, (s+1)*split_len).  split_len == 0: the range (from lo rounded
// down to a tile) is cut evenly into at most max_splits pieces of whole tiles, so that every
// token uses the whole grid whatever its length.
struct SplitInfo {
    int first, last, len, base;
};
__device__ __forceinline__ SplitInfo split_info(int lo, int hi, int split_len, int max_splits) {
    SplitInfo s;
    if (split_len > 0) {
        s.first = lo / split_len;
        s.last = (hi - 1) / split_len;
        s.len = split_len;
        s.base = 0;
    } else {
        s.base = (lo / KT) * KT;
        const int span = hi - s.base;
        s.len = ((span + max_splits - 1) / max_splits + KT - 1) / KT * KT;
        s.first = 0;
        s.last = (span - 1) / s.len;
    }
    return s;
}

// ---------------------------------------------------------------------------
// prefill
//   tiles: int32 [n_tiles, 4] = (request index, first token row, rows in the tile, position of the first row)
// ---------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attention_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ tiles,
    const int32_t* __restrict__ block_table, int table_width, int page_size, int H, int G, int window, float scale_log2) {
    constexpr int STRIDE = HD + 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [64][STRIDE]
    __nv_bfloat16* sK = sQ + 64 * STRIDE;                            // [2][64][STRIDE]
    __nv_bfloat16* sV = sK + 2 * KT * STRIDE;                        // [2][64][STRIDE]

    // the host lists a request's tiles in ascending position; later tiles see more keys, so walk the list backwards:
    // the longest tiles start first and the short ones fill the tail
    // heads fastest, later (longer) tiles first: the longest tiles of every head start in the first wave
    const int tile = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;
    const int g = (h * G) / H;
    const int req = tiles[tile * 4 + 0], row0 = tiles[tile * 4 + 1], n_rows = tiles[tile * 4 + 2], pos0 = tiles[tile * 4 + 3];
    const int32_t* table = block_table + (size_t)req * table_width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // key range needed by the tile: from the first row's lower bound to the last row's position
    const int hi_all = pos0 + n_rows;                                     // exclusive
    const int lo_all = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int kt_begin = lo_all / KT, kt_end = (hi_all + KT - 1) / KT;

    // Q tile → shared (rows beyond n_rows are zero)
    for (int c = threadIdx.x; c < 64 * (HD / 8); c += ATT_THREADS) {
        const int r = c / (HD / 8), part = c - r * (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + r) * H + h) * HD + part * 8);
        *reinterpret_cast<uint4*>(sQ + r * STRIDE + part * 8) = v;
    }
    // first K/V tile
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    load_kv_tile<HD>(sK, sV, k_pages, v_pages, table, kt_begin * KT, lo_all, hi_all, G, g, page_size, page_shift);
    cp_async_commit();
    __syncthreads();

    // Q fragments of this warp's 16 rows
    uint32_t qf[KSTEPS][4];
    {
        const int id = lane >> 3, rr = lane & 7;
        const int r = warp * 16 + (id & 1) * 8 + rr;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
            ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], sQ + r * STRIDE + ks * 16 + (id >> 1) * 8);
    }
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;   // the two rows this thread holds
    const int pos_lo = pos0 + r_lo, pos_hi = pos0 + r_hi;
    const int wlo_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
    const int wlo_hi = (window > 0 && pos_hi + 1 > window) ? pos_hi + 1 - window : 0;
    const bool valid_lo = r_lo < n_rows, valid_hi = r_hi < n_rows;

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) {
            load_kv_tile<HD>(sK + (buf ^ 1) * KT * STRIDE, sV + (buf ^ 1) * KT * STRIDE, k_pages, v_pages, table, (kt + 1) * KT,
                             lo_all, hi_all, G, g, page_size, page_shift);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* tK = sK + buf * KT * STRIDE;
        const __nv_bfloat16* tV = sV + buf * KT * STRIDE;
        const int key0 = kt * KT;
        // a warp whose rows all lie before this tile has nothing to do in it
        const bool warp_active = (pos0 + warp * 16 + 15 >= key0) && (warp * 16 < n_rows);
        if (warp_active) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {   // pairs of 8-key tiles
                    uint32_t b0, b1, b2, b3;
                    const int id = lane >> 3, rr = lane & 7;
                    const int n = jp * 16 + (id >> 1) * 8 + rr;
                    ldmatrix_x4(b0, b1, b2, b3, tK + n * STRIDE + ks * 16 + (id & 1) * 8);
                    mma_bf16(s[jp * 2], qf[ks], b0, b1);
                    mma_bf16(s[jp * 2 + 1], qf[ks], b2, b3);
                }
            }
            // mask (only tiles that touch the diagonal, the window's edge or the tile's ragged end), running max of
            // the raw scores; the scale is folded into the exponent: p = exp2(s * c - m * c), c = scale * log2(e)
            const bool interior = (key0 + KT - 1 <= pos0 + warp * 16) && (warp * 16 + 15 < n_rows) && (window == 0 || key0 >= pos0 + warp * 16 + 16 - window);
            float mx_lo = m_lo, mx_hi = m_hi;
            if (!interior) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                        const bool hi_row = e >= 2;
                        const bool ok = hi_row ? (valid_hi && key <= pos_hi && key >= wlo_hi) : (valid_lo && key <= pos_lo && key >= wlo_lo);
                        if (!ok) s[j][e] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
                mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
            }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float use_lo = (mx_lo == -INFINITY) ? 0.0f : mx_lo * scale_log2;
            const float use_hi = (mx_hi == -INFINITY) ? 0.0f : mx_hi * scale_log2;
            const float a_lo = exp2f(m_lo * scale_log2 - use_lo), a_hi = exp2f(m_hi * scale_log2 - use_hi);
            m_lo = mx_lo;
            m_hi = mx_hi;
            float sum_lo = 0.0f, sum_hi = 0.0f;
            uint32_t pf[4][4];   // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float p0 = exp2f(fmaf(s[j][0], scale_log2, -use_lo)), p1 = exp2f(fmaf(s[j][1], scale_log2, -use_lo));
                const float p2 = exp2f(fmaf(s[j][2], scale_log2, -use_hi)), p3 = exp2f(fmaf(s[j][3], scale_log2, -use_hi));
                sum_lo += p0 + p1;
                sum_hi += p2 + p3;
                pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
            l_lo = l_lo * a_lo + sum_lo;
            l_hi = l_hi * a_hi + sum_hi;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= a_lo; o[j][1] *= a_lo; o[j][2] *= a_hi; o[j][3] *= a_hi;
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                for (int jp = 0; jp < NT_O / 2; ++jp) {
                    uint32_t b0, b1, b2, b3;
                    const int id = lane >> 3, rr = lane & 7;
                    const int key = ks * 16 + (id & 1) * 8 + rr;
                    ldmatrix_x4_trans(b0, b1, b2, b3, tV + key * STRIDE + (jp * 2 + (id >> 1)) * 8);
                    mma_bf16(o[jp * 2], pf[ks], b0, b1);
                    mma_bf16(o[jp * 2 + 1], pf[ks], b2, b3);
                }
            }
        }
        __syncthreads();   // the buffer is refilled two iterations later
    }
    // row sums live in the four threads of a quad
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = l_lo > 0.0f ? 1.0f / l_lo : 0.0f, inv_hi = l_hi > 0.0f ? 1.0f / l_hi : 0.0f;
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
        const int col = j * 8 + (lane & 3) * 2;
        if (valid_lo)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_lo) * H + h) * HD + col) = pack_bf16(o[j][0] * inv_lo, o[j][1] * inv_lo);
        if (valid_hi)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_hi) * H + h) * HD + col) = pack_bf16(o[j][2] * inv_hi, o[j][3] * inv_hi);
    }
}

// ---------------------------------------------------------------------------
// decode (split keys)
//   items: int32 [n_items] token rows (null: item i is token i)
//   part_o: fp32 [n_items, H, max_splits, HD], part_ml: fp32 [n_items, H, max_splits, 2]
// ---------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(ATT_THREADS) attention_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, const int32_t* __restrict__ items, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ token_req, const int32_t* __restrict__ block_table, int table_width, int page_size,
    int H, int G, int window, float scale_log2, int split_len, int max_splits) {
    constexpr int STRIDE = HD + 8;
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [DEC_STAGES][64][STRIDE]
    __nv_bfloat16* sV = sK + DEC_STAGES * KT * STRIDE;               // [DEC_STAGES][64][STRIDE]

    const int item = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int t = items ? items[item] : item;
    const int pos = positions[t];
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const SplitInfo sp = split_info(lo, hi, split_len, max_splits);
    if (split < sp.first || split > sp.last) return;
    const bool single = sp.first == sp.last;
    const int k_begin = max(lo, sp.base + split * sp.len), k_end = min(hi, sp.base + (split + 1) * sp.len);
    const int kt_begin = k_begin / KT, kt_end = (k_end + KT - 1) / KT;
    const int32_t* table = block_table + (size_t)token_req[t] * table_width;
    const int qpg = H / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;

    // prologue: the first DEC_STAGES - 1 tiles, one commit group each (empty groups keep the count uniform)
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
        if (kt_begin + st < kt_end)
            load_kv_tile<HD>(sK + st * KT * STRIDE, sV + st * KT * STRIDE, k_pages, v_pages, table, (kt_begin + st) * KT,
                             k_begin, k_end, G, g, page_size, page_shift);
        cp_async_commit();
    }

    // Q fragments: rows are the query heads of this KV head (rows >= qpg are zero)
    uint32_t qf[KSTEPS][4];
    {
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
        const __nv_bfloat16* q_lo = q + ((size_t)t * H + g * qpg + r_lo) * HD;
        const __nv_bfloat16* q_hi = q + ((size_t)t * H + g * qpg + r_hi) * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int c = ks * 16 + (lane & 3) * 2;
            qf[ks][0] = r_lo < qpg ? *reinterpret_cast<const uint32_t*>(q_lo + c) : 0u;
            qf[ks][1] = r_hi < qpg ? *reinterpret_cast<const uint32_t*>(q_hi + c) : 0u;
            qf[ks][2] = r_lo < qpg ? *reinterpret_cast<const uint32_t*>(q_lo + c + 8) : 0u;
            qf[ks][3] = r_hi < qpg ? *reinterpret_cast<const uint32_t*>(q_hi + c + 8) : 0u;
        }
    }
    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) % DEC_STAGES;
        {
            const int nxt = kt + DEC_STAGES - 1;
            if (nxt < kt_end) {
                const int nb = (nxt - kt_begin) % DEC_STAGES;
                load_kv_tile<HD>(sK + nb * KT * STRIDE, sV + nb * KT * STRIDE, k_pages, v_pages, table, nxt * KT, k_begin, k_end,
                                 G, g, page_size, page_shift);
            }
            cp_async_commit();
            cp_async_wait<DEC_STAGES - 1>();
        }
        __syncthreads();
        const __nv_bfloat16* tK = sK + buf * KT * STRIDE + warp * 16 * STRIDE;   // this warp's 16 keys
        const __nv_bfloat16* tV = sV + buf * KT * STRIDE + warp * 16 * STRIDE;
        const int key0 = kt * KT + warp * 16;
        if (key0 < k_end && key0 + 16 > k_begin) {
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.0f;
            s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t b0, b1, b2, b3;
                const int id = lane >> 3, rr = lane & 7;
                ldmatrix_x4(b0, b1, b2, b3, tK + ((id >> 1) * 8 + rr) * STRIDE + ks * 16 + (id & 1) * 8);
                mma_bf16(s[0], qf[ks], b0, b1);
                mma_bf16(s[1], qf[ks], b2, b3);
            }
            float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    const float v = (key >= k_begin && key < k_end) ? s[j][e] * scale_log2 : -INFINITY;
                    s[j][e] = v;
                    if (e >= 2) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
                }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float use_lo = (mx_lo == -INFINITY) ? 0.0f : mx_lo;
            const float use_hi = (mx_hi == -INFINITY) ? 0.0f : mx_hi;
            const float a_lo = exp2f(m_lo - use_lo), a_hi = exp2f(m_hi - use_hi);
            m_lo = mx_lo;
            m_hi = mx_hi;
            uint32_t pf[4];
            const float p00 = exp2f(s[0][0] - use_lo), p01 = exp2f(s[0][1] - use_lo);
            const float p02 = exp2f(s[0][2] - use_hi), p03 = exp2f(s[0][3] - use_hi);
            const float p10 = exp2f(s[1][0] - use_lo), p11 = exp2f(s[1][1] - use_lo);
            const float p12 = exp2f(s[1][2] - use_hi), p13 = exp2f(s[1][3] - use_hi);
            pf[0] = pack_bf16(p00, p01);
            pf[1] = pack_bf16(p02, p03);
            pf[2] = pack_bf16(p10, p11);
            pf[3] = pack_bf16(p12, p13);
            l_lo = l_lo * a_lo + (p00 + p01 + p10 + p11);
            l_hi = l_hi * a_hi + (p02 + p03 + p12 + p13);
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= a_lo; o[j][1] *= a_lo; o[j][2] *= a_hi; o[j][3] *= a_hi;
            }
#pragma unroll
            for (int jp = 0; jp < NT_O / 2; ++jp) {
                uint32_t b0, b1, b2, b3;
                const int id = lane >> 3, rr = lane & 7;
                ldmatrix_x4_trans(b0, b1, b2, b3, tV + ((id & 1) * 8 + rr) * STRIDE + (jp * 2 + (id >> 1)) * 8);
                mma_bf16(o[jp * 2], pf, b0, b1);
                mma_bf16(o[jp * 2 + 1], pf, b2, b3);
            }
        }
        __syncthreads();
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    cp_async_wait<0>();
    // merge the four warps through shared memory (the K/V buffers are free now)
    float* mo = reinterpret_cast<float*>(smem_raw);         // [4][16][HD]
    float* mml = mo + 4 * 16 * HD;                          // [4][16][2]
    {
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            const int col = j * 8 + (lane & 3) * 2;
            float* base = mo + (size_t)warp * 16 * HD;
            base[r_lo * HD + col] = o[j][0];
            base[r_lo * HD + col + 1] = o[j][1];
            base[r_hi * HD + col] = o[j][2];
            base[r_hi * HD + col + 1] = o[j][3];
        }
        if ((lane & 3) == 0) {
            mml[(warp * 16 + r_lo) * 2] = m_lo;
            mml[(warp * 16 + r_lo) * 2 + 1] = l_lo;
            mml[(warp * 16 + r_hi) * 2] = m_hi;
            mml[(warp * 16 + r_hi) * 2 + 1] = l_hi;
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < qpg * HD; idx += ATT_THREADS) {
        const int r = idx / HD, col = idx - r * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, mml[(w * 16 + r) * 2]);
        const float mu = (m == -INFINITY) ? 0.0f : m;
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(mml[(w * 16 + r) * 2] - mu);
            l += mml[(w * 16 + r) * 2 + 1] * f;
            acc += mo[((size_t)w * 16 + r) * HD + col] * f;
        }
        const int h = g * qpg + r;
        if (single) {
            out[((size_t)t * H + h) * HD + col] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
        } else {
            const size_t p = ((size_t)item * H + h) * max_splits + split;
            part_o[p * HD + col] = acc;
            if (col == 0) {
                part_ml[p * 2] = m;
                part_ml[p * 2 + 1] = l;
            }
        }
    }
}

template <int HD>
__global__ void attention_merge_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ part_o,
                                       const float* __restrict__ part_ml, const int32_t* __restrict__ items,
                                       const int32_t* __restrict__ positions, int H, int window, int split_len,
                                       int max_splits) {
    const int item = blockIdx.x, h = blockIdx.y;
    const int t = items ? items[item] : item;
    const int hi = positions[t] + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const SplitInfo sp = split_info(lo, hi, split_len, max_splits);
    const int first_split = sp.first, last_split = sp.last;
    if (first_split == last_split) return;   // written by the attention kernel itself
    const size_t base = ((size_t)item * H + h) * max_splits;
    const int n = last_split - first_split + 1;
    // Up to MERGE_SMEM splits: every thread fetches the (maximum, sum) of a few splits, the weights 2^(m_s - m) go to
    // shared memory, and the sum over the splits then runs with sixteen loads in flight (in ascending order of the
    // splits).  Longer lists take the plain loop below.
    constexpr int MERGE_SMEM = 1024;
    __shared__ float w_s[MERGE_SMEM];
    __shared__ float l_s[MERGE_SMEM];
    __shared__ float red_s[32];
    __shared__ float inv_s;
    if (n <= MERGE_SMEM) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
        float m = -INFINITY;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base + first_split + i) * 2);
            w_s[i] = ml.x;
            l_s[i] = ml.y;
            m = fmaxf(m, ml.x);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red_s[warp] = m;
        __syncthreads();
        m = red_s[0];
        for (int i = 1; i < n_warps; ++i) m = fmaxf(m, red_s[i]);
        const float mu = (m == -INFINITY) ? 0.0f : m;
        for (int i = threadIdx.x; i < n; i += blockDim.x) w_s[i] = exp2f(w_s[i] - mu);
        __syncthreads();
        if (warp == 0) {
            // lane j adds the splits j, j + 32, ... in ascending order, then a fixed shuffle tree adds the lanes
            float l = 0.0f;
            for (int i = lane; i < n; i += 32) l += l_s[i] * w_s[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            if (lane == 0) inv_s = l > 0.0f ? 1.0f / l : 0.0f;
        }
        __syncthreads();
        const float inv = inv_s;
        for (int col = threadIdx.x; col < HD; col += blockDim.x) {
            const float* po = part_o + (base + first_split) * HD + col;
            float acc = 0.0f;
            int i = 0;
            for (; i + 16 <= n; i += 16) {
                float v[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) v[u] = po[(size_t)(i + u) * HD];
#pragma unroll
                for (int u = 0; u < 16; ++u) acc += v[u] * w_s[i + u];
            }
            for (; i < n; ++i) acc += po[(size_t)i * HD] * w_s[i];
            out[((size_t)t * H + h) * HD + col] = __float2bfloat16_rn(acc * inv);
        }
        return;
    }
    float m = -INFINITY;
    for (int s = first_split; s <= last_split; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
    const float mu = (m == -INFINITY) ? 0.0f : m;
    float l = 0.0f;
    for (int s = first_split; s <= last_split; ++s) l += part_ml[(base + s) * 2 + 1] * exp2f(part_ml[(base + s) * 2] - mu);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    for (int col = threadIdx.x; col < HD; col += blockDim.x) {
        float acc = 0.0f;
        for (int s = first_split; s <= last_split; ++s)
            acc += part_o[(base + s) * HD + col] * exp2f(part_ml[(base + s) * 2] - mu);
        out[((size_t)t * H + h) * HD + col] = __float2bfloat16_rn(acc * inv);
    }
}

static const float LOG2E = 1.4426950408889634f;

template <int HD>
static int launch_prefill(const void* q, const void* k, const void* v, void* out, const void* tiles, int n_tiles,
                          const void* table, int table_width, int page_size, int H, int G, int window, float scale,
                          cudaStream_t s) {
    const size_t smem = (size_t)(64 + 4 * KT) * (HD + 8) * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = true;
    }
    dim3 grid(H, n_tiles);
    attention_prefill_kernel<HD><<<grid, ATT_THREADS, smem, s>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out,
        (const int32_t*)tiles, (const int32_t*)table, table_width, page_size, H, G, window, scale * LOG2E);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                        const void* tiles, int n_tiles, const void* block_table, int table_width,
                                        int page_size, int H, int G, int hd, int window, float scale, void* stream) {
    MM_REQUIRE(n_tiles >= 0 && H > 0 && G > 0 && H % G == 0, "attention_prefill: bad head counts");
    MM_REQUIRE(n_tiles <= 65535, "attention_prefill: more than 65535 tiles in one launch");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0, "attention_prefill: bad page geometry or window");
    if (n_tiles == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return launch_prefill<64>(q, k_pages, v_pages, out, tiles, n_tiles, block_table, table_width, page_size, H, G, window, scale, s);
    if (hd == 128) return launch_prefill<128>(q, k_pages, v_pages, out, tiles, n_tiles, block_table, table_width, page_size, H, G, window, scale, s);
    mm_set_last_error("attention_prefill: the tensor-core kernel is built for head_dim 64 and 128");
    return MM_ERR_UNSUPPORTED;
}

template <int HD>
static int launch_decode(const void* q, const void* k, const void* v, void* out, void* part_o, void* part_ml,
                         const void* items, int n_items, const void* positions, const void* token_req,
                         const void* table, int table_width, int page_size, int H, int G, int window, float scale,
                         int split_len, int max_splits, cudaStream_t s) {
    size_t smem = (size_t)(2 * DEC_STAGES * KT) * (HD + 8) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)(4 * 16 * HD + 4 * 16 * 2) * sizeof(float);
    if (merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = true;
    }
    dim3 grid(n_items, G, max_splits);
    mm_launch(attention_decode_kernel<HD>, grid, dim3(ATT_THREADS), smem, s,
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, (float*)part_o,
        (float*)part_ml, (const int32_t*)items, (const int32_t*)positions, (const int32_t*)token_req,
        (const int32_t*)table, table_width, page_size, H, G, window, scale * LOG2E, split_len, max_splits);
    MM_CHECK_LAUNCH();
    if (max_splits > 1) {
        dim3 mgrid(n_items, H);
        mm_launch(attention_merge_kernel<HD>, mgrid, dim3(HD >= 128 ? 128 : 64), 0, s, (__nv_bfloat16*)out, (const float*)part_o,
                                                                         (const float*)part_ml, (const int32_t*)items,
                                                                         (const int32_t*)positions, H, window, split_len,
                                                                         max_splits);
        MM_CHECK_LAUNCH();
    }
    return MM_OK;
}

// Scratch: part_o needs n_items*H*max_splits*hd floats, part_ml n_items*H*max_splits*2 floats
// (both may be null when max_splits == 1).  With split_len > 0, max_splits must cover
// ceil((max position + 1) / split_len); with split_len == 0 each token's range is cut evenly into
// at most max_splits pieces.
MM_EXPORT int mm_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, void* part_o,
                                       void* part_ml, const void* items, int n_items, const void* positions,
                                       const void* token_req, const void* block_table, int table_width, int page_size,
                                       int H, int G, int hd, int window, float scale, int split_len, int max_splits,
                                       void* stream) {
    MM_REQUIRE(n_items >= 0 && H > 0 && G > 0 && H % G == 0, "attention_decode: bad head counts");
    MM_REQUIRE(H / G <= 16, "attention_decode: more than 16 query heads per KV head");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0, "attention_decode: bad page geometry or window");
    MM_REQUIRE(split_len >= 0 && split_len % KT == 0 && max_splits >= 1 && max_splits <= 65535, "attention_decode: split_len must be 0 (even cut) or a positive multiple of 64");
    MM_REQUIRE(max_splits == 1 || (part_o != nullptr && part_ml != nullptr), "attention_decode: scratch missing");
    MM_REQUIRE(G <= 65535, "attention_decode: too many KV heads");
    if (n_items == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return launch_decode<64>(q, k_pages, v_pages, out, part_o, part_ml, items, n_items, positions, token_req, block_table, table_width, page_size, H, G, window, scale, split_len, max_splits, s);
    if (hd == 128) return launch_decode<128>(q, k_pages, v_pages, out, part_o, part_ml, items, n_items, positions, token_req, block_table, table_width, page_size, H, G, window, scale, split_len, max_splits, s);
    mm_set_last_error("attention_decode: the tensor-core kernel is built for head_dim 64 and 128");
    return MM_ERR_UNSUPPORTED;
}

// The merge pass alone, for the decode kernel of attention_decode_tma.cu, which writes the same partial results.
MM_EXPORT int mm_attention_decode_merge_bf16(void* out, const void* part_o, const void* part_ml, const void* items, int n_items,
                                             const void* positions, int H, int hd, int window, int split_len, int max_splits,
                                             void* stream) {
    MM_REQUIRE(hd == 64 || hd == 128, "attention_decode_merge: head_dim must be 64 or 128");
    MM_REQUIRE(n_items >= 0 && H > 0 && max_splits >= 1 && part_o != nullptr && part_ml != nullptr, "attention_decode_merge: bad arguments");
    if (n_items == 0 || max_splits == 1) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 mgrid(n_items, H);
    if (hd == 128)
        mm_launch(attention_merge_kernel<128>, mgrid, dim3(128), 0, s, (__nv_bfloat16*)out, (const float*)part_o, (const float*)part_ml,
                      (const int32_t*)items, (const int32_t*)positions, H, window, split_len, max_splits);
    else
        mm_launch(attention_merge_kernel<64>, mgrid, dim3(64), 0, s, (__nv_bfloat16*)out, (const float*)part_o, (const float*)part_ml,
                      (const int32_t*)items, (const int32_t*)positions, H, window, split_len, max_splits);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------
// Split-key decode attention for callers that cannot allocate (see no_alloc.h).
// ---------------------------------------------------------------------------
#include "no_alloc.h"
#include <stdio.h>

// The scratch of the no-allocation entry point.  In host code this name is only a handle
// for cudaGetSymbolAddress: it is not a device address and must never be passed to a kernel.
static __device__ __align__(256) float g_no_alloc_scratch[MM_NO_ALLOC_SCRATCH_FLOATS];

#define MM_NO_ALLOC_MAX_DEVICES 64
static float* g_no_alloc_scratch_ptr[MM_NO_ALLOC_MAX_DEVICES];   // device address of the array, per device

MM_EXPORT int mm_attention_decode_bf16_no_alloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                                const void* items, int n_items, const void* positions,
                                                const void* token_req, const void* block_table, int table_width,
                                                int page_size, int H, int G, int hd, int window, float scale,
                                                int split_len, int max_splits, void* stream) {
    MM_REQUIRE(n_items >= 0 && H > 0 && hd > 0 && max_splits >= 1, "attention_decode_no_alloc: bad sizes");
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (max_splits > 1) {
        const long long rows = (long long)n_items * H * max_splits;
        const long long need = rows * ((long long)hd + 2);
        if (need > (long long)MM_NO_ALLOC_SCRATCH_FLOATS) {
            char msg[256];
            snprintf(msg, sizeof(msg),
                     "attention_decode_no_alloc: this call needs %lld floats of scratch (items %d x heads %d x splits %d x "
                     "(head_dim %d + 2)), the built-in scratch holds %d",
                     need, n_items, H, max_splits, hd, (int)MM_NO_ALLOC_SCRATCH_FLOATS);
            mm_set_last_error(msg);
            return MM_ERR_BAD_ARG;
        }
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MM_NO_ALLOC_MAX_DEVICES) {
            mm_set_last_error("attention_decode_no_alloc: no current CUDA device (or its index is above 63)");
            return MM_ERR_DRIVER;
        }
        if (g_no_alloc_scratch_ptr[dev] == nullptr) {
            // one-time set-up for this device, with this device current
            void* p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
            if (e != cudaSuccess || p == nullptr) {
                mm_set_last_error(cudaGetErrorString(e));
                return MM_ERR_DRIVER;
            }
            g_no_alloc_scratch_ptr[dev] = (float*)p;
        }
        part_o = g_no_alloc_scratch_ptr[dev];        // [rows, hd]
        part_ml = part_o + rows * hd;                // [rows, 2]; rows * hd * 4 bytes is a multiple of 8
    }
    return mm_attention_decode_bf16(q, k_pages, v_pages, out, part_o, part_ml, items, n_items, positions, token_req,
                                    block_table, table_width, page_size, H, G, hd, window, scale, split_len, max_splits,
                                    stream);
}
