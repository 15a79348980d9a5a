// Split-key paged decode attention with a TMA producer warp (bfloat16, head size 64 or 128).
//
// Same arithmetic, work split and partial-result format as attention_decode_kernel in
// attention_mma.cu (one CTA per (token, KV head, split); rows of the mma tile are the query
// heads sharing the KV head; four consumer warps take 16 keys each of every 64-key tile; the
// merge kernel of that file combines the splits), but the keys and values are fetched by a
// fifth warp with cp.async.bulk.tensor, page by page (a page of one KV head is one contiguous
// [page_size, head] block in the pool), into a ring of STAGES tiles with full/empty mbarriers.
// The consumer warps issue no loads, compute no addresses and never meet at a CTA barrier in
// the loop, so the bytes in flight per SM are set by the ring depth alone.
//
// Tiles are written with the 128-byte swizzle; ldmatrix row addresses apply the same xor.
// Waits are bounded; on a time-out the CTA gives up and sets `err`.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int DT_KT = 64;                 // keys per tile
constexpr int DT_CONSUMERS = 4;           // warps
constexpr int DT_THREADS = (DT_CONSUMERS + 1) * 32;

struct SplitRange {
    int first, last, len, base;
};
// identical to split_info of attention_mma.cu (the merge kernel there must see the same cut)
__device__ __forceinline__ SplitRange split_range(int lo, int hi, int split_len, int max_splits) {
    SplitRange s;
    if (split_len > 0) {
        s.first = lo / split_len;
        s.last = (hi - 1) / split_len;
        s.len = split_len;
        s.base = 0;
    } else {
        s.base = (lo / DT_KT) * DT_KT;
        const int span = hi - s.base;
        s.len = ((span + max_splits - 1) / max_splits + DT_KT - 1) / DT_KT * DT_KT;
        s.first = 0;
        s.last = (span - 1) / s.len;
    }
    return s;
}

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2bf(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int STAGES>
struct DecCtl {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t done;            // the four consumer warps have written their partial results to shared memory
    int abort_flag;
};

// byte offset of (row, 16-byte chunk c of the head) inside a [64 keys x HD] tile stored as HD/64 column halves of
// [64 x 64] (128 bytes per row) with the 128-byte swizzle
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * (DT_KT * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int HD, int STAGES>
__global__ void __launch_bounds__(DT_THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                            float* __restrict__ part_ml, const int32_t* __restrict__ items, const int32_t* __restrict__ positions,
                            const int32_t* __restrict__ token_req, const int32_t* __restrict__ block_table, int table_width,
                            int page_size, int H, int G, int window, float scale_log2, int split_len, int max_splits,
                            int* __restrict__ err) {
    constexpr int KSTEPS = HD / 16;
    constexpr int NT_O = HD / 8;
    constexpr int HALVES = HD / 64;
    constexpr int TILE = DT_KT * HD * 2;                       // bytes of one K (or V) tile
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* sK = smem_raw;                              // STAGES * TILE
    unsigned char* sV = sK + STAGES * TILE;                    // STAGES * TILE
    DecCtl<STAGES>* ctl = reinterpret_cast<DecCtl<STAGES>*>(sV + STAGES * TILE);
    volatile int* abort_flag = &ctl->abort_flag;

    const int item = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int t = items ? items[item] : item;
    const int pos = positions[t];
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const SplitRange sp = split_range(lo, hi, split_len, max_splits);
    if (split < sp.first || split > sp.last) return;
    const bool single = sp.first == sp.last;
    const int k_begin = max(lo, sp.base + split * sp.len), k_end = min(hi, sp.base + (split + 1) * sp.len);
    const int kt_begin = k_begin / DT_KT, kt_end = (k_end + DT_KT - 1) / DT_KT;
    const int32_t* table = block_table + (size_t)token_req[t] * table_width;
    const int qpg = H / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0 && err != nullptr) atomicExch(err, 5);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), DT_CONSUMERS);
        }
        mbar_init(smem_u32(&ctl->done), DT_CONSUMERS);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // value rows that are never fetched (beyond the split's last key) are multiplied by P = 0: they must be finite
    for (int i = threadIdx.x; i < STAGES * TILE / 16; i += DT_THREADS) reinterpret_cast<uint4*>(sV)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    if (warp == DT_CONSUMERS) {
        // ---- producer: lane = (page of the tile, K or V, column half), all copies of a tile issued at once ----
        const int pages_per_tile = DT_KT / page_size;
        const uint32_t page_bytes = (uint32_t)page_size * 128u;          // one column half of a page
        const int per_page = 2 * HALVES;                                 // copies per page: K and V, each column half
        const int j = lane / per_page, sub = lane % per_page;
        const bool is_v = sub >= HALVES;
        const int hf = sub % HALVES;
        uint32_t it = 0;
        bool ok = true;
        for (int kt = kt_begin; kt < kt_end && ok; ++kt, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            int pid = -1;
            if (j < pages_per_tile) {
                const int key_lo = kt * DT_KT + j * page_size;
                if (key_lo < k_end && key_lo + page_size > k_begin) pid = table[kt * pages_per_tile + j];
            }
            const uint32_t have = __ballot_sync(0xffffffffu, pid >= 0);
            const uint32_t full = smem_u32(&ctl->full[s]);
            if (lane == 0) {
                ok = mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1, abort_flag);
                if (ok) mbar_expect_tx(full, (uint32_t)__popc(have) * page_bytes);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok && pid >= 0)
                tma_load_2d(smem_u32((is_v ? sV : sK) + s * TILE) + hf * (DT_KT * 128) + (uint32_t)j * page_bytes, is_v ? &tmV : &tmK,
                            hf * 64, (pid * G + g) * page_size, full);
        }
        return;     // the producer warp takes no part in the merge
    }

    // ---- consumers ----
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
    bool ok = true;
    uint32_t it = 0;
    for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(smem_u32(&ctl->full[s]), ph, abort_flag)) { ok = false; break; }
        const uint32_t tK = smem_u32(sK + s * TILE), tV = smem_u32(sV + s * TILE);
        const int key0 = kt * DT_KT + warp * 16;                 // this warp's 16 keys
        if (key0 < k_end && key0 + 16 > k_begin) {
            float sc[2][4];
            sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = 0.0f;
            sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.0f;
            const int id = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, tK + tile_off<HD>(warp * 16 + (id >> 1) * 8 + rr, ks * 2 + (id & 1)));
                mma16816(sc[0], qf[ks], b0, b1);
                mma16816(sc[1], qf[ks], b2, b3);
            }
            float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                    const float v = (key >= k_begin && key < k_end) ? sc[j][e] * scale_log2 : -INFINITY;
                    sc[j][e] = v;
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
            const float p00 = exp2f(sc[0][0] - use_lo), p01 = exp2f(sc[0][1] - use_lo);
            const float p02 = exp2f(sc[0][2] - use_hi), p03 = exp2f(sc[0][3] - use_hi);
            const float p10 = exp2f(sc[1][0] - use_lo), p11 = exp2f(sc[1][1] - use_lo);
            const float p12 = exp2f(sc[1][2] - use_hi), p13 = exp2f(sc[1][3] - use_hi);
            pf[0] = pack2bf(p00, p01);
            pf[1] = pack2bf(p02, p03);
            pf[2] = pack2bf(p10, p11);
            pf[3] = pack2bf(p12, p13);
            l_lo = l_lo * a_lo + (p00 + p01 + p10 + p11);
            l_hi = l_hi * a_hi + (p02 + p03 + p12 + p13);
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= a_lo; o[j][1] *= a_lo; o[j][2] *= a_hi; o[j][3] *= a_hi;
            }
#pragma unroll
            for (int jp = 0; jp < NT_O / 2; ++jp) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(b0, b1, b2, b3, tV + tile_off<HD>(warp * 16 + (id & 1) * 8 + rr, jp * 2 + (id >> 1)));
                mma16816(o[jp * 2], pf, b0, b1);
                mma16816(o[jp * 2 + 1], pf, b2, b3);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctl->empty[s]));
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    // merge the four warps through shared memory.  All tiles this warp waited for have landed and every consumer has
    // released every stage it read, so once all four warps are here the K ring is free to be reused.
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctl->done));
    if (!ok || !mbar_wait(smem_u32(&ctl->done), 0, abort_flag)) {
        if (lane == 0 && err != nullptr) atomicExch(err, 4);
        return;
    }
    float* mo = reinterpret_cast<float*>(sK);                 // [4][16][HD]
    float* mml = mo + 4 * 16 * HD;                            // [4][16][2]
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
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ctl->done));          // second phase: the partial results are in shared memory
    if (!mbar_wait(smem_u32(&ctl->done), 1, abort_flag)) {
        if (lane == 0 && err != nullptr) atomicExch(err, 4);
        return;
    }
    for (int idx = threadIdx.x; idx < qpg * HD; idx += DT_CONSUMERS * 32) {
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

template <int HD, int STAGES>
int launch_decode_tma(const CUtensorMap& tk, const CUtensorMap& tv, const void* q, void* out, void* part_o, void* part_ml,
                      const void* items, int n_items, const void* positions, const void* token_req, const void* table,
                      int table_width, int page_size, int H, int G, int window, float scale, int split_len, int max_splits,
                      int* err, cudaStream_t s) {
    constexpr int TILE = DT_KT * HD * 2;
    const size_t smem = (size_t)2 * STAGES * TILE + sizeof(DecCtl<STAGES>);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_decode_tma_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            mm_set_last_error("attention_decode_tma: cannot reserve shared memory");
            return MM_ERR_LAUNCH;
        }
        configured = true;
    }
    dim3 grid(n_items, G, max_splits);
    attention_decode_tma_kernel<HD, STAGES><<<grid, DT_THREADS, smem, s>>>(
        tk, tv, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (float*)part_o, (float*)part_ml, (const int32_t*)items,
        (const int32_t*)positions, (const int32_t*)token_req, (const int32_t*)table, table_width, page_size, H, G, window,
        scale * 1.4426950408889634f, split_len, max_splits, err);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

}  // namespace

// The attention part only: the caller runs the merge of attention_mma.cu afterwards when max_splits > 1
// (mm_attention_decode_merge_bf16).  Arguments as mm_attention_decode_bf16, plus the pool size for the tensor maps.
MM_EXPORT int mm_attention_decode_tma_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, void* part_o,
                                           void* part_ml, const void* items, int n_items, const void* positions,
                                           const void* token_req, const void* block_table, int table_width, int page_size,
                                           int num_pages, int H, int G, int hd, int window, float scale, int split_len,
                                           int max_splits, int stages, void* err, void* stream) {
    MM_REQUIRE(hd == 64 || hd == 128, "attention_decode_tma: built for head_dim 64 and 128");
    MM_REQUIRE(n_items >= 0 && H > 0 && G > 0 && H % G == 0 && H / G <= 16 && num_pages > 0, "attention_decode_tma: bad head counts");
    MM_REQUIRE(page_size >= 8 && page_size <= 64 && (64 % page_size) == 0, "attention_decode_tma: page_size must be 8, 16, 32 or 64");
    MM_REQUIRE(split_len >= 0 && split_len % 64 == 0 && max_splits >= 1 && max_splits <= 65535 && G <= 65535, "attention_decode_tma: bad split");
    MM_REQUIRE(max_splits == 1 || (part_o != nullptr && part_ml != nullptr), "attention_decode_tma: scratch missing");
    MM_REQUIRE(stages == 3 || stages == 6, "attention_decode_tma: stages must be 3 or 6");
    if (n_items == 0) return MM_OK;
    CUtensorMap tk, tv;
    const long long pool_rows = (long long)num_pages * G * page_size;
    if (!tc::make_map_bf16(&tk, k_pages, pool_rows, hd, hd, page_size) || !tc::make_map_bf16(&tv, v_pages, pool_rows, hd, hd, page_size)) {
        mm_set_last_error("attention_decode_tma: cuTensorMapEncodeTiled failed or is not available");
        return MM_ERR_DRIVER;
    }
    cudaStream_t s = (cudaStream_t)stream;
#define MM_DT(HDV, ST) launch_decode_tma<HDV, ST>(tk, tv, q, out, part_o, part_ml, items, n_items, positions, token_req, block_table, \
                                                  table_width, page_size, H, G, window, scale, split_len, max_splits, (int*)err, s)
    if (hd == 128) return stages == 3 ? MM_DT(128, 3) : MM_DT(128, 6);
    return stages == 3 ? MM_DT(64, 3) : MM_DT(64, 6);
#undef MM_DT
}
