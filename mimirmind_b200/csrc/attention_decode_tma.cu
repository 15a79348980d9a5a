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
//
// CLUSTER variant (at most 8 splits): the splits of one (token, KV head) are one thread-block cluster.  Each CTA
// leaves its partial result in its own shared memory; after a cluster barrier every CTA merges a slice of the
// output columns, reading the partials of its peers through distributed shared memory, and writes bf16 output:
// no scratch in global memory and no merge launch.  Every thread of every CTA reaches both cluster barriers on
// every path (a CTA without keys, a failed wait), so the barriers cannot be left waiting.
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

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
    return r;
}
// value of a float in the shared memory of CTA `rank` of this cluster, at the place `local` has in this CTA's
__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

template <int HD, int STAGES, bool CLUSTER>
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
    const bool has_keys = split >= sp.first && split <= sp.last;
    if (!CLUSTER && !has_keys) return;
    const bool single = sp.first == sp.last;
    const int k_begin = max(lo, sp.base + split * sp.len), k_end = min(hi, sp.base + (split + 1) * sp.len);
    const int kt_begin = k_begin / DT_KT, kt_end = (k_end + DT_KT - 1) / DT_KT;
    const int32_t* table = block_table + (size_t)token_req[t] * table_width;
    const int qpg = H / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // the partial result of this CTA for the cluster merge: [16 heads][HD] sums, then [16][2] (max, sum of weights);
    // behind the scratch of the four-warp merge inside the key ring
    float* fin_o = reinterpret_cast<float*>(sK) + 4 * 16 * HD + 4 * 16 * 2;
    float* fin_ml = fin_o + 16 * HD;
    static_assert((4 * 16 * HD + 4 * 16 * 2 + 16 * HD + 16 * 2) * sizeof(float) <= (size_t)STAGES * TILE, "merge scratch must fit in the key ring");
    bool good = (smem_u32(smem_raw) & 1023u) == 0;
    if (!good) {
        if (threadIdx.x == 0 && err != nullptr) atomicExch(err, 5);
        if (!CLUSTER) return;
    }
    if (threadIdx.x == DT_CONSUMERS * 32) {
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
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

    if (good && has_keys && warp == DT_CONSUMERS) {
        // ---- producer: lane = (page of the tile, K or V, column half), all copies of a tile issued at once ----
        const int pages_per_tile = DT_KT / page_size;
        const uint32_t page_bytes = (uint32_t)page_size * 128u;          // one column half of a page
        const int per_page = 2 * HALVES;                                 // copies per page: K and V, each column half
        const int j = lane / per_page, sub = lane % per_page;
        const bool is_v = sub >= HALVES;
        const int hf = sub % HALVES;
        uint32_t it = 0;
        bool ok = true;
        // page ids are read a few tiles ahead: the load from the block table would otherwise sit, with its full
        // latency, between every two tiles
        auto page_of = [&](int kt) -> int {
            if (kt >= kt_end || j >= pages_per_tile) return -1;
            const int key_lo = kt * DT_KT + j * page_size;
            return (key_lo < k_end && key_lo + page_size > k_begin) ? table[kt * pages_per_tile + j] : -1;
        };
        constexpr int AHEAD = 4;
        int ahead[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) ahead[i] = page_of(kt_begin + i);
        for (int kt = kt_begin; kt < kt_end && ok; ++kt, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            const int pid = ahead[0];
#pragma unroll
            for (int i = 0; i + 1 < AHEAD; ++i) ahead[i] = ahead[i + 1];
            ahead[AHEAD - 1] = page_of(kt + AHEAD);
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
        if (!CLUSTER) return;     // the producer warp takes no part in the merge inside the CTA
    } else if (good && has_keys) {
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
        if (!CLUSTER) return;
        good = false;
    }
    float* mo = reinterpret_cast<float*>(sK);                 // [4][16][HD]
    float* mml = mo + 4 * 16 * HD;                            // [4][16][2]
    if (good) {
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
        if (!CLUSTER) return;
        good = false;
    }
    }
    if (good)
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
        if (CLUSTER) {
            fin_o[r * HD + col] = acc;
            if (col == 0) {
                fin_ml[r * 2] = m;
                fin_ml[r * 2 + 1] = l;
            }
        } else if (single) {
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
    }   // consumers

    if constexpr (CLUSTER) {
        // a CTA without keys (or one that gave up) contributes nothing: weight 0
        if ((!has_keys || !good) && threadIdx.x < 16) {
            fin_ml[threadIdx.x * 2] = -INFINITY;
            fin_ml[threadIdx.x * 2 + 1] = 0.0f;
        }
        cluster_sync_all();
        // this CTA's slice of the qpg * HD output values; partials in split order, as the merge kernel sums them
        const int n_ranks = (int)cluster_size(), rank = (int)cluster_rank();
        const int total = qpg * HD, chunk = (total + n_ranks - 1) / n_ranks;
        const int end = min(total, (rank + 1) * chunk);
        for (int idx = rank * chunk + (int)threadIdx.x; idx < end; idx += DT_THREADS) {
            const int r = idx / HD, col = idx - r * HD;
            float m = -INFINITY;
            for (int sI = 0; sI < n_ranks; ++sI) m = fmaxf(m, ld_peer_f32(&fin_ml[r * 2], sI));
            const float mu = (m == -INFINITY) ? 0.0f : m;
            float l = 0.0f, acc = 0.0f;
            for (int sI = 0; sI < n_ranks; ++sI) {
                const float lp = ld_peer_f32(&fin_ml[r * 2 + 1], sI);
                if (lp > 0.0f) {                       // a peer without keys holds no sums
                    const float f = exp2f(ld_peer_f32(&fin_ml[r * 2], sI) - mu);
                    l += lp * f;
                    acc += ld_peer_f32(&fin_o[r * HD + col], sI) * f;
                }
            }
            out[((size_t)t * H + g * qpg + r) * HD + col] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
        }
        cluster_sync_all();                            // peers may still be reading this CTA's shared memory
    }
}

template <int HD, int STAGES, bool CLUSTER>
int launch_decode_tma(const CUtensorMap& tk, const CUtensorMap& tv, const void* q, void* out, void* part_o, void* part_ml,
                      const void* items, int n_items, const void* positions, const void* token_req, const void* table,
                      int table_width, int page_size, int H, int G, int window, float scale, int split_len, int max_splits,
                      int* err, cudaStream_t s) {
    constexpr int TILE = DT_KT * HD * 2;
    const size_t smem = (size_t)2 * STAGES * TILE + sizeof(DecCtl<STAGES>);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_decode_tma_kernel<HD, STAGES, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            mm_set_last_error("attention_decode_tma: cannot reserve shared memory");
            return MM_ERR_LAUNCH;
        }
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_items, G, max_splits);
    cfg.blockDim = dim3(DT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = max_splits;       // the splits of one (token, KV head) are one cluster
    cfg.attrs = attr;
    cfg.numAttrs = CLUSTER ? 1 : 0;
    cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel<HD, STAGES, CLUSTER>, tk, tv, (const __nv_bfloat16*)q, (__nv_bfloat16*)out,
                       (float*)part_o, (float*)part_ml, (const int32_t*)items, (const int32_t*)positions, (const int32_t*)token_req,
                       (const int32_t*)table, table_width, page_size, H, G, window, scale * 1.4426950408889634f, split_len,
                       max_splits, err);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// How many clusters of `cluster_size` CTAs of the cluster variant can be resident on the device at once.
template <int HD>
int max_active_clusters(int cluster_size, int* out) {
    constexpr int STAGES = 3, TILE = DT_KT * HD * 2;
    const size_t smem = (size_t)2 * STAGES * TILE + sizeof(DecCtl<STAGES>);
    if (cudaFuncSetAttribute(attention_decode_tma_kernel<HD, STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        mm_set_last_error("attention_decode_tma: cannot reserve shared memory");
        return MM_ERR_LAUNCH;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, cluster_size);
    cfg.blockDim = dim3(DT_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = cluster_size;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(out, attention_decode_tma_kernel<HD, STAGES, true>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        mm_set_last_error("attention_decode_tma: cudaOccupancyMaxActiveClusters failed");
        return MM_ERR_LAUNCH;
    }
    return MM_OK;
}

}  // namespace

// The attention part only: the caller runs the merge of attention_mma.cu afterwards when max_splits > 1
// (mm_attention_decode_merge_bf16), unless `cluster` is set: then 2 <= max_splits <= 8, the splits are merged inside the
// kernel by a thread-block cluster, no scratch is used and `out` is final.
// Arguments as mm_attention_decode_bf16, plus the pool size for the tensor maps.
MM_EXPORT int mm_attention_decode_tma_bf16(const void* q, const void* k_pages, const void* v_pages, void* out, void* part_o,
                                           void* part_ml, const void* items, int n_items, const void* positions,
                                           const void* token_req, const void* block_table, int table_width, int page_size,
                                           int num_pages, int H, int G, int hd, int window, float scale, int split_len,
                                           int max_splits, int stages, int cluster, void* err, void* stream) {
    MM_REQUIRE(hd == 64 || hd == 128, "attention_decode_tma: built for head_dim 64 and 128");
    MM_REQUIRE(n_items >= 0 && H > 0 && G > 0 && H % G == 0 && H / G <= 16 && num_pages > 0, "attention_decode_tma: bad head counts");
    MM_REQUIRE(page_size >= 8 && page_size <= 64 && (64 % page_size) == 0, "attention_decode_tma: page_size must be 8, 16, 32 or 64");
    MM_REQUIRE(split_len >= 0 && split_len % 64 == 0 && max_splits >= 1 && max_splits <= 65535 && G <= 65535, "attention_decode_tma: bad split");
    MM_REQUIRE(cluster || max_splits == 1 || (part_o != nullptr && part_ml != nullptr), "attention_decode_tma: scratch missing");
    MM_REQUIRE(!cluster || (max_splits >= 2 && max_splits <= 8), "attention_decode_tma: a cluster merges 2 to 8 splits");
    MM_REQUIRE(stages == 3 || stages == 6, "attention_decode_tma: stages must be 3 or 6");
    if (n_items == 0) return MM_OK;
    CUtensorMap tk, tv;
    const long long pool_rows = (long long)num_pages * G * page_size;
    if (!tc::make_map_bf16(&tk, k_pages, pool_rows, hd, hd, page_size) || !tc::make_map_bf16(&tv, v_pages, pool_rows, hd, hd, page_size)) {
        mm_set_last_error("attention_decode_tma: cuTensorMapEncodeTiled failed or is not available");
        return MM_ERR_DRIVER;
    }
    cudaStream_t s = (cudaStream_t)stream;
#define MM_DT(HDV, ST, CL) launch_decode_tma<HDV, ST, CL>(tk, tv, q, out, part_o, part_ml, items, n_items, positions, token_req, block_table, \
                                                          table_width, page_size, H, G, window, scale, split_len, max_splits, (int*)err, s)
    if (cluster) return hd == 128 ? MM_DT(128, 3, true) : MM_DT(64, 3, true);
    if (hd == 128) return stages == 3 ? MM_DT(128, 3, false) : MM_DT(128, 6, false);
    return stages == 3 ? MM_DT(64, 3, false) : MM_DT(64, 6, false);
#undef MM_DT
}

// Clusters of `cluster_size` (2..8) CTAs of the cluster variant that fit on the current device at the same time; a
// launch with more clusters than this runs in waves.
MM_EXPORT int mm_attention_decode_tma_max_clusters(int hd, int cluster_size, int* out) {
    MM_REQUIRE(hd == 64 || hd == 128, "attention_decode_tma: built for head_dim 64 and 128");
    MM_REQUIRE(cluster_size >= 2 && cluster_size <= 8 && out != nullptr, "attention_decode_tma: cluster size must be 2..8");
    return hd == 128 ? max_active_clusters<128>(cluster_size, out) : max_active_clusters<64>(cluster_size, out);
}
