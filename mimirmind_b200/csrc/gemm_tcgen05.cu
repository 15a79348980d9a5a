// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the fifth-generation tensor cores of sm_100a:
// operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), products
// issued by one thread with tcgen05.mma (UMMA 128x256x16, cta_group::1), accumulators in
// tensor memory (two 256-column accumulators so the epilogue of one tile overlaps the main
// loop of the next), read back with tcgen05.ld by four epilogue warps.
//
// Persistent, warp-specialised: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue.  Tiles are walked M-fastest so that CTAs working at the same time
// share a weight tile in L2.
//
// Epilogues (fused, so the product's output makes one trip to memory):
//   0  store bf16 (+ bias)
//   1  SwiGLU: columns interleave gate and up in blocks of 8 (the fused gate/up weight);
//      writes silu(gate) * up, [M, N/2] bf16
//   2  store fp32 (+ bias)
//
// Two kernels.  The single-CTA one works on 128 x 256 tiles.  The pair kernel (cta_group::2) runs a cluster of two
// CTAs on a 256 x 256 tile: each CTA loads its 128 rows of A and 128 of the 256 weight rows, so a stage is 32 KB
// instead of 48 KB (six stages instead of four in flight, a third less traffic from L2 per product), the leader's
// thread issues tcgen05.mma.cta_group::2 for both, and each CTA's epilogue reads its own half of the accumulator
// from its own tensor memory.  Loads are plain per-CTA TMA copies (no multicast).
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel raises an abort
// flag that all roles watch, lets copies in flight land, frees its tensor memory, writes an
// error code to `err` and returns, so a fault in the pipeline can never hang the GPU.
//
// The reference's counterparts are its wmma 16x16x16 bf16 kernel, one warp per output tile and
// no pipelining (kernels/cuda/common/matmul_bf16_gemm_tc.cu:37-99), and its cuBLASLt route
// (src/compute/cuda/GpuMatmul.cpp:786-884).
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int EPI_STAGE_BYTES = 32 * 256;     // per epilogue warp: 32 rows of 128 bf16, staged so that global stores are whole rows
constexpr int GEMM_THREADS = 192;

enum { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_F32 = 2 };

// K-major tile written by TMA with the 128-byte swizzle: groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) { return smem_desc_sw128(smem_addr, 16, 1024); }

// fp32 accumulate, bf16 x bf16, both K-major, N = 256, M = 128
constexpr uint32_t IDESC = idesc_bf16(BM, BN, false);

__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    umma_bf16(d_tmem, a_desc, b_desc, IDESC, accumulate);
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

struct SharedCtl {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// Partial sums of a 128 x 256 accumulator travel between pairs of CTAs column by column (fp32 [256][128]): a thread
// owns a row, so the 32 lanes of a warp then write, and read, 32 consecutive floats of a column at a time.
// r[0..32) += columns c0 .. c0 + 31 of this thread's row, read past L1 (another SM wrote them).
__device__ __forceinline__ void add_partial(uint32_t* r, const float* p_col0_row) {
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __ldcg(p_col0_row + (size_t)i * BM));
}

// The same for n blocks `stride` floats apart, two blocks' loads in flight at a time, added in the order of the blocks
__device__ __forceinline__ void add_partials(uint32_t* r, const float* p, int n, size_t stride) {
    int pi = 0;
    for (; pi + 2 <= n; pi += 2) {
        float a[32], b[32];
        const float* pa = p + pi * stride;
        const float* pb = pa + stride;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            a[i] = __ldcg(pa + (size_t)i * BM);
            b[i] = __ldcg(pb + (size_t)i * BM);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint((__uint_as_float(r[i]) + a[i]) + b[i]);
    }
    if (pi < n) add_partial(r, p + pi * stride);
}

// One warp's 32 rows of a 128 x 256 accumulator, as they are, to `ws` (fp32 [256][128])
__device__ __forceinline__ void dump_rows(uint32_t taddr, int q, int lane, float* __restrict__ ws) {
    float* wcol = ws + q * 32 + lane;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
#pragma unroll
        for (int i = 0; i < 32; ++i) __stcg(wcol + (size_t)(c * 32 + i) * BM, __uint_as_float(r[i]));
    }
}

// The epilogue of one warp for its 32 rows (TMEM lanes) of a 128 x 256 accumulator at `taddr`: rows m0 + 32 q + lane,
// columns n0 .. n0 + 255 of the product.
template <int EPI>
__device__ __forceinline__ void epilogue_rows(uint32_t taddr, int m0, int n0, int q, int lane, unsigned char* wstage,
                                              void* __restrict__ out, const void* __restrict__ bias, int bias_dtype, int M,
                                              int N, int ldo, const float* partial = nullptr, int n_partial = 0,
                                              size_t partial_stride = 0) {
    const int row = m0 + q * 32 + lane;
    // `partial`: n_partial blocks (partial_stride floats apart) of fp32 [256][128] sums (column by column) that other
    // pairs of CTAs computed for K segments of this tile; added in their order
    const float* prow = partial ? partial + (q * 32 + lane) : nullptr;
    if (EPI == EPI_F32) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            const int col0 = n0 + c * 32;
            if (col0 >= N) break;                      // uniform over the warp
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
            add_partials(r, prow + (size_t)(c * 32) * BM, n_partial, partial_stride);
            if (row >= M) continue;
            float* o = (float*)out + (size_t)row * ldo + col0;
            for (int i = 0; i < 32 && col0 + i < N; ++i) {
                float v = __uint_as_float(r[i]);
                if (bias != nullptr) v += (bias_dtype == MM_F32) ? ((const float*)bias)[col0 + i] : __bfloat162float(((const __nv_bfloat16*)bias)[col0 + i]);
                o[i] = v;
            }
        }
    } else {
        // bf16 outputs: each thread owns a row of the accumulator, which would make every global store a
        // 64-byte piece of a different row.  The warp stages 128 output columns of its 32 rows in shared memory
        // (16-byte unit u of row r at u ^ (r & 15): conflict-free both ways) and then stores whole 256-byte rows.
        constexpr int GROUP_CHUNKS = (EPI == EPI_SWIGLU) ? 8 : 4;      // 32-column accumulator chunks per 128 outputs
        const int n_out = (EPI == EPI_SWIGLU) ? N / 2 : N;
#pragma unroll 1
        for (int grp = 0; grp < BN / 32 / GROUP_CHUNKS; ++grp) {
            if (n0 + grp * GROUP_CHUNKS * 32 >= N) break;              // uniform over the warp
#pragma unroll 1
            for (int cc = 0; cc < GROUP_CHUNKS; ++cc) {
                const int c = grp * GROUP_CHUNKS + cc;
                const int col0 = n0 + c * 32;
                if (col0 >= N) break;                                 // uniform over the warp
                uint32_t r[32];
                tmem_ld32(taddr + c * 32, r);
                add_partials(r, prow + (size_t)(c * 32) * BM, n_partial, partial_stride);
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                unsigned char* srow = wstage + lane * 256;
                if (EPI == EPI_BF16) {
                    if (bias != nullptr) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < N)
                                v[i] += (bias_dtype == MM_F32) ? ((const float*)bias)[col0 + i] : __bfloat162float(((const __nv_bfloat16*)bias)[col0 + i]);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        *reinterpret_cast<uint4*>(srow + (((cc * 4 + i) ^ (lane & 15)) << 4)) =
                            make_uint4(pack2(v[i * 8], v[i * 8 + 1]), pack2(v[i * 8 + 2], v[i * 8 + 3]), pack2(v[i * 8 + 4], v[i * 8 + 5]), pack2(v[i * 8 + 6], v[i * 8 + 7]));
                } else {
                    // columns: 8 gate, 8 up, 8 gate, 8 up  ->  16 outputs
                    float a[16];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        a[i] = silu_mul(v[i], v[8 + i]);
                        a[8 + i] = silu_mul(v[16 + i], v[24 + i]);
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i)
                        *reinterpret_cast<uint4*>(srow + (((cc * 2 + i) ^ (lane & 15)) << 4)) =
                            make_uint4(pack2(a[i * 8], a[i * 8 + 1]), pack2(a[i * 8 + 2], a[i * 8 + 3]), pack2(a[i * 8 + 4], a[i * 8 + 5]), pack2(a[i * 8 + 6], a[i * 8 + 7]));
                }
            }
            __syncwarp();
            const int out_base = (EPI == EPI_SWIGLU) ? n0 / 2 : n0 + grp * 128;
#pragma unroll 4
            for (int it = 0; it < 16; ++it) {
                const int r = it * 2 + (lane >> 4), u = lane & 15;
                const int grow = m0 + q * 32 + r, gcol = out_base + u * 8;
                if (grow < M && gcol < n_out)
                    *reinterpret_cast<uint4*>((__nv_bfloat16*)out + (size_t)grow * ldo + gcol) =
                        *reinterpret_cast<const uint4*>(wstage + r * 256 + ((u ^ (r & 15)) << 4));
            }
            __syncwarp();
        }
    }
}

template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ out,
                    const void* __restrict__ bias, int bias_dtype, int M, int N, int K, int ldo, int* __restrict__ err) {
    extern __shared__ unsigned char smem_raw[];
    // 128-byte swizzle wants 1024-byte aligned tiles
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + STAGES * STAGE_BYTES;                     // 4 epilogue warps x [32 rows][256 bytes]
    SharedCtl* ctl = reinterpret_cast<SharedCtl*>(staging + 4 * EPI_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &ctl->abort_flag;

    if (threadIdx.x == 32) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctl->tmem_empty[a]), 4);   // one arrival per epilogue warp
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN, k_blocks = (K + BK - 1) / BK;
    const int total = m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ----
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t full = smem_u32(&ctl->full[s]);
                    mbar_expect_tx(full, STAGE_BYTES);
                    const uint32_t a_dst = smem_u32(tiles + s * STAGE_BYTES);
                    tma_load_2d(a_dst, &tmA, kb * BK, m0, full);
                    tma_load_2d(a_dst + A_BYTES, &tmB, kb * BK, n0, full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++local) {
                const uint32_t acc = local & 1, acc_ph = (local >> 1) & 1;
                if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(smem_u32(&ctl->full[s]), ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
                    const uint64_t a_desc = make_desc(a_addr), b_desc = make_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advancing 16 elements (32 bytes) along K inside the swizzled row: +2 in the address field
                        umma(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), (kb | k) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&ctl->empty[s]));      // the stage is free once these products have read it
                }
                if (ok) umma_commit(smem_u32(&ctl->tmem_full[acc]));
            }
        }
    } else {
        // ---- epilogue: warp w reads TMEM lanes 32*(w%4) .. +31 ----
        const int q = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++local) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const uint32_t acc = local & 1, acc_ph = (local >> 1) & 1;
            if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            epilogue_rows<EPI>(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN, m0, n0, q, lane, staging + q * EPI_STAGE_BYTES,
                               out, bias, bias_dtype, M, N, ldo);
            // the accumulator may be overwritten once all four warps have read it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
        }
    }

    // ---- teardown ----
    if (*abort_flag) {
        // give copies and products in flight time to land before the tensor memory is given back
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0 && ctl->abort_flag && err != nullptr) atomicExch(err, 1);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The pair kernel: a cluster of two CTAs per 256 x 256 tile.
// ---------------------------------------------------------------------------------------------------------------
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_BYTES = 128 * BK * 2;                       // this CTA's half of the tile's 256 weight rows
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;         // 32 KB
constexpr uint32_t IDESC_PAIR = idesc_bf16(256, BN, false);      // M = 256 over the two CTAs

struct PairCtl {
    uint64_t full[PAIR_STAGES];      // the leader's count the bytes of both CTAs' loads
    uint64_t empty[PAIR_STAGES];     // each CTA's own, signalled by the leader's commit
    uint64_t tmem_full[2];           // each CTA's own, signalled by the leader's commit
    uint64_t tmem_empty[2];          // the leader's: eight arrivals, four epilogue warps of each CTA
    uint64_t epi_sync;               // stream-K: the four epilogue warps of this CTA meet here (a bounded wait, unlike bar.sync)
    uint32_t tmem_base;
    int abort_flag;
};

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ out,
                         const void* __restrict__ bias, int bias_dtype, int M, int N, int K, int ldo, int* __restrict__ err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + PAIR_STAGES * PAIR_STAGE_BYTES;
    PairCtl* ctl = reinterpret_cast<PairCtl*>(staging + 4 * EPI_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    volatile int* abort_flag = &ctl->abort_flag;
    const uint32_t peer_abort = map_to_rank(smem_u32(&ctl->abort_flag), rank ^ 1u);

    if (threadIdx.x == 32) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctl->tmem_empty[a]), 8);
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // one warp of each CTA of the pair takes part in the allocation; both get the same columns
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    pair_sync();                 // the peer's barriers exist before anything of this CTA signals them
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    const int m_tiles = (M + 255) / 256, n_tiles = (N + BN - 1) / BN, k_blocks = (K + BK - 1) / BK;
    const int total = m_tiles * n_tiles;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer of this CTA's halves; the bytes of both CTAs are counted on the leader's barrier ----
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < total && ok; tile += pairs) {
                const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * BN + (int)rank * 128;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t ph = (it / PAIR_STAGES) & 1;
                    if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1, abort_flag)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(smem_u32(&ctl->full[s]), 2 * PAIR_STAGE_BYTES);
                    const uint32_t full = map_to_rank(smem_u32(&ctl->full[s]), 0);
                    const uint32_t a_dst = smem_u32(tiles + s * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(a_dst, &tmA, kb * BK, m0, full);
                    tma_load_2d_pair(a_dst + A_BYTES, &tmB, kb * BK, n0, full);
                }
            }
            if (!ok) st_cluster_u32(peer_abort, 1u);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer for the pair ----
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < total && ok; tile += pairs, ++local) {
                const uint32_t acc = local & 1, acc_ph = (local >> 1) & 1;
                if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t ph = (it / PAIR_STAGES) & 1;
                    if (!mbar_wait(smem_u32(&ctl->full[s]), ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + s * PAIR_STAGE_BYTES);
                    const uint64_t a_desc = make_desc(a_addr), b_desc = make_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), IDESC_PAIR, (kb | k) ? 1u : 0u);
                    umma_commit_pair(smem_u32(&ctl->empty[s]), 3);      // frees the stage in both CTAs
                }
                if (ok) umma_commit_pair(smem_u32(&ctl->tmem_full[acc]), 3);
            }
            if (!ok) st_cluster_u32(peer_abort, 1u);
        }
    } else {
        // ---- epilogue of this CTA's 128 rows ----
        const int q = warp & 3;
        const uint32_t leader_empty0 = map_to_rank(smem_u32(&ctl->tmem_empty[0]), 0);
        const uint32_t leader_empty1 = map_to_rank(smem_u32(&ctl->tmem_empty[1]), 0);
        uint32_t local = 0;
        bool ok = true;
        for (int tile = pair; tile < total && ok; tile += pairs, ++local) {
            const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * BN;
            const uint32_t acc = local & 1, acc_ph = (local >> 1) & 1;
            if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            epilogue_rows<EPI>(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN, m0, n0, q, lane, staging + q * EPI_STAGE_BYTES,
                               out, bias, bias_dtype, M, N, ldo);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
        }
        if (!ok && lane == 0) st_cluster_u32(peer_abort, 1u);
    }

    // ---- teardown: neither CTA leaves, or gives its tensor memory back, while the other may still signal it ----
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    pair_sync();
    tc_fence_after();
    if (threadIdx.x == 0 && ctl->abort_flag && err != nullptr) atomicExch(err, 1);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The pair kernel for products whose tiles do not fill a whole number of rounds (2,048 x 3,584: 112 tiles for 74
// pairs).  Whole rounds run as in the pair kernel (tile = pair + round x pairs: pairs that run together work on
// neighbouring tiles and share operands in L2).  The k blocks of the tiles that are left form one sequence that the
// pairs share out evenly ("stream-K"), so every pair is busy to the end.  A tile of that part is cut between
// consecutive pairs: the pair that holds its first k blocks finishes it; the others write their accumulators to
// their slot of `ws` and raise their flag.  The finisher comes to the tile last in its share (the others come to it
// first), waits for their flags (bounded), adds their sums in the order of the pairs and runs the epilogue; the
// result does not depend on timing.  The flags are left at zero again.
// ---------------------------------------------------------------------------------------------------------------
constexpr int SK_FLAG_POLLS = 1 << 22;

struct StreamKPlan {
    int pairs, pair, rounds, tiles, KB;
    long long u0, u1;              // this pair's k blocks of the sequence over the left-over tiles
    __device__ void init(int m_tiles, int n_tiles, int kb, int pair_, int pairs_) {
        pairs = pairs_; pair = pair_; KB = kb;
        tiles = m_tiles * n_tiles;
        rounds = tiles / pairs;
        const long long units = (long long)(tiles - rounds * pairs) * KB;
        u0 = units * pair / pairs;
        u1 = units * (pair + 1) / pairs;
    }
    __device__ long long share_begin(int q) const { return (long long)(tiles - rounds * pairs) * KB * q / pairs; }
    // item number i of this pair: false when there is none
    __device__ bool item(int i, long long& pos, int& tile, int& kb0, int& kb1) const {
        if (i < rounds) {
            tile = pair + i * pairs; kb0 = 0; kb1 = KB;
            return true;
        }
        if (pos >= u1) return false;
        const int t = (int)(pos / KB);
        kb0 = (int)(pos - (long long)t * KB);
        const long long left = u1 - (long long)t * KB;
        kb1 = left < KB ? (int)left : KB;
        tile = rounds * pairs + t;
        pos = (long long)t * KB + kb1;
        return true;
    }
};

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_streamk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, void* __restrict__ out,
                            const void* __restrict__ bias, int bias_dtype, int M, int N, int K, int ldo, float* __restrict__ ws,
                            int* __restrict__ flags, int* __restrict__ err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + PAIR_STAGES * PAIR_STAGE_BYTES;
    PairCtl* ctl = reinterpret_cast<PairCtl*>(staging + 4 * EPI_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    volatile int* abort_flag = &ctl->abort_flag;
    const uint32_t peer_abort = map_to_rank(smem_u32(&ctl->abort_flag), rank ^ 1u);

    if (threadIdx.x == 32) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctl->tmem_empty[a]), 8);
        }
        mbar_init(smem_u32(&ctl->epi_sync), 4);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    pair_sync();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;

    const int m_tiles = (M + 255) / 256, n_tiles = (N + BN - 1) / BN;
    StreamKPlan plan;
    plan.init(m_tiles, n_tiles, (K + BK - 1) / BK, blockIdx.x >> 1, gridDim.x >> 1);
    const int KB = plan.KB, pair = plan.pair;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            long long pos = plan.u0;
            int tile, kb0, kb1;
            for (int i = 0; ok && plan.item(i, pos, tile, kb0, kb1); ++i) {
                const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * BN + (int)rank * 128;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t ph = (it / PAIR_STAGES) & 1;
                    if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1, abort_flag)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(smem_u32(&ctl->full[s]), 2 * PAIR_STAGE_BYTES);
                    const uint32_t full = map_to_rank(smem_u32(&ctl->full[s]), 0);
                    const uint32_t a_dst = smem_u32(tiles + s * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(a_dst, &tmA, kb * BK, m0, full);
                    tma_load_2d_pair(a_dst + A_BYTES, &tmB, kb * BK, n0, full);
                }
            }
            if (!ok) st_cluster_u32(peer_abort, 1u);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t it = 0;
            bool ok = true;
            long long pos = plan.u0;
            int tile, kb0, kb1;
            for (int i = 0; ok && plan.item(i, pos, tile, kb0, kb1); ++i) {
                const uint32_t acc = (uint32_t)i & 1, acc_ph = ((uint32_t)i >> 1) & 1;
                if (!mbar_wait(smem_u32(&ctl->tmem_empty[acc]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t ph = (it / PAIR_STAGES) & 1;
                    if (!mbar_wait(smem_u32(&ctl->full[s]), ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + s * PAIR_STAGE_BYTES);
                    const uint64_t a_desc = make_desc(a_addr), b_desc = make_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), IDESC_PAIR, (kb > kb0 || k) ? 1u : 0u);
                    umma_commit_pair(smem_u32(&ctl->empty[s]), 3);
                }
                if (ok) umma_commit_pair(smem_u32(&ctl->tmem_full[acc]), 3);
            }
            if (!ok) st_cluster_u32(peer_abort, 1u);
        }
    } else {
        const int q = warp & 3;
        const uint32_t leader_empty0 = map_to_rank(smem_u32(&ctl->tmem_empty[0]), 0);
        const uint32_t leader_empty1 = map_to_rank(smem_u32(&ctl->tmem_empty[1]), 0);
        uint32_t meet_ph = 0;
        bool ok = true;
        // the four epilogue warps meet (every wait in this kernel is bounded, so no bar.sync among a subset of warps)
        auto meet = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->epi_sync));
            const bool met = mbar_wait(smem_u32(&ctl->epi_sync), meet_ph, abort_flag);
            meet_ph ^= 1;
            return met;
        };
        long long pos = plan.u0;
        int tile, kb0, kb1;
        for (int i = 0; ok && plan.item(i, pos, tile, kb0, kb1); ++i) {
            const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * BN;
            const uint32_t acc = (uint32_t)i & 1, acc_ph = ((uint32_t)i >> 1) & 1;
            if (!mbar_wait(smem_u32(&ctl->tmem_full[acc]), acc_ph, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
            if (kb0 > 0) {
                // k blocks in the middle or at the end of a tile that another pair finishes: hand the sums over
                dump_rows(taddr, q, lane, ws + ((size_t)pair * 2 + rank) * BM * BN);
                __threadfence();
                if (!meet()) { ok = false; break; }
                if (q == 0 && lane == 0) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flags + pair * 2 + rank), "r"(1) : "memory");
            } else if (kb1 < KB) {
                // the first k blocks of a cut tile: the pairs after this one whose shares begin inside the tile hold the
                // rest; wait for their sums, add them in their order, finish
                const long long tile_end = (long long)(tile - plan.rounds * plan.pairs + 1) * KB;
                int others = 0;
                while (pair + 1 + others < plan.pairs && plan.share_begin(pair + 1 + others) < tile_end) ++others;
                if (q == 0 && lane == 0) {
                    for (int o = 0; o < others && !*abort_flag; ++o) {
                        const int* flag = flags + (pair + 1 + o) * 2 + rank;
                        int v = 0;
                        for (int polls = 0; polls < SK_FLAG_POLLS; ++polls) {
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                            if (v != 0 || *abort_flag) break;
                            __nanosleep(100);
                        }
                        if (v == 0) *abort_flag = 1;
                    }
                }
                if (!meet() || *abort_flag) { ok = false; break; }
                epilogue_rows<EPI>(taddr, m0, n0, q, lane, staging + q * EPI_STAGE_BYTES, out, bias, bias_dtype, M, N, ldo,
                                   ws + ((size_t)(pair + 1) * 2 + rank) * BM * BN, others, (size_t)2 * BM * BN);
                if (!meet()) { ok = false; break; }                            // all four warps have read the slots
                if (q == 0 && lane == 0)
                    for (int o = 0; o < others; ++o) flags[(pair + 1 + o) * 2 + rank] = 0;
            } else {
                epilogue_rows<EPI>(taddr, m0, n0, q, lane, staging + q * EPI_STAGE_BYTES, out, bias, bias_dtype, M, N, ldo);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
        }
        if (!ok && lane == 0) st_cluster_u32(peer_abort, 1u);
    }

    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    pair_sync();
    tc_fence_after();
    if (threadIdx.x == 0 && ctl->abort_flag && err != nullptr) atomicExch(err, 1);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ws: fp32 [pairs][2][128][256], flags: int32 [pairs + 1][2], zero before the first launch (the kernel leaves them zero)
template <int EPI>
int launch_streamk(const CUtensorMap& a, const CUtensorMap& b, void* out, const void* bias, int bias_dtype, int M, int N, int K,
                   int ldo, float* ws, int* flags, int pairs, int* err, cudaStream_t s) {
    const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 4 * EPI_STAGE_BYTES + 1024 + sizeof(PairCtl);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_streamk_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            mm_set_last_error("gemm_tcgen05: cannot reserve shared memory for the stream-K kernel");
            return MM_ERR_LAUNCH;
        }
        configured = true;
    }
    gemm_tcgen05_streamk_kernel<EPI><<<2 * pairs, GEMM_THREADS, smem, s>>>(a, b, out, bias, bias_dtype, M, N, K, ldo, ws, flags, err);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

template <int EPI>
int launch_pair(const CUtensorMap& a, const CUtensorMap& b, void* out, const void* bias, int bias_dtype, int M, int N, int K,
                int ldo, int* err, int max_ctas, cudaStream_t s) {
    const size_t smem = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 4 * EPI_STAGE_BYTES + 1024 + sizeof(PairCtl);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            mm_set_last_error("gemm_tcgen05: cannot reserve shared memory for the pair kernel");
            return MM_ERR_LAUNCH;
        }
        configured = true;
    }
    const int total = ((M + 255) / 256) * ((N + BN - 1) / BN);
    const int max_pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
    const int pairs = total < max_pairs ? total : max_pairs;
    gemm_tcgen05_pair_kernel<EPI><<<2 * pairs, GEMM_THREADS, smem, s>>>(a, b, out, bias, bias_dtype, M, N, K, ldo, err);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

template <int EPI>
int launch(const CUtensorMap& a, const CUtensorMap& b, void* out, const void* bias, int bias_dtype, int M, int N, int K,
           int ldo, int* err, int max_ctas, cudaStream_t s) {
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 4 * EPI_STAGE_BYTES + 1024 + sizeof(SharedCtl);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            mm_set_last_error("gemm_tcgen05: cannot reserve shared memory");
            return MM_ERR_LAUNCH;
        }
        configured = true;
    }
    const int total = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = total < max_ctas ? total : max_ctas;
    gemm_tcgen05_kernel<EPI><<<grid, GEMM_THREADS, smem, s>>>(a, b, out, bias, bias_dtype, M, N, K, ldo, err);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

}  // namespace

// A [M, lda] bf16 (K leading columns used), W [N, K] bf16, out [M, ldo] (bf16, fp32, or with the SwiGLU epilogue bf16
// [M, N/2]).  `err`: device int set to 1 if a bounded wait ran out (may be null).  `pair`: the cta_group::2 kernel.
static int gemm_tcgen05_common(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue, int M,
                               int N, int K, int lda, int ldo, void* err, void* stream, bool pair) {
    MM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes");
    MM_REQUIRE(K % 8 == 0 && lda % 8 == 0 && lda >= K, "gemm_tcgen05: K and the row stride of A must be multiples of 8 (16-byte TMA rows)");
    MM_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)out & 15) == 0, "gemm_tcgen05: pointers must be 16-byte aligned");
    MM_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tcgen05: unknown epilogue");
    MM_REQUIRE(epilogue != EPI_SWIGLU || (N % 16 == 0 && bias == nullptr && ldo >= N / 2), "gemm_tcgen05: the SwiGLU epilogue needs N a multiple of 16 and no bias");
    MM_REQUIRE(ldo % 8 == 0 && (epilogue == EPI_SWIGLU || ldo >= N), "gemm_tcgen05: the row stride of the output must be a multiple of 8 and at least N");
    CUtensorMap ta, tb;
    if (!tc::make_map_bf16(&ta, A, M, K, lda, BM) || !tc::make_map_bf16(&tb, W, N, K, K, pair ? 128 : BN)) {
        mm_set_last_error("gemm_tcgen05: cuTensorMapEncodeTiled failed or is not available");
        return MM_ERR_DRIVER;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaStream_t s = (cudaStream_t)stream;
    if (pair) {
        if (epilogue == EPI_BF16) return launch_pair<EPI_BF16>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (int*)err, sms, s);
        if (epilogue == EPI_SWIGLU) return launch_pair<EPI_SWIGLU>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (int*)err, sms, s);
        return launch_pair<EPI_F32>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (int*)err, sms, s);
    }
    if (epilogue == EPI_BF16) return launch<EPI_BF16>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (int*)err, sms, s);
    if (epilogue == EPI_SWIGLU) return launch<EPI_SWIGLU>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (int*)err, sms, s);
    return launch<EPI_F32>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (int*)err, sms, s);
}

MM_EXPORT int mm_gemm_tcgen05(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue, int M,
                              int N, int K, int lda, int ldo, void* err, void* stream) {
    return gemm_tcgen05_common(A, W, bias, bias_dtype, out, epilogue, M, N, K, lda, ldo, err, stream, false);
}

MM_EXPORT int mm_gemm_tcgen05_pair(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue, int M,
                                   int N, int K, int lda, int ldo, void* err, void* stream) {
    return gemm_tcgen05_common(A, W, bias, bias_dtype, out, epilogue, M, N, K, lda, ldo, err, stream, true);
}


// The stream-K kernel.  pairs: CTA pairs to launch (at most half the SMs); ws: fp32 scratch of pairs * 2 * 128 * 256 floats; flags: (pairs + 1) * 2 int32,
// zero before the first launch.
MM_EXPORT int mm_gemm_tcgen05_streamk(const void* A, const void* W, const void* bias, int bias_dtype, void* out, int epilogue,
                                      int M, int N, int K, int lda, int ldo, void* ws, void* flags, int pairs, void* err,
                                      void* stream) {
    MM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes");
    MM_REQUIRE(K % 8 == 0 && lda % 8 == 0 && lda >= K, "gemm_tcgen05: K and the row stride of A must be multiples of 8 (16-byte TMA rows)");
    MM_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)ws & 15) == 0, "gemm_tcgen05: pointers must be 16-byte aligned");
    MM_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tcgen05: unknown epilogue");
    MM_REQUIRE(epilogue != EPI_SWIGLU || (N % 16 == 0 && bias == nullptr && ldo >= N / 2), "gemm_tcgen05: the SwiGLU epilogue needs N a multiple of 16 and no bias");
    MM_REQUIRE(ldo % 8 == 0 && (epilogue == EPI_SWIGLU || ldo >= N), "gemm_tcgen05: the row stride of the output must be a multiple of 8 and at least N");
    MM_REQUIRE(ws != nullptr && flags != nullptr && pairs >= 1, "gemm_tcgen05: the stream-K kernel needs its scratch");
    {
        // a pair's share of the left-over tiles must hold at least one k block (else some pairs have nothing to hand over
        // or finish, which is fine) and a tile may be cut among many pairs, but never more than there are flags
        const long long KB = (K + BK - 1) / BK, tiles = (long long)((M + 255) / 256) * ((N + BN - 1) / BN);
        const long long left = tiles % pairs;
        MM_REQUIRE(left == 0 || left * KB >= pairs, "gemm_tcgen05: too few k blocks in the left-over tiles for every pair to get one");
    }
    CUtensorMap ta, tb;
    if (!tc::make_map_bf16(&ta, A, M, K, lda, BM) || !tc::make_map_bf16(&tb, W, N, K, K, 128)) {
        mm_set_last_error("gemm_tcgen05: cuTensorMapEncodeTiled failed or is not available");
        return MM_ERR_DRIVER;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == EPI_BF16) return launch_streamk<EPI_BF16>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (float*)ws, (int*)flags, pairs, (int*)err, s);
    if (epilogue == EPI_SWIGLU) return launch_streamk<EPI_SWIGLU>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (float*)ws, (int*)flags, pairs, (int*)err, s);
    return launch_streamk<EPI_F32>(ta, tb, out, bias, bias_dtype, M, N, K, ldo, (float*)ws, (int*)flags, pairs, (int*)err, s);
}
