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

// The epilogue of one warp for its 32 rows (TMEM lanes) of a 128 x 256 accumulator at `taddr`: rows m0 + 32 q + lane,
// columns n0 .. n0 + 255 of the product.
template <int EPI>
__device__ __forceinline__ void epilogue_rows(uint32_t taddr, int m0, int n0, int q, int lane, unsigned char* wstage,
                                              void* __restrict__ out, const void* __restrict__ bias, int bias_dtype, int M,
                                              int N, int ldo) {
    const int row = m0 + q * 32 + lane;
    if (EPI == EPI_F32) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            const int col0 = n0 + c * 32;
            if (col0 >= N) break;                      // uniform over the warp
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
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
