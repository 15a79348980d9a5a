// y[M,N] = x[M,K] * W[N,K]^T for 9..128 rows of x (decode batches, short prompt portions): weight streaming on
// the fifth-generation tensor cores.  The operands are swapped: a 128-row tile of W is the 128-row operand of
// tcgen05.mma, the (zero-padded) batch is its N dimension (16..128), so every weight byte is fetched once, by TMA
// (cp.async.bulk.tensor, 16 KB boxes, 128-byte swizzle) into an mbarrier ring, and the accumulator [128 weight
// rows x batch] lives in tensor memory.
//
// Products with few weight rows (N = hidden) split K over a thread-block cluster of 2, 4 or 8 CTAs: every CTA owns
// a slice of the tile's rows; each CTA stores its partial sums for a slice straight into the owner's shared memory
// (distributed shared memory stores, nobody waits for a remote load), and after one cluster barrier the owner adds
// the S pieces in rank order (deterministic) and finishes its slice.
//
// The ring is as deep as shared memory allows when the grid has at most one CTA per SM (few tiles: the bytes in
// flight per SM are what bounds the stream), and shallow enough for two CTAs per SM otherwise.
//
// Epilogues, per unit of (batch row, 16 weight rows), the same four as the weight-streaming GEMV of gemv_bf16.cu
// and with the same weight layouts, so a decode layer is five launches at these batch sizes too:
//   PLAIN   bias; fp32 or bf16 output
//   SWIGLU  rows interleave gate and up in blocks of 8; writes silu(gate) * up
//   RESID   adds into the fp32 residual stream; with a norm weight also writes residual * weight (bf16) and the
//           unit's sum of squares (the next product applies 1/rms to its accumulators: `in_ss`)
//   ROPE    q/k/v projection: bias, rotation of q and k (rows interleave each head's halves in blocks of 8), q to
//           [M, H*hd], k and v into their cache pages
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2..5 epilogue.  Every mbarrier wait is
// bounded (tcgen05.cuh); after a time-out the roles fall through to the cluster barriers, which every thread of
// every CTA reaches on every path, and the error flag is set.
//
// The reference's counterparts: its scalar small-M bf16 product (kernels/cuda/common/matmul_bf16_gemm.cu, M <= 16) and
// the library route above that (src/compute/cuda/GpuMatmul.cpp:786-884).
#include "tcgen05.cuh"


#include <map>
#include <utility>

namespace {

using namespace tc;

constexpr int SK_ROWS = 128;            // weight rows per tile (the MMA's M)
constexpr int SK_BK = 64;               // k per stage: one 128-byte swizzled row
constexpr int SK_THREADS = 192;
constexpr int SK_A_BYTES = SK_ROWS * SK_BK * 2;

enum { SK_PLAIN = 0, SK_SWIGLU = 1, SK_RESID = 2, SK_ROPE = 3 };

struct SkinnyArgs {
    void* out;                  // PLAIN [M, ldo] bf16/fp32; SWIGLU [M, ldo] (N/2 columns)
    const void* bias;           // [N] or null (PLAIN, ROPE)
    int bias_dtype, out_dtype;
    int M, N, K, ldo;
    int S;                      // K splits = cluster size
    int stages;                 // depth of the TMA ring
    // deferred 1/rms of the input rows: partial sums of squares [in_tiles][ss_ld] (null: none)
    const float* in_ss;
    int in_tiles, in_dim, in_ld;
    float in_eps;
    // RESID
    float* residual;            // [M, N]
    const void* norm_w;         // [N] or null
    int norm_w_dtype;
    __nv_bfloat16* xw_out;      // [M, N]
    float* out_ss;              // [N / 16][out_ld]
    int out_ld;
    // ROPE
    __nv_bfloat16* q_out;       // [M, H * hd]
    __nv_bfloat16* k_pages;     // [pages, G, page_size, hd] or null
    __nv_bfloat16* v_pages;
    const float* rope_table;    // [M, hd]: cos then sin of the hd/2 angles
    const int32_t* slots;       // [M] or null
    int page_size, H, G, hd;
    int* err;
};

constexpr int SK_MAX_STAGES = 12;

long long g_sk_last_count = -1;            // the library's launch count right after the last launch from this file
cudaStream_t g_sk_last_stream = nullptr;

struct SkinnyCtl {
    uint64_t full[SK_MAX_STAGES];
    uint64_t empty[SK_MAX_STAGES];
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void sk_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t sk_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ float sk_w(const void* p, int dtype, int i) {
    return dtype == MM_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ uint32_t sk_pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void sk_store8_bf16(__nv_bfloat16* dst, const float* v) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(sk_pack2(v[0], v[1]), sk_pack2(v[2], v[3]), sk_pack2(v[4], v[5]), sk_pack2(v[6], v[7]));
}

// MP: batch rows the tile is padded to (the MMA's N and the accumulator's columns)
template <int MP, int EPI>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const SkinnyArgs a) {
    constexpr int B_BYTES = MP * SK_BK * 2;
    constexpr int STAGE_BYTES = SK_A_BYTES + B_BYTES;
    constexpr int TMEM_COLS = MP < 32 ? 32 : MP;
    constexpr uint32_t IDESC = idesc_bf16(SK_ROWS, MP, false);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int STAGES = a.stages;
    unsigned char* ring = smem_raw;
    // recv[s][m][row of my slice]: the partial sums of K split s for the rows this CTA finishes.  With one split it
    // lies over the ring (only this CTA writes it, after its own products); with several it has memory of its own,
    // because a peer may be done, and store, while this CTA's products still read the ring.
    float* recv = reinterpret_cast<float*>(a.S == 1 ? ring : ring + STAGES * STAGE_BYTES);
    SkinnyCtl* ctl = reinterpret_cast<SkinnyCtl*>(ring + STAGES * STAGE_BYTES + (a.S == 1 ? 0 : MP * SK_ROWS * 4));
    float* in_scale = reinterpret_cast<float*>(ctl + 1);                 // [MP]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &ctl->abort_flag;

    const int tile = blockIdx.x;
    const int S = a.S;
    const int rank = S > 1 ? (int)sk_cluster_rank() : 0;
    const int n_tile0 = tile * SK_ROWS;
    const int k_blocks = (a.K + SK_BK - 1) / SK_BK;
    const int kb_per = (k_blocks + S - 1) / S;
    const int kb_begin = min(rank * kb_per, k_blocks), kb_end = min(kb_begin + kb_per, k_blocks);
    const int n_kb = kb_end - kb_begin;
    bool good = (smem_u32(smem_raw) & 1023u) == 0;
    if (!good && threadIdx.x == 0 && a.err != nullptr) atomicExch(a.err, 5);

    if (threadIdx.x == 32) {
        prefetch_tensormap(&tmW);
        prefetch_tensormap(&tmX);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        mbar_init(smem_u32(&ctl->acc_full), 1);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the first round of the ring needs nobody else: its copies go out before this CTA's other warps have
        // allocated tensor memory and met at the barrier
        if (good) {
            for (int i = 0; i < n_kb && i < STAGES; ++i) {
                const uint32_t full = smem_u32(&ctl->full[i]);
                mbar_expect_tx(full, STAGE_BYTES);
                tma_load_2d(smem_u32(ring + i * STAGE_BYTES), &tmW, (kb_begin + i) * SK_BK, n_tile0, full);
            }
        }
        // Launched dependently, this kernel may have started before the one ahead of it has finished: the weights above do
        // not depend on that kernel, the batch does.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (good) {
            for (int i = 0; i < n_kb && i < STAGES; ++i)
                tma_load_2d(smem_u32(ring + i * STAGE_BYTES) + SK_A_BYTES, &tmX, (kb_begin + i) * SK_BK, 0, smem_u32(&ctl->full[i]));
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        if (lane == 0 && good) {
            // ---- TMA producer: this CTA's k blocks of the weight tile and of the batch (after the first round) ----
            for (int i = STAGES; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1, abort_flag)) break;
                const uint32_t full = smem_u32(&ctl->full[s]);
                mbar_expect_tx(full, STAGE_BYTES);
                const uint32_t dst = smem_u32(ring + s * STAGE_BYTES);
                tma_load_2d(dst, &tmW, (kb_begin + i) * SK_BK, n_tile0, full);
                tma_load_2d(dst + SK_A_BYTES, &tmX, (kb_begin + i) * SK_BK, 0, full);
            }
        }
        // this CTA's weights have been asked for: a dependent kernel's blocks may move in and ask for theirs
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    } else if (warp == 1) {
        if (lane == 0 && good) {
            // ---- MMA issuer ----
            bool ok = true;
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (!mbar_wait(smem_u32(&ctl->full[s]), ph, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(ring + s * STAGE_BYTES);
                const uint64_t a_desc = smem_desc_sw128(a_addr, 16, 1024), b_desc = smem_desc_sw128(a_addr + SK_A_BYTES, 16, 1024);
#pragma unroll
                for (int k = 0; k < SK_BK / 16; ++k)
                    umma_bf16(tmem_base, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), IDESC, (i | k) ? 1u : 0u);
                umma_commit(smem_u32(&ctl->empty[s]));
            }
            if (ok) umma_commit(smem_u32(&ctl->acc_full));      // arrives when every product above has finished
        }
    } else {
        // ---- epilogue warps, part 1: 1/rms of the input rows while the weights stream, then the accumulator
        //      (TMEM lanes = weight rows, columns = batch rows) goes to shared memory as part[m][row] ----
        const int q = warp & 3, et = q * 32 + lane;               // 0..127
        if (a.in_ss != nullptr) {
            for (int m = et; m < a.M; m += 128) {
                float ssum = 0.0f;
                for (int j = 0; j < a.in_tiles; ++j) ssum += a.in_ss[(size_t)j * a.in_ld + m];
                in_scale[m] = 1.0f / sqrtf(ssum / (float)a.in_dim + a.in_eps);
            }
        }
        if (good && n_kb > 0) {
            if (!mbar_wait(smem_u32(&ctl->acc_full), 0, abort_flag)) good = false;
        }
        tc_fence_after();
        if (good) {
            // row `et` of the tile belongs to the slice of CTA et / R: its M partial sums go to that CTA's recv[rank]
            const int R = SK_ROWS / S;
            const int owner = et / R, rl = et - owner * R;
            uint32_t dst = smem_u32(recv + (size_t)rank * MP * R + rl);
            if (S > 1) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(dst) : "r"(dst), "r"(owner));
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < TMEM_COLS / 32; ++c) {
                if (c * 32 >= a.M) break;                          // uniform
                uint32_t r[32];
                if (n_kb > 0) {
                    tmem_ld32(taddr + c * 32, r);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                }
                if (S == 1) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < a.M) recv[(c * 32 + i) * SK_ROWS + et] = __uint_as_float(r[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < a.M)
                            asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(dst + (uint32_t)((c * 32 + i) * R) * 4u), "f"(__uint_as_float(r[i])) : "memory");
                }
            }
        } else if (lane == 0 && a.err != nullptr) {
            atomicExch(a.err, 1);
        }
        tc_fence_before();
    }

    // every split's partial sums for this CTA's slice are in its recv buffer
    __syncthreads();
    if (S > 1) sk_cluster_sync();

    if (warp >= 2 && *abort_flag == 0) {
        // ---- epilogue warps, part 2: this CTA's slice of the tile's rows, units of (batch row, 16 weight rows) ----
        const int et = (warp & 3) * 32 + lane;
        const int R = SK_ROWS / S, nb = R / 16;                   // rows and 16-row blocks of a slice
        const int row0 = rank * R;
        for (int u = et; u < a.M * nb; u += 128) {
            const int m = u / nb, b = u - m * nb;
            const int r_in_tile = row0 + b * 16;
            const int n0 = n_tile0 + r_in_tile;                  // first weight row (output column) of the unit
            if (n0 >= a.N) continue;
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.0f;
            for (int sp = 0; sp < S; ++sp) {                     // rank order: the sum does not depend on timing
                const float* piece = recv + ((size_t)sp * MP + m) * R + b * 16;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 t4 = *reinterpret_cast<const float4*>(piece + 4 * i);
                    v[4 * i] += t4.x; v[4 * i + 1] += t4.y; v[4 * i + 2] += t4.z; v[4 * i + 3] += t4.w;
                }
            }
            if (a.in_ss != nullptr) {
                const float sc = in_scale[m];
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] *= sc;
            }
            if constexpr (EPI == SK_PLAIN) {
                if (a.bias != nullptr) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] += sk_w(a.bias, a.bias_dtype, n0 + i);
                }
                if (a.out_dtype == MM_F32) {
                    float* o = (float*)a.out + (size_t)m * a.ldo + n0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(o + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                } else {
                    __nv_bfloat16* o = (__nv_bfloat16*)a.out + (size_t)m * a.ldo + n0;
                    sk_store8_bf16(o, v);
                    sk_store8_bf16(o + 8, v + 8);
                }
            } else if constexpr (EPI == SK_SWIGLU) {
                float act[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) act[i] = v[i] / (1.0f + expf(-v[i])) * v[8 + i];
                if (a.out_dtype == MM_F32) {
                    float* o = (float*)a.out + (size_t)m * a.ldo + n0 / 2;
                    *reinterpret_cast<float4*>(o) = make_float4(act[0], act[1], act[2], act[3]);
                    *reinterpret_cast<float4*>(o + 4) = make_float4(act[4], act[5], act[6], act[7]);
                } else {
                    sk_store8_bf16((__nv_bfloat16*)a.out + (size_t)m * a.ldo + n0 / 2, act);
                }
            } else if constexpr (EPI == SK_RESID) {
                float* res = a.residual + (size_t)m * a.N + n0;
                float sq = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 t4 = *reinterpret_cast<const float4*>(res + 4 * i);
                    v[4 * i] += t4.x; v[4 * i + 1] += t4.y; v[4 * i + 2] += t4.z; v[4 * i + 3] += t4.w;
                    *reinterpret_cast<float4*>(res + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
                if (a.norm_w != nullptr) {
                    float xw[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        sq = fmaf(v[i], v[i], sq);
                        xw[i] = v[i] * sk_w(a.norm_w, a.norm_w_dtype, n0 + i);
                    }
                    __nv_bfloat16* o = a.xw_out + (size_t)m * a.N + n0;
                    sk_store8_bf16(o, xw);
                    sk_store8_bf16(o + 8, xw + 8);
                    a.out_ss[(size_t)(n0 / 16) * a.out_ld + m] = sq;
                }
            } else {
                const int hd = a.hd, head = n0 / hd, within = n0 - head * hd;
                if (a.bias != nullptr) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] += sk_w(a.bias, a.bias_dtype, n0 + i);
                }
                __nv_bfloat16* dst = nullptr;
                if (head < a.H) {
                    dst = a.q_out + ((size_t)m * a.H + head) * hd;
                } else if (a.slots != nullptr && a.slots[m] >= 0) {
                    const bool is_v = head >= a.H + a.G;
                    const int g = head - a.H - (is_v ? a.G : 0);
                    const int slot = a.slots[m], page = slot / a.page_size, in_page = slot - page * a.page_size;
                    dst = (is_v ? a.v_pages : a.k_pages) + (((size_t)page * a.G + g) * a.page_size + in_page) * hd;
                }
                if (dst == nullptr) continue;
                if (head < a.H + a.G) {
                    // the block holds elements i0..i0+7 of the head's first half and their partners of the second half
                    const int i0 = within / 2;
                    const float* cs = a.rope_table + (size_t)m * hd;
                    float ra[8], rb[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float c = cs[i0 + i], sn = cs[hd / 2 + i0 + i];
                        ra[i] = v[i] * c - v[8 + i] * sn;
                        rb[i] = v[i] * sn + v[8 + i] * c;
                    }
                    sk_store8_bf16(dst + i0, ra);
                    sk_store8_bf16(dst + hd / 2 + i0, rb);
                } else {
                    sk_store8_bf16(dst + within, v);
                    sk_store8_bf16(dst + within + 8, v + 8);
                }
            }
        }
    }

    // ---- teardown (no CTA touches a peer's shared memory after the barrier above) ----
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);       // let copies and products in flight land
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0 && ctl->abort_flag && a.err != nullptr) atomicExch(a.err, 1);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int MP, int EPI>
int sk_launch(const CUtensorMap& tw, const CUtensorMap& tx, SkinnyArgs& a, cudaStream_t s) {
    constexpr int STAGE_BYTES = SK_A_BYTES + MP * SK_BK * 2;
    constexpr int RECV_BYTES = MP * SK_ROWS * 4;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = (a.N + SK_ROWS - 1) / SK_ROWS;
    const size_t fixed = sizeof(SkinnyCtl) + MP * sizeof(float) + (a.S > 1 ? RECV_BYTES : 0);
    // the kernel's shared-memory ceiling only ever goes up
    static size_t ceiling = 48 * 1024;
    auto allow = [&](size_t need) -> bool {
        if (need <= ceiling) return true;
        if (cudaFuncSetAttribute(gemm_skinny_kernel<MP, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        ceiling = need;
        return true;
    };
    // As deep a ring as shared memory allows if the whole grid is then still resident at once (few tiles: the bytes
    // in flight per SM bound the stream); else room for two CTAs per SM.  The answer per (tiles, splits) is kept.
    size_t budget = 110 * 1024;
    if (tiles * a.S <= sms) {
        static std::map<std::pair<int, int>, bool> deep_fits;
        const std::pair<int, int> key(tiles, a.S);
        auto it = deep_fits.find(key);
        if (it == deep_fits.end()) {
            int deep_stages = (int)((200 * 1024 - fixed) / STAGE_BYTES);
            deep_stages = deep_stages > SK_MAX_STAGES ? SK_MAX_STAGES : deep_stages;
            const size_t deep_smem = (size_t)deep_stages * STAGE_BYTES + fixed;
            bool fits = false;
            if (allow(deep_smem)) {
                cudaLaunchConfig_t probe = {};
                probe.gridDim = dim3(tiles, a.S);
                probe.blockDim = dim3(SK_THREADS);
                probe.dynamicSmemBytes = deep_smem;
                cudaLaunchAttribute pattr[1];
                pattr[0].id = cudaLaunchAttributeClusterDimension;
                pattr[0].val.clusterDim.x = 1;
                pattr[0].val.clusterDim.y = a.S;
                pattr[0].val.clusterDim.z = 1;
                probe.attrs = pattr;
                probe.numAttrs = 1;
                int clusters = 0;
                if (cudaOccupancyMaxActiveClusters(&clusters, gemm_skinny_kernel<MP, EPI>, &probe) == cudaSuccess) fits = clusters >= tiles;
                else cudaGetLastError();
            }
            it = deep_fits.emplace(key, fits).first;
        }
        if (it->second) budget = 200 * 1024;
    }
    int stages = (int)((budget - fixed) / STAGE_BYTES);
    if (a.S == 1 && stages * STAGE_BYTES < RECV_BYTES) stages = (RECV_BYTES + STAGE_BYTES - 1) / STAGE_BYTES;   // recv lies over the ring
    stages = stages < 2 ? 2 : (stages > SK_MAX_STAGES ? SK_MAX_STAGES : stages);
    a.stages = stages;
    const size_t smem = (size_t)stages * STAGE_BYTES + fixed;
    if (!allow(smem)) {
        mm_set_last_error("gemm_skinny: cannot reserve shared memory");
        return MM_ERR_LAUNCH;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, a.S);
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (a.S > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = a.S;          // the K splits of a tile are one cluster
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    // Directly behind another product of this file (a layer's products follow each other) the launch is a dependent one:
    // the blocks start as that kernel's blocks leave (shared memory lets no third block onto an SM), ask for their first
    // weights and wait for it to finish before they touch the batch.
    if (g_mm_pdl != 0 && g_sk_last_count == g_mm_launch_count && g_sk_last_stream == s) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<MP, EPI>, tw, tx, a);
    MM_CHECK_LAUNCH();
    g_sk_last_count = g_mm_launch_count;
    g_sk_last_stream = s;
    return MM_OK;
}

template <int EPI>
int sk_dispatch(const void* W, const void* x, int ldx, SkinnyArgs& a, cudaStream_t s) {
    const int mp = a.M <= 16 ? 16 : (a.M <= 32 ? 32 : (a.M <= 64 ? 64 : 128));
    CUtensorMap tw, tx;
    if (!tc::make_map_bf16(&tw, W, a.N, a.K, a.K, SK_ROWS) || !tc::make_map_bf16(&tx, x, a.M, a.K, ldx, mp)) {
        mm_set_last_error("gemm_skinny: cuTensorMapEncodeTiled failed or is not available");
        return MM_ERR_DRIVER;
    }
    switch (mp) {
        case 16: return sk_launch<16, EPI>(tw, tx, a, s);
        case 32: return sk_launch<32, EPI>(tw, tx, a, s);
        case 64: return sk_launch<64, EPI>(tw, tx, a, s);
        default: return sk_launch<128, EPI>(tw, tx, a, s);
    }
}

int sk_common(SkinnyArgs& a, const void* W, const void* x, int M, int N, int K, int ldx, int splits, const void* in_ss,
              int in_tiles, int in_dim, int in_ld, float in_eps, void* err) {
    MM_REQUIRE(M >= 1 && M <= 128, "gemm_skinny: M must be in 1..128");
    MM_REQUIRE(N > 0 && N % 16 == 0, "gemm_skinny: N must be a multiple of 16");
    MM_REQUIRE(K > 0 && K % 8 == 0 && ldx >= K && ldx % 8 == 0, "gemm_skinny: K and the row stride of x must be multiples of 8 (16-byte TMA rows)");
    MM_REQUIRE(((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x)) & 15) == 0, "gemm_skinny: pointers must be 16-byte aligned");
    MM_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "gemm_skinny: K splits must be 1, 2, 4 or 8");
    MM_REQUIRE(in_ss == nullptr || (in_tiles >= 1 && in_dim >= 1 && in_ld >= M && in_eps > 0.0f), "gemm_skinny: bad input-scale sizes");
    a = SkinnyArgs();
    a.M = M; a.N = N; a.K = K; a.S = splits;
    a.in_ss = (const float*)in_ss; a.in_tiles = in_tiles; a.in_dim = in_dim; a.in_ld = in_ld; a.in_eps = in_eps;
    a.err = (int*)err;
    return MM_OK;
}

}  // namespace

// out[M, ldo] = x[M, ldx(K)] * W[N,K]^T (+ bias), or with swiglu != 0: out[M, N/2] = silu(gate) * up for W rows
// interleaved gate/up in blocks of 8.  splits: K splits (cluster size).  in_ss (or null): partial sums of squares
// [in_tiles][in_ld] of the rows x was made from; row m of the product is scaled by 1/sqrt(sum/in_dim + in_eps).
// err: device int set non-zero if a bounded wait ran out.
MM_EXPORT int mm_gemm_skinny(const void* W, const void* x, const void* bias, int bias_dtype, void* out, int out_dtype, int M,
                             int N, int K, int ldx, int ldo, int splits, int swiglu, const void* in_ss, int in_tiles,
                             int in_dim, int in_ld, float in_eps, void* err, void* stream) {
    SkinnyArgs a;
    const int rc = sk_common(a, W, x, M, N, K, ldx, splits, in_ss, in_tiles, in_dim, in_ld, in_eps, err);
    if (rc != MM_OK) return rc;
    MM_REQUIRE(out_dtype == MM_F32 || out_dtype == MM_BF16, "gemm_skinny: out dtype must be float32 or bfloat16");
    MM_REQUIRE(!swiglu || (bias == nullptr && ldo >= N / 2), "gemm_skinny: the SwiGLU epilogue takes no bias and writes N/2 columns");
    MM_REQUIRE(swiglu || ldo >= N, "gemm_skinny: ldo too small");
    MM_REQUIRE(ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "gemm_skinny: output rows must be 16-byte aligned");
    a.out = out; a.out_dtype = out_dtype; a.ldo = ldo; a.bias = bias; a.bias_dtype = bias_dtype;
    cudaStream_t s = (cudaStream_t)stream;
    return swiglu ? sk_dispatch<SK_SWIGLU>(W, x, ldx, a, s) : sk_dispatch<SK_PLAIN>(W, x, ldx, a, s);
}

// residual[M, N] (fp32) += x * W^T.  With norm_w: also xw_out[M, N] = bf16(residual * norm_w) and
// out_ss[N/16][out_ld] = sums of squares of the new residual over each 16 columns (entry m of a row is batch row m).
MM_EXPORT int mm_gemm_skinny_residual(const void* W, const void* x, void* residual, const void* norm_w, int norm_w_dtype,
                                      void* xw_out, void* out_ss, int out_ld, int M, int N, int K, int ldx, int splits,
                                      const void* in_ss, int in_tiles, int in_dim, int in_ld, float in_eps, void* err,
                                      void* stream) {
    SkinnyArgs a;
    const int rc = sk_common(a, W, x, M, N, K, ldx, splits, in_ss, in_tiles, in_dim, in_ld, in_eps, err);
    if (rc != MM_OK) return rc;
    MM_REQUIRE(residual != nullptr && (reinterpret_cast<uintptr_t>(residual) & 15) == 0, "gemm_skinny: residual missing or not 16-byte aligned");
    MM_REQUIRE(norm_w == nullptr || (xw_out != nullptr && out_ss != nullptr && out_ld >= M && (reinterpret_cast<uintptr_t>(xw_out) & 15) == 0),
               "gemm_skinny: a norm weight needs both outputs");
    MM_REQUIRE(norm_w_dtype == MM_F32 || norm_w_dtype == MM_BF16, "gemm_skinny: norm weight dtype must be float32 or bfloat16");
    a.residual = (float*)residual; a.norm_w = norm_w; a.norm_w_dtype = norm_w_dtype;
    a.xw_out = (__nv_bfloat16*)xw_out; a.out_ss = (float*)out_ss; a.out_ld = out_ld;
    return sk_dispatch<SK_RESID>(W, x, ldx, a, (cudaStream_t)stream);
}

// q/k/v projection with bias, rotation and cache write; layouts as mm_gemv_bf16_qkv_rope.
MM_EXPORT int mm_gemm_skinny_qkv_rope(const void* W, const void* x, const void* bias, int bias_dtype, void* q_out,
                                      void* k_pages, void* v_pages, const void* rope_table, const void* slots,
                                      int page_size, int H, int G, int hd, int M, int K, int ldx, int splits,
                                      const void* in_ss, int in_tiles, int in_dim, int in_ld, float in_eps, void* err,
                                      void* stream) {
    MM_REQUIRE(H >= 1 && G >= 1 && hd >= 16 && hd % 16 == 0, "gemm_skinny qkv: head size must be a multiple of 16");
    SkinnyArgs a;
    const int rc = sk_common(a, W, x, M, (H + 2 * G) * hd, K, ldx, splits, in_ss, in_tiles, in_dim, in_ld, in_eps, err);
    if (rc != MM_OK) return rc;
    MM_REQUIRE(q_out != nullptr && rope_table != nullptr, "gemm_skinny qkv: q_out and the rotation table are needed");
    MM_REQUIRE((k_pages == nullptr) == (v_pages == nullptr), "gemm_skinny qkv: k_pages and v_pages go together");
    MM_REQUIRE(k_pages == nullptr || (slots != nullptr && page_size >= 1), "gemm_skinny qkv: a cache write needs the slots");
    MM_REQUIRE(((reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages)) & 15) == 0,
               "gemm_skinny qkv: outputs must be 16-byte aligned");
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.q_out = (__nv_bfloat16*)q_out; a.k_pages = (__nv_bfloat16*)k_pages; a.v_pages = (__nv_bfloat16*)v_pages;
    a.rope_table = (const float*)rope_table; a.slots = k_pages ? (const int32_t*)slots : nullptr;
    a.page_size = page_size > 0 ? page_size : 1; a.H = H; a.G = G; a.hd = hd;
    return sk_dispatch<SK_ROPE>(W, x, ldx, a, (cudaStream_t)stream);
}
