// y[M,N] = x[M,K] * W[N,K]^T for a handful of rows (M <= 16): the decode-time matrix
// products, which are pure weight streaming.  Each weight element is read from HBM exactly
// once, with 16-byte loads straight into registers, and multiplied on the tensor cores
// (mma.sync m16n8k16, the weight rows as the 16-row operand, the batch rows as the 8 columns).
//
// Trick that makes the register loads line up with the mma fragments: a dot product does
// not care in which order k is visited, so the kernel lets thread t of a quad own the 8
// consecutive k values [kb + 8t, kb + 8t + 8) of a 32-wide k block for both operands and
// feeds them to two mma steps; the mma's own idea of "k index" is a permutation of memory
// order that is the same for W and x, so the sum is unchanged.
//
// A CTA has 8 warps arranged as RT row tiles (16 weight rows each) x KS splits of K; the
// splits of one row tile are summed through shared memory in a fixed order.  x is read from
// global memory through L1 (it is small and stays in L2; a copy per CTA into shared memory
// measured slower).  Loads are software-pipelined two batches deep in registers.
// Epilogues (one template instance each), chosen so that a decode layer is five launches:
//   PLAIN   bias; fp32 or bf16 output.
//   SWIGLU  the weight rows interleave gate and up in blocks of 8 (rows 16j..16j+7 = gate[8j..],
//           rows 16j+8..16j+15 = up[8j..]): one thread holds a gate value and its up value.
//   RESID   the product is added to the fp32 residual stream in place; if a norm weight is given,
//           the rows of residual * weight (bf16) and, per 16-column tile, the partial sums of
//           squares of the new residual are written too: RMSNorm(x) = (x * w) / rms(x), and the
//           1/rms factor commutes with the next matrix product, which applies it (below).
//   ROPE    q/k/v projection: bias, rotary position encoding of q and k (split-half pairs; the
//           weight rows of each q and k head interleave the two halves in blocks of 8, so a thread
//           holds a pair), q written as [M, H * hd], k and v written into their cache pages.
// Two builds (MINB = resident blocks per SM the compiler is asked for): 3 with 80 registers a thread, 2 with more and
// nothing spilled; the launch code takes the second when the grid has at most two blocks per SM.  Launched directly behind
// another launch of this kernel, a launch is a dependent one (common.cuh): the first weight loads go out before the wait.
// Input row scale: with `in_ss` the accumulators of row m are multiplied by
// 1 / sqrt(sum_j in_ss[j][m] / in_dim + eps) before the epilogue (the deferred 1/rms of RESID).
//
// The reference's counterparts are its bf16 GEMV and small-M GEMM
// (kernels/cuda/common/matmul_bf16_vec.cu:53-99: warp per output row, M launches;
// matmul_bf16_gemm.cu: scalar, M <= 16).
#include "common.cuh"

#define GEMV_THREADS 256
#define GEMV_WARPS 8

struct GemvArgs {
    const __nv_bfloat16* W;
    const __nv_bfloat16* x;
    const void* bias;
    void* out;
    int M, N, K, ldx, ldo;
    int bias_dtype, out_dtype;
    int RT, KS;
    // deferred 1/rms of the input rows (null: none): partial sums of squares [in_tiles][16]
    const float* in_ss;
    int in_tiles, in_dim;
    float in_eps;
    // RESID
    float* residual;            // [M, N] fp32, updated in place
    const void* norm_w;         // [N] or null
    int norm_w_dtype;
    __nv_bfloat16* xw_out;      // [M, N]
    float* out_ss;              // [N / 16][16]
    // ROPE
    __nv_bfloat16* q_out;       // [M, H * hd]
    __nv_bfloat16* k_pages;     // [pages, G, page_size, hd] or null
    __nv_bfloat16* v_pages;
    const float* rope_table;    // [M, hd]: cos of the hd/2 angles of the row's position, then their sin
    const int32_t* slots;       // [M]: page * page_size + place in the page of the row's position, or -1 (null: no cache write)
    int page_size, H, G, hd;
};

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_ROPE = 3 };

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// activations were written by the kernel before this one: plain loads, never .nc
__device__ __forceinline__ uint4 ld_act(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// shared memory of a CTA, reused by every item and phase
struct GemvSmem {
    float red[GEMV_WARPS][32][8];                 // K-split partial sums (4 floats per batch tile)
    float in_scale[16];                           // 1/rms of the input rows
    __align__(16) float stage_a[GEMV_WARPS * 16 * 16];   // RESID: residual [rt][m][16 cols]; ROPE: cos[8], sin[8] per [rt][m]
    __align__(16) float stage_b[GEMV_WARPS * 16];        // RESID: norm weights [rt][16]; ROPE: bias [rt][16]
    int slot_s[16];                               // ROPE: cache slot of each row
};

template <int U>
struct GemvFirst {                                // the first batch of weight loads of an item, issued ahead of its turn
    uint4 lo[U], hi[U];
};

// this warp's place in an item: row tile, K split, its 32-wide k blocks
struct GemvPlace {
    int rt, ks, n0, kb_begin, kb_count;
    bool active;
};
__device__ __forceinline__ GemvPlace gemv_place(const GemvArgs& a, int item) {
    GemvPlace p;
    const int warp = threadIdx.x >> 5;
    p.rt = warp / a.KS;
    p.ks = warp - p.rt * a.KS;
    p.n0 = (item * a.RT + p.rt) * 16;
    p.active = p.n0 < a.N;
    const int nkb = a.K / 32, base = nkb / a.KS, rem = nkb % a.KS;
    p.kb_begin = p.ks * base + min(p.ks, rem);
    p.kb_count = base + (p.ks < rem ? 1 : 0);
    return p;
}

template <int U>
__device__ __forceinline__ void gemv_first_weights(const GemvArgs& a, int item, GemvFirst<U>& f) {
    const GemvPlace p = gemv_place(a, item);
    const int lane = threadIdx.x & 31, t = lane & 3, r = lane >> 2;
    const __nv_bfloat16* wlo = a.W + (size_t)(p.n0 + r) * a.K + (size_t)p.kb_begin * 32 + t * 8;
    const __nv_bfloat16* whi = wlo + (size_t)8 * a.K;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        if (p.active && u < p.kb_count) {
            f.lo[u] = ldg_stream(wlo + (size_t)u * 32);
            f.hi[u] = ldg_stream(whi + (size_t)u * 32);
        } else {
            f.lo[u] = make_uint4(0, 0, 0, 0);
            f.hi[u] = make_uint4(0, 0, 0, 0);
        }
    }
}

// One work item (RT row tiles of 16 weight rows, all of K) of one product, by the whole CTA.  `first` holds the
// item's first weight batch, already requested.  Ends with the item's results written to global memory; the
// caller separates items that share `sm` by a CTA barrier.
template <int NT, int U, int EPI>
__device__ __forceinline__ void gemv_item(const GemvArgs& a, int item, const GemvFirst<U>& first, GemvSmem& sm, float* ss_s) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = lane & 3, r = lane >> 2;
    const int K = a.K;
    const GemvPlace pl = gemv_place(a, item);
    const int rt = pl.rt, ks = pl.ks, n0 = pl.n0;
    const bool active = pl.active;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    // Small operands of the epilogue are copied to shared memory with cp.async while the weights stream (no register
    // is held and no warp waits for them before the epilogue):
    //   every EPI  the producer's partial sums of squares of the input rows, [in_tiles][M4] (dynamic shared memory)
    //   RESID      the residual values [rt][m][16 cols] and the norm weights [rt][16] of this CTA's columns
    //   ROPE       cos and sin [rt][m][8] of every (row, pair) of this CTA's tiles, the bias [rt][16], each row's slot
    constexpr bool kStaged = (EPI == EPI_RESID || EPI == EPI_ROPE);
    float* stage_a = sm.stage_a;
    float* stage_b = sm.stage_b;
    int* slot_s = sm.slot_s;
    const int M4 = (a.M + 3) & ~3;
    auto stage = [&]() {
        if (a.in_ss != nullptr) {
            const int per = M4 / 4;                                   // 16-byte pieces per tile
            for (int idx = threadIdx.x; idx < a.in_tiles * per; idx += GEMV_THREADS) {
                const int j = idx / per, c = idx - j * per;
                cp_async16(&ss_s[j * M4 + c * 4], a.in_ss + j * 16 + c * 4);
            }
        }
        if constexpr (EPI == EPI_RESID) {
            for (int idx = threadIdx.x; idx < a.RT * 64; idx += GEMV_THREADS) {     // (tile, row, 4 columns)
                const int ti = idx >> 6, m = (idx >> 2) & 15, c4 = idx & 3;
                const int col = (item * a.RT + ti) * 16 + c4 * 4;
                if (m < a.M && col < a.N) cp_async16(&stage_a[(ti * 16 + m) * 16 + c4 * 4], a.residual + (size_t)m * a.N + col);
            }
            if (a.norm_w != nullptr) {
                const int bytes16 = (a.norm_w_dtype == MM_F32) ? 4 : 2;             // 16-byte pieces per tile
                for (int idx = threadIdx.x; idx < a.RT * bytes16; idx += GEMV_THREADS) {
                    const int ti = idx / bytes16, c = idx - ti * bytes16;
                    const int col = (item * a.RT + ti) * 16;
                    if (col < a.N)
                        cp_async16(reinterpret_cast<char*>(&stage_b[ti * 16]) + c * 16,
                                   reinterpret_cast<const char*>(a.norm_w) + (size_t)col * (a.norm_w_dtype == MM_F32 ? 4 : 2) + c * 16);
                }
            }
        }
        if constexpr (EPI == EPI_ROPE) {
            for (int idx = threadIdx.x; idx < a.RT * 64; idx += GEMV_THREADS) {     // (tile, row, cos|sin, 4 pairs)
                const int ti = idx >> 6, m = (idx >> 2) & 15, part = idx & 3;
                const int tile0 = (item * a.RT + ti) * 16;
                const int head = tile0 / a.hd, within = tile0 - head * a.hd;
                if (m < a.M && tile0 < a.N && head < a.H + a.G)
                    cp_async16(&stage_a[(ti * 16 + m) * 16 + part * 4],
                               a.rope_table + (size_t)m * a.hd + (part >> 1) * (a.hd / 2) + within / 2 + (part & 1) * 4);
            }
            if (a.bias != nullptr) {
                const int bytes16 = (a.bias_dtype == MM_F32) ? 4 : 2;
                for (int idx = threadIdx.x; idx < a.RT * bytes16; idx += GEMV_THREADS) {
                    const int ti = idx / bytes16, c = idx - ti * bytes16;
                    const int row = (item * a.RT + ti) * 16;
                    if (row < a.N)
                        cp_async16(reinterpret_cast<char*>(&stage_b[ti * 16]) + c * 16,
                                   reinterpret_cast<const char*>(a.bias) + (size_t)row * (a.bias_dtype == MM_F32 ? 4 : 2) + c * 16);
                }
            }
            if (threadIdx.x < 16) slot_s[threadIdx.x] = (threadIdx.x < a.M && a.slots != nullptr) ? a.slots[threadIdx.x] : -1;
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    auto staged_f32 = [&](const float* base, int dtype, int i) -> float {
        return dtype == MM_F32 ? base[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
    };

    if (active) {
        const int kb_count = pl.kb_count;
        const __nv_bfloat16* wlo = a.W + (size_t)(n0 + r) * K + (size_t)pl.kb_begin * 32 + t * 8;
        const __nv_bfloat16* whi = wlo + (size_t)8 * K;
        const __nv_bfloat16* xg[NT];
        bool xok[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int n = j * 8 + r;
            xok[j] = n < a.M;
            xg[j] = a.x + (size_t)(xok[j] ? n : 0) * a.ldx + (size_t)pl.kb_begin * 32 + t * 8;
        }
        // Two register buffers: the loads of the next U k-blocks are issued before the mma of the
        // current ones, so a warp always has a full batch of loads in flight.
        uint4 alo[2][U], ahi[2][U], xb[2][U][NT];
        auto load_w = [&](int buf, int kb) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (kb + u < kb_count) {
                    alo[buf][u] = ldg_stream(wlo + (size_t)(kb + u) * 32);
                    ahi[buf][u] = ldg_stream(whi + (size_t)(kb + u) * 32);
                } else {
                    alo[buf][u] = make_uint4(0, 0, 0, 0);
                    ahi[buf][u] = make_uint4(0, 0, 0, 0);
                }
            }
        };
        auto load_x = [&](int buf, int kb) {
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int j = 0; j < NT; ++j)
                    xb[buf][u][j] = (kb + u < kb_count && xok[j]) ? ld_act(xg[j] + (size_t)(kb + u) * 32) : make_uint4(0, 0, 0, 0);
        };
        auto mma_batch = [&](int buf, int kb) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint4 xv = xb[buf][u][j];
                    mma_16816(acc[j], alo[buf][u].x, ahi[buf][u].x, alo[buf][u].y, ahi[buf][u].y, xv.x, xv.y);
                    mma_16816(acc[j], alo[buf][u].z, ahi[buf][u].z, alo[buf][u].w, ahi[buf][u].w, xv.z, xv.w);
                }
            }
        };
#pragma unroll
        for (int u = 0; u < U; ++u) {
            alo[0][u] = first.lo[u];
            ahi[0][u] = first.hi[u];
        }
        load_x(0, 0);
        stage();
        for (int kb = 0; kb < kb_count; kb += 2 * U) {
            load_w(1, kb + U);
            load_x(1, kb + U);
            mma_batch(0, kb);
            load_w(0, kb + 2 * U);
            load_x(0, kb + 2 * U);
            mma_batch(1, kb + U);
        }
    } else {
        stage();
    }
    // the weights are through: the next kernel's blocks may move in beside this one's epilogue and request theirs
    pdl_trigger();
    asm volatile("cp.async.wait_all;\n" ::: "memory");
    // sum the K splits of each row tile in a fixed order
    const bool need_sync = a.KS > 1 || a.in_ss != nullptr || kStaged;
    if (a.KS > 1) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sm.red[warp][lane][j * 4 + e] = acc[j][e];
    }
    if (need_sync) __syncthreads();
    if (a.in_ss != nullptr) {
        // 1/rms of the input rows: thread (m, part) adds every 16th partial of row m, a shuffle tree adds the 16 parts
        const int m = threadIdx.x >> 4, part = threadIdx.x & 15;
        float ssum = 0.0f;
        if (m < a.M)
            for (int j = part; j < a.in_tiles; j += 16) ssum += ss_s[j * M4 + m];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
        if (part == 0) sm.in_scale[m] = 1.0f / sqrtf(ssum / (float)a.in_dim + a.in_eps);
        __syncthreads();
    }
    if (a.KS > 1 && ks == 0) {
        for (int sI = 1; sI < a.KS; ++sI)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][e] += sm.red[warp + sI][lane][j * 4 + e];
    }
    if (!active || ks != 0) return;

    // acc[j] = {(row r, col 2t), (row r, col 2t+1), (row r+8, col 2t), (row r+8, col 2t+1)} of batch tile j
    if (a.in_ss != nullptr) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float sc = sm.in_scale[j * 8 + t * 2 + e];
                acc[j][e] *= sc;
                acc[j][2 + e] *= sc;
            }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int m = j * 8 + t * 2 + e;
            const bool live = m < a.M;
            if constexpr (EPI == EPI_SWIGLU) {
                if (!live) continue;
                const float g = acc[j][e], u = acc[j][2 + e];
                const float v = g / (1.0f + expf(-g)) * u;
                const size_t o = (size_t)m * a.ldo + n0 / 2 + r;
                if (a.out_dtype == MM_F32) ((float*)a.out)[o] = v; else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(v);
            } else if constexpr (EPI == EPI_RESID) {
                float sq = 0.0f;
                if (live) {
#pragma unroll
                    for (int hi = 0; hi < 2; ++hi) {
                        const int c = r + hi * 8, col = n0 + c;
                        const size_t o = (size_t)m * a.N + col;
                        const float v = stage_a[(rt * 16 + m) * 16 + c] + acc[j][hi * 2 + e];
                        a.residual[o] = v;
                        if (a.norm_w != nullptr) {
                            a.xw_out[o] = __float2bfloat16_rn(v * staged_f32(&stage_b[rt * 16], a.norm_w_dtype, c));
                            sq = fmaf(v, v, sq);
                        }
                    }
                }
                // the 16 columns of this tile for row m: lanes with the same t (every r)
                sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                sq += __shfl_xor_sync(0xffffffffu, sq, 16);
                if (live && r == 0 && a.norm_w != nullptr) a.out_ss[(n0 / 16) * 16 + m] = sq;
            } else if constexpr (EPI == EPI_ROPE) {
                if (!live) continue;
                const int hd = a.hd, head = n0 / hd, within = n0 - head * hd;
                float x1 = acc[j][e], x2 = acc[j][2 + e];
                if (a.bias) {
                    x1 += staged_f32(&stage_b[rt * 16], a.bias_dtype, r);
                    x2 += staged_f32(&stage_b[rt * 16], a.bias_dtype, 8 + r);
                }
                int i1, i2;
                if (head < a.H + a.G) {
                    // rows interleave the halves: this thread holds element i of the first half and its partner
                    const int i = within / 2 + r;
                    const float c = stage_a[(rt * 16 + m) * 16 + r], sn = stage_a[(rt * 16 + m) * 16 + 8 + r];
                    const float ra = x1 * c - x2 * sn, rb = x1 * sn + x2 * c;
                    x1 = ra; x2 = rb; i1 = i; i2 = i + hd / 2;
                } else {
                    i1 = within + r; i2 = i1 + 8;
                }
                __nv_bfloat16* dst = nullptr;
                if (head < a.H) {
                    dst = a.q_out + ((size_t)m * a.H + head) * hd;
                } else if (slot_s[m] >= 0) {
                    // slot = page * page_size + place in the page; the pool is [pages, G, page_size, hd]
                    const bool is_v = head >= a.H + a.G;
                    const int g = head - a.H - (is_v ? a.G : 0);
                    const int page = slot_s[m] / a.page_size, in_page = slot_s[m] - page * a.page_size;
                    dst = (is_v ? a.v_pages : a.k_pages) + (((size_t)page * a.G + g) * a.page_size + in_page) * hd;
                }
                if (dst != nullptr) {
                    dst[i1] = __float2bfloat16_rn(x1);
                    dst[i2] = __float2bfloat16_rn(x2);
                }
            } else {
                if (!live) continue;
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const int row = n0 + r + hi * 8;
                    float v = acc[j][hi * 2 + e];
                    if (a.bias) v += (a.bias_dtype == MM_F32) ? ((const float*)a.bias)[row] : __bfloat162float(((const __nv_bfloat16*)a.bias)[row]);
                    const size_t o = (size_t)m * a.ldo + row;
                    if (a.out_dtype == MM_F32) ((float*)a.out)[o] = v; else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(v);
                }
            }
        }
    }
}


template <int NT, int U, int EPI, int MINB>
__global__ void __launch_bounds__(GEMV_THREADS, MINB) gemv_bf16_kernel(const GemvArgs a) {
    __shared__ GemvSmem sm;
    extern __shared__ __align__(16) float ss_s[];
    // The weights do not depend on the previous kernel: their first loads go out before this kernel waits for
    // it, so the stream from HBM is already running when the activations become readable.
    GemvFirst<U> first;
    gemv_first_weights<U>(a, blockIdx.x, first);
    pdl_wait();
    gemv_item<NT, U, EPI>(a, blockIdx.x, first, sm, ss_s);
}

static int g_gemv_blocks = 0;   // 0: by the grid's size; 2 or 3: that build always (for measurements)
MM_EXPORT int mm_set_gemv_blocks(int n) {
    const int old = g_gemv_blocks;
    if (n == 0 || n == 2 || n == 3) g_gemv_blocks = n;
    return old;
}

static size_t gemv_dynamic_smem(const GemvArgs& a) {
    return a.in_ss ? (size_t)a.in_tiles * ((a.M + 3) & ~3) * sizeof(float) : 0;   // the staged partial sums of the input rows
}

template <int EPI>
static int launch_gemv_now(const GemvArgs& a, cudaStream_t s) {
    const int tiles = a.N / 16;
    const int blocks = (tiles + a.RT - 1) / a.RT;
    const size_t smem = gemv_dynamic_smem(a);
    // Two builds of the kernel: for two resident blocks per SM (more registers, nothing spilled, and a third block never
    // fits) and for three (80 registers).  A grid of at most two blocks per SM takes the first, larger grids the second.
    // A launch directly behind another launch of this kernel is a dependent one: with the residency that the chosen build
    // allows used up by the two grids, its early blocks can only take the places that the blocks of the kernel before it
    // leave, and every SM ends with its share (measured: 7B shapes 3.05 -> 2.97 ms per step, 14B 6.39 -> 6.25, 32B
    // 13.04 -> 12.75).  Behind attention or a norm the launch stays plain: there the early blocks land unevenly.
    int sms = 148;
    {
        static int cached = 0;
        if (cached == 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
        }
        sms = cached;
    }
    const bool two = g_gemv_blocks == 2 || (g_gemv_blocks == 0 && blocks <= 2 * sms);
    const bool dependent = g_mm_pdl != 0 && g_mm_dep_count == g_mm_launch_count && g_mm_dep_stream == (void*)s;
    if (two) {
        if (a.M <= 8) mm_launch_dependent(dependent, gemv_bf16_kernel<1, 4, EPI, 2>, dim3(blocks), dim3(GEMV_THREADS), smem, s, a);
        else mm_launch_dependent(dependent, gemv_bf16_kernel<2, 2, EPI, 2>, dim3(blocks), dim3(GEMV_THREADS), smem, s, a);
    } else {
        if (a.M <= 8) mm_launch_dependent(dependent, gemv_bf16_kernel<1, 4, EPI, 3>, dim3(blocks), dim3(GEMV_THREADS), smem, s, a);
        else mm_launch_dependent(dependent, gemv_bf16_kernel<2, 2, EPI, 3>, dim3(blocks), dim3(GEMV_THREADS), smem, s, a);
    }
    MM_CHECK_LAUNCH();
    g_mm_dep_count = g_mm_launch_count;
    g_mm_dep_stream = (void*)s;
    return MM_OK;
}

template <int EPI>
static int launch_gemv(const GemvArgs& a, cudaStream_t s) {
    if (gemv_dynamic_smem(a) > 16 * 1024) {
        mm_set_last_error("gemv: too many partial sums for the input scale (rows x producer tiles above 4096)");
        return MM_ERR_UNSUPPORTED;
    }
    return launch_gemv_now<EPI>(a, s);
}

// Checks shared by the entry points; fills the common fields.
static int gemv_common(GemvArgs& a, const void* W, const void* x, int M, int N, int K, int ldx, int rt, int ks,
                       const void* in_ss, int in_tiles, int in_dim, float in_eps) {
    MM_REQUIRE(M >= 1 && M <= 16, "gemv: M must be in 1..16");
    MM_REQUIRE(N > 0 && N % 16 == 0, "gemv: N must be a multiple of 16");
    MM_REQUIRE(K > 0 && K % 32 == 0, "gemv: K must be a multiple of 32");
    MM_REQUIRE(ldx >= K && ldx % 8 == 0, "gemv: x rows must be 16-byte aligned");
    MM_REQUIRE(rt >= 1 && ks >= 1 && rt * ks == GEMV_WARPS, "gemv: rt * ks must be 8");
    MM_REQUIRE(ks <= K / 32, "gemv: more K splits than 32-wide blocks");
    MM_REQUIRE(in_ss == nullptr || (in_tiles >= 1 && in_dim >= 1 && in_eps > 0.0f), "gemv: bad input-scale sizes");
    MM_REQUIRE((reinterpret_cast<uintptr_t>(in_ss) & 15) == 0, "gemv: the partial sums must be 16-byte aligned");
    a = GemvArgs();
    a.W = (const __nv_bfloat16*)W; a.x = (const __nv_bfloat16*)x;
    a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.RT = rt; a.KS = ks;
    a.in_ss = (const float*)in_ss; a.in_tiles = in_tiles; a.in_dim = in_dim; a.in_eps = in_eps;
    return MM_OK;
}

// out[M, ldo] = x[M, ldx(K)] * W[N,K]^T (+ bias), or with swiglu != 0: out[M, N/2] = silu(gate) * up for
// W rows interleaved gate/up in blocks of 8.  rt * ks must be 8.  in_ss (or null): partial sums of squares
// [in_tiles][16] of the rows that x was made from; row m of the product is scaled by 1/sqrt(sum/in_dim + in_eps).
MM_EXPORT int mm_gemv_bf16(const void* W, const void* x, const void* bias, int bias_dtype, void* out, int out_dtype,
                           int M, int N, int K, int ldx, int ldo, int rt, int ks, int swiglu,
                           const void* in_ss, int in_tiles, int in_dim, float in_eps, void* stream) {
    GemvArgs a;
    const int rc = gemv_common(a, W, x, M, N, K, ldx, rt, ks, in_ss, in_tiles, in_dim, in_eps);
    if (rc != MM_OK) return rc;
    MM_REQUIRE(out_dtype == MM_F32 || out_dtype == MM_BF16, "gemv: out dtype must be float32 or bfloat16");
    MM_REQUIRE(!swiglu || (bias == nullptr && ldo >= N / 2), "gemv: the SwiGLU epilogue takes no bias and writes N/2 columns");
    MM_REQUIRE(swiglu || ldo >= N, "gemv: ldo too small");
    a.bias = bias; a.bias_dtype = bias_dtype; a.out = out; a.out_dtype = out_dtype; a.ldo = ldo;
    cudaStream_t s = (cudaStream_t)stream;
    return swiglu ? launch_gemv<EPI_SWIGLU>(a, s) : launch_gemv<EPI_PLAIN>(a, s);
}

// residual[M, N] (fp32) += x * W^T.  With norm_w: also xw_out[M, N] = bf16(residual * norm_w) and
// out_ss[N/16][16] = per-tile sums of squares of the new residual rows (column m of a tile's 16 is row m).
MM_EXPORT int mm_gemv_bf16_residual(const void* W, const void* x, void* residual, const void* norm_w, int norm_w_dtype,
                                    void* xw_out, void* out_ss, int M, int N, int K, int ldx, int rt, int ks,
                                    const void* in_ss, int in_tiles, int in_dim, float in_eps, void* stream) {
    GemvArgs a;
    const int rc = gemv_common(a, W, x, M, N, K, ldx, rt, ks, in_ss, in_tiles, in_dim, in_eps);
    if (rc != MM_OK) return rc;
    MM_REQUIRE(residual != nullptr, "gemv: no residual");
    MM_REQUIRE(norm_w == nullptr || (xw_out != nullptr && out_ss != nullptr), "gemv: a norm weight needs both outputs");
    MM_REQUIRE(norm_w_dtype == MM_F32 || norm_w_dtype == MM_BF16, "gemv: norm weight dtype must be float32 or bfloat16");
    MM_REQUIRE(((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(norm_w)) & 15) == 0, "gemv: residual and norm weight must be 16-byte aligned");
    a.residual = (float*)residual; a.norm_w = norm_w; a.norm_w_dtype = norm_w_dtype;
    a.xw_out = (__nv_bfloat16*)xw_out; a.out_ss = (float*)out_ss;
    return launch_gemv<EPI_RESID>(a, (cudaStream_t)stream);
}

// q/k/v projection with bias, rotary encoding and cache write.  W [(H + 2G) * hd, K]: the rows of every q and k
// head interleave the head's two halves in blocks of 8 (rows 16b..16b+7 = elements 8b.. of the first half, rows
// 16b+8..16b+15 = the same elements of the second half); v rows and the layout of bias follow W.
// rope_table [M, hd] fp32 (mm_rope_table) and slots [M] (mm_slot_mapping) are per step, shared by all layers.
MM_EXPORT int mm_gemv_bf16_qkv_rope(const void* W, const void* x, const void* bias, int bias_dtype, void* q_out,
                                    void* k_pages, void* v_pages, const void* rope_table, const void* slots,
                                    int page_size, int H, int G, int hd, int M, int K, int ldx, int rt, int ks,
                                    const void* in_ss, int in_tiles, int in_dim, float in_eps, void* stream) {
    MM_REQUIRE(H >= 1 && G >= 1 && hd >= 16 && hd % 16 == 0, "gemv qkv: head size must be a multiple of 16");
    GemvArgs a;
    const int rc = gemv_common(a, W, x, M, (H + 2 * G) * hd, K, ldx, rt, ks, in_ss, in_tiles, in_dim, in_eps);
    if (rc != MM_OK) return rc;
    MM_REQUIRE(q_out != nullptr && rope_table != nullptr, "gemv qkv: q_out and the rotation table are needed");
    MM_REQUIRE((k_pages == nullptr) == (v_pages == nullptr), "gemv qkv: k_pages and v_pages go together");
    MM_REQUIRE(k_pages == nullptr || (slots != nullptr && page_size >= 1), "gemv qkv: a cache write needs the slots");
    MM_REQUIRE(((reinterpret_cast<uintptr_t>(rope_table) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0, "gemv qkv: table and bias must be 16-byte aligned");
    a.bias = bias; a.bias_dtype = bias_dtype;
    a.q_out = (__nv_bfloat16*)q_out; a.k_pages = (__nv_bfloat16*)k_pages; a.v_pages = (__nv_bfloat16*)v_pages;
    a.rope_table = (const float*)rope_table; a.slots = k_pages ? (const int32_t*)slots : nullptr;
    a.page_size = page_size > 0 ? page_size : 1; a.H = H; a.G = G; a.hd = hd;
    return launch_gemv<EPI_ROPE>(a, (cudaStream_t)stream);
}
