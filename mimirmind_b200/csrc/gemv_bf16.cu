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
// Epilogues: bias; fp32 or bf16 output; SwiGLU when the weight rows interleave gate and up
// in blocks of 8 (rows 16j..16j+7 = gate[8j..], rows 16j+8..16j+15 = up[8j..]), so that one
// thread holds a gate value and its up value.
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
    int swiglu;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, int U>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_bf16_kernel(const GemvArgs a) {
    __shared__ float red[GEMV_WARPS][32][4 * NT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = lane & 3, r = lane >> 2;
    const int K = a.K;

    const int rt = warp / a.KS, ks = warp - rt * a.KS;
    const int n0 = (blockIdx.x * a.RT + rt) * 16;
    const bool active = n0 < a.N;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    if (active) {
        // this warp's share of the 32-wide k blocks
        const int nkb = K / 32, base = nkb / a.KS, rem = nkb % a.KS;
        const int kb_begin = ks * base + min(ks, rem);
        const int kb_count = base + (ks < rem ? 1 : 0);
        const __nv_bfloat16* wlo = a.W + (size_t)(n0 + r) * K + (size_t)kb_begin * 32 + t * 8;
        const __nv_bfloat16* whi = wlo + (size_t)8 * K;
        const __nv_bfloat16* xg[NT];
        bool xok[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int n = j * 8 + r;
            xok[j] = n < a.M;
            xg[j] = a.x + (size_t)(xok[j] ? n : 0) * a.ldx + (size_t)kb_begin * 32 + t * 8;
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
                    xb[buf][u][j] = (kb + u < kb_count && xok[j])
                                        ? __ldg(reinterpret_cast<const uint4*>(xg[j] + (size_t)(kb + u) * 32))
                                        : make_uint4(0, 0, 0, 0);
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
        // The weights do not depend on the previous kernel: their first loads go out before this kernel waits for
        // it, so the stream from HBM is already running when the activations become readable.
        load_w(0, 0);
        pdl_wait();
        pdl_trigger();
        load_x(0, 0);
        for (int kb = 0; kb < kb_count; kb += 2 * U) {
            load_w(1, kb + U);
            load_x(1, kb + U);
            mma_batch(0, kb);
            load_w(0, kb + 2 * U);
            load_x(0, kb + 2 * U);
            mma_batch(1, kb + U);
        }
    } else {
        pdl_wait();
        pdl_trigger();
    }
    // sum the K splits of each row tile in a fixed order
    if (a.KS > 1) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) red[warp][lane][j * 4 + e] = acc[j][e];
        __syncthreads();
        if (ks == 0) {
            for (int s = 1; s < a.KS; ++s)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[j][e] += red[warp + s][lane][j * 4 + e];
        }
    }
    if (!active || ks != 0) return;

    // epilogue: acc[j] = {(row r, col 2t), (row r, col 2t+1), (row r+8, col 2t), (row r+8, col 2t+1)} of batch tile j
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int m = j * 8 + t * 2 + e;
            if (m >= a.M) continue;
            if (a.swiglu) {
                const float g = acc[j][e], u = acc[j][2 + e];
                const float v = g / (1.0f + expf(-g)) * u;
                const size_t o = (size_t)m * a.ldo + n0 / 2 + r;
                if (a.out_dtype == MM_F32) ((float*)a.out)[o] = v; else ((__nv_bfloat16*)a.out)[o] = __float2bfloat16_rn(v);
            } else {
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

template <int NT, int U>
static int launch_gemv(const GemvArgs& a, cudaStream_t s) {
    const int tiles = a.N / 16;
    const int blocks = (tiles + a.RT - 1) / a.RT;
    mm_launch_pdl(gemv_bf16_kernel<NT, U>, dim3(blocks), dim3(GEMV_THREADS), 0, s, a);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// out[M, ldo] = x[M, ldx(K)] * W[N,K]^T (+ bias), or with swiglu != 0: out[M, N/2] = silu(gate) * up for
// W rows interleaved gate/up in blocks of 8.  rt * ks must be 8.
MM_EXPORT int mm_gemv_bf16(const void* W, const void* x, const void* bias, int bias_dtype, void* out, int out_dtype,
                           int M, int N, int K, int ldx, int ldo, int rt, int ks, int swiglu, void* stream) {
    MM_REQUIRE(M >= 1 && M <= 16, "gemv: M must be in 1..16");
    MM_REQUIRE(N > 0 && N % 16 == 0, "gemv: N must be a multiple of 16");
    MM_REQUIRE(K > 0 && K % 32 == 0, "gemv: K must be a multiple of 32");
    MM_REQUIRE(ldx >= K && ldx % 8 == 0, "gemv: x rows must be 16-byte aligned");
    MM_REQUIRE(rt >= 1 && ks >= 1 && rt * ks == GEMV_WARPS, "gemv: rt * ks must be 8");
    MM_REQUIRE(ks <= K / 32, "gemv: more K splits than 32-wide blocks");
    MM_REQUIRE(out_dtype == MM_F32 || out_dtype == MM_BF16, "gemv: out dtype must be float32 or bfloat16");
    MM_REQUIRE(!swiglu || (bias == nullptr && ldo >= N / 2), "gemv: the SwiGLU epilogue takes no bias and writes N/2 columns");
    MM_REQUIRE(swiglu || ldo >= N, "gemv: ldo too small");
    GemvArgs a;
    a.W = (const __nv_bfloat16*)W; a.x = (const __nv_bfloat16*)x; a.bias = bias; a.out = out;
    a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldo = ldo; a.bias_dtype = bias_dtype; a.out_dtype = out_dtype;
    a.RT = rt; a.KS = ks; a.swiglu = swiglu;
    const int nt = M <= 8 ? 1 : 2;
    cudaStream_t s = (cudaStream_t)stream;
    return nt == 1 ? launch_gemv<1, 4>(a, s) : launch_gemv<2, 2>(a, s);
}
