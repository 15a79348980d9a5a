// Memory-bound parts of a step: embedding gather, residual-add + RMSNorm, SiLU·up,
// and bias + rotary position encoding + paged K/V write.  All arithmetic is fp32;
// the template type is only what is stored.
//
// Formulas (reference, file:line):
//   embedding   x[t,:] = E[id_t,:], an id outside [0,V) gives a zero row
//               (src/compute/Embedding.cpp:46-67)
//   RMSNorm     y = x * w * (1 / sqrt(mean(x^2) + eps))      (src/compute/Norm.cpp:21-37)
//   add+norm    x += delta, then RMSNorm of the sum          (kernels/cuda/common/add_rmsnorm.cu:32-81)
//   SiLU·up     a = g / (1 + exp(-g)) * u                     (src/compute/Activations.cpp:25-36,
//                                                             kernels/cuda/common/silu_mul.cu:37-41)
//   rotary      pairs (i, i+half): theta = pos * base^(-2i/dim)
//               x'_i = x_i cos - x_{i+half} sin, x'_{i+half} = x_i sin + x_{i+half} cos
//               (src/compute/Rope.cpp:23-41), applied to q and k after the bias
//               (src/runtime/arch/Qwen2Backend.cpp:316-325, 369-375)
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int vocab, int d, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * d;
    if (id < 0 || id >= vocab) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32<T>(row[i]) * scale;
}

// bfloat16 table whose width is a multiple of 8: one 16-byte load and two 16-byte stores per thread and step, so a
// row's loads are all in flight at once (a handful of decode tokens otherwise waits for one load after the other)
__global__ void embedding_bf16x8_kernel(const int32_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                        float* __restrict__ out, int vocab, int d, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * d;
    const bool known = id >= 0 && id < vocab;
    const __nv_bfloat16* row = table + (size_t)(known ? id : 0) * d;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
        float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
        if (known) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 a = __bfloat1622float2(p2[0]), b = __bfloat1622float2(p2[1]);
            const float2 e = __bfloat1622float2(p2[2]), f = __bfloat1622float2(p2[3]);
            lo = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
            hi = make_float4(e.x * scale, e.y * scale, f.x * scale, f.y * scale);
        }
        *reinterpret_cast<float4*>(o + c) = lo;
        *reinterpret_cast<float4*>(o + c + 4) = hi;
    }
}

MM_EXPORT int mm_embedding(const void* ids, const void* table, int table_dtype, void* out, int n_tokens,
                           int vocab, int d, float scale, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && vocab > 0 && d > 0, "embedding: bad sizes");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == MM_F32)
        mm_launch(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const int32_t*)ids, (const float*)table, (float*)out, vocab, d, scale);
    else if (table_dtype == MM_BF16 && d % 8 == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)out & 15) == 0)
        mm_launch(embedding_bf16x8_kernel, dim3(n_tokens), dim3(d >= 4096 ? 512 : (d >= 2048 ? 256 : 128)), 0, s,
                      (const int32_t*)ids, (const __nv_bfloat16*)table, (float*)out, vocab, d, scale);
    else if (table_dtype == MM_BF16)
        mm_launch(embedding_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, (const int32_t*)ids, (const __nv_bfloat16*)table, (float*)out, vocab, d, scale);
    else
        MM_REQUIRE(false, "embedding: table dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------
// residual add + RMSNorm
//   residual: fp32 [*, d]; delta: T [*, d] or null; rows: int32 [n_rows] or null.
//   Output row i is made from source row r = rows ? rows[i] : i.
//   Without `rows` the sum is written back to the residual (it stays the running
//   residual stream); with `rows` (a gather for the output head) it is not.
// ---------------------------------------------------------------------------
template <typename T, typename WT>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const int32_t* __restrict__ rows, const WT* __restrict__ weight,
                                   T* __restrict__ out, int d, float eps) {
    extern __shared__ float row_cache[];
    __shared__ float red[32];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    float* res = residual + r * d;
    const T* dl = delta ? delta + r * d : nullptr;
    float ss = 0.0f;
    for (int k = threadIdx.x; k < d; k += blockDim.x) {
        float v = res[k];
        if (dl) v += to_f32<T>(dl[k]);
        row_cache[k] = v;
        ss = fmaf(v, v, ss);
    }
    const float total = block_sum(ss, red);
    const float inv_rms = 1.0f / sqrtf(total / (float)d + eps);
    T* o = out + (size_t)i * d;
    const bool write_back = (rows == nullptr) && (dl != nullptr);
    for (int k = threadIdx.x; k < d; k += blockDim.x) {
        const float v = row_cache[k];
        if (write_back) res[k] = v;
        o[k] = from_f32<T>(v * to_f32<WT>(weight[k]) * inv_rms);
    }
}

// f[0..8) += p[0..8), p aligned to 8 elements: 16-byte loads instead of eight scalar ones (a warp whose threads are
// 16 elements apart would otherwise touch 32 sectors with every scalar load).
__device__ __forceinline__ void add8(const float* __restrict__ p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
    f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
}
__device__ __forceinline__ void add8(const __nv_bfloat16* __restrict__ p, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 x = __bfloat1622float2(p2[k]);
        f[2 * k] += x.x;
        f[2 * k + 1] += x.y;
    }
}

// bfloat16 activations, width a multiple of 8 and at most 8192: every thread keeps 8 consecutive elements in
// registers (two float4 of the residual, one 16-byte load of the branch output), so a row makes one trip.
template <typename WT>
__global__ void add_rmsnorm_bf16x8_kernel(float* __restrict__ residual, const __nv_bfloat16* __restrict__ delta,
                                          const int32_t* __restrict__ rows, const WT* __restrict__ weight,
                                          __nv_bfloat16* __restrict__ out, int d, float eps) {
    __shared__ float red[32];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    const int c = threadIdx.x * 8;
    const bool active = c < d;
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = 0.0f;
    if (active) {
        const float4 a = *reinterpret_cast<const float4*>(residual + r * d + c);
        const float4 b = *reinterpret_cast<const float4*>(residual + r * d + c + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        if (delta) {
            const uint4 dv = *reinterpret_cast<const uint4*>(delta + r * d + c);
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(d2[k]);
                v[2 * k] += f.x;
                v[2 * k + 1] += f.y;
            }
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
    const float total = block_sum(ss, red);
    const float inv_rms = 1.0f / sqrtf(total / (float)d + eps);
    if (!active) return;
    if (rows == nullptr && delta != nullptr) {
        *reinterpret_cast<float4*>(residual + r * d + c) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(residual + r * d + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
    float w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) w[k] = 0.0f;
    add8(weight + c, w);
#pragma unroll
    for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(v[2 * k] * w[2 * k] * inv_rms, v[2 * k + 1] * w[2 * k + 1] * inv_rms);
    *reinterpret_cast<uint4*>(out + (size_t)i * d + c) = ov;
}

template <typename T, typename WT>
static int launch_add_rmsnorm(float* residual, const void* delta, const int32_t* rows, const void* weight, void* out,
                              int n_rows, int d, float eps, cudaStream_t s) {
    if constexpr (sizeof(T) == 2) {
        if (d % 8 == 0 && d <= 8192) {
            const int threads = ((d / 8 + 31) / 32) * 32;
            mm_launch(add_rmsnorm_bf16x8_kernel<WT>, dim3(n_rows), dim3(threads), 0, s, residual, (const __nv_bfloat16*)delta, rows,
                          (const WT*)weight, (__nv_bfloat16*)out, d, eps);
            MM_CHECK_LAUNCH();
            return MM_OK;
        }
    }
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) {
            mm_set_last_error("rmsnorm: width above 51200 is not supported");
            return MM_ERR_UNSUPPORTED;
        }
        cudaFuncSetAttribute(add_rmsnorm_kernel<T, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    mm_launch(add_rmsnorm_kernel<T, WT>, dim3(n_rows), dim3(threads), smem, s, residual, (const T*)delta, rows, (const WT*)weight, (T*)out, d, eps);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_add_rmsnorm(void* residual, const void* delta, const void* rows, const void* weight, int weight_dtype,
                             void* out, int act_dtype, int n_rows, int d, float eps, void* stream) {
    MM_REQUIRE(n_rows >= 0 && d > 0 && eps > 0.0f, "rmsnorm: bad sizes");
    if (n_rows == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    float* res = (float*)residual;
    const int32_t* rw = (const int32_t*)rows;
    if (act_dtype == MM_F32 && weight_dtype == MM_F32) return launch_add_rmsnorm<float, float>(res, delta, rw, weight, out, n_rows, d, eps, s);
    if (act_dtype == MM_F32 && weight_dtype == MM_BF16) return launch_add_rmsnorm<float, __nv_bfloat16>(res, delta, rw, weight, out, n_rows, d, eps, s);
    if (act_dtype == MM_BF16 && weight_dtype == MM_F32) return launch_add_rmsnorm<__nv_bfloat16, float>(res, delta, rw, weight, out, n_rows, d, eps, s);
    if (act_dtype == MM_BF16 && weight_dtype == MM_BF16) return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(res, delta, rw, weight, out, n_rows, d, eps, s);
    MM_REQUIRE(false, "rmsnorm: dtypes must be float32 or bfloat16");
}

// residual += delta only (the last layer's pending sum when no norm follows it)
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ residual, const T* __restrict__ delta, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) residual[i] += to_f32<T>(delta[i]);
}

MM_EXPORT int mm_add_residual(void* residual, const void* delta, int act_dtype, long long n, void* stream) {
    MM_REQUIRE(n >= 0, "add_residual: bad size");
    if (n == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (act_dtype == MM_F32) add_residual_kernel<float><<<blocks, 256, 0, s>>>((float*)residual, (const float*)delta, (size_t)n);
    else if (act_dtype == MM_BF16) add_residual_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((float*)residual, (const __nv_bfloat16*)delta, (size_t)n);
    else MM_REQUIRE(false, "add_residual: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------
// SiLU(gate) * up over a [n, 2F] buffer.  interleave == 0: gate in columns [0,F), up in
// [F,2F).  interleave == 8: blocks of 8 gate columns alternate with blocks of 8 up columns
// (gate f at (f/8)*16 + f%8, up f eight columns later), the layout of the fused weight.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int n, int F, int interleave) {
    const size_t total = (size_t)n * F;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t row = i / F, col = i - row * F;
        const size_t gc = interleave ? (col / 8) * 16 + col % 8 : col;
        const size_t uc = interleave ? gc + 8 : F + col;
        const float g = to_f32<T>(gu[row * 2 * F + gc]);
        const float u = to_f32<T>(gu[row * 2 * F + uc]);
        out[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// 8 bf16 values per thread when F is a multiple of 8
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int n, int F, int interleave) {
    const int F8 = F / 8;
    const size_t total = (size_t)n * F8;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t row = i / F8, c8 = i - row * F8;
        const size_t gc = interleave ? c8 * 16 : c8 * 8;
        const size_t uc = interleave ? gc + 8 : (size_t)F + c8 * 8;
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + row * 2 * F + gc);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + row * 2 * F + uc);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(g2[k]);
            const float2 u = __bfloat1622float2(u2[k]);
            float2 r;
            r.x = g.x / (1.0f + expf(-g.x)) * u.x;
            r.y = g.y / (1.0f + expf(-g.y)) * u.y;
            o2[k] = __float22bfloat162_rn(r);
        }
        *reinterpret_cast<uint4*>(out + row * F + c8 * 8) = ov;
    }
}

MM_EXPORT int mm_silu_mul(const void* gu, void* out, int act_dtype, int n, int F, int interleave, void* stream) {
    MM_REQUIRE(n >= 0 && F > 0, "silu_mul: bad sizes");
    MM_REQUIRE(interleave == 0 || (interleave == 8 && F % 8 == 0), "silu_mul: interleave must be 0, or 8 with F a multiple of 8");
    if (n == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)n * F;
    if (act_dtype == MM_BF16 && F % 8 == 0) {
        const size_t work = total / 8;
        const int blocks = (int)((work + 255) / 256 < 148 * 32 ? (work + 255) / 256 : 148 * 32);
        mm_launch(silu_mul_bf16x8_kernel, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n, F, interleave);
    } else {
        const int blocks = (int)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
        if (act_dtype == MM_F32) mm_launch(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, n, F, interleave);
        else if (act_dtype == MM_BF16) mm_launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n, F, interleave);
        else MM_REQUIRE(false, "silu_mul: dtype must be float32 or bfloat16");
    }
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------
// bias + rotary + paged K/V write
//   qkv      T [n, (H + 2G) * hd]  : q heads, then k heads, then v heads of each token
//   bias     WT [(H + 2G) * hd] or null
//   q_out    T [n, H * hd]
//   k_pages, v_pages  T [num_pages, G, page_size, hd] of this layer (null: nothing cached)
//   positions int32 [n], token_req int32 [n], block_table int32 [n_req, table_width]
//   rotary_dim: leading dims of each head that are rotated (0: no position encoding)
// ---------------------------------------------------------------------------
template <typename T, typename WT>
__global__ void qkv_rope_kvwrite_kernel(const T* __restrict__ qkv, const WT* __restrict__ bias, T* __restrict__ q_out,
                                        T* __restrict__ k_pages, T* __restrict__ v_pages,
                                        const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                                        const int32_t* __restrict__ block_table, int table_width, int page_size,
                                        int H, int G, int hd, int rotary_dim, float theta_base) {
    extern __shared__ float cs[];  // cos[half], sin[half]
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rotary_dim / 2;
    float* cosv = cs;
    float* sinv = cs + half;
    if (half > 0) {
        const float inv_dim = 1.0f / (float)rotary_dim;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float freq = powf(theta_base, -(float)(2 * i) * inv_dim);
            const float ang = (float)pos * freq;
            cosv[i] = cosf(ang);
            sinv[i] = sinf(ang);
        }
    }
    __syncthreads();

    const int row_width = (H + 2 * G) * hd;
    const T* src = qkv + (size_t)t * row_width;
    // destination of this token's K/V rows
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (k_pages != nullptr) {
        const int req = token_req[t];
        const int page = block_table[(size_t)req * table_width + pos / page_size];
        if (page >= 0) {
            const size_t base = ((size_t)page * G * page_size + (size_t)(pos % page_size)) * hd;
            kdst = k_pages + base;
            vdst = v_pages + base;
        }
    }
    const size_t head_stride_in_page = (size_t)page_size * hd;

    // rotated part of q and k heads: one thread per (head, pair)
    const int rot_heads = H + G;
    for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const int c0 = h * hd + i, c1 = c0 + half;
        float a = to_f32<T>(src[c0]), b = to_f32<T>(src[c1]);
        if (bias) {
            a += to_f32<WT>(bias[c0]);
            b += to_f32<WT>(bias[c1]);
        }
        const float c = cosv[i], s = sinv[i];
        const float ra = a * c - b * s;
        const float rb = a * s + b * c;
        if (h < H) {
            T* q = q_out + (size_t)t * H * hd + (size_t)h * hd;
            q[i] = from_f32<T>(ra);
            q[i + half] = from_f32<T>(rb);
        } else if (kdst) {
            T* k = kdst + (size_t)(h - H) * head_stride_in_page;
            k[i] = from_f32<T>(ra);
            k[i + half] = from_f32<T>(rb);
        }
    }
    // unrotated tail of q and k heads
    const int tail = hd - rotary_dim;
    if (tail > 0) {
        for (int idx = threadIdx.x; idx < rot_heads * tail; idx += blockDim.x) {
            const int h = idx / tail, i = rotary_dim + (idx - h * tail);
            const int c0 = h * hd + i;
            float a = to_f32<T>(src[c0]);
            if (bias) a += to_f32<WT>(bias[c0]);
            if (h < H) q_out[(size_t)t * H * hd + (size_t)h * hd + i] = from_f32<T>(a);
            else if (kdst) kdst[(size_t)(h - H) * head_stride_in_page + i] = from_f32<T>(a);
        }
    }
    // v heads
    if (vdst) {
        for (int idx = threadIdx.x; idx < G * hd; idx += blockDim.x) {
            const int g = idx / hd, i = idx - g * hd;
            const int c0 = (H + G) * hd + idx;
            float a = to_f32<T>(src[c0]);
            if (bias) a += to_f32<WT>(bias[c0]);
            vdst[(size_t)g * head_stride_in_page + i] = from_f32<T>(a);
        }
    }
}

// bfloat16, full rotary (rotary_dim == hd) with hd a multiple of 16: a thread rotates 8 consecutive pairs, two
// 16-byte loads and two 16-byte stores.  `interleave`: the columns of qkv (and bias) of every q and k head hold
// the head's halves alternating in blocks of 8 (the row order of the weight that the fused decode product wants,
// see gemv_bf16.cu); the outputs are in natural order either way.
template <typename WT>
__global__ void qkv_rope_kvwrite_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const WT* __restrict__ bias,
                                               __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages,
                                               __nv_bfloat16* __restrict__ v_pages, const int32_t* __restrict__ positions,
                                               const int32_t* __restrict__ token_req, const int32_t* __restrict__ block_table,
                                               int table_width, int page_size, int H, int G, int hd, float theta_base,
                                               int interleave) {
    extern __shared__ float cs[];  // cos[half], sin[half]
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = hd / 2;
    float* cosv = cs;
    float* sinv = cs + half;
    {
        const float inv_dim = 1.0f / (float)hd;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float freq = powf(theta_base, -(float)(2 * i) * inv_dim);
            const float ang = (float)pos * freq;
            cosv[i] = cosf(ang);
            sinv[i] = sinf(ang);
        }
    }
    __syncthreads();
    const int row_width = (H + 2 * G) * hd;
    const __nv_bfloat16* src = qkv + (size_t)t * row_width;
    __nv_bfloat16* kdst = nullptr;
    __nv_bfloat16* vdst = nullptr;
    if (k_pages != nullptr) {
        const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
        if (page >= 0) {
            const size_t base = ((size_t)page * G * page_size + (size_t)(pos % page_size)) * hd;
            kdst = k_pages + base;
            vdst = v_pages + base;
        }
    }
    const size_t head_stride_in_page = (size_t)page_size * hd;
    const int chunks = half / 8;                      // 8-pair chunks per head
    auto load8 = [&](int col, float* f) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + col);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 x = __bfloat1622float2(p2[k]);
            f[2 * k] = x.x;
            f[2 * k + 1] = x.y;
        }
        if (bias) add8(bias + col, f);
    };
    auto store8 = [&](__nv_bfloat16* dst, const float* f) {
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
        *reinterpret_cast<uint4*>(dst) = ov;
    };
    for (int idx = threadIdx.x; idx < (H + G) * chunks; idx += blockDim.x) {
        const int h = idx / chunks, i0 = (idx - h * chunks) * 8;
        float a[8], b[8], ra[8], rb[8];
        // interleaved input: the two halves of a q or k head alternate in blocks of 8 columns
        load8(interleave ? h * hd + 2 * i0 : h * hd + i0, a);
        load8(interleave ? h * hd + 2 * i0 + 8 : h * hd + i0 + half, b);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float c = cosv[i0 + k], sn = sinv[i0 + k];
            ra[k] = a[k] * c - b[k] * sn;
            rb[k] = a[k] * sn + b[k] * c;
        }
        __nv_bfloat16* dst = nullptr;
        if (h < H) dst = q_out + (size_t)t * H * hd + (size_t)h * hd;
        else if (kdst) dst = kdst + (size_t)(h - H) * head_stride_in_page;
        if (dst) {
            store8(dst + i0, ra);
            store8(dst + i0 + half, rb);
        }
    }
    if (vdst) {
        for (int idx = threadIdx.x; idx < G * hd / 8; idx += blockDim.x) {
            const int g = (idx * 8) / hd, i0 = idx * 8 - g * hd;
            float a[8];
            load8((H + G) * hd + idx * 8, a);
            store8(vdst + (size_t)g * head_stride_in_page + i0, a);
        }
    }
}

// The same with the step's tables: rotation factors from rope_table [n, hd] (cos of the hd/2 angles, then sin) and
// the cache place from slots [n] (page * page_size + place in the page, -1: not cached), both made once per step
// for all layers.  No arithmetic on angles and no dependent look-ups here: every load of a thread is issued at once.
template <typename WT>
__global__ void __launch_bounds__(384, 4) qkv_rope_tables_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const WT* __restrict__ bias,
                                              __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages,
                                              __nv_bfloat16* __restrict__ v_pages, const float* __restrict__ rope_table,
                                              const int32_t* __restrict__ slots, int page_size, int H, int G, int hd,
                                              int interleave) {
    const int t = blockIdx.x;
    const int half = hd / 2;
    const float* cosv = rope_table + (size_t)t * hd;
    const float* sinv = cosv + half;
    const int row_width = (H + 2 * G) * hd;
    const __nv_bfloat16* src = qkv + (size_t)t * row_width;
    __nv_bfloat16* kdst = nullptr;
    __nv_bfloat16* vdst = nullptr;
    if (k_pages != nullptr && slots != nullptr) {
        const int slot = slots[t];
        if (slot >= 0) {
            const int page = slot / page_size;
            const size_t base = ((size_t)page * G * page_size + (size_t)(slot - page * page_size)) * hd;
            kdst = k_pages + base;
            vdst = v_pages + base;
        }
    }
    const size_t head_stride_in_page = (size_t)page_size * hd;
    const int chunks = half / 8;
    auto load8 = [&](int col, float* f) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + col);
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 x = __bfloat1622float2(p2[k]);
            f[2 * k] = x.x;
            f[2 * k + 1] = x.y;
        }
        if (bias) add8(bias + col, f);
    };
    auto store8 = [&](__nv_bfloat16* dst, const float* f) {
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int k = 0; k < 4; ++k) o2[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
        *reinterpret_cast<uint4*>(dst) = ov;
    };
    const int rot_items = (H + G) * chunks;
    const int v_items = vdst ? G * hd / 8 : 0;
    for (int idx = threadIdx.x; idx < rot_items + v_items; idx += blockDim.x) {
        if (idx < rot_items) {
            const int h = idx / chunks, i0 = (idx - h * chunks) * 8;
            __nv_bfloat16* dst = nullptr;
            if (h < H) dst = q_out + (size_t)t * H * hd + (size_t)h * hd;
            else if (kdst) dst = kdst + (size_t)(h - H) * head_stride_in_page;
            if (!dst) continue;
            float a[8], b[8], c[8], sn[8], ra[8], rb[8];
            *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cosv + i0);
            *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cosv + i0 + 4);
            *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sinv + i0);
            *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sinv + i0 + 4);
            load8(interleave ? h * hd + 2 * i0 : h * hd + i0, a);
            load8(interleave ? h * hd + 2 * i0 + 8 : h * hd + i0 + half, b);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                ra[k] = a[k] * c[k] - b[k] * sn[k];
                rb[k] = a[k] * sn[k] + b[k] * c[k];
            }
            store8(dst + i0, ra);
            store8(dst + i0 + half, rb);
        } else {
            const int j = idx - rot_items;
            const int g = (j * 8) / hd, i0 = j * 8 - g * hd;
            float a[8];
            load8((H + G) * hd + j * 8, a);
            store8(vdst + (size_t)g * head_stride_in_page + i0, a);
        }
    }
}

MM_EXPORT int mm_qkv_rope_tables(const void* qkv, const void* bias, int bias_dtype, void* q_out, void* k_pages,
                                 void* v_pages, const void* rope_table, const void* slots, int page_size, int n_tokens,
                                 int H, int G, int hd, int interleave, void* stream) {
    typedef __nv_bfloat16 bf;
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && hd > 0 && hd % 16 == 0,
               "qkv_rope_tables: the head size must be a positive multiple of 16");
    MM_REQUIRE(page_size > 0, "qkv_rope_tables: bad page geometry");
    MM_REQUIRE((k_pages == nullptr) == (v_pages == nullptr), "qkv_rope_tables: k and v pools must both be given or both be null");
    MM_REQUIRE(k_pages == nullptr || slots != nullptr, "qkv_rope_tables: a cache needs the slots of the tokens");
    MM_REQUIRE(rope_table != nullptr, "qkv_rope_tables: no rotation table");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int items = (H + G) * (hd / 16) + G * hd / 8;
    int threads = ((items + 31) / 32) * 32;
    if (threads > 384) threads = 384;          // the kernel's launch bound (40 registers: five blocks of 320 threads per SM)
    if (bias == nullptr || bias_dtype == MM_F32)
        mm_launch(qkv_rope_tables_bf16x8_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const bf*)qkv, (const float*)bias,
                      (bf*)q_out, (bf*)k_pages, (bf*)v_pages, (const float*)rope_table, (const int32_t*)slots, page_size, H, G,
                      hd, interleave);
    else if (bias_dtype == MM_BF16)
        mm_launch(qkv_rope_tables_bf16x8_kernel<bf>, dim3(n_tokens), dim3(threads), 0, s, (const bf*)qkv, (const bf*)bias,
                      (bf*)q_out, (bf*)k_pages, (bf*)v_pages, (const float*)rope_table, (const int32_t*)slots, page_size, H, G,
                      hd, interleave);
    else MM_REQUIRE(false, "qkv_rope_tables: the bias must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

MM_EXPORT int mm_qkv_rope_kvwrite(const void* qkv, const void* bias, int bias_dtype, void* q_out, void* k_pages,
                                  void* v_pages, int act_dtype, const void* positions, const void* token_req,
                                  const void* block_table, int table_width, int page_size, int n_tokens, int H, int G,
                                  int hd, int rotary_dim, float theta_base, int interleave, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && hd > 0, "qkv_rope_kvwrite: bad sizes");
    MM_REQUIRE(interleave == 0 || (act_dtype == MM_BF16 && rotary_dim == hd && hd % 16 == 0),
               "qkv_rope_kvwrite: interleaved halves need bfloat16, full rotation and a head size that is a multiple of 16");
    MM_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0, "qkv_rope_kvwrite: rotary_dim must be even and at most head_dim");
    MM_REQUIRE(page_size > 0 && table_width > 0, "qkv_rope_kvwrite: bad page geometry");
    MM_REQUIRE((k_pages == nullptr) == (v_pages == nullptr), "qkv_rope_kvwrite: k and v pools must both be given or both be null");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)rotary_dim * sizeof(float);
    const int threads = 256;
#define MM_LAUNCH_QKV(T, WT)                                                                                       \
    mm_launch(qkv_rope_kvwrite_kernel<T, WT>, dim3(n_tokens), dim3(threads), smem, s,                           \
        (const T*)qkv, (const WT*)bias, (T*)q_out, (T*)k_pages, (T*)v_pages, (const int32_t*)positions,            \
        (const int32_t*)token_req, (const int32_t*)block_table, table_width, page_size, H, G, hd, rotary_dim,      \
        theta_base)
    if (bias == nullptr) bias_dtype = MM_F32;
    if (act_dtype == MM_BF16 && rotary_dim == hd && hd % 16 == 0) {
        typedef __nv_bfloat16 bf;
        if (bias_dtype == MM_F32)
            mm_launch(qkv_rope_kvwrite_bf16x8_kernel<float>, dim3(n_tokens), dim3(threads), smem, s, (const bf*)qkv, (const float*)bias,
                          (bf*)q_out, (bf*)k_pages, (bf*)v_pages, (const int32_t*)positions, (const int32_t*)token_req,
                          (const int32_t*)block_table, table_width, page_size, H, G, hd, theta_base, interleave);
        else
            mm_launch(qkv_rope_kvwrite_bf16x8_kernel<bf>, dim3(n_tokens), dim3(threads), smem, s, (const bf*)qkv, (const bf*)bias,
                          (bf*)q_out, (bf*)k_pages, (bf*)v_pages, (const int32_t*)positions, (const int32_t*)token_req,
                          (const int32_t*)block_table, table_width, page_size, H, G, hd, theta_base, interleave);
        MM_CHECK_LAUNCH();
        return MM_OK;
    }
    if (act_dtype == MM_F32 && bias_dtype == MM_F32) MM_LAUNCH_QKV(float, float);
    else if (act_dtype == MM_F32 && bias_dtype == MM_BF16) MM_LAUNCH_QKV(float, __nv_bfloat16);
    else if (act_dtype == MM_BF16 && bias_dtype == MM_F32) MM_LAUNCH_QKV(__nv_bfloat16, float);
    else if (act_dtype == MM_BF16 && bias_dtype == MM_BF16) MM_LAUNCH_QKV(__nv_bfloat16, __nv_bfloat16);
    else MM_REQUIRE(false, "qkv_rope_kvwrite: dtypes must be float32 or bfloat16");
#undef MM_LAUNCH_QKV
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------
// gather rows of a T [*, d] matrix: out[i,:] = src[rows[i],:]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ rows, T* __restrict__ out, int d) {
    const T* s = src + (size_t)rows[blockIdx.x] * d;
    T* o = out + (size_t)blockIdx.x * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = s[i];
}

MM_EXPORT int mm_gather_rows(const void* src, const void* rows, void* out, int dtype, int n_rows, int d, void* stream) {
    MM_REQUIRE(n_rows >= 0 && d > 0, "gather_rows: bad sizes");
    if (n_rows == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MM_F32) gather_rows_kernel<float><<<n_rows, 256, 0, s>>>((const float*)src, (const int32_t*)rows, (float*)out, d);
    else if (dtype == MM_BF16) gather_rows_kernel<__nv_bfloat16><<<n_rows, 256, 0, s>>>((const __nv_bfloat16*)src, (const int32_t*)rows, (__nv_bfloat16*)out, d);
    else MM_REQUIRE(false, "gather_rows: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}

// ---------------------------------------------------------------------------
// Per-step tables shared by all layers of a cache group / rotary encoding (read by the fused decode projection):
//   rope_table[t, 0:half] = cos(pos_t * theta^(-2i/dim)), rope_table[t, half:dim] = sin(...), i < half = dim / 2
//   slots[t] = page * page_size + pos_t % page_size with page = block_table[req_t, pos_t / page_size], or -1
// Same angle arithmetic as the rotary kernels above.
// ---------------------------------------------------------------------------
__global__ void rope_table_kernel(const int32_t* __restrict__ positions, float* __restrict__ out, int dim, float theta_base) {
    const int t = blockIdx.x, half = dim / 2;
    const int pos = positions[t];
    const float inv_dim = 1.0f / (float)dim;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float freq = powf(theta_base, -(float)(2 * i) * inv_dim);
        const float ang = (float)pos * freq;
        out[(size_t)t * dim + i] = cosf(ang);
        out[(size_t)t * dim + half + i] = sinf(ang);
    }
}

MM_EXPORT int mm_rope_table(const void* positions, void* out, int n_tokens, int dim, float theta_base, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && dim >= 2 && dim % 2 == 0 && theta_base > 0.0f, "rope_table: bad sizes");
    if (n_tokens == 0) return MM_OK;
    rope_table_kernel<<<n_tokens, 64, 0, (cudaStream_t)stream>>>((const int32_t*)positions, (float*)out, dim, theta_base);
    MM_CHECK_LAUNCH();
    return MM_OK;
}

__global__ void slot_mapping_kernel(const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                                    const int32_t* __restrict__ block_table, int table_width, int page_size, int n,
                                    int32_t* __restrict__ out) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
    out[t] = page >= 0 ? page * page_size + pos % page_size : -1;
}

MM_EXPORT int mm_slot_mapping(const void* positions, const void* token_req, const void* block_table, int table_width,
                              int page_size, int n_tokens, void* out, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && table_width >= 1 && page_size >= 1, "slot_mapping: bad sizes");
    if (n_tokens == 0) return MM_OK;
    slot_mapping_kernel<<<(n_tokens + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        (const int32_t*)positions, (const int32_t*)token_req, (const int32_t*)block_table, table_width, page_size, n_tokens, (int32_t*)out);
    MM_CHECK_LAUNCH();
    return MM_OK;
}
