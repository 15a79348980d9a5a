// Paged causal attention with grouped KV heads, fp32 arithmetic, any head size.
//
// One warp per (token, query head).  The key range of a token is cut into chunks of 32
// keys aligned to absolute position, and the running (max, sum, output) is updated
// chunk by chunk, so the result for a token depends only on its own position and keys:
// never on how the tokens were cut into steps or on what else is in the batch.  This is
// the kernel of the 32-bit path and the fallback of the bfloat16 path for head sizes the
// tensor-core kernels are not built for.
//
// Formula (reference src/compute/Attention.cpp:43-94): kv head g = (h*G)/H; a query at
// absolute position a sees keys [max(0, a+1-W), a] (W = 0: all); s_j = (q.k_j)*scale;
// p = softmax(s); o = sum_j p_j v_j.
#include "common.cuh"

#define ATT_MAX_ACC 16  // head_dim <= 512

template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                         const T* __restrict__ v_pages, T* __restrict__ out,
                                         const int32_t* __restrict__ positions, const int32_t* __restrict__ token_req,
                                         const int32_t* __restrict__ block_table, int table_width, int page_size,
                                         int n_tokens, int H, int G, int hd, int window, float scale) {
    extern __shared__ float q_smem[];  // [warps][hd]
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * warps_per_block + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const int g = (h * G) / H;
    const int pos = positions[t];
    const int req = token_req[t];
    const int32_t* table = block_table + (size_t)req * table_width;
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;

    float* qs = q_smem + warp * hd;
    const T* qrow = q + ((size_t)t * H + h) * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32<T>(qrow[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.0f;
    float acc[ATT_MAX_ACC];
#pragma unroll
    for (int a = 0; a < ATT_MAX_ACC; ++a) acc[a] = 0.0f;
    const size_t head_off = (size_t)g * page_size * hd;
    const size_t page_stride = (size_t)G * page_size * hd;

    for (int c = (lo / 32) * 32; c < hi; c += 32) {
        const int j = c + lane;
        const bool valid = (j >= lo) && (j < hi);
        float s = -INFINITY;
        if (valid) {
            const int page = table[j / page_size];
            const T* kr = k_pages + (size_t)page * page_stride + head_off + (size_t)(j % page_size) * hd;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f32<T>(kr[d]), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);  // m = -inf on the first chunk gives 0
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int a = 0; a < ATT_MAX_ACC; ++a) acc[a] *= alpha;
        for (int jj = 0; jj < 32; ++jj) {
            const int key = c + jj;
            if (key < lo || key >= hi) continue;  // uniform over the warp
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int page = table[key / page_size];
            const T* vr = v_pages + (size_t)page * page_stride + head_off + (size_t)(key % page_size) * hd;
#pragma unroll
            for (int a = 0; a < ATT_MAX_ACC; ++a) {
                const int d = a * 32 + lane;
                if (d < hd) acc[a] = fmaf(pj, to_f32<T>(vr[d]), acc[a]);
            }
        }
        m = m_new;
    }
    const float inv_l = (l > 0.0f) ? 1.0f / l : 0.0f;
    T* orow = out + ((size_t)t * H + h) * hd;
#pragma unroll
    for (int a = 0; a < ATT_MAX_ACC; ++a) {
        const int d = a * 32 + lane;
        if (d < hd) orow[d] = from_f32<T>(acc[a] * inv_l);
    }
}

MM_EXPORT int mm_attention_generic(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype,
                                   const void* positions, const void* token_req, const void* block_table,
                                   int table_width, int page_size, int n_tokens, int H, int G, int hd, int window,
                                   float scale, void* stream) {
    MM_REQUIRE(n_tokens >= 0 && H > 0 && G > 0 && hd > 0 && H % G == 0, "attention: heads must be a positive multiple of kv heads");
    MM_REQUIRE(hd <= 32 * ATT_MAX_ACC, "attention: head_dim above 512 is not supported");
    MM_REQUIRE(page_size > 0 && table_width > 0 && window >= 0, "attention: bad page geometry or window");
    if (n_tokens == 0) return MM_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    const size_t smem = (size_t)warps * hd * sizeof(float);
    const long long items = (long long)n_tokens * H;
    const int blocks = (int)((items + warps - 1) / warps);
    if (dtype == MM_F32)
        attention_generic_kernel<float><<<blocks, warps * 32, smem, s>>>(
            (const float*)q, (const float*)k_pages, (const float*)v_pages, (float*)out, (const int32_t*)positions,
            (const int32_t*)token_req, (const int32_t*)block_table, table_width, page_size, n_tokens, H, G, hd, window, scale);
    else if (dtype == MM_BF16)
        attention_generic_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, s>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out,
            (const int32_t*)positions, (const int32_t*)token_req, (const int32_t*)block_table, table_width, page_size,
            n_tokens, H, G, hd, window, scale);
    else
        MM_REQUIRE(false, "attention: dtype must be float32 or bfloat16");
    MM_CHECK_LAUNCH();
    return MM_OK;
}
