// Memory, descriptions, the part registry and the matrix-product dispatch of the native step executor.
#include <cublasLt.h>
#include <dlfcn.h>

#include <cstdio>
#include <cstring>
#include <tuple>

#include "exec.h"
#include "kernels_api.h"

namespace mmx {

void check_kernel(int code, const char* what) {
    if (code != 0) throw ExecError(std::string(what) + " failed (code " + std::to_string(code) + "): " + mm_last_error());
}

void check_cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw ExecError(std::string(what) + ": " + cudaGetErrorString(e));
}

// ---- Arena --------------------------------------------------------------------------------------------------------
Arena::~Arena() {
    for (auto& c : chunks_) cudaFree(c.base);
}

size_t Arena::capacity() const {
    size_t n = 0;
    for (auto& c : chunks_) n += c.size;
    return n;
}

void* Arena::alloc(size_t bytes) {
    bytes = (bytes + 255) & ~(size_t)255;
    if (bytes == 0) bytes = 256;
    while (cur_ < chunks_.size()) {
        Chunk& c = chunks_[cur_];
        if (off_ + bytes <= c.size) {
            void* p = c.base + off_;
            off_ += bytes;
            return p;
        }
        ++cur_;
        off_ = 0;
    }
    // a new chunk: at least what is asked for, and growing so that a few chunks serve any step
    size_t size = next_chunk_ > bytes ? next_chunk_ : bytes;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, size);
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw ExecError("the executor could not grow its device memory by " + std::to_string(size >> 20) + " MiB (" +
                        cudaGetErrorString(e) + "); a step larger than any before it cannot be run while a stream captures");
    }
    chunks_.push_back({static_cast<char*>(p), size});
    next_chunk_ = size * 2;
    cur_ = chunks_.size() - 1;
    off_ = bytes;
    return p;
}

// ---- PartDesc -------------------------------------------------------------------------------------------------------
double PartDesc::get(const std::string& key) const {
    auto it = num.find(key);
    if (it == num.end()) throw ExecError("part '" + kind + "': no parameter '" + key + "'");
    return it->second;
}
double PartDesc::get(const std::string& key, double fallback) const {
    auto it = num.find(key);
    return it == num.end() ? fallback : it->second;
}
const Tensor& PartDesc::tensor(const std::string& key) const {
    auto it = tensors.find(key);
    if (it == tensors.end()) throw ExecError("part '" + kind + "': no tensor '" + key + "'");
    return it->second;
}
const Tensor* PartDesc::tensor_or_null(const std::string& key) const {
    auto it = tensors.find(key);
    return it == tensors.end() ? nullptr : &it->second;
}
const PartDesc& PartDesc::child(const std::string& key) const {
    auto it = children.find(key);
    if (it == children.end()) throw ExecError("part '" + kind + "': no part '" + key + "'");
    return *it->second;
}

// ---- registry --------------------------------------------------------------------------------------------------------
static std::map<std::string, PartFactory>& registry() {
    static std::map<std::string, PartFactory> r;
    return r;
}
void register_part(const std::string& category, const std::string& kind, PartFactory f) {
    registry()[category + "/" + kind] = std::move(f);
}
std::unique_ptr<Part> build_part(const std::string& category, const PartDesc& d) {
    auto it = registry().find(category + "/" + d.kind);
    if (it == registry().end()) {
        std::string known;
        for (auto& kv : registry())
            if (kv.first.compare(0, category.size() + 1, category + "/") == 0) known += (known.empty() ? "" : ", ") + kv.first.substr(category.size() + 1);
        throw ExecError("no native " + category + " of kind '" + d.kind + "' (known: " + known + ")");
    }
    return it->second(d);
}

Options& options() {
    static Options o;
    return o;
}

// ---- the library product ------------------------------------------------------------------------------------------
struct Blas::Impl {
    void* so = nullptr;
    cublasLtHandle_t handle = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 32u << 20;
    decltype(&cublasLtCreate) create = nullptr;
    decltype(&cublasLtDestroy) destroy = nullptr;
    decltype(&cublasLtMatmul) matmul = nullptr;
    decltype(&cublasLtMatmulDescCreate) desc_create = nullptr;
    decltype(&cublasLtMatmulDescDestroy) desc_destroy = nullptr;
    decltype(&cublasLtMatmulDescSetAttribute) desc_set = nullptr;
    decltype(&cublasLtMatrixLayoutCreate) layout_create = nullptr;
    decltype(&cublasLtMatrixLayoutDestroy) layout_destroy = nullptr;
    decltype(&cublasLtMatmulPreferenceCreate) pref_create = nullptr;
    decltype(&cublasLtMatmulPreferenceDestroy) pref_destroy = nullptr;
    decltype(&cublasLtMatmulPreferenceSetAttribute) pref_set = nullptr;
    decltype(&cublasLtMatmulAlgoGetHeuristic) heuristic = nullptr;

    struct Plan {
        cublasLtMatmulDesc_t op = nullptr;
        cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
        cublasLtMatmulAlgo_t algo;
    };
    std::map<std::tuple<int, int, int, int>, Plan> plans;

    template <typename F>
    void sym(F& f, const char* name) {
        f = reinterpret_cast<F>(dlsym(so, name));
        if (!f) throw ExecError(std::string("cuBLASLt: symbol ") + name + " not found");
    }
    void ck(cublasStatus_t st, const char* what) {
        if (st != CUBLAS_STATUS_SUCCESS) throw ExecError(std::string("cuBLASLt: ") + what + " failed with status " + std::to_string((int)st));
    }
};

Blas::Blas() : impl_(new Impl) {
    Impl& m = *impl_;
    // the copy the process has loaded already (the one the host framework brought), else the loader's search path
    const char* names[] = {"libcublasLt.so.12", "libcublasLt.so", "/usr/local/cuda/lib64/libcublasLt.so.12"};
    for (const char* n : names)
        if ((m.so = dlopen(n, RTLD_NOW | RTLD_NOLOAD))) break;
    if (!m.so)
        for (const char* n : names)
            if ((m.so = dlopen(n, RTLD_NOW | RTLD_LOCAL))) break;
    if (!m.so) throw ExecError("cuBLASLt (libcublasLt.so.12) was not found; the plain bf16 products of more than a few rows need it");
    m.sym(m.create, "cublasLtCreate");
    m.sym(m.destroy, "cublasLtDestroy");
    m.sym(m.matmul, "cublasLtMatmul");
    m.sym(m.desc_create, "cublasLtMatmulDescCreate");
    m.sym(m.desc_destroy, "cublasLtMatmulDescDestroy");
    m.sym(m.desc_set, "cublasLtMatmulDescSetAttribute");
    m.sym(m.layout_create, "cublasLtMatrixLayoutCreate");
    m.sym(m.layout_destroy, "cublasLtMatrixLayoutDestroy");
    m.sym(m.pref_create, "cublasLtMatmulPreferenceCreate");
    m.sym(m.pref_destroy, "cublasLtMatmulPreferenceDestroy");
    m.sym(m.pref_set, "cublasLtMatmulPreferenceSetAttribute");
    m.sym(m.heuristic, "cublasLtMatmulAlgoGetHeuristic");
    m.ck(m.create(&m.handle), "cublasLtCreate");
    check_cuda(cudaMalloc(&m.workspace, m.workspace_bytes), "cuBLASLt workspace");
}

Blas::~Blas() {
    Impl& m = *impl_;
    for (auto& kv : m.plans) {
        if (kv.second.a) m.layout_destroy(kv.second.a);
        if (kv.second.b) m.layout_destroy(kv.second.b);
        if (kv.second.c) m.layout_destroy(kv.second.c);
        if (kv.second.op) m.desc_destroy(kv.second.op);
    }
    if (m.handle) m.destroy(m.handle);
    if (m.workspace) cudaFree(m.workspace);
}

void Blas::gemm_nt(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K, cudaStream_t s) {
    Impl& m = *impl_;
    auto key = std::make_tuple(M, N, K, out_dtype);
    auto it = m.plans.find(key);
    if (it == m.plans.end()) {
        // Row-major out[M, N] = x[M, K] W[N, K]^T is, in the library's column-major terms, out^T[N, M] = W'[K, N]^T x'[K, M]
        Impl::Plan p;
        m.ck(m.desc_create(&p.op, CUBLAS_COMPUTE_32F, CUDA_R_32F), "MatmulDescCreate");
        cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
        m.ck(m.desc_set(p.op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)), "set TRANSA");
        m.ck(m.desc_set(p.op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)), "set TRANSB");
        const cudaDataType_t ct = out_dtype == F32 ? CUDA_R_32F : CUDA_R_16BF;
        m.ck(m.layout_create(&p.a, CUDA_R_16BF, K, N, K), "layout A");
        m.ck(m.layout_create(&p.b, CUDA_R_16BF, K, M, K), "layout B");
        m.ck(m.layout_create(&p.c, ct, N, M, N), "layout C");
        cublasLtMatmulPreference_t pref = nullptr;
        m.ck(m.pref_create(&pref), "PreferenceCreate");
        m.ck(m.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &m.workspace_bytes, sizeof(m.workspace_bytes)), "set workspace");
        cublasLtMatmulHeuristicResult_t res;
        int found = 0;
        cublasStatus_t st = m.heuristic(m.handle, p.op, p.a, p.b, p.c, p.c, pref, 1, &res, &found);
        m.pref_destroy(pref);
        if (st != CUBLAS_STATUS_SUCCESS || found < 1)
            throw ExecError("cuBLASLt has no algorithm for a bf16 product of " + std::to_string(M) + " x " + std::to_string(N) + " x " + std::to_string(K));
        p.algo = res.algo;
        it = m.plans.emplace(key, p).first;
    }
    const Impl::Plan& p = it->second;
    const float one = 1.f, zero = 0.f;
    m.ck(m.matmul(m.handle, p.op, &one, W, p.a, x, p.b, &zero, out, p.c, out, p.c, &p.algo, m.workspace, m.workspace_bytes, s), "Matmul");
}

// ---- dispatch ---------------------------------------------------------------------------------------------------------
void Step::fork() const {
    check_cuda(cudaEventRecord(forked, stream), "forking the side stream");
    check_cuda(cudaStreamWaitEvent(side, forked, 0), "forking the side stream");
}
void Step::join() const {
    check_cuda(cudaEventRecord(joined, side), "joining the side stream");
    check_cuda(cudaStreamWaitEvent(stream, joined, 0), "joining the side stream");
}

bool gemv_supported(int m, int n, int k) { return 1 <= m && m <= options().gemv_max_rows && n % 16 == 0 && k % 32 == 0 && k >= 256; }
bool skinny_supported(int m, int n, int k) {
    return options().gemv_max_rows < m && m <= options().skinny_max_rows && n % 16 == 0 && k % 8 == 0 && k >= 64;
}

static int skinny_pad(int m) { return m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128)); }

// K splits (= cluster size) of the tcgen05 weight-streaming product: enough CTAs to fill the GPU when the weight has
// few 128-row tiles, no more clusters than are resident at once, at least 6 blocks of 64 along K per CTA, a power of two.
static int skinny_splits(int n, int k) {
    const int tiles = (n + 127) / 128, k_blocks = (k + 63) / 64;
    int s = 1;
    while (s < 8 && tiles * s * 2 <= 256 && k_blocks / (s * 2) >= 6) s *= 2;
    return s;
}

// 8 warps per CTA of the register-streaming kernel as row tiles x K splits: as many row tiles per CTA (8, 4, 2, 1) as
// still leave one and a half CTAs per SM; fewer CTAs than that do not keep enough loads in flight, many more only add
// CTAs that wait their turn.  Measured per product at 8 rows (us, best first): 1,728 tiles of 5,120: 4 tiles per CTA 45.9,
// 2: 47.5, 8: 50.8, 1: 51.7; 2,368 tiles of 3,584: 8: 44.6, 2: 49.4; 608 of 896: 2: 6.4, 4: 7.3, 1: 8.3; 448 of 5,120:
// 2: 15.3, 1: 18.7; 320 tiles and fewer: 1.
static void gemv_layout(int n, int k, int* rt, int* ks) {
    const int tiles = n / 16;
    int r = 8;
    while (r > 1 && (tiles + r - 1) / r < 222) r /= 2;
    int s = 8 / r;
    while (s > k / 32) {
        s /= 2;
        r *= 2;
    }
    *rt = r;
    *ks = s;
}

Rows linear(Step& st, Arena& mem, const Rows& x, const Tensor& W, int out_dtype, void* into) {
    if (out_dtype < 0) out_dtype = x.dtype;
    const int m = x.n, k = x.width, n = (int)W.shape[0];
    if (W.ndim != 2 || W.shape[1] != k) throw ExecError("linear: the weight's inner size does not match the rows");
    Rows out{into ? into : mem.alloc((size_t)m * n * dtype_size(out_dtype)), out_dtype, m, n};
    void* s = st.stream;
    if (x.dtype == BF16 && W.dtype == BF16 && !st.simt) {
        if (gemv_supported(m, n, k)) {
            int rt, ks;
            gemv_layout(n, k, &rt, &ks);
            check_kernel(mm_gemv_bf16(W.ptr, x.ptr, nullptr, F32, out.ptr, out_dtype, m, n, k, k, n, rt, ks, 0, nullptr, 0, 0, 0.f, s), "gemv_bf16");
        } else {
            st.blas->gemm_nt(x.ptr, W.ptr, out.ptr, out_dtype, m, n, k, st.stream);
        }
        return out;
    }
    check_kernel(mm_gemm_simt(x.ptr, x.dtype, W.ptr, W.dtype, nullptr, F32, out.ptr, out_dtype, m, n, k, k, n, s), "gemm_simt");
    return out;
}

Rows small_product(Step& st, Arena& mem, const Act& x, const Tensor& W, int out_dtype, bool swiglu) {
    const void* xin = x.factored ? x.f.xw : x.rows.ptr;
    const int m = x.n(), k = x.factored ? x.f.width : x.rows.width, n = (int)W.shape[0];
    if (W.shape[1] != k || !small_batch_supported(m, n, k)) throw ExecError("small product: sizes are not supported");
    const int cols = swiglu ? n / 2 : n;
    Rows out{mem.alloc((size_t)m * cols * dtype_size(out_dtype)), out_dtype, m, cols};
    const float* ss = x.factored ? x.f.ss : nullptr;
    if (m > options().gemv_max_rows) {
        if (cols % 8) throw ExecError("small product: the tcgen05 product needs output rows of a multiple of 8 columns");
        check_kernel(mm_gemm_skinny(W.ptr, xin, nullptr, F32, out.ptr, out_dtype, m, n, k, k, cols, skinny_splits(n, k), swiglu ? 1 : 0, ss,
                                    ss ? x.f.tiles : 0, ss ? x.f.dim : 0, ss ? x.f.ld : 0, ss ? x.f.eps : 0.f, st.err, st.stream), "gemm_skinny");
        return out;
    }
    int rt, ks;
    gemv_layout(n, k, &rt, &ks);
    check_kernel(mm_gemv_bf16(W.ptr, xin, nullptr, F32, out.ptr, out_dtype, m, n, k, k, cols, rt, ks, swiglu ? 1 : 0, ss, ss ? x.f.tiles : 0,
                              ss ? x.f.dim : 0, ss ? x.f.eps : 0.f, st.stream), "gemv_bf16");
    return out;
}

Out small_product_residual(Step& st, Arena& mem, const Rows& x, const Tensor& W, const Sink& sink) {
    const int m = x.n, k = x.width, n = (int)W.shape[0];
    if (W.shape[1] != k || !small_batch_supported(m, n, k)) throw ExecError("small product: sizes are not supported");
    const bool skinny = m > options().gemv_max_rows;
    Out out;
    void* xw = nullptr;
    float* ss = nullptr;
    const int ld = skinny ? skinny_pad(m) : 16;
    if (sink.norm_w) {
        if (sink.norm_w->shape[0] != n) throw ExecError("small product: the norm weight has the wrong length");
        xw = mem.alloc((size_t)m * n * 2);
        ss = mem.alloc_n<float>((size_t)(n / 16) * ld);
        out.kind = Out::FACTORED;
        out.f = Factored{xw, ss, m, n, n / 16, ld, n, sink.eps};
    }
    const void* nw = sink.norm_w ? sink.norm_w->ptr : nullptr;
    const int nwd = sink.norm_w ? sink.norm_w->dtype : F32;
    if (skinny) {
        check_kernel(mm_gemm_skinny_residual(W.ptr, x.ptr, sink.residual, nw, nwd, xw, ss, ss ? ld : 0, m, n, k, k, skinny_splits(n, k), nullptr, 0,
                                             0, 0, 0.f, st.err, st.stream), "gemm_skinny_residual");
    } else {
        int rt, ks;
        gemv_layout(n, k, &rt, &ks);
        check_kernel(mm_gemv_bf16_residual(W.ptr, x.ptr, sink.residual, nw, nwd, xw, ss, m, n, k, k, rt, ks, nullptr, 0, 0, 0.f, st.stream),
                     "gemv_bf16_residual");
    }
    return out;
}

// used by the attention mixer's fused projection (parts_builtin.cu)
void qkv_rope_small(Step& st, const Act& x, const Tensor& W, const Tensor* bias, void* q_out, void* k_pages, void* v_pages, const void* table,
                    const void* slots, int page_size, int H, int G, int hd) {
    const void* xin = x.factored ? x.f.xw : x.rows.ptr;
    const int m = x.n(), k = x.factored ? x.f.width : x.rows.width, n = (H + 2 * G) * hd;
    if (W.shape[0] != n || W.shape[1] != k || !small_batch_supported(m, n, k) || hd % 16) throw ExecError("fused q/k/v product: sizes are not supported");
    const float* ss = x.factored ? x.f.ss : nullptr;
    const void* b = bias ? bias->ptr : nullptr;
    const int bd = bias ? bias->dtype : F32;
    const void* sl = k_pages ? slots : nullptr;
    if (m > options().gemv_max_rows) {
        check_kernel(mm_gemm_skinny_qkv_rope(W.ptr, xin, b, bd, q_out, k_pages, v_pages, table, sl, page_size, H, G, hd, m, k, k, skinny_splits(n, k), ss,
                                             ss ? x.f.tiles : 0, ss ? x.f.dim : 0, ss ? x.f.ld : 0, ss ? x.f.eps : 0.f, st.err, st.stream),
                     "gemm_skinny_qkv_rope");
        return;
    }
    int rt, ks;
    gemv_layout(n, k, &rt, &ks);
    check_kernel(mm_gemv_bf16_qkv_rope(W.ptr, xin, b, bd, q_out, k_pages, v_pages, table, sl, page_size, H, G, hd, m, k, k, rt, ks, ss, ss ? x.f.tiles : 0,
                                       ss ? x.f.dim : 0, ss ? x.f.eps : 0.f, st.stream), "gemv_bf16_qkv_rope");
}

}  // namespace mmx
