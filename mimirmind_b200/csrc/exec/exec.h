// The native step executor: the launch sequence of a whole step, issued from C++.
//
// A model is a tree of part descriptions (kind, numbers, tensors, children) handed over by the loader; every kind
// that can run natively has a factory in a registry (register_part), so another mixer, feed-forward, norm,
// position encoding or block arrangement is one more class with one more registration.  A model whose parts all
// have native classes runs its steps here: one call assembles the step's integers (token ids, positions,
// token -> request, block tables, wanted rows, attention work lists), copies them to the device once and launches
// every layer, the final norm and the head, with activations from memory the executor owns.  The reference runs a
// block the same way, as one native call that issues all of its kernels
// (src/runtime/arch/Qwen2Backend.cpp:132-466), inside a native generate loop
// (src/runtime/InferenceEngine.cpp:1304-2131).
//
// Nothing here synchronises with the device except the growth of the executor's memory (outside stream capture)
// and the reuse of a pinned staging buffer whose last copy has not run yet.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace mmx {

constexpr int F32 = 0, BF16 = 1;
constexpr int MAX_GROUPS = 8;

inline size_t dtype_size(int dt) { return dt == F32 ? 4 : 2; }

// What a step refuses before anything runs (a bad token id, an unknown request, no pages): the caller's mistake.
struct StepRefused : std::runtime_error {
    using std::runtime_error::runtime_error;
};
// Anything else: a kernel that refused its sizes, a failed launch, a failed allocation.
struct ExecError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

void check_kernel(int code, const char* what);       // throws ExecError with the kernel library's message
void check_cuda(cudaError_t e, const char* what);

// ---- memory ---------------------------------------------------------------------------------------------------
// Device memory handed out front to back and taken back all at once.  It grows by whole chunks and never moves or
// frees one before the executor goes, so addresses recorded in a captured graph stay valid.
class Arena {
  public:
    explicit Arena(size_t first_chunk) : next_chunk_(first_chunk) {}
    ~Arena();
    Arena(const Arena&) = delete;
    Arena& operator=(const Arena&) = delete;
    void* alloc(size_t bytes);
    template <typename T>
    T* alloc_n(size_t n) { return static_cast<T*>(alloc(n * sizeof(T))); }
    void reset() { cur_ = 0; off_ = 0; }
    size_t capacity() const;

  private:
    struct Chunk {
        char* base;
        size_t size;
    };
    std::vector<Chunk> chunks_;
    size_t cur_ = 0, off_ = 0, next_chunk_;
};

// ---- descriptions -----------------------------------------------------------------------------------------------
struct Tensor {
    void* ptr = nullptr;
    int dtype = F32;
    int ndim = 0;
    long long shape[4] = {0, 0, 0, 0};
    bool ok() const { return ptr != nullptr; }
};

struct PartDesc {
    std::string kind;
    std::map<std::string, double> num;
    std::map<std::string, Tensor> tensors;
    std::map<std::string, std::unique_ptr<PartDesc>> children;

    double get(const std::string& key) const;
    double get(const std::string& key, double fallback) const;
    int geti(const std::string& key) const { return (int)get(key); }
    const Tensor& tensor(const std::string& key) const;
    const Tensor* tensor_or_null(const std::string& key) const;
    const PartDesc& child(const std::string& key) const;
};

// ---- activations --------------------------------------------------------------------------------------------------
struct Rows {                 // [n, width] contiguous
    void* ptr = nullptr;
    int dtype = F32;
    int n = 0, width = 0;
};

// Rows of norm(x) in factored form, for norms of the kind x * w / rms(x): xw holds x * w (bf16) and ss the partial
// sums of squares per 16-column tile of the producer, [tiles, ld]; a matrix product applies 1/rms to its result.
struct Factored {
    void* xw = nullptr;
    float* ss = nullptr;
    int n = 0, width = 0, tiles = 0, ld = 0, dim = 0;
    float eps = 0.f;
};

struct Act {                  // what a mixer or feed-forward gets
    bool factored = false;
    Rows rows;
    Factored f;
    int n() const { return factored ? f.n : rows.n; }
};

struct Out {                  // what it gives back
    enum Kind { NONE, ROWS, FACTORED } kind = NONE;
    Rows rows;
    Factored f;
};

// Where a fusing part adds its output itself: the fp32 residual stream and, if a norm follows whose consumer takes
// factored rows, that norm's weight and eps.
struct Sink {
    float* residual = nullptr;
    const Tensor* norm_w = nullptr;
    float eps = 0.f;
};

struct LayerCache {
    void* k_pages = nullptr;
    void* v_pages = nullptr;
    const int* table = nullptr;      // device, [requests, table_width]
    int table_width = 0, page_size = 0, num_pages = 0, group = -1;
    bool writes = true;
};

class Blas;
class Executor;

// One batch: tokens of several requests, portions of prompts beside single decoded tokens.
struct Step {
    int n_tokens = 0, n_requests = 0, n_logit_rows = 0, max_kv_len = 0, max_q_len = 0, page_size = 0, table_width = 0;
    const int* token_ids = nullptr;       // device
    const int* positions = nullptr;
    const int* token_req = nullptr;
    const int* logit_rows = nullptr;
    const int* tables[MAX_GROUPS] = {};
    std::vector<int> q_start, q_len, kv_len;   // host, per request
    int act_dtype = BF16;
    bool simt = false;
    cudaStream_t stream = nullptr;
    void* err = nullptr;                  // device int the tcgen05 kernels set when a bounded wait ran out
    // a second stream with two events (or null): independent kernels of a part may run there beside the step's own,
    // between step.fork() and step.join()
    cudaStream_t side = nullptr;
    cudaEvent_t forked = nullptr, joined = nullptr;
    void fork() const;                    // the side stream waits for what the step has launched so far
    void join() const;                    // the step waits for what the side stream has been given
    Arena* step_mem = nullptr;            // lives until the step has been launched
    Arena* layer_mem = nullptr;           // the running layer's; the one before it keeps its memory one layer longer
    Blas* blas = nullptr;
    // device buffers derived from the step's inputs and shared between layers (rotation tables, cache slots)
    std::map<std::string, const void*> derived;
    // launch plans made once per step on the host and shared between layers
    std::map<std::string, std::shared_ptr<void>> plans;
    // integers a plan wants on the device: collected while the step is prepared, copied with the step's one copy
    struct Upload {
        std::vector<int> data;
        const int** where;                // receives the device address
    };
    std::vector<Upload> uploads;
};

// ---- parts -----------------------------------------------------------------------------------------------------------
struct Part {
    virtual ~Part() = default;
    // host-only planning for a step, before its integers are copied (may add to step.uploads)
    virtual void prepare(Step&, const LayerCache*) {}
};

struct Norm : Part {
    // residual (fp32 [n, width]) += delta; the normalised rows in the activation dtype.  With rows only those rows
    // are produced and the residual is not written.
    virtual Rows forward(Step&, Arena&, float* residual, const Rows* delta, const int* rows, int n_rows) = 0;
    // weight and eps if the norm is x * weight / sqrt(mean(x^2) + eps), else false
    virtual bool factors(const Tensor** weight, float* eps) const { return false; }
};

struct PositionEncoding : Part {
    // (rotary_dim, theta) of a split-half rotation the fused kernels apply
    virtual bool fused_rotary(int* rotary_dim, float* theta) const = 0;
};

struct Mixer : Part {
    virtual bool fuses(const Step&, int n_tokens) const { return false; }
    virtual Out forward(Step&, Arena&, const Act& x, LayerCache& cache, const Sink* sink) = 0;
};

struct FeedForward : Part {
    virtual bool fuses(const Step&, int n_tokens) const { return false; }
    virtual Out forward(Step&, Arena&, const Act& x, const Sink* sink) = 0;
};

// A branch output not yet added to the residual stream, or the factored rows prepared for a block's first norm.
struct Pending {
    enum Kind { NONE, DELTA, FACTORED } kind = NONE;
    Rows delta;
    Factored f;
};

struct Block : Part {
    virtual Pending forward(Step&, float* residual, const Pending& pending, LayerCache& cache, Block* successor) = 0;
    virtual bool entry_norm(const Step&, int n_tokens, const Tensor** weight, float* eps) const { return false; }
};

struct Embedding : Part {
    virtual float* forward(Step&, Arena&) = 0;        // fp32 [n_tokens, width]
    virtual int width() const = 0;
};

struct Head : Part {
    virtual void forward(Step&, Arena&, const Rows& x, float* logits) = 0;   // fp32 [x.n, vocab]
    virtual int vocab() const = 0;
};

// The registry: kind -> factory.  A factory may throw ExecError when it cannot take the description (then the
// model runs through the loader's own part classes instead).
using PartFactory = std::function<std::unique_ptr<Part>(const PartDesc&)>;
void register_part(const std::string& category, const std::string& kind, PartFactory f);
std::unique_ptr<Part> build_part(const std::string& category, const PartDesc& d);

template <typename T>
std::unique_ptr<T> build_as(const std::string& category, const PartDesc& d) {
    std::unique_ptr<Part> p = build_part(category, d);
    T* t = dynamic_cast<T*>(p.get());
    if (!t) throw ExecError("part kind '" + d.kind + "' is not a " + category);
    p.release();
    return std::unique_ptr<T>(t);
}

struct Registrar {
    Registrar(const char* category, const char* kind, PartFactory f) { register_part(category, kind, std::move(f)); }
};

// ---- matrix products ------------------------------------------------------------------------------------------------
// The library's bf16 product (cuBLASLt, found at run time in the process or on the loader's path), for the plain
// products of more rows than the weight-streaming kernels take; the reference's bf16 library route is the same
// (src/compute/cuda/GpuMatmul.cpp:786-884).
class Blas {
  public:
    Blas();
    ~Blas();
    // out[M, N] (bf16 or fp32) = x[M, K] (bf16) * W[N, K]^T (bf16), fp32 accumulation
    void gemm_nt(const void* x, const void* W, void* out, int out_dtype, int M, int N, int K, cudaStream_t s);

  private:
    struct Impl;
    std::unique_ptr<Impl> impl_;
};

// Tunables of the dispatch (the measured thresholds; tests move them to reach every kernel).
struct Options {
    int prefill_min = 16;             // shorter portions go token by token through the decode kernel
    int use_tcgen05_prefill = 1;
    int use_tma_decode = 1;
    int tma_decode_stages = 3;
    int target_ctas = 2 * 148;        // decode CTAs wanted
    int use_cluster_merge = 1;
    int cluster_max_wanted = 12;
    int fixed_split = 0;              // > 0: cut keys by absolute position into splits of this length
    int gemv_max_rows = 8;
    int skinny_max_rows = 64;
    int tcgen05_swiglu_min_rows = 256;
    int tcgen05_pair_min_rows = 256;
    int use_side_stream = 1;          // a mixed step's decode attention runs beside its prefill attention
};
Options& options();

bool gemv_supported(int m, int n, int k);
bool skinny_supported(int m, int n, int k);
inline bool small_batch_supported(int m, int n, int k) { return gemv_supported(m, n, k) || skinny_supported(m, n, k); }

// y = x * W^T in out_dtype (-1: x's dtype), W stored [out, in]; into `into` if given, else into memory of `mem`
Rows linear(Step&, Arena& mem, const Rows& x, const Tensor& W, int out_dtype = -1, void* into = nullptr);
// the weight-streaming products of a few rows with their fused epilogues
Rows small_product(Step&, Arena& mem, const Act& x, const Tensor& W, int out_dtype, bool swiglu);
Out small_product_residual(Step&, Arena& mem, const Rows& x, const Tensor& W, const Sink& sink);

}  // namespace mmx
