// Native classes of the part kinds this library ships: RMSNorm, the split-half rotary encoding (and "none"),
// grouped-query attention over the paged cache, the gated feed-forward, the pre-norm block, the token embedding and
// the output head.  Each takes its sizes and constants from its description; none knows which model it is in.
// The formulas and their places in the reference are cited at the kernels they launch (csrc/*.cu).
#include <algorithm>
#include <cmath>

#include "exec.h"
#include "kernels_api.h"

namespace mmx {

void qkv_rope_small(Step& st, const Act& x, const Tensor& W, const Tensor* bias, void* q_out, void* k_pages, void* v_pages, const void* table,
                    const void* slots, int page_size, int H, int G, int hd);

namespace {

// ---- RMSNorm: y = x * w / sqrt(mean(x^2) + eps), the residual add before it fused in ------------------------------
struct RMSNorm : Norm {
    int width;
    float eps;
    Tensor weight;
    explicit RMSNorm(const PartDesc& d) : width(d.geti("width")), eps((float)d.get("eps")), weight(d.tensor("weight")) {
        if (weight.ndim != 1 || weight.shape[0] != width) throw ExecError("rmsnorm: the weight does not have the norm's width");
    }
    Rows forward(Step& st, Arena& mem, float* residual, const Rows* delta, const int* rows, int n_rows) override {
        const int n = rows ? n_rows : st.n_tokens;
        Rows out{mem.alloc((size_t)n * width * dtype_size(st.act_dtype)), st.act_dtype, n, width};
        if (delta && (delta->dtype != st.act_dtype || delta->width != width)) throw ExecError("rmsnorm: delta and residual differ");
        check_kernel(mm_add_rmsnorm(residual, delta ? delta->ptr : nullptr, rows, weight.ptr, weight.dtype, out.ptr, st.act_dtype, n, width, eps,
                                    st.stream), "rmsnorm");
        return out;
    }
    bool factors(const Tensor** w, float* e) const override {
        *w = &weight;
        *e = eps;
        return true;
    }
};
Registrar r_rmsnorm("norm", "rmsnorm", [](const PartDesc& d) { return std::unique_ptr<Part>(new RMSNorm(d)); });

// ---- position encodings the fused kernels apply -----------------------------------------------------------------------
struct RotaryHalf : PositionEncoding {
    int rotary_dim;
    float theta;
    explicit RotaryHalf(const PartDesc& d) : rotary_dim(d.geti("rotary_dim")), theta((float)d.get("theta")) {
        if (rotary_dim % 2) throw ExecError("rotary_half: rotary_dim must be even");
    }
    bool fused_rotary(int* rd, float* th) const override {
        *rd = rotary_dim;
        *th = theta;
        return true;
    }
};
Registrar r_rotary("position", "rotary_half", [](const PartDesc& d) { return std::unique_ptr<Part>(new RotaryHalf(d)); });

struct NoPosition : PositionEncoding {
    bool fused_rotary(int* rd, float* th) const override {
        *rd = 0;
        *th = 1.f;
        return true;
    }
};
Registrar r_nopos("position", "none", [](const PartDesc&) { return std::unique_ptr<Part>(new NoPosition()); });

// ---- attention ---------------------------------------------------------------------------------------------------------
// Launch plan of the tensor-core attention kernels, made once per step for each head geometry: portions of at least
// prefill_min tokens become tiles of query rows of one request, the other tokens decode items; the decode kernel
// cuts each token's key range into splits so that the grid fills the GPU.
struct AttentionPlan {
    int n_tiles = 0, tile_rows = 0, n_items = 0, split_len = 0, max_splits = 1;
    bool cluster = false, all_items = false;
    const int* tiles = nullptr;       // device int32 [n_tiles, 4]: request, first row, rows, first position
    const int* items = nullptr;       // device int32 [n_items]; null with all_items
    float* part_o = nullptr;
    float* part_ml = nullptr;
};

int cluster_capacity(int head_dim, int size) {
    static std::map<std::pair<int, int>, int> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    auto key = std::make_pair(dev * 1024 + head_dim, size);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    int n = 0;
    check_kernel(mm_attention_decode_tma_max_clusters(head_dim, size, &n), "attention_decode_tma_max_clusters");
    cache[key] = n;
    return n;
}

bool tma_page(int ps) { return ps == 8 || ps == 16 || ps == 32 || ps == 64; }

// (split_len, max_splits, cluster) of the decode kernel.  split_len 0: every token's key range is cut evenly into at
// most max_splits pieces of whole 64-key tiles.  cluster: the splits of a token are one thread-block cluster that
// merges itself through distributed shared memory.
void choose_split(int n_items, int G, int max_kv_len, int head_dim, int page_size, AttentionPlan& p) {
    const Options& o = options();
    if (o.fixed_split > 0) {
        p.split_len = o.fixed_split;
        p.max_splits = std::max(1, (max_kv_len + o.fixed_split - 1) / o.fixed_split);
        p.cluster = false;
        return;
    }
    p.split_len = 0;
    p.max_splits = 1;
    p.cluster = false;
    const int ctas = std::max(1, n_items * G);
    if (ctas >= o.target_ctas / 2) return;      // one CTA per SM or more already: a split would only add the merge pass
    const int wanted = std::max(1, std::min(o.target_ctas / ctas, (max_kv_len + 63) / 64));
    if (o.use_tma_decode && o.use_cluster_merge && (head_dim == 64 || head_dim == 128) && tma_page(page_size) && wanted >= 2) {
        int size = 1;
        while (size * 2 <= std::min(wanted, 8)) size *= 2;
        if ((wanted >= 8 || 4 * size >= 3 * wanted) && wanted <= o.cluster_max_wanted && ctas <= cluster_capacity(head_dim, size)) {
            p.max_splits = size;
            p.cluster = true;
            return;
        }
    }
    p.max_splits = wanted;
}

bool tensor_core_attention(int hd, int H, int G) { return (hd == 64 || hd == 128) && H % G == 0 && H / G <= 16; }

struct GQAAttention : Mixer {
    int hidden, H, G, hd, window;
    float scale;
    bool interleaved;
    Tensor w_qkv, w_o;
    const Tensor* b_qkv = nullptr;
    Tensor bias_store;
    std::unique_ptr<PositionEncoding> position;

    explicit GQAAttention(const PartDesc& d)
        : hidden(d.geti("hidden")), H(d.geti("num_heads")), G(d.geti("num_kv_heads")), hd(d.geti("head_dim")), window(d.geti("window")),
          scale((float)d.get("scale")), interleaved(d.geti("interleaved") != 0), w_qkv(d.tensor("w_qkv")), w_o(d.tensor("w_o")) {
        if (const Tensor* b = d.tensor_or_null("b_qkv")) {
            bias_store = *b;
            b_qkv = &bias_store;
        }
        position = build_as<PositionEncoding>("position", d.child("position"));
        if (G < 1 || H % G) throw ExecError("gqa_attention: num_heads must be a multiple of num_kv_heads");
        const long long width = (long long)(H + 2 * G) * hd;
        if (w_qkv.ndim != 2 || w_qkv.shape[0] != width || w_qkv.shape[1] != hidden || w_o.ndim != 2 || w_o.shape[0] != hidden ||
            w_o.shape[1] != (long long)H * hd)
            throw ExecError("gqa_attention: projection weights do not have the sizes of the description");
    }

    bool fuses(const Step&, int n) const override {
        const int width = (H + 2 * G) * hd;
        return interleaved && small_batch_supported(n, width, hidden) && small_batch_supported(n, hidden, H * hd);
    }

    std::string plan_key() const { return "attention_bf16/" + std::to_string(H) + "/" + std::to_string(G) + "/" + std::to_string(hd); }

    bool uses_plan(const Step& st) const { return st.act_dtype == BF16 && tensor_core_attention(hd, H, G); }

    void prepare(Step& st, const LayerCache* cache) override {
        if (!uses_plan(st) || !cache || st.plans.count(plan_key())) return;
        const Options& o = options();
        auto plan = std::make_shared<AttentionPlan>();
        const bool tc = o.use_tcgen05_prefill && (hd == 128 || hd == 64) && (tma_page(st.page_size) || st.page_size == 128);
        plan->tile_rows = tc ? 128 : 64;
        struct Tile {
            int r, first, rows, pos;
        };
        std::vector<Tile> tiles;
        std::vector<int> items;
        for (int r = 0; r < st.n_requests; ++r) {
            const int s = st.q_start[r], n = st.q_len[r], kv = st.kv_len[r];
            if (n >= o.prefill_min) {
                for (int off = 0; off < n; off += plan->tile_rows) tiles.push_back({r, s + off, std::min(plan->tile_rows, n - off), kv - n + off});
            } else {
                for (int i = s; i < s + n; ++i) items.push_back(i);
            }
        }
        // by keys seen, ascending: the kernels start from the far end
        std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& a, const Tile& b) { return a.pos + a.rows < b.pos + b.rows; });
        plan->n_tiles = (int)tiles.size();
        plan->n_items = (int)items.size();
        plan->all_items = plan->n_items == st.n_tokens;
        if (plan->n_tiles) {
            Step::Upload up;
            up.data.reserve(tiles.size() * 4);
            for (auto& t : tiles) {
                up.data.push_back(t.r);
                up.data.push_back(t.first);
                up.data.push_back(t.rows);
                up.data.push_back(t.pos);
            }
            up.where = &plan->tiles;
            st.uploads.push_back(std::move(up));
        }
        if (plan->n_items && !plan->all_items) {
            Step::Upload up;
            up.data = std::move(items);
            up.where = &plan->items;
            st.uploads.push_back(std::move(up));
        }
        if (plan->n_items) choose_split(plan->n_items, G, st.max_kv_len, hd, st.page_size, *plan);
        st.plans[plan_key()] = plan;
    }

    void attention(Step& st, const void* q, void* out, LayerCache& cache) {
        void* s = st.stream;
        if (!uses_plan(st)) {
            check_kernel(mm_attention_generic(q, cache.k_pages, cache.v_pages, out, st.act_dtype, st.positions, st.token_req, cache.table,
                                              cache.table_width, cache.page_size, st.n_tokens, H, G, hd, window, scale, s), "attention_generic");
            return;
        }
        auto it = st.plans.find(plan_key());
        if (it == st.plans.end()) throw ExecError("attention: the step was not prepared");
        AttentionPlan& p = *static_cast<AttentionPlan*>(it->second.get());
        const Options& o = options();
        // prompt portions and single tokens are two kernels over disjoint rows of q and out: in a step that has both, the
        // second runs beside the first on the step's side stream (measured at the 7B shape, 8 single tokens beside a
        // portion: 192 tokens 6.11 -> 5.70 ms per step, 100 tokens 5.19 -> 5.15, 56 tokens no gain)
        const bool beside = p.n_tiles && p.n_items && st.side != nullptr && o.use_side_stream && st.n_tokens - p.n_items >= 128;
        if (beside) st.fork();
        if (p.n_tiles && p.tile_rows == 128) {
            check_kernel(mm_attention_prefill_tcgen05(q, cache.k_pages, cache.v_pages, out, p.tiles, p.n_tiles, cache.table, cache.table_width,
                                                      cache.page_size, cache.num_pages, st.n_tokens, H, G, hd, window, scale, st.err, s),
                         "attention_prefill_tcgen05");
        } else if (p.n_tiles) {
            check_kernel(mm_attention_prefill_bf16(q, cache.k_pages, cache.v_pages, out, p.tiles, p.n_tiles, cache.table, cache.table_width,
                                                   cache.page_size, H, G, hd, window, scale, s), "attention_prefill_bf16");
        }
        if (!p.n_items) return;
        if (beside) s = st.side;
        if (p.max_splits > 1 && !p.cluster && !p.part_o) {
            p.part_o = st.step_mem->alloc_n<float>((size_t)p.n_items * H * p.max_splits * hd);
            p.part_ml = st.step_mem->alloc_n<float>((size_t)p.n_items * H * p.max_splits * 2);
        }
        if (o.use_tma_decode && tma_page(cache.page_size)) {
            check_kernel(mm_attention_decode_tma_bf16(q, cache.k_pages, cache.v_pages, out, p.part_o, p.part_ml, p.items, p.n_items, st.positions,
                                                      st.token_req, cache.table, cache.table_width, cache.page_size, cache.num_pages, H, G, hd, window,
                                                      scale, p.split_len, p.max_splits, o.tma_decode_stages, p.cluster ? 1 : 0, st.err, s),
                         "attention_decode_tma_bf16");
            if (p.max_splits > 1 && !p.cluster)
                check_kernel(mm_attention_decode_merge_bf16(out, p.part_o, p.part_ml, p.items, p.n_items, st.positions, H, hd, window, p.split_len,
                                                            p.max_splits, s), "attention_decode_merge_bf16");
        } else {
            check_kernel(mm_attention_decode_bf16(q, cache.k_pages, cache.v_pages, out, p.part_o, p.part_ml, p.items, p.n_items, st.positions,
                                                  st.token_req, cache.table, cache.table_width, cache.page_size, H, G, hd, window, scale, p.split_len,
                                                  p.max_splits, s), "attention_decode_bf16");
        }
        if (beside) st.join();
    }

    Out forward(Step& st, Arena& mem, const Act& x, LayerCache& cache, const Sink* sink) override {
        const int n = st.n_tokens;
        void* s = st.stream;
        void* k_pages = cache.writes ? cache.k_pages : nullptr;
        void* v_pages = cache.writes ? cache.v_pages : nullptr;
        int rotary_dim = 0;
        float theta = 1.f;
        position->fused_rotary(&rotary_dim, &theta);
        const size_t esz = dtype_size(st.act_dtype);
        void* q = mem.alloc((size_t)n * H * hd * esz);
        // rotation factors and cache places are the same in every layer that shares them: made once per step
        const bool tables = rotary_dim == hd && hd % 16 == 0 && st.act_dtype == BF16;
        const void* table = nullptr;
        const void* slots = nullptr;
        if (tables) {
            const std::string key = "rope_table/" + std::to_string(hd) + "/" + std::to_string(theta);
            auto it = st.derived.find(key);
            if (it == st.derived.end()) {
                float* t = st.step_mem->alloc_n<float>((size_t)n * hd);
                check_kernel(mm_rope_table(st.positions, t, n, hd, theta, s), "rope_table");
                it = st.derived.emplace(key, t).first;
            }
            table = it->second;
            if (k_pages) {
                const std::string skey = "slots/" + std::to_string(cache.group);
                auto is = st.derived.find(skey);
                if (is == st.derived.end()) {
                    int* sl = st.step_mem->alloc_n<int>(n);
                    check_kernel(mm_slot_mapping(st.positions, st.token_req, cache.table, cache.table_width, cache.page_size, n, sl, s), "slot_mapping");
                    is = st.derived.emplace(skey, sl).first;
                }
                slots = is->second;
            }
        }
        if (fuses(st, n)) {
            // a few tokens: projection, 1/rms of a factored input, bias, rotation and cache write in one launch
            qkv_rope_small(st, x, w_qkv, b_qkv, q, k_pages, v_pages, table, slots, cache.page_size, H, G, hd);
        } else {
            if (x.factored) throw ExecError("attention: factored rows handed to a projection that does not fuse");
            Rows qkv = linear(st, mem, x.rows, w_qkv);
            const void* b = b_qkv ? b_qkv->ptr : nullptr;
            const int bd = b_qkv ? b_qkv->dtype : F32;
            if (tables && qkv.dtype == BF16) {
                check_kernel(mm_qkv_rope_tables(qkv.ptr, b, bd, q, k_pages, v_pages, table, slots, cache.page_size, n, H, G, hd, interleaved ? 1 : 0, s),
                             "qkv_rope_tables");
            } else {
                check_kernel(mm_qkv_rope_kvwrite(qkv.ptr, b, bd, q, k_pages, v_pages, st.act_dtype, st.positions, st.token_req, cache.table,
                                                 cache.table_width, cache.page_size, n, H, G, hd, rotary_dim, theta, interleaved ? 1 : 0, s),
                             "qkv_rope_kvwrite");
            }
        }
        void* attn = mem.alloc((size_t)n * H * hd * esz);
        attention(st, q, attn, cache);
        Rows a{attn, st.act_dtype, n, H * hd};
        if (!sink) {
            Out out;
            out.kind = Out::ROWS;
            out.rows = linear(st, mem, a, w_o);
            return out;
        }
        return small_product_residual(st, mem, a, w_o, *sink);
    }
};
Registrar r_gqa("mixer", "gqa_attention", [](const PartDesc& d) { return std::unique_ptr<Part>(new GQAAttention(d)); });

// ---- gated feed-forward: y = (silu(x Wg^T) * x Wu^T) Wd^T -----------------------------------------------------------------
struct SwiGLU : FeedForward {
    int hidden, intermediate, interleave;
    Tensor w_gate_up, w_down;
    explicit SwiGLU(const PartDesc& d)
        : hidden(d.geti("hidden")), intermediate(d.geti("intermediate")), interleave(d.geti("interleave")), w_gate_up(d.tensor("w_gate_up")),
          w_down(d.tensor("w_down")) {
        if (w_gate_up.ndim != 2 || w_gate_up.shape[0] != 2LL * intermediate || w_gate_up.shape[1] != hidden || w_down.ndim != 2 ||
            w_down.shape[0] != hidden || w_down.shape[1] != intermediate)
            throw ExecError("swiglu: weights do not have the sizes of the description");
    }
    bool tensor_cores(const Step& st) const {
        return interleave != 0 && st.act_dtype == BF16 && w_gate_up.dtype == BF16 && w_down.dtype == BF16 && !st.simt;
    }
    bool fuses(const Step& st, int m) const override {
        return tensor_cores(st) && small_batch_supported(m, 2 * intermediate, hidden) && small_batch_supported(m, hidden, intermediate);
    }
    Out forward(Step& st, Arena& mem, const Act& x, const Sink* sink) override {
        const int m = x.n();
        Out out;
        if (fuses(st, m)) {
            // a few tokens: two weight-streaming products; 1/rms and activation in the first one's epilogue, residual add
            // and the next norm in the second one's
            Rows act = small_product(st, mem, x, w_gate_up, BF16, true);
            if (!sink) {
                Act a;
                a.rows = act;
                out.kind = Out::ROWS;
                out.rows = small_product(st, mem, a, w_down, BF16, false);
                return out;
            }
            return small_product_residual(st, mem, act, w_down, *sink);
        }
        if (x.factored || sink) throw ExecError("swiglu: factored rows or a sink handed to a feed-forward that does not fuse");
        const Options& o = options();
        Rows act;
        const int n2 = 2 * intermediate;
        if (tensor_cores(st) && m >= o.tcgen05_swiglu_min_rows && hidden % 8 == 0 && n2 % 16 == 0 && hidden >= 64) {
            // prefill-sized: tcgen05 product with the activation as its epilogue (the [m, 2F] intermediate never exists)
            act = Rows{mem.alloc((size_t)m * intermediate * 2), BF16, m, intermediate};
            const bool pair = m >= o.tcgen05_pair_min_rows && (m - 1) % 256 >= 128;
            auto fn = pair ? mm_gemm_tcgen05_pair : mm_gemm_tcgen05;
            check_kernel(fn(x.rows.ptr, w_gate_up.ptr, nullptr, F32, act.ptr, 1 /* SwiGLU epilogue */, m, n2, hidden, hidden, intermediate, st.err,
                            st.stream), "gemm_tcgen05");
        } else {
            Rows gu = linear(st, mem, x.rows, w_gate_up);
            act = Rows{mem.alloc((size_t)m * intermediate * dtype_size(gu.dtype)), gu.dtype, m, intermediate};
            check_kernel(mm_silu_mul(gu.ptr, act.ptr, act.dtype, m, intermediate, interleave, st.stream), "silu_mul");
        }
        out.kind = Out::ROWS;
        out.rows = linear(st, mem, act, w_down);
        return out;
    }
};
Registrar r_swiglu("feed_forward", "swiglu", [](const PartDesc& d) { return std::unique_ptr<Part>(new SwiGLU(d)); });

// ---- pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x)) ----------------------------------------------------
// The last add of a layer is left pending so that it fuses into the norm that follows, whichever layer owns it.  With
// parts that fuse (a few tokens in bfloat16) the residual add and the norm move into the epilogue of the branch's
// last product and the 1/rms into the next product: a layer is five launches.
struct PreNormBlock : Block {
    std::unique_ptr<Norm> mixer_norm, ffn_norm;
    std::unique_ptr<Mixer> mixer;
    std::unique_ptr<FeedForward> feed_forward;
    explicit PreNormBlock(const PartDesc& d) {
        mixer_norm = build_as<Norm>("norm", d.child("mixer_norm"));
        mixer = build_as<Mixer>("mixer", d.child("mixer"));
        ffn_norm = build_as<Norm>("norm", d.child("ffn_norm"));
        feed_forward = build_as<FeedForward>("feed_forward", d.child("feed_forward"));
    }
    void prepare(Step& st, const LayerCache* cache) override {
        mixer_norm->prepare(st, cache);
        mixer->prepare(st, cache);
        ffn_norm->prepare(st, cache);
        feed_forward->prepare(st, cache);
    }
    bool entry_norm(const Step& st, int n, const Tensor** w, float* eps) const override {
        return mixer_norm->factors(w, eps) && mixer->fuses(st, n);
    }
    Pending forward(Step& st, float* residual, const Pending& pending, LayerCache& cache, Block* successor) override {
        const int n = st.n_tokens;
        Arena& mem = *st.layer_mem;
        const bool mixer_fuses = mixer->fuses(st, n), ffn_fuses = feed_forward->fuses(st, n);
        Act h;
        if (pending.kind == Pending::FACTORED) {
            h.factored = true;
            h.f = pending.f;
        } else {
            h.rows = mixer_norm->forward(st, mem, residual, pending.kind == Pending::DELTA ? &pending.delta : nullptr, nullptr, 0);
        }
        const Tensor* w = nullptr;
        float eps = 0.f;
        const bool between = mixer_fuses && ffn_fuses && ffn_norm->factors(&w, &eps);
        Act h2;
        if (between) {
            Sink sink{residual, w, eps};
            Out o = mixer->forward(st, mem, h, cache, &sink);
            h2.factored = true;
            h2.f = o.f;
        } else {
            Out o = mixer->forward(st, mem, h, cache, nullptr);
            h2.rows = ffn_norm->forward(st, mem, residual, &o.rows, nullptr, 0);
        }
        Pending result;
        auto plain = [&]() {
            Out o = feed_forward->forward(st, mem, h2, nullptr);
            result.kind = Pending::DELTA;
            result.delta = o.rows;
        };
        if (!ffn_fuses) {
            plain();
            return result;
        }
        const Tensor* aw = nullptr;
        float aeps = 0.f;
        const bool after = successor && successor->entry_norm(st, n, &aw, &aeps);
        if (successor && !after) {      // the next block wants a plain pending sum
            plain();
            return result;
        }
        Sink sink{residual, after ? aw : nullptr, aeps};
        Out o = feed_forward->forward(st, mem, h2, &sink);
        if (o.kind == Out::FACTORED) {
            result.kind = Pending::FACTORED;
            result.f = o.f;
        }
        return result;
    }
};
Registrar r_prenorm("block", "pre_norm", [](const PartDesc& d) { return std::unique_ptr<Part>(new PreNormBlock(d)); });

// ---- embedding and head ------------------------------------------------------------------------------------------------------
struct TokenEmbedding : Embedding {
    int vocab_, width_;
    float scale;
    Tensor table;
    explicit TokenEmbedding(const PartDesc& d) : vocab_(d.geti("vocab")), width_(d.geti("width")), scale((float)d.get("scale", 1.0)), table(d.tensor("table")) {
        if (table.ndim != 2 || table.shape[0] != vocab_ || table.shape[1] != width_) throw ExecError("token_embedding: the table does not have the sizes of the description");
    }
    int width() const override { return width_; }
    float* forward(Step& st, Arena& mem) override {
        float* out = mem.alloc_n<float>((size_t)st.n_tokens * width_);
        check_kernel(mm_embedding(st.token_ids, table.ptr, table.dtype, out, st.n_tokens, vocab_, width_, scale, st.stream), "embedding");
        return out;
    }
};
Registrar r_embedding("embedding", "token_embedding", [](const PartDesc& d) { return std::unique_ptr<Part>(new TokenEmbedding(d)); });

struct LMHead : Head {
    int vocab_;
    Tensor weight;
    explicit LMHead(const PartDesc& d) : vocab_(d.geti("vocab")), weight(d.tensor("weight")) {
        if (weight.ndim != 2 || weight.shape[0] != vocab_) throw ExecError("lm_head: the weight does not have the sizes of the description");
    }
    int vocab() const override { return vocab_; }
    void forward(Step& st, Arena& mem, const Rows& x, float* logits) override { linear(st, mem, x, weight, F32, logits); }
};
Registrar r_head("head", "lm_head", [](const PartDesc& d) { return std::unique_ptr<Part>(new LMHead(d)); });

}  // namespace
}  // namespace mmx
