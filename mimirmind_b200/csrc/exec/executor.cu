// The native step: from (request, its next tokens) entries to logits at the wanted places, in one call.
//
// mmx_exec_run checks the entries against the cache manager (csrc/host/runtime.cpp), reserves their pages when asked
// to, writes the step's integers (token ids, absolute positions, token -> request, wanted rows, one block-table row
// per request and cache group, the attention work lists) into a pinned buffer, copies them to the device once, and
// launches embedding, every schedule entry's block, the final norm on the wanted rows and the head.  mmx_exec_forward
// runs the same launches on buffers the caller keeps on the device (a decode step captured in a CUDA graph).
// The reference has a one-token-per-slot step and a per-request prefill as separate native calls
// (src/runtime/engine/ServingSession.cpp:856-947, 949-1093); here any mix is one call.
#include <algorithm>
#include <cstring>
#include <unordered_set>

#include "../host/runtime_api.h"
#include "exec.h"
#include "kernels_api.h"

#define MMX_EXPORT extern "C" __attribute__((visibility("default")))

namespace mmx {

struct ScheduleEntry {
    int layer, cache_from;
};

struct Model {
    std::unique_ptr<Embedding> embedding;
    std::unique_ptr<Norm> final_norm;
    std::unique_ptr<Head> head;
    std::vector<std::unique_ptr<Block>> layers;
    std::vector<ScheduleEntry> schedule;
    int act_dtype = BF16;
    bool simt = false;
};

struct EntryCache {
    void* k_pages;
    void* v_pages;
    int group;       // -1: the entry keeps no keys and values
    bool writes;
};

// what the caller of mmx_exec_forward describes: device arrays it keeps, host facts about the batch
struct StepDesc {
    int n_tokens, n_requests, n_logit_rows, max_kv_len, max_q_len, table_width;
    const int* token_ids;
    const int* positions;
    const int* token_req;
    const int* logit_rows;
    const int* tables[MAX_GROUPS];
    const int* q_start;      // host, [n_requests]
    const int* q_len;
    const int* kv_len;
};

constexpr int RUN_RESERVE = 1, RUN_COMMIT = 2;

class Executor {
  public:
    Executor(Model* model, void* cache, int page_size, std::vector<int> group_pages, std::vector<EntryCache> entries, int vocab, int max_seq_len, void* err)
        : model_(model), cache_(cache), page_size_(page_size), group_pages_(std::move(group_pages)), entries_(std::move(entries)), vocab_(vocab),
          max_seq_len_(max_seq_len), err_(err), step_mem_(8u << 20), layer_mem_{Arena(16u << 20), Arena(16u << 20)} {
        if (entries_.size() != model_->schedule.size()) throw ExecError("executor: one cache entry per schedule entry");
        if ((int)group_pages_.size() > MAX_GROUPS) throw ExecError("executor: too many cache groups");
        check_cuda(cudaMallocHost((void**)&err_host_, sizeof(int)), "pinned error flag");
        *err_host_ = 0;
        check_cuda(cudaStreamCreateWithFlags(&side_, cudaStreamNonBlocking), "the executor's side stream");
        check_cuda(cudaEventCreateWithFlags(&forked_, cudaEventDisableTiming), "fork event");
        check_cuda(cudaEventCreateWithFlags(&joined_, cudaEventDisableTiming), "join event");
    }
    ~Executor() {
        for (auto& s : ring_) {
            if (s.host) cudaFreeHost(s.host);
            if (s.copied) cudaEventDestroy(s.copied);
        }
        if (err_host_) cudaFreeHost(err_host_);
        if (forked_) cudaEventDestroy(forked_);
        if (joined_) cudaEventDestroy(joined_);
        if (side_) cudaStreamDestroy(side_);
    }

    int n_groups() const { return (int)group_pages_.size(); }

    // ---- the launches of a step whose integers are on the device -------------------------------------------------------
    void forward(Step& st, float* logits) {
        Model& m = *model_;
        float* residual = m.embedding->forward(st, *st.step_mem);
        Pending pending;
        const int last = (int)m.schedule.size() - 1;
        for (int i = 0; i <= last; ++i) {
            Arena& mem = layer_mem_[i & 1];
            mem.reset();
            st.layer_mem = &mem;
            LayerCache lc = layer_cache(i, st);
            Block* successor = i < last ? m.layers[m.schedule[i + 1].layer].get() : nullptr;
            pending = m.layers[m.schedule[i].layer]->forward(st, residual, pending, lc, successor);
        }
        if (st.n_logit_rows == 0) return;
        if (pending.kind == Pending::FACTORED) throw ExecError("the last block left factored rows that no block takes");
        Arena& mem = layer_mem_[(last + 1) & 1];
        mem.reset();
        Rows normed = m.final_norm->forward(st, mem, residual, pending.kind == Pending::DELTA ? &pending.delta : nullptr, st.logit_rows, st.n_logit_rows);
        m.head->forward(st, mem, normed, logits);
    }

    LayerCache layer_cache(int entry, const Step& st) const {
        const EntryCache& e = entries_[entry];
        LayerCache lc;
        lc.page_size = page_size_;
        lc.writes = e.writes;
        lc.group = e.group;
        if (e.group >= 0) {
            lc.k_pages = e.k_pages;
            lc.v_pages = e.v_pages;
            lc.table = st.tables[e.group];
            lc.table_width = st.table_width;
            lc.num_pages = std::max(group_pages_[e.group], 1);
        }
        return lc;
    }

    void init_step(Step& st, cudaStream_t stream) {
        st.act_dtype = model_->act_dtype;
        st.simt = model_->simt;
        st.stream = stream;
        st.err = err_;
        st.page_size = page_size_;
        step_mem_.reset();
        st.step_mem = &step_mem_;
        if (!blas_) blas_.reset(new Blas());
        st.blas = blas_.get();
        st.side = side_;
        st.forked = forked_;
        st.joined = joined_;
    }

    void prepare(Step& st) {
        Model& m = *model_;
        for (size_t i = 0; i < m.schedule.size(); ++i) {
            LayerCache lc = layer_cache((int)i, st);
            m.layers[m.schedule[i].layer]->prepare(st, &lc);
        }
    }

    // ---- staging: a ring of pinned buffers, each reused only after its last copy has run -----------------------------------
    struct Staging {
        int* host = nullptr;
        size_t cap = 0;
        cudaEvent_t copied = nullptr;
        bool in_flight = false;
    };
    Staging& next_staging(size_t ints) {
        Staging& s = ring_[ring_next_];
        ring_next_ = (ring_next_ + 1) % (int)(sizeof(ring_) / sizeof(ring_[0]));
        if (s.in_flight) {
            check_cuda(cudaEventSynchronize(s.copied), "waiting for a staging buffer");
            s.in_flight = false;
        }
        if (s.cap < ints) {
            if (s.host) cudaFreeHost(s.host);
            s.host = nullptr;
            s.cap = std::max(ints * 2, (size_t)16384);
            check_cuda(cudaMallocHost((void**)&s.host, s.cap * sizeof(int)), "pinned staging buffer");
        }
        if (!s.copied) check_cuda(cudaEventCreateWithFlags(&s.copied, cudaEventDisableTiming), "staging event");
        return s;
    }

    // copies `fixed` ints (already in s.host) and the step's uploads to the device in one copy; returns the device base
    const int* copy_step(Step& st, Staging& s, size_t fixed) {
        size_t total = fixed;
        for (auto& u : st.uploads) total += (u.data.size() + 3) & ~(size_t)3;
        if (total == 0) return nullptr;
        if (total > s.cap) throw ExecError("executor: staging buffer too small");     // sized by the caller
        size_t off = fixed;
        std::vector<size_t> offs;
        for (auto& u : st.uploads) {
            std::memcpy(s.host + off, u.data.data(), u.data.size() * sizeof(int));
            offs.push_back(off);
            off += (u.data.size() + 3) & ~(size_t)3;
        }
        int* dev = st.step_mem->alloc_n<int>(total);
        check_cuda(cudaMemcpyAsync(dev, s.host, total * sizeof(int), cudaMemcpyHostToDevice, st.stream), "copying the step's integers");
        check_cuda(cudaEventRecord(s.copied, st.stream), "staging event");
        s.in_flight = true;
        for (size_t i = 0; i < st.uploads.size(); ++i) *st.uploads[i].where = dev + offs[i];
        st.uploads.clear();
        return dev;
    }

    size_t upload_ints(const Step& st) const {
        size_t n = 0;
        for (auto& u : st.uploads) n += (u.data.size() + 3) & ~(size_t)3;
        return n;
    }

    // ---- one step from entries -------------------------------------------------------------------------------------------------
    // Returns the number of logits rows written.
    int run(int n_entries, const long long* rids, const int* counts, const int* tokens, const int* n_want, const int* want, int flags, float* logits,
            long long logits_rows_cap, cudaStream_t stream) {
        if (n_entries <= 0) return 0;
        const int G = n_groups(), ps = page_size_;
        // -- what the step refuses, before anything changes
        std::unordered_set<long long> seen;
        std::vector<int> start(n_entries);
        int n_tok = 0, n_rows = 0;
        for (int r = 0; r < n_entries; ++r) {
            if (counts[r] < 1) throw StepRefused("request " + std::to_string(r) + " of the step: an entry needs at least one token");
            if (!seen.insert(rids[r]).second) throw StepRefused("a request appears twice in one step");
            if (!mmh_cache_has(cache_, rids[r])) throw StepRefused("unknown request");
            start[r] = mmh_cache_request(cache_, rids[r], 0);
            if (start[r] + counts[r] > max_seq_len_)
                throw StepRefused(std::to_string(start[r] + counts[r]) + " tokens exceed the context of " + std::to_string(max_seq_len_));
            for (int i = 0; i < counts[r]; ++i)
                if (tokens[n_tok + i] < 0 || tokens[n_tok + i] >= vocab_) throw StepRefused("token id outside [0, " + std::to_string(vocab_) + ")");
            for (int i = 0; i < n_want[r]; ++i)
                if (want[n_rows + i] < 0 || want[n_rows + i] >= counts[r])
                    throw StepRefused("wanted place " + std::to_string(want[n_rows + i]) + " is outside the entry's " + std::to_string(counts[r]) + " tokens");
            n_tok += counts[r];
            n_rows += n_want[r];
        }
        if (logits != nullptr && n_rows > logits_rows_cap) throw ExecError("executor: the logits buffer is too small for the wanted rows");
        if (flags & RUN_RESERVE) {
            // pages for every entry: the step runs fully or not at all
            std::vector<int> need(G, 0), one(std::max(G, 1));
            for (int r = 0; r < n_entries; ++r) {
                if (mmh_cache_pages_needed(cache_, rids[r], start[r] + counts[r], one.data()) != 0) throw ExecError(mmh_last_error());
                for (int g = 0; g < G; ++g) need[g] += one[g];
            }
            for (int g = 0; g < G; ++g) {
                const int free_pages = mmh_cache_info(cache_, 3, g);
                if (need[g] > free_pages)
                    throw StepRefused("out of cache pages in group " + std::to_string(g) + ": the step needs " + std::to_string(need[g]) + ", " +
                                      std::to_string(free_pages) + " of " + std::to_string(mmh_cache_info(cache_, 2, g)) + " are free");
            }
            for (int r = 0; r < n_entries; ++r)
                if (mmh_cache_reserve(cache_, rids[r], start[r] + counts[r]) != 1) throw ExecError("executor: reserving checked pages failed");
        }
        for (int r = 0; r < n_entries; ++r) mmh_cache_request(cache_, rids[r], 3);      // the request has started (its state slot is in use)

        // -- the batch
        Step st;
        init_step(st, stream);
        st.n_tokens = n_tok;
        st.n_requests = n_entries;
        st.n_logit_rows = n_rows;
        st.q_start.resize(n_entries);
        st.q_len.assign(counts, counts + n_entries);
        st.kv_len.resize(n_entries);
        int at = 0;
        for (int r = 0; r < n_entries; ++r) {
            st.q_start[r] = at;
            st.kv_len[r] = start[r] + counts[r];
            st.max_kv_len = std::max(st.max_kv_len, st.kv_len[r]);
            st.max_q_len = std::max(st.max_q_len, counts[r]);
            at += counts[r];
        }
        st.table_width = std::max(1, (st.max_kv_len + ps - 1) / ps);
        prepare(st);

        // -- one pinned buffer, one copy: ids | positions | token -> request | wanted rows | a table per group | work lists
        auto pad4 = [](size_t n) { return (n + 3) & ~(size_t)3; };
        const size_t o_ids = 0, o_pos = o_ids + pad4(n_tok), o_req = o_pos + pad4(n_tok), o_rows = o_req + pad4(n_tok),
                     o_tab = o_rows + pad4(std::max(n_rows, 1)), tab = pad4((size_t)n_entries * st.table_width), fixed = o_tab + tab * G;
        Staging& sg = next_staging(fixed + upload_ints(st));
        int* h = sg.host;
        std::memcpy(h + o_ids, tokens, sizeof(int) * n_tok);
        int row = 0, wi = 0;
        for (int r = 0; r < n_entries; ++r) {
            for (int i = 0; i < counts[r]; ++i) {
                h[o_pos + st.q_start[r] + i] = start[r] + i;
                h[o_req + st.q_start[r] + i] = r;
            }
            for (int i = 0; i < n_want[r]; ++i) h[o_rows + row++] = st.q_start[r] + want[wi++];
        }
        for (int g = 0; g < G; ++g)
            if (mmh_cache_tables(cache_, g, n_entries, rids, st.table_width, h + o_tab + tab * g) != 0) throw ExecError(mmh_last_error());
        const int* dev = copy_step(st, sg, fixed);
        st.token_ids = dev + o_ids;
        st.positions = dev + o_pos;
        st.token_req = dev + o_req;
        st.logit_rows = dev + o_rows;
        for (int g = 0; g < G; ++g) st.tables[g] = dev + o_tab + tab * g;

        if (logits == nullptr && n_rows > 0) logits = st.step_mem->alloc_n<float>((size_t)n_rows * vocab_);      // the caller samples from them itself
        own_logits_ = logits;
        forward(st, logits);
        check_cuda(cudaMemcpyAsync(err_host_, err_, sizeof(int), cudaMemcpyDeviceToHost, stream), "reading the kernels' error flag");
        if (flags & RUN_COMMIT)
            for (int r = 0; r < n_entries; ++r)
                if (mmh_cache_commit(cache_, rids[r], start[r] + counts[r]) != 0) throw ExecError(mmh_last_error());
        ++steps_;
        return n_rows;
    }

    // ---- the same launches over the caller's device buffers ------------------------------------------------------------------------
    void forward_described(const StepDesc& d, float* logits, cudaStream_t stream) {
        Step st;
        init_step(st, stream);
        st.n_tokens = d.n_tokens;
        st.n_requests = d.n_requests;
        st.n_logit_rows = d.n_logit_rows;
        st.max_kv_len = d.max_kv_len;
        st.max_q_len = d.max_q_len;
        st.table_width = d.table_width;
        st.token_ids = d.token_ids;
        st.positions = d.positions;
        st.token_req = d.token_req;
        st.logit_rows = d.logit_rows;
        for (int g = 0; g < n_groups(); ++g) st.tables[g] = d.tables[g];
        st.q_start.assign(d.q_start, d.q_start + d.n_requests);
        st.q_len.assign(d.q_len, d.q_len + d.n_requests);
        st.kv_len.assign(d.kv_len, d.kv_len + d.n_requests);
        prepare(st);
        if (!st.uploads.empty()) {
            cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
            cudaStreamIsCapturing(stream, &cs);
            if (cs != cudaStreamCaptureStatusNone)
                throw ExecError("this step needs work lists copied from the host (it holds a prompt portion); it cannot be captured");
            Staging& sg = next_staging(upload_ints(st));
            copy_step(st, sg, 0);
        }
        forward(st, logits);
        ++steps_;
    }


    // ---- one scheduler step, sampled and committed ------------------------------------------------------------------------------------
    // Asks the scheduler (csrc/host/runtime.cpp) for the next step's plan, runs it, draws a token for every entry whose last
    // token was fed (greedy, or temperature / top-k / top-p with the request's own seed and draw counter, after soft-cap and
    // repetition / frequency / presence penalties over its recent tokens: src/compute/Sampling.cpp:119-264), waits for the tokens,
    // and commits them: cache lengths advance, finished requests give back what they hold.  Returns the number of sampled tokens
    // (out_rids / out_tokens); the plan it ran stays readable from the scheduler, what happened to requests from events().
    int run_plan(void* sched, long long* out_rids, int* out_tokens, int cap, cudaStream_t stream) {
        events_.clear();
        planned_ = 0;
        const int n = mmh_sched_schedule(sched);
        if (n < 0) throw ExecError(mmh_last_error());
        take_events(sched);
        if (n == 0) return 0;
        std::vector<long long> rids(n);
        std::vector<int> starts(n), counts(n), samples(n), n_want(n), want, sampled(n, 0);
        mmh_sched_plan(sched, rids.data(), starts.data(), counts.data(), samples.data(), n);
        planned_ = n;
        size_t total = 0;
        for (int i = 0; i < n; ++i) total += counts[i];
        std::vector<int> tokens(total);
        size_t at = 0;
        int rows = 0;
        for (int i = 0; i < n; ++i) {
            if (mmh_sched_tokens(sched, rids[i], starts[i], counts[i], tokens.data() + at) < 0) throw ExecError(mmh_last_error());
            at += counts[i];
            n_want[i] = samples[i] ? 1 : 0;
            if (samples[i]) {
                want.push_back(counts[i] - 1);
                ++rows;
            }
        }
        if (rows > cap) throw ExecError("executor: more sampled tokens than the caller has room for");
        run(n, rids.data(), counts.data(), tokens.data(), n_want.data(), want.data(), 0, nullptr, 0, stream);
        if (rows > 0) {
            std::vector<long long> row_rids;
            for (int i = 0; i < n; ++i)
                if (samples[i]) row_rids.push_back(rids[i]);
            int* dev_tokens = sample(sched, row_rids, own_logits_, stream);
            Staging& sg = next_staging(rows);
            check_cuda(cudaMemcpyAsync(sg.host, dev_tokens, rows * sizeof(int), cudaMemcpyDeviceToHost, stream), "reading the sampled tokens");
            check_cuda(cudaStreamSynchronize(stream), "waiting for the step");
            if (take_error_flag() != 0) {
                cudaMemsetAsync(err_, 0, sizeof(int), stream);
                throw ExecError("a kernel of the step gave up waiting on its pipeline; the step's output is not valid");
            }
            int r = 0;
            for (int i = 0; i < n; ++i)
                if (samples[i]) {
                    if (sg.host[r] < 0 || sg.host[r] >= vocab_) throw ExecError("the sampler returned a token outside the vocabulary");
                    sampled[i] = sg.host[r];
                    out_rids[r] = rids[i];
                    out_tokens[r] = sg.host[r];
                    ++r;
                }
        }
        if (mmh_sched_commit(sched, n, rids.data(), starts.data(), counts.data(), samples.data(), sampled.data()) != 0) throw ExecError(mmh_last_error());
        take_events(sched);
        return rows;
    }

    struct Event {
        long long rid;
        int kind, code;
    };
    const std::vector<Event>& events() const { return events_; }
    int planned() const { return planned_; }

  private:
    void take_events(void* sched) {
        std::vector<long long> r(256);
        std::vector<int> k(256), c(256);
        int n = mmh_sched_events(sched, r.data(), k.data(), c.data(), 256);
        if (n > 256) {                      // more than fit the first time: the list stays until the scheduler's next call
            r.resize(n);
            k.resize(n);
            c.resize(n);
            n = mmh_sched_events(sched, r.data(), k.data(), c.data(), n);
        }
        for (int i = 0; i < n; ++i) events_.push_back({r[i], k[i], c[i]});
    }

    // Draws one token per row of logits [rows, vocab] for the requests `rids`; returns device int32 [rows].
    int* sample(void* sched, const std::vector<long long>& rids, float* logits, cudaStream_t stream) {
        const int R = (int)rids.size(), V = vocab_;
        struct P {
            float f[6];      // temperature, top_p, repetition, frequency, presence, softcap
            int i[4];        // top_k, penalty window, generated, tokens
            long long seed;
        };
        std::vector<P> p(R);
        bool need_pen = false, need_cap = false, all_greedy = true;
        int w = 0;
        auto greedy = [](const P& x) { return x.f[0] <= 0.f || x.i[0] == 1; };
        auto pen = [](const P& x) { return x.i[1] > 0 && (x.f[2] != 1.f || x.f[3] != 0.f || x.f[4] != 0.f); };
        for (int r = 0; r < R; ++r) {
            if (mmh_sched_get_sampling(sched, rids[r], p[r].f, p[r].i, &p[r].seed) != 0) throw ExecError(mmh_last_error());
            if (pen(p[r]) && p[r].i[3] > 0) {
                need_pen = true;
                w = std::max(w, std::min(p[r].i[1], p[r].i[3]));
            }
            need_cap = need_cap || p[r].f[5] > 0.f;
            all_greedy = all_greedy && greedy(p[r]);
        }
        Arena& mem = step_mem_;
        int* out = mem.alloc_n<int>(R);
        void* s = stream;
        auto argmax = [&]() {
            if (V > 16384) {          // wide rows: several blocks per row, then one to reduce them
                const int parts = std::min(256, (V + 4095) / 4096);
                float* pv = mem.alloc_n<float>((size_t)R * parts);
                int* pi = mem.alloc_n<int>((size_t)R * parts);
                check_kernel(mm_argmax_rows_split(logits, out, pv, pi, R, V, parts, s), "argmax_rows_split");
            } else {
                check_kernel(mm_argmax_rows(logits, out, R, V, s), "argmax_rows");
            }
            return out;
        };
        // greedy without penalties: the soft-cap is monotonic and leaves the maximum where it is
        if (all_greedy && !need_pen) return argmax();
        // the rows' parameters in one pinned block, one copy: 64-bit values first, then floats and integers
        const int W = std::max(w, 1);
        const size_t o_seed = 0, o_cnt = o_seed + 2 * (size_t)R, o_f = o_cnt + 2 * (size_t)R, o_k = o_f + 6 * (size_t)R, o_recent = o_k + R,
                     total = o_recent + (size_t)R * W;
        Staging& sg = next_staging(total);
        long long* h_seed = reinterpret_cast<long long*>(sg.host + o_seed);
        long long* h_cnt = reinterpret_cast<long long*>(sg.host + o_cnt);
        float* h_f = reinterpret_cast<float*>(sg.host + o_f);      // rep | freq | pres | cap | temperature | top_p, R each
        int* h_k = sg.host + o_k;
        int* h_recent = sg.host + o_recent;
        std::vector<int> hist;
        for (int r = 0; r < R; ++r) {
            const bool on = pen(p[r]);
            h_seed[r] = p[r].seed & 0x7FFFFFFFFFFFFFFFLL;
            h_cnt[r] = p[r].i[2];
            h_f[0 * R + r] = on ? p[r].f[2] : 1.f;
            h_f[1 * R + r] = on ? p[r].f[3] : 0.f;
            h_f[2 * R + r] = on ? p[r].f[4] : 0.f;
            h_f[3 * R + r] = p[r].f[5];
            h_f[4 * R + r] = greedy(p[r]) ? 0.f : p[r].f[0];
            h_f[5 * R + r] = p[r].f[1];
            h_k[r] = p[r].i[0];
            for (int j = 0; j < W; ++j) h_recent[(size_t)r * W + j] = -1;
            const int k = on ? std::min(p[r].i[1], p[r].i[3]) : 0;
            if (k > 0) {
                hist.resize(k);
                if (mmh_sched_tokens(sched, rids[r], p[r].i[3] - k, k, hist.data()) < 0) throw ExecError(mmh_last_error());
                for (int j = 0; j < k; ++j) h_recent[(size_t)r * W + j] = hist[j];
            }
        }
        int* dev = mem.alloc_n<int>(total);
        check_cuda(cudaMemcpyAsync(dev, sg.host, total * sizeof(int), cudaMemcpyHostToDevice, stream), "copying the sampling parameters");
        check_cuda(cudaEventRecord(sg.copied, stream), "staging event");
        sg.in_flight = true;
        const float* d_f = reinterpret_cast<const float*>(dev + o_f);
        if (need_pen || need_cap) {
            check_kernel(mm_apply_penalties(logits, R, V, w > 0 ? dev + o_recent : nullptr, w > 0 ? W : 0, d_f, d_f + R, d_f + 2 * R,
                                            need_cap ? d_f + 3 * R : nullptr, s), "apply_penalties");
            if (all_greedy) return argmax();
        }
        check_kernel(mm_sample_rows(logits, out, R, V, d_f + 4 * R, dev + o_k, d_f + 5 * R, dev + o_seed, dev + o_cnt, s), "sample_rows");
        return out;
    }

  public:
    void* error_flag_device() const { return err_; }
    void* cache() const { return cache_; }
    int page_size() const { return page_size_; }
    int vocab() const { return vocab_; }
    std::vector<Event>& events_buffer() { return events_; }

    int take_error_flag() {
        const int v = *err_host_;
        *err_host_ = 0;
        return v;
    }
    long long steps() const { return steps_; }
    size_t memory() const { return step_mem_.capacity() + layer_mem_[0].capacity() + layer_mem_[1].capacity(); }

  private:
    Model* model_;
    void* cache_;
    int page_size_;
    std::vector<int> group_pages_;
    std::vector<EntryCache> entries_;
    int vocab_, max_seq_len_;
    void* err_;
    int* err_host_ = nullptr;
    Arena step_mem_;
    Arena layer_mem_[2];
    std::unique_ptr<Blas> blas_;
    cudaStream_t side_ = nullptr;
    cudaEvent_t forked_ = nullptr, joined_ = nullptr;
    Staging ring_[4];
    int ring_next_ = 0;
    long long steps_ = 0;
    float* own_logits_ = nullptr;
    std::vector<Event> events_;
    int planned_ = 0;
};


// ---- steady-state decoding of a fixed set of requests as one replayed CUDA graph ---------------------------------------------------
// When every running request is decoding, a step is the same launches with the same shapes each time: only token ids,
// positions and block-table entries change, and they live in device buffers that the graph reads.  The step (forward,
// penalties, sampling, position advance) is captured once and replayed; pages for a number of steps (the horizon) are
// reserved at binding, so no host work is needed between replays except committing lengths.  The reference has graph
// replay of its decode blocks as an opt-in (src/runtime/InferenceEngine.cpp:1826-1842, 1944-1998).
class DecodeSession {
  public:
    DecodeSession(Executor* ex, void* cache, int n_groups, int page_size, int vocab, int batch, int kv_bound, bool greedy, bool feed_back, int window)
        : ex_(ex), cache_(cache), G_(n_groups), ps_(page_size), V_(vocab), b_(batch), bound_(kv_bound), greedy_(greedy), feed_back_(feed_back), W_(window) {
        width_ = std::max(1, (bound_ + ps_ - 1) / ps_);
        parts_ = V_ > 16384 ? std::min(256, (V_ + 4095) / 4096) : 0;
        auto pad = [](size_t n) { return (n + 63) & ~(size_t)63; };
        // one block of device memory: 64-bit values first, then 32-bit ones
        size_t off = 0;
        auto take = [&](size_t bytes) { const size_t at = off; off += pad(bytes); return at; };
        const size_t o_seeds = take(8 * b_), o_counters = take(8 * b_), o_lengths = take(8 * b_), o_ids = take(4 * b_), o_pos = take(4 * b_),
                     o_req = take(4 * b_), o_out = take(4 * (b_ + 1)), o_topk = take(4 * b_), o_widths = take(4 * b_), o_temp = take(4 * b_),
                     o_topp = take(4 * b_), o_pen = take(16 * b_), o_recent = take(4 * (size_t)b_ * std::max(W_, 1)),
                     o_tables = take(4 * (size_t)G_ * b_ * width_), o_pv = take(4 * (size_t)b_ * std::max(parts_, 1)),
                     o_pi = take(4 * (size_t)b_ * std::max(parts_, 1)), o_logits = take(4 * (size_t)b_ * V_);
        check_cuda(cudaMalloc((void**)&mem_, off), "decode session memory");
        check_cuda(cudaMemset(mem_, 0, off - pad(4 * (size_t)b_ * V_)), "decode session memory");
        seeds_ = (long long*)(mem_ + o_seeds); counters_ = (long long*)(mem_ + o_counters); lengths_ = (long long*)(mem_ + o_lengths);
        ids_ = (int*)(mem_ + o_ids); pos_ = (int*)(mem_ + o_pos); req_ = (int*)(mem_ + o_req); out_ = (int*)(mem_ + o_out);
        topk_ = (int*)(mem_ + o_topk); widths_ = (int*)(mem_ + o_widths); temp_ = (float*)(mem_ + o_temp); topp_ = (float*)(mem_ + o_topp);
        pen_ = (float*)(mem_ + o_pen); recent_ = (int*)(mem_ + o_recent); tables_ = (int*)(mem_ + o_tables);
        part_val_ = (float*)(mem_ + o_pv); part_idx_ = (int*)(mem_ + o_pi); logits_ = (float*)(mem_ + o_logits);
        std::vector<int> ar(b_);
        for (int i = 0; i < b_; ++i) ar[i] = i;
        check_cuda(cudaMemcpy(req_, ar.data(), 4 * b_, cudaMemcpyHostToDevice), "decode session set-up");
        q_start_ = ar;
        q_len_.assign(b_, 1);
        kv_len_.assign(b_, bound_);
        // pinned: the step's results (tokens, then the kernels' error flag) twice, the tokens fed back, and what a binding uploads
        const size_t up = (size_t)G_ * b_ * width_ + (size_t)b_ * (std::max(W_, 1) + 24);
        check_cuda(cudaMallocHost((void**)&pin_, 4 * (3 * (size_t)(b_ + 1) + up)), "decode session pinned memory");
        pin_out_[0] = pin_;
        pin_out_[1] = pin_ + (b_ + 1);
        pin_in_ = pin_ + 2 * (b_ + 1);
        pin_up_ = pin_ + 3 * (b_ + 1);
        check_cuda(cudaStreamCreateWithFlags(&capture_stream_, cudaStreamNonBlocking), "decode session stream");
    }
    ~DecodeSession() {
        if (graph_) cudaGraphExecDestroy(graph_);
        if (capture_stream_) cudaStreamDestroy(capture_stream_);
        if (pin_) cudaFreeHost(pin_);
        if (mem_) cudaFree(mem_);
    }

    // Points the session at `rids` for `horizon` steps.  Returns 0; 1 when the pages for the horizon are not free (nothing
    // changed); 2 when a request would outgrow the bound the session was made for.
    int bind(const long long* rids, int horizon, const int* first_tokens, const float* temperature, const int* top_k, const float* top_p,
             const long long* seeds, const long long* counters, const int* recent, const int* widths, const long long* lengths, const float* pen,
             cudaStream_t s) {
        std::vector<int> len(b_), need(std::max(G_, 1), 0), one(std::max(G_, 1));
        for (int i = 0; i < b_; ++i) {
            len[i] = mmh_cache_request(cache_, rids[i], 0);
            if (len[i] < 0) throw ExecError(mmh_last_error());
            if (len[i] + horizon > bound_) return 2;
        }
        for (int i = 0; i < b_; ++i) {
            if (mmh_cache_pages_needed(cache_, rids[i], len[i] + horizon, one.data()) != 0) throw ExecError(mmh_last_error());
            for (int g = 0; g < G_; ++g) need[g] += one[g];
        }
        for (int g = 0; g < G_; ++g)
            if (need[g] > mmh_cache_info(cache_, 3, g)) return 1;
        for (int i = 0; i < b_; ++i)
            if (mmh_cache_reserve(cache_, rids[i], len[i] + horizon) != 1) throw ExecError("decode session: reserving checked pages failed");
        rids_.assign(rids, rids + b_);
        alive_.assign(b_, 1);
        horizon_ = horizon;
        done_ = 0;
        // one pinned block, copied piece by piece (a binding is rare)
        check_cuda(cudaStreamSynchronize(s), "decode session bind");       // the pinned block may still be read by an earlier copy
        int* h = pin_up_;
        auto up = [&](void* dst, const void* src, size_t bytes) {
            std::memcpy(h, src, bytes);
            check_cuda(cudaMemcpyAsync(dst, h, bytes, cudaMemcpyHostToDevice, s), "decode session bind");
            h += (bytes + 7) / 8 * 2;
        };
        for (int g = 0; g < G_; ++g) {
            if (mmh_cache_tables(cache_, g, b_, rids, width_, h) != 0) throw ExecError(mmh_last_error());
            check_cuda(cudaMemcpyAsync(tables_ + (size_t)g * b_ * width_, h, 4 * (size_t)b_ * width_, cudaMemcpyHostToDevice, s), "decode session bind");
            h += ((size_t)b_ * width_ + 1) / 2 * 2;
        }
        up(pos_, len.data(), 4 * b_);
        up(ids_, first_tokens, 4 * b_);
        if (!greedy_) {
            if (!temperature || !top_k || !top_p || !seeds || !counters) throw ExecError("decode session: a sampling session needs the sampling parameters");
            up(temp_, temperature, 4 * b_);
            up(topk_, top_k, 4 * b_);
            up(topp_, top_p, 4 * b_);
            up(seeds_, seeds, 8 * b_);
            up(counters_, counters, 8 * b_);
        }
        if (W_ > 0) {
            if (!recent || !widths || !lengths || !pen) throw ExecError("decode session: a session with penalties needs the recent tokens");
            check_cuda(cudaStreamSynchronize(s), "decode session bind");
            h = pin_up_;
            up(recent_, recent, 4 * (size_t)b_ * W_);
            up(widths_, widths, 4 * b_);
            up(lengths_, lengths, 8 * b_);
            up(pen_, pen, 16 * b_);
        }
        check_cuda(cudaStreamSynchronize(s), "decode session bind");
        return 0;
    }

    // one decode step for every bound request: launched eagerly the first time (and then captured), replayed afterwards
    void step(cudaStream_t s) {
        if (done_ >= horizon_) throw ExecError("decode session is past its horizon");
        if (!graph_) {
            launch(s);                               // a valid step of its own, and the warm-up of every kernel and workspace
            check_cuda(cudaStreamSynchronize(s), "decode session warm-up");
            check_cuda(cudaStreamBeginCapture(capture_stream_, cudaStreamCaptureModeThreadLocal), "decode session capture");
            cudaGraph_t graph = nullptr;
            try {
                launch(capture_stream_);             // records the launches; nothing runs, the buffers keep their contents
            } catch (...) {
                cudaStreamEndCapture(capture_stream_, &graph);
                if (graph) cudaGraphDestroy(graph);
                throw;
            }
            check_cuda(cudaStreamEndCapture(capture_stream_, &graph), "decode session capture");
            const cudaError_t e = cudaGraphInstantiate(&graph_, graph, 0);
            cudaGraphDestroy(graph);
            check_cuda(e, "decode session graph");
        } else {
            check_cuda(cudaGraphLaunch(graph_, s), "decode session replay");
        }
        for (long long rid : rids_)
            if (mmh_cache_has(cache_, rid)) {        // a request may have been retired while this step was already in flight
                const int n = mmh_cache_request(cache_, rid, 0);
                if (mmh_cache_commit(cache_, rid, n + 1) != 0) throw ExecError(mmh_last_error());
            }
        ++done_;
    }

    // starts the copy of the step's results (tokens and error flag) into pinned buffer `which`
    void read_out(int which, cudaStream_t s) {
        check_cuda(cudaMemcpyAsync(pin_out_[which], out_, 4 * (b_ + 1), cudaMemcpyDeviceToHost, s), "reading the sampled tokens");
    }

    // The loop of a decode run, one call per step: waits for the step in flight, launches the next one with that step's
    // tokens copied back from pinned memory as its inputs, and accounts for the finished step in the scheduler (tokens
    // appended, finished requests retired).  out_tokens[b], out_done[b] (1: finished with this token, -1: not accounted,
    // the request had left earlier).  Returns 1 if a request finished in this step, else 0.
    int cycle(void* sched, bool launch_next, int* out_tokens, int* out_done, std::vector<Executor::Event>* events, cudaStream_t s) {
        check_cuda(cudaStreamSynchronize(s), "waiting for the decode step");
        const int* got = pin_out_[cur_];
        if (got[b_] != 0) {
            cudaMemsetAsync(ex_->error_flag_device(), 0, sizeof(int), s);
            throw ExecError("a kernel of the decode step gave up waiting on its pipeline; the step's output is not valid");
        }
        for (int i = 0; i < b_; ++i)
            if (got[i] < 0 || got[i] >= V_) throw ExecError("the sampler returned a token outside the vocabulary");
        std::memcpy(out_tokens, got, 4 * b_);
        if (launch_next && done_ < horizon_) {
            if (!feed_back_) {
                std::memcpy(pin_in_, got, 4 * b_);
                check_cuda(cudaMemcpyAsync(ids_, pin_in_, 4 * b_, cudaMemcpyHostToDevice, s), "feeding the tokens back");      // next step's inputs, from pinned memory
            }
            step(s);
            read_out(cur_ ^ 1, s);
        }
        cur_ ^= 1;
        int stop = 0;
        for (int i = 0; i < b_; ++i) {
            out_done[i] = -1;
            if (!alive_[i]) continue;
            out_done[i] = 0;
            if (sched != nullptr) {
                const int rc = mmh_sched_accept_token(sched, rids_[i], out_tokens[i]);
                if (rc < 0) throw ExecError(mmh_last_error());
                long long r[8];
                int k[8], c[8];
                const int n = mmh_sched_events(sched, r, k, c, 8);
                for (int j = 0; j < n && j < 8; ++j) events->push_back({r[j], k[j], c[j]});
                if (rc == 1) {
                    out_done[i] = 1;
                    alive_[i] = 0;
                    stop = 1;
                }
            }
        }
        return stop;
    }

    void begin(cudaStream_t s) {
        cur_ = 0;
        step(s);
        read_out(0, s);
    }
    void drop(int i) {
        if (i >= 0 && i < b_) alive_[i] = 0;
    }
    int remaining() const { return horizon_ - done_; }
    int steps_done() const { return done_; }
    bool captured() const { return graph_ != nullptr; }
    int* device_tokens() { return out_; }
    int* device_inputs() { return ids_; }

  private:
    void launch(cudaStream_t s) {
        StepDesc d{};
        d.n_tokens = d.n_requests = d.n_logit_rows = b_;
        d.max_kv_len = bound_;
        d.max_q_len = 1;
        d.table_width = width_;
        d.token_ids = ids_;
        d.positions = pos_;
        d.token_req = req_;
        d.logit_rows = req_;
        for (int g = 0; g < G_; ++g) d.tables[g] = tables_ + (size_t)g * b_ * width_;
        d.q_start = q_start_.data();
        d.q_len = q_len_.data();
        d.kv_len = kv_len_.data();
        ex_->forward_described(d, logits_, s);
        if (W_ > 0) check_kernel(mm_apply_penalties(logits_, b_, V_, recent_, W_, pen_, pen_ + b_, pen_ + 2 * b_, pen_ + 3 * b_, s), "apply_penalties");
        if (greedy_) {
            if (parts_ > 0) check_kernel(mm_argmax_rows_split(logits_, out_, part_val_, part_idx_, b_, V_, parts_, s), "argmax_rows_split");
            else check_kernel(mm_argmax_rows(logits_, out_, b_, V_, s), "argmax_rows");
        } else {
            check_kernel(mm_sample_rows(logits_, out_, b_, V_, temp_, topk_, topp_, seeds_, counters_, s), "sample_rows");
        }
        if (W_ > 0) check_kernel(mm_window_push(recent_, b_, W_, widths_, lengths_, out_, s), "window_push");
        check_kernel(mm_advance_step(pos_, greedy_ ? nullptr : counters_, feed_back_ ? ids_ : nullptr, out_, b_, s), "advance_step");
        check_cuda(cudaMemcpyAsync(out_ + b_, ex_->error_flag_device(), sizeof(int), cudaMemcpyDeviceToDevice, s), "copying the error flag");
    }

    Executor* ex_;
    void* cache_;
    int G_, ps_, V_, b_, bound_;
    bool greedy_, feed_back_;
    int W_, width_ = 1, parts_ = 0, horizon_ = 0, done_ = 0, cur_ = 0;
    char* mem_ = nullptr;
    long long *seeds_ = nullptr, *counters_ = nullptr, *lengths_ = nullptr;
    int *ids_ = nullptr, *pos_ = nullptr, *req_ = nullptr, *out_ = nullptr, *topk_ = nullptr, *widths_ = nullptr, *recent_ = nullptr, *tables_ = nullptr,
        *part_idx_ = nullptr;
    float *temp_ = nullptr, *topp_ = nullptr, *pen_ = nullptr, *part_val_ = nullptr, *logits_ = nullptr;
    int* pin_ = nullptr;
    int* pin_out_[2] = {nullptr, nullptr};
    int* pin_in_ = nullptr;
    int* pin_up_ = nullptr;
    std::vector<int> q_start_, q_len_, kv_len_;
    std::vector<long long> rids_;
    std::vector<char> alive_;
    cudaStream_t capture_stream_ = nullptr;
    cudaGraphExec_t graph_ = nullptr;
};

}  // namespace mmx

// ---- C interface -----------------------------------------------------------------------------------------------------------------
using namespace mmx;

static thread_local std::string g_mmx_error;
static int set_error(int code, const std::exception& e) {
    g_mmx_error = e.what();
    return code;
}
#define MMX_GUARD(body)                                 \
    try {                                               \
        body                                            \
    } catch (const StepRefused& e) {                    \
        return set_error(-10, e);                       \
    } catch (const std::exception& e) {                 \
        return set_error(-1, e);                        \
    }

MMX_EXPORT const char* mmx_last_error() { return g_mmx_error.c_str(); }

// descriptions: built by the loader, consumed by mmx_model_create
MMX_EXPORT void* mmx_desc_new(const char* kind) {
    auto* d = new PartDesc();
    d->kind = kind;
    return d;
}
MMX_EXPORT void mmx_desc_free(void* d) { delete static_cast<PartDesc*>(d); }
MMX_EXPORT void mmx_desc_num(void* d, const char* key, double v) { static_cast<PartDesc*>(d)->num[key] = v; }
MMX_EXPORT int mmx_desc_tensor(void* d, const char* key, void* ptr, int dtype, int ndim, const long long* shape) {
    if (ndim < 0 || ndim > 4 || (dtype != F32 && dtype != BF16)) return -1;
    Tensor t;
    t.ptr = ptr;
    t.dtype = dtype;
    t.ndim = ndim;
    for (int i = 0; i < ndim; ++i) t.shape[i] = shape[i];
    static_cast<PartDesc*>(d)->tensors[key] = t;
    return 0;
}
// the child belongs to the parent from here on
MMX_EXPORT void mmx_desc_child(void* d, const char* key, void* child) {
    static_cast<PartDesc*>(d)->children[key] = std::unique_ptr<PartDesc>(static_cast<PartDesc*>(child));
}

// A model from descriptions (which stay the caller's).  Null, with a message, when a part has no native class.
MMX_EXPORT void* mmx_model_create(void* embedding, void* final_norm, void* head, int n_layers, void** blocks, int n_schedule, const int* sched_layer,
                                  const int* sched_cache_from, int act_dtype, int simt) {
    try {
        std::unique_ptr<Model> m(new Model());
        m->act_dtype = act_dtype;
        m->simt = simt != 0;
        m->embedding = build_as<Embedding>("embedding", *static_cast<PartDesc*>(embedding));
        m->final_norm = build_as<Norm>("norm", *static_cast<PartDesc*>(final_norm));
        m->head = build_as<Head>("head", *static_cast<PartDesc*>(head));
        for (int i = 0; i < n_layers; ++i) m->layers.push_back(build_as<Block>("block", *static_cast<PartDesc*>(blocks[i])));
        for (int i = 0; i < n_schedule; ++i) {
            if (sched_layer[i] < 0 || sched_layer[i] >= n_layers) throw ExecError("schedule entry names a layer the model does not have");
            m->schedule.push_back({sched_layer[i], sched_cache_from[i]});
        }
        return m.release();
    } catch (const std::exception& e) {
        g_mmx_error = e.what();
        return nullptr;
    }
}
MMX_EXPORT void mmx_model_destroy(void* m) { delete static_cast<Model*>(m); }

// entry_group[i] < 0: schedule entry i keeps no keys and values; k_pages/v_pages: the pools of the entry whose cache it uses
MMX_EXPORT void* mmx_exec_create(void* model, void* cache, int n_groups, int page_size, const int* group_pages, int n_entries, void** k_pages,
                                 void** v_pages, const int* entry_group, const int* entry_writes, int vocab, int max_seq_len, void* err_flag) {
    try {
        std::vector<EntryCache> entries;
        for (int i = 0; i < n_entries; ++i) entries.push_back({k_pages[i], v_pages[i], entry_group[i], entry_writes[i] != 0});
        return new Executor(static_cast<Model*>(model), cache, page_size, std::vector<int>(group_pages, group_pages + n_groups), std::move(entries), vocab,
                            max_seq_len, err_flag);
    } catch (const std::exception& e) {
        g_mmx_error = e.what();
        return nullptr;
    }
}
MMX_EXPORT void mmx_exec_destroy(void* ex) { delete static_cast<Executor*>(ex); }

// One step.  rids, counts, n_want: per entry; tokens and want: the entries' tokens and wanted places, one after the other.
// flags: 1 reserve the pages first (all or nothing), 2 commit the lengths after the launches.  Returns the number of
// logits rows (fp32 [rows, vocab] at `logits`), -10 when the step is refused (nothing ran, nothing changed), -1 on
// any other error; the text is mmx_last_error().
MMX_EXPORT int mmx_exec_run(void* ex, int n_entries, const long long* rids, const int* counts, const int* tokens, const int* n_want, const int* want,
                            int flags, void* logits, long long logits_rows_cap, void* stream) {
    MMX_GUARD(return static_cast<Executor*>(ex)->run(n_entries, rids, counts, tokens, n_want, want, flags, (float*)logits, logits_rows_cap,
                                                     (cudaStream_t)stream);)
}

MMX_EXPORT int mmx_exec_forward(void* ex, const StepDesc* d, void* logits, void* stream) {
    MMX_GUARD(static_cast<Executor*>(ex)->forward_described(*d, (float*)logits, (cudaStream_t)stream); return 0;)
}

// One step of the scheduler `sched` (a handle of csrc/host/runtime.cpp made over the same cache manager): plan, launches,
// sampling, the wait for the tokens, commit.  Returns the number of sampled tokens written to out_rids / out_tokens (at most
// cap), -1 on an error (the plan it was running stays readable from the scheduler, so that the caller can fail its requests).
MMX_EXPORT int mmx_exec_run_plan(void* ex, void* sched, long long* out_rids, int* out_tokens, int cap, void* stream) {
    MMX_GUARD(return static_cast<Executor*>(ex)->run_plan(sched, out_rids, out_tokens, cap, (cudaStream_t)stream);)
}
// entries of the plan of the last mmx_exec_run_plan (0: the scheduler had nothing to run)
MMX_EXPORT int mmx_exec_planned(void* ex) { return static_cast<Executor*>(ex)->planned(); }
// what the last mmx_exec_run_plan did to requests (admitted, preempted, finished: the scheduler's event kinds and codes)
MMX_EXPORT int mmx_exec_events(void* ex, long long* rids, int* kinds, int* codes, int cap) {
    const auto& ev = static_cast<Executor*>(ex)->events();
    const int n = (int)ev.size();
    for (int i = 0; i < n && i < cap; ++i) {
        rids[i] = ev[i].rid;
        kinds[i] = ev[i].kind;
        codes[i] = ev[i].code;
    }
    return n;
}

// ---- decode sessions: see DecodeSession above.  Codes: 0 ok, -1 error (mmx_last_error), bind: 1 no pages, 2 beyond the bound ----
MMX_EXPORT void* mmx_decode_create(void* ex, int batch, int kv_bound, int greedy, int feed_back, int penalty_window) {
    try {
        Executor* e = static_cast<Executor*>(ex);
        return new DecodeSession(e, e->cache(), e->n_groups(), e->page_size(), e->vocab(), batch, kv_bound, greedy != 0, feed_back != 0, penalty_window);
    } catch (const std::exception& e) {
        g_mmx_error = e.what();
        return nullptr;
    }
}
MMX_EXPORT void mmx_decode_destroy(void* sess) { delete static_cast<DecodeSession*>(sess); }
MMX_EXPORT int mmx_decode_bind(void* sess, const long long* rids, int horizon, const int* first_tokens, const float* temperature, const int* top_k,
                               const float* top_p, const long long* seeds, const long long* counters, const int* recent, const int* widths,
                               const long long* lengths, const float* pen, void* stream) {
    MMX_GUARD(return static_cast<DecodeSession*>(sess)->bind(rids, horizon, first_tokens, temperature, top_k, top_p, seeds, counters, recent, widths,
                                                             lengths, pen, (cudaStream_t)stream);)
}
// one step (launch or replay, lengths committed); the tokens stay on the device
MMX_EXPORT int mmx_decode_step(void* sess, void* stream) {
    MMX_GUARD(static_cast<DecodeSession*>(sess)->step((cudaStream_t)stream); return 0;)
}
// the first step of a run whose results come back through mmx_decode_cycle
MMX_EXPORT int mmx_decode_begin(void* sess, void* stream) {
    MMX_GUARD(static_cast<DecodeSession*>(sess)->begin((cudaStream_t)stream); return 0;)
}
// One turn of the decode loop: waits for the step in flight, launches the next (launch_next != 0 and steps are left), accounts
// for the finished one in `sched` (may be null).  Returns 1 if a request finished with this step, 0 if none, -1 on an error.
// What happened to requests is read with mmx_exec_events of the executor the session belongs to.
MMX_EXPORT int mmx_decode_cycle(void* ex, void* sess, void* sched, int launch_next, int* out_tokens, int* out_done, void* stream) {
    MMX_GUARD(auto& ev = static_cast<Executor*>(ex)->events_buffer(); ev.clear();
              return static_cast<DecodeSession*>(sess)->cycle(sched, launch_next != 0, out_tokens, out_done, &ev, (cudaStream_t)stream);)
}
MMX_EXPORT void mmx_decode_drop(void* sess, int index) { static_cast<DecodeSession*>(sess)->drop(index); }
// what: 0 steps left of the horizon, 1 steps done since the binding, 2 whether the step has been captured
MMX_EXPORT int mmx_decode_info(void* sess, int what) {
    DecodeSession* d = static_cast<DecodeSession*>(sess);
    return what == 0 ? d->remaining() : (what == 1 ? d->steps_done() : (d->captured() ? 1 : 0));
}
// device int32 arrays of the session: 0 the step's tokens [batch] (then the error flag), 1 the next step's input ids [batch]
MMX_EXPORT void* mmx_decode_buffer(void* sess, int what) {
    DecodeSession* d = static_cast<DecodeSession*>(sess);
    return what == 0 ? (void*)d->device_tokens() : (void*)d->device_inputs();
}

// The kernels' error flag as the last mmx_exec_run copied it back (valid once the stream has been synchronised); reading clears it.
MMX_EXPORT int mmx_exec_take_error_flag(void* ex) { return static_cast<Executor*>(ex)->take_error_flag(); }
MMX_EXPORT long long mmx_exec_stat(void* ex, int what) {
    Executor* e = static_cast<Executor*>(ex);
    return what == 0 ? e->steps() : (long long)e->memory();
}

// Tunables of the dispatch by name; returns the old value, or -1 for an unknown name.  value < 0 only reads.
MMX_EXPORT int mmx_option(const char* name, int value) {
    Options& o = options();
    struct {
        const char* n;
        int* p;
    } table[] = {{"prefill_min", &o.prefill_min}, {"use_tcgen05_prefill", &o.use_tcgen05_prefill}, {"use_tma_decode", &o.use_tma_decode},
                 {"tma_decode_stages", &o.tma_decode_stages}, {"target_ctas", &o.target_ctas}, {"use_cluster_merge", &o.use_cluster_merge},
                 {"cluster_max_wanted", &o.cluster_max_wanted}, {"fixed_split", &o.fixed_split}, {"gemv_max_rows", &o.gemv_max_rows},
                 {"skinny_max_rows", &o.skinny_max_rows}, {"tcgen05_swiglu_min_rows", &o.tcgen05_swiglu_min_rows},
                 {"tcgen05_pair_min_rows", &o.tcgen05_pair_min_rows}, {"use_side_stream", &o.use_side_stream}};
    for (auto& t : table)
        if (std::strcmp(t.n, name) == 0) {
            const int old = *t.p;
            if (value >= 0) *t.p = value;
            return old;
        }
    return -1;
}
