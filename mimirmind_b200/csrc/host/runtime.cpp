// Host runtime of the engine: page allocator, cache manager (block tables per request and cache group, state
// slots) and the continuous-batching scheduler.  Pure C++17, no CUDA: the library is built with the host compiler
// and driven from Python through the C interface at the end of this file.
//
// What it does and where the reference does the same:
//  * pages come from a LIFO free list, ids first handed out in ascending order, exhaustion is a sentinel
//    (src/runtime/serving/PagedKvBlockAllocator.cpp:11-60); freeing a page twice or one never given is an error;
//  * a request has one block table per cache group, indexed by absolute position / page size; reserve is all or
//    nothing across groups (src/runtime/serving/PagedKvSequence.cpp:41-74); tokens count after commit
//    (src/runtime/KvCache.hpp:90-103); a windowed group gives back pages no later query can reach; release gives
//    everything back (PagedKvSequence.cpp:76-87); every request owns a state slot (src/runtime/SsmState.hpp:39-86);
//  * per step decodes first, then prompt portions under the token budget, in admission order
//    (src/runtime/serving/ChunkedPrefillScheduler.cpp:20-51); first-in first-out admission up to max_active
//    (src/runtime/serving/RequestScheduler.cpp:84-103); out of pages: the most recently admitted running request
//    is preempted, last in first out (RequestScheduler.cpp:164-188), keeps its generated tokens and is recomputed;
//    a lone request that does not fit fails (src/runtime/serving/PreemptionPolicy.hpp:32-41).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

thread_local std::string g_error;
int fail(const std::string& msg) {
    g_error = msg;
    return -2;
}
}  // namespace

// the library's other source files report their errors through the same message
void mmh_set_error(const std::string& msg) { g_error = msg; }

namespace {

constexpr int32_t INVALID_PAGE = -1;

class PageAllocator {
  public:
    explicit PageAllocator(int n) : n_(n), out_(n, 0), ever_(n, 0) {
        free_.reserve(n);
        for (int p = n - 1; p >= 0; --p) free_.push_back(p);   // pop_back gives 0, 1, 2, ...
    }
    int num_pages() const { return n_; }
    int num_free() const { return (int)free_.size(); }
    int num_used() const { return n_ - (int)free_.size(); }
    long long total_allocs() const { return allocs_; }
    long long reuses() const { return reuses_; }
    int alloc() {
        if (free_.empty()) return INVALID_PAGE;
        const int p = free_.back();
        free_.pop_back();
        out_[p] = 1;
        ++allocs_;
        if (ever_[p]) ++reuses_;
        ever_[p] = 1;
        return p;
    }
    int free(int p) {
        if (p < 0 || p >= n_) return fail("page " + std::to_string(p) + " is outside the pool of " + std::to_string(n_));
        if (!out_[p]) return fail("page " + std::to_string(p) + " freed twice or never allocated");
        out_[p] = 0;
        free_.push_back(p);
        return 0;
    }
    bool is_allocated(int p) const { return p >= 0 && p < n_ && out_[p]; }
    int check() const {
        std::vector<int> seen(n_, 0);
        for (int p : free_) ++seen[p];
        for (int p = 0; p < n_; ++p) {
            if (seen[p] > 1) return fail("page " + std::to_string(p) + " is on the free list " + std::to_string(seen[p]) + " times");
            if (seen[p] == 1 && out_[p]) return fail("page " + std::to_string(p) + " is both free and allocated");
            if (seen[p] == 0 && !out_[p]) return fail("page " + std::to_string(p) + " is lost: neither free nor allocated");
        }
        return 0;
    }

  private:
    int n_;
    std::vector<int> free_;
    std::vector<char> out_, ever_;
    long long allocs_ = 0, reuses_ = 0;
};

struct CacheRequest {
    int length = 0, reserved = 0, slot = -1;
    bool started = false;
    std::vector<std::vector<int32_t>> tables;     // per group
};

class CacheManager {
  public:
    CacheManager(int n_groups, const int* pages, const int* windows, int page_size, int max_requests)
        : page_size_(page_size), slots_(max_requests) {
        for (int g = 0; g < n_groups; ++g) {
            allocs_.emplace_back(pages[g]);
            windows_.push_back(windows[g]);
        }
    }
    int n_groups() const { return (int)allocs_.size(); }
    int page_size() const { return page_size_; }
    PageAllocator& allocator(int g) { return allocs_[g]; }
    int window(int g) const { return windows_[g]; }
    bool has(int64_t rid) const { return reqs_.count(rid) != 0; }
    CacheRequest* find(int64_t rid) {
        auto it = reqs_.find(rid);
        if (it == reqs_.end()) {
            fail("unknown request");
            return nullptr;
        }
        return &it->second;
    }
    int add(int64_t rid) {
        if (has(rid)) return fail("request already exists");
        const int slot = slots_.alloc();
        if (slot == INVALID_PAGE) return -1;
        CacheRequest r;
        r.slot = slot;
        r.tables.resize(allocs_.size());
        reqs_.emplace(rid, std::move(r));
        return slot;
    }
    int blocks_for(int length) const { return (length + page_size_ - 1) / page_size_; }
    int pages_needed(int64_t rid, int new_len, int* out) {
        CacheRequest* r = find(rid);
        if (!r) return -2;
        const int first = r->length / page_size_, last = blocks_for(new_len);
        for (size_t g = 0; g < allocs_.size(); ++g) {
            const auto& t = r->tables[g];
            int n = 0;
            for (int b = first; b < last; ++b)
                if (b >= (int)t.size() || t[b] == INVALID_PAGE) ++n;
            out[g] = n;
        }
        return 0;
    }
    int reserve(int64_t rid, int new_len) {
        CacheRequest* r = find(rid);
        if (!r) return -2;
        if (new_len < r->length) return fail("cannot reserve " + std::to_string(new_len) + " below the length " + std::to_string(r->length));
        std::vector<int> need(allocs_.size());
        pages_needed(rid, new_len, need.data());
        for (size_t g = 0; g < allocs_.size(); ++g)
            if (allocs_[g].num_free() < need[g]) return 0;
        const int first = r->length / page_size_, last = blocks_for(new_len);
        for (size_t g = 0; g < allocs_.size(); ++g) {
            auto& t = r->tables[g];
            if ((int)t.size() < last) t.resize(last, INVALID_PAGE);
            for (int b = first; b < last; ++b)
                if (t[b] == INVALID_PAGE) t[b] = allocs_[g].alloc();
        }
        r->reserved = std::max(r->reserved, new_len);
        return 1;
    }
    int commit(int64_t rid, int new_len) {
        CacheRequest* r = find(rid);
        if (!r) return -2;
        if (new_len < r->length || new_len > r->reserved)
            return fail("commit to " + std::to_string(new_len) + " outside [" + std::to_string(r->length) + ", " + std::to_string(r->reserved) + "]");
        r->length = new_len;
        // the next query sits at position new_len and sees keys >= new_len + 1 - W
        for (size_t g = 0; g < allocs_.size(); ++g) {
            if (windows_[g] <= 0) continue;
            const int dead_before = new_len + 1 - windows_[g];
            if (dead_before <= 0) continue;
            auto& t = r->tables[g];
            const int upto = std::min(dead_before / page_size_, (int)t.size());
            for (int b = 0; b < upto; ++b)
                if (t[b] != INVALID_PAGE) {
                    if (allocs_[g].free(t[b]) != 0) return -2;
                    t[b] = INVALID_PAGE;
                }
        }
        return 0;
    }
    int release(int64_t rid) {
        auto it = reqs_.find(rid);
        if (it == reqs_.end()) return fail("unknown request");
        for (size_t g = 0; g < allocs_.size(); ++g)
            for (int32_t p : it->second.tables[g])
                if (p != INVALID_PAGE && allocs_[g].free(p) != 0) return -2;
        if (slots_.free(it->second.slot) != 0) return -2;
        reqs_.erase(it);
        return 0;
    }
    int total_pages(int g) const { return allocs_[g].num_pages(); }
    int check() {
        for (size_t g = 0; g < allocs_.size(); ++g) {
            if (allocs_[g].check() != 0) return -2;
            std::vector<char> seen(allocs_[g].num_pages(), 0);
            int count = 0;
            for (auto& kv : reqs_)
                for (int32_t p : kv.second.tables[g]) {
                    if (p == INVALID_PAGE) continue;
                    if (p < 0 || p >= allocs_[g].num_pages() || !allocs_[g].is_allocated(p))
                        return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " of a request is not allocated");
                    if (seen[p]) return fail("group " + std::to_string(g) + ": page " + std::to_string(p) + " is in two block tables");
                    seen[p] = 1;
                    ++count;
                }
            if (count != allocs_[g].num_used())
                return fail("group " + std::to_string(g) + ": " + std::to_string(allocs_[g].num_used()) + " pages are out but tables hold " + std::to_string(count));
        }
        if (slots_.check() != 0) return -2;
        std::vector<char> seen(slots_.num_pages(), 0);
        for (auto& kv : reqs_) {
            const int s = kv.second.slot;
            if (s < 0 || s >= slots_.num_pages() || seen[s]) return fail("state slots are inconsistent");
            seen[s] = 1;
        }
        if ((int)reqs_.size() != slots_.num_used()) return fail("state slots are inconsistent");
        return 0;
    }
    const std::unordered_map<int64_t, CacheRequest>& requests() const { return reqs_; }
    PageAllocator& slots() { return slots_; }

  private:
    int page_size_;
    std::vector<PageAllocator> allocs_;
    std::vector<int> windows_;
    PageAllocator slots_;
    std::unordered_map<int64_t, CacheRequest> reqs_;
};

// ---- scheduler ---------------------------------------------------------------------------------------------
enum State { WAITING = 0, RUNNING = 1, FINISHED = 2 };
enum Finish { NONE = 0, STOP = 1, LENGTH = 2, CONTEXT = 3, OUT_OF_PAGES = 4, REJECTED = 5, CANCELLED = 6 };
enum Event { EV_ADMITTED = 1, EV_PREEMPTED = 2, EV_FINISHED = 3 };

struct SchedRequest {
    int64_t id = 0;
    std::vector<int32_t> tokens;        // prompt, then what was generated
    int prompt_len = 0, max_new = 0, generated = 0;
    std::vector<int32_t> stop_ids;
    int state = WAITING, finish = NONE, preemptions = 0;
    long long admit_seq = -1;
    std::string reject_reason;
    // how its tokens are drawn (names and meanings of the reference's sampler, src/compute/Sampling.hpp:40-87); kept here so
    // that a step which samples inside the library needs nothing from the caller
    float temperature = 0.f, top_p = 1.f, repetition = 1.f, frequency = 0.f, presence = 0.f, softcap = 0.f;
    int top_k = 0, penalty_window = 0;
    long long seed = 0;
};

struct PlanEntry {
    int64_t rid;
    int start, count, samples;
};

struct SchedEvent {
    int64_t rid;
    int kind, code;
};

class Scheduler {
  public:
    Scheduler(CacheManager* mgr, int token_budget, int max_active, int prefill_chunk, int max_seq_len)
        : mgr_(mgr), budget_(token_budget), max_active_(max_active), chunk_(prefill_chunk), max_seq_(max_seq_len) {}

    SchedRequest* find(int64_t rid) {
        auto it = reqs_.find(rid);
        if (it == reqs_.end()) {
            fail("unknown request");
            return nullptr;
        }
        return &it->second;
    }
    int add(int64_t rid, const int32_t* prompt, int n, int max_new, const int32_t* stop, int n_stop) {
        if (reqs_.count(rid)) return fail("request id already used");
        SchedRequest r;
        r.id = rid;
        r.tokens.assign(prompt, prompt + n);
        r.prompt_len = n;
        r.max_new = max_new;
        r.stop_ids.assign(stop, stop + n_stop);
        std::string reason;
        if (n == 0) reason = "empty prompt";
        else if (max_new < 1) reason = "max_new must be at least 1";
        else if (n >= max_seq_) reason = "prompt of " + std::to_string(n) + " tokens does not fit the context of " + std::to_string(max_seq_);
        else {
            const int need = (n + mgr_->page_size() - 1) / mgr_->page_size();
            for (int g = 0; g < mgr_->n_groups(); ++g)
                if (mgr_->window(g) <= 0 && need > mgr_->total_pages(g))
                    reason = "prompt needs " + std::to_string(need) + " pages, the pool has " + std::to_string(mgr_->total_pages(g));
        }
        if (!reason.empty()) {
            r.state = FINISHED;
            r.finish = REJECTED;
            r.reject_reason = reason;
            reqs_.emplace(rid, std::move(r));
            finished_.push_back(rid);
            ++m_rejected_;
            return 0;
        }
        reqs_.emplace(rid, std::move(r));
        waiting_.push_back(rid);
        return 1;
    }
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    int remaining(const SchedRequest& r) {
        CacheRequest* c = mgr_->find(r.id);
        return (int)r.tokens.size() - (c ? c->length : 0);
    }
    int portion(int remaining_tokens, int budget) const {
        int n = std::min(remaining_tokens, budget);
        if (chunk_ > 0 && n > 1) n = std::min(n, chunk_);
        return n;
    }
    void finish(SchedRequest& r, int why) {
        r.state = FINISHED;
        r.finish = why;
        finished_.push_back(r.id);
        events_.push_back({r.id, EV_FINISHED, why});
    }
    int schedule() {
        plan_.clear();
        events_.clear();
        bool preempted_now = false;
        while (true) {
            int budget = budget_;
            plan_.clear();
            bool failed = false;
            // decodes first, then prompt portions, both in admission order
            std::vector<int64_t> order;
            for (int64_t rid : running_)
                if (remaining(reqs_[rid]) == 1) order.push_back(rid);
            for (int64_t rid : running_)
                if (remaining(reqs_[rid]) > 1) order.push_back(rid);
            for (int64_t rid : order) {
                if (budget <= 0) break;
                SchedRequest& r = reqs_[rid];
                const int start = mgr_->find(rid)->length;
                const int n = portion((int)r.tokens.size() - start, budget);
                const int rc = mgr_->reserve(rid, start + n);
                if (rc < 0) return -2;
                if (rc == 0) {
                    failed = true;
                    break;
                }
                plan_.push_back({rid, start, n, start + n == (int)r.tokens.size() ? 1 : 0});
                budget -= n;
            }
            if (failed) {
                // pages ran out: reserved pages stay with their requests; the most recently admitted goes
                const int64_t vid = running_.back();
                SchedRequest& victim = reqs_[vid];
                if (mgr_->release(vid) != 0) return -2;
                running_.pop_back();
                if (running_.empty()) {
                    // it was alone and still did not fit: it fails, and nothing is left that its pages must serve
                    // first, so waiting requests may be admitted in this same call (else the plan would be empty
                    // with work left)
                    finish(victim, OUT_OF_PAGES);
                    ++m_finished_;
                    preempted_now = false;
                } else {
                    victim.state = WAITING;
                    ++victim.preemptions;
                    waiting_.push_front(vid);
                    ++m_preempted_;
                    events_.push_back({vid, EV_PREEMPTED, victim.preemptions});
                    preempted_now = true;
                }
                continue;
            }
            // admit waiting requests, first in first out (not in a step that had to preempt: the freed pages
            // first serve the requests that were short of them)
            while (!preempted_now && !waiting_.empty() && (int)running_.size() < max_active_ && budget > 0) {
                const int64_t rid = waiting_.front();
                SchedRequest& r = reqs_[rid];
                if (!mgr_->has(rid)) {
                    const int slot = mgr_->add(rid);
                    if (slot == -2) return -2;
                    if (slot < 0) break;           // no state slot free
                }
                const int n = portion((int)r.tokens.size(), budget);
                const int rc = mgr_->reserve(rid, n);
                if (rc < 0) return -2;
                if (rc == 0) {
                    if (mgr_->release(rid) != 0) return -2;
                    if (running_.empty() && plan_.empty()) {
                        // alone and still too large for the free pages: it can never run
                        waiting_.pop_front();
                        finish(r, OUT_OF_PAGES);
                        ++m_finished_;
                        continue;
                    }
                    break;
                }
                waiting_.pop_front();
                r.state = RUNNING;
                r.admit_seq = seq_++;
                running_.push_back(rid);
                ++m_admitted_;
                events_.push_back({rid, EV_ADMITTED, (int)r.admit_seq});
                plan_.push_back({rid, 0, n, n == (int)r.tokens.size() ? 1 : 0});
                budget -= n;
            }
            if (!plan_.empty()) ++m_steps_;
            for (auto& p : plan_) m_tokens_ += p.count;
            return (int)plan_.size();
        }
    }
    // 1: finished, 0: goes on
    int accept_token(int64_t rid, int tok) {
        SchedRequest* r = find(rid);
        if (!r) return -2;
        r->tokens.push_back(tok);
        ++r->generated;
        int why = NONE;
        if (std::find(r->stop_ids.begin(), r->stop_ids.end(), tok) != r->stop_ids.end()) why = STOP;
        else if (r->generated >= r->max_new) why = LENGTH;
        else if ((int)r->tokens.size() >= max_seq_) why = CONTEXT;
        if (why == NONE) return 0;
        if (mgr_->release(rid) != 0) return -2;
        running_.erase(std::remove(running_.begin(), running_.end(), rid), running_.end());
        finish(*r, why);
        ++m_finished_;
        return 1;
    }
    int commit(int n, const int64_t* rids, const int* starts, const int* counts, const int* samples, const int* sampled) {
        events_.clear();
        for (int i = 0; i < n; ++i) {
            if (mgr_->commit(rids[i], starts[i] + counts[i]) != 0) return -2;
            if (!samples[i]) continue;
            if (accept_token(rids[i], sampled[i]) < 0) return -2;
        }
        return 0;
    }
    bool all_decoding() {
        if (running_.empty() || !waiting_.empty()) return false;
        for (int64_t rid : running_)
            if (remaining(reqs_[rid]) != 1) return false;
        return true;
    }
    int cancel(int64_t rid) {
        auto it = reqs_.find(rid);
        if (it == reqs_.end() || it->second.state == FINISHED) return 0;
        SchedRequest& r = it->second;
        if (r.state == RUNNING) {
            if (mgr_->release(rid) != 0) return -2;
            running_.erase(std::remove(running_.begin(), running_.end(), rid), running_.end());
        } else {
            waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), rid), waiting_.end());
            if (mgr_->has(rid) && mgr_->release(rid) != 0) return -2;
        }
        r.state = FINISHED;
        r.finish = CANCELLED;
        finished_.push_back(rid);
        return 1;
    }

    CacheManager* mgr_;
    int budget_, max_active_, chunk_, max_seq_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_, finished_;
    std::unordered_map<int64_t, SchedRequest> reqs_;
    std::vector<PlanEntry> plan_;
    std::vector<SchedEvent> events_;
    long long seq_ = 0;
    long long m_admitted_ = 0, m_finished_ = 0, m_preempted_ = 0, m_rejected_ = 0, m_steps_ = 0, m_tokens_ = 0;
};

}  // namespace

#define MMH extern "C" __attribute__((visibility("default")))

MMH const char* mmh_last_error() { return g_error.c_str(); }

// ---- page allocator ----
MMH void* mmh_alloc_create(int n) { return n < 0 ? nullptr : new PageAllocator(n); }
MMH void mmh_alloc_destroy(void* h) { delete static_cast<PageAllocator*>(h); }
MMH int mmh_alloc_alloc(void* h) { return static_cast<PageAllocator*>(h)->alloc(); }
MMH int mmh_alloc_free(void* h, int page) { return static_cast<PageAllocator*>(h)->free(page); }
MMH int mmh_alloc_is_allocated(void* h, int page) { return static_cast<PageAllocator*>(h)->is_allocated(page) ? 1 : 0; }
MMH int mmh_alloc_check(void* h) { return static_cast<PageAllocator*>(h)->check(); }
// what: 0 pages, 1 free, 2 used, 3 allocations so far, 4 allocations of a page used before
MMH long long mmh_alloc_stat(void* h, int what) {
    PageAllocator* a = static_cast<PageAllocator*>(h);
    switch (what) {
        case 0: return a->num_pages();
        case 1: return a->num_free();
        case 2: return a->num_used();
        case 3: return a->total_allocs();
        default: return a->reuses();
    }
}

// ---- cache manager ----
MMH void* mmh_cache_create(int n_groups, const int* pages, const int* windows, int page_size, int max_requests) {
    if (n_groups < 0 || page_size <= 0 || max_requests < 0) return nullptr;
    return new CacheManager(n_groups, pages, windows, page_size, max_requests);
}
MMH void mmh_cache_destroy(void* h) { delete static_cast<CacheManager*>(h); }
MMH int mmh_cache_has(void* h, long long rid) { return static_cast<CacheManager*>(h)->has(rid) ? 1 : 0; }
MMH int mmh_cache_add(void* h, long long rid) { return static_cast<CacheManager*>(h)->add(rid); }
// what: 0 length, 1 slot, 2 reserved, 3 "first call?" (marks the request started)
MMH int mmh_cache_request(void* h, long long rid, int what) {
    CacheRequest* r = static_cast<CacheManager*>(h)->find(rid);
    if (!r) return -2;
    switch (what) {
        case 0: return r->length;
        case 1: return r->slot;
        case 2: return r->reserved;
        default: {
            const int first = r->started ? 0 : 1;
            r->started = true;
            return first;
        }
    }
}
MMH int mmh_cache_pages_needed(void* h, long long rid, int new_len, int* out) { return static_cast<CacheManager*>(h)->pages_needed(rid, new_len, out); }
MMH int mmh_cache_reserve(void* h, long long rid, int new_len) { return static_cast<CacheManager*>(h)->reserve(rid, new_len); }
MMH int mmh_cache_commit(void* h, long long rid, int new_len) { return static_cast<CacheManager*>(h)->commit(rid, new_len); }
MMH int mmh_cache_release(void* h, long long rid) { return static_cast<CacheManager*>(h)->release(rid); }
// copies up to cap entries of the request's block table of a group; returns the table's length
MMH int mmh_cache_table(void* h, long long rid, int group, int* out, int cap) {
    CacheManager* m = static_cast<CacheManager*>(h);
    CacheRequest* r = m->find(rid);
    if (!r) return -2;
    if (group < 0 || group >= m->n_groups()) return fail("no such cache group");
    const auto& t = r->tables[group];
    const int n = std::min((int)t.size(), cap);
    if (n > 0) std::memcpy(out, t.data(), sizeof(int32_t) * n);
    return (int)t.size();
}
// fills rows [n, width] of block tables (entries beyond a table's end are -1): the batch's tables in one call
MMH int mmh_cache_tables(void* h, int group, int n, const long long* rids, int width, int* out) {
    CacheManager* m = static_cast<CacheManager*>(h);
    if (group < 0 || group >= m->n_groups()) return fail("no such cache group");
    for (int i = 0; i < n; ++i) {
        CacheRequest* r = m->find(rids[i]);
        if (!r) return -2;
        const auto& t = r->tables[group];
        const int k = std::min((int)t.size(), width);
        if (k > 0) std::memcpy(out + (size_t)i * width, t.data(), sizeof(int32_t) * k);
        for (int j = k; j < width; ++j) out[(size_t)i * width + j] = INVALID_PAGE;
    }
    return 0;
}
// what: 0 number of groups, 1 page size, 2 pages of a group, 3 free pages of a group
MMH int mmh_cache_info(void* h, int what, int group) {
    CacheManager* m = static_cast<CacheManager*>(h);
    if (what == 0) return m->n_groups();
    if (what == 1) return m->page_size();
    if (group < 0 || group >= m->n_groups()) return fail("no such cache group");
    return what == 2 ? m->allocator(group).num_pages() : m->allocator(group).num_free();
}
MMH void* mmh_cache_allocator(void* h, int group) {
    CacheManager* m = static_cast<CacheManager*>(h);
    if (group == -1) return &m->slots();
    return (group < 0 || group >= m->n_groups()) ? nullptr : &m->allocator(group);
}
MMH int mmh_cache_live(void* h, long long* out, int cap) {
    CacheManager* m = static_cast<CacheManager*>(h);
    int n = 0;
    for (auto& kv : m->requests()) {
        if (n < cap) out[n] = kv.first;
        ++n;
    }
    return n;
}
MMH int mmh_cache_check(void* h) { return static_cast<CacheManager*>(h)->check(); }

// ---- scheduler ----
MMH void* mmh_sched_create(void* cache, int token_budget, int max_active, int prefill_chunk, int max_seq_len) {
    if (cache == nullptr) return nullptr;
    return new Scheduler(static_cast<CacheManager*>(cache), token_budget, max_active, prefill_chunk, max_seq_len);
}
MMH void mmh_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }
// 1 queued, 0 rejected (finished at once; the reason: mmh_sched_reject_reason), -2 error
MMH int mmh_sched_add(void* h, long long rid, const int* prompt, int n, int max_new, const int* stop, int n_stop) {
    return static_cast<Scheduler*>(h)->add(rid, prompt, n, max_new, stop, n_stop);
}
MMH const char* mmh_sched_reject_reason(void* h, long long rid) {
    SchedRequest* r = static_cast<Scheduler*>(h)->find(rid);
    return r ? r->reject_reason.c_str() : "";
}
MMH int mmh_sched_has_work(void* h) { return static_cast<Scheduler*>(h)->has_work() ? 1 : 0; }
MMH int mmh_sched_all_decoding(void* h) { return static_cast<Scheduler*>(h)->all_decoding() ? 1 : 0; }
// plans the next step (reserves its pages; may preempt or fail requests); returns the number of entries
MMH int mmh_sched_schedule(void* h) { return static_cast<Scheduler*>(h)->schedule(); }
MMH int mmh_sched_plan(void* h, long long* rids, int* starts, int* counts, int* samples, int cap) {
    Scheduler* s = static_cast<Scheduler*>(h);
    const int n = std::min((int)s->plan_.size(), cap);
    for (int i = 0; i < n; ++i) {
        rids[i] = s->plan_[i].rid;
        starts[i] = s->plan_[i].start;
        counts[i] = s->plan_[i].count;
        samples[i] = s->plan_[i].samples;
    }
    return (int)s->plan_.size();
}
// what the last schedule / commit / accept_token did to requests: (request, kind 1 admitted 2 preempted 3 finished, code)
MMH int mmh_sched_events(void* h, long long* rids, int* kinds, int* codes, int cap) {
    Scheduler* s = static_cast<Scheduler*>(h);
    const int n = std::min((int)s->events_.size(), cap);
    for (int i = 0; i < n; ++i) {
        rids[i] = s->events_[i].rid;
        kinds[i] = s->events_[i].kind;
        codes[i] = s->events_[i].code;
    }
    return (int)s->events_.size();
}
MMH int mmh_sched_commit(void* h, int n, const long long* rids, const int* starts, const int* counts, const int* samples, const int* sampled) {
    return static_cast<Scheduler*>(h)->commit(n, reinterpret_cast<const int64_t*>(rids), starts, counts, samples, sampled);
}
// how a request's tokens are drawn; values as the caller resolved them (seed != 0)
MMH int mmh_sched_set_sampling(void* h, long long rid, float temperature, int top_k, float top_p, long long seed, float frequency,
                               float presence, float repetition, int penalty_window, float softcap) {
    SchedRequest* r = static_cast<Scheduler*>(h)->find(rid);
    if (!r) return -2;
    r->temperature = temperature; r->top_k = top_k; r->top_p = top_p; r->seed = seed;
    r->frequency = frequency; r->presence = presence; r->repetition = repetition; r->penalty_window = penalty_window; r->softcap = softcap;
    return 0;
}
// f: temperature, top_p, repetition, frequency, presence, softcap; i: top_k, penalty_window, tokens generated so far, tokens in all
MMH int mmh_sched_get_sampling(void* h, long long rid, float* f, int* i, long long* seed) {
    SchedRequest* r = static_cast<Scheduler*>(h)->find(rid);
    if (!r) return -2;
    f[0] = r->temperature; f[1] = r->top_p; f[2] = r->repetition; f[3] = r->frequency; f[4] = r->presence; f[5] = r->softcap;
    i[0] = r->top_k; i[1] = r->penalty_window; i[2] = r->generated; i[3] = (int)r->tokens.size();
    *seed = r->seed;
    return 0;
}
MMH int mmh_sched_accept_token(void* h, long long rid, int tok) {
    Scheduler* s = static_cast<Scheduler*>(h);
    s->events_.clear();
    return s->accept_token(rid, tok);
}
MMH int mmh_sched_cancel(void* h, long long rid) { return static_cast<Scheduler*>(h)->cancel(rid); }
// what: 0 state, 1 finish code, 2 preemptions, 3 generated, 4 tokens, 5 admission number
MMH long long mmh_sched_request(void* h, long long rid, int what) {
    SchedRequest* r = static_cast<Scheduler*>(h)->find(rid);
    if (!r) return -2;
    switch (what) {
        case 0: return r->state;
        case 1: return r->finish;
        case 2: return r->preemptions;
        case 3: return r->generated;
        case 4: return (long long)r->tokens.size();
        default: return r->admit_seq;
    }
}
MMH int mmh_sched_tokens(void* h, long long rid, int start, int count, int* out) {
    SchedRequest* r = static_cast<Scheduler*>(h)->find(rid);
    if (!r) return -2;
    if (start < 0 || count < 0 || start + count > (int)r->tokens.size()) return fail("token range outside the request");
    if (count > 0) std::memcpy(out, r->tokens.data() + start, sizeof(int32_t) * count);
    return count;
}
// which: 0 waiting, 1 running, 2 finished (in their order)
MMH int mmh_sched_list(void* h, int which, long long* out, int cap) {
    Scheduler* s = static_cast<Scheduler*>(h);
    int n = 0;
    auto put = [&](int64_t rid) {
        if (n < cap) out[n] = rid;
        ++n;
    };
    if (which == 0) for (int64_t r : s->waiting_) put(r);
    else if (which == 1) for (int64_t r : s->running_) put(r);
    else for (int64_t r : s->finished_) put(r);
    return n;
}
// what: 0 admitted, 1 finished, 2 preempted, 3 rejected, 4 steps, 5 tokens scheduled
MMH long long mmh_sched_metric(void* h, int what) {
    Scheduler* s = static_cast<Scheduler*>(h);
    switch (what) {
        case 0: return s->m_admitted_;
        case 1: return s->m_finished_;
        case 2: return s->m_preempted_;
        case 3: return s->m_rejected_;
        case 4: return s->m_steps_;
        default: return s->m_tokens_;
    }
}
