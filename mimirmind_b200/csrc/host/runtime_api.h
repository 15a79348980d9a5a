// C interface of the host runtime (runtime.cpp: page allocator, cache manager, scheduler) as other native code
// of this project uses it.  Handles are the opaque pointers the create functions return; a result of -2 means an
// error whose text is mmh_last_error().
#pragma once

extern "C" {
const char* mmh_last_error();

// cache manager
int mmh_cache_has(void* cache, long long rid);
int mmh_cache_request(void* cache, long long rid, int what);   // what: 0 length, 1 state slot, 2 reserved, 3 first step? (marks it)
int mmh_cache_pages_needed(void* cache, long long rid, int new_len, int* out_per_group);
int mmh_cache_reserve(void* cache, long long rid, int new_len);
int mmh_cache_commit(void* cache, long long rid, int new_len);
int mmh_cache_tables(void* cache, int group, int n, const long long* rids, int width, int* out);
int mmh_cache_info(void* cache, int what, int group);           // what: 0 groups, 1 page size, 2 pages of group, 3 free pages of group

// scheduler
int mmh_sched_schedule(void* sched);
int mmh_sched_plan(void* sched, long long* rids, int* starts, int* counts, int* samples, int cap);
int mmh_sched_tokens(void* sched, long long rid, int start, int count, int* out);
long long mmh_sched_request(void* sched, long long rid, int what);
int mmh_sched_events(void* sched, long long* rids, int* kinds, int* codes, int cap);
int mmh_sched_get_sampling(void* sched, long long rid, float* f6, int* i4, long long* seed);
int mmh_sched_accept_token(void* sched, long long rid, int token);    // 1: the request finished, 0: it goes on
int mmh_sched_commit(void* sched, int n, const long long* rids, const int* starts, const int* counts, const int* samples,
                     const int* sampled);
}
