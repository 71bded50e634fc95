// C entry points of the host runtime (cache manager and scheduler), called
// from Python through ctypes.  Handles are opaque pointers; every function
// returns a status or a count, never throws across the boundary.
#include <cstring>

#include "cache_manager.hpp"
#include "scheduler.hpp"

using namespace railgun;

#define RG_GUARD(expr) try { expr; } catch (...) { return CACHE_CORRUPT; }

extern "C" {

void* rg_cache_create(int n_groups, const int* page_size, const int* num_pages, const int* window, int max_slots) {
    if (n_groups < 0 || max_slots < 0) return nullptr;
    for (int g = 0; g < n_groups; ++g)
        if (page_size[g] <= 0 || num_pages[g] < 0 || window[g] < 0) return nullptr;
    try { return new CacheManager(n_groups, page_size, num_pages, window, max_slots); } catch (...) { return nullptr; }
}
void rg_cache_destroy(void* h) { delete (CacheManager*)h; }
int rg_cache_add_request(void* h, long long id) { RG_GUARD(return ((CacheManager*)h)->add_request(id)) }
int rg_cache_reserve(void* h, long long id, int new_len) { RG_GUARD(return ((CacheManager*)h)->reserve(id, new_len)) }
int rg_cache_can_reserve(void* h, long long id, int new_len, int spare) {
    RG_GUARD(return ((CacheManager*)h)->can_reserve(id, new_len, spare) ? 1 : 0)
}
int rg_cache_commit(void* h, long long id, int new_len) { RG_GUARD(return ((CacheManager*)h)->commit(id, new_len)) }
int rg_cache_release(void* h, long long id) { RG_GUARD(return ((CacheManager*)h)->release(id)) }
int rg_cache_has(void* h, long long id) { return ((CacheManager*)h)->has(id) ? 1 : 0; }
int rg_cache_num_computed(void* h, long long id) {
    const CacheRequest* r = ((CacheManager*)h)->find(id);
    return r ? r->num_computed : CACHE_UNKNOWN_REQUEST;
}
int rg_cache_slot(void* h, long long id) {
    const CacheRequest* r = ((CacheManager*)h)->find(id);
    return r ? r->slot : CACHE_UNKNOWN_REQUEST;
}
// Copies the request's block table of one group; returns its length (may exceed cap: call again).
int rg_cache_table(void* h, long long id, int group, int* out, int cap) {
    CacheManager* c = (CacheManager*)h;
    const CacheRequest* r = c->find(id);
    if (!r) return CACHE_UNKNOWN_REQUEST;
    if (group < 0 || group >= c->num_groups()) return CACHE_BAD_ARGUMENT;
    const std::vector<int>& t = r->tables[group];
    const int n = (int)t.size();
    if (n && cap > 0) std::memcpy(out, t.data(), sizeof(int) * (size_t)(n < cap ? n : cap));
    return n;
}
// Packs a pure-decode step (one new token per request) for `R` requests into `out`, laid out for a static
// batch of `B` rows and block tables `MB` wide:
//   positions[B] | context_lens[B] | start_pos[B] | state_slots[B] | per group: slots[B] | per group: table[B*MB]
// Rows R..B-1 are padding: position 0, context 1, slot -1 (nothing is written), table of zeros.
// Pages for the new token are reserved here.  Returns 0, or a negative status (nothing half-reserved matters:
// a failed request keeps what it had).
int rg_cache_pack_decode(void* h, const long long* ids, int R, int B, int MB, int* out) {
    try {
        CacheManager* c = (CacheManager*)h;
        const int G = c->num_groups();
        int* positions = out;
        int* context = out + B;
        int* start = out + 2 * B;
        int* slots_state = out + 3 * B;
        int* slot_map = out + 4 * B;                       // G blocks of B
        int* tables = out + (4 + G) * B;                   // G blocks of B*MB
        std::memset(out, 0, sizeof(int) * ((size_t)(4 + G) * B + (size_t)G * B * MB));
        for (int b = R; b < B; ++b) {
            context[b] = 1;
            for (int g = 0; g < G; ++g) slot_map[g * B + b] = -1;
        }
        for (int b = 0; b < R; ++b) {
            const CacheRequest* r = c->find(ids[b]);
            if (!r) return CACHE_UNKNOWN_REQUEST;
            const int pos = r->num_computed;
            const int st = c->reserve(ids[b], pos + 1);
            if (st != CACHE_OK) return st;
            r = c->find(ids[b]);
            positions[b] = pos;
            context[b] = pos + 1;
            start[b] = pos;
            slots_state[b] = r->slot;
            for (int g = 0; g < G; ++g) {
                const std::vector<int>& t = r->tables[g];
                const int ps = c->group(g).page_size;
                if ((int)t.size() > MB) return CACHE_BAD_ARGUMENT;
                int* row = tables + ((size_t)g * B + b) * MB;
                for (size_t i = 0; i < t.size(); ++i) row[i] = t[i] < 0 ? 0 : t[i];
                slot_map[g * B + b] = t[pos / ps] * ps + pos % ps;
            }
        }
        return CACHE_OK;
    } catch (...) { return CACHE_CORRUPT; }
}
// Every listed request now holds `n` more tokens.
int rg_cache_advance(void* h, const long long* ids, int R, int n) {
    try {
        CacheManager* c = (CacheManager*)h;
        for (int b = 0; b < R; ++b) {
            const CacheRequest* r = c->find(ids[b]);
            if (!r) return CACHE_UNKNOWN_REQUEST;
            const int st = c->commit(ids[b], r->num_computed + n);
            if (st != CACHE_OK) return st;
        }
        return CACHE_OK;
    } catch (...) { return CACHE_CORRUPT; }
}
int rg_cache_free_pages(void* h, int group) { return ((CacheManager*)h)->free_pages(group); }
int rg_cache_free_slots(void* h) { return ((CacheManager*)h)->free_slots(); }
int rg_cache_num_requests(void* h) { return ((CacheManager*)h)->num_requests(); }
int rg_cache_check(void* h) { RG_GUARD(return ((CacheManager*)h)->check()) }

void* rg_sched_create(void* cache, int max_num_batched_tokens, int max_num_seqs, int max_prefill_chunk,
                      int max_model_len) {
    if (!cache || max_num_batched_tokens < 1 || max_num_seqs < 1 || max_prefill_chunk < 0 || max_model_len < 1)
        return nullptr;
    SchedConfig cfg;
    cfg.max_num_batched_tokens = max_num_batched_tokens;
    cfg.max_num_seqs = max_num_seqs;
    cfg.max_prefill_chunk = max_prefill_chunk;
    cfg.max_model_len = max_model_len;
    try { return new Scheduler((CacheManager*)cache, cfg); } catch (...) { return nullptr; }
}
void rg_sched_destroy(void* h) { delete (Scheduler*)h; }
int rg_sched_add_request(void* h, long long id, const int* prompt, int n, int max_new_tokens, const int* stop,
                         int n_stop) {
    RG_GUARD(return ((Scheduler*)h)->add_request(id, prompt, n, max_new_tokens, stop, n_stop))
}
// Decides the next step and writes it flat: per entry id/start/count/want_last, and all entries' tokens
// one after the other.  Returns the number of entries, or -(needed token capacity) - 1000000 if a buffer is
// too small (nothing is lost: call rg_sched_fetch with larger buffers).
static int write_step(Scheduler* s, long long* ids, int* start, int* count, int* want, int cap_entries,
                      int* tokens, int cap_tokens) {
    const auto& es = s->entries();
    int total = 0;
    for (const StepEntry& e : es) total += e.count;
    if ((int)es.size() > cap_entries || total > cap_tokens) return -1000000 - total;
    int off = 0;
    for (size_t i = 0; i < es.size(); ++i) {
        const StepEntry& e = es[i];
        ids[i] = e.id; start[i] = e.start; count[i] = e.count; want[i] = e.want_last;
        const SchedRequest* r = s->find(e.id);
        std::memcpy(tokens + off, r->tokens.data() + e.start, sizeof(int) * (size_t)e.count);
        off += e.count;
    }
    return (int)es.size();
}
int rg_sched_schedule(void* h, long long* ids, int* start, int* count, int* want, int cap_entries,
                      int* tokens, int cap_tokens) {
    try {
        Scheduler* s = (Scheduler*)h;
        s->schedule();
        return write_step(s, ids, start, count, want, cap_entries, tokens, cap_tokens);
    } catch (...) { return CACHE_CORRUPT; }
}
int rg_sched_fetch(void* h, long long* ids, int* start, int* count, int* want, int cap_entries,
                   int* tokens, int cap_tokens) {
    RG_GUARD(return write_step((Scheduler*)h, ids, start, count, want, cap_entries, tokens, cap_tokens))
}
int rg_sched_preempted(void* h, long long* out, int cap) {
    const auto& p = ((Scheduler*)h)->preempted();
    for (int i = 0; i < (int)p.size() && i < cap; ++i) out[i] = p[i];
    return (int)p.size();
}
int rg_sched_update(void* h, const long long* ids, const int* tokens, int n) {
    RG_GUARD(return ((Scheduler*)h)->update((const int64_t*)ids, tokens, n))
}
int rg_sched_abort(void* h, long long id) { RG_GUARD(return ((Scheduler*)h)->abort(id)) }
int rg_sched_finished(void* h, long long* out, int cap) {
    const auto& f = ((Scheduler*)h)->finished();
    for (int i = 0; i < (int)f.size() && i < cap; ++i) out[i] = f[i];
    return (int)f.size();
}
// finish reason (0 while alive), or SCHED_UNKNOWN
int rg_sched_finish_reason(void* h, long long id) {
    const SchedRequest* r = ((Scheduler*)h)->find(id);
    return r ? r->finish : SCHED_UNKNOWN;
}
int rg_sched_num_generated(void* h, long long id) {
    const SchedRequest* r = ((Scheduler*)h)->find(id);
    return r ? r->num_generated() : SCHED_UNKNOWN;
}
int rg_sched_num_preemptions(void* h, long long id) {
    const SchedRequest* r = ((Scheduler*)h)->find(id);
    return r ? r->num_preemptions : SCHED_UNKNOWN;
}
// generated tokens of a request; returns their number
int rg_sched_outputs(void* h, long long id, int* out, int cap) {
    const SchedRequest* r = ((Scheduler*)h)->find(id);
    if (!r) return SCHED_UNKNOWN;
    const int n = r->num_generated();
    for (int i = 0; i < n && i < cap; ++i) out[i] = r->tokens[r->prompt_len + i];
    return n;
}
int rg_sched_error(void* h, long long id, char* out, int cap) {
    const std::string& e = ((Scheduler*)h)->error_of(id);
    if (cap > 0) {
        std::strncpy(out, e.c_str(), (size_t)cap - 1);
        out[cap - 1] = 0;
    }
    return (int)e.size();
}
void rg_sched_forget(void* h, long long id) { ((Scheduler*)h)->forget(id); }
int rg_sched_num_waiting(void* h) { return ((Scheduler*)h)->num_waiting(); }
int rg_sched_num_running(void* h) { return ((Scheduler*)h)->num_running(); }

}  // extern "C"
