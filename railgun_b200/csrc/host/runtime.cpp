// C entry points of the host runtime (cache manager and scheduler), called
// from Python through ctypes.  Handles are opaque pointers; every function
// returns a status or a count, never throws across the boundary.
#include <cstring>
#include <unordered_map>
#include <vector>

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
    const RequestRecord* r = ((CacheManager*)h)->record(id);
    return r ? r->num_computed : CACHE_UNKNOWN_REQUEST;
}
// The records of all state slots, in place: max_slots records of rg_cache_record_bytes() bytes, record s for
// slot s (request_id -1: free).  The memory lives as long as the cache manager.
const void* rg_cache_records(void* h) { return ((CacheManager*)h)->records(); }
int rg_cache_record_bytes() { return (int)sizeof(RequestRecord); }
// Sets what the cache manager does not work out itself in a live request's record (a scheduler does this at
// admission; callers without one, to have decode steps sample).
int rg_cache_set_request(void* h, long long id, int prompt_len, int num_generated, int max_new_tokens,
                         float temperature, int top_k, float top_p, unsigned long long seed) {
    RequestRecord* r = ((CacheManager*)h)->record(id);
    if (!r) return CACHE_UNKNOWN_REQUEST;
    if (!(temperature >= 0.f) || top_k < 0 || !(top_p > 0.f && top_p <= 1.f) || num_generated < 0) return CACHE_BAD_ARGUMENT;
    r->prompt_len = prompt_len; r->num_generated = num_generated; r->max_new_tokens = max_new_tokens;
    r->temperature = temperature; r->top_k = top_k; r->top_p = top_p; r->seed = seed;
    return CACHE_OK;
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
// Rows R..B-1 are padding: position 0, context 1, cache slot -1 (nothing is written), state slot -1 (no
// request: a part with per-request state leaves such rows alone), table of zeros.
// Pages for the new token are reserved here.  `ahead` > 0 packs the step that many steps after the next one (for a
// step launched before the one before it has been committed): its position is num_computed + ahead.
// `sampling` (may be null): the rows' sampling parameters from the requests' records, as 7 B 32-bit words:
//   seed[B] (64-bit) | draw counter[B] (64-bit) = num_generated + draw_ahead | temperature[B] | top_k[B] | top_p[B]
// with padding rows greedy; *any_sampled says whether a row has a temperature above zero.  Returns 0, or
// a negative status (nothing half-reserved matters: a failed request keeps what it had).
int rg_cache_pack_decode(void* h, const long long* ids, int R, int B, int MB, int* out, int ahead, int* sampling,
                         int draw_ahead, int* any_sampled) {
    try {
        CacheManager* c = (CacheManager*)h;
        if (ahead < 0 || draw_ahead < 0) return CACHE_BAD_ARGUMENT;
        if (any_sampled) *any_sampled = 0;
        if (sampling) {
            std::memset(sampling, 0, sizeof(int) * (size_t)7 * B);
            float* top_p = reinterpret_cast<float*>(sampling + 6 * B);
            for (int b = 0; b < B; ++b) top_p[b] = 1.f;
        }
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
            slots_state[b] = -1;
            for (int g = 0; g < G; ++g) slot_map[g * B + b] = -1;
        }
        for (int b = 0; b < R; ++b) {
            const CacheRequest* r = c->find(ids[b]);
            if (!r) return CACHE_UNKNOWN_REQUEST;
            const RequestRecord* rec = c->record(ids[b]);
            const int pos = rec->num_computed + ahead;
            const int st = c->reserve(ids[b], pos + 1);
            if (st != CACHE_OK) return st;
            r = c->find(ids[b]);
            if (sampling) {
                reinterpret_cast<unsigned long long*>(sampling)[b] = rec->seed;
                reinterpret_cast<long long*>(sampling + 2 * B)[b] = (long long)rec->num_generated + draw_ahead;
                reinterpret_cast<float*>(sampling + 4 * B)[b] = rec->temperature;
                sampling[5 * B + b] = rec->top_k;
                reinterpret_cast<float*>(sampling + 6 * B)[b] = rec->top_p;
                if (any_sampled && rec->temperature > 0.f) *any_sampled = 1;
            }
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
// Plans a step of any shape: request b brings counts[b] >= 1 next tokens and asks for the logits at the places
// want[want_offsets[b] .. want_offsets[b+1]) among them.  Everything is checked before anything is reserved; then
// unknown requests are added and pages reserved for every request (a request added here is released again if a
// reservation fails).  Writes every request's start position and, per group, the width of the widest block table
// rounded up to a power of two.  Returns CACHE_OK, or a status with *bad = the entry it is about:
// CACHE_DUPLICATE (a request twice in one step), CACHE_BAD_ARGUMENT (no tokens), STEP_BEYOND_MAX_POSITION,
// STEP_BAD_WANT (a wanted place outside the entry's tokens; *bad_value = the place), or a reservation's status.
enum StepStatus : int { STEP_BEYOND_MAX_POSITION = -7, STEP_BAD_WANT = -8 };

int rg_cache_plan_step(void* h, const long long* ids, const int* counts, int R, const int* want,
                       const int* want_offsets, int max_position, int* starts, int* max_blocks, int* bad,
                       int* bad_value) {
    try {
        CacheManager* c = (CacheManager*)h;
        const int G = c->num_groups();
        std::unordered_map<long long, int> seen;
        seen.reserve((size_t)R * 2);
        for (int b = 0; b < R; ++b) {
            *bad = b;
            if (!seen.emplace(ids[b], b).second) return CACHE_DUPLICATE;
            if (counts[b] < 1) return CACHE_BAD_ARGUMENT;
            starts[b] = c->num_computed(ids[b]);
            if ((long long)starts[b] + counts[b] > max_position) return STEP_BEYOND_MAX_POSITION;
            for (int w = want_offsets[b]; w < want_offsets[b + 1]; ++w)
                if (want[w] < 0 || want[w] >= counts[b]) { *bad_value = want[w]; return STEP_BAD_WANT; }
        }
        std::vector<long long> added;
        int status = CACHE_OK;
        for (int b = 0; b < R && status == CACHE_OK; ++b) {
            *bad = b;
            if (!c->has(ids[b])) {
                const int slot = c->add_request(ids[b]);
                if (slot < 0) { status = slot; break; }
                added.push_back(ids[b]);
            }
            status = c->reserve(ids[b], starts[b] + counts[b]);
        }
        if (status != CACHE_OK) {
            for (long long id : added) c->release(id);
            return status;
        }
        for (int g = 0; g < G; ++g) {
            size_t widest = 1;
            for (int b = 0; b < R; ++b) {
                const size_t n = c->find(ids[b])->tables[g].size();
                if (n > widest) widest = n;
            }
            int p2 = 1;
            while ((size_t)p2 < widest) p2 <<= 1;
            max_blocks[g] = p2;
        }
        return CACHE_OK;
    } catch (...) { return CACHE_CORRUPT; }
}

// Writes a planned step into its packed buffer.  seg[i] is the offset (in ints) of segment i of `out`:
//   0 token ids [T] | 1 positions [T] | 2 request of token [T] | 3 wanted rows [W] | 4 cu_seqlens [R+1] |
//   5 context lens [R] | 6 start positions [R] | 7 state slots [R] | per group g: 8+2g cache slot of each token [T],
//   9+2g block table [R, max_blocks[g]] (released pages as 0: they are never read) |
//   8+2G tiles of <= tile_rows consecutive rows of requests with several tokens, (first row, rows, request) |
//   9+2G rows of requests with one token | 10+2G the same tiles with <= 2 * tile_rows rows.
int rg_cache_fill_step(void* h, const long long* ids, const int* counts, const int* starts, int R,
                       const long long* tokens, const int* want, const int* want_offsets, const int* max_blocks,
                       int tile_rows, const long long* seg, int* out) {
    try {
        CacheManager* c = (CacheManager*)h;
        const int G = c->num_groups();
        int* tok = out + seg[0];
        int* pos = out + seg[1];
        int* req = out + seg[2];
        int* want_rows = out + seg[3];
        int* cu = out + seg[4];
        int* ctx = out + seg[5];
        int* start = out + seg[6];
        int* slots = out + seg[7];
        int* tiles = out + seg[8 + 2 * G];
        int* dec = out + seg[9 + 2 * G];
        int* tiles2 = out + seg[10 + 2 * G];
        int off = 0, nw = 0;
        cu[0] = 0;
        for (int b = 0; b < R; ++b) {
            const CacheRequest* r = c->find(ids[b]);
            if (!r) return CACHE_UNKNOWN_REQUEST;
            const int n = counts[b], s = starts[b];
            for (int k = 0; k < n; ++k) {
                tok[off + k] = (int)tokens[off + k];
                pos[off + k] = s + k;
                req[off + k] = b;
            }
            for (int w = want_offsets[b]; w < want_offsets[b + 1]; ++w) want_rows[nw++] = off + want[w];
            cu[b + 1] = off + n;
            ctx[b] = s + n;
            start[b] = s;
            slots[b] = r->slot;
            for (int g = 0; g < G; ++g) {
                const std::vector<int>& t = r->tables[g];
                const int ps = c->group(g).page_size, MB = max_blocks[g];
                if ((int)t.size() > MB || (size_t)(s + n - 1) / ps >= t.size()) return CACHE_BAD_ARGUMENT;
                int* row = out + seg[9 + 2 * g] + (size_t)b * MB;
                for (int i = 0; i < MB; ++i) row[i] = i < (int)t.size() && t[i] > 0 ? t[i] : 0;
                int* sm = out + seg[8 + 2 * g] + off;
                for (int k = 0; k < n; ++k) {
                    const int p = s + k;
                    sm[k] = row[p / ps] * ps + p % ps;
                }
            }
            if (n == 1) {
                *dec++ = off;
            } else {
                for (int k = 0; k < n; k += tile_rows) {
                    *tiles++ = off + k; *tiles++ = n - k < tile_rows ? n - k : tile_rows; *tiles++ = b;
                }
                for (int k = 0; k < n; k += 2 * tile_rows) {
                    *tiles2++ = off + k; *tiles2++ = n - k < 2 * tile_rows ? n - k : 2 * tile_rows; *tiles2++ = b;
                }
            }
            off += n;
        }
        return CACHE_OK;
    } catch (...) { return CACHE_CORRUPT; }
}
// Request b now holds new_len[b] tokens (the step that was packed for them ran).
int rg_cache_commit_many(void* h, const long long* ids, const int* new_len, int R) {
    try {
        CacheManager* c = (CacheManager*)h;
        for (int b = 0; b < R; ++b) {
            const int st = c->commit(ids[b], new_len[b]);
            if (st != CACHE_OK) return st;
        }
        return CACHE_OK;
    } catch (...) { return CACHE_CORRUPT; }
}
// Every listed request now holds `n` more tokens.
int rg_cache_advance(void* h, const long long* ids, int R, int n) {
    try {
        CacheManager* c = (CacheManager*)h;
        for (int b = 0; b < R; ++b) {
            if (!c->has(ids[b])) return CACHE_UNKNOWN_REQUEST;
            const int st = c->commit(ids[b], c->num_computed(ids[b]) + n);
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
                         int n_stop, float temperature, int top_k, float top_p, unsigned long long seed) {
    RG_GUARD(return ((Scheduler*)h)->add_request(id, prompt, n, max_new_tokens, stop, n_stop, temperature, top_k,
                                                 top_p, seed))
}
// The sampling parameters of n requests (waiting, running or finished), and the number of each one's next draw.
int rg_sched_sampling_many(void* h, const long long* ids, int n, float* temperature, int* top_k, float* top_p,
                           long long* seed, long long* counter) {
    try {
        for (int i = 0; i < n; ++i) {
            const SchedRequest* r = ((Scheduler*)h)->find(ids[i]);
            if (!r) return SCHED_UNKNOWN;
            temperature[i] = r->temperature; top_k[i] = r->top_k; top_p[i] = r->top_p;
            seed[i] = (long long)r->seed; counter[i] = r->num_generated();
        }
        return 0;
    } catch (...) { return SCHED_BAD_ARGUMENT; }
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
// How many tokens each of the n requests has generated; returns 0, or SCHED_UNKNOWN at the first unknown id.
int rg_sched_num_generated_many(void* h, const long long* ids, int n, long long* out) {
    try {
        for (int i = 0; i < n; ++i) {
            const SchedRequest* r = ((Scheduler*)h)->find(ids[i]);
            if (!r) return SCHED_UNKNOWN;
            out[i] = r->num_generated();
        }
        return 0;
    } catch (...) { return SCHED_BAD_ARGUMENT; }
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
int rg_sched_next_step_predictable(void* h) { RG_GUARD(return ((Scheduler*)h)->next_step_predictable() ? 1 : 0) }
int rg_sched_num_waiting(void* h) { return ((Scheduler*)h)->num_waiting(); }
int rg_sched_num_running(void* h) { return ((Scheduler*)h)->num_running(); }

}  // extern "C"
