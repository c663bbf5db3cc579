#include "iian_b200/c_api.h"

#include <cstring>
#include <string>

#include "iian_b200/scheduler.h"

using namespace iian_b200;

namespace {
thread_local std::string g_error;

template <typename F> int guarded(F && f) {
    try {
        f();
        return 0;
    } catch (const PoolError & e) {
        g_error = e.what();
        return 1;
    } catch (const std::exception & e) {
        g_error = e.what();
        return 2;
    }
}

struct SchedHandle {
    Scheduler sched;
    SchedulerOutput last;
    SchedHandle(const SchedulerConfig & c, CacheManager * m) : sched(c, m) {}
};

std::vector<std::vector<int>> unpack_tables(const int * tables, const int * lens, int n_groups, int cap) {
    std::vector<std::vector<int>> out(n_groups);
    for (int g = 0; g < n_groups; g++) out[g].assign(tables + (size_t) g * cap, tables + (size_t) g * cap + lens[g]);
    return out;
}
}  // namespace

extern "C" {

const char * iian_host_last_error(void) { return g_error.c_str(); }
uint64_t iian_hash_block(uint64_t parent, const int32_t * tokens, int n, uint64_t salt) { return hash_block(parent, tokens, n, salt); }

// ---- block pool -------------------------------------------------------------------------------------
void * iian_pool_new(int num_blocks, int block_size, int caching) {
    BlockPool * p = nullptr;
    guarded([&] { p = new BlockPool(num_blocks, block_size, caching != 0); });
    return p;
}
void iian_pool_delete(void * pool) { delete static_cast<BlockPool *>(pool); }
long long iian_pool_get(void * pool, int what, int b) {
    auto * p = static_cast<BlockPool *>(pool);
    switch (what) {
        case 0: return p->num_blocks();
        case 1: return p->block_size();
        case 2: return p->caching();
        case 3: return p->num_free();
        case 4: return p->num_cached();
        case 5: return b >= 0 && b < p->num_blocks() ? p->ref(b) : -1;
        case 6: return b >= 0 && b < p->num_blocks() ? p->is_cached(b) : 0;
        case 7: return p->evictions;
        case 8: return p->cache_queries;
        case 9: return p->cache_hits;
    }
    return -1;
}
uint64_t iian_pool_hash(void * pool, int b) { return static_cast<BlockPool *>(pool)->hash(b); }
int iian_pool_free_list(void * pool, int * out, int cap) {
    const auto list = static_cast<BlockPool *>(pool)->free_list();
    for (size_t i = 0; i < list.size() && (int) i < cap; i++) out[i] = list[i];
    return (int) list.size();
}
int iian_pool_get_cached_block(void * pool, uint64_t h, const int32_t * tokens, int n) {
    return static_cast<BlockPool *>(pool)->get_cached_block(h, tokens, n);
}
int iian_pool_cache_block(void * pool, int b, uint64_t h, const int32_t * tokens, int n) {
    return guarded([&] { static_cast<BlockPool *>(pool)->cache_block(b, h, tokens, n); });
}
int iian_pool_reset_prefix_cache(void * pool) { return static_cast<BlockPool *>(pool)->reset_prefix_cache() ? 1 : 0; }
int iian_pool_touch(void * pool, int b) { return guarded([&] { static_cast<BlockPool *>(pool)->touch(b); }); }
int iian_pool_get_new_blocks(void * pool, int n, int * out) {
    return guarded([&] {
        std::vector<int> v;
        static_cast<BlockPool *>(pool)->get_new_blocks(n, v);
        std::memcpy(out, v.data(), sizeof(int) * v.size());
    });
}
int iian_pool_free_blocks(void * pool, const int * blocks, int n) {
    return guarded([&] { static_cast<BlockPool *>(pool)->free_blocks(blocks, n); });
}
int iian_pool_check(void * pool) { return guarded([&] { static_cast<BlockPool *>(pool)->check_invariants(); }); }

// ---- cache manager ------------------------------------------------------------------------------------
void * iian_cache_new(const int * windows, const int * num_blocks, int n_groups, int block_size, int caching, int state_slots) {
    CacheManager * m = nullptr;
    guarded([&] {
        std::vector<PageGroup> groups;
        for (int g = 0; g < n_groups; g++) groups.push_back({windows[g], num_blocks[g]});
        m = new CacheManager(groups, block_size, caching != 0, state_slots);
    });
    return m;
}
void iian_cache_delete(void * mgr) { delete static_cast<CacheManager *>(mgr); }
void * iian_cache_pool(void * mgr, int g) { return &static_cast<CacheManager *>(mgr)->pool(g); }
int iian_cache_slots(void * mgr, int what, int arg, int * out) {
    auto & s = static_cast<CacheManager *>(mgr)->slots();
    return guarded([&] {
        switch (what) {
            case 0: *out = s.num_slots(); break;
            case 1: *out = s.num_free(); break;
            case 2: *out = s.allot(); break;
            case 3: s.release(arg); *out = 0; break;
            default: throw std::invalid_argument("iian_cache_slots: unknown request");
        }
    });
}
long long iian_cache_counter(void * mgr, int what, long long add) {
    auto * m = static_cast<CacheManager *>(mgr);
    long long & c = what == 0 ? m->prefix_queries : m->prefix_hits;
    c += add;
    return c;
}
void * iian_rc_new(void * mgr) { return static_cast<CacheManager *>(mgr)->new_request(); }
void iian_rc_delete(void * rc) { delete static_cast<RequestCache *>(rc); }
int iian_rc_get(void * rc, int what, int g) {
    auto * r = static_cast<RequestCache *>(rc);
    switch (what) {
        case 0: return r->state_slot;
        case 1: return r->state_fresh;
        case 2: return r->epoch;
        case 3: return g >= 0 && g < (int) r->tables.size() ? (int) r->tables[g].size() : -1;
        case 4: return (int) r->hashes.size();
        case 5: return g >= 0 && g < (int) r->committed.size() ? r->committed[g] : -1;
        case 6: return r->holds_pages();
        case 7: return (int) r->tables.size();
    }
    return -1;
}
void iian_rc_set_state_fresh(void * rc, int fresh) { static_cast<RequestCache *>(rc)->state_fresh = fresh != 0; }
const int * iian_rc_table(void * rc, int g) { return static_cast<RequestCache *>(rc)->tables[g].data(); }
const uint64_t * iian_rc_hashes(void * rc) { return static_cast<RequestCache *>(rc)->hashes.data(); }
int iian_cache_allot_state(void * mgr, void * rc) {
    return static_cast<CacheManager *>(mgr)->allot_state(*static_cast<RequestCache *>(rc)) ? 1 : 0;
}
int iian_cache_first_needed_block(void * mgr, int g, int n_computed) {
    return static_cast<CacheManager *>(mgr)->first_needed_block(g, n_computed);
}
int iian_cache_update_hashes(void * mgr, void * rc, const int32_t * tokens, int n, uint64_t salt) {
    return guarded([&] { static_cast<CacheManager *>(mgr)->update_hashes(static_cast<RequestCache *>(rc)->hashes, tokens, n, salt); });
}
int iian_cache_find_prefix(void * mgr, const int32_t * tokens, int n, const uint64_t * hashes, int n_hashes,
                           int * tables, int * lens, int cap) {
    int found = -1;
    auto * m = static_cast<CacheManager *>(mgr);
    const int rc = guarded([&] {
        std::vector<std::vector<int>> t;
        found = m->find_cached_prefix(tokens, n, hashes, n_hashes, t);
        for (int g = 0; g < m->num_groups(); g++) {
            if ((int) t[g].size() > cap) throw std::invalid_argument("iian_cache_find_prefix: table buffer too small");
            lens[g] = (int) t[g].size();
            std::memcpy(tables + (size_t) g * cap, t[g].data(), sizeof(int) * t[g].size());
        }
    });
    return rc == 0 ? found : -1;
}
int iian_cache_commit(void * mgr, void * rc, const int32_t * tokens, int n, int n_computed) {
    return guarded([&] { static_cast<CacheManager *>(mgr)->commit(*static_cast<RequestCache *>(rc), tokens, n, n_computed); });
}
int iian_cache_release_passed(void * mgr, void * rc, int n_computed, int * released) {
    return guarded([&] { *released = static_cast<CacheManager *>(mgr)->release_passed(*static_cast<RequestCache *>(rc), n_computed); });
}
int iian_cache_allocate(void * mgr, void * rc, int n_computed, int n_new, const int * tables, const int * lens, int cap, int * ok) {
    auto * m = static_cast<CacheManager *>(mgr);
    return guarded([&] {
        if (tables != nullptr) {
            const auto computed = unpack_tables(tables, lens, m->num_groups(), cap);
            *ok = m->allocate(*static_cast<RequestCache *>(rc), n_computed, n_new, &computed) ? 1 : 0;
        } else {
            *ok = m->allocate(*static_cast<RequestCache *>(rc), n_computed, n_new, nullptr) ? 1 : 0;
        }
    });
}
int iian_cache_free(void * mgr, void * rc) {
    return guarded([&] { static_cast<CacheManager *>(mgr)->free(*static_cast<RequestCache *>(rc)); });
}
int iian_cache_slot_of(void * mgr, void * rc, int g, int token_idx, long long * out) {
    return guarded([&] { *out = static_cast<CacheManager *>(mgr)->slot_of(*static_cast<RequestCache *>(rc), g, token_idx); });
}
double iian_cache_usage(void * mgr) { return static_cast<CacheManager *>(mgr)->usage(); }
int iian_cache_check(void * mgr) { return guarded([&] { static_cast<CacheManager *>(mgr)->check_invariants(); }); }

// ---- requests and scheduler ---------------------------------------------------------------------------
void * iian_req_new(long long id, const int32_t * tokens, int n, int priority, double arrival, uint64_t salt) {
    auto * r = new SchedRequest();
    r->id = id;
    r->tokens.assign(tokens, tokens + n);
    r->priority = priority;
    r->arrival = arrival;
    r->cache_salt = salt;
    return r;
}
void iian_req_delete(void * req) { delete static_cast<SchedRequest *>(req); }
int iian_req_get(void * req, int what) {
    auto * r = static_cast<SchedRequest *>(req);
    switch (what) {
        case 0: return r->status;
        case 1: return r->num_computed_tokens;
        case 2: return r->num_cached_tokens;
        case 3: return r->num_preemptions;
        case 4: return r->n_tokens();
    }
    return -1;
}
void iian_req_set(void * req, int what, int value) {
    auto * r = static_cast<SchedRequest *>(req);
    switch (what) {
        case 0: r->status = value; break;
        case 1: r->num_computed_tokens = value; break;
        case 2: r->num_cached_tokens = value; break;
        case 3: r->num_preemptions = value; break;
    }
}
void iian_req_append(void * req, const int32_t * tokens, int n) {
    auto * r = static_cast<SchedRequest *>(req);
    r->tokens.insert(r->tokens.end(), tokens, tokens + n);
}
void * iian_req_cache(void * req) { return static_cast<SchedRequest *>(req)->cache.get(); }
void iian_req_adopt_cache(void * req, void * rc) { static_cast<SchedRequest *>(req)->cache.reset(static_cast<RequestCache *>(rc)); }

void * iian_sched_new(void * mgr, int max_num_seqs, int max_num_batched_tokens, int long_prefill_token_threshold,
                      int enable_chunked_prefill, int priority_policy) {
    SchedHandle * h = nullptr;
    guarded([&] {
        SchedulerConfig c;
        c.max_num_seqs = max_num_seqs;
        c.max_num_batched_tokens = max_num_batched_tokens;
        c.long_prefill_token_threshold = long_prefill_token_threshold;
        c.enable_chunked_prefill = enable_chunked_prefill != 0;
        c.priority_policy = priority_policy != 0;
        h = new SchedHandle(c, static_cast<CacheManager *>(mgr));
    });
    return h;
}
void iian_sched_delete(void * sched) { delete static_cast<SchedHandle *>(sched); }
int iian_sched_add(void * sched, void * req) {
    return guarded([&] { static_cast<SchedHandle *>(sched)->sched.add_request(static_cast<SchedRequest *>(req)); });
}
int iian_sched_finish(void * sched, void * req, int status) {
    return guarded([&] { static_cast<SchedHandle *>(sched)->sched.finish_request(static_cast<SchedRequest *>(req), status); });
}
int iian_sched_schedule(void * sched, void ** reqs, int * n_new, int * resumed, int cap, int * n_scheduled,
                        void ** preempted, int * n_preempted, int * total_tokens) {
    auto * h = static_cast<SchedHandle *>(sched);
    return guarded([&] {
        h->last = h->sched.schedule();
        const auto & out = h->last;
        if ((int) out.scheduled.size() > cap || (int) out.preempted.size() > cap)
            throw std::invalid_argument("iian_sched_schedule: output buffers too small");
        for (size_t i = 0; i < out.scheduled.size(); i++) {
            reqs[i] = out.scheduled[i].req;
            n_new[i] = out.scheduled[i].n_new_tokens;
            resumed[i] = out.scheduled[i].resumed;
        }
        for (size_t i = 0; i < out.preempted.size(); i++) preempted[i] = out.preempted[i];
        *n_scheduled = (int) out.scheduled.size();
        *n_preempted = (int) out.preempted.size();
        *total_tokens = out.total_tokens;
    });
}
int iian_sched_update(void * sched) {
    auto * h = static_cast<SchedHandle *>(sched);
    return guarded([&] { h->sched.update_after_step(h->last); });
}
int iian_sched_queue(void * sched, int which, void ** out, int cap) {
    auto & s = static_cast<SchedHandle *>(sched)->sched;
    int n = 0;
    if (which == 0) {
        for (auto * r : s.waiting()) {
            if (n < cap) out[n] = r;
            n++;
        }
    } else {
        for (auto * r : s.running()) {
            if (n < cap) out[n] = r;
            n++;
        }
    }
    return n;
}
long long iian_sched_num_preemptions(void * sched) { return static_cast<SchedHandle *>(sched)->sched.num_preemptions; }

// ---- step packing ---------------------------------------------------------------------------------------
int iian_pack_decode_step(void * mgr, void ** caches, const int32_t * tokens, const int32_t * starts, int n, int S,
                          int max_blocks, int32_t * host, long long * sig, int rewrite_all, int * fresh_slots) {
    auto * m = static_cast<CacheManager *>(mgr);
    int n_fresh = 0;
    const int rc = guarded([&] {
        const int G = m->num_groups(), bs = m->block_size();
        if (n > S) throw std::invalid_argument("iian_pack_decode_step: more requests than rows");
        int32_t * tok = host, * pos = tok + S, * seq = pos + S, * cu = seq + S, * ctx = cu + S + 1, * state = ctx + S,
                * rows = state + S, * cells = rows + S, * bt = cells + (size_t) G * S;
        if (rewrite_all) {              // the padding: sequences of one token that is stored nowhere
            for (int s = 0; s < S; s++) {
                tok[s] = 0; pos[s] = 0; seq[s] = -1; cu[s] = s; ctx[s] = 1; state[s] = -1; rows[s] = s;
            }
            cu[S] = S;
            for (size_t i = 0; i < (size_t) G * S; i++) cells[i] = -1;
            for (size_t i = 0; i < (size_t) G * S * max_blocks; i++) bt[i] = 0;
            for (size_t i = 0; i < (size_t) G * S * 3; i++) sig[i] = 0;
        }
        for (int s = 0; s < n; s++) {
            auto * rc = static_cast<RequestCache *>(caches[s]);
            const int start = starts[s];
            tok[s] = tokens[s];
            pos[s] = start;
            seq[s] = s;
            ctx[s] = start + 1;
            state[s] = rc->state_slot;
            if (rc->state_fresh) {
                fresh_slots[n_fresh++] = rc->state_slot;
                rc->state_fresh = false;
            }
            const int need = start / bs + 1;
            if (need > max_blocks) throw std::invalid_argument("iian_pack_decode_step: the context is longer than the graph's block table");
            for (int g = 0; g < G; g++) {
                const auto & table = rc->tables[g];
                if ((int) table.size() < need)
                    throw std::invalid_argument("request holds " + std::to_string(table.size()) + " pages in group " +
                                                std::to_string(g) + ", needs " + std::to_string(need));
                int32_t * row = bt + ((size_t) g * S + s) * max_blocks;
                long long * sg = sig + ((size_t) g * S + s) * 3;
                const long long who = rc->serial;                         // 0 marks a row nobody wrote
                if (sg[0] != who || sg[1] != rc->epoch || sg[2] > need) {
                    for (int i = 0; i < max_blocks; i++) row[i] = -1;
                    for (int i = 0; i < need; i++) row[i] = table[i];
                } else {
                    for (int i = (int) sg[2]; i < need; i++) row[i] = table[i];
                }
                sg[0] = who; sg[1] = rc->epoch; sg[2] = need;
                const int page = table[need - 1];
                if (page < 0) throw PoolError("a token of this step lies in a page that was given back");
                cells[(size_t) g * S + s] = page * bs + start % bs;
            }
        }
    });
    return rc == 0 ? n_fresh : -1;
}

}  // extern "C"
