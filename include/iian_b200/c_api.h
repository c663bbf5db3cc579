// C interface of the host runtime (block pool, cache manager, scheduler, step packing), for bindings.
// Handles are opaque pointers.  Functions that can fail return 0 on success, 1 for a pool error (out of
// pages, double free, page given back), 2 for any other error; iian_host_last_error() then gives the text.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char * iian_host_last_error(void);
uint64_t iian_hash_block(uint64_t parent, const int32_t * tokens, int n, uint64_t salt);

// ---- block pool -------------------------------------------------------------------------------------
void * iian_pool_new(int num_blocks, int block_size, int caching);
void iian_pool_delete(void * pool);
// what: 0 num_blocks, 1 block_size, 2 caching, 3 num_free, 4 num_cached, 5 ref[b], 6 is_cached(b), 7 evictions,
// 8 cache_queries, 9 cache_hits
long long iian_pool_get(void * pool, int what, int b);
uint64_t iian_pool_hash(void * pool, int b);
int iian_pool_free_list(void * pool, int * out, int cap);                 // returns the length
int iian_pool_get_cached_block(void * pool, uint64_t h, const int32_t * tokens, int n);
int iian_pool_cache_block(void * pool, int b, uint64_t h, const int32_t * tokens, int n);
int iian_pool_reset_prefix_cache(void * pool);                            // 1 if reset
int iian_pool_touch(void * pool, int b);
int iian_pool_get_new_blocks(void * pool, int n, int * out);
int iian_pool_free_blocks(void * pool, const int * blocks, int n);
int iian_pool_check(void * pool);

// ---- cache manager ------------------------------------------------------------------------------------
void * iian_cache_new(const int * windows, const int * num_blocks, int n_groups, int block_size, int caching, int state_slots);
void iian_cache_delete(void * mgr);
void * iian_cache_pool(void * mgr, int g);                                // borrowed
int iian_cache_slots(void * mgr, int what, int arg, int * out);           // what: 0 num_slots, 1 num_free, 2 allot, 3 release(arg)
long long iian_cache_counter(void * mgr, int what, long long add);        // what: 0 prefix_queries, 1 prefix_hits; returns the new value
void * iian_rc_new(void * mgr);
void iian_rc_delete(void * rc);
// what: 0 state_slot, 1 state_fresh, 2 epoch, 3 len(tables[g]), 4 len(hashes), 5 committed[g], 6 holds_pages
int iian_rc_get(void * rc, int what, int g);
void iian_rc_set_state_fresh(void * rc, int fresh);
const int * iian_rc_table(void * rc, int g);                              // valid until the table changes
const uint64_t * iian_rc_hashes(void * rc);
int iian_cache_allot_state(void * mgr, void * rc);                        // 1 if the request has a slot now
int iian_cache_first_needed_block(void * mgr, int g, int n_computed);
int iian_cache_update_hashes(void * mgr, void * rc, const int32_t * tokens, int n, uint64_t salt);
// tables: [n_groups * cap] ints, lens: [n_groups]; returns the number of reusable tokens (-1: error)
int iian_cache_find_prefix(void * mgr, const int32_t * tokens, int n, const uint64_t * hashes, int n_hashes,
                           int * tables, int * lens, int cap);
int iian_cache_commit(void * mgr, void * rc, const int32_t * tokens, int n, int n_computed);
int iian_cache_release_passed(void * mgr, void * rc, int n_computed, int * released);
// computed tables as for iian_cache_find_prefix, or null; *ok = 1 if the pages were taken
int iian_cache_allocate(void * mgr, void * rc, int n_computed, int n_new, const int * tables, const int * lens, int cap, int * ok);
int iian_cache_free(void * mgr, void * rc);
int iian_cache_slot_of(void * mgr, void * rc, int g, int token_idx, long long * out);
double iian_cache_usage(void * mgr);
int iian_cache_check(void * mgr);

// ---- requests and scheduler ---------------------------------------------------------------------------
void * iian_req_new(long long id, const int32_t * tokens, int n, int priority, double arrival, uint64_t salt);
void iian_req_delete(void * req);
// what: 0 status, 1 num_computed_tokens, 2 num_cached_tokens, 3 num_preemptions, 4 n_tokens
int iian_req_get(void * req, int what);
void iian_req_set(void * req, int what, int value);
void iian_req_append(void * req, const int32_t * tokens, int n);
void * iian_req_cache(void * req);                                        // borrowed; null before the request is added
void iian_req_adopt_cache(void * req, void * rc);                         // the request owns rc from now on
void * iian_sched_new(void * mgr, int max_num_seqs, int max_num_batched_tokens, int long_prefill_token_threshold,
                      int enable_chunked_prefill, int priority_policy);
void iian_sched_delete(void * sched);
int iian_sched_add(void * sched, void * req);
int iian_sched_finish(void * sched, void * req, int status);
// Fills the scheduled requests (handles, new tokens, resumed flags) and the preempted ones; the output is also
// kept for iian_sched_update.  Returns 0, or an error code as above.
int iian_sched_schedule(void * sched, void ** reqs, int * n_new, int * resumed, int cap, int * n_scheduled,
                        void ** preempted, int * n_preempted, int * total_tokens);
int iian_sched_update(void * sched);                                      // after the step that ran the last schedule
int iian_sched_queue(void * sched, int which, void ** out, int cap);      // which: 0 waiting, 1 running; returns the length
long long iian_sched_num_preemptions(void * sched);

// ---- step packing ---------------------------------------------------------------------------------------
// Writes the integers of a step in which every request brings one token into `host` (the layout of
// ModelRunner's decode graphs: tokens, positions, sequence of token, cu_q, context lengths, state slots, output
// rows, per group the cells, per group the block table [S, max_blocks]).  Rows [0, n) are the requests, rows
// [n, S) padding.  sig: [n_groups * S * 3] longs kept by the caller between calls (request identity, epoch,
// pages written), from which the function knows what it may skip; pass rewrite_all = 1 after anything else
// changed the buffer.  fresh_slots receives the state slots that must be zeroed (at most n); returns their
// number, or -1 on error.
int iian_pack_decode_step(void * mgr, void ** caches, const int32_t * tokens, const int32_t * starts, int n, int S,
                          int max_blocks, int32_t * host, long long * sig, int rewrite_all, int * fresh_slots);

#ifdef __cplusplus
}
#endif
