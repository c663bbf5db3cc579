// The cache manager: pages per group of layers, a block table per request and group, prefix reuse, and
// slots for per-request state of fixed size.
//
// The reference has one group (every layer shares one block table, src/iian/kv_cache.cpp:156-169) and no
// fixed-size state; its per-request record is KVRequestState (include/iian/kv_cache.h:93-97) and its
// operations are get_computed_blocks (kv_cache.cpp:199-212), allocate_slots (:214-229, all or nothing),
// cache_blocks (:231-238), free in reverse order (:240-246) and update_hashes (:190-197).  Those semantics
// are kept per group.  New here:
//  * several groups, each with a pool of its own; a group with a window needs only the last `window` keys,
//    so pages the window has passed are given back while the request is still running;
//  * a prefix hit must be usable by every group: all leading pages for a group that needs all keys, the
//    pages inside the window for a windowed one;
//  * StateSlots: one fixed-size slot per running request for mixers that keep a summary instead of
//    per-token entries.
// Everything here is host bookkeeping on page numbers.
#pragma once
#include <memory>
#include <vector>

#include "iian_b200/block_pool.h"

namespace iian_b200 {

struct PageGroup {
    int window;          // -1: every key stays; n: a query sees itself and the n - 1 keys before it
    int num_blocks;
};

// What one request holds.
struct RequestCache {
    std::vector<std::vector<int>> tables;     // per group: page of logical block i, -1 = not held
    std::vector<uint64_t> hashes;             // chained hashes of the full pages of its tokens
    std::vector<int> committed;               // per group: leading blocks offered to the prefix index
    int state_slot = -1;
    bool state_fresh = false;                 // the slot was just allotted and must start from zero
    int epoch = 0;                            // bumped whenever a table changes other than by growing
    long long serial = 0;                     // unique per object for the life of the process (an address may come back)
    bool holds_pages() const;
};

class StateSlots {
public:
    explicit StateSlots(int num_slots);
    int num_slots() const { return num_slots_; }
    int num_free() const { return (int) free_.size(); }
    int allot();                              // -1: none free
    void release(int slot);                   // throws PoolError if the slot is not held
private:
    int num_slots_;
    std::vector<int> free_;
    std::vector<char> held_;
};

class CacheManager {
public:
    CacheManager(const std::vector<PageGroup> & groups, int block_size, bool enable_prefix_caching, int num_state_slots);

    int num_groups() const { return (int) groups_.size(); }
    int block_size() const { return block_size_; }
    bool prefix_caching() const { return prefix_caching_; }
    const PageGroup & group(int g) const { return groups_[g]; }
    BlockPool & pool(int g) { return *pools_[g]; }
    StateSlots & slots() { return slots_; }

    RequestCache * new_request() const;       // the caller owns it
    bool allot_state(RequestCache & rc);      // false if no slot is free (a request that has one keeps it)

    int first_needed_block(int g, int n_computed) const;
    int blocks_for(int n_tokens) const { return (n_tokens + block_size_ - 1) / block_size_; }

    void update_hashes(std::vector<uint64_t> & hashes, const int32_t * tokens, int n_tokens, uint64_t salt) const;
    // Longest reusable prefix in tokens (a multiple of the page size, at most n_tokens - 1 so that the last
    // token is always computed for its logits) and per group the table to start from.  Nothing is referenced.
    int find_cached_prefix(const int32_t * tokens, int n_tokens, const uint64_t * hashes, int n_hashes,
                           std::vector<std::vector<int>> & tables);
    void commit(RequestCache & rc, const int32_t * tokens, int n_tokens, int n_computed);
    int release_passed(RequestCache & rc, int n_computed);
    // Make sure the request holds pages for tokens [0, n_computed + n_new) in every group.  Either every group
    // gets what it needs or nothing is taken and false is returned.
    bool allocate(RequestCache & rc, int n_computed, int n_new, const std::vector<std::vector<int>> * computed);
    void free(RequestCache & rc);
    long long slot_of(const RequestCache & rc, int g, int token_idx) const;
    double usage() const;
    void check_invariants() const;

    long long prefix_queries = 0, prefix_hits = 0;

private:
    std::vector<PageGroup> groups_;
    int block_size_;
    bool prefix_caching_;
    std::vector<std::unique_ptr<BlockPool>> pools_;
    StateSlots slots_;
};

}  // namespace iian_b200
