// A pool of fixed-size cache pages with reference counts, a free list and a prefix index.
//
// Behaviour follows the reference's BlockPool (include/iian/kv_cache.h:40-90, src/iian/kv_cache.cpp:34-132):
//  * new pages come from the head of the free list; a page that still carries a prefix hash loses it at
//    that moment, not when it is freed (kv_cache.cpp:93-102);
//  * a freed page without a hash goes to the head (used again first), one with a hash to the tail (kept
//    for prefix reuse, least recently used evicted first) (kv_cache.cpp:104-116);
//  * a prefix hit must match the stored token ids, not just the hash (kv_cache.cpp:77-85);
//  * taking more pages than are free, or freeing a page twice, is an error (kv_cache.cpp:94, :108).
// No device memory is touched here; pages are numbers.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace iian_b200 {

constexpr uint64_t kHashNone = 0;

struct PoolError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// Chained 64-bit hash of one full page of token ids (role of kv_cache.cpp:24-29; the mixing function is
// this engine's own, hits are verified against the stored ids anyway).  Never returns kHashNone.
uint64_t hash_block(uint64_t parent, const int32_t * tokens, int n, uint64_t salt);

class BlockPool {
public:
    BlockPool(int num_blocks, int block_size, bool enable_caching);

    int num_blocks() const { return num_blocks_; }
    int block_size() const { return block_size_; }
    bool caching() const { return caching_; }
    int num_free() const { return num_free_; }
    int num_cached() const { return num_cached_; }
    int ref(int b) const { return ref_[b]; }
    uint64_t hash(int b) const { return hash_[b]; }
    bool is_cached(int b) const { return hash_[b] != kHashNone; }
    double usage() const { return 1.0 - (double) num_free_ / num_blocks_; }
    std::vector<int> free_list() const;

    int get_cached_block(uint64_t h, const int32_t * tokens, int n) const;     // -1: no page holds these tokens
    void cache_block(int b, uint64_t h, const int32_t * tokens, int n);
    bool reset_prefix_cache();                                                 // only when nothing is held

    void touch(int b);                       // take a reference; a free page leaves the free list
    void get_new_blocks(int n, std::vector<int> & out);
    void free_blocks(const int * blocks, int n);
    void check_invariants() const;           // throws std::logic_error naming the broken invariant

    long long cache_queries = 0, cache_hits = 0, evictions = 0;

private:
    void remove(int b);
    void push_front(int b);
    void push_back(int b);
    void evict_hash(int b);

    int num_blocks_, block_size_;
    bool caching_;
    std::vector<int> ref_, prev_, next_;
    std::vector<char> in_free_;
    std::vector<uint64_t> hash_;
    std::vector<int32_t> tokens_;            // [num_blocks * block_size], valid where hash_ is set
    std::unordered_map<uint64_t, std::vector<int>> index_;     // hash -> pages carrying it, in the order they registered
    int head_ = -1, tail_ = -1, num_free_ = 0, num_cached_ = 0;
};

}  // namespace iian_b200
