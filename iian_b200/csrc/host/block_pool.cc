#include "iian_b200/block_pool.h"

#include <algorithm>
#include <cstring>
#include <set>

namespace iian_b200 {

static inline uint64_t mix64(uint64_t h) {
    h ^= h >> 33;
    h *= 0xFF51AFD7ED558CCDull;
    h ^= h >> 33;
    h *= 0xC4CEB9FE1A85EC53ull;
    h ^= h >> 33;
    return h;
}

uint64_t hash_block(uint64_t parent, const int32_t * tokens, int n, uint64_t salt) {
    uint64_t h = mix64(parent ^ 0x9E3779B97F4A7C15ull) ^ mix64(salt + 0x2545F4914F6CDD1Dull);
    for (int i = 0; i < n; i++) {
        const uint64_t t = (uint64_t) (uint32_t) tokens[i];
        h = mix64(h ^ (t + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2)));
    }
    return h != kHashNone ? h : 1;
}

BlockPool::BlockPool(int num_blocks, int block_size, bool enable_caching)
    : num_blocks_(num_blocks), block_size_(block_size), caching_(enable_caching) {
    if (num_blocks < 1 || block_size < 1) throw std::invalid_argument("BlockPool needs at least one block of at least one token");
    ref_.assign(num_blocks, 0);
    prev_.assign(num_blocks, -1);
    next_.assign(num_blocks, -1);
    in_free_.assign(num_blocks, 0);
    hash_.assign(num_blocks, kHashNone);
    tokens_.assign((size_t) num_blocks * block_size, 0);
    for (int b = 0; b < num_blocks; b++) push_back(b);
}

void BlockPool::remove(int b) {
    if (!in_free_[b]) return;
    const int p = prev_[b], n = next_[b];
    if (p >= 0) next_[p] = n; else head_ = n;
    if (n >= 0) prev_[n] = p; else tail_ = p;
    prev_[b] = next_[b] = -1;
    in_free_[b] = 0;
    num_free_--;
}

void BlockPool::push_front(int b) {
    prev_[b] = -1;
    next_[b] = head_;
    if (head_ >= 0) prev_[head_] = b; else tail_ = b;
    head_ = b;
    in_free_[b] = 1;
    num_free_++;
}

void BlockPool::push_back(int b) {
    next_[b] = -1;
    prev_[b] = tail_;
    if (tail_ >= 0) next_[tail_] = b; else head_ = b;
    tail_ = b;
    in_free_[b] = 1;
    num_free_++;
}

std::vector<int> BlockPool::free_list() const {
    std::vector<int> out;
    for (int b = head_; b >= 0; b = next_[b]) out.push_back(b);
    return out;
}

void BlockPool::evict_hash(int b) {
    const uint64_t h = hash_[b];
    if (h == kHashNone) return;
    auto it = index_.find(h);
    if (it != index_.end()) {
        auto & pages = it->second;
        auto at = std::find(pages.begin(), pages.end(), b);
        if (at != pages.end()) {
            pages.erase(at);
            num_cached_--;
        }
        if (pages.empty()) index_.erase(it);
    }
    hash_[b] = kHashNone;
    evictions++;
}

int BlockPool::get_cached_block(uint64_t h, const int32_t * tokens, int n) const {
    if (!caching_ || n != block_size_) return -1;
    auto it = index_.find(h);
    if (it == index_.end()) return -1;
    for (int b : it->second)
        if (std::memcmp(&tokens_[(size_t) b * block_size_], tokens, sizeof(int32_t) * n) == 0) return b;
    return -1;
}

void BlockPool::cache_block(int b, uint64_t h, const int32_t * tokens, int n) {
    if (!caching_ || hash_[b] != kHashNone || n != block_size_) return;
    hash_[b] = h;
    std::memcpy(&tokens_[(size_t) b * block_size_], tokens, sizeof(int32_t) * n);
    index_[h].push_back(b);
    num_cached_++;
}

bool BlockPool::reset_prefix_cache() {
    if (num_free_ != num_blocks_) return false;
    std::fill(hash_.begin(), hash_.end(), kHashNone);
    index_.clear();
    num_cached_ = 0;
    return true;
}

void BlockPool::touch(int b) {
    if (ref_[b] == 0) remove(b);
    ref_[b]++;
}

void BlockPool::get_new_blocks(int n, std::vector<int> & out) {
    if (n > num_free_)
        throw PoolError("BlockPool: out of blocks (asked " + std::to_string(n) + ", free " + std::to_string(num_free_) + ")");
    for (int i = 0; i < n; i++) {
        const int b = head_;
        remove(b);
        if (hash_[b] != kHashNone) evict_hash(b);
        ref_[b] = 1;
        out.push_back(b);
    }
}

void BlockPool::free_blocks(const int * blocks, int n) {
    std::vector<int> uncached, cached;
    for (int i = 0; i < n; i++) {
        const int b = blocks[i];
        if (b < 0 || b >= num_blocks_ || ref_[b] <= 0) throw PoolError("BlockPool: double free of block " + std::to_string(b));
        if (--ref_[b] == 0) {
            if (hash_[b] == kHashNone || !caching_) uncached.push_back(b);
            else cached.push_back(b);
        }
    }
    for (auto it = uncached.rbegin(); it != uncached.rend(); ++it) push_front(*it);
    for (int b : cached) push_back(b);
}

void BlockPool::check_invariants() const {
    const std::vector<int> on_list = free_list();
    const std::set<int> free_set(on_list.begin(), on_list.end());
    if (free_set.size() != on_list.size()) throw std::logic_error("a page is on the free list twice");
    if ((int) on_list.size() != num_free_)
        throw std::logic_error("free list holds " + std::to_string(on_list.size()) + " pages, counter says " + std::to_string(num_free_));
    for (int b = 0; b < num_blocks_; b++) {
        if (ref_[b] < 0) throw std::logic_error("page " + std::to_string(b) + " has a negative reference count");
        if ((ref_[b] == 0) != (free_set.count(b) > 0))
            throw std::logic_error("page " + std::to_string(b) + ": ref " + std::to_string(ref_[b]) + ", on free list " +
                                   std::to_string((int) free_set.count(b)));
    }
}

}  // namespace iian_b200
