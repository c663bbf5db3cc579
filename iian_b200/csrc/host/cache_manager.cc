#include "iian_b200/cache_manager.h"

#include <algorithm>
#include <atomic>

namespace iian_b200 {

// Serial numbers of request records: unique for the life of the process, also when this source is part of more than
// one loaded library (each copy then counts in a range of its own, set apart by where the copy was loaded).
static std::atomic<long long> g_next_serial{0};
static long long next_serial() {
    const long long base = (long long) ((reinterpret_cast<uintptr_t>(&g_next_serial) >> 4) & 0x3FFFFFF) << 36;
    return base + 1 + g_next_serial++;
}

bool RequestCache::holds_pages() const {
    for (const auto & t : tables)
        for (int p : t)
            if (p >= 0) return true;
    return false;
}

StateSlots::StateSlots(int num_slots) : num_slots_(num_slots), held_(num_slots, 0) {
    for (int s = num_slots - 1; s >= 0; s--) free_.push_back(s);
}

int StateSlots::allot() {
    if (free_.empty()) return -1;
    const int s = free_.back();
    free_.pop_back();
    held_[s] = 1;
    return s;
}

void StateSlots::release(int slot) {
    if (slot < 0) return;
    if (slot >= num_slots_ || !held_[slot]) throw PoolError("StateSlots: slot " + std::to_string(slot) + " released twice");
    held_[slot] = 0;
    free_.push_back(slot);
}

CacheManager::CacheManager(const std::vector<PageGroup> & groups, int block_size, bool enable_prefix_caching, int num_state_slots)
    : groups_(groups), block_size_(block_size), prefix_caching_(enable_prefix_caching), slots_(num_state_slots) {
    if (block_size < 1) throw std::invalid_argument("block_size must be >= 1");
    for (const auto & g : groups_) pools_.emplace_back(new BlockPool(g.num_blocks, block_size, enable_prefix_caching));
}

RequestCache * CacheManager::new_request() const {
    auto * rc = new RequestCache();
    rc->serial = next_serial();
    rc->tables.resize(groups_.size());
    rc->committed.assign(groups_.size(), 0);
    return rc;
}

bool CacheManager::allot_state(RequestCache & rc) {
    if (rc.state_slot >= 0 || slots_.num_slots() == 0) return true;
    const int s = slots_.allot();
    if (s < 0) return false;
    rc.state_slot = s;
    rc.state_fresh = true;
    return true;
}

int CacheManager::first_needed_block(int g, int n_computed) const {
    const int w = groups_[g].window;
    if (w < 0) return 0;
    return std::max(0, n_computed - w + 1) / block_size_;
}

void CacheManager::update_hashes(std::vector<uint64_t> & hashes, const int32_t * tokens, int n_tokens, uint64_t salt) const {
    const int n_full = n_tokens / block_size_;
    while ((int) hashes.size() < n_full) {
        const size_t i = hashes.size();
        const uint64_t parent = i == 0 ? kHashNone : hashes[i - 1];
        hashes.push_back(hash_block(parent, tokens + i * block_size_, block_size_, salt));
    }
}

int CacheManager::find_cached_prefix(const int32_t * tokens, int n_tokens, const uint64_t * hashes, int n_hashes,
                                     std::vector<std::vector<int>> & tables) {
    const int G = num_groups();
    tables.assign(G, {});
    if (!prefix_caching_ || n_tokens < 2 || G == 0) return 0;      // without page groups there is nothing to share
    const int bs = block_size_;
    const int max_blocks = std::min((n_tokens - 1) / bs, n_hashes);
    std::vector<std::vector<int>> found(G);
    for (int g = 0; g < G; g++)
        for (int i = 0; i < max_blocks; i++) found[g].push_back(pools_[g]->get_cached_block(hashes[i], tokens + (size_t) i * bs, bs));
    int n = max_blocks;
    for (int g = 0; g < G; g++)
        if (groups_[g].window < 0) {
            int k = 0;
            while (k < n && found[g][k] >= 0) k++;
            n = k;
        }
    while (n > 0) {
        bool ok = true;
        for (int g = 0; g < G && ok; g++) {
            if (groups_[g].window < 0) continue;
            for (int i = first_needed_block(g, n * bs); i < n; i++)
                if (found[g][i] < 0) { ok = false; break; }
        }
        if (ok) break;
        n--;
    }
    if (n == 0) return 0;
    for (int g = 0; g < G; g++) {
        const int first = first_needed_block(g, n * bs);
        tables[g].assign(first, -1);
        for (int i = first; i < n; i++) tables[g].push_back(found[g][i]);
    }
    return n * bs;
}

void CacheManager::commit(RequestCache & rc, const int32_t * tokens, int n_tokens, int n_computed) {
    if (!prefix_caching_) return;
    const int bs = block_size_;
    const int n_full = std::min(std::min(n_computed, n_tokens) / bs, (int) rc.hashes.size());
    for (int g = 0; g < num_groups(); g++) {
        const auto & table = rc.tables[g];
        const int upto = std::min(n_full, (int) table.size());
        for (int i = rc.committed[g]; i < upto; i++)
            if (table[i] >= 0) pools_[g]->cache_block(table[i], rc.hashes[i], tokens + (size_t) i * bs, bs);
        rc.committed[g] = std::max(rc.committed[g], upto);
    }
}

int CacheManager::release_passed(RequestCache & rc, int n_computed) {
    int released = 0;
    for (int g = 0; g < num_groups(); g++) {
        if (groups_[g].window < 0) continue;
        auto & table = rc.tables[g];
        const int first = std::min(first_needed_block(g, n_computed), (int) table.size());
        std::vector<int> gone;
        for (int i = first - 1; i >= 0; i--)
            if (table[i] >= 0) gone.push_back(table[i]);          // in reverse order, like a free
        if (!gone.empty()) {
            pools_[g]->free_blocks(gone.data(), (int) gone.size());
            for (int i = 0; i < first; i++) table[i] = -1;
            released += (int) gone.size();
        }
    }
    if (released) rc.epoch++;
    return released;
}

bool CacheManager::allocate(RequestCache & rc, int n_computed, int n_new, const std::vector<std::vector<int>> * computed) {
    release_passed(rc, n_computed);
    const int need_total = blocks_for(n_computed + n_new);
    const int G = num_groups();
    std::vector<char> use(G, 0);
    std::vector<int> fresh(G, 0);
    for (int g = 0; g < G; g++) {
        const auto & table = rc.tables[g];
        const bool use_computed = computed != nullptr && table.empty() && !(*computed)[g].empty();
        const int have = use_computed ? (int) (*computed)[g].size() : (int) table.size();
        const int n_fresh = std::max(0, need_total - have);
        int n_touch_free = 0;
        if (use_computed)
            for (int p : (*computed)[g])
                if (p >= 0 && pools_[g]->ref(p) == 0) n_touch_free++;
        if (n_fresh + n_touch_free > pools_[g]->num_free()) return false;
        use[g] = use_computed;
        fresh[g] = n_fresh;
    }
    for (int g = 0; g < G; g++) {
        auto & table = rc.tables[g];
        if (use[g]) {
            for (int p : (*computed)[g]) {
                if (p >= 0) pools_[g]->touch(p);
                table.push_back(p);
            }
            rc.committed[g] = (int) table.size();
        }
        if (fresh[g]) pools_[g]->get_new_blocks(fresh[g], table);
    }
    return true;
}

void CacheManager::free(RequestCache & rc) {
    for (int g = 0; g < num_groups(); g++) {
        auto & table = rc.tables[g];
        std::vector<int> held;
        for (auto it = table.rbegin(); it != table.rend(); ++it)
            if (*it >= 0) held.push_back(*it);
        if (!held.empty()) pools_[g]->free_blocks(held.data(), (int) held.size());
        table.clear();
        rc.committed[g] = 0;
    }
    rc.epoch++;
    if (rc.state_slot >= 0) {
        slots_.release(rc.state_slot);
        rc.state_slot = -1;
        rc.state_fresh = false;
    }
}

long long CacheManager::slot_of(const RequestCache & rc, int g, int token_idx) const {
    const int page = rc.tables[g].at(token_idx / block_size_);
    if (page < 0) throw PoolError("token " + std::to_string(token_idx) + " lies in a page that was given back");
    return (long long) page * block_size_ + token_idx % block_size_;
}

double CacheManager::usage() const {
    double u = 0.0;
    for (const auto & p : pools_) u = std::max(u, p->usage());
    return u;
}

void CacheManager::check_invariants() const {
    for (const auto & p : pools_) p->check_invariants();
}

}  // namespace iian_b200
