#include "iian_b200/scheduler.h"

#include <algorithm>

namespace iian_b200 {

Scheduler::Scheduler(const SchedulerConfig & cfg, CacheManager * cache) : cfg_(cfg), cache_(cache) {
    if (cfg.max_num_seqs < 1 || cfg.max_num_batched_tokens < 1) throw std::invalid_argument("scheduler limits must be positive");
}

void Scheduler::enqueue(SchedRequest * req) {
    if (!cfg_.priority_policy) {
        waiting_.push_back(req);
        return;
    }
    auto pos = std::upper_bound(waiting_.begin(), waiting_.end(), req, [](const SchedRequest * a, const SchedRequest * b) {
        return a->priority != b->priority ? a->priority < b->priority : a->arrival < b->arrival;
    });
    waiting_.insert(pos, req);
}

void Scheduler::add_request(SchedRequest * req) {
    req->status = WAITING;
    if (!req->cache) req->cache.reset(cache_->new_request());
    enqueue(req);
}

void Scheduler::finish_request(SchedRequest * req, int status) {
    req->status = status;
    if (req->cache) cache_->free(*req->cache);
    auto r = std::find(running_.begin(), running_.end(), req);
    if (r != running_.end()) {
        running_.erase(r);
        return;
    }
    auto w = std::find(waiting_.begin(), waiting_.end(), req);
    if (w != waiting_.end()) waiting_.erase(w);
}

void Scheduler::preempt(SchedRequest * req) {
    cache_->free(*req->cache);
    req->status = PREEMPTED;
    req->num_computed_tokens = 0;
    req->num_preemptions++;
    num_preemptions++;
    running_.erase(std::find(running_.begin(), running_.end(), req));
    if (cfg_.priority_policy) enqueue(req);
    else waiting_.push_front(req);
}

SchedulerOutput Scheduler::schedule() {
    SchedulerOutput out;
    int budget = cfg_.max_num_batched_tokens;
    const int cap = cfg_.long_prefill_token_threshold;

    size_t idx = 0;
    while (idx < running_.size() && budget > 0) {
        SchedRequest * req = running_[idx];
        int n_new = req->n_tokens() - req->num_computed_tokens;
        if (cap > 0) n_new = std::min(n_new, cap);
        n_new = std::min(n_new, budget);
        if (n_new == 0) {
            idx++;
            continue;
        }
        bool ok = true;
        while (!cache_->allocate(*req->cache, req->num_computed_tokens, n_new, nullptr)) {
            SchedRequest * victim = running_.back();
            if (victim == req) {
                preempt(req);
                out.preempted.push_back(req);
                ok = false;
                break;
            }
            for (auto it = out.scheduled.begin(); it != out.scheduled.end(); ++it)
                if (it->req == victim) {
                    budget += it->n_new_tokens;
                    out.total_tokens -= it->n_new_tokens;
                    out.scheduled.erase(it);
                    break;
                }
            preempt(victim);
            out.preempted.push_back(victim);
        }
        if (!ok) break;
        out.scheduled.push_back({req, n_new, false});
        out.total_tokens += n_new;
        budget -= n_new;
        idx++;
    }

    if (out.preempted.empty()) {
        while (!waiting_.empty() && budget > 0 && (int) running_.size() < cfg_.max_num_seqs) {
            SchedRequest * req = waiting_.front();
            std::vector<std::vector<int>> computed;
            bool have_computed = false;
            int n_computed = req->num_computed_tokens;
            if (n_computed == 0) {
                cache_->update_hashes(req->cache->hashes, req->tokens.data(), req->n_tokens(), req->cache_salt);
                n_computed = cache_->find_cached_prefix(req->tokens.data(), req->n_tokens(), req->cache->hashes.data(),
                                                        (int) req->cache->hashes.size(), computed);
                have_computed = true;
                cache_->prefix_queries += req->n_tokens() / cache_->block_size();
                cache_->prefix_hits += n_computed / cache_->block_size();
            }
            int n_new = req->n_tokens() - n_computed;
            if (cap > 0) n_new = std::min(n_new, cap);
            if (!cfg_.enable_chunked_prefill && n_new > budget) break;
            n_new = std::min(n_new, budget);
            if (n_new == 0) break;
            if (!cache_->allot_state(*req->cache)) break;
            if (!cache_->allocate(*req->cache, n_computed, n_new, have_computed ? &computed : nullptr)) {
                cache_->free(*req->cache);      // holds no pages; gives the state slot back
                break;
            }
            waiting_.pop_front();
            const bool resumed = req->status == PREEMPTED;
            req->status = RUNNING;
            req->num_computed_tokens = n_computed;
            if (!resumed) req->num_cached_tokens = n_computed;
            running_.push_back(req);
            out.scheduled.push_back({req, n_new, resumed});
            out.total_tokens += n_new;
            budget -= n_new;
        }
    }
    return out;
}

void Scheduler::update_after_step(const SchedulerOutput & out) {
    for (const auto & s : out.scheduled) {
        SchedRequest * r = s.req;
        if (r->is_finished()) continue;
        r->num_computed_tokens += s.n_new_tokens;
        cache_->update_hashes(r->cache->hashes, r->tokens.data(), r->n_tokens(), r->cache_salt);
        cache_->commit(*r->cache, r->tokens.data(), r->n_tokens(), std::min(r->num_computed_tokens, r->n_tokens()));
    }
}

}  // namespace iian_b200
