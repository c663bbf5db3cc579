// The scheduler: which requests run in the next step, and how many tokens of each.
//
// The algorithm is the reference's (src/iian/scheduler.cpp:84-160, docs/ARCHITECTURE.md:129-145):
//  * a request has num_computed_tokens and every step schedules work so that it catches up with its number
//    of tokens; there are no separate prefill and decode phases;
//  * phase 1, running requests in order: n_new = min(remaining, long-prefill cap, budget); pages are
//    allocated for computed + n_new tokens (scheduler.cpp:89-124);
//  * when pages run out, the LAST running request is preempted (its pages freed, its computed count set to
//    zero, itself put back at the front of the waiting queue) and the allocation is tried again; a victim
//    that was already scheduled in this step gets its tokens refunded; if the victim is the request itself,
//    scheduling stops (scheduler.cpp:105-118, :70-82);
//  * phase 2, admission from the waiting queue, only in a step that preempted nobody: look up the cached
//    prefix, allocate, never preempt on behalf of a waiting request (scheduler.cpp:126-158);
//  * after the step the computed counts advance and full pages are offered to the prefix index
//    (scheduler.cpp:162-171).
// No speculative tokens.  New here: a request also needs a state slot before it is admitted.
#pragma once
#include <deque>
#include <memory>
#include <vector>

#include "iian_b200/cache_manager.h"

namespace iian_b200 {

// ordering matters: finished states compare greater than PREEMPTED (include/iian/request.h:20-21)
enum RequestStatus : int {
    WAITING = 0, RUNNING = 1, PREEMPTED = 2, FINISHED_STOPPED = 3, FINISHED_LENGTH = 4, FINISHED_ABORTED = 5, FINISHED_ERROR = 6,
};

// What the scheduler keeps of a request (include/iian/request.h:64-109 without text, sampling and outputs,
// which stay with the caller).
struct SchedRequest {
    long long id = 0;
    std::vector<int32_t> tokens;             // prompt + generated
    int priority = 0;
    double arrival = 0.0;
    uint64_t cache_salt = 0;
    int status = WAITING;
    int num_computed_tokens = 0;             // catches up with tokens.size() (request.h:74)
    int num_cached_tokens = 0;               // prefix hit at first admission
    int num_preemptions = 0;
    std::unique_ptr<RequestCache> cache;
    int n_tokens() const { return (int) tokens.size(); }
    bool is_finished() const { return status > PREEMPTED; }
};

struct SchedulerConfig {
    int max_num_seqs = 32;
    int max_num_batched_tokens = 1024;
    int long_prefill_token_threshold = 0;
    bool enable_chunked_prefill = true;
    bool priority_policy = false;            // false: first come, first served
};

struct ScheduledRequest {
    SchedRequest * req;
    int n_new_tokens;
    bool resumed;
};

struct SchedulerOutput {
    std::vector<ScheduledRequest> scheduled;
    std::vector<SchedRequest *> preempted;
    int total_tokens = 0;
};

class Scheduler {
public:
    Scheduler(const SchedulerConfig & cfg, CacheManager * cache);

    void add_request(SchedRequest * req);    // the caller keeps the request alive until it is finished
    void finish_request(SchedRequest * req, int status);
    bool has_requests() const { return !waiting_.empty() || !running_.empty(); }
    const std::deque<SchedRequest *> & waiting() const { return waiting_; }
    const std::vector<SchedRequest *> & running() const { return running_; }

    SchedulerOutput schedule();
    void update_after_step(const SchedulerOutput & out);

    long long num_preemptions = 0;

private:
    void enqueue(SchedRequest * req);
    void preempt(SchedRequest * req);

    SchedulerConfig cfg_;
    CacheManager * cache_;
    std::deque<SchedRequest *> waiting_;
    std::vector<SchedRequest *> running_;
};

}  // namespace iian_b200
