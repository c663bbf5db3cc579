// Engine: the loop above the step function (include/iian_b200/engine.h).
//
// Behaviour follows the reference's Engine (src/iian/engine.cpp): submit validates and queues a tokenized prompt
// (:290-326); step schedules, runs one mixed batch, advances the computed counts, samples one token for every
// request whose last token was in the batch, applies the stop rules and frees finished requests (:456-637,
// :639-762).  Sampling runs on the device over the step's logits (iian_b200/csrc/sampling.cu); a request's
// uniform numbers are a hash of (its seed, the index of the output token), so its tokens do not depend on what
// else is in the batch.
#include "iian_b200/engine.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cmath>
#include <map>
#include <stdexcept>

namespace iian_b200 {

namespace {

constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

uint64_t splitmix64(uint64_t x) {
    x += kGolden;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// number `index` of the stream `seed`: a float32-exact value in [0, 1)
float uniform(uint64_t seed, uint64_t index) {
    const uint64_t h = splitmix64(splitmix64(seed) ^ (index * 0xD1B54A32D192ED03ull));
    return (float) (h >> 40) / (float) (1 << 24);
}

struct Req {
    SchedRequest sched;
    SamplingOptions params;
    int n_prompt = 0;
    uint64_t seed = 0;
    std::deque<OutputChunk> outputs;
    std::vector<int32_t> pending;
    int finish_reason = FINISH_NONE;
    std::string error;
    int n_output() const { return sched.n_tokens() - n_prompt; }
};

using S = cudaStream_t;

}  // namespace

struct Engine::Impl {
    StepFunction * step_fn;
    CacheManager * cache;
    EngineOptions opt;
    Scheduler scheduler;
    std::map<long long, std::unique_ptr<Req>> requests;      // live and finished-but-unread
    std::vector<Req *> fresh;
    std::vector<long long> aborts;
    long long next_id = 1;
    EngineStats st;
    mutable std::mutex mu;
    void * sampling_lib = nullptr;
    int (*argmax)(const float *, int, int, long long, int *, S) = nullptr;
    int (*argmax_wide)(const float *, int, int, long long, void *, int *, S) = nullptr;
    int (*sample)(const float *, int, int, long long, const float *, const int *, const float *, const float *, const float *, int *, S) = nullptr;
    int (*logit_edits)(float *, int, int, long long, const int *, const int *, const int *, const int *, const float *, const float *,
                       const float *, const float *, S) = nullptr;
    int * d_edit_i = nullptr; float * d_edit_f = nullptr; size_t cap_edit = 0;
    // device and pinned buffers of the sampler
    int * d_out = nullptr; float * d_par = nullptr; int * d_topk = nullptr; void * d_scratch = nullptr;
    int * h_out = nullptr; float * h_par = nullptr; int * h_topk = nullptr;
    int cap_rows = 0;

    Impl(StepFunction * s, CacheManager * c, const EngineOptions & o) : step_fn(s), cache(c), opt(o), scheduler(o.sched, c) {}

    void reserve(int rows) {
        if (rows <= cap_rows) return;
        release();
        cap_rows = std::max(rows, 64);
        cudaMalloc(reinterpret_cast<void **>(&d_out), cap_rows * sizeof(int));
        cudaMalloc(reinterpret_cast<void **>(&d_par), 4 * cap_rows * sizeof(float));
        cudaMalloc(reinterpret_cast<void **>(&d_topk), cap_rows * sizeof(int));
        cudaMalloc(&d_scratch, (size_t) cap_rows * 64 * 2 * sizeof(float));
        cudaMallocHost(reinterpret_cast<void **>(&h_out), cap_rows * sizeof(int));
        cudaMallocHost(reinterpret_cast<void **>(&h_par), 4 * cap_rows * sizeof(float));
        cudaMallocHost(reinterpret_cast<void **>(&h_topk), cap_rows * sizeof(int));
    }
    void release() {
        if (d_out) cudaFree(d_out);
        if (d_par) cudaFree(d_par);
        if (d_topk) cudaFree(d_topk);
        if (d_scratch) cudaFree(d_scratch);
        if (d_edit_i) cudaFree(d_edit_i);
        if (d_edit_f) cudaFree(d_edit_f);
        d_edit_i = nullptr; d_edit_f = nullptr; cap_edit = 0;
        if (h_out) cudaFreeHost(h_out);
        if (h_par) cudaFreeHost(h_par);
        if (h_topk) cudaFreeHost(h_topk);
        d_out = nullptr; d_par = nullptr; d_topk = nullptr; d_scratch = nullptr; h_out = nullptr; h_par = nullptr; h_topk = nullptr;
    }

    void deliver(Req & r, bool final) {
        OutputChunk ch;
        ch.tokens.swap(r.pending);
        ch.finished = final;
        ch.finish_reason = r.finish_reason;
        ch.error = r.error;
        ch.n_prompt_tokens = r.n_prompt;
        ch.n_output_tokens = r.n_output();
        ch.n_cached_tokens = r.sched.num_cached_tokens;
        r.outputs.push_back(std::move(ch));
    }
    void finish(Req & r, int status, int why, const std::string & error = "") {
        r.finish_reason = why;
        r.error = error;
        scheduler.finish_request(&r.sched, status);
        st.requests_finished++;
        if (why == FINISH_ABORT) st.requests_aborted++;
        st.cached_prompt_tokens += r.sched.num_cached_tokens;
        deliver(r, true);
    }
    bool is_eos(int32_t t) const {
        for (int32_t e : opt.eos_token_ids) if (e == t) return true;
        return false;
    }

    // While a request has produced fewer than min_tokens tokens, the ids that would end it may not be produced
    // (src/iian/sampler.cpp:89-91): their logits are set to -inf by the logits-processor kernel.
    void ban_end_tokens(float * logits, const std::vector<Req *> & reqs, S stream) {
        const int r = (int) reqs.size(), v = step_fn->vocab();
        std::vector<int> ints(2 * (r + 1), 0);                 // allow_off [r + 1] (no allow lists), edit_off [r + 1]
        std::vector<int> toks;
        for (int i = 0; i < r; i++) {
            const Req & q = *reqs[i];
            if (q.n_output() < q.params.min_tokens) {
                for (int32_t t : opt.eos_token_ids) if (t >= 0 && t < v) toks.push_back(t);
                for (int32_t t : q.params.stop_token_ids) toks.push_back(t);
            }
            ints[r + 1 + i + 1] = (int) toks.size();
        }
        if (toks.empty()) return;
        const size_t n = toks.size();
        ints.insert(ints.end(), toks.begin(), toks.end());
        std::vector<float> vals(4 * n);
        for (size_t i = 0; i < n; i++) { vals[i] = -INFINITY; vals[n + i] = 1.0f; vals[2 * n + i] = 1.0f; vals[3 * n + i] = 0.0f; }
        if (cap_edit < ints.size() + vals.size()) {
            if (d_edit_i) cudaFree(d_edit_i);
            if (d_edit_f) cudaFree(d_edit_f);
            cap_edit = 2 * (ints.size() + vals.size());
            cudaMalloc(reinterpret_cast<void **>(&d_edit_i), cap_edit * sizeof(int));
            cudaMalloc(reinterpret_cast<void **>(&d_edit_f), cap_edit * sizeof(float));
        }
        cudaMemcpyAsync(d_edit_i, ints.data(), ints.size() * sizeof(int), cudaMemcpyHostToDevice, stream);
        cudaMemcpyAsync(d_edit_f, vals.data(), vals.size() * sizeof(float), cudaMemcpyHostToDevice, stream);
        cudaStreamSynchronize(stream);                          // the host vectors go out of scope
        const int * allow_off = d_edit_i, * edit_off = d_edit_i + (r + 1), * allow_ids = d_edit_i + 2 * (r + 1), * edit_tok = allow_ids;
        const int code = logit_edits(logits, r, v, v, allow_off, allow_ids, edit_off, edit_tok, d_edit_f, d_edit_f + n, d_edit_f + 2 * n,
                                     d_edit_f + 3 * n, stream);
        if (code != 0) throw std::runtime_error("logit_edits failed with code " + std::to_string(code));
    }

    // one token per logits row (greedy rows by argmax with ties to the lowest id; the others by the sampling kernel)
    void sample_rows(const float * logits, const std::vector<Req *> & reqs, S stream) {
        const int r = (int) reqs.size(), v = step_fn->vocab();
        reserve(r);
        ban_end_tokens(const_cast<float *>(logits), reqs, stream);
        bool all_greedy = true;
        for (Req * q : reqs) all_greedy = all_greedy && q->params.temperature < 1e-5f;
        int code;
        if (all_greedy) {
            code = v >= 16384 ? argmax_wide(logits, r, v, v, d_scratch, d_out, stream) : argmax(logits, r, v, v, d_out, stream);
        } else {
            for (int i = 0; i < r; i++) {
                const SamplingOptions & p = reqs[i]->params;
                h_par[i] = p.temperature;
                h_par[r + i] = p.top_p;
                h_par[2 * r + i] = p.min_p;
                h_par[3 * r + i] = uniform(reqs[i]->seed, (uint64_t) reqs[i]->n_output());
                h_topk[i] = std::max(p.top_k, 0);
            }
            cudaMemcpyAsync(d_par, h_par, 4 * r * sizeof(float), cudaMemcpyHostToDevice, stream);
            cudaMemcpyAsync(d_topk, h_topk, r * sizeof(int), cudaMemcpyHostToDevice, stream);
            code = sample(logits, r, v, v, d_par, d_topk, d_par + r, d_par + 2 * r, d_par + 3 * r, d_out, stream);
        }
        if (code != 0) throw std::runtime_error("sampling kernel failed with code " + std::to_string(code));
        cudaMemcpyAsync(h_out, d_out, r * sizeof(int), cudaMemcpyDeviceToHost, stream);
        if (cudaStreamSynchronize(stream) != cudaSuccess) throw std::runtime_error(std::string("sampling: ") + cudaGetErrorString(cudaGetLastError()));
    }
};

Engine::Engine(StepFunction * step, CacheManager * cache, const EngineOptions & opt, const std::string & sampling_library)
    : impl_(new Impl(step, cache, opt)) {
    if (opt.max_model_len <= 0) throw std::invalid_argument("max_model_len must be positive");
    void * h = dlopen(sampling_library.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) throw std::runtime_error("cannot load the sampling kernels " + sampling_library + ": " + dlerror());
    impl_->sampling_lib = h;
    impl_->argmax = reinterpret_cast<decltype(impl_->argmax)>(dlsym(h, "iian_argmax"));
    impl_->argmax_wide = reinterpret_cast<decltype(impl_->argmax_wide)>(dlsym(h, "iian_argmax_wide"));
    impl_->sample = reinterpret_cast<decltype(impl_->sample)>(dlsym(h, "iian_sample"));
    impl_->logit_edits = reinterpret_cast<decltype(impl_->logit_edits)>(dlsym(h, "iian_logit_edits"));
    if (!impl_->argmax || !impl_->argmax_wide || !impl_->sample || !impl_->logit_edits) throw std::runtime_error("the sampling library lacks an entry point");
}

Engine::~Engine() {
    impl_->release();
    if (impl_->sampling_lib) dlclose(impl_->sampling_lib);
}

long long Engine::submit(const std::vector<int32_t> & prompt, const SamplingOptions & p, int priority) {
    Impl & m = *impl_;
    const int v = m.step_fn->vocab();
    if (prompt.empty()) throw std::invalid_argument("prompt must not be empty");
    if (p.temperature < 0.0f) throw std::invalid_argument("temperature must be >= 0");
    if (!(p.top_p > 0.0f && p.top_p <= 1.0f)) throw std::invalid_argument("top_p must be in (0, 1]");
    if (p.top_k < -1) throw std::invalid_argument("top_k must be -1, 0 or positive");
    if (!(p.min_p >= 0.0f && p.min_p <= 1.0f)) throw std::invalid_argument("min_p must be in [0, 1]");
    if (p.max_tokens < -1 || p.max_tokens == 0) throw std::invalid_argument("max_tokens must be >= 1");
    if (p.min_tokens < 0 || (p.max_tokens > 0 && p.min_tokens > p.max_tokens)) throw std::invalid_argument("min_tokens must be in [0, max_tokens]");
    for (int32_t t : prompt)
        if (t < 0 || t >= v) throw std::invalid_argument("prompt token id out of range: " + std::to_string(t));
    for (int32_t t : p.stop_token_ids)
        if (t < 0 || t >= v) throw std::invalid_argument("stop_token_ids out of range: " + std::to_string(t));
    if ((int) prompt.size() >= m.opt.max_model_len)
        throw std::invalid_argument("prompt is too long: " + std::to_string(prompt.size()) + " tokens, max_model_len is " + std::to_string(m.opt.max_model_len));
    std::lock_guard<std::mutex> lock(m.mu);
    auto r = std::make_unique<Req>();
    const long long id = m.next_id++;
    r->sched.id = id;
    r->sched.tokens = prompt;
    r->sched.priority = priority;
    r->sched.arrival = std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
    r->sched.cache.reset(m.cache->new_request());
    r->params = p;
    r->n_prompt = (int) prompt.size();
    r->seed = p.seed >= 0 ? (uint64_t) p.seed : (uint64_t) m.opt.seed + (uint64_t) id * kGolden;
    m.fresh.push_back(r.get());
    m.requests[id] = std::move(r);
    m.st.requests_total++;
    return id;
}

void Engine::abort(long long id) {
    std::lock_guard<std::mutex> lock(impl_->mu);
    impl_->aborts.push_back(id);
}

bool Engine::step(void * stream_) {
    Impl & m = *impl_;
    S stream = static_cast<S>(stream_);
    std::vector<Req *> fresh;
    std::vector<long long> aborts;
    {
        std::lock_guard<std::mutex> lock(m.mu);
        fresh.swap(m.fresh);
        aborts.swap(m.aborts);
    }
    for (Req * r : fresh) m.scheduler.add_request(&r->sched);
    for (long long id : aborts) {
        auto it = m.requests.find(id);
        if (it != m.requests.end() && !it->second->sched.is_finished()) m.finish(*it->second, FINISHED_ABORTED, FINISH_ABORT);
    }
    if (!m.scheduler.has_requests()) return false;
    SchedulerOutput so = m.scheduler.schedule();
    m.st.preemptions = m.scheduler.num_preemptions;
    if (so.scheduled.empty()) {
        if (!so.preempted.empty()) return true;
        if (m.scheduler.running().empty()) {              // cannot fit even alone (src/iian/engine.cpp:477-485)
            std::vector<SchedRequest *> stuck(m.scheduler.waiting().begin(), m.scheduler.waiting().end());
            for (SchedRequest * s : stuck) m.finish(*m.requests.at(s->id), FINISHED_ERROR, FINISH_ERROR, "request does not fit in the KV cache");
        }
        return false;
    }
    StepBatch batch;
    std::vector<Req *> sampled;
    std::vector<int32_t> wants(so.scheduled.size());
    long long n_prompt_done = 0;
    for (size_t i = 0; i < so.scheduled.size(); i++) {
        const ScheduledRequest & s = so.scheduled[i];
        SchedRequest * r = s.req;
        const int start = r->num_computed_tokens;
        const bool reaches_end = start + s.n_new_tokens >= r->n_tokens();
        StepEntry e;
        e.cache = r->cache.get();
        e.tokens = r->tokens.data() + start;
        e.n_tokens = s.n_new_tokens;
        e.start = start;
        wants[i] = s.n_new_tokens - 1;
        e.want = reaches_end ? &wants[i] : nullptr;
        e.n_want = reaches_end ? 1 : 0;
        batch.entries.push_back(e);
        Req * q = m.requests.at(r->id).get();
        if (reaches_end) sampled.push_back(q);
        if (start < q->n_prompt) n_prompt_done += std::min(s.n_new_tokens, q->n_prompt - start);
    }
    int n_rows = 0;
    const float * logits = m.step_fn->step(batch, stream, &n_rows);
    m.st.steps++;
    m.scheduler.update_after_step(so);
    m.st.prompt_tokens += n_prompt_done;
    if (sampled.empty()) return true;
    if (n_rows != (int) sampled.size() || logits == nullptr) throw std::runtime_error("the step returned " + std::to_string(n_rows) + " rows of logits, expected " + std::to_string(sampled.size()));
    m.sample_rows(logits, sampled, stream);
    for (size_t i = 0; i < sampled.size(); i++) {
        Req & r = *sampled[i];
        int32_t tok = m.h_out[i];
        r.sched.tokens.push_back(tok);
        r.pending.push_back(tok);
        m.st.generation_tokens++;
        const SamplingOptions & p = r.params;
        bool stop = false;
        int why = FINISH_NONE;
        if (m.is_eos(tok) && !p.ignore_eos) { stop = true; why = FINISH_STOP; }
        if (!stop)
            for (int32_t t : p.stop_token_ids) if (t == tok) { stop = true; why = FINISH_STOP; break; }
        if (!stop && p.max_tokens > 0 && r.n_output() >= p.max_tokens) { stop = true; why = FINISH_LENGTH; }
        if (!stop && r.sched.n_tokens() >= m.opt.max_model_len) { stop = true; why = FINISH_LENGTH; }
        if (stop) m.finish(r, why == FINISH_LENGTH ? FINISHED_LENGTH : FINISHED_STOPPED, why);
        else m.deliver(r, false);
    }
    return true;
}

bool Engine::poll(long long id, OutputChunk & out) {
    Impl & m = *impl_;
    auto it = m.requests.find(id);
    if (it == m.requests.end() || it->second->outputs.empty()) return false;
    out = std::move(it->second->outputs.front());
    it->second->outputs.pop_front();
    if (out.finished && it->second->outputs.empty()) m.requests.erase(it);
    return true;
}

bool Engine::has_unfinished() const {
    const Impl & m = *impl_;
    std::lock_guard<std::mutex> lock(m.mu);
    return m.scheduler.has_requests() || !m.fresh.empty();
}

EngineStats Engine::stats() const {
    const Impl & m = *impl_;
    EngineStats s = m.st;
    s.num_running = (int) m.scheduler.running().size();
    s.num_waiting = (int) m.scheduler.waiting().size();
    s.kv_usage = m.cache->usage();
    s.prefix_cache_queries = m.cache->prefix_queries;
    s.prefix_cache_hits = m.cache->prefix_hits;
    s.preemptions = m.scheduler.num_preemptions;
    return s;
}

}  // namespace iian_b200
