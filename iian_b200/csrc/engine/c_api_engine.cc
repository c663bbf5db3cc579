// C interface of the native step function and engine loop (include/iian_b200/engine_c_api.h).
#include "iian_b200/engine_c_api.h"

#include <string>

#include "iian_b200/engine.h"

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

MatrixDesc matrix(const IianMatrix & m) {
    MatrixDesc d;
    d.ptr = m.ptr; d.dtype = m.dtype; d.rows = m.rows; d.cols = m.cols;
    return d;
}

struct EngineHandle {
    std::unique_ptr<Engine> engine;
};
}  // namespace

extern "C" {

const char * iian_engine_last_error(void) { return g_error.c_str(); }

void * iian_runner_new(const IianModel * model, const char * const * libs, void * cache, const IianRunnerOptions * o) {
    NativeRunner * r = nullptr;
    guarded([&] {
        ModelDesc m;
        m.dtype = model->dtype; m.hidden = model->hidden; m.vocab = model->vocab;
        m.embedding = matrix(model->embedding); m.head = matrix(model->head);
        m.final_norm_w = model->final_norm_w; m.final_norm_eps = model->final_norm_eps;
        m.page_size = model->page_size; m.num_groups = model->num_groups;
        for (int i = 0; i < model->n_layers; i++) {
            const IianLayer & s = model->layers[i];
            LayerDesc L;
            L.mixer_norm_w = s.mixer_norm_w; L.mixer_norm_eps = s.mixer_norm_eps;
            L.ffn_norm_w = s.ffn_norm_w; L.ffn_norm_eps = s.ffn_norm_eps;
            L.w_qkv = matrix(s.w_qkv); L.w_o = matrix(s.w_o);
            L.b_qkv = s.b_qkv; L.b_o = s.b_o;
            L.q_norm_w = s.q_norm_w; L.k_norm_w = s.k_norm_w; L.qk_norm_eps = s.qk_norm_eps;
            L.num_heads = s.num_heads; L.num_kv_heads = s.num_kv_heads; L.head_dim = s.head_dim;
            L.scale = s.scale; L.window = s.window;
            L.inv_freq = s.inv_freq; L.rot_dim = s.rot_dim; L.rope_style = s.rope_style; L.rope_key = s.rope_key;
            L.w_gate_up = matrix(s.w_gate_up); L.w_down = matrix(s.w_down);
            L.intermediate = s.intermediate; L.interleave = s.interleave;
            m.layers.push_back(L);
        }
        for (int i = 0; i < model->n_calls; i++) {
            const IianCall & s = model->calls[i];
            if (s.layer < 0 || s.layer >= model->n_layers) throw std::invalid_argument("run order names a layer the model does not have");
            if (s.group < 0 || s.group >= model->num_groups) throw std::invalid_argument("run order names a page group the cache does not have");
            CallDesc c;
            c.layer = s.layer; c.group = s.group; c.writes_cache = s.writes_cache;
            c.k_cache = s.k_cache; c.v_cache = s.v_cache; c.num_pages = s.num_pages;
            m.calls.push_back(c);
        }
        KernelLibraries kl;
        std::string * slots[11] = {&kl.elementwise, &kl.rope_kv, &kl.attention_generic, &kl.gemm_simt, &kl.sampling, &kl.gemm_skinny,
                                   &kl.attention_mma, &kl.prefetch, &kl.gemm_tcgen05, &kl.attention_tc, &kl.gemm_stream};
        for (int i = 0; i < 11; i++) if (libs[i] != nullptr) *slots[i] = libs[i];
        RunnerOptions opt;
        opt.max_num_seqs = o->max_num_seqs; opt.max_model_len = o->max_model_len; opt.cuda_graphs = o->cuda_graphs != 0;
        opt.weight_prefetch = o->weight_prefetch != 0; opt.prefetch_window_mb = o->prefetch_window_mb;
        opt.tcgen05_min_tiles = o->tcgen05_min_tiles; opt.library_gemm_only = o->library_gemm_only != 0;
        opt.fuse_norm = o->fuse_norm != 0; opt.fused_decode = o->fused_decode != 0; opt.attention_tc = o->attention_tc != 0;
        opt.cluster_merge = o->cluster_merge != 0; opt.tcgen05_pair = o->tcgen05_pair != 0; opt.decode_stages = o->decode_stages;
        opt.max_splits = o->max_splits; opt.decode_ctas_per_sm = o->decode_ctas_per_sm;
        opt.stream_product = o->stream_product != 0; opt.stream_stages = o->stream_stages; opt.pdl_stream = o->pdl_stream != 0;
        opt.decode_tma = o->decode_tma != 0; opt.split_mixed = o->split_mixed != 0;
        r = new NativeRunner(m, kl, static_cast<CacheManager *>(cache), opt);
    });
    return r;
}

void iian_runner_delete(void * runner) { delete static_cast<NativeRunner *>(runner); }

int iian_runner_step(void * runner, void * const * caches, const int32_t * tokens, const int * n_tokens, const int * starts,
                     const int32_t * want, const int * n_want, int n_entries, void * stream, const float ** logits, int * n_rows) {
    return guarded([&] {
        StepBatch b;
        b.entries.reserve(n_entries);
        const int32_t * t = tokens, * w = want;
        for (int i = 0; i < n_entries; i++) {
            StepEntry e;
            e.cache = static_cast<RequestCache *>(caches[i]);
            e.tokens = t; e.n_tokens = n_tokens[i]; e.start = starts[i];
            e.want = w; e.n_want = n_want[i];
            t += n_tokens[i];
            w += n_want[i];
            b.entries.push_back(e);
        }
        *logits = static_cast<NativeRunner *>(runner)->step(b, stream, n_rows);
    });
}

long long iian_runner_get(void * runner, int what) {
    auto * r = static_cast<NativeRunner *>(runner);
    switch (what) {
        case 0: return r->launches();
        case 1: return r->num_graphs();
        case 2: return r->last_upload_bytes();
    }
    return -1;
}
long long iian_runner_launches_of(void * runner, const char * entry) { return static_cast<NativeRunner *>(runner)->launches_of(entry); }
void iian_runner_set_cuda_graphs(void * runner, int on) { static_cast<NativeRunner *>(runner)->set_cuda_graphs(on != 0); }
int iian_runner_check_status(void * runner) { return guarded([&] { static_cast<NativeRunner *>(runner)->check_status(); }); }

void * iian_engine_new(void * step_fn, void * cache, const IianEngineOptions * o, const char * sampling_library) {
    EngineHandle * h = nullptr;
    guarded([&] {
        EngineOptions opt;
        opt.max_model_len = o->max_model_len;
        opt.seed = o->seed;
        opt.eos_token_ids.assign(o->eos_token_ids, o->eos_token_ids + o->n_eos);
        opt.sched.max_num_seqs = o->max_num_seqs;
        opt.sched.max_num_batched_tokens = o->max_num_batched_tokens;
        opt.sched.long_prefill_token_threshold = o->long_prefill_token_threshold;
        opt.sched.enable_chunked_prefill = o->enable_chunked_prefill != 0;
        opt.sched.priority_policy = o->priority_policy != 0;
        auto eng = std::make_unique<Engine>(static_cast<StepFunction *>(static_cast<NativeRunner *>(step_fn)), static_cast<CacheManager *>(cache), opt,
                                            sampling_library);
        h = new EngineHandle{std::move(eng)};
    });
    return h;
}
void iian_engine_delete(void * engine) { delete static_cast<EngineHandle *>(engine); }

long long iian_engine_submit(void * engine, const int32_t * prompt, int n, const IianSampling * p, int priority) {
    long long id = -1;
    guarded([&] {
        SamplingOptions s;
        s.temperature = p->temperature; s.top_k = p->top_k; s.top_p = p->top_p; s.min_p = p->min_p; s.seed = p->seed;
        s.max_tokens = p->max_tokens; s.min_tokens = p->min_tokens; s.ignore_eos = p->ignore_eos != 0;
        s.stop_token_ids.assign(p->stop_token_ids, p->stop_token_ids + p->n_stop);
        id = static_cast<EngineHandle *>(engine)->engine->submit(std::vector<int32_t>(prompt, prompt + n), s, priority);
    });
    return id;
}
int iian_engine_abort(void * engine, long long id) { return guarded([&] { static_cast<EngineHandle *>(engine)->engine->abort(id); }); }
int iian_engine_step(void * engine, void * stream, int * did_work) {
    return guarded([&] { *did_work = static_cast<EngineHandle *>(engine)->engine->step(stream) ? 1 : 0; });
}
int iian_engine_poll(void * engine, long long id, int32_t * tokens, int cap, int * n_tokens, int * info) {
    int got = 0;
    const int rc = guarded([&] {
        OutputChunk ch;
        if (!static_cast<EngineHandle *>(engine)->engine->poll(id, ch)) return;
        if ((int) ch.tokens.size() > cap) throw std::invalid_argument("iian_engine_poll: the token buffer is too small");
        for (size_t i = 0; i < ch.tokens.size(); i++) tokens[i] = ch.tokens[i];
        *n_tokens = (int) ch.tokens.size();
        info[0] = ch.finished ? 1 : 0; info[1] = ch.finish_reason; info[2] = ch.n_prompt_tokens; info[3] = ch.n_output_tokens;
        info[4] = ch.n_cached_tokens;
        if (!ch.error.empty()) g_error = ch.error;
        got = 1;
    });
    return rc == 0 ? got : -1;
}
int iian_engine_has_unfinished(void * engine) { return static_cast<EngineHandle *>(engine)->engine->has_unfinished() ? 1 : 0; }
int iian_engine_stats(void * engine, long long * out, double * kv_usage) {
    return guarded([&] {
        const EngineStats s = static_cast<EngineHandle *>(engine)->engine->stats();
        out[0] = s.requests_total; out[1] = s.requests_finished; out[2] = s.requests_aborted; out[3] = s.prompt_tokens;
        out[4] = s.generation_tokens; out[5] = s.cached_prompt_tokens; out[6] = s.steps; out[7] = s.preemptions;
        out[8] = s.num_running; out[9] = s.num_waiting; out[10] = s.prefix_cache_queries; out[11] = s.prefix_cache_hits;
        *kv_usage = s.kv_usage;
    });
}

}  // extern "C"
