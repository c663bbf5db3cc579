// C interface of the native step function and engine loop (include/iian_b200/engine.h), for bindings.
// Functions that can fail return 0 on success and non-zero otherwise; iian_engine_last_error() gives the text.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct { const void * ptr; int dtype, rows, cols; } IianMatrix;      // dtype: 0 float32, 1 bfloat16

typedef struct {
    const float * mixer_norm_w; float mixer_norm_eps;
    const float * ffn_norm_w; float ffn_norm_eps;
    IianMatrix w_qkv, w_o;
    const float * b_qkv; const float * b_o;
    const float * q_norm_w; const float * k_norm_w; float qk_norm_eps;
    int num_heads, num_kv_heads, head_dim;
    float scale;
    int window;
    const float * inv_freq; int rot_dim, rope_style, rope_key;
    IianMatrix w_gate_up, w_down;
    int intermediate, interleave;
} IianLayer;

typedef struct { int layer, group, writes_cache; void * k_cache; void * v_cache; int num_pages; } IianCall;

typedef struct {
    int dtype, hidden, vocab;
    IianMatrix embedding, head;
    const float * final_norm_w; float final_norm_eps;
    const IianLayer * layers; int n_layers;
    const IianCall * calls; int n_calls;
    int page_size, num_groups;
} IianModel;

typedef struct {
    int max_num_seqs, max_model_len, cuda_graphs, weight_prefetch, prefetch_window_mb, tcgen05_min_tiles, library_gemm_only,
        fuse_norm, fused_decode, attention_tc, cluster_merge, tcgen05_pair, decode_stages, max_splits, decode_ctas_per_sm,
        stream_product, stream_stages, pdl_stream, decode_tma, split_mixed;
} IianRunnerOptions;

const char * iian_engine_last_error(void);

// libs: paths of the kernel libraries in the order elementwise, rope_kv, attention_generic, gemm_simt, sampling,
// gemm_skinny, attention_mma, prefetch, gemm_tcgen05, attention_tc, gemm_stream (null or "": not needed); cache: a cache manager
// of the host runtime (iian_cache_new).  Null on failure.
void * iian_runner_new(const IianModel * model, const char * const * libs, void * cache, const IianRunnerOptions * opt);
void iian_runner_delete(void * runner);
// One step: entry e brings n_tokens[e] tokens (concatenated in tokens) after starts[e] tokens in caches[e], and wants
// the logits at n_want[e] places (concatenated in want).  *logits: float32 [*n_rows, vocab] on the device, valid
// until the next step (null if nothing is wanted).
int iian_runner_step(void * runner, void * const * caches, const int32_t * tokens, const int * n_tokens, const int * starts,
                     const int32_t * want, const int * n_want, int n_entries, void * stream, const float ** logits, int * n_rows);
// what: 0 launches, 1 graphs captured, 2 bytes of the last upload
long long iian_runner_get(void * runner, int what);
long long iian_runner_launches_of(void * runner, const char * entry);
int iian_runner_check_status(void * runner);
void iian_runner_set_cuda_graphs(void * runner, int on);

typedef struct {
    float temperature; int top_k; float top_p, min_p; long long seed; int max_tokens, min_tokens, ignore_eos;
    const int32_t * stop_token_ids; int n_stop;
} IianSampling;

typedef struct {
    int max_model_len; long long seed; const int32_t * eos_token_ids; int n_eos;
    int max_num_seqs, max_num_batched_tokens, long_prefill_token_threshold, enable_chunked_prefill, priority_policy;
} IianEngineOptions;

// step_fn: a runner (iian_runner_new); cache: the same cache manager the runner was given.
void * iian_engine_new(void * step_fn, void * cache, const IianEngineOptions * opt, const char * sampling_library);
void iian_engine_delete(void * engine);
long long iian_engine_submit(void * engine, const int32_t * prompt, int n, const IianSampling * params, int priority);    // id, or -1
int iian_engine_abort(void * engine, long long id);
int iian_engine_step(void * engine, void * stream, int * did_work);
// The request's next chunk: up to cap tokens into tokens, *n_tokens how many, info = {finished, finish_reason,
// n_prompt, n_output, n_cached}; returns 1 if there was a chunk, 0 if none, -1 on error.
int iian_engine_poll(void * engine, long long id, int32_t * tokens, int cap, int * n_tokens, int * info);
int iian_engine_has_unfinished(void * engine);
// out: requests_total, requests_finished, requests_aborted, prompt_tokens, generation_tokens, cached_prompt_tokens, steps,
// preemptions, num_running, num_waiting, prefix_cache_queries, prefix_cache_hits (12 values); *kv_usage
int iian_engine_stats(void * engine, long long * out, double * kv_usage);

#ifdef __cplusplus
}
#endif
