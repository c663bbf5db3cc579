// The engine in C++: a model as a flat description, the step function that walks it, and the engine loop.
//
// Surface and behaviour follow the reference's Engine (include/iian/engine.h:67-94: Engine(model, cfg), submit,
// abort, step, start / stop, stats; OutputChunk, include/iian/request.h:26-39) without text and log-probabilities,
// plus what the reference reaches only through a scheduler: a public, scheduler-free step(StepBatch) (its nearest
// piece is a hand-built UBatch, tests/e2e/test-attn-parity.cpp:24-66).
//
//  * ModelDesc is what the architecture-neutral layer description (layers of parts, the run order over them)
//    looks like once the weights are bound: device pointers and the constants of every part.  The host language
//    builds it (it owns loading and device memory); nothing in here knows an architecture by name.
//  * NativeRunner::step packs the step's integers, uploads them with one copy and issues the kernel sequence
//    from C++ through the kernels' C entry points: embedding, per run-order entry norm / mixer / norm /
//    feed-forward with the fused forms where the sizes allow them, final norm, head.  Steps in which every
//    request brings one token are replayed from CUDA graphs keyed by (padded batch, context bucket).
//  * Engine is the loop above it: admission checks, scheduling (iian_b200/scheduler.h), the step, greedy or
//    temperature sampling on the device, finish rules, output chunks.
// Only the built-in parts (RMSNorm, attention with rotary or no positions, gated feed-forward, token embedding,
// head) have a native form; a model with other parts runs through the host language's own step function.
#pragma once
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "iian_b200/scheduler.h"

namespace iian_b200 {

enum : int { DT_F32 = 0, DT_BF16 = 1 };

struct MatrixDesc {                 // [rows, cols] row-major, as files hold it ([out features, in features])
    const void * ptr = nullptr;
    int dtype = DT_BF16;
    int rows = 0, cols = 0;
};

struct LayerDesc {
    // norm before the mixer, norm before the feed-forward: x * rsqrt(mean(x^2) + eps) * w
    const float * mixer_norm_w = nullptr;
    float mixer_norm_eps = 0.0f;
    const float * ffn_norm_w = nullptr;
    float ffn_norm_eps = 0.0f;
    // attention mixer
    MatrixDesc w_qkv, w_o;          // Wq | Wk | Wv stacked; Wo
    const float * b_qkv = nullptr;  // optional biases (float32)
    const float * b_o = nullptr;
    const float * q_norm_w = nullptr, * k_norm_w = nullptr;     // per-head RMSNorm of Q and K (null: none)
    float qk_norm_eps = 0.0f;
    int num_heads = 0, num_kv_heads = 0, head_dim = 0;
    float scale = 0.0f;
    int window = 0;                 // 0: every key stays visible
    const float * inv_freq = nullptr;   // rotary: base^(-2j/dim), null: no rotation
    int rot_dim = 0, rope_style = 0, rope_key = 0;      // rope_key: layers with equal keys share one table per step
    // gated feed-forward: rows of gate and up interleaved in groups of `interleave` (8) or stacked (0)
    MatrixDesc w_gate_up, w_down;
    int intermediate = 0, interleave = 0;
};

struct CallDesc {                   // one entry of the run order
    int layer = 0;
    int group = 0;                  // page group of its cache (block table and cells in the step's integers)
    int writes_cache = 1;
    void * k_cache = nullptr;       // [pages, kv_heads, page_size, head_dim] of the cache this call works on
    void * v_cache = nullptr;
    int num_pages = 0;
};

struct ModelDesc {
    int dtype = DT_BF16;            // activation and cache dtype; DT_F32: everything in true 32-bit
    int hidden = 0, vocab = 0;
    MatrixDesc embedding, head;     // head may point at the embedding (tied)
    const float * final_norm_w = nullptr;
    float final_norm_eps = 0.0f;
    std::vector<LayerDesc> layers;
    std::vector<CallDesc> calls;
    int page_size = 16;
    int num_groups = 1;
};

struct StepEntry {                  // one request's share of a step
    RequestCache * cache = nullptr;
    const int32_t * tokens = nullptr;   // its next tokens, following the `start` tokens already in its cache
    int n_tokens = 0;
    int start = 0;
    const int32_t * want = nullptr;     // places among these tokens whose logits are returned
    int n_want = 0;
};

struct StepBatch {
    std::vector<StepEntry> entries;
};

struct RunnerOptions {
    int max_num_seqs = 4;
    int max_model_len = 0;          // sizes the block tables of captured graphs
    bool cuda_graphs = false;
    bool weight_prefetch = false;   // L2 prefetch of the next weights on a side stream inside captured graphs
    int prefetch_window_mb = 8;
    int tcgen05_min_tiles = 300;    // the own tcgen05 product from this many tiles of 256 x 256 on (else the library)
    bool library_gemm_only = false;
    bool fuse_norm = true;
    bool fused_decode = true;
    bool attention_tc = true;
    bool cluster_merge = true;
    bool tcgen05_pair = true;
    int decode_stages = 2;
    int max_splits = 32;
    int decode_ctas_per_sm = 27;    // in tenths: CTAs per SM a decode attention launch with split keys may use
    bool stream_product = true;     // products of up to 8 rows: weights through shared memory by bulk copies (gemm_stream.cu)
    int stream_stages = 12;         // 12: one CTA per SM with the deep ring; 6: two CTAs per SM
    bool pdl_stream = true;         // launch the streaming product with programmatic stream serialization
    bool decode_tma = true;         // decode attention fetches K/V tiles by TMA (head size 128) instead of cp.async
    bool split_mixed = true;        // mixed steps: decoded tokens' attention on the decode kernel, on a second stream
};

// Paths of the kernel libraries (one shared object per source, see iian_b200/csrc/build.py); empty: not needed.
struct KernelLibraries {
    std::string elementwise, rope_kv, attention_generic, gemm_simt, sampling, gemm_skinny, attention_mma, prefetch,
        gemm_tcgen05, attention_tc, gemm_stream;
};

class StepFunction {
public:
    virtual ~StepFunction() = default;
    // Runs the batch (pages for every entry's tokens must be allocated) on `stream` and returns float32 logits
    // [*n_rows, vocab] on the device, in the order of the entries and of their `want` lists (null if nothing is
    // wanted).  The buffer stays valid until the next step.
    virtual const float * step(const StepBatch & batch, void * stream, int * n_rows) = 0;
    virtual int vocab() const = 0;
};

class NativeRunner : public StepFunction {
public:
    NativeRunner(const ModelDesc & model, const KernelLibraries & libs, CacheManager * cache, const RunnerOptions & opt);
    ~NativeRunner() override;
    const float * step(const StepBatch & batch, void * stream, int * n_rows) override;
    int vocab() const override;
    long long launches() const;             // kernel launches issued so far (graph replays count what they hold)
    int num_graphs() const;
    int last_upload_bytes() const;
    long long launches_of(const char * entry) const;    // by entry point ("attention_tc", "library_gemm", ...)
    void check_status();                    // throws if a tcgen05 kernel gave up on a barrier since the last call
    void set_cuda_graphs(bool on);          // replay decode-only steps from captured graphs from now on (or stop doing so)
    struct Impl;
private:
    std::unique_ptr<Impl> impl_;
};

// ---- the engine loop ------------------------------------------------------------------------------------------
struct SamplingOptions {                    // include/iian/sampling.h:15-46, the part that needs no text
    float temperature = 1.0f;               // < 1e-5: greedy, ties to the lowest id
    int top_k = 0;
    float top_p = 1.0f;
    float min_p = 0.0f;
    long long seed = -1;                    // -1: engine seed + id * 0x9E3779B97F4A7C15
    int max_tokens = -1;                    // -1: until the context is full
    int min_tokens = 0;
    bool ignore_eos = false;
    std::vector<int32_t> stop_token_ids;
};

enum FinishReason : int { FINISH_NONE = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_ABORT = 3, FINISH_ERROR = 4 };

struct OutputChunk {
    std::vector<int32_t> tokens;
    bool finished = false;
    int finish_reason = FINISH_NONE;
    std::string error;
    int n_prompt_tokens = 0, n_output_tokens = 0, n_cached_tokens = 0;
};

struct EngineStats {
    long long requests_total = 0, requests_finished = 0, requests_aborted = 0;
    long long prompt_tokens = 0, generation_tokens = 0, cached_prompt_tokens = 0, steps = 0, preemptions = 0;
    int num_running = 0, num_waiting = 0;
    double kv_usage = 0.0;
    long long prefix_cache_queries = 0, prefix_cache_hits = 0;
};

struct EngineOptions {
    int max_model_len = 0;
    long long seed = 0;
    std::vector<int32_t> eos_token_ids;
    SchedulerConfig sched;
};

class Engine {
public:
    // `step` and `cache` outlive the engine; `sampling_library` is the path of the sampling kernels.
    Engine(StepFunction * step, CacheManager * cache, const EngineOptions & opt, const std::string & sampling_library);
    ~Engine();
    long long submit(const std::vector<int32_t> & prompt, const SamplingOptions & params, int priority = 0);   // throws std::invalid_argument
    void abort(long long id);
    bool step(void * stream = nullptr);     // schedule and run one batch; false when there was nothing to do
    bool poll(long long id, OutputChunk & out);         // the request's next chunk, if any
    bool has_unfinished() const;
    EngineStats stats() const;
    struct Impl;
private:
    std::unique_ptr<Impl> impl_;
};

}  // namespace iian_b200
