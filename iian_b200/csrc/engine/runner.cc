// NativeRunner: the step function in C++ (include/iian_b200/engine.h).
//
// It packs the step's integers, uploads them with one copy and issues the kernel sequence of a ModelDesc through
// the C entry points of the kernel libraries (iian_b200/csrc/*.cu, one shared object each, opened with dlopen).
// The sequence and every choice of kernel are those of the Python parts (iian_b200/parts/*.py) and of their
// kernel layer (iian_b200/ops/cuda_backend.py): the same kernels with the same arguments in the same order, so
// the 32-bit logits of both step functions are the same bits.  The reference builds the corresponding graph per
// step from its scheduler's output (src/iian/engine.cpp:491-535, src/iian/arch/qwen3.cpp:61-104).
#include "iian_b200/engine.h"

#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace iian_b200 {

namespace {

[[noreturn]] void fail(const std::string & what) { throw std::runtime_error(what); }

void cuda_ok(cudaError_t e, const char * what) {
    if (e != cudaSuccess) fail(std::string(what) + ": " + cudaGetErrorString(e));
}

const char * kernel_error(int code) {
    switch (code) {
        case 1: return "element types not supported by this kernel";
        case 2: return "a size this kernel refuses";
        case 3: return "a pointer or stride is not aligned as the kernel requires";
        case 4: return "beyond the kernel's stated maximum";
        default: return "error";
    }
}

// ---- the kernels' entry points ------------------------------------------------------------------------------
using S = cudaStream_t;
struct Kernels {
    int (*embedding)(const void *, int, const int *, float *, int, int, int, S) = nullptr;
    int (*add_rms_norm)(float *, const void *, const float *, void *, int, int, int, float, S) = nullptr;
    int (*swiglu)(const void *, void *, int, int, int, int, S) = nullptr;
    int (*gather_rows)(const void *, const int *, void *, int, int, int, int, S) = nullptr;
    int (*add_bias)(void *, const float *, int, int, int, S) = nullptr;
    int (*rotary_table)(const float *, const int *, void *, int, int, S) = nullptr;
    int (*qk_norm_rope_store)(const void *, const float *, void *, void *, void *, const float *, const float *, const float *,
                              const void *, const int *, const int *, int, int, int, int, int, int, int, float, int, int, int, S) = nullptr;
    int (*attention_generic)(const void *, const void *, const void *, void *, const int *, const int *, const int *, int,
                             const int *, int, int, int, int, int, int, int, float, int, S) = nullptr;
    int (*gemm_simt)(const void *, int, const void *, int, void *, int, int, int, int, S) = nullptr;
    int (*gemm_skinny_cfg)(const void *, const void *, void *, int, int, int, int, int, int, float *, int *, int, S) = nullptr;
    int (*gemm_skinny_fused)(const void *, const void *, void *, int, int, int, int, int, const float *, int, float, float,
                             float *, const float *, float *, S) = nullptr;
    int (*gemm_tcgen05)(const void *, const void *, void *, int, int, int, int, int, int, int *, S) = nullptr;
    int (*gemm_tcgen05_fused)(const void *, const void *, void *, int, int, int, int, int, int, int *, const float *, int, float,
                              float, float *, const float *, float *, S) = nullptr;
    int (*attention_tc)(const void *, const void *, const void *, void *, const int *, const int *, const int *, int, int, int,
                        int, int, int, int, int, int, float, int, int *, S) = nullptr;
    int (*attention_mma)(const void *, const void *, const void *, void *, float *, float *, int *, const int *, const int *,
                         const int *, int, int, int, int, int, int, int, int, int, float, int, int, int, int *, S) = nullptr;
    int (*attention_decode_fused)(const void *, void *, void *, void *, float *, float *, int *, const int *, const int *,
                                  const int *, int, int, int, int, int, int, int, float, int, int, int, const float *,
                                  const float *, const float *, const int *, float, int, int *, S) = nullptr;
    int (*attention_decode_stages)(int) = nullptr;
    int (*gemm_stream)(const void *, const void *, void *, int, int, int, int, int, const float *, int, float, float, float *,
                       const float *, float *, int *, S) = nullptr;
    int (*gemm_stream_stages)(int) = nullptr;
    int (*prefetch_l2)(const void *, long long, S) = nullptr;
};

template <typename F> void bind(void * lib, const char * name, F & fn, const std::string & path) {
    void * p = dlsym(lib, name);
    if (p == nullptr) fail("kernel library " + path + " has no entry point " + name);
    fn = reinterpret_cast<F>(p);
}

void * open_library(const std::string & path) {
    void * h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) fail("cannot load kernel library " + path + ": " + dlerror());
    return h;
}

// ---- device buffers by name, grown on demand (as the Python runner's workspace) -----------------------------------
struct Workspace {
    struct Buf { void * ptr = nullptr; size_t cap = 0; };
    std::map<std::string, Buf> bufs;
    std::vector<void *> retired;      // buffers a captured graph may still point at are kept until the end
    bool frozen = false;
    void * get(const std::string & name, size_t bytes) {
        Buf & b = bufs[name];
        if (b.cap < bytes || b.ptr == nullptr) {
            if (frozen) fail("workspace buffer '" + name + "' would have to grow while a captured graph uses it");
            if (b.ptr != nullptr) retired.push_back(b.ptr);
            const size_t cap = std::max<size_t>(bytes, 256);
            cuda_ok(cudaMalloc(&b.ptr, cap), "cudaMalloc (workspace)");
            b.cap = cap;
        }
        return b.ptr;
    }
    ~Workspace() {
        for (auto & kv : bufs) if (kv.second.ptr) cudaFree(kv.second.ptr);
        for (void * p : retired) cudaFree(p);
    }
};

// The step's integers on the device: one buffer, views into it.
struct StepInts {
    int N = 0, S = 0, R = 0;
    int max_q_len = 0, max_ctx = 0;
    bool decode_only = false, rows_identity = false;
    const int * tokens = nullptr, * positions = nullptr, * seq_of_token = nullptr, * cu_q = nullptr, * ctx_len = nullptr,
              * state_slots = nullptr, * out_rows = nullptr;
    std::vector<const int *> slots, block_table;      // per group
    std::vector<int> max_blocks;                      // per group
    int n_split = 0;                                  // fixed number of key splits (captured graphs); 0: chosen per launch
    int upload_bytes = 0;
    // A step that brings single decoded tokens beside portions of prompts has the sequences of the former first:
    int decode_seqs = 0;                              // how many (0 unless the step is mixed), and their longest context
    int decode_max_ctx = 0;
};

struct Staging {
    int32_t * host = nullptr;       // pinned
    int32_t * dev = nullptr;
    size_t cap = 0;                 // ints
    cudaEvent_t copy_done = nullptr;
    bool pending = false;
    void reserve(size_t n) {
        if (cap >= n) return;
        wait();
        if (host) cudaFreeHost(host);
        if (dev) cudaFree(dev);
        cap = std::max<size_t>(4096, 2 * n);
        cuda_ok(cudaMallocHost(reinterpret_cast<void **>(&host), cap * sizeof(int32_t)), "cudaMallocHost");
        cuda_ok(cudaMalloc(reinterpret_cast<void **>(&dev), cap * sizeof(int32_t)), "cudaMalloc (step integers)");
        if (copy_done == nullptr) cuda_ok(cudaEventCreateWithFlags(&copy_done, cudaEventDisableTiming), "cudaEventCreate");
    }
    void wait() {                    // the last upload has left the host buffer
        if (pending) { cudaEventSynchronize(copy_done); pending = false; }
    }
    void upload(size_t n, cudaStream_t stream) {
        cuda_ok(cudaMemcpyAsync(dev, host, n * sizeof(int32_t), cudaMemcpyHostToDevice, stream), "upload of the step's integers");
        cuda_ok(cudaEventRecord(copy_done, stream), "cudaEventRecord");
        pending = true;
    }
    ~Staging() {
        if (copy_done) cudaEventDestroy(copy_done);
        if (host) cudaFreeHost(host);
        if (dev) cudaFree(dev);
    }
};

// What a sub-layer hands to the next one: rows, or rows that still lack the factor per row of a folded norm.
struct Rows {
    void * x = nullptr;             // [n, width] in the activation dtype (null: nothing to add yet)
    bool prenormed = false;
    const float * partials = nullptr;   // [n, parts] sums of squares of the residual's rows
    int parts = 0;
    int width = 0;
    float eps = 0.0f;
    const float * for_norm = nullptr;   // the norm weight these rows were prepared for
};

struct GraphSlot {
    int num_seqs = 0, ctx_bucket = 0, max_blocks = 0, n_split = 1;
    Staging staging;
    Workspace ws;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    const float * logits = nullptr;
    long long launches = 0;
    StepInts ints;
    std::vector<long long> sig;
    int n_last = -1;
    ~GraphSlot() {
        if (exec) cudaGraphExecDestroy(exec);
        if (graph) cudaGraphDestroy(graph);
    }
};

}  // namespace

extern "C" int iian_pack_decode_step(void * mgr, void ** caches, const int32_t * tokens, const int32_t * starts, int n, int S,
                                     int max_blocks, int32_t * host, long long * sig, int rewrite_all, int * fresh_slots);
extern "C" const char * iian_host_last_error(void);

struct NativeRunner::Impl {
    ModelDesc model;
    RunnerOptions opt;
    CacheManager * cache;
    Kernels k;
    std::vector<void *> libs;
    int act_dtype;
    size_t act_size;
    int sm_count = 148;
    cudaStream_t stream = nullptr;          // where the current step's kernels go
    Workspace ws;                           // of eager steps
    Workspace * cur_ws = nullptr;
    Staging staging;
    int * tc_status = nullptr;
    bool tc_used = false;
    cublasHandle_t blas = nullptr;
    void * blas_ws = nullptr;
    // scratch of split attention and split products (shared by all launches: the stream orders them)
    float * attn_scratch = nullptr; size_t attn_scratch_floats = 0;
    int * attn_counters = nullptr; size_t attn_counters_n = 0;
    std::vector<void *> retired_scratch;
    long long launches = 0;
    std::unordered_map<std::string, long long> by_entry;
    int last_upload = 0;
    std::map<std::pair<int, int>, std::unique_ptr<GraphSlot>> graphs;
    // weight prefetch inside captured graphs
    std::vector<std::pair<const void *, size_t>> * weight_log = nullptr;
    struct Prefetcher {
        std::vector<std::pair<const void *, size_t>> weights;
        std::vector<size_t> starts;
        size_t total = 0, window = 0, cursor = 0;
        size_t index = 0;
        cudaStream_t side = nullptr;
    };
    Prefetcher * prefetcher = nullptr;
    cudaStream_t cap_stream = nullptr, side_stream = nullptr;
    cudaStream_t mixed_stream = nullptr;              // the decoded tokens' attention of a mixed step
    cudaEvent_t mixed_fork = nullptr, mixed_join = nullptr;
    std::map<int, void *> rotary_tables;    // rope_key -> table of the current forward pass
    std::vector<int32_t> scratch_tokens, scratch_starts, scratch_fresh;
    std::vector<void *> scratch_caches;

    void check(int code, const char * what) {
        if (code == 0) { launches++; by_entry[what]++; return; }
        if (code >= 1000) fail(std::string(what) + ": CUDA launch failed: " + cudaGetErrorString((cudaError_t) (code - 1000)));
        fail(std::string(what) + ": " + kernel_error(code));
    }
    void * buf(const char * name, size_t bytes) { return cur_ws->get(name, bytes); }

    // ---- dispatch rules (iian_b200/ops/cuda_backend.py) ---------------------------------------------------------
    static bool aligned16(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
    bool bf16_mode() const { return act_dtype == DT_BF16; }
    bool tcgen05_rows_ok(int n, int m) const {
        return n >= 128 && (long long) ((n + 255) / 256) * ((m + 255) / 256) >= opt.tcgen05_min_tiles;
    }
    bool tcgen05_ok(const void * x, int x_dtype, const MatrixDesc & w, int n) const {
        return !opt.library_gemm_only && tcgen05_rows_ok(n, w.rows) && w.cols % 8 == 0 && x_dtype == DT_BF16 && w.dtype == DT_BF16 &&
               aligned16(x) && aligned16(w.ptr);
    }
    bool skinny_ok(const void * x, int x_dtype, const MatrixDesc & w, int n) const {
        return n <= 8 && w.cols % 32 == 0 && x_dtype == DT_BF16 && w.dtype == DT_BF16 && aligned16(x) && aligned16(w.ptr);
    }
    bool can_fuse_norm(const void * x, const MatrixDesc & w, int n) const {
        return opt.fuse_norm && (skinny_ok(x, act_dtype, w, n) || tcgen05_ok(x, act_dtype, w, n));
    }
    bool can_take_prenormed(int n_rows, const MatrixDesc & w) const {
        if (!opt.fuse_norm || !bf16_mode() || w.dtype != DT_BF16 || !aligned16(w.ptr)) return false;
        if (n_rows <= 8) return w.cols % 32 == 0;
        return tcgen05_rows_ok(n_rows, w.rows) && w.cols % 8 == 0 && !opt.library_gemm_only;
    }
    int tcgen05_tile(int n_rows, int n) const {
        const bool wide = n % 256 == 0 || n > 4096;
        if (wide && opt.tcgen05_pair && n_rows > 128) return 512;
        return wide ? 256 : 128;
    }
    int norm_parts(const MatrixDesc & w, int n_rows) const {
        if (n_rows > 8) { const int cols = std::min(256, tcgen05_tile(n_rows, w.rows)); return (w.rows + cols - 1) / cols; }
        return (w.rows + 15) / 16;
    }
    int attention_splits(int num_seqs, int num_kv_heads, int max_ctx) const {
        const int tiles = std::max(1, (max_ctx + 63) / 64);
        const int base = std::max(1, num_seqs * num_kv_heads);
        const int slots = opt.decode_ctas_per_sm * sm_count / 10;      // tenths: 2.7 CTAs per SM by default
        int n = std::max(1, std::min(std::min(slots / base, (tiles + 1) / 2), opt.max_splits));
        // a power of two, merged inside a thread-block cluster of up to 16 (of which only a few fit the GPU at once);
        // 32 through scratch memory for a single sequence from 32k of context on
        if (n >= 32 && tiles >= 512) return n;
        if (n >= 16) return base * 16 <= 2 * sm_count ? 16 : 8;
        return n >= 8 ? 8 : n >= 4 ? 4 : n >= 2 ? 2 : 1;
    }

    // ---- products ---------------------------------------------------------------------------------------------
    void prefetch_head(size_t j) {
        Prefetcher & pf = *prefetcher;
        if (j >= pf.weights.size()) return;
        const size_t begin = std::max(pf.cursor, pf.starts[j]);
        const size_t end = std::min(pf.total, pf.starts[j] + pf.window);
        if (end <= begin) return;
        cudaEvent_t ev;
        cuda_ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
        cuda_ok(cudaEventRecord(ev, stream), "cudaEventRecord");
        cuda_ok(cudaStreamWaitEvent(pf.side, ev, 0), "cudaStreamWaitEvent");
        cudaEventDestroy(ev);
        while (j < pf.weights.size() && pf.starts[j] < end) {
            const size_t lo = std::max(begin, pf.starts[j]) - pf.starts[j];
            const size_t hi = std::min(end, pf.starts[j] + pf.weights[j].second) - pf.starts[j];
            if (hi > lo) check(k.prefetch_l2(static_cast<const char *>(pf.weights[j].first) + lo, (long long) (hi - lo), pf.side), "prefetch_l2");
            j++;
        }
        pf.cursor = end;
    }
    void before_stream_product() { if (prefetcher) prefetch_head(prefetcher->index + 1); }
    void after_stream_product(const MatrixDesc & w) {
        if (weight_log) weight_log->push_back({w.ptr, (size_t) w.rows * w.cols * 2});
        if (prefetcher) prefetcher->index++;
    }

    void plain_stream_product(const void * x, const MatrixDesc & w, void * out, int out_dtype, int n, int epilogue) {
        if (opt.stream_product) {
            tc_used = true;
            check(k.gemm_stream(x, w.ptr, out, out_dtype, n, w.rows, w.cols, epilogue, nullptr, 0, 0.0f, 0.0f, nullptr, nullptr, nullptr,
                                tc_status, stream), "gemm_stream");
        } else {
            check(k.gemm_skinny_cfg(x, w.ptr, out, out_dtype, n, w.rows, w.cols, 0, 1, nullptr, nullptr, epilogue, stream), "gemm_skinny");
        }
    }
    void gemm_skinny_fused(const void * x, const MatrixDesc & w, void * out, int out_dtype, int n, int epilogue, const Rows * scale,
                           float * res, const float * norm_w, float * out_partial) {
        before_stream_product();
        if (opt.stream_product) {
            tc_used = true;
            check(k.gemm_stream(x, w.ptr, out, out_dtype, n, w.rows, w.cols, epilogue,
                                scale ? scale->partials : nullptr, scale ? scale->parts : 0,
                                scale ? 1.0f / (float) scale->width : 0.0f, scale ? scale->eps : 0.0f,
                                res, norm_w, out_partial, tc_status, stream), "gemm_stream");
        } else {
            check(k.gemm_skinny_fused(x, w.ptr, out, out_dtype, n, w.rows, w.cols, epilogue,
                                      scale ? scale->partials : nullptr, scale ? scale->parts : 0,
                                      scale ? 1.0f / (float) scale->width : 0.0f, scale ? scale->eps : 0.0f,
                                      res, norm_w, out_partial, stream), "gemm_skinny_fused");
        }
        after_stream_product(w);
    }
    void gemm_tcgen05(const void * x, const MatrixDesc & w, void * out, int out_dtype, int n, int epilogue, const Rows * scale,
                      float * res, const float * norm_w, float * out_partial) {
        tc_used = true;
        const int bn = tcgen05_tile(n, w.rows);
        if (scale == nullptr && res == nullptr) {
            check(k.gemm_tcgen05(x, w.ptr, out, out_dtype, n, w.rows, w.cols, epilogue, bn, tc_status, stream), "gemm_tcgen05");
            return;
        }
        check(k.gemm_tcgen05_fused(x, w.ptr, out, out_dtype, n, w.rows, w.cols, res != nullptr ? 2 : epilogue, bn, tc_status,
                                   scale ? scale->partials : nullptr, scale ? scale->parts : 0,
                                   scale ? 1.0f / (float) scale->width : 0.0f, scale ? scale->eps : 0.0f,
                                   res, norm_w, out_partial, stream), "gemm_tcgen05");
    }
    bool library_gemm(const void * x, const MatrixDesc & w, void * out, int out_dtype, int n) {
        // out[n, m] (row-major) = x[n, k] w[m, k]^T; in column-major terms out^T[m, n] = w (as [k, m], transposed) x^T
        if (blas == nullptr) {
            if (cublasCreate(&blas) != CUBLAS_STATUS_SUCCESS) fail("cublasCreate failed");
            cuda_ok(cudaMalloc(&blas_ws, (size_t) 32 << 20), "cudaMalloc (library workspace)");
            cublasSetWorkspace(blas, blas_ws, (size_t) 32 << 20);
        }
        cublasSetStream(blas, stream);
        const float one = 1.0f, zero = 0.0f;
        const cudaDataType_t ct = out_dtype == DT_BF16 ? CUDA_R_16BF : CUDA_R_32F;
        const cublasStatus_t st = cublasGemmEx(blas, CUBLAS_OP_T, CUBLAS_OP_N, w.rows, n, w.cols, &one, w.ptr, CUDA_R_16BF, w.cols,
                                               x, CUDA_R_16BF, w.cols, &zero, out, ct, w.rows, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
        if (st != CUBLAS_STATUS_SUCCESS) return false;
        by_entry["library_gemm"]++;
        return true;
    }
    // out[n, m] = x . w^T, with the fused forms when asked for (scale: rows lack a folded norm's factor; res / norm_w /
    // out_partial: add to the residual and prepare the next norm)
    void linear(const void * x, int x_dtype, const MatrixDesc & w, void * out, int out_dtype, int n, const Rows * scale = nullptr,
                float * res = nullptr, const float * norm_w = nullptr, float * out_partial = nullptr) {
        if (n == 0) return;
        if (scale != nullptr || res != nullptr) {
            if (tcgen05_ok(x, x_dtype, w, n)) gemm_tcgen05(x, w, out, out_dtype, n, 0, scale, res, norm_w, out_partial);
            else gemm_skinny_fused(x, w, out, out_dtype, n, res != nullptr ? 2 : 0, scale, res, norm_w, out_partial);
            return;
        }
        if (x_dtype == DT_BF16 && w.dtype == DT_BF16) {
            if (tcgen05_ok(x, x_dtype, w, n)) { gemm_tcgen05(x, w, out, out_dtype, n, 0, nullptr, nullptr, nullptr, nullptr); return; }
            if (n <= 8 && w.cols % 32 == 0 && aligned16(x) && aligned16(w.ptr)) {
                before_stream_product();
                plain_stream_product(x, w, out, out_dtype, n, 0);
                after_stream_product(w);
                return;
            }
            if (n > 8 && library_gemm(x, w, out, out_dtype, n)) return;
        }
        check(k.gemm_simt(x, x_dtype, w.ptr, w.dtype, out, out_dtype, n, w.rows, w.cols, stream), "gemm_simt");
    }
    bool can_fuse_swiglu(const void * x, const MatrixDesc & w, int n, int interleave) const {
        return interleave == 8 && w.rows % 16 == 0 && (tcgen05_ok(x, act_dtype, w, n) || skinny_ok(x, act_dtype, w, n));
    }
    void linear_swiglu(const void * x, const MatrixDesc & w, void * out, int n, const Rows * scale) {
        if (scale != nullptr) {
            if (tcgen05_ok(x, act_dtype, w, n)) gemm_tcgen05(x, w, out, act_dtype, n, 1, scale, nullptr, nullptr, nullptr);
            else gemm_skinny_fused(x, w, out, act_dtype, n, 1, scale, nullptr, nullptr, nullptr);
            return;
        }
        if (tcgen05_ok(x, act_dtype, w, n)) { gemm_tcgen05(x, w, out, act_dtype, n, 1, nullptr, nullptr, nullptr, nullptr); return; }
        before_stream_product();
        plain_stream_product(x, w, out, act_dtype, n, 1);
        after_stream_product(w);
    }

    // ---- attention --------------------------------------------------------------------------------------------
    float * scratch_for(size_t floats) {
        if (attn_scratch_floats < floats) {
            if (attn_scratch) retired_scratch.push_back(attn_scratch);       // a captured graph may still point at it
            attn_scratch_floats = std::max<size_t>(floats, (size_t) 1 << 20);
            cuda_ok(cudaMalloc(reinterpret_cast<void **>(&attn_scratch), attn_scratch_floats * sizeof(float)), "cudaMalloc (attention scratch)");
        }
        return attn_scratch;
    }
    int * counters_for(size_t n) {
        if (attn_counters_n < n) {
            if (attn_counters) retired_scratch.push_back(attn_counters);
            attn_counters_n = std::max<size_t>(n, (size_t) 1 << 16);
            cuda_ok(cudaMalloc(reinterpret_cast<void **>(&attn_counters), attn_counters_n * sizeof(int)), "cudaMalloc (attention counters)");
            cuda_ok(cudaMemset(attn_counters, 0, attn_counters_n * sizeof(int)), "cudaMemset");
        }
        return attn_counters;
    }
    // The decode kernel's TMA form reports a wait that gave up in the status words the tcgen05 kernels use; without
    // them it copies with cp.async.
    int * decode_status() {
        if (!opt.decode_tma) return nullptr;
        tc_used = true;
        return tc_status;
    }
    void paged_attention(const void * q, const CallDesc & c, const LayerDesc & L, void * out, const StepInts & si) {
        const int g = c.group, nh = L.num_heads, nkv = L.num_kv_heads, hd = L.head_dim, ps = model.page_size;
        const int * bt = si.block_table[g];
        const int mb = si.max_blocks[g];
        const bool pow2_page = ps == 8 || ps == 16 || ps == 32 || ps == 64 || ps == 128;
        if (opt.attention_tc && bf16_mode() && hd == 128 && pow2_page && nkv > 0 && nh % nkv == 0 && si.max_q_len * (nh / nkv) >= 64) {
            tc_used = true;
            const int Sd = si.decode_seqs;
            if (Sd > 0 && opt.split_mixed && nh / nkv <= 16) {
                // A mixed step: the single decoded tokens (the first Sd sequences) go to the decode kernel, which reads
                // their K/V at the memory's rate, on a second stream, while the portions of prompts run on the tensor
                // cores beside it; in the prefill kernel a decoded token would be a CTA of 256 rows with one token's
                // heads in it, walking its sequence's keys alone.
                if (mixed_stream == nullptr) {
                    cuda_ok(cudaStreamCreateWithFlags(&mixed_stream, cudaStreamNonBlocking), "cudaStreamCreate");
                    cuda_ok(cudaEventCreateWithFlags(&mixed_fork, cudaEventDisableTiming), "cudaEventCreate");
                    cuda_ok(cudaEventCreateWithFlags(&mixed_join, cudaEventDisableTiming), "cudaEventCreate");
                }
                cuda_ok(cudaEventRecord(mixed_fork, stream), "cudaEventRecord");
                cuda_ok(cudaStreamWaitEvent(mixed_stream, mixed_fork, 0), "cudaStreamWaitEvent");
                const int n_split = attention_splits(Sd, nkv, si.decode_max_ctx);
                const bool cluster = opt.cluster_merge && (n_split == 2 || n_split == 4 || n_split == 8 || n_split == 16);
                float * part_o = nullptr, * part_lse = nullptr;
                int * counters = nullptr;
                if (n_split > 1 && !cluster) {
                    const size_t rows = (size_t) Sd * nh;
                    part_o = scratch_for(rows * n_split * (hd + 1));
                    part_lse = part_o + rows * n_split * hd;
                    counters = counters_for((size_t) Sd * nkv);
                }
                check(k.attention_mma(q, c.k_cache, c.v_cache, out, part_o, part_lse, counters, si.cu_q, si.ctx_len, bt, mb, Sd, Sd, 1,
                                      nh, nkv, hd, ps, c.num_pages, L.scale, L.window, n_split, cluster ? 2 : 1, decode_status(),
                                      mixed_stream), "attention_mma");
                check(k.attention_tc(q, c.k_cache, c.v_cache, out, si.cu_q + Sd, si.ctx_len + Sd, bt + (size_t) Sd * mb, mb, si.N,
                                     si.S - Sd, si.max_q_len, nh, nkv, hd, ps, c.num_pages, L.scale, L.window, tc_status, stream),
                      "attention_tc");
                cuda_ok(cudaEventRecord(mixed_join, mixed_stream), "cudaEventRecord");
                cuda_ok(cudaStreamWaitEvent(stream, mixed_join, 0), "cudaStreamWaitEvent");
                return;
            }
            check(k.attention_tc(q, c.k_cache, c.v_cache, out, si.cu_q, si.ctx_len, bt, mb, si.N, si.S, si.max_q_len, nh, nkv, hd, ps,
                                 c.num_pages, L.scale, L.window, tc_status, stream), "attention_tc");
            return;
        }
        if (bf16_mode() && (hd == 64 || hd == 128)) {
            const bool decode = si.max_q_len * (nh / nkv) <= 16;
            const bool small_tiles = decode;
            int n_split = si.n_split > 0 ? si.n_split : (decode ? attention_splits(si.S, nkv, si.max_ctx) : 1);
            const bool cluster = opt.cluster_merge && small_tiles && (n_split == 2 || n_split == 4 || n_split == 8 || n_split == 16);
            float * part_o = nullptr, * part_lse = nullptr;
            int * counters = nullptr;
            if (n_split > 1 && !cluster) {
                const size_t rows = (size_t) si.N * nh;
                part_o = scratch_for(rows * n_split * (hd + 1));
                part_lse = part_o + rows * n_split * hd;
                if (small_tiles) {
                    const int row_tiles = (si.max_q_len * (nh / nkv) + 15) / 16;
                    counters = counters_for((size_t) si.S * nkv * row_tiles);
                }
            }
            check(k.attention_mma(q, c.k_cache, c.v_cache, out, part_o, part_lse, counters, si.cu_q, si.ctx_len, bt, mb, si.N, si.S,
                                  si.max_q_len, nh, nkv, hd, ps, c.num_pages, L.scale, L.window, n_split,
                                  small_tiles ? (cluster ? 2 : 1) : 0, decode_status(), stream), "attention_mma");
            if (n_split > 1 && !small_tiles) launches++;
            return;
        }
        check(k.attention_generic(q, c.k_cache, c.v_cache, out, si.positions, si.seq_of_token, bt, mb, si.ctx_len, act_dtype, si.N, nh, nkv,
                                  hd, ps, c.num_pages, L.scale, L.window, stream), "paged_attention_generic");
    }
    const void * rotary_table(const LayerDesc & L, const StepInts & si) {
        auto it = rotary_tables.find(L.rope_key);
        if (it != rotary_tables.end()) return it->second;
        const int half = L.rot_dim / 2;
        const std::string name = "rotary_table_" + std::to_string(rotary_tables.size());
        void * t = cur_ws->get(name, (size_t) si.N * half * 2 * sizeof(float));
        check(k.rotary_table(L.inv_freq, si.positions, t, si.N, half, stream), "rotary_table");
        rotary_tables[L.rope_key] = t;
        return t;
    }

    // ---- parts -------------------------------------------------------------------------------------------------
    void * add_rms_norm(float * residual, const void * delta, const float * w, float eps, int n) {
        void * out = buf("normed", (size_t) n * model.hidden * act_size);
        check(k.add_rms_norm(residual, delta, w, out, act_dtype, n, model.hidden, eps, stream), "add_rms_norm");
        return out;
    }
    // the product that ends a sub-layer, asked to add to the residual and prepare `norm_w`'s input
    Rows take_norm_out(const void * x, const MatrixDesc & w, int n, float * residual, const float * norm_w, float eps, const char * name) {
        Rows r;
        r.prenormed = true;
        r.width = w.rows;
        r.eps = eps;
        r.for_norm = norm_w;
        r.parts = norm_parts(w, n);
        r.x = buf((std::string("prenormed_") + name).c_str(), (size_t) n * w.rows * act_size);
        float * partials = static_cast<float *>(buf((std::string("norm_partials_") + name).c_str(), (size_t) n * r.parts * sizeof(float)));
        r.partials = partials;
        linear(x, act_dtype, w, r.x, act_dtype, n, nullptr, residual, norm_w, partials);
        return r;
    }
    Rows attention(const Rows & h, const CallDesc & c, const LayerDesc & L, const StepInts & si, float * residual,
                   const float * out_norm_w, float out_norm_eps) {
        const int n = si.N, nh = L.num_heads, hd = L.head_dim;
        const int q_size = nh * hd;
        const int nkv = c.writes_cache ? L.num_kv_heads : 0;
        MatrixDesc w = L.w_qkv;
        const float * bias = L.b_qkv;
        const int width = q_size + 2 * nkv * hd;
        w.rows = width;                                   // a call that reads another call's cache projects Q only
        void * qkv = buf("qkv", (size_t) n * width * act_size);
        linear(h.x, act_dtype, w, qkv, act_dtype, n, h.prenormed ? &h : nullptr);
        void * attn = buf("attn", (size_t) n * q_size * act_size);
        const int rot_dim = L.inv_freq != nullptr ? L.rot_dim : 0;
        const void * table = L.inv_freq != nullptr ? rotary_table(L, si) : nullptr;
        const int g = c.group;
        const bool fuse = c.writes_cache && opt.fused_decode && si.decode_only && si.N == si.S && bf16_mode() && (hd == 64 || hd == 128) &&
                          bias == nullptr && (rot_dim == 0 || rot_dim == hd) && (L.rope_style == 0 || rot_dim == 0) &&
                          L.num_kv_heads > 0 && nh % L.num_kv_heads == 0 && nh / L.num_kv_heads <= 16 && (rot_dim == 0 || table != nullptr);
        if (fuse) {
            int n_split = si.n_split > 0 ? si.n_split : attention_splits(si.S, L.num_kv_heads, si.max_ctx);
            const bool cluster = opt.cluster_merge && n_split >= 2 && n_split <= 16;
            float * part_o = nullptr, * part_lse = nullptr;
            int * counters = nullptr;
            if (n_split > 1 && !cluster) {
                const size_t rows = (size_t) si.S * nh;
                part_o = scratch_for(rows * n_split * (hd + 1));
                part_lse = part_o + rows * n_split * hd;
                counters = counters_for((size_t) si.S * L.num_kv_heads);
            }
            check(k.attention_decode_fused(qkv, c.k_cache, c.v_cache, attn, part_o, part_lse, counters, si.cu_q, si.ctx_len,
                                           si.block_table[g], si.max_blocks[g], si.S, nh, L.num_kv_heads, hd, model.page_size, c.num_pages,
                                           L.scale, L.window, n_split, cluster ? 1 : 0, L.q_norm_w, L.k_norm_w,
                                           rot_dim ? static_cast<const float *>(table) : nullptr, si.slots[g], L.qk_norm_eps, 1,
                                           decode_status(), stream),
                  "attention_decode_fused");
        } else {
            void * q = buf("q", (size_t) n * q_size * act_size);
            check(k.qk_norm_rope_store(qkv, bias, q, c.writes_cache ? c.k_cache : nullptr, c.writes_cache ? c.v_cache : nullptr,
                                       L.q_norm_w, L.k_norm_w, L.inv_freq, table, si.positions, c.writes_cache ? si.slots[g] : nullptr,
                                       act_dtype, n, nh, nkv, hd, rot_dim, L.rope_style, L.qk_norm_eps,
                                       c.writes_cache ? model.page_size : 0, c.writes_cache ? c.num_pages : 0, c.writes_cache ? 1 : 0, stream),
                  "qk_norm_rope_store");
            paged_attention(q, c, L, attn, si);
        }
        if (out_norm_w != nullptr && L.b_o == nullptr && can_fuse_norm(attn, L.w_o, n))
            return take_norm_out(attn, L.w_o, n, residual, out_norm_w, out_norm_eps, "mixer");
        Rows r;
        r.x = buf("mixer_out", (size_t) n * model.hidden * act_size);
        linear(attn, act_dtype, L.w_o, r.x, act_dtype, n);
        if (L.b_o != nullptr) check(k.add_bias(r.x, L.b_o, act_dtype, n, model.hidden, stream), "add_bias");
        return r;
    }
    Rows feed_forward(const Rows & h, const LayerDesc & L, int n, float * residual, const float * out_norm_w, float out_norm_eps) {
        void * act = buf("ffn_act", (size_t) n * L.intermediate * act_size);
        if (h.prenormed) linear_swiglu(h.x, L.w_gate_up, act, n, &h);
        else if (can_fuse_swiglu(h.x, L.w_gate_up, n, L.interleave)) linear_swiglu(h.x, L.w_gate_up, act, n, nullptr);
        else {
            void * gate_up = buf("gate_up", (size_t) n * 2 * L.intermediate * act_size);
            linear(h.x, act_dtype, L.w_gate_up, gate_up, act_dtype, n);
            check(k.swiglu(gate_up, act, act_dtype, n, L.intermediate, L.interleave, stream), "swiglu");
        }
        if (out_norm_w != nullptr && can_fuse_norm(act, L.w_down, n))
            return take_norm_out(act, L.w_down, n, residual, out_norm_w, out_norm_eps, "feed_forward");
        Rows r;
        r.x = buf("ffn_out", (size_t) n * model.hidden * act_size);
        linear(act, act_dtype, L.w_down, r.x, act_dtype, n);
        return r;
    }

    // ---- the forward pass (iian_b200/engine/model.py: embedding, run order, final norm, head) ---------------------
    const float * forward(const StepInts & si) {
        rotary_tables.clear();
        const int H = model.hidden;
        float * residual = static_cast<float *>(buf("residual", (size_t) si.N * H * sizeof(float)));
        check(k.embedding(model.embedding.ptr, model.embedding.dtype, si.tokens, residual, si.N, H, model.embedding.rows, stream), "embedding");
        Rows delta;                                            // nothing to add yet
        int n = si.N;
        const size_t n_calls = model.calls.size();
        for (size_t idx = 0; idx < n_calls; idx++) {
            const CallDesc & c = model.calls[idx];
            const LayerDesc & L = model.layers[c.layer];
            const bool last = idx + 1 == n_calls;
            Rows h;
            if (delta.prenormed) {
                if (delta.for_norm != L.mixer_norm_w) fail("block: received rows prepared for another norm");
                h = delta;
            } else {
                h.x = add_rms_norm(residual, delta.x, L.mixer_norm_w, L.mixer_norm_eps, n);
            }
            const bool gathers = last && !si.rows_identity;
            const bool fold_ffn_norm = !gathers && L.interleave == 8 && can_take_prenormed(n, L.w_gate_up);
            Rows y = attention(h, c, L, si, residual, fold_ffn_norm ? L.ffn_norm_w : nullptr, L.ffn_norm_eps);
            if (gathers) {
                float * res_sel = static_cast<float *>(buf("residual_rows", (size_t) si.R * H * sizeof(float)));
                void * y_sel = buf("mixer_out_rows", (size_t) si.R * H * act_size);
                check(k.gather_rows(residual, si.out_rows, res_sel, DT_F32, si.R, H, n, stream), "gather_rows");
                check(k.gather_rows(y.x, si.out_rows, y_sel, act_dtype, si.R, H, n, stream), "gather_rows");
                residual = res_sel;
                y.x = y_sel;
                n = si.R;
            }
            Rows h2;
            if (y.prenormed) h2 = y;
            else h2.x = add_rms_norm(residual, y.x, L.ffn_norm_w, L.ffn_norm_eps, n);
            const float * next_w = nullptr;
            float next_eps = 0.0f;
            if (!last) {
                const LayerDesc & nx = model.layers[model.calls[idx + 1].layer];
                if (can_take_prenormed(n, nx.w_qkv)) { next_w = nx.mixer_norm_w; next_eps = nx.mixer_norm_eps; }
            }
            delta = feed_forward(h2, L, n, residual, next_w, next_eps);
        }
        if (n_calls == 0 && !si.rows_identity) {
            float * sel = static_cast<float *>(buf("residual_rows", (size_t) si.R * H * sizeof(float)));
            check(k.gather_rows(residual, si.out_rows, sel, DT_F32, si.R, H, n, stream), "gather_rows");
            residual = sel;
            n = si.R;
        } else if (n_calls == 0) {
            n = si.R;
        }
        if (si.R == 0) return nullptr;
        void * normed = add_rms_norm(residual, delta.x, model.final_norm_w, model.final_norm_eps, n);
        float * logits = static_cast<float *>(buf("logits", (size_t) n * model.vocab * sizeof(float)));
        linear(normed, act_dtype, model.head, logits, DT_F32, n);
        return logits;
    }

    // ---- the step's integers (iian_b200/engine/runner.py: build_context) ----------------------------------------
    void pack(const StepBatch & batch, Staging & st, StepInts & si, GraphSlot * slot) {
        const int bs = cache->block_size(), G = cache->num_groups();
        const int n_real = (int) batch.entries.size();
        int S, N, R;
        std::vector<int> max_blocks(G, 1);
        if (slot == nullptr) {
            S = n_real; N = 0; R = 0;
            for (const auto & e : batch.entries) {
                if (e.n_tokens <= 0) throw std::invalid_argument("a step entry must bring at least one token");
                N += e.n_tokens;
                R += e.n_want;
                for (int g = 0; g < G; g++) max_blocks[g] = std::max(max_blocks[g], cache->blocks_for(e.start + e.n_tokens));
            }
        } else {
            S = N = R = slot->num_seqs;
            for (int g = 0; g < G; g++) max_blocks[g] = slot->max_blocks;
        }
        size_t total = (size_t) 3 * N + (S + 1) + 2 * S + R;
        for (int g = 0; g < G; g++) total += (size_t) N + (size_t) S * max_blocks[g];
        st.reserve(total);
        st.wait();
        int32_t * host = st.host;
        size_t off = 0;
        auto take = [&](size_t count) { const size_t at = off; off += count; return at; };
        const size_t o_tok = take(N), o_pos = take(N), o_seq = take(N), o_cu = take(S + 1), o_ctx = take(S), o_state = take(S), o_rows = take(R);
        std::vector<size_t> o_slots(G), o_bt(G);
        for (int g = 0; g < G; g++) o_slots[g] = take(N);
        for (int g = 0; g < G; g++) o_bt[g] = take((size_t) S * max_blocks[g]);
        if (slot != nullptr) {                                    // padding first; real sequences overwrite the front
            for (int i = 0; i < N; i++) { host[o_tok + i] = 0; host[o_pos + i] = 0; host[o_seq + i] = -1; }
            for (int s = 0; s <= S; s++) host[o_cu + s] = s;
            for (int s = 0; s < S; s++) { host[o_ctx + s] = 1; host[o_state + s] = -1; host[o_rows + s] = s; }
            for (int g = 0; g < G; g++) {
                for (int i = 0; i < N; i++) host[o_slots[g] + i] = -1;
                for (size_t i = 0; i < (size_t) S * max_blocks[g]; i++) host[o_bt[g] + i] = 0;
            }
        }
        // The sequences of a step are laid out with the single decoded tokens first (in their given order), the
        // portions of prompts after them, so that attention can give each kind to its kernel; the wanted rows keep
        // the order of the entries as given.
        std::vector<int> order(n_real), row_base(n_real + 1, 0);
        int n_single = 0;
        for (int i = 0; i < n_real; i++) {
            row_base[i + 1] = row_base[i] + batch.entries[i].n_want;
            if (batch.entries[i].n_tokens == 1) n_single++;
        }
        const bool mixed = slot == nullptr && n_single > 0 && n_single < n_real;
        {
            int a = 0, b = mixed ? n_single : 0;
            for (int i = 0; i < n_real; i++) {
                if (!mixed) order[i] = i;
                else if (batch.entries[i].n_tokens == 1) order[a++] = i;
                else order[b++] = i;
            }
        }
        int t0 = 0, max_q = 0, max_ctx = 0, decode_max_ctx = 0;
        host[o_cu] = 0;
        for (int s = 0; s < n_real; s++) {
            const StepEntry & e = batch.entries[order[s]];
            int r = row_base[order[s]];
            const int n = e.n_tokens;
            for (int i = 0; i < n; i++) {
                host[o_tok + t0 + i] = e.tokens[i];
                host[o_pos + t0 + i] = e.start + i;
                host[o_seq + t0 + i] = s;
            }
            host[o_cu + s + 1] = t0 + n;
            host[o_ctx + s] = e.start + n;
            host[o_state + s] = e.cache->state_slot;
            e.cache->state_fresh = false;       // no mixer of a native model keeps state of its own: nothing to zero
            if (slot == nullptr) {
                for (int i = 0; i < e.n_want; i++) {
                    const int w = e.want[i];
                    if (w < 0 || w >= n) throw std::invalid_argument("wanted place " + std::to_string(w) + " is outside this step's " + std::to_string(n) + " tokens");
                    host[o_rows + r++] = t0 + w;
                }
            }
            const int need = cache->blocks_for(e.start + n);
            for (int g = 0; g < G; g++) {
                const auto & table = e.cache->tables[g];
                if ((int) table.size() < need)
                    throw std::invalid_argument("request holds " + std::to_string(table.size()) + " pages in group " + std::to_string(g) + ", needs " + std::to_string(need));
                const int mb = max_blocks[g];
                int32_t * row = host + o_bt[g] + (size_t) s * mb;
                for (int i = 0; i < mb; i++) row[i] = i < need ? table[i] : -1;
                for (int i = 0; i < n; i++) {
                    const int p = e.start + i;
                    const int page = row[p / bs];
                    if (page < 0) throw PoolError("a token of this step lies in a page that was given back");
                    host[o_slots[g] + t0 + i] = page * bs + p % bs;
                }
            }
            max_q = std::max(max_q, n);
            max_ctx = std::max(max_ctx, e.start + n);
            if (mixed && s < n_single) decode_max_ctx = std::max(decode_max_ctx, e.start + n);
            t0 += n;
        }
        bool identity = R == N;                               // every token's logits wanted, in the order of the tokens
        if (slot == nullptr)
            for (int i = 0; identity && i < R; i++) identity = host[o_rows + i] == i;
        st.upload(total, stream);
        const int32_t * dev = st.dev;
        si = StepInts();
        si.N = N; si.S = S; si.R = R;
        si.tokens = dev + o_tok; si.positions = dev + o_pos; si.seq_of_token = dev + o_seq; si.cu_q = dev + o_cu; si.ctx_len = dev + o_ctx;
        si.state_slots = dev + o_state; si.out_rows = dev + o_rows;
        for (int g = 0; g < G; g++) { si.slots.push_back(dev + o_slots[g]); si.block_table.push_back(dev + o_bt[g]); }
        si.max_blocks = max_blocks;
        si.max_q_len = max_q; si.max_ctx = max_ctx;
        if (slot != nullptr) { si.max_q_len = 1; si.max_ctx = slot->ctx_bucket; si.n_split = slot->n_split; }
        si.decode_only = si.max_q_len == 1;
        si.decode_seqs = mixed ? n_single : 0;
        si.decode_max_ctx = decode_max_ctx;
        si.rows_identity = slot != nullptr || identity;
        si.upload_bytes = (int) (total * sizeof(int32_t));
    }

    const float * step_eager(const StepBatch & batch, int * n_rows) {
        StepInts si;
        pack(batch, staging, si, nullptr);
        cur_ws = &ws;
        const float * out = forward(si);
        last_upload = si.upload_bytes;
        *n_rows = si.R;
        return out;
    }

    // ---- decode-only steps replayed from captured graphs (iian_b200/engine/runner.py: _step_graph, _capture) ------
    GraphSlot * capture(int num_seqs, int ctx_bucket, cudaStream_t user_stream) {
        auto slot = std::make_unique<GraphSlot>();
        slot->num_seqs = num_seqs;
        slot->ctx_bucket = ctx_bucket;
        slot->max_blocks = std::max(1, cache->blocks_for(std::max(opt.max_model_len, ctx_bucket)));
        int min_kv = 0;
        for (const auto & c : model.calls) {
            const int nkv = model.layers[c.layer].num_kv_heads;
            min_kv = min_kv == 0 ? nkv : std::min(min_kv, nkv);
        }
        slot->n_split = min_kv > 0 ? attention_splits(num_seqs, min_kv, ctx_bucket) : 1;
        // warm up eagerly on padding sequences only (kernels get loaded, buffers sized, the order of the streamed
        // weights recorded; nothing is stored), then capture the same launches
        StepBatch none;
        stream = user_stream;
        pack(none, slot->staging, slot->ints, slot.get());
        cur_ws = &slot->ws;
        std::vector<std::pair<const void *, size_t>> log;
        const bool prefetch = opt.weight_prefetch && k.prefetch_l2 != nullptr;
        if (prefetch) weight_log = &log;
        try { forward(slot->ints); } catch (...) { weight_log = nullptr; throw; }
        weight_log = nullptr;
        cuda_ok(cudaStreamSynchronize(user_stream), "cudaStreamSynchronize");
        slot->ws.frozen = true;
        if (cap_stream == nullptr) {
            cuda_ok(cudaStreamCreateWithFlags(&cap_stream, cudaStreamNonBlocking), "cudaStreamCreate");
            cuda_ok(cudaStreamCreateWithFlags(&side_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        }
        const long long before = launches;
        Prefetcher pf;
        if (prefetch && !log.empty()) {
            pf.weights = log;
            size_t pos = 0;
            for (const auto & w : log) { pf.starts.push_back(pos); pos += w.second; }
            pf.total = pos;
            pf.window = (size_t) opt.prefetch_window_mb << 20;
            pf.side = side_stream;
        }
        stream = cap_stream;
        cuda_ok(cudaStreamBeginCapture(cap_stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
        bool ok = false;
        try {
            if (!pf.weights.empty()) prefetcher = &pf;
            slot->logits = forward(slot->ints);
            if (prefetcher != nullptr) {                          // the side stream joins before the capture ends
                cudaEvent_t ev;
                cuda_ok(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
                cuda_ok(cudaEventRecord(ev, side_stream), "cudaEventRecord");
                cuda_ok(cudaStreamWaitEvent(cap_stream, ev, 0), "cudaStreamWaitEvent");
                cudaEventDestroy(ev);
            }
            ok = true;
        } catch (...) {
            prefetcher = nullptr;
            cudaGraph_t g = nullptr;
            cudaStreamEndCapture(cap_stream, &g);
            if (g) cudaGraphDestroy(g);
            stream = user_stream;
            throw;
        }
        prefetcher = nullptr;
        cuda_ok(cudaStreamEndCapture(cap_stream, &slot->graph), "cudaStreamEndCapture");
        (void) ok;
        cuda_ok(cudaGraphInstantiate(&slot->exec, slot->graph, 0), "cudaGraphInstantiate");
        slot->launches = launches - before;
        stream = user_stream;
        GraphSlot * raw = slot.get();
        graphs[{num_seqs, ctx_bucket}] = std::move(slot);
        return raw;
    }

    const float * step_graph(const StepBatch & batch, int * n_rows) {
        const int n = (int) batch.entries.size();
        // batches are padded to 1, 2, 4, 8, then to multiples of 4 up to 32, of 8 up to 64, of 16 up to 128 and of 32
        // beyond: padding sequences are CTAs of the attention launch too, and whether those fit the GPU at once decides
        // its form
        int bucket = 1;
        if (n <= 8) { while (bucket < n) bucket *= 2; }
        else { const int step = n <= 32 ? 4 : n <= 64 ? 8 : n <= 128 ? 16 : 32; bucket = (n + step - 1) / step * step; }
        bucket = std::min(bucket, std::max(opt.max_num_seqs, n));
        int max_ctx = 0;
        for (const auto & e : batch.entries) max_ctx = std::max(max_ctx, e.start + 1);
        int ctx_bucket = 256;
        while (ctx_bucket < max_ctx) ctx_bucket *= 2;
        auto it = graphs.find({bucket, ctx_bucket});
        GraphSlot * slot = it != graphs.end() ? it->second.get() : capture(bucket, ctx_bucket, stream);
        const int S = slot->num_seqs, mb = slot->max_blocks, G = cache->num_groups();
        slot->staging.wait();
        if (slot->sig.empty()) slot->sig.assign((size_t) std::max(1, G) * S * 3, 0);
        scratch_caches.resize(n); scratch_tokens.resize(n); scratch_starts.resize(n); scratch_fresh.resize(std::max(n, 1));
        for (int s = 0; s < n; s++) {
            scratch_caches[s] = batch.entries[s].cache;
            scratch_tokens[s] = batch.entries[s].tokens[0];
            scratch_starts[s] = batch.entries[s].start;
        }
        const int n_fresh = iian_pack_decode_step(cache, scratch_caches.data(), scratch_tokens.data(), scratch_starts.data(), n, S, mb,
                                                  slot->staging.host, slot->sig.data(), slot->n_last != n ? 1 : 0, scratch_fresh.data());
        if (n_fresh < 0) { slot->n_last = -1; fail(iian_host_last_error()); }
        slot->n_last = n;
        size_t total = (size_t) 3 * S + (S + 1) + 3 * S + (size_t) G * (S + (size_t) S * mb);
        slot->staging.upload(total, stream);
        cuda_ok(cudaGraphLaunch(slot->exec, stream), "cudaGraphLaunch");
        launches += slot->launches;
        last_upload = (int) (total * sizeof(int32_t));
        *n_rows = n;
        return slot->logits;
    }
};

NativeRunner::NativeRunner(const ModelDesc & model, const KernelLibraries & libs, CacheManager * cache, const RunnerOptions & opt)
    : impl_(new Impl()) {
    Impl & m = *impl_;
    m.model = model;
    m.opt = opt;
    m.cache = cache;
    m.act_dtype = model.dtype;
    m.act_size = model.dtype == DT_BF16 ? 2 : 4;
    if (cache->num_groups() != model.num_groups) fail("the cache manager and the model disagree on the number of page groups");
    if (cache->block_size() != model.page_size) fail("the cache manager and the model disagree on the page size");
    int dev = 0;
    cuda_ok(cudaGetDevice(&dev), "cudaGetDevice");
    if (cudaDeviceGetAttribute(&m.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || m.sm_count <= 0) m.sm_count = 148;
    auto open = [&](const std::string & path) -> void * {
        if (path.empty()) return nullptr;
        void * h = open_library(path);
        m.libs.push_back(h);
        return h;
    };
    Kernels & k = m.k;
    if (void * h = open(libs.elementwise)) {
        bind(h, "iian_embedding", k.embedding, libs.elementwise);
        bind(h, "iian_add_rms_norm", k.add_rms_norm, libs.elementwise);
        bind(h, "iian_swiglu", k.swiglu, libs.elementwise);
        bind(h, "iian_gather_rows", k.gather_rows, libs.elementwise);
        bind(h, "iian_add_bias", k.add_bias, libs.elementwise);
    } else fail("the elementwise kernel library is required");
    if (void * h = open(libs.rope_kv)) {
        bind(h, "iian_rotary_table", k.rotary_table, libs.rope_kv);
        bind(h, "iian_qk_norm_rope_store", k.qk_norm_rope_store, libs.rope_kv);
    } else fail("the rope_kv kernel library is required");
    if (void * h = open(libs.attention_generic)) bind(h, "iian_paged_attention_generic", k.attention_generic, libs.attention_generic);
    else fail("the attention_generic kernel library is required");
    if (void * h = open(libs.gemm_simt)) bind(h, "iian_gemm_simt", k.gemm_simt, libs.gemm_simt);
    else fail("the gemm_simt kernel library is required");
    if (model.dtype == DT_BF16) {
        if (void * h = open(libs.gemm_skinny)) {
            bind(h, "iian_gemm_skinny_cfg", k.gemm_skinny_cfg, libs.gemm_skinny);
            bind(h, "iian_gemm_skinny_fused", k.gemm_skinny_fused, libs.gemm_skinny);
        } else fail("the gemm_skinny kernel library is required for bfloat16");
        if (void * h = open(libs.gemm_tcgen05)) {
            bind(h, "iian_gemm_tcgen05", k.gemm_tcgen05, libs.gemm_tcgen05);
            bind(h, "iian_gemm_tcgen05_fused", k.gemm_tcgen05_fused, libs.gemm_tcgen05);
        } else fail("the gemm_tcgen05 kernel library is required for bfloat16");
        if (void * h = open(libs.attention_tc)) bind(h, "iian_attention_tc", k.attention_tc, libs.attention_tc);
        else fail("the attention_tc kernel library is required for bfloat16");
        if (void * h = open(libs.attention_mma)) {
            bind(h, "iian_attention_mma", k.attention_mma, libs.attention_mma);
            bind(h, "iian_attention_decode_fused", k.attention_decode_fused, libs.attention_mma);
            bind(h, "iian_attention_decode_stages", k.attention_decode_stages, libs.attention_mma);
            if (k.attention_decode_stages(opt.decode_stages) != 0) fail("attention: the decode kernel has 2 or 3 stages");
        } else fail("the attention_mma kernel library is required for bfloat16");
        if (void * h = open(libs.prefetch)) bind(h, "iian_prefetch_l2", k.prefetch_l2, libs.prefetch);
        if (void * h = open(libs.gemm_stream)) {
            bind(h, "iian_gemm_stream", k.gemm_stream, libs.gemm_stream);
            bind(h, "iian_gemm_stream_stages", k.gemm_stream_stages, libs.gemm_stream);
            if (k.gemm_stream_stages(opt.stream_stages) != 0) fail("gemm_stream: the ring is chosen by 6 or 12");
            void (*set_pdl)(int) = nullptr;
            bind(h, "iian_set_pdl", set_pdl, libs.gemm_stream);
            set_pdl(opt.pdl_stream ? 1 : 0);
        } else if (opt.stream_product) fail("the gemm_stream kernel library is required for bfloat16");
        cuda_ok(cudaMalloc(reinterpret_cast<void **>(&m.tc_status), 2 * sizeof(int)), "cudaMalloc (status)");
        cuda_ok(cudaMemset(m.tc_status, 0, 2 * sizeof(int)), "cudaMemset");
    }
}

NativeRunner::~NativeRunner() {
    Impl & m = *impl_;
    cudaDeviceSynchronize();
    m.graphs.clear();
    if (m.blas) cublasDestroy(m.blas);
    if (m.blas_ws) cudaFree(m.blas_ws);
    if (m.tc_status) cudaFree(m.tc_status);
    if (m.attn_scratch) cudaFree(m.attn_scratch);
    if (m.attn_counters) cudaFree(m.attn_counters);
    for (void * p : m.retired_scratch) cudaFree(p);
    if (m.cap_stream) cudaStreamDestroy(m.cap_stream);
    if (m.mixed_stream) { cudaStreamDestroy(m.mixed_stream); cudaEventDestroy(m.mixed_fork); cudaEventDestroy(m.mixed_join); }
    if (m.side_stream) cudaStreamDestroy(m.side_stream);
    for (void * h : m.libs) dlclose(h);
}

const float * NativeRunner::step(const StepBatch & batch, void * stream, int * n_rows) {
    Impl & m = *impl_;
    *n_rows = 0;
    if (batch.entries.empty()) return nullptr;
    if ((int) batch.entries.size() > m.opt.max_num_seqs)
        throw std::invalid_argument(std::to_string(batch.entries.size()) + " requests in one step, the runner was built for " + std::to_string(m.opt.max_num_seqs));
    m.stream = static_cast<cudaStream_t>(stream);
    bool decode = m.opt.cuda_graphs;
    if (decode)
        for (const auto & e : batch.entries)
            if (e.n_tokens != 1 || e.n_want != 1 || e.want[0] != 0) { decode = false; break; }
    return decode ? m.step_graph(batch, n_rows) : m.step_eager(batch, n_rows);
}

int NativeRunner::vocab() const { return impl_->model.vocab; }
long long NativeRunner::launches() const { return impl_->launches; }
int NativeRunner::num_graphs() const { return (int) impl_->graphs.size(); }
int NativeRunner::last_upload_bytes() const { return impl_->last_upload; }
long long NativeRunner::launches_of(const char * entry) const {
    auto it = impl_->by_entry.find(entry);
    return it == impl_->by_entry.end() ? 0 : it->second;
}

void NativeRunner::set_cuda_graphs(bool on) { impl_->opt.cuda_graphs = on; }

void NativeRunner::check_status() {
    Impl & m = *impl_;
    if (!m.tc_used || m.tc_status == nullptr) return;
    m.tc_used = false;
    int host[2] = {0, 0};
    cuda_ok(cudaMemcpy(host, m.tc_status, sizeof(host), cudaMemcpyDeviceToHost), "cudaMemcpy (status)");
    if (host[0] != 0) {
        cudaMemset(m.tc_status, 0, sizeof(host));
        fail("a kernel gave up waiting on a barrier (wait " + std::to_string(host[0]) + ", iteration " + std::to_string(host[1]) + "); its result is not valid");
    }
}

}  // namespace iian_b200
