// Sampling over float32 logits rows on the device: greedy argmax and temperature sampling with
// min-p, top-k and top-p truncation.
//
// Semantics follow the reference's CPU sampler (src/iian/sampler.cpp:111-171):
//  * temperature < 1e-5 -> greedy; ties resolve to the lowest id (src/iian/vec_math.h:78-82);
//  * else z = logit / T; min_p keeps z >= max(z) + log(min_p) (:122-126); top_k keeps the k largest
//    with (value desc, id asc) order, only if k is smaller than the candidate count (:131-134);
//    probabilities are exp(z - max) normalised over the candidates (:139-156); top_p keeps the
//    shortest prefix in that order whose mass reaches top_p (:158-163); a uniform draw over the kept
//    mass picks the token by walking the candidates and subtracting (:165-171).
// Differences: the walk is in vocabulary order for every setting (the reference walks in sorted
// order when it sorted), and the uniform number comes from the caller (a counter-based stream per
// request) instead of a per-request mt19937_64.  The distribution is the same.
//
// One block per row.  The k-th largest value and the top-p cut are found exactly by bisection over
// the order-preserving integer image of the float values (32 counting passes over the row, which
// stays in L2).
#include "common.cuh"

namespace iian {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned order_key(float f) {
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ int block_sum_int(int v, int * scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int t = lane < (blockDim.x >> 5) ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// (max value, lowest index holding it) over a row
__device__ __forceinline__ void block_argmax(const float * row, int V, float scale, float & best, int & best_idx,
                                             float * fs, int * is) {
    float b = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i] * scale;
        if (v > b || (v == b && i < bi)) { b = v; bi = i; }   // NaN compares false: treated as smaller
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, b, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { fs[warp] = b; is[warp] = bi; }
    __syncthreads();
    b = lane < (blockDim.x >> 5) ? fs[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? is[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, b, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
    }
    best = b;
    best_idx = bi == 0x7fffffff ? 0 : bi;
}

__global__ void __launch_bounds__(kSampleThreads) argmax_kernel(const float * __restrict__ logits, int V, size_t stride,
                                                                int * __restrict__ out) {
    __shared__ float fs[32];
    __shared__ int is[32];
    float b; int bi;
    block_argmax(logits + (size_t) blockIdx.x * stride, V, 1.0f, b, bi, fs, is);
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
}

// Two-stage argmax for wide rows: `parts` blocks per row each reduce a contiguous slice to (value, id),
// a second launch reduces the parts.  Ties still go to the lowest id.
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float * __restrict__ logits, int V, size_t stride,
                                                             int parts, float * __restrict__ part_val,
                                                             int * __restrict__ part_idx) {
    __shared__ float fs[32];
    __shared__ int is[32];
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.y, part = blockIdx.x;
    const int per = (V + parts - 1) / parts;
    const int begin = min(V, part * per), end = min(V, begin + per);
    const float * r = logits + (size_t) row * stride;
    float b = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = r[i];
        if (v > b || (v == b && i < bi)) { b = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, b, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { fs[warp] = b; is[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        b = lane < (blockDim.x >> 5) ? fs[lane] : -INFINITY;
        bi = lane < (blockDim.x >> 5) ? is[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, b, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
        }
        if (lane == 0) { part_val[(size_t) row * parts + part] = b; part_idx[(size_t) row * parts + part] = bi; }
    }
}

__global__ void argmax_final_kernel(const float * __restrict__ part_val, const int * __restrict__ part_idx, int parts,
                                    int * __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x, lane = threadIdx.x;       // one warp per row
    float b = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lane; i < parts; i += 32) {
        const float v = part_val[(size_t) row * parts + i];
        const int idx = part_idx[(size_t) row * parts + i];
        if (v > b || (v == b && idx < bi)) { b = v; bi = idx; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, b, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(
    const float * __restrict__ logits, int V, size_t stride,
    const float * __restrict__ temperature, const int * __restrict__ top_k, const float * __restrict__ top_p,
    const float * __restrict__ min_p, const float * __restrict__ uniform, int * __restrict__ out) {
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ float chunk_mass[kSampleThreads];
    __shared__ int chunk_ties[kSampleThreads];
    __shared__ int pick_thread;
    __shared__ float pick_before;
    __shared__ int pick_ties_before;

    const float * row = logits + (size_t) blockIdx.x * stride;
    const float T = temperature[blockIdx.x];
    if (T < 1e-5f) {
        float b; int bi;
        block_argmax(row, V, 1.0f, b, bi, fs, is);
        if (threadIdx.x == 0) out[blockIdx.x] = bi;
        return;
    }
    const float inv_t = 1.0f / T;
    float zmax; int imax;
    block_argmax(row, V, inv_t, zmax, imax, fs, is);

    // candidate set: key > cut, plus the first n_tie elements (by id) with key == cut
    unsigned cut = 0u;                 // 0 is below every finite or infinite value's key
    int n_tie = 0x7fffffff;
    const float mp = min_p[blockIdx.x];
    if (mp > 0.0f) cut = order_key(zmax + logf(mp)), n_tie = 0x7fffffff;
    // keys >= cut are candidates; express "all ties" as n_tie = INT_MAX

    int count = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) count += order_key(row[i] * inv_t) >= cut;
    count = block_sum_int(count, is);

    const int k = top_k[blockIdx.x];
    if (k > 0 && k < count) {
        unsigned K = 0u;
        for (int bit = 31; bit >= 0; bit--) {
            const unsigned trial = K | (1u << bit);
            int c = 0;
            for (int i = threadIdx.x; i < V; i += blockDim.x) c += order_key(row[i] * inv_t) >= trial;
            c = block_sum_int(c, is);
            if (c >= k) K = trial;
        }
        int gt = 0;
        for (int i = threadIdx.x; i < V; i += blockDim.x) gt += order_key(row[i] * inv_t) > K;
        gt = block_sum_int(gt, is);
        cut = K;
        n_tie = k - gt;
    }

    const float P = top_p[blockIdx.x];
    if (P < 1.0f) {
        // mass of the current set; ties at `cut` all have the same value, so only their count matters
        float mass_gt = 0.0f;
        int ties = 0;
        float cut_val = 0.0f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float z = row[i] * inv_t;
            const unsigned key = order_key(z);
            if (key > cut) mass_gt += expf(z - zmax);
            else if (key == cut) { ties++; cut_val = z; }
        }
        mass_gt = block_sum(mass_gt, fs);
        ties = block_sum_int(ties, is);
        // every thread needs the tied value: take it from the key itself
        const unsigned cb = (cut & 0x80000000u) ? (cut & 0x7fffffffu) : ~cut;
        cut_val = __uint_as_float(cb);
        const int ties_in = min(ties, n_tie);
        const float pe_cut = ties_in > 0 ? expf(cut_val - zmax) : 0.0f;
        const float total = mass_gt + (float) ties_in * pe_cut;
        const float target = P * total;
        // largest key Kp (> cut) with mass(key >= Kp) >= target; if none, the cut itself stays
        unsigned Kp = cut;
        bool moved = false;
        {
            unsigned K = 0u;
            for (int bit = 31; bit >= 0; bit--) {
                const unsigned trial = K | (1u << bit);
                bool ok;
                if (trial <= cut) ok = true;
                else {
                    float ms = 0.0f;
                    for (int i = threadIdx.x; i < V; i += blockDim.x) {
                        const float z = row[i] * inv_t;
                        if (order_key(z) >= trial) ms += expf(z - zmax);
                    }
                    ms = block_sum(ms, fs);
                    ok = ms >= target;
                }
                if (ok) K = trial;
            }
            if (K > cut) { Kp = K; moved = true; }
        }
        if (moved) {
            float above = 0.0f;
            int tie_p = 0;
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float z = row[i] * inv_t;
                const unsigned key = order_key(z);
                if (key > Kp) above += expf(z - zmax);
                else if (key == Kp) tie_p++;
            }
            above = block_sum(above, fs);
            tie_p = block_sum_int(tie_p, is);
            const unsigned pb = (Kp & 0x80000000u) ? (Kp & 0x7fffffffu) : ~Kp;
            const float pe = expf(__uint_as_float(pb) - zmax);
            int need = pe > 0.0f ? (int) ceilf((target - above) / pe) : tie_p;
            need = max(1, min(need, tie_p));
            cut = Kp;
            n_tie = need;
        } else if (ties_in > 0 && pe_cut > 0.0f) {
            int need = (int) ceilf((target - mass_gt) / pe_cut);
            n_tie = max(mass_gt >= target ? 0 : 1, min(need, ties_in));
            if (mass_gt <= 0.0f) n_tie = max(n_tie, 1);
        }
    }

    // inverse CDF in vocabulary order: thread t owns ids [t * per, (t + 1) * per)
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int begin = min(V, (int) threadIdx.x * per), end = min(V, begin + per);
    float cm = 0.0f;
    int ct = 0;
    for (int i = begin; i < end; i++) {
        const unsigned key = order_key(row[i] * inv_t);
        if (key == cut) ct++;
    }
    chunk_ties[threadIdx.x] = ct;
    __syncthreads();
    if (threadIdx.x == 0) {     // exclusive scan of tie counts (1024 entries)
        int run = 0;
        for (int t = 0; t < blockDim.x; t++) { const int c = chunk_ties[t]; chunk_ties[t] = run; run += c; }
    }
    __syncthreads();
    int tie_rank = chunk_ties[threadIdx.x];
    const int tie_rank0 = tie_rank;
    for (int i = begin; i < end; i++) {
        const float z = row[i] * inv_t;
        const unsigned key = order_key(z);
        if (key > cut) cm += expf(z - zmax);
        else if (key == cut) { if (tie_rank < n_tie) cm += expf(z - zmax); tie_rank++; }
    }
    chunk_mass[threadIdx.x] = cm;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int t = 0; t < blockDim.x; t++) total += chunk_mass[t];
        const float r = uniform[blockIdx.x] * total;
        float run = 0.0f;
        int pt = -1;
        for (int t = 0; t < blockDim.x; t++) {
            if (chunk_mass[t] > 0.0f && run + chunk_mass[t] > r) { pt = t; break; }
            run += chunk_mass[t];
        }
        if (pt < 0) {           // r == total (rounding): last chunk that holds mass
            run = 0.0f;
            float before = 0.0f;
            for (int t = 0; t < blockDim.x; t++) { if (chunk_mass[t] > 0.0f) { pt = t; before = run; } run += chunk_mass[t]; }
            run = before;
        }
        pick_thread = pt;
        pick_before = run;
        pick_ties_before = 0;
        (void) pick_ties_before;
        // r is re-derived by the owner from `uniform` and `total`
        fs[0] = r;
    }
    __syncthreads();
    if ((int) threadIdx.x == pick_thread) {
        const float r = fs[0];
        float run = pick_before;
        int tr = tie_rank0;
        int chosen = -1, last = -1;
        for (int i = begin; i < end; i++) {
            const float z = row[i] * inv_t;
            const unsigned key = order_key(z);
            float pe = 0.0f;
            if (key > cut) pe = expf(z - zmax);
            else if (key == cut) { if (tr < n_tie) pe = expf(z - zmax); tr++; }
            if (pe > 0.0f) {
                last = i;
                run += pe;
                if (run > r) { chosen = i; break; }
            }
        }
        if (chosen < 0) chosen = last >= 0 ? last : imax;
        out[blockIdx.x] = chosen;
    }
    if (pick_thread < 0 && threadIdx.x == 0) out[blockIdx.x] = imax;
}

// Logits processors in the reference's order (src/iian/sampler.cpp:72-109), as lists the host prepares per row:
//  * allowed ids (sorted; an empty list allows everything): every other logit becomes -inf (:72-76);
//  * one edit per touched token: l += pre (logit bias; -inf for a banned token or the end of a bad word, :77-88),
//    then l = l > 0 ? l * mul_pos : l * mul_neg (repetition penalty: 1 / r and r, :106), then l += post
//    (-(frequency * count + presence) for tokens that were produced, :107).
// One block per row; a row's lists are the ranges [off[r], off[r + 1]).
__global__ void logit_edits_kernel(float * __restrict__ logits, int V, size_t stride,
                                   const int * __restrict__ allow_off, const int * __restrict__ allow_ids,
                                   const int * __restrict__ edit_off, const int * __restrict__ edit_tok,
                                   const float * __restrict__ pre, const float * __restrict__ mul_pos,
                                   const float * __restrict__ mul_neg, const float * __restrict__ post) {
    const int r = blockIdx.x;
    float * row = logits + (size_t) r * stride;
    const int a0 = allow_off[r], a1 = allow_off[r + 1];
    if (a1 > a0) {
        for (int v = threadIdx.x; v < V; v += blockDim.x) {
            int lo = a0, hi = a1;                 // is v among the sorted ids [a0, a1)?
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (allow_ids[mid] < v) lo = mid + 1; else hi = mid;
            }
            if (lo == a1 || allow_ids[lo] != v) row[v] = -INFINITY;
        }
        __syncthreads();
    }
    for (int e = edit_off[r] + threadIdx.x; e < edit_off[r + 1]; e += blockDim.x) {
        const int t = edit_tok[e];
        if (t < 0 || t >= V) continue;
        float l = row[t] + pre[e];
        l = l > 0.0f ? l * mul_pos[e] : l * mul_neg[e];
        row[t] = l + post[e];
    }
}

// Log-probabilities of the raw distribution (src/iian/sampler.cpp:63-70, 174-182): log softmax of the row at the
// chosen token and at the k largest logits (value descending, lowest id first among equals).  One block per row;
// the k-th pick is the largest entry that comes after the pick before it in that order, so no entry is marked.
__global__ void __launch_bounds__(kSampleThreads) logprobs_kernel(
    const float * __restrict__ logits, int V, size_t stride, const int * __restrict__ tokens, const int * __restrict__ want_k,
    int kmax, float * __restrict__ out_lp, int * __restrict__ top_ids, float * __restrict__ top_lp) {
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ float red[32];
    const int r = blockIdx.x;
    const int k = want_k[r];
    if (k < 0) return;
    const float * row = logits + (size_t) r * stride;
    float mx; int mi;
    block_argmax(row, V, 1.0f, mx, mi, fs, is);
    float acc = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) acc += expf(row[i] - mx);
    __syncthreads();
    const float lse = mx + logf(block_sum(acc, red));
    if (threadIdx.x == 0) {
        const int t = tokens[r];
        out_lp[r] = (t >= 0 && t < V) ? row[t] - lse : -INFINITY;
    }
    float pv = INFINITY;
    int pi = -1;
    for (int j = 0; j < kmax; j++) {
        if (j >= k || j >= V) {
            if (threadIdx.x == 0) { top_ids[(size_t) r * kmax + j] = -1; top_lp[(size_t) r * kmax + j] = -INFINITY; }
            continue;
        }
        float b = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            const bool after = v < pv || (v == pv && i > pi);          // after the pick before, in (value desc, id asc) order
            if (after && (v > b || (v == b && i < bi))) { b = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, b, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
        }
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        __syncthreads();
        if (lane == 0) { fs[warp] = b; is[warp] = bi; }
        __syncthreads();
        b = lane < (blockDim.x >> 5) ? fs[lane] : -INFINITY;
        bi = lane < (blockDim.x >> 5) ? is[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, b, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > b || (ob == b && oi < bi)) { b = ob; bi = oi; }
        }
        pv = b; pi = bi;
        if (threadIdx.x == 0) {
            top_ids[(size_t) r * kmax + j] = bi == 0x7fffffff ? -1 : bi;
            top_lp[(size_t) r * kmax + j] = bi == 0x7fffffff ? -INFINITY : b - lse;
        }
    }
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_argmax(const float * logits, int R, int V, long long stride, int * out, cudaStream_t stream) {
    if (R <= 0) return IIAN_OK;
    if (V <= 0) return IIAN_ERR_SHAPE;
    argmax_kernel<<<R, kSampleThreads, 0, stream>>>(logits, V, (size_t) stride, out);
    return iian_launch_status();
}

// Wide rows: scratch must hold R * parts floats followed by R * parts ints (parts = iian_argmax_parts(V)).
IIAN_API int iian_argmax_parts(int V) { return V >= 16384 ? 64 : 0; }

IIAN_API int iian_argmax_wide(const float * logits, int R, int V, long long stride, void * scratch, int * out,
                              cudaStream_t stream) {
    if (R <= 0) return IIAN_OK;
    const int parts = iian_argmax_parts(V);
    if (V <= 0 || parts == 0 || scratch == nullptr || R > 65535) return IIAN_ERR_SHAPE;
    float * pv = (float *) scratch;
    int * pi = (int *) (pv + (size_t) R * parts);
    const int rc = iian_launch(argmax_partial_kernel, dim3(parts, R), dim3(256), 0, stream, logits, V, (size_t) stride, parts, pv, pi);
    if (rc != IIAN_OK) return rc;
    return iian_launch(argmax_final_kernel, dim3(R), dim3(32), 0, stream, (const float *) pv, (const int *) pi, parts, out);
}

IIAN_API int iian_sample(const float * logits, int R, int V, long long stride, const float * temperature,
                         const int * top_k, const float * top_p, const float * min_p, const float * uniform,
                         int * out, cudaStream_t stream) {
    if (R <= 0) return IIAN_OK;
    if (V <= 0) return IIAN_ERR_SHAPE;
    sample_kernel<<<R, kSampleThreads, 0, stream>>>(logits, V, (size_t) stride, temperature, top_k, top_p, min_p,
                                                    uniform, out);
    return iian_launch_status();
}

// logits [R, V] float32, changed in place.  allow_off / edit_off: [R + 1] int32 prefix sums; a token may appear in
// at most one edit of its row.
IIAN_API int iian_logit_edits(float * logits, int R, int V, long long stride, const int * allow_off, const int * allow_ids,
                              const int * edit_off, const int * edit_tok, const float * pre, const float * mul_pos,
                              const float * mul_neg, const float * post, cudaStream_t stream) {
    if (R <= 0) return IIAN_OK;
    if (V <= 0 || allow_off == nullptr || edit_off == nullptr) return IIAN_ERR_SHAPE;
    logit_edits_kernel<<<R, 256, 0, stream>>>(logits, V, (size_t) stride, allow_off, allow_ids, edit_off, edit_tok, pre,
                                              mul_pos, mul_neg, post);
    return iian_launch_status();
}

// Raw log-probabilities: out_lp [R] at tokens [R]; the want_k[r] (at most kmax; negative: skip the row) largest
// entries of row r into top_ids / top_lp [R, kmax], the rest of a row filled with -1 / -inf.
IIAN_API int iian_logprobs(const float * logits, int R, int V, long long stride, const int * tokens, const int * want_k,
                           int kmax, float * out_lp, int * top_ids, float * top_lp, cudaStream_t stream) {
    if (R <= 0) return IIAN_OK;
    if (V <= 0 || kmax < 0 || kmax > 64) return IIAN_ERR_SHAPE;
    logprobs_kernel<<<R, kSampleThreads, 0, stream>>>(logits, V, (size_t) stride, tokens, want_k, kmax, out_lp, top_ids, top_lp);
    return iian_launch_status();
}
