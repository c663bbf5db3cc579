// Paged attention, general form: any element type, head size, number of heads and groups, page
// size and window.  One warp per (token, head); keys are walked in tiles of 32 that start at
// multiples of 32 of the ABSOLUTE key position, so the order of every sum depends only on the
// token's own position -- not on how the request was cut into steps or what else is in the batch.
// This is the whole attention of the 32-bit path and the fallback of the bfloat16 path for sizes
// the tensor-core kernels do not take.
//
// Formula (reference): head h reads KV head h / (nh / nkv); s_j = (q . k_j) * scale; key j is
// visible iff j <= pos and (window == 0 or pos - j < window); softmax in float32; o = sum p_j v_j
// (src/iian/paged_attn.cpp:112-145, window test :124).
#include "common.cuh"

namespace iian {

constexpr int kGenMaxHeadDim = 512;
constexpr int kGenWarps = 4;

template <typename A>
__global__ void paged_attention_generic_kernel(
    const A * __restrict__ q, const A * __restrict__ k_cache, const A * __restrict__ v_cache,
    A * __restrict__ out, const int * __restrict__ positions, const int * __restrict__ seq_of_token,
    const int * __restrict__ block_table, int max_blocks, const int * __restrict__ ctx_len,
    int N, int nh, int nkv, int hd, int page_size, int num_pages, float scale, int window) {
    __shared__ float qs[kGenWarps][kGenMaxHeadDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long) blockIdx.x * kGenWarps + warp;
    if (item >= (long long) N * nh) return;
    const int t = (int) (item / nh), h = (int) (item % nh);
    const int kvh = h / (nh / nkv);
    A * o = out + ((size_t) t * nh + h) * hd;
    const int s = seq_of_token[t];
    if (s < 0) {   // padding token
        for (int d = lane; d < hd; d += 32) o[d] = from_f32<A>(0.0f);
        return;
    }
    const int p = positions[t];
    int hi = p;
    if (ctx_len != nullptr) hi = min(hi, ctx_len[s] - 1);
    const int lo = window > 0 ? max(0, p - window + 1) : 0;

    const A * qp = q + ((size_t) t * nh + h) * hd;
    for (int d = lane; d < hd; d += 32) qs[warp][d] = to_f32(qp[d]);
    __syncwarp();

    constexpr int kAcc = kGenMaxHeadDim / 32;
    float acc[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; i++) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    const int * bt = block_table + (size_t) s * max_blocks;

    for (int kb = (lo / 32) * 32; kb <= hi; kb += 32) {
        const int j = kb + lane;
        bool valid = j >= lo && j <= hi;
        const A * kp = nullptr;
        const A * vp = nullptr;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) {
                valid = false;      // a page that was given back is never inside the window; never read it
            } else {
                const size_t cell = (((size_t) page * nkv + kvh) * page_size + (j % page_size)) * hd;
                kp = k_cache + cell;
                vp = v_cache + cell;
            }
        }
        float sc = -INFINITY;
        if (valid) {
            float dot = 0.0f;
            for (int d = 0; d < hd; d++) dot += qs[warp][d] * to_f32(kp[d]);
            sc = dot * scale;
        }
        const float tile_max = warp_max(sc);
        if (tile_max == -INFINITY) continue;
        const float m_new = fmaxf(m, tile_max);
        const float pj = valid ? expf(sc - m_new) : 0.0f;
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < kAcc; i++) acc[i] *= corr;
        m = m_new;
        for (int jj = 0; jj < 32; jj++) {
            const float pjj = __shfl_sync(0xffffffffu, pj, jj);
            const unsigned long long vaddr = __shfl_sync(0xffffffffu, (unsigned long long) vp, jj);
            if (pjj == 0.0f) continue;
            const A * vrow = (const A *) vaddr;
#pragma unroll
            for (int i = 0; i < kAcc; i++) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] += pjj * to_f32(vrow[d]);
            }
        }
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;     // a row that sees no key yields zeros
#pragma unroll
    for (int i = 0; i < kAcc; i++) {
        const int d = lane + 32 * i;
        if (d < hd) o[d] = from_f32<A>(acc[i] * inv);
    }
}

}  // namespace iian

using namespace iian;

// q: [N, nh, hd]; caches: [num_pages, nkv, page_size, hd]; out: [N, nh * hd];
// block_table: [S, max_blocks]; ctx_len may be null (then only causality bounds the keys).
IIAN_API int iian_paged_attention_generic(
    const void * q, const void * k_cache, const void * v_cache, void * out,
    const int * positions, const int * seq_of_token, const int * block_table, int max_blocks,
    const int * ctx_len, int act_dtype, int N, int nh, int nkv, int hd, int page_size, int num_pages,
    float scale, int window, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (hd <= 0 || hd > kGenMaxHeadDim || nkv <= 0 || nh % nkv != 0 || page_size <= 0) return IIAN_ERR_SHAPE;
    const long long items = (long long) N * nh;
    const unsigned blocks = (unsigned) ((items + kGenWarps - 1) / kGenWarps);
    const int threads = kGenWarps * 32;
    if (act_dtype == IIAN_F32)
        paged_attention_generic_kernel<float><<<blocks, threads, 0, stream>>>(
            (const float *) q, (const float *) k_cache, (const float *) v_cache, (float *) out, positions,
            seq_of_token, block_table, max_blocks, ctx_len, N, nh, nkv, hd, page_size, num_pages, scale, window);
    else if (act_dtype == IIAN_BF16)
        paged_attention_generic_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
            (const __nv_bfloat16 *) q, (const __nv_bfloat16 *) k_cache, (const __nv_bfloat16 *) v_cache,
            (__nv_bfloat16 *) out, positions, seq_of_token, block_table, max_blocks, ctx_len, N, nh, nkv, hd,
            page_size, num_pages, scale, window);
    else return IIAN_ERR_DTYPE;
    return iian_launch_status();
}
