// Fused per-head RMSNorm of Q and K, rotary position encoding, and the write of K and V into
// the paged cache.  One block per token; its warps share the heads of the concatenated projection
// output Q | K | V.
//
// Reference order (src/iian/arch/qwen3.cpp:80-87): norm over the head axis with one weight
// [head_dim] shared by all heads, then rotation; V is stored untouched.  Rotation, NEOX pairing
// (third_party/ggml/src/ggml-cpu/ops.cpp:5958-5990, 6063-6079): for j < n_rot/2,
// theta = pos * base^(-2j/n_rot); (x_j, x_{j+n_rot/2}) <- (x_j cos - x_{j+n_rot/2} sin,
// x_j sin + x_{j+n_rot/2} cos).  base^(-2j/n_rot) comes in as a float32 table, the product and
// sin/cos are float32.  Cache cell of a token: page * page_size + offset
// (include/iian/kv_cache.h:135-137); K and V use the same cell (src/iian/graph.cpp:66).
//
// Cache layout per layer: [num_pages, num_kv_heads, page_size, head_dim], so one (page, head)
// tile is contiguous.
#include "common.cuh"

namespace iian {

constexpr int kMaxHeadDim = 512;
constexpr int kWarpsPerBlock = 8;


// One block per token; its warps take the heads in turn.  A lane owns rotation pairs p = lane, lane + 32,
// ...: elements (p, p + half) in NEOX style, (2p, 2p + 1) interleaved, and beyond the rotated part single
// elements.  Both members of a pair sit in the same lane, so the rotation needs no exchange, and the
// sines and cosines of a token are computed once per warp and reused for every head.
template <typename A>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) qk_norm_rope_store_kernel(
    const A * __restrict__ qkv, const float * __restrict__ bias,
    A * __restrict__ q_out, A * __restrict__ k_cache, A * __restrict__ v_cache,
    const float * __restrict__ q_weight, const float * __restrict__ k_weight,
    const float * __restrict__ inv_freq, const int * __restrict__ positions,
    const int * __restrict__ slots,
    int N, int nh, int nkv, int hd, int rot_dim, int rope_style, float eps,
    int page_size, int num_pages, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nh + 2 * nkv;
    const int t = blockIdx.x;
    const int slot = slots != nullptr ? slots[t] : -1;
    const bool store_kv = write_kv && slot >= 0 && slot < num_pages * page_size;   // a padding token stores nothing
    constexpr int kMaxPairs = kMaxHeadDim / 64;      // per lane
    const bool has_rope = inv_freq != nullptr && rot_dim > 0;
    const int half = has_rope ? rot_dim / 2 : 0;
    float cs[kMaxPairs], sn[kMaxPairs];
    if (has_rope) {
        const float pos = (float) positions[t];
#pragma unroll
        for (int k = 0; k < kMaxPairs; k++) {
            const int p = lane + 32 * k;
            if (p < half) sincosf(pos * inv_freq[p], &sn[k], &cs[k]);
        }
    }
    for (int h = warp; h < heads_total; h += kWarpsPerBlock) {
        const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
        if (!is_q && !store_kv) continue;
        const A * src = qkv + (size_t) t * heads_total * hd + (size_t) h * hd;
        const float * b = bias != nullptr ? bias + (size_t) h * hd : nullptr;
        A * dst;
        if (is_q) {
            dst = q_out + ((size_t) t * nh + h) * hd;
        } else {
            const int kvh = is_k ? h - nh : h - nh - nkv;
            const int page = slot / page_size, off = slot % page_size;
            A * base = is_k ? k_cache : v_cache;
            dst = base + (((size_t) page * nkv + kvh) * page_size + off) * hd;
        }
        const float * w = is_q ? q_weight : (is_k ? k_weight : nullptr);
        const bool rotate = (is_q || is_k) && has_rope;
        if (w == nullptr && !rotate) {          // V (or an unnormalised, unrotated head): a copy
            for (int i = lane; i < hd; i += 32) {
                float v = to_f32(src[i]);
                if (b != nullptr) v += b[i];
                dst[i] = from_f32<A>(v);
            }
            continue;
        }
        const int hr = rotate ? half : 0;
        float x0[kMaxPairs], x1[kMaxPairs], tail[kMaxPairs * 2];
        float ss = 0.0f;
#pragma unroll
        for (int k = 0; k < kMaxPairs; k++) {
            const int p = lane + 32 * k;
            if (p < hr) {
                const int i0 = rope_style == 0 ? p : 2 * p, i1 = rope_style == 0 ? p + hr : 2 * p + 1;
                float a0 = to_f32(src[i0]), a1 = to_f32(src[i1]);
                if (b != nullptr) { a0 += b[i0]; a1 += b[i1]; }
                x0[k] = a0; x1[k] = a1;
                ss += a0 * a0 + a1 * a1;
            }
        }
#pragma unroll
        for (int k = 0; k < kMaxPairs * 2; k++) {
            const int i = 2 * hr + lane + 32 * k;
            if (i < hd) {
                float a = to_f32(src[i]);
                if (b != nullptr) a += b[i];
                tail[k] = a;
                ss += a * a;
            }
        }
        float inv = 1.0f;
        if (w != nullptr) {
            ss = warp_sum(ss);
            inv = rsqrtf(ss / (float) hd + eps);
        }
#pragma unroll
        for (int k = 0; k < kMaxPairs; k++) {
            const int p = lane + 32 * k;
            if (p < hr) {
                const int i0 = rope_style == 0 ? p : 2 * p, i1 = rope_style == 0 ? p + hr : 2 * p + 1;
                float a0 = x0[k], a1 = x1[k];
                if (w != nullptr) { a0 = a0 * inv * w[i0]; a1 = a1 * inv * w[i1]; }
                dst[i0] = from_f32<A>(a0 * cs[k] - a1 * sn[k]);
                dst[i1] = from_f32<A>(a0 * sn[k] + a1 * cs[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < kMaxPairs * 2; k++) {
            const int i = 2 * hr + lane + 32 * k;
            if (i < hd) {
                float a = tail[k];
                if (w != nullptr) a = a * inv * w[i];
                dst[i] = from_f32<A>(a);
            }
        }
    }
}

}  // namespace iian

using namespace iian;

// qkv: [N, (nh + 2 nkv) * hd].  q_weight / k_weight / inv_freq / bias / slots may be null.
IIAN_API int iian_qk_norm_rope_store(
    const void * qkv, const float * bias, void * q_out, void * k_cache, void * v_cache,
    const float * q_weight, const float * k_weight, const float * inv_freq,
    const int * positions, const int * slots, int act_dtype,
    int N, int nh, int nkv, int hd, int rot_dim, int rope_style, float eps,
    int page_size, int num_pages, int write_kv, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (hd <= 0 || hd > kMaxHeadDim) return IIAN_ERR_SHAPE;
    if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1)) return IIAN_ERR_SHAPE;
    if (write_kv && (slots == nullptr || k_cache == nullptr || v_cache == nullptr)) return IIAN_ERR_SHAPE;
    const unsigned blocks = (unsigned) N;
    const int threads = kWarpsPerBlock * 32;
    if (act_dtype == IIAN_F32)
        return iian_launch(qk_norm_rope_store_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
            (const float *) qkv, bias, (float *) q_out, (float *) k_cache, (float *) v_cache, q_weight, k_weight,
            inv_freq, positions, slots, N, nh, nkv, hd, rot_dim, rope_style, eps, page_size, num_pages, write_kv);
    if (act_dtype == IIAN_BF16)
        return iian_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
            (const __nv_bfloat16 *) qkv, bias, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache,
            (__nv_bfloat16 *) v_cache, q_weight, k_weight, inv_freq, positions, slots, N, nh, nkv, hd, rot_dim,
            rope_style, eps, page_size, num_pages, write_kv);
    return IIAN_ERR_DTYPE;
}
