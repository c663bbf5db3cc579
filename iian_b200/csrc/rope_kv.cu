// Fused per-head RMSNorm of Q and K, rotary position encoding, and the write of K and V into
// the paged cache.  One warp per (token, head) of the concatenated projection output Q | K | V.
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
constexpr int kWarpsPerBlock = 4;

template <typename A>
__global__ void qk_norm_rope_store_kernel(
    const A * __restrict__ qkv, const float * __restrict__ bias,
    A * __restrict__ q_out, A * __restrict__ k_cache, A * __restrict__ v_cache,
    const float * __restrict__ q_weight, const float * __restrict__ k_weight,
    const float * __restrict__ inv_freq, const int * __restrict__ positions,
    const int * __restrict__ slots,
    int N, int nh, int nkv, int hd, int rot_dim, int rope_style, float eps,
    int page_size, int num_pages, int write_kv) {
    __shared__ float stage[kWarpsPerBlock][kMaxHeadDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nh + 2 * nkv;
    const long long item = (long long) blockIdx.x * kWarpsPerBlock + warp;
    if (item >= (long long) N * heads_total) return;
    const int t = (int) (item / heads_total);
    const int h = (int) (item % heads_total);
    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    if (!is_q && !write_kv) return;
    const int slot = slots != nullptr ? slots[t] : -1;
    if (!is_q && (slot < 0 || slot >= num_pages * page_size)) return;   // padding token: nothing to store

    const size_t in_off = (size_t) t * heads_total * hd + (size_t) h * hd;
    float * s = stage[warp];
    float ss = 0.0f;
    for (int i = lane; i < hd; i += 32) {
        float v = to_f32(qkv[in_off + i]);
        if (bias != nullptr) v += bias[(size_t) h * hd + i];
        s[i] = v;
        ss += v * v;
    }
    const float * w = is_q ? q_weight : (is_k ? k_weight : nullptr);
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float) hd + eps);
        for (int i = lane; i < hd; i += 32) s[i] = s[i] * inv * w[i];
    }
    __syncwarp();

    A * dst;
    if (is_q) {
        dst = q_out + ((size_t) t * nh + h) * hd;
    } else {
        const int kvh = is_k ? h - nh : h - nh - nkv;
        const int page = slot / page_size, off = slot % page_size;
        A * base = is_k ? k_cache : v_cache;
        dst = base + (((size_t) page * nkv + kvh) * page_size + off) * hd;
    }
    const bool rotate = (is_q || is_k) && inv_freq != nullptr && rot_dim > 0;
    const float pos = rotate ? (float) positions[t] : 0.0f;
    const int half = rot_dim / 2;
    for (int i = lane; i < hd; i += 32) {
        float o;
        if (rotate && i < rot_dim) {
            int j, i0, i1;
            bool first;
            if (rope_style == 0) {          // NEOX: (j, j + half)
                first = i < half;
                j = first ? i : i - half;
                i0 = j; i1 = j + half;
            } else {                         // interleaved: (2j, 2j + 1)
                j = i >> 1;
                first = (i & 1) == 0;
                i0 = 2 * j; i1 = 2 * j + 1;
            }
            float sn, cs;
            sincosf(pos * inv_freq[j], &sn, &cs);
            const float x0 = s[i0], x1 = s[i1];
            o = first ? x0 * cs - x1 * sn : x0 * sn + x1 * cs;
        } else {
            o = s[i];
        }
        dst[i] = from_f32<A>(o);
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
    const long long items = (long long) N * (nh + 2 * nkv);
    const unsigned blocks = (unsigned) ((items + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const int threads = kWarpsPerBlock * 32;
    if (act_dtype == IIAN_F32)
        qk_norm_rope_store_kernel<float><<<blocks, threads, 0, stream>>>(
            (const float *) qkv, bias, (float *) q_out, (float *) k_cache, (float *) v_cache, q_weight, k_weight,
            inv_freq, positions, slots, N, nh, nkv, hd, rot_dim, rope_style, eps, page_size, num_pages, write_kv);
    else if (act_dtype == IIAN_BF16)
        qk_norm_rope_store_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
            (const __nv_bfloat16 *) qkv, bias, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache,
            (__nv_bfloat16 *) v_cache, q_weight, k_weight, inv_freq, positions, slots, N, nh, nkv, hd, rot_dim,
            rope_style, eps, page_size, num_pages, write_kv);
    else return IIAN_ERR_DTYPE;
    return iian_launch_status();
}
