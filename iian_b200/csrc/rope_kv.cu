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


// cos and sin of pos * inv_freq[p] for every token of the step and every rotation pair: computed once per
// step and shared by all layers that rotate alike (the angles do not depend on the layer).
__global__ void rotary_table_kernel(const float * __restrict__ inv_freq, const int * __restrict__ positions,
                                    float2 * __restrict__ table, int half, long long total) {
    pdl_wait();
    pdl_launch_dependents();
    const long long idx = (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int) (idx / half), p = (int) (idx % half);
    float sn, cs;
    sincosf((float) positions[t] * inv_freq[p], &sn, &cs);
    table[idx] = make_float2(cs, sn);
}

template <typename A> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float * p) { return *reinterpret_cast<const float2 *>(p); }
    static __device__ __forceinline__ void store(float * p, float2 v) { *reinterpret_cast<float2 *>(p) = v; }
};
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16 * p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 * p, float2 v) {
        *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(v.x, v.y);
    }
};

// Fast form: one warp per (token, head); NEOX pairs over the whole head (or no rotation), head size a
// multiple of 4, angles from the table.  A lane owns two adjacent pairs at a time, i.e. two adjacent
// elements in each half of the head, so every access is a 2-element vector.
template <typename A>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) qk_norm_rope_store_fast_kernel(
    const A * __restrict__ qkv, A * __restrict__ q_out, A * __restrict__ k_cache, A * __restrict__ v_cache,
    const float * __restrict__ q_weight, const float * __restrict__ k_weight, const float2 * __restrict__ table,
    const int * __restrict__ slots, int N, int nh, int nkv, int hd, float eps, int page_size, int num_pages, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
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
    const A * src = qkv + (size_t) t * heads_total * hd + (size_t) h * hd;
    A * dst;
    if (is_q) {
        dst = q_out + ((size_t) t * nh + h) * hd;
    } else {
        const int kvh = is_k ? h - nh : h - nh - nkv;
        const int page = slot / page_size, off = slot % page_size;
        A * base = is_k ? k_cache : v_cache;
        dst = base + (((size_t) page * nkv + kvh) * page_size + off) * hd;
    }
    const int half = hd >> 1;
    const float * w = is_q ? q_weight : (is_k ? k_weight : nullptr);
    const bool rotate = (is_q || is_k) && table != nullptr;
    constexpr int kIter = kMaxHeadDim / 128;       // a pass covers 64 pairs
    float2 lo[kIter], hi[kIter];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kIter; k++) {
        const int p0 = 2 * lane + 64 * k;
        if (p0 < half) {
            lo[k] = Pair<A>::load(src + p0);
            hi[k] = Pair<A>::load(src + half + p0);
            ss += lo[k].x * lo[k].x + lo[k].y * lo[k].y + hi[k].x * hi[k].x + hi[k].y * hi[k].y;
        }
    }
    float inv = 1.0f;
    if (w != nullptr) {
        ss = warp_sum(ss);
        inv = rsqrtf(ss / (float) hd + eps);
    }
#pragma unroll
    for (int k = 0; k < kIter; k++) {
        const int p0 = 2 * lane + 64 * k;
        if (p0 < half) {
            float2 a = lo[k], c = hi[k];
            if (w != nullptr) {
                const float2 wl = *reinterpret_cast<const float2 *>(w + p0), wh = *reinterpret_cast<const float2 *>(w + half + p0);
                a.x = a.x * inv * wl.x; a.y = a.y * inv * wl.y;
                c.x = c.x * inv * wh.x; c.y = c.y * inv * wh.y;
            }
            if (rotate) {
                const float4 cssn = *reinterpret_cast<const float4 *>(table + (size_t) t * half + p0);   // cos0 sin0 cos1 sin1
                const float2 r0 = make_float2(rot_lo(a.x, c.x, cssn.x, cssn.y), rot_lo(a.y, c.y, cssn.z, cssn.w));
                const float2 r1 = make_float2(rot_hi(a.x, c.x, cssn.x, cssn.y), rot_hi(a.y, c.y, cssn.z, cssn.w));
                a = r0; c = r1;
            }
            Pair<A>::store(dst + p0, a);
            Pair<A>::store(dst + half + p0, c);
        }
    }
}

// The fast form for head sizes up to 128 with several heads per warp: a warp takes HPW consecutive heads of a token
// and has all their loads in flight before it touches the first (a head of 128 bfloat16 is only 256 bytes; one head
// per warp leaves the memory system mostly idle: 27.6 us for 2048 tokens of 32 + 2 x 8 heads, against 50 MB to move).
template <typename A, int HPW>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) qk_norm_rope_store_wide_kernel(
    const A * __restrict__ qkv, A * __restrict__ q_out, A * __restrict__ k_cache, A * __restrict__ v_cache,
    const float * __restrict__ q_weight, const float * __restrict__ k_weight, const float2 * __restrict__ table,
    const int * __restrict__ slots, int N, int nh, int nkv, int hd, float eps, int page_size, int num_pages, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nh + 2 * nkv;
    const int groups = (heads_total + HPW - 1) / HPW;
    const long long item = (long long) blockIdx.x * kWarpsPerBlock + warp;
    if (item >= (long long) N * groups) return;
    const int t = (int) (item / groups);
    const int h0 = (int) (item % groups) * HPW;
    const int slot = slots != nullptr ? slots[t] : -1;
    const bool slot_ok = slot >= 0 && slot < num_pages * page_size;
    const int half = hd >> 1;
    const int p0 = 2 * lane;
    const bool mine = p0 < half;
    const A * row = qkv + (size_t) t * heads_total * hd;
    float2 lo[HPW], hi[HPW];
    bool live[HPW];
#pragma unroll
    for (int j = 0; j < HPW; j++) {
        const int h = h0 + j;
        live[j] = h < heads_total && (h < nh || (write_kv && slot_ok));     // a padding token stores no K/V
        lo[j] = hi[j] = make_float2(0.0f, 0.0f);
        if (live[j] && mine) {
            lo[j] = Pair<A>::load(row + (size_t) h * hd + p0);
            hi[j] = Pair<A>::load(row + (size_t) h * hd + half + p0);
        }
    }
    float4 cssn = make_float4(1.0f, 0.0f, 1.0f, 0.0f);                        // cos0 sin0 cos1 sin1
    if (table != nullptr && mine) cssn = *reinterpret_cast<const float4 *>(table + (size_t) t * half + p0);
#pragma unroll
    for (int j = 0; j < HPW; j++) {
        if (!live[j]) continue;                                              // uniform over the warp
        const int h = h0 + j;
        const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
        A * dst;
        if (is_q) {
            dst = q_out + ((size_t) t * nh + h) * hd;
        } else {
            const int kvh = is_k ? h - nh : h - nh - nkv;
            const int page = slot / page_size, off = slot % page_size;
            dst = (is_k ? k_cache : v_cache) + (((size_t) page * nkv + kvh) * page_size + off) * hd;
        }
        const float * w = is_q ? q_weight : (is_k ? k_weight : nullptr);
        float2 a = lo[j], c = hi[j];
        if (w != nullptr) {
            const float ss = warp_sum(a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y);
            const float inv = rsqrtf(ss / (float) hd + eps);
            if (mine) {
                const float2 wl = *reinterpret_cast<const float2 *>(w + p0), wh = *reinterpret_cast<const float2 *>(w + half + p0);
                a.x = a.x * inv * wl.x; a.y = a.y * inv * wl.y;
                c.x = c.x * inv * wh.x; c.y = c.y * inv * wh.y;
            }
        }
        if ((is_q || is_k) && table != nullptr) {
            const float2 r0 = make_float2(rot_lo(a.x, c.x, cssn.x, cssn.y), rot_lo(a.y, c.y, cssn.z, cssn.w));
            const float2 r1 = make_float2(rot_hi(a.x, c.x, cssn.x, cssn.y), rot_hi(a.y, c.y, cssn.z, cssn.w));
            a = r0; c = r1;
        }
        if (mine) {
            Pair<A>::store(dst + p0, a);
            Pair<A>::store(dst + half + p0, c);
        }
    }
}

// Head size 128 in bfloat16, the serving case: the kernel above is bound by instruction issue (64 % of the issue
// slots at 2048 tokens), not by memory, so this form moves 8 bytes per access.  Sixteen lanes own a head: lane s of
// them has elements 4 s .. 4 s + 3 of each half, i.e. four rotation pairs; a warp works on two heads at a time and
// on HPW heads of a token in all.
template <int HPW>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) qk_norm_rope_store_vec128_kernel(
    const __nv_bfloat16 * __restrict__ qkv, __nv_bfloat16 * __restrict__ q_out, __nv_bfloat16 * __restrict__ k_cache,
    __nv_bfloat16 * __restrict__ v_cache, const float * __restrict__ q_weight, const float * __restrict__ k_weight,
    const float2 * __restrict__ table, const int * __restrict__ slots, int N, int nh, int nkv, float eps, int page_size,
    int num_pages, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int hd = 128, half = 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane & 15, hsel = lane >> 4;
    const int heads_total = nh + 2 * nkv;
    const int groups = (heads_total + HPW - 1) / HPW;
    const long long item = (long long) blockIdx.x * kWarpsPerBlock + warp;
    if (item >= (long long) N * groups) return;
    const int t = (int) (item / groups);
    const int h0 = (int) (item % groups) * HPW;
    const int slot = slots != nullptr ? slots[t] : -1;
    const bool slot_ok = slot >= 0 && slot < num_pages * page_size;
    const int page = slot_ok ? slot / page_size : 0, off = slot_ok ? slot % page_size : 0;
    const __nv_bfloat16 * row = qkv + (size_t) t * heads_total * hd;
    uint2 lo[HPW / 2], hi[HPW / 2];
#pragma unroll
    for (int j = 0; j < HPW / 2; j++) {
        const int h = h0 + 2 * j + hsel;
        lo[j] = hi[j] = make_uint2(0u, 0u);
        if (h < heads_total && (h < nh || (write_kv && slot_ok))) {
            lo[j] = *reinterpret_cast<const uint2 *>(row + (size_t) h * hd + 4 * sub);
            hi[j] = *reinterpret_cast<const uint2 *>(row + (size_t) h * hd + half + 4 * sub);
        }
    }
    float cs[4] = {1.0f, 1.0f, 1.0f, 1.0f}, sn[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (table != nullptr) {
        const float4 t0 = *reinterpret_cast<const float4 *>(table + (size_t) t * half + 4 * sub);
        const float4 t1 = *reinterpret_cast<const float4 *>(table + (size_t) t * half + 4 * sub + 2);
        cs[0] = t0.x; sn[0] = t0.y; cs[1] = t0.z; sn[1] = t0.w; cs[2] = t1.x; sn[2] = t1.y; cs[3] = t1.z; sn[3] = t1.w;
    }
#pragma unroll
    for (int j = 0; j < HPW / 2; j++) {
        const int h = h0 + 2 * j + hsel;
        const bool live = h < heads_total && (h < nh || (write_kv && slot_ok));     // a padding token stores no K/V
        const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
        const float * w = is_q ? q_weight : (is_k ? k_weight : nullptr);
        float a[4], c[4];
        {
            const float2 a01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&lo[j].x));
            const float2 a23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&lo[j].y));
            const float2 c01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&hi[j].x));
            const float2 c23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&hi[j].y));
            a[0] = a01.x; a[1] = a01.y; a[2] = a23.x; a[3] = a23.y;
            c[0] = c01.x; c[1] = c01.y; c[2] = c23.x; c[3] = c23.y;
        }
        // sum of squares over the sixteen lanes of this head (all lanes take part in the shuffles)
        float ss = (a[0] * a[0] + a[1] * a[1]) + (a[2] * a[2] + a[3] * a[3]) + (c[0] * c[0] + c[1] * c[1]) + (c[2] * c[2] + c[3] * c[3]);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (!live) continue;
        if (w != nullptr) {
            const float inv = rsqrtf(ss / (float) hd + eps);
            const float4 wl = *reinterpret_cast<const float4 *>(w + 4 * sub), wh = *reinterpret_cast<const float4 *>(w + half + 4 * sub);
            a[0] *= inv * wl.x; a[1] *= inv * wl.y; a[2] *= inv * wl.z; a[3] *= inv * wl.w;
            c[0] *= inv * wh.x; c[1] *= inv * wh.y; c[2] *= inv * wh.z; c[3] *= inv * wh.w;
        }
        if ((is_q || is_k) && table != nullptr) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float r0 = rot_lo(a[i], c[i], cs[i], sn[i]), r1 = rot_hi(a[i], c[i], cs[i], sn[i]);
                a[i] = r0; c[i] = r1;
            }
        }
        __nv_bfloat16 * dst;
        if (is_q) {
            dst = q_out + ((size_t) t * nh + h) * hd;
        } else {
            const int kvh = is_k ? h - nh : h - nh - nkv;
            dst = (is_k ? k_cache : v_cache) + (((size_t) page * nkv + kvh) * page_size + off) * hd;
        }
        uint2 o0, o1;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a[0], a[1]), p1 = __floats2bfloat162_rn(a[2], a[3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(c[0], c[1]), p3 = __floats2bfloat162_rn(c[2], c[3]);
        o0.x = *reinterpret_cast<unsigned *>(&p0); o0.y = *reinterpret_cast<unsigned *>(&p1);
        o1.x = *reinterpret_cast<unsigned *>(&p2); o1.y = *reinterpret_cast<unsigned *>(&p3);
        *reinterpret_cast<uint2 *>(dst + 4 * sub) = o0;
        *reinterpret_cast<uint2 *>(dst + half + 4 * sub) = o1;
    }
}

// General form: one warp per (token, head); any head size, partial rotation, either pairing style, bias.
// A lane owns rotation pairs p = lane, lane + 32, ...: elements (p, p + half) in NEOX style, (2p, 2p + 1)
// interleaved; beyond the rotated part it owns single elements.  Both members of a pair sit in the same
// lane, so the rotation needs no exchange.
template <typename A>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) qk_norm_rope_store_kernel(
    const A * __restrict__ qkv, const float * __restrict__ bias,
    A * __restrict__ q_out, A * __restrict__ k_cache, A * __restrict__ v_cache,
    const float * __restrict__ q_weight, const float * __restrict__ k_weight,
    const float * __restrict__ inv_freq, const float2 * __restrict__ table, const int * __restrict__ positions,
    const int * __restrict__ slots,
    int N, int nh, int nkv, int hd, int rot_dim, int rope_style, float eps,
    int page_size, int num_pages, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
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
    const bool rotate = (is_q || is_k) && inv_freq != nullptr && rot_dim > 0;

    if (w == nullptr && !rotate) {          // V (or an unnormalised, unrotated head): a copy
        for (int i = lane; i < hd; i += 32) {
            float v = to_f32(src[i]);
            if (b != nullptr) v += b[i];
            dst[i] = from_f32<A>(v);
        }
        return;
    }
    constexpr int kMaxPairs = kMaxHeadDim / 64;      // per lane
    const int half = rotate ? rot_dim / 2 : 0;
    float x0[kMaxPairs], x1[kMaxPairs], tail[kMaxPairs * 2];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kMaxPairs; k++) {
        const int p = lane + 32 * k;
        if (p < half) {
            const int i0 = rope_style == 0 ? p : 2 * p, i1 = rope_style == 0 ? p + half : 2 * p + 1;
            float a0 = to_f32(src[i0]), a1 = to_f32(src[i1]);
            if (b != nullptr) { a0 += b[i0]; a1 += b[i1]; }
            x0[k] = a0; x1[k] = a1;
            ss += a0 * a0 + a1 * a1;
        }
    }
#pragma unroll
    for (int k = 0; k < kMaxPairs * 2; k++) {
        const int i = 2 * half + lane + 32 * k;
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
    const float pos = rotate ? (float) positions[t] : 0.0f;
#pragma unroll
    for (int k = 0; k < kMaxPairs; k++) {
        const int p = lane + 32 * k;
        if (p < half) {
            const int i0 = rope_style == 0 ? p : 2 * p, i1 = rope_style == 0 ? p + half : 2 * p + 1;
            float a0 = x0[k], a1 = x1[k];
            if (w != nullptr) { a0 = a0 * inv * w[i0]; a1 = a1 * inv * w[i1]; }
            float sn, cs;
            if (table != nullptr) { const float2 e = table[(size_t) t * half + p]; cs = e.x; sn = e.y; }
            else sincosf(pos * inv_freq[p], &sn, &cs);
            dst[i0] = from_f32<A>(rot_lo(a0, a1, cs, sn));
            dst[i1] = from_f32<A>(rot_hi(a0, a1, cs, sn));
        }
    }
#pragma unroll
    for (int k = 0; k < kMaxPairs * 2; k++) {
        const int i = 2 * half + lane + 32 * k;
        if (i < hd) {
            float a = tail[k];
            if (w != nullptr) a = a * inv * w[i];
            dst[i] = from_f32<A>(a);
        }
    }
}

}  // namespace iian

using namespace iian;

// table[t, p] = (cos, sin)(positions[t] * inv_freq[p]) for p < half; float2 per entry.
IIAN_API int iian_rotary_table(const float * inv_freq, const int * positions, void * table, int N, int half,
                               cudaStream_t stream) {
    const long long total = (long long) N * half;
    if (total <= 0) return IIAN_OK;
    const int threads = 256;
    return iian_launch(rotary_table_kernel, dim3((unsigned) ((total + threads - 1) / threads)), dim3(threads), 0, stream,
                       inv_freq, positions, (float2 *) table, half, total);
}

// qkv: [N, (nh + 2 nkv) * hd].  q_weight / k_weight / inv_freq / bias / slots / table may be null.  With a
// table (from iian_rotary_table for the same positions and rot_dim / 2 pairs) no sine or cosine is computed
// here.
IIAN_API int iian_qk_norm_rope_store(
    const void * qkv, const float * bias, void * q_out, void * k_cache, void * v_cache,
    const float * q_weight, const float * k_weight, const float * inv_freq, const void * table,
    const int * positions, const int * slots, int act_dtype,
    int N, int nh, int nkv, int hd, int rot_dim, int rope_style, float eps,
    int page_size, int num_pages, int write_kv, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (hd <= 0 || hd > kMaxHeadDim) return IIAN_ERR_SHAPE;
    if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1)) return IIAN_ERR_SHAPE;
    if (write_kv && (slots == nullptr || k_cache == nullptr || v_cache == nullptr)) return IIAN_ERR_SHAPE;
    if (act_dtype != IIAN_F32 && act_dtype != IIAN_BF16) return IIAN_ERR_DTYPE;
    const long long items = (long long) N * (nh + 2 * nkv);
    const unsigned blocks = (unsigned) ((items + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const int threads = kWarpsPerBlock * 32;
    const bool no_rope = inv_freq == nullptr || rot_dim == 0;
    const bool fast = bias == nullptr && hd % 4 == 0 && (no_rope || (rope_style == 0 && rot_dim == hd && table != nullptr)) &&
                      ((uintptr_t) qkv & 7) == 0 && ((uintptr_t) q_out & 7) == 0 && ((uintptr_t) k_cache & 7) == 0 &&
                      ((uintptr_t) v_cache & 7) == 0 && ((uintptr_t) q_weight & 7) == 0 && ((uintptr_t) k_weight & 7) == 0 &&
                      ((uintptr_t) table & 15) == 0;
    const float2 * tab = no_rope ? nullptr : (const float2 *) table;
    if (fast && hd == 128 && act_dtype == IIAN_BF16 && ((uintptr_t) q_weight & 15) == 0 && ((uintptr_t) k_weight & 15) == 0) {
        constexpr int HPW = 4;
        const long long witems = (long long) N * ((nh + 2 * nkv + HPW - 1) / HPW);
        const unsigned wblocks = (unsigned) ((witems + kWarpsPerBlock - 1) / kWarpsPerBlock);
        return iian_launch(qk_norm_rope_store_vec128_kernel<HPW>, dim3(wblocks), dim3(threads), 0, stream,
            (const __nv_bfloat16 *) qkv, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache, (__nv_bfloat16 *) v_cache,
            q_weight, k_weight, tab, slots, N, nh, nkv, eps, page_size, num_pages, write_kv);
    }
    if (fast && hd <= 128) {
        constexpr int HPW = 4;          // measured at 2048 tokens of 32 + 2 x 8 heads: 2 and 4 heads per warp 21 us, 8: 25 us, 16: 34 us
        const long long witems = (long long) N * ((nh + 2 * nkv + HPW - 1) / HPW);
        const unsigned wblocks = (unsigned) ((witems + kWarpsPerBlock - 1) / kWarpsPerBlock);
        if (act_dtype == IIAN_F32)
            return iian_launch(qk_norm_rope_store_wide_kernel<float, HPW>, dim3(wblocks), dim3(threads), 0, stream,
                (const float *) qkv, (float *) q_out, (float *) k_cache, (float *) v_cache, q_weight, k_weight, tab, slots,
                N, nh, nkv, hd, eps, page_size, num_pages, write_kv);
        return iian_launch(qk_norm_rope_store_wide_kernel<__nv_bfloat16, HPW>, dim3(wblocks), dim3(threads), 0, stream,
            (const __nv_bfloat16 *) qkv, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache, (__nv_bfloat16 *) v_cache,
            q_weight, k_weight, tab, slots, N, nh, nkv, hd, eps, page_size, num_pages, write_kv);
    }
    if (fast) {
        if (act_dtype == IIAN_F32)
            return iian_launch(qk_norm_rope_store_fast_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
                (const float *) qkv, (float *) q_out, (float *) k_cache, (float *) v_cache, q_weight, k_weight, tab, slots,
                N, nh, nkv, hd, eps, page_size, num_pages, write_kv);
        return iian_launch(qk_norm_rope_store_fast_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
            (const __nv_bfloat16 *) qkv, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache, (__nv_bfloat16 *) v_cache,
            q_weight, k_weight, tab, slots, N, nh, nkv, hd, eps, page_size, num_pages, write_kv);
    }
    if (act_dtype == IIAN_F32)
        return iian_launch(qk_norm_rope_store_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
            (const float *) qkv, bias, (float *) q_out, (float *) k_cache, (float *) v_cache, q_weight, k_weight,
            inv_freq, tab, positions, slots, N, nh, nkv, hd, rot_dim, rope_style, eps, page_size, num_pages, write_kv);
    return iian_launch(qk_norm_rope_store_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
        (const __nv_bfloat16 *) qkv, bias, (__nv_bfloat16 *) q_out, (__nv_bfloat16 *) k_cache,
        (__nv_bfloat16 *) v_cache, q_weight, k_weight, inv_freq, tab, positions, slots, N, nh, nkv, hd, rot_dim,
        rope_style, eps, page_size, num_pages, write_kv);
}
