// Row-wise kernels: embedding gather, residual add + RMSNorm, SwiGLU, row gather, bias add.
//
// The residual stream is always float32; `A` is the activation type (float in the 32-bit path,
// bfloat16 in the serving path).  Each row is reduced in an order that depends only on the
// block size, so a row's result does not depend on which other rows are in the batch.
//
// Formulas (reference): RMSNorm x * rsqrt(mean(x^2) + eps) * w, normalise first, weight second
// (src/iian/graph.cpp:105-114); SwiGLU silu(gate) * up with silu(z) = z / (1 + exp(-z))
// (src/iian/graph.cpp:135, third_party/ggml/src/ggml-cpu/vec.h:1046-1048); embedding = row gather
// (src/iian/graph.cpp:39-46); row selection = row gather (src/iian/graph.cpp:356-358).
#include "common.cuh"

namespace iian {

template <typename W>
__global__ void embedding_kernel(const W * __restrict__ table, const int * __restrict__ tokens,
                                 float * __restrict__ out, int H, int V) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = tokens[t];
    float * o = out + (size_t) t * H;
    if (id < 0 || id >= V) {   // never read outside the table
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const W * row = table + (size_t) id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

// residual (f32, in place) += delta (A, optional); out (A) = rmsnorm(residual) * weight (f32)
// General form: two passes over the row, any H.
template <typename A>
__global__ void add_rms_norm_kernel(float * __restrict__ residual, const A * __restrict__ delta,
                                    const float * __restrict__ weight, A * __restrict__ out,
                                    int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float * r = residual + base;
    float ss = 0.0f;
    if (delta != nullptr) {
        const A * d = delta + base;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = r[i] + to_f32(d[i]);
            r[i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = r[i];
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float) H + eps);
    A * o = out + base;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<A>(r[i] * inv * weight[i]);
}

template <typename A> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float * p) { return *reinterpret_cast<const float4 *>(p); }
    static __device__ __forceinline__ void store(float * p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16 * p) {
        const uint2 raw = *reinterpret_cast<const uint2 *>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 * p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned *>(&a);
        raw.y = *reinterpret_cast<unsigned *>(&b);
        *reinterpret_cast<uint2 *>(p) = raw;
    }
};

// Fast form for H % 4 == 0 and H <= 4 * VPT * blockDim: the row stays in registers, one pass over
// memory, 16-byte accesses.  Thread t owns the float4 groups t, t + blockDim, ... (fixed by H alone).
template <typename A, int VPT>
__global__ void add_rms_norm_vec_kernel(float * __restrict__ residual, const A * __restrict__ delta,
                                        const float * __restrict__ weight, A * __restrict__ out,
                                        int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    const int groups = H >> 2;
    float4 v[VPT];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int gi = threadIdx.x + k * blockDim.x;
        if (gi < groups) {
            float4 x = Vec4<float>::load(residual + base + 4 * gi);
            if (delta != nullptr) {
                const float4 d = Vec4<A>::load(delta + base + 4 * gi);
                x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
                Vec4<float>::store(residual + base + 4 * gi, x);
            }
            v[k] = x;
            ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float) H + eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int gi = threadIdx.x + k * blockDim.x;
        if (gi < groups) {
            const float4 w = Vec4<float>::load(weight + 4 * gi);
            Vec4<A>::store(out + base + 4 * gi, make_float4(v[k].x * inv * w.x, v[k].y * inv * w.y,
                                                             v[k].z * inv * w.z, v[k].w * inv * w.w));
        }
    }
}

// x (A, read only) -> out (A) = rmsnorm(x) * weight; no residual
template <typename A>
__global__ void rms_norm_kernel(const A * __restrict__ x, const float * __restrict__ weight,
                                A * __restrict__ out, int H, float eps) {
    __shared__ float scratch[32];
    const size_t base = (size_t) blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32(x[base + i]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float) H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        out[base + i] = from_f32<A>(to_f32(x[base + i]) * inv * weight[i]);
}

// gate_up rows are [gate (F) | up (F)] (interleave 0) or groups of 16 columns holding 8 gate values and
// then the 8 up values of the same features (interleave 8, the layout the fused product kernels want)
template <typename A>
__global__ void swiglu_kernel(const A * __restrict__ gate_up, A * __restrict__ out, int F, size_t total, int interleave) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t idx = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / F;
    const int col = (int) (idx - row * F);
    const size_t gi = interleave ? row * 2 * F + (size_t) (col / 8) * 16 + col % 8 : row * 2 * F + col;
    const size_t ui = interleave ? gi + 8 : gi + F;
    const float g = to_f32(gate_up[gi]);
    const float u = to_f32(gate_up[ui]);
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_f32<A>(s * u);
}

// 8 elements per thread with 16-byte (bf16) or 2 x 16-byte (f32) accesses; needs F % 8 == 0
template <typename A>
__global__ void swiglu_vec_kernel(const A * __restrict__ gate_up, A * __restrict__ out, int F, size_t groups, int interleave) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t gidx = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (gidx >= groups) return;
    const int per_row = F >> 3;
    const size_t row = gidx / per_row;
    const int col = (int) (gidx - row * per_row) << 3;
    const A * g = gate_up + row * 2 * F + (interleave ? 2 * col : col);
    const A * u = g + (interleave ? 8 : F);
    A * o = out + row * F + col;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float4 gv = Vec4<A>::load(g + 4 * h), uv = Vec4<A>::load(u + 4 * h);
        float4 r;
        r.x = gv.x / (1.0f + expf(-gv.x)) * uv.x;
        r.y = gv.y / (1.0f + expf(-gv.y)) * uv.y;
        r.z = gv.z / (1.0f + expf(-gv.z)) * uv.z;
        r.w = gv.w / (1.0f + expf(-gv.w)) * uv.w;
        Vec4<A>::store(o + 4 * h, r);
    }
}

template <typename T>
__global__ void gather_rows_kernel(const T * __restrict__ src, const int * __restrict__ rows,
                                   T * __restrict__ out, int H, int n_src) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = rows[blockIdx.x];
    T * o = out + (size_t) blockIdx.x * H;
    if (r < 0 || r >= n_src) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>(0.0f);
        return;
    }
    const T * s = src + (size_t) r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = s[i];
}

template <typename A>
__global__ void add_bias_kernel(A * __restrict__ x, const float * __restrict__ bias, int M, size_t total) {
    const size_t idx = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    x[idx] = from_f32<A>(to_f32(x[idx]) + bias[idx % M]);
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_embedding(const void * table, int table_dtype, const int * tokens, float * out,
                            int N, int H, int V, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == IIAN_F32) return iian_launch(embedding_kernel<float>, dim3(N), dim3(threads), 0, stream, (const float *) table, tokens, out, H, V);
    if (table_dtype == IIAN_BF16) return iian_launch(embedding_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, (const __nv_bfloat16 *) table, tokens, out, H, V);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_add_rms_norm(float * residual, const void * delta, const float * weight, void * out,
                               int act_dtype, int N, int H, float eps, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    if (act_dtype != IIAN_F32 && act_dtype != IIAN_BF16) return IIAN_ERR_DTYPE;
    // the launch shape is a function of H alone, so the order of every sum does not depend on the batch
    const bool aligned = H % 4 == 0 && ((uintptr_t) residual & 15) == 0 && ((uintptr_t) weight & 15) == 0 &&
                         ((uintptr_t) out & 7) == 0 && ((uintptr_t) delta & 7) == 0;
    if (aligned && H <= 4 * 4 * 1024) {
        const int groups = H / 4;
        int threads = 128;
        while (threads < 1024 && threads * 2 <= groups) threads *= 2;      // >= 2 groups per thread up to 1024 threads
        while (threads * 4 < groups) threads *= 2;
        if (threads > 1024) threads = 1024;
        if (act_dtype == IIAN_F32) return iian_launch(add_rms_norm_vec_kernel<float, 4>, dim3(N), dim3(threads), 0, stream, residual, (const float *) delta, weight, (float *) out, H, eps);
        return iian_launch(add_rms_norm_vec_kernel<__nv_bfloat16, 4>, dim3(N), dim3(threads), 0, stream, residual, (const __nv_bfloat16 *) delta, weight, (__nv_bfloat16 *) out, H, eps);
    }
    const int threads = 256;
    if (act_dtype == IIAN_F32) return iian_launch(add_rms_norm_kernel<float>, dim3(N), dim3(threads), 0, stream, residual, (const float *) delta, weight, (float *) out, H, eps);
    return iian_launch(add_rms_norm_kernel<__nv_bfloat16>, dim3(N), dim3(threads), 0, stream, residual, (const __nv_bfloat16 *) delta, weight, (__nv_bfloat16 *) out, H, eps);
}

IIAN_API int iian_rms_norm(const void * x, const float * weight, void * out, int act_dtype, int N, int H,
                           float eps, cudaStream_t stream) {
    if (N <= 0) return IIAN_OK;
    const int threads = H >= 512 ? 256 : 32;
    if (act_dtype == IIAN_F32) rms_norm_kernel<float><<<N, threads, 0, stream>>>((const float *) x, weight, (float *) out, H, eps);
    else if (act_dtype == IIAN_BF16) rms_norm_kernel<__nv_bfloat16><<<N, threads, 0, stream>>>((const __nv_bfloat16 *) x, weight, (__nv_bfloat16 *) out, H, eps);
    else return IIAN_ERR_DTYPE;
    return iian_launch_status();
}

IIAN_API int iian_swiglu(const void * gate_up, void * out, int act_dtype, int N, int F, int interleave, cudaStream_t stream) {
    if (interleave != 0 && (interleave != 8 || F % 8 != 0)) return IIAN_ERR_SHAPE;
    const size_t total = (size_t) N * F;
    if (total == 0) return IIAN_OK;
    const int threads = 256;
    if (F % 8 == 0 && ((uintptr_t) gate_up & 15) == 0 && ((uintptr_t) out & 15) == 0 && (act_dtype == IIAN_F32 || act_dtype == IIAN_BF16)) {
        const size_t groups = total / 8;
        const unsigned vblocks = (unsigned) ((groups + threads - 1) / threads);
        if (act_dtype == IIAN_F32) return iian_launch(swiglu_vec_kernel<float>, dim3(vblocks), dim3(threads), 0, stream, (const float *) gate_up, (float *) out, F, groups, interleave);
        return iian_launch(swiglu_vec_kernel<__nv_bfloat16>, dim3(vblocks), dim3(threads), 0, stream, (const __nv_bfloat16 *) gate_up, (__nv_bfloat16 *) out, F, groups, interleave);
    }
    const unsigned blocks = (unsigned) ((total + threads - 1) / threads);
    if (act_dtype == IIAN_F32) return iian_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float *) gate_up, (float *) out, F, total, interleave);
    if (act_dtype == IIAN_BF16) return iian_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16 *) gate_up, (__nv_bfloat16 *) out, F, total, interleave);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_gather_rows(const void * src, const int * rows, void * out, int dtype, int R, int H,
                              int n_src, cudaStream_t stream) {
    if (R <= 0) return IIAN_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == IIAN_F32) return iian_launch(gather_rows_kernel<float>, dim3(R), dim3(threads), 0, stream, (const float *) src, rows, (float *) out, H, n_src);
    if (dtype == IIAN_BF16) return iian_launch(gather_rows_kernel<__nv_bfloat16>, dim3(R), dim3(threads), 0, stream, (const __nv_bfloat16 *) src, rows, (__nv_bfloat16 *) out, H, n_src);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_add_bias(void * x, const float * bias, int act_dtype, int N, int M, cudaStream_t stream) {
    const size_t total = (size_t) N * M;
    if (total == 0) return IIAN_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned) ((total + threads - 1) / threads);
    if (act_dtype == IIAN_F32) add_bias_kernel<float><<<blocks, threads, 0, stream>>>((float *) x, bias, M, total);
    else if (act_dtype == IIAN_BF16) add_bias_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16 *) x, bias, M, total);
    else return IIAN_ERR_DTYPE;
    return iian_launch_status();
}
