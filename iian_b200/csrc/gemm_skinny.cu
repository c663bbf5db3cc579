// out[n, m] = sum_k x[n, k] * w[m, k] for a handful of rows n (decode batches, 1..64): a
// weight-streaming kernel.  Every weight is read from HBM exactly once with 16-byte loads and fed
// straight into tensor-core MMAs (mma.sync m16n8k16, bf16 in, float32 accumulate); the weights sit in
// the 16-row operand, the batch in the 8-column operand ("swap AB"), so the batch size does not change
// how weights are fetched.
//
// The dot product does not care in which order k is walked, as long as both operands agree.  A thread
// therefore takes the 8 consecutive k of its 16-byte load as ITS k's of two MMA steps, and loads the
// activations at the same offsets: no shuffle, no shared-memory staging of the weights.
//
// A block owns 16 weight rows; its 8 warps split K in interleaved 32-wide chunks and add their partial
// sums through shared memory in a fixed order, so a result does not depend on the batch it is part of.
// The reference covers this regime with its own mat-vec kernels
// (third_party/ggml/src/ggml-cuda/mmvf.cu:8, mmf.cuh:50) before it falls back to cuBLAS.
#include "common.cuh"

namespace iian {

constexpr int kSkinnyWarps = 8;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ld_stream(const uint4 * p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float * c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, typename OutT>
__global__ void __launch_bounds__(kSkinnyWarps * 32) gemm_skinny_kernel(
    const __nv_bfloat16 * __restrict__ x, const __nv_bfloat16 * __restrict__ w, OutT * __restrict__ out,
    int B, int M, int K) {
    __shared__ float red[kSkinnyWarps][16][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.x * 16;
    const int r0 = min(m0 + g, M - 1), r1 = min(m0 + g + 8, M - 1);
    const uint4 * w0 = reinterpret_cast<const uint4 *>(w + (size_t) r0 * K) + t;
    const uint4 * w1 = reinterpret_cast<const uint4 *>(w + (size_t) r1 * K) + t;
    const uint4 * xr[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int n = min(nt * 8 + g, B - 1);
        xr[nt] = reinterpret_cast<const uint4 *>(x + (size_t) n * K) + t;
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;

    const int nchunks = K / 32;                      // a chunk = 32 k = 4 x 16 bytes per row
    int c = warp;
    for (; c + (kUnroll - 1) * kSkinnyWarps < nchunks; c += kUnroll * kSkinnyWarps) {
        uint4 a0[kUnroll], a1[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            a0[u] = ld_stream(w0 + (size_t) (c + u * kSkinnyWarps) * 4);
            a1[u] = ld_stream(w1 + (size_t) (c + u * kSkinnyWarps) * 4);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint4 b = __ldg(xr[nt] + (size_t) (c + u * kSkinnyWarps) * 4);
                mma_bf16_16816(acc[nt], a0[u].x, a1[u].x, a0[u].y, a1[u].y, b.x, b.y);
                mma_bf16_16816(acc[nt], a0[u].z, a1[u].z, a0[u].w, a1[u].w, b.z, b.w);
            }
        }
    }
    for (; c < nchunks; c += kSkinnyWarps) {
        const uint4 a0 = ld_stream(w0 + (size_t) c * 4);
        const uint4 a1 = ld_stream(w1 + (size_t) c * 4);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint4 b = __ldg(xr[nt] + (size_t) c * 4);
            mma_bf16_16816(acc[nt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
            mma_bf16_16816(acc[nt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        red[warp][g][nt * 8 + 2 * t] = acc[nt][0];
        red[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
        red[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
        red[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += blockDim.x) {
        const int n = idx / 16, r = idx % 16;
        const int m = m0 + r;
        if (n >= B || m >= M) continue;
        float s = 0.0f;
#pragma unroll
        for (int wv = 0; wv < kSkinnyWarps; wv++) s += red[wv][r][n];
        out[(size_t) n * M + m] = from_f32<OutT>(s);
    }
}

template <typename OutT>
static int launch_skinny(const void * x, const void * w, void * out, int B, int M, int K, cudaStream_t stream) {
    const unsigned blocks = (unsigned) ((M + 15) / 16);
    const int threads = kSkinnyWarps * 32;
    const __nv_bfloat16 * xp = (const __nv_bfloat16 *) x;
    const __nv_bfloat16 * wp = (const __nv_bfloat16 *) w;
    OutT * op = (OutT *) out;
    if (B <= 8) gemm_skinny_kernel<1, OutT><<<blocks, threads, 0, stream>>>(xp, wp, op, B, M, K);
    else if (B <= 16) gemm_skinny_kernel<2, OutT><<<blocks, threads, 0, stream>>>(xp, wp, op, B, M, K);
    else if (B <= 32) gemm_skinny_kernel<4, OutT><<<blocks, threads, 0, stream>>>(xp, wp, op, B, M, K);
    else gemm_skinny_kernel<8, OutT><<<blocks, threads, 0, stream>>>(xp, wp, op, B, M, K);
    return iian_launch_status();
}

}  // namespace iian

using namespace iian;

// x: [B, K] bf16, w: [M, K] bf16, out: [B, M] bf16 or f32.  Needs 1 <= B <= 64, K a multiple of 32
// and 16-byte aligned x and w (rows are then aligned too).
IIAN_API int iian_gemm_skinny(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K,
                              cudaStream_t stream) {
    if (B <= 0 || M <= 0) return IIAN_OK;
    if (B > 64) return IIAN_ERR_LIMIT;
    if (K <= 0 || K % 32 != 0) return IIAN_ERR_SHAPE;
    if (((uintptr_t) x & 15) || ((uintptr_t) w & 15)) return IIAN_ERR_ALIGN;
    if (out_dtype == IIAN_BF16) return launch_skinny<__nv_bfloat16>(x, w, out, B, M, K, stream);
    if (out_dtype == IIAN_F32) return launch_skinny<float>(x, w, out, B, M, K, stream);
    return IIAN_ERR_DTYPE;
}
