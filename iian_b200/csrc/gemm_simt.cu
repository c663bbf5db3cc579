// out[n, m] = sum_k x[n, k] * w[m, k]: the plain matrix product of the 32-bit path, and the
// fallback for element-type combinations the tensor-core kernels do not take.
//
// Weights are row-major [out_features, in_features] exactly as the file stores them, which is
// also the reference's layout (ggml_mul_mat(W, x) = W x, src/iian/graph.cpp:121-160).  Products
// and sums are float32 FMAs (no reduced-precision matrix mode); every output element adds its
// K products in the order k = 0, 1, 2, ..., so a row's result does not depend on how many other
// rows the batch has.
#include "common.cuh"

namespace iian {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TX * __restrict__ x, const TW * __restrict__ w,
                                                        TO * __restrict__ out, int N, int M, int K) {
    __shared__ float xs[BK][BN + 4];
    __shared__ float ws[BK][BM + 4];
    const int tid = threadIdx.x;
    const int n0 = blockIdx.y * BN, m0 = blockIdx.x * BM;
    const int tx = tid % 16, ty = tid / 16;          // thread computes rows n0 + ty*4.., cols m0 + tx*4..
    const int lrow = tid / 4, lk = (tid % 4) * 4;    // loader: row of the tile, first k of 4
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int k = k0 + lk + e;
            const int n = n0 + lrow, m = m0 + lrow;
            xs[lk + e][lrow] = (n < N && k < K) ? to_f32(x[(size_t) n * K + k]) : 0.0f;
            ws[lk + e][lrow] = (m < M && k < K) ? to_f32(w[(size_t) m * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int n = n0 + ty * 4 + i;
        if (n >= N) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + tx * 4 + j;
            if (m < M) out[(size_t) n * M + m] = from_f32<TO>(acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TO>
static int launch(const void * x, const void * w, void * out, int N, int M, int K, cudaStream_t stream) {
    dim3 grid((M + BM - 1) / BM, (N + BN - 1) / BN);
    gemm_simt_kernel<TX, TW, TO><<<grid, 256, 0, stream>>>((const TX *) x, (const TW *) w, (TO *) out, N, M, K);
    return iian_launch_status();
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_gemm_simt(const void * x, int x_dtype, const void * w, int w_dtype, void * out, int out_dtype,
                            int N, int M, int K, cudaStream_t stream) {
    if (N <= 0 || M <= 0) return IIAN_OK;
    if (K <= 0) return IIAN_ERR_SHAPE;
    if ((M + BM - 1) / BM > 2147483647 || (N + BN - 1) / BN > 65535) return IIAN_ERR_LIMIT;
    typedef __nv_bfloat16 bf;
    const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case 0: return launch<float, float, float>(x, w, out, N, M, K, stream);
        case 1: return launch<float, float, bf>(x, w, out, N, M, K, stream);
        case 2: return launch<float, bf, float>(x, w, out, N, M, K, stream);
        case 3: return launch<float, bf, bf>(x, w, out, N, M, K, stream);
        case 4: return launch<bf, float, float>(x, w, out, N, M, K, stream);
        case 5: return launch<bf, float, bf>(x, w, out, N, M, K, stream);
        case 6: return launch<bf, bf, float>(x, w, out, N, M, K, stream);
        case 7: return launch<bf, bf, bf>(x, w, out, N, M, K, stream);
    }
    return IIAN_ERR_DTYPE;
}
