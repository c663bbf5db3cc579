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

// Weights are read once per step: their lines are marked as the first to leave the L2, so that the matrix that
// is streaming through does not push out what other kernels of the step keep there (activations, the cache
// pages of the live requests, what the prefetcher brought in for the next product).  Measured on B200 at the
// Qwen3-8B sizes: 3.48 -> 3.36 ms per decode step at batch 1.
__device__ __forceinline__ uint64_t stream_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// (The policy is made anew beside every load on purpose: one policy kept in registers for the whole kernel
// measured 3.41 ms per step against 3.23 ms -- the compiler then fits the 8-warp kernels into 64 registers with
// spills for a fourth CTA per SM, and the loads of a round are issued less densely.)
__device__ __forceinline__ uint4 ld_stream(const uint4 * p) {
    uint4 v;
    const uint64_t policy = stream_policy();
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(policy));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float * c, unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// What the fused forms of the epilogue need (all null / zero: plain product).
//  * in_partial: the activations are a residual stream times a norm weight, not yet normalised; the sums of
//    squares of its rows come as in_tiles partial sums per row ([B, in_tiles]); the kernel multiplies row n
//    of its result by rsqrt(sum / width + eps) (RMSNorm commutes with the product: it is a factor per row,
//    src/iian/graph.cpp:105-114).
//  * res / norm_w / out_partial (EPI 2): the product is the output of a sub-layer.  The kernel rounds it to
//    bfloat16 as the unfused route would store it, adds it to the float32 residual stream res [B, M] in
//    place, stores res * norm_w as bfloat16 (the input of the next product, not yet normalised) and leaves
//    the sum of squares of its 16 columns of every row in out_partial [B, tiles] for the consumer above.
struct SkinnyExtra {
    const float * in_partial;
    int in_tiles;
    float inv_width, eps;
    float * res;
    const float * norm_w;
    float * out_partial;
};

// NT: 8-column tiles of the batch; MT: 16-row tiles of weights per block (they share the activation
// fragments); WARPS: how many warps split K; UNROLL: 32-wide k chunks whose weight loads are issued
// before the first of them is used.
// EPI 0: store the products.  EPI 1: the weight rows hold gate and up projections interleaved in groups of
// 8 (rows 16j..16j+7 gate, 16j+8..16j+15 up, same 8 features); the kernel stores silu(gate) * up, half as
// many columns (src/iian/graph.cpp:135).
// (No minimum of CTAs per SM is stated on purpose: 2, 3 and 4 all measured slower than the compiler's own
// choice of 78 to 80 registers for the 8-warp forms, three CTAs per SM.)
template <int NT, int MT, int WARPS, int UNROLL, int EPI, typename OutT>
__global__ void __launch_bounds__(WARPS * 32) gemm_skinny_kernel(
    const __nv_bfloat16 * __restrict__ x, const __nv_bfloat16 * __restrict__ w, OutT * __restrict__ out,
    int B, int M, int K, float * __restrict__ part, int * __restrict__ counters, const SkinnyExtra ex) {
    extern __shared__ float red_raw[];
    __shared__ int s_last;
    __shared__ float s_rs[8];
    float (*red)[MT * 16][NT * 8 + 1] = reinterpret_cast<float (*)[MT * 16][NT * 8 + 1]>(red_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.x * (16 * MT);
    const uint4 * w0[MT];
    const uint4 * w1[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const int r0 = min(m0 + mt * 16 + g, M - 1), r1 = min(m0 + mt * 16 + g + 8, M - 1);
        w0[mt] = reinterpret_cast<const uint4 *>(w + (size_t) r0 * K) + t;
        w1[mt] = reinterpret_cast<const uint4 *>(w + (size_t) r1 * K) + t;
    }
    const uint4 * xr[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int n = min(nt * 8 + g, B - 1);
        xr[nt] = reinterpret_cast<const uint4 *>(x + (size_t) n * K) + t;
    }
    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[mt][nt][i] = 0.0f;

    const int nchunks = K / 32;                      // a chunk = 32 k = 4 x 16 bytes per row
    uint4 a0[UNROLL][MT], a1[UNROLL][MT];
    auto load_round = [&](int c) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                a0[u][mt] = ld_stream(w0[mt] + (size_t) (c + u * WARPS) * 4);
                a1[u][mt] = ld_stream(w1[mt] + (size_t) (c + u * WARPS) * 4);
            }
    };
    auto compute_round = [&](int c) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint4 b = __ldg(xr[nt] + (size_t) (c + u * WARPS) * 4);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    mma_bf16_16816(acc[mt][nt], a0[u][mt].x, a1[u][mt].x, a0[u][mt].y, a1[u][mt].y, b.x, b.y);
                    mma_bf16_16816(acc[mt][nt], a0[u][mt].z, a1[u][mt].z, a0[u][mt].w, a1[u][mt].w, b.z, b.w);
                }
            }
        }
    };
    // The weights do not depend on the kernel before this one: the first round of loads is in flight
    // before this kernel waits for its activations.
    // gridDim.y CTAs split K between them (contiguous ranges of chunks); inside a CTA the warps interleave
    const int ksplit = gridDim.y, ks = blockIdx.y;
    const int c_begin = (int) ((long long) nchunks * ks / ksplit), c_end = (int) ((long long) nchunks * (ks + 1) / ksplit);
    int c = c_begin + warp;
    const bool scaled = NT == 1 && ex.in_partial != nullptr;
    auto row_factors = [&]() {                       // row n's factor: one warp adds its partial sums in a fixed order
        if constexpr (NT == 1) {
            if (scaled) {
                for (int n = warp; n < B; n += WARPS) {
                    float a = 0.0f;
                    for (int i = lane; i < ex.in_tiles; i += 32) a += ex.in_partial[(size_t) n * ex.in_tiles + i];
                    a = warp_sum(a);
                    if (lane == 0) s_rs[n] = rsqrtf(a * ex.inv_width + ex.eps);
                }
            }
        }
    };
    const bool first_round = c + (UNROLL - 1) * WARPS < c_end;
    if (first_round) load_round(c);
    pdl_wait();
    row_factors();
    if (first_round) {
        compute_round(c);
        c += UNROLL * WARPS;
    }
    for (; c + (UNROLL - 1) * WARPS < c_end; c += UNROLL * WARPS) {
        load_round(c);
        compute_round(c);
    }
    for (; c < c_end; c += WARPS) {
        uint4 t0[MT], t1[MT];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            t0[mt] = ld_stream(w0[mt] + (size_t) c * 4);
            t1[mt] = ld_stream(w1[mt] + (size_t) c * 4);
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint4 b = __ldg(xr[nt] + (size_t) c * 4);
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                mma_bf16_16816(acc[mt][nt], t0[mt].x, t1[mt].x, t0[mt].y, t1[mt].y, b.x, b.y);
                mma_bf16_16816(acc[mt][nt], t0[mt].z, t1[mt].z, t0[mt].w, t1[mt].w, b.z, b.w);
            }
        }
    }
    // The weights are read: let the next kernel of the chain start (it waits for this grid's results
    // before it touches them).  Triggering earlier would let a whole cascade of future kernels become
    // resident and spin, taking registers and shared memory from the kernel that is actually running.
    pdl_launch_dependents();
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            red[warp][mt * 16 + g][nt * 8 + 2 * t] = acc[mt][nt][0];
            red[warp][mt * 16 + g][nt * 8 + 2 * t + 1] = acc[mt][nt][1];
            red[warp][mt * 16 + g + 8][nt * 8 + 2 * t] = acc[mt][nt][2];
            red[warp][mt * 16 + g + 8][nt * 8 + 2 * t + 1] = acc[mt][nt][3];
        }
    __syncthreads();
    constexpr int ROWS = MT * 16;
    constexpr int CELLS = ROWS * NT * 8;
    if (EPI == 1) {                                  // (ksplit is 1 here)
        for (int idx = threadIdx.x; idx < CELLS / 2; idx += blockDim.x) {
            const int n = idx / (ROWS / 2), f = idx % (ROWS / 2);
            const int r = (f / 8) * 16 + f % 8;      // gate row; its up row is 8 further
            const int m = m0 + r;
            if (n >= B || m + 8 >= M) continue;
            float g = 0.0f, u = 0.0f;
#pragma unroll
            for (int wv = 0; wv < WARPS; wv++) { g += red[wv][r][n]; u += red[wv][r + 8][n]; }
            if (scaled) { g *= s_rs[n]; u *= s_rs[n]; }
            out[(size_t) n * (M / 2) + (m0 / 2 + f)] = from_f32<OutT>(g / (1.0f + expf(-g)) * u);
        }
        return;
    }
    if (EPI == 2) {                                  // (ksplit is 1, NT is 1: CELLS is a multiple of 32)
        for (int idx = threadIdx.x; idx < CELLS; idx += blockDim.x) {
            const int n = idx / ROWS, r = idx % ROWS;
            const int m = m0 + r;
            float s = 0.0f;
#pragma unroll
            for (int wv = 0; wv < WARPS; wv++) s += red[wv][r][n];
            if (scaled) s *= s_rs[n];
            float rn = 0.0f;
            if (n < B && m < M) {
                const size_t at = (size_t) n * M + m;
                rn = ex.res[at] + __bfloat162float(__float2bfloat16_rn(s));
                ex.res[at] = rn;
                out[at] = from_f32<OutT>(rn * ex.norm_w[m]);
            }
            float sq = rn * rn;                      // the ROWS cells of a row of the batch are consecutive lanes
#pragma unroll
            for (int o = ROWS / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (r == 0 && n < B) ex.out_partial[(size_t) n * gridDim.x + blockIdx.x] = sq;
        }
        return;
    }
    if (ksplit == 1) {
        for (int idx = threadIdx.x; idx < CELLS; idx += blockDim.x) {
            const int n = idx / ROWS, r = idx % ROWS;
            const int m = m0 + r;
            if (n >= B || m >= M) continue;
            float s = 0.0f;
#pragma unroll
            for (int wv = 0; wv < WARPS; wv++) s += red[wv][r][n];      // fixed order: independent of the batch
            if (scaled) s *= s_rs[n];
            out[(size_t) n * M + m] = from_f32<OutT>(s);
        }
        return;
    }
    // split K: every CTA leaves its partial sums in scratch; the CTA that arrives last for this row block
    // adds the parts in the order of their index (not of their arrival) and writes the result
    float * mine = part + ((size_t) blockIdx.x * ksplit + ks) * CELLS;
    for (int idx = threadIdx.x; idx < CELLS; idx += blockDim.x) {
        const int n = idx / ROWS, r = idx % ROWS;
        float s = 0.0f;
#pragma unroll
        for (int wv = 0; wv < WARPS; wv++) s += red[wv][r][n];
        mine[idx] = s;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(counters + blockIdx.x, 1) == ksplit - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float * all = part + (size_t) blockIdx.x * ksplit * CELLS;
    for (int idx = threadIdx.x; idx < CELLS; idx += blockDim.x) {
        const int n = idx / ROWS, r = idx % ROWS;
        const int m = m0 + r;
        if (n >= B || m >= M) continue;
        float s = 0.0f;
        for (int i = 0; i < ksplit; i++) s += __ldcg(all + (size_t) i * CELLS + idx);
        out[(size_t) n * M + m] = from_f32<OutT>(s);
    }
    if (threadIdx.x == 0) counters[blockIdx.x] = 0;
}

template <int NT, int MT, int WARPS, int UNROLL, int EPI, typename OutT>
static int launch_cfg(const void * x, const void * w, void * out, int B, int M, int K, int ksplit, float * part,
                      int * counters, const SkinnyExtra & ex, cudaStream_t stream) {
    const unsigned blocks = (unsigned) ((M + 16 * MT - 1) / (16 * MT));
    constexpr size_t smem = sizeof(float) * WARPS * MT * 16 * (NT * 8 + 1);
    if (smem > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NT, MT, WARPS, UNROLL, EPI, OutT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
            if (e != cudaSuccess) return 1000 + (int) e;
            configured = true;
        }
    }
    return iian_launch(gemm_skinny_kernel<NT, MT, WARPS, UNROLL, EPI, OutT>, dim3(blocks, ksplit), dim3(WARPS * 32), smem, stream,
                       (const __nv_bfloat16 *) x, (const __nv_bfloat16 *) w, (OutT *) out, B, M, K, part, counters, ex);
}

// cfg = MT * 100 + WARPS * 10 + UNROLL; 0 = the default for this (B, M)
template <int NT, int EPI, typename OutT>
static int launch_nt(const void * x, const void * w, void * out, int B, int M, int K, int cfg, int ksplit, float * part,
                     int * counters, const SkinnyExtra & ex, cudaStream_t stream) {
    if (cfg == 0) {
        if (NT == 1) cfg = M >= 65536 ? 144 : (K >= 8192 ? 188 : 184);
        else if (NT == 2) cfg = 284;
        else cfg = 282;
    }
    if (NT == 1) {
        switch (cfg) {
            case 184: return launch_cfg<1, 1, 8, 4, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, ex, stream);
            case 188: return launch_cfg<1, 1, 8, 8, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, ex, stream);
            case 144: return launch_cfg<1, 1, 4, 4, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, ex, stream);
            case 148: return launch_cfg<1, 1, 4, 8, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, ex, stream);
        }
        return IIAN_ERR_SHAPE;
    }
    switch (cfg) {
        case 284: return launch_cfg<NT, 2, 8, 4, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, ex, stream);
        case 282: return launch_cfg<NT, 2, 8, 2, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, ex, stream);
    }
    return IIAN_ERR_SHAPE;
}

template <int EPI, typename OutT>
static int launch_skinny(const void * x, const void * w, void * out, int B, int M, int K, int cfg, int ksplit, float * part,
                         int * counters, const SkinnyExtra & ex, cudaStream_t stream) {
    if (B <= 8) return launch_nt<1, EPI, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, ex, stream);
    if (EPI != 0 || ex.in_partial != nullptr) return IIAN_ERR_LIMIT;      // the fused forms are built for up to 8 rows
    if (B <= 16) return launch_nt<2, 0, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, ex, stream);
    if (B <= 32) return launch_nt<4, 0, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, ex, stream);
    return launch_nt<8, 0, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, ex, stream);
}

}  // namespace iian

using namespace iian;

// x: [B, K] bf16, w: [M, K] bf16, out: [B, M] bf16 or f32.  Needs 1 <= B <= 64, K a multiple of 32
// and 16-byte aligned x and w (rows are then aligned too).  cfg selects a tile configuration
// (MT * 100 + WARPS * 10 + UNROLL); 0 takes the default.  ksplit > 1 cuts K over that many CTAs per row
// block and needs scratch: part = ceil(M / rows per block) * ksplit * (rows per block * 8 * ceil(B / 8))
// floats and counters = ceil(M / rows per block) ints that are zero before the first launch (the kernel
// leaves them zero).  epilogue 1 stores silu(gate) * up for gate/up rows interleaved in groups of 8 (out is
// [B, M / 2] bf16; up to 8 rows, no split).
static int skinny_entry(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K,
                        int cfg, int ksplit, float * part, int * counters, int epilogue, const SkinnyExtra & ex,
                        cudaStream_t stream) {
    if (B <= 0 || M <= 0) return IIAN_OK;
    if (B > 64) return IIAN_ERR_LIMIT;
    if (K <= 0 || K % 32 != 0) return IIAN_ERR_SHAPE;
    if (((uintptr_t) x & 15) || ((uintptr_t) w & 15)) return IIAN_ERR_ALIGN;
    if (ksplit < 1 || ksplit > 64 || ksplit > K / 32) return IIAN_ERR_SHAPE;
    if (ksplit > 1 && (part == nullptr || counters == nullptr)) return IIAN_ERR_SHAPE;
    if (ex.in_partial != nullptr && (B > 8 || ex.in_tiles <= 0 || ksplit != 1)) return IIAN_ERR_SHAPE;
    if (epilogue == 1) {
        if (M % 16 != 0 || ksplit != 1 || out_dtype != IIAN_BF16) return IIAN_ERR_SHAPE;
        return launch_skinny<1, __nv_bfloat16>(x, w, out, B, M, K, cfg, 1, nullptr, nullptr, ex, stream);
    }
    if (epilogue == 2) {
        if (B > 8 || ksplit != 1 || out_dtype != IIAN_BF16 || ex.res == nullptr || ex.norm_w == nullptr ||
            ex.out_partial == nullptr) return IIAN_ERR_SHAPE;
        return launch_skinny<2, __nv_bfloat16>(x, w, out, B, M, K, cfg, 1, nullptr, nullptr, ex, stream);
    }
    if (epilogue != 0) return IIAN_ERR_SHAPE;
    if (out_dtype == IIAN_BF16) return launch_skinny<0, __nv_bfloat16>(x, w, out, B, M, K, cfg, ksplit, part, counters, ex, stream);
    if (out_dtype == IIAN_F32) return launch_skinny<0, float>(x, w, out, B, M, K, cfg, ksplit, part, counters, ex, stream);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_gemm_skinny_cfg(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K,
                                  int cfg, int ksplit, float * part, int * counters, int epilogue, cudaStream_t stream) {
    if (epilogue == 2) return IIAN_ERR_SHAPE;
    const SkinnyExtra none = {nullptr, 0, 0.0f, 0.0f, nullptr, nullptr, nullptr};
    return skinny_entry(x, w, out, out_dtype, B, M, K, cfg, ksplit, part, counters, epilogue, none, stream);
}

// The product with its fused forms (up to 8 rows).  in_partial [B, in_tiles] (or null): sums of squares of the
// rows of the not yet normalised input, in parts; the result's row n is multiplied by
// rsqrt(sum / width + eps) with inv_width = 1 / width.  epilogue 2: out = bf16(res * norm_w) after
// res [B, M] float32 += bf16(product), and out_partial [B, tiles_out] receives the sums of squares of res per
// block of rows of w (iian_gemm_skinny_tiles says how many blocks there are).
IIAN_API int iian_gemm_skinny_fused(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K, int epilogue,
                                    const float * in_partial, int in_tiles, float inv_width, float eps,
                                    float * res, const float * norm_w, float * out_partial, cudaStream_t stream) {
    const SkinnyExtra ex = {in_partial, in_tiles, inv_width, eps, res, norm_w, out_partial};
    return skinny_entry(x, w, out, out_dtype, B, M, K, 0, 1, nullptr, nullptr, epilogue, ex, stream);
}

// blocks of rows of w the default configuration for up to 8 rows cuts M into (16 rows each)
IIAN_API int iian_gemm_skinny_tiles(int M) { return (M + 15) / 16; }

IIAN_API int iian_gemm_skinny(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K,
                              cudaStream_t stream) {
    return iian_gemm_skinny_cfg(x, w, out, out_dtype, B, M, K, 0, 1, nullptr, nullptr, 0, stream);
}
