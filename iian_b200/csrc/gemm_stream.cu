// out[n, m] = sum_k x[n, k] * w[m, k] for up to 8 rows n (decode steps): the weights stream through a ring of
// shared-memory stages filled by bulk asynchronous copies, so that the bytes in flight per SM do not depend on
// registers and the stream does not stop between row blocks.
//
// A CTA is persistent: it walks the 16-row blocks b = blockIdx.x, blockIdx.x + gridDim.x, ...  One producer warp
// issues, per stage, sixteen `cp.async.bulk` copies of 1 KB -- 512 k of one weight row each, contiguous in
// memory -- that complete on the stage's mbarrier; it runs ahead of the consumers by the depth of the ring, also
// across row blocks.  Eight consumer warps split the 32-k chunks of a stage between them (chunk c goes to warp
// c mod 8, the split of gemm_skinny.cu), read their 16 bytes of two weight rows from shared memory and the same
// k of the activations from global memory, and feed `mma.sync` m16n8k16 (weights in the 16-row operand, the
// batch in the 8-column operand).  A row's stage occupies 1088 bytes, 64 more than it holds, so that the eight
// rows a quarter warp reads lie in different banks.  Sums per warp are added through shared memory in a fixed
// order: the result is the one gemm_skinny.cu gives, bit for bit, and the epilogues are the same (store; SiLU(gate)
// * up for interleaved gate / up rows; residual add + next norm's weight + sums of squares; a factor per row from
// such sums).  Weight lines carry the evict-first L2 policy: they are read once per step.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records where it gave up in `status`
// and raises a flag in shared memory; every role then runs to the common exit without computing (the producer
// first waits, bounded again, for the copies it has in flight).
#include "common.cuh"

namespace iian {

constexpr int GS_ROWS = 16;                 // weight rows of a block
// k per stage: a bulk copy brings GS_KC * 2 bytes of one weight row.  The copy engine of an SM handles a limited
// number of requests per second, whatever their size: with 1 KB requests (512 k) the kernel reached 2.8 to 5.2 TB/s,
// with 2 KB 3.9 to 6.8, with 4 KB 4.1 to 7.0 (output projection / vocabulary projection of the Qwen3-8B shape).
#ifndef IIAN_GS_KC
#define IIAN_GS_KC 2048
#endif
#ifndef IIAN_GS_STAGES_2
#define IIAN_GS_STAGES_2 1                  // ring depth with two CTAs per SM
#endif
#ifndef IIAN_GS_STAGES_1
#define IIAN_GS_STAGES_1 3                  // ring depth with one CTA per SM
#endif
constexpr int GS_KC = IIAN_GS_KC;           // k per stage
constexpr int GS_ROW_STRIDE = GS_KC * 2 + 64;   // bytes between the rows of a stage (64 more than it holds: bank spread)
constexpr int GS_STAGE_BYTES = GS_ROWS * GS_ROW_STRIDE;
constexpr int GS_WARPS = 8;                 // consumer warps
constexpr int GS_THREADS = (GS_WARPS + 1) * 32;
constexpr unsigned kGsSpinLimit = 2u * 1000u * 1000u;

struct StreamExtra {                        // as SkinnyExtra of gemm_skinny.cu
    const float * in_partial;
    int in_tiles;
    float inv_width, eps;
    float * res;
    const float * norm_w;
    float * out_partial;
};

__device__ __forceinline__ unsigned gs_smem(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void gs_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void gs_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gs_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool gs_wait(unsigned bar, unsigned parity) {
    for (unsigned spin = 0; spin < kGsSpinLimit; spin++) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void gs_bulk_load(unsigned dst, const void * src, unsigned bytes, unsigned bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
__device__ __forceinline__ void gs_mma(float * c, unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void gs_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GS_WARPS * 32) : "memory"); }

template <int STAGES, int EPI, int XREG, typename OutT>
__global__ void __launch_bounds__(GS_THREADS) gemm_stream_kernel(
    const __nv_bfloat16 * __restrict__ x, const __nv_bfloat16 * __restrict__ w, OutT * __restrict__ out,
    int B, int M, int K, const StreamExtra ex, int * __restrict__ status) {
    extern __shared__ __align__(128) unsigned char gs_raw[];
    unsigned char * ring = gs_raw;                                              // [STAGES][16][1088]
    float (*red)[GS_ROWS][9] = reinterpret_cast<float (*)[GS_ROWS][9]>(gs_raw + (size_t) STAGES * GS_STAGE_BYTES);   // [8][16][9]
    __shared__ __align__(8) unsigned long long full[STAGES], empty[STAGES];
    __shared__ float s_rs[8];
    __shared__ int s_failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_blocks = (M + GS_ROWS - 1) / GS_ROWS;
    const int n_st = (K + GS_KC - 1) / GS_KC;
    const int nchunks = K / 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            gs_mbar_init(gs_smem(&full[s]), 1);
            gs_mbar_init(gs_smem(&empty[s]), GS_WARPS);
        }
        s_failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Launched with programmatic stream serialization, this grid may start while the one before it drains: the
    // producer fills the ring at once (weights do not depend on the kernel before), the consumers first wait for
    // the grid before to complete.  The grid after this one may be launched as soon as SMs become free.
    pdl_launch_dependents();
    const bool scaled = ex.in_partial != nullptr;
    if (warp < GS_WARPS) {
        pdl_wait();
        if (scaled) {                           // row n's factor: one warp adds its partial sums in a fixed order
            for (int n = warp; n < B; n += GS_WARPS) {
                float a = 0.0f;
                for (int i = lane; i < ex.in_tiles; i += 32) a += ex.in_partial[(size_t) n * ex.in_tiles + i];
                a = warp_sum(a);
                if (lane == 0) s_rs[n] = rsqrtf(a * ex.inv_width + ex.eps);
            }
        }
        gs_consumer_sync();
    }
    volatile int * failed = &s_failed;

    if (warp == GS_WARPS) {
        // ---- producer -------------------------------------------------------------------------------------
        uint64_t policy;
        asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
        unsigned it = 0;
        bool ok = true;
        for (int b = blockIdx.x; ok && b < n_blocks; b += gridDim.x) {
            const int m0 = b * GS_ROWS;
            const int rows_valid = min(GS_ROWS, M - m0);
            for (int s = 0; s < n_st; s++, it++) {
                const unsigned slot = it % STAGES, ph = (it / STAGES) & 1u;
                const unsigned bytes_row = (unsigned) min(GS_KC, K - s * GS_KC) * 2u;
                int good = 1;
                if (lane == 0) {
                    if (*failed || !gs_wait(gs_smem(&empty[slot]), ph ^ 1u)) {
                        if (!*failed) { status[0] = 21; status[1] = (int) it; s_failed = 1; }
                        good = 0;
                    } else {
                        gs_expect_tx(gs_smem(&full[slot]), bytes_row * (unsigned) rows_valid);
                    }
                }
                good = __shfl_sync(0xffffffffu, good, 0);
                if (!good) { ok = false; break; }
                if (lane < rows_valid)
                    gs_bulk_load(gs_smem(ring + (size_t) slot * GS_STAGE_BYTES + lane * GS_ROW_STRIDE),
                                 w + (size_t) (m0 + lane) * K + (size_t) s * GS_KC, bytes_row, gs_smem(&full[slot]), policy);
            }
        }
        if (!ok && lane == 0) {                  // the copies in flight land in this CTA's shared memory: wait for them
            const unsigned issued = it < (unsigned) STAGES ? it : (unsigned) STAGES;
            for (unsigned j = 0; j < issued; j++) {
                const unsigned jt = it - 1 - j;
                gs_wait(gs_smem(&full[jt % STAGES]), (jt / STAGES) & 1u);
            }
        }
        return;
    }

    // ---- consumers -------------------------------------------------------------------------------------------
    // The activations a thread needs do not change from row block to row block: chunk c of row g, 16 bytes at t.
    // XREG > 0 (K up to XREG * 256): they are loaded once into XREG registers of 16 bytes.  XREG == 0: they are
    // fetched from global memory (they stay in L2) one stage ahead of their use, round and round.
    const int g = lane >> 2, t = lane & 3;
    const uint4 * xr = reinterpret_cast<const uint4 *>(x + (size_t) min(g, B - 1) * K) + t;
    constexpr int PER_STAGE = GS_KC / 32 / GS_WARPS;      // chunks of a stage per warp
    constexpr int XR = XREG > 0 ? XREG : 1;
    uint4 xb[XR];
    if (XREG > 0) {
#pragma unroll
        for (int i = 0; i < XR; i++) {
            const int c = (i / PER_STAGE) * (GS_KC / 32) + (i % PER_STAGE) * GS_WARPS + warp;
            xb[i] = c < nchunks ? __ldg(xr + (size_t) c * 4) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    auto fetch = [&](int s_, uint4 * dst) {                // the activations of stage s_ (of any row block) for this warp
#pragma unroll
        for (int i = 0; i < PER_STAGE; i++) {
            const int c = s_ * (GS_KC / 32) + i * GS_WARPS + warp;
            dst[i] = c < nchunks ? __ldg(xr + (size_t) c * 4) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    auto stage = [&](unsigned it, int s_, float * acc, const uint4 * bx) {
        const unsigned slot = it % STAGES, ph = (it / STAGES) & 1u;
        const int last = min(nchunks, (s_ + 1) * (GS_KC / 32));
        if (!*failed && !gs_wait(gs_smem(&full[slot]), ph)) {
            if (lane == 0 && !*failed) { status[0] = 22; status[1] = (int) it; }
            s_failed = 1;
        }
        if (*failed) return;
        const unsigned char * st = ring + (size_t) slot * GS_STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < PER_STAGE; i++) {
            const int cl = i * GS_WARPS + warp;             // chunk within the stage
            if (s_ * (GS_KC / 32) + cl < last) {
                const uint4 a0 = *reinterpret_cast<const uint4 *>(st + g * GS_ROW_STRIDE + (cl * 4 + t) * 16);
                const uint4 a1 = *reinterpret_cast<const uint4 *>(st + (g + 8) * GS_ROW_STRIDE + (cl * 4 + t) * 16);
                gs_mma(acc, a0.x, a1.x, a0.y, a1.y, bx[i].x, bx[i].y);
                gs_mma(acc, a0.z, a1.z, a0.w, a1.w, bx[i].z, bx[i].w);
            }
        }
        __syncwarp();
        if (lane == 0) gs_arrive(gs_smem(&empty[slot]));
    };
    // the eight warps' sums of row block b, in a fixed order; then the epilogue; the sums start again at zero
    auto finish_block = [&](int b, float * acc) {
        const int m0 = b * GS_ROWS;
        // ---- the eight warps' sums, in a fixed order; then the epilogue --------------------------------------
        gs_consumer_sync();                         // the block before has been written out: red is free
        red[warp][g][2 * t] = acc[0];
        red[warp][g][2 * t + 1] = acc[1];
        red[warp][g + 8][2 * t] = acc[2];
        red[warp][g + 8][2 * t + 1] = acc[3];
        gs_consumer_sync();
        if (*failed) return;
        constexpr int CELLS = GS_ROWS * 8;
        const int tid = threadIdx.x;                // 0 .. 255
        if (EPI == 1) {
            if (tid < CELLS / 2) {
                const int n = tid / (GS_ROWS / 2), f = tid % (GS_ROWS / 2);
                const int r = f;                    // gate row (rows 0..7); its up row is 8 further
                const int m = m0 + r;
                if (n < B && m + 8 < M) {
                    float gt = 0.0f, up = 0.0f;
#pragma unroll
                    for (int wv = 0; wv < GS_WARPS; wv++) { gt += red[wv][r][n]; up += red[wv][r + 8][n]; }
                    if (scaled) { gt *= s_rs[n]; up *= s_rs[n]; }
                    out[(size_t) n * (M / 2) + (m0 / 2 + f)] = from_f32<OutT>(gt / (1.0f + expf(-gt)) * up);
                }
            }
        } else if (EPI == 2) {
            if (tid < CELLS) {                      // the 16 cells of a row of the batch are consecutive lanes
                const int n = tid / GS_ROWS, r = tid % GS_ROWS;
                const int m = m0 + r;
                float sum = 0.0f;
#pragma unroll
                for (int wv = 0; wv < GS_WARPS; wv++) sum += red[wv][r][n];
                if (scaled) sum *= s_rs[n];
                float rn = 0.0f;
                if (n < B && m < M) {
                    const size_t at = (size_t) n * M + m;
                    rn = ex.res[at] + __bfloat162float(__float2bfloat16_rn(sum));
                    ex.res[at] = rn;
                    out[at] = from_f32<OutT>(rn * ex.norm_w[m]);
                }
                float sq = rn * rn;
#pragma unroll
                for (int o = GS_ROWS / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (r == 0 && n < B) ex.out_partial[(size_t) n * n_blocks + b] = sq;
            }
        } else {
            if (tid < CELLS) {
                const int n = tid / GS_ROWS, r = tid % GS_ROWS;
                const int m = m0 + r;
                if (n < B && m < M) {
                    float sum = 0.0f;
#pragma unroll
                    for (int wv = 0; wv < GS_WARPS; wv++) sum += red[wv][r][n];
                    if (scaled) sum *= s_rs[n];
                    out[(size_t) n * M + m] = from_f32<OutT>(sum);
                }
            }
        }
        acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
    };
    unsigned it = 0;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (XREG > 0) {
        for (int b = blockIdx.x; b < n_blocks; b += gridDim.x) {
#pragma unroll
            for (int s_ = 0; s_ < XR / PER_STAGE; s_++)
                if (s_ < n_st) { stage(it, s_, acc, xb + s_ * PER_STAGE); it++; }
            finish_block(b, acc);
        }
    } else {
        // two sets of registers: while a stage is multiplied with one, the next stage's activations arrive in the other
        uint4 pa[PER_STAGE], pb[PER_STAGE];
        int b = blockIdx.x, s_ = 0;
        if (b >= n_blocks) return;
        fetch(0, pa);
        for (;;) {
            fetch(s_ + 1 == n_st ? 0 : s_ + 1, pb);
            stage(it++, s_, acc, pa);
            if (++s_ == n_st) { finish_block(b, acc); s_ = 0; b += gridDim.x; if (b >= n_blocks) break; }
            fetch(s_ + 1 == n_st ? 0 : s_ + 1, pa);
            stage(it++, s_, acc, pb);
            if (++s_ == n_st) { finish_block(b, acc); s_ = 0; b += gridDim.x; if (b >= n_blocks) break; }
        }
    }
}

static int gs_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms = n;
    }
    return sms;
}

static int g_stream_stages = 12;            // 12: one CTA per SM with the deep ring; 6: two CTAs per SM with the shallow one

template <int STAGES, int EPI, int XREG, typename OutT>
static int gs_launch_x(const void * x, const void * w, void * out, int B, int M, int K, const StreamExtra & ex, int * status,
                       cudaStream_t stream) {
    constexpr size_t smem = (size_t) STAGES * GS_STAGE_BYTES + sizeof(float) * GS_WARPS * GS_ROWS * 9;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<STAGES, EPI, XREG, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return 1000 + (int) e;
        configured = true;
    }
    const int n_blocks = (M + GS_ROWS - 1) / GS_ROWS;
    const int per_sm = STAGES == IIAN_GS_STAGES_2 ? 2 : 1;
    const int grid = n_blocks < per_sm * gs_sm_count() ? n_blocks : per_sm * gs_sm_count();
    return iian_launch(gemm_stream_kernel<STAGES, EPI, XREG, OutT>, dim3((unsigned) grid), dim3(GS_THREADS), smem, stream,
                       (const __nv_bfloat16 *) x, (const __nv_bfloat16 *) w, (OutT *) out, B, M, K, ex, status);
}

// activations in registers for K up to 4096 (16 registers of 16 bytes a thread), fetched ahead from L2 beyond
template <int STAGES, int EPI, typename OutT>
static int gs_launch(const void * x, const void * w, void * out, int B, int M, int K, const StreamExtra & ex, int * status,
                     cudaStream_t stream) {
    if (K <= 16 * 256) return gs_launch_x<STAGES, EPI, 16, OutT>(x, w, out, B, M, K, ex, status, stream);
    return gs_launch_x<STAGES, EPI, 0, OutT>(x, w, out, B, M, K, ex, status, stream);
}

template <int EPI, typename OutT>
static int gs_launch_stages(const void * x, const void * w, void * out, int B, int M, int K, const StreamExtra & ex, int * status,
                            cudaStream_t stream) {
    if (g_stream_stages >= 12) return gs_launch<IIAN_GS_STAGES_1, EPI, OutT>(x, w, out, B, M, K, ex, status, stream);
    return gs_launch<IIAN_GS_STAGES_2, EPI, OutT>(x, w, out, B, M, K, ex, status, stream);
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_gemm_stream_stages(int stages) {
    if (stages != 6 && stages != 12) return IIAN_ERR_SHAPE;
    g_stream_stages = stages;
    return IIAN_OK;
}

// x: [B, K] bf16 with 1 <= B <= 8, w: [M, K] bf16, K a multiple of 32, both 16-byte aligned.  out: [B, M] (epilogue 0:
// bf16 or f32; 2: bf16) or [B, M / 2] bf16 (epilogue 1, gate / up rows interleaved in groups of 8, M a multiple of 16).
// in_partial [B, in_tiles] (or null): sums of squares of the rows of the not yet normalised input, in parts; row n of
// the result is multiplied by rsqrt(sum / width + eps) with inv_width = 1 / width.  Epilogue 2: out = bf16(res *
// norm_w) after res [B, M] float32 += bf16(product); out_partial [B, ceil(M / 16)] receives the sums of squares of res
// per block of 16 rows of w.  status: two ints on the device, zero before the launch; non-zero afterwards means a wait
// gave up and the output is not valid.  The results are those of iian_gemm_skinny_fused, bit for bit.
IIAN_API int iian_gemm_stream(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K, int epilogue,
                              const float * in_partial, int in_tiles, float inv_width, float eps,
                              float * res, const float * norm_w, float * out_partial, int * status, cudaStream_t stream) {
    if (B <= 0 || M <= 0) return IIAN_OK;
    if (B > 8) return IIAN_ERR_LIMIT;
    if (K <= 0 || K % 32 != 0) return IIAN_ERR_SHAPE;
    if (((uintptr_t) x & 15) || ((uintptr_t) w & 15)) return IIAN_ERR_ALIGN;
    if (status == nullptr) return IIAN_ERR_SHAPE;
    if (in_partial != nullptr && in_tiles <= 0) return IIAN_ERR_SHAPE;
    const StreamExtra ex = {in_partial, in_tiles, inv_width, eps, res, norm_w, out_partial};
    if (epilogue == 1) {
        if (M % 16 != 0 || out_dtype != IIAN_BF16) return IIAN_ERR_SHAPE;
        return gs_launch_stages<1, __nv_bfloat16>(x, w, out, B, M, K, ex, status, stream);
    }
    if (epilogue == 2) {
        if (out_dtype != IIAN_BF16 || res == nullptr || norm_w == nullptr || out_partial == nullptr) return IIAN_ERR_SHAPE;
        return gs_launch_stages<2, __nv_bfloat16>(x, w, out, B, M, K, ex, status, stream);
    }
    if (epilogue != 0) return IIAN_ERR_SHAPE;
    if (out_dtype == IIAN_BF16) return gs_launch_stages<0, __nv_bfloat16>(x, w, out, B, M, K, ex, status, stream);
    if (out_dtype == IIAN_F32) return gs_launch_stages<0, float>(x, w, out, B, M, K, ex, status, stream);
    return IIAN_ERR_DTYPE;
}
