// out[t, n] = sum_k x[t, k] * w[n, k] for many rows t (prefill portions, large decode batches) on the
// fifth-generation tensor cores: tcgen05.mma with the accumulator in tensor memory, operands brought
// into shared memory by TMA (cp.async.bulk.tensor, no multicast), an mbarrier pipeline between one
// producer thread, one MMA-issuing thread and four epilogue warps.
//
// Both operands are K-major (activations [T, K] and weights [N, K], k contiguous), which is how the
// weights are stored in the file and in the reference (ggml_mul_mat(W, x), src/iian/graph.cpp:121-160).
// The reference hands products of this size to cuBLAS (third_party/ggml/src/ggml-cuda/ggml-cuda.cu:
// 1548-1608); this kernel is the engine's own, so that what follows the product can ride in its
// epilogue: a plain store, or SiLU(gate) * up for a gate|up matrix whose rows are interleaved in groups
// of 8 (gate rows 16j..16j+7, up rows 16j+8..16j+15 hold the same 8 features).
//
// Tile: 128 rows x BN columns (BN = 128 or 256), K in blocks of 64 (one 128-byte swizzle atom), STAGES
// shared-memory stages; one persistent CTA per SM walks the tiles.  Roles: warp 0 lane 0 issues TMA
// loads; warp 1 allocates tensor memory (two accumulators) and its lane 0 issues the MMAs (4 per K
// block, K = 16 each) and commits; warps 2..5 read an accumulator (tcgen05.ld, 32 lanes each), convert
// and store while the next tile is already being multiplied into the other accumulator.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records where it gave up in
// `status`, and every role falls through to the common exit, where tensor memory is freed.  A kernel
// that gave up has written garbage; the host checks `status` after the stream has been synchronised.
#include <cuda.h>

#include "common.cuh"

namespace iian {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;                 // 64 bf16 = 128 bytes = one swizzle atom
constexpr int TC_THREADS = 192;           // warp 0: TMA, warp 1: MMA + TMEM, warps 2..5: epilogue
constexpr unsigned kSpinLimit = 2u * 1000u * 1000u;

enum { EPI_STORE = 0, EPI_SWIGLU8 = 1, EPI_RESNORM = 2 };

struct TcStatus { int code; int where; };

// The fused forms of the epilogue (all null / zero: plain product), as in the weight-streaming kernel.
//  * in_partial [T, in_tiles]: the activations are a residual stream times a norm weight, not yet normalised; row t
//    of the result is multiplied by rsqrt(sum_i in_partial[t, i] / width + eps) (RMSNorm's factor per row commutes
//    with the product, src/iian/graph.cpp:105-114).
//  * res / norm_w / out_partial (EPI_RESNORM): the product is the output of a sub-layer: it is rounded to bfloat16 as
//    the unfused route would store it, added to the float32 residual stream res [T, N] in place, res * norm_w is
//    stored as bfloat16, and the sum of squares of the tile's columns of every row goes to out_partial [T, n_tiles].
struct TcExtra {
    const float * in_partial;
    int in_tiles;
    float inv_width, eps;
    float * res;
    const float * norm_w;
    float * out_partial;
};

__device__ __forceinline__ unsigned smem_addr(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait for the phase with this parity; false: gave up
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned spin = 0; spin < kSpinLimit; spin++) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap * map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: thread i of the warp gets lane i's 32 columns
__device__ __forceinline__ void tc_ld32(unsigned taddr, unsigned * r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile with 128-byte rows, 128-byte swizzle, groups of 8 rows
// 1024 bytes apart.  Start address and offsets are in units of 16 bytes.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long) ((addr & 0x3FFFF) >> 4);           // bits  0-13: start address
    d |= (unsigned long long) 1 << 16;                            // bits 16-29: leading byte offset (unused with swizzle)
    d |= (unsigned long long) (1024 >> 4) << 32;                  // bits 32-45: stride byte offset (8 rows)
    d |= (unsigned long long) 1 << 46;                            // bits 46-47: descriptor version of this architecture
    d |= (unsigned long long) 2 << 61;                            // bits 61-63: 128-byte swizzle
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N tile.
__host__ __device__ constexpr unsigned instr_desc_bf16(int m, int n) {
    return (1u << 4)                      // accumulator format f32
         | (1u << 7) | (1u << 10)         // A and B are bf16
         | ((unsigned) (n >> 3) << 17)    // N / 8
         | ((unsigned) (m >> 4) << 24);   // M / 16
}

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// One accumulator tile (128 x BN, float32, in tensor memory) -> global memory.  `r` holds 32 consecutive
// columns of this thread's row.
template <int EPI, typename OutT>
__device__ __forceinline__ void epilogue_store32(unsigned * r, OutT * __restrict__ out, int row, int col0, int N, int ldo, float rs) {
    if (rs != 1.0f) {
#pragma unroll
        for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * rs);
    }
    if (EPI == EPI_STORE) {
        OutT * dst = out + (size_t) row * ldo + col0;
        if (col0 + 32 <= N && (((uintptr_t) dst) & 15) == 0) {
            if (sizeof(OutT) == 2) {
#pragma unroll
                for (int v = 0; v < 4; v++) {
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                    pk.x = *reinterpret_cast<unsigned *>(&h0); pk.y = *reinterpret_cast<unsigned *>(&h1);
                    pk.z = *reinterpret_cast<unsigned *>(&h2); pk.w = *reinterpret_cast<unsigned *>(&h3);
                    *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(dst) + 8 * v) = pk;
                }
            } else {
#pragma unroll
                for (int v = 0; v < 8; v++)
                    *reinterpret_cast<uint4 *>(reinterpret_cast<float *>(dst) + 4 * v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            }
        } else {
            for (int i = 0; i < 32; i++)
                if (col0 + i < N) dst[i] = from_f32<OutT>(__uint_as_float(r[i]));
        }
    } else {
        // columns come in groups of 16: 8 gate values, then the 8 up values of the same features; the
        // output has N / 2 columns
        OutT * dst = out + (size_t) row * ldo + col0 / 2;
#pragma unroll
        for (int grp = 0; grp < 2; grp++) {
            float a[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float g = __uint_as_float(r[16 * grp + i]), u = __uint_as_float(r[16 * grp + 8 + i]);
                a[i] = g / (1.0f + __expf(-g)) * u;
            }
            if (col0 + 16 * grp + 16 <= N) {
                if (sizeof(OutT) == 2 && (((uintptr_t) (dst + 8 * grp)) & 15) == 0) {
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(a[0], a[1]), h1 = __floats2bfloat162_rn(a[2], a[3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(a[4], a[5]), h3 = __floats2bfloat162_rn(a[6], a[7]);
                    pk.x = *reinterpret_cast<unsigned *>(&h0); pk.y = *reinterpret_cast<unsigned *>(&h1);
                    pk.z = *reinterpret_cast<unsigned *>(&h2); pk.w = *reinterpret_cast<unsigned *>(&h3);
                    *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(dst) + 8 * grp) = pk;
                } else {
                    for (int i = 0; i < 8; i++) dst[8 * grp + i] = from_f32<OutT>(a[i]);
                }
            }
        }
    }
}

// EPI_RESNORM for 32 columns of one row: returns the sum of squares of the new residual values.
__device__ __forceinline__ float epilogue_resnorm32(const unsigned * r, __nv_bfloat16 * __restrict__ out, float * __restrict__ res,
                                                   const float * __restrict__ norm_w, int row, int col0, int N, float rs) {
    float sq = 0.0f;
    float * rp = res + (size_t) row * N + col0;
    __nv_bfloat16 * op = out + (size_t) row * N + col0;
    if (col0 + 32 <= N && (((uintptr_t) rp) & 15) == 0 && (((uintptr_t) op) & 15) == 0) {
#pragma unroll
        for (int v = 0; v < 4; v++) {
            float x[8];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const float4 old = *reinterpret_cast<const float4 *>(rp + 8 * v + 4 * h);
                float4 nw;
                nw.x = old.x + __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[8 * v + 4 * h + 0]) * rs));
                nw.y = old.y + __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[8 * v + 4 * h + 1]) * rs));
                nw.z = old.z + __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[8 * v + 4 * h + 2]) * rs));
                nw.w = old.w + __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[8 * v + 4 * h + 3]) * rs));
                *reinterpret_cast<float4 *>(rp + 8 * v + 4 * h) = nw;
                sq += nw.x * nw.x + nw.y * nw.y + nw.z * nw.z + nw.w * nw.w;
                const float4 w4 = __ldg(reinterpret_cast<const float4 *>(norm_w + col0 + 8 * v + 4 * h));
                x[4 * h + 0] = nw.x * w4.x; x[4 * h + 1] = nw.y * w4.y; x[4 * h + 2] = nw.z * w4.z; x[4 * h + 3] = nw.w * w4.w;
            }
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(x[0], x[1]), h1 = __floats2bfloat162_rn(x[2], x[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(x[4], x[5]), h3 = __floats2bfloat162_rn(x[6], x[7]);
            pk.x = *reinterpret_cast<unsigned *>(&h0); pk.y = *reinterpret_cast<unsigned *>(&h1);
            pk.z = *reinterpret_cast<unsigned *>(&h2); pk.w = *reinterpret_cast<unsigned *>(&h3);
            *reinterpret_cast<uint4 *>(op + 8 * v) = pk;
        }
    } else {
        for (int i = 0; i < 32; i++)
            if (col0 + i < N) {
                const float nw = rp[i] + __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i]) * rs));
                rp[i] = nw;
                sq += nw * nw;
                op[i] = __float2bfloat16_rn(nw * norm_w[col0 + i]);
            }
    }
    return sq;
}

// Persistent: gridDim.x CTAs (one per SM) walk the output tiles round-robin, row tiles fastest, so the
// CTAs that run together share a few weight tiles (read from HBM once, then from L2) and sweep the
// activations, which stay in L2 as a whole.  Tensor memory holds two accumulators: while the epilogue
// warps drain one, the MMA thread already fills the other with the next tile.
template <int BN, int STAGES, int EPI, typename OutT>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
    OutT * __restrict__ out, int T, int N, int K, int ldo, TcStatus * status, const TcExtra ex) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the swizzle pattern is a function of the address: tiles start on 1024-byte boundaries
    unsigned char * smem = (unsigned char *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr unsigned TMEM_COLS = 2 * BN;
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    const int m_tiles = (T + TC_BM - 1) / TC_BM, n_tiles = (N + BN - 1) / BN;
    const int num_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(smem_addr(&full_bar[s]), 1); mbar_init(smem_addr(&empty_bar[s]), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(smem_addr(&acc_full[b]), 1); mbar_init(smem_addr(&acc_empty[b]), 4); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {          // tensor memory: two accumulators of BN columns (128 lanes x 32 bits each)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---- producer: the stage ring runs on across tiles -------------------------------------------
        int it = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
            for (int kb = 0; kb < num_kb; kb++, it++) {
                const int s = it % STAGES;
                const unsigned phase = (it / STAGES) & 1;
                if (!mbar_wait(smem_addr(&empty_bar[s]), phase ^ 1)) { status->code = 1; status->where = it; failed = 1; goto done; }
                const unsigned bar = smem_addr(&full_bar[s]);
                mbar_expect_tx(bar, STAGE_BYTES);
                tma_load_2d(smem_addr(smem + s * STAGE_BYTES), &map_a, kb * TC_BK, m0, bar);
                tma_load_2d(smem_addr(smem + s * STAGE_BYTES + A_BYTES), &map_b, kb * TC_BK, n0, bar);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer -----------------------------------------------------------------------------
        constexpr unsigned idesc = instr_desc_bf16(TC_BM, BN);
        int it = 0, use = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, use++) {
            const int buf = use & 1;
            const unsigned acc_phase = (use >> 1) & 1;
            if (!mbar_wait(smem_addr(&acc_empty[buf]), acc_phase ^ 1)) { status->code = 4; status->where = use; failed = 1; goto done; }
            tc_fence_after();
            const unsigned d_tmem = tmem_base + (unsigned) (buf * BN);
            for (int kb = 0; kb < num_kb; kb++, it++) {
                const int s = it % STAGES;
                const unsigned phase = (it / STAGES) & 1;
                if (!mbar_wait(smem_addr(&full_bar[s]), phase)) { status->code = 2; status->where = it; failed = 1; goto done; }
                tc_fence_after();
                const unsigned long long da = smem_desc_sw128(smem_addr(smem + s * STAGE_BYTES));
                const unsigned long long db = smem_desc_sw128(smem_addr(smem + s * STAGE_BYTES + A_BYTES));
#pragma unroll
                for (int k = 0; k < TC_BK / 16; k++)      // 32 bytes further along K per step, inside the swizzle atom
                    tc_mma(d_tmem, da + (unsigned long long) (k * 2), db + (unsigned long long) (k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                tc_commit(smem_addr(&empty_bar[s]));      // the stage is free once these MMAs have read it
            }
            tc_commit(smem_addr(&acc_full[buf]));         // this accumulator is complete
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads tensor-memory lanes 32 * (w % 4) .. + 31 ----------------------------
        const int q = warp & 3;
        int use = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, use++) {
            const int buf = use & 1;
            const unsigned acc_phase = (use >> 1) & 1;
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * BN;
            if (!mbar_wait(smem_addr(&acc_full[buf]), acc_phase)) {
                if (lane == 0) { status->code = 3; status->where = use; }
                failed = 1;
                break;
            }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            float rs = 1.0f;
            if (ex.in_partial != nullptr && row < T) {          // this row's factor: its partial sums in a fixed order
                float a = 0.0f;
                for (int i = 0; i < ex.in_tiles; i++) a += ex.in_partial[(size_t) row * ex.in_tiles + i];
                rs = rsqrtf(a * ex.inv_width + ex.eps);
            }
            float sq = 0.0f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned r[32];
                tc_ld32(tmem_base + ((unsigned) (q * 32) << 16) + (unsigned) (buf * BN + c0), r);
                tc_wait_ld();
                if (row < T) {
                    if constexpr (EPI == EPI_RESNORM)
                        sq += epilogue_resnorm32(r, reinterpret_cast<__nv_bfloat16 *>(out), ex.res, ex.norm_w, row, n0 + c0, N, rs);
                    else
                        epilogue_store32<EPI, OutT>(r, out, row, n0 + c0, N, ldo, rs);
                }
            }
            if constexpr (EPI == EPI_RESNORM) {
                if (row < T) ex.out_partial[(size_t) row * n_tiles + tile / m_tiles] = sq;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&acc_empty[buf]));     // four arrivals free the accumulator
        }
    }
done:
    // ---- common exit: everybody arrives here, also after a wait that gave up -------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- the same product on pairs of SMs ---------------------------------------------------------------
// A cluster of two CTAs owns a tile of 256 rows x BN columns: CTA r of the pair holds rows 128 r .. 128 r + 127 of
// the activations and columns BN / 2 * r .. of the weights in its shared memory, and its 128 rows of the
// accumulator in its tensor memory.  One thread of CTA 0 issues tcgen05.mma.cta_group::2 (M = 256), which reads
// both CTAs' shared memory and writes both tensor memories; each SM therefore fills 32 KB of shared memory per K
// block instead of 48 KB, which leaves room for six stages and lowers the traffic (and the power) per flop.
// Both CTAs' TMA loads complete on CTA 0's `full` barrier; tcgen05.commit with a CTA mask arrives on the `empty`
// and `accumulator full` barriers of both; the epilogue warps of both arrive on CTA 0's `accumulator empty`.
__device__ __forceinline__ unsigned cluster_cta_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned map_to_cta(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// no multicast: the tile lands in this CTA's shared memory; only the completion goes to the barrier of CTA 0
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap * map, int x, int y, unsigned bar_cluster) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(unsigned bar) {      // arrives on the barrier at this offset in both CTAs
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short) 3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc,
                                            unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

template <int BN, int STAGES, int KPS, int EPI, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1) gemm_tcgen05_pair_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
    OutT * __restrict__ out, int T, int N, int K, int ldo, TcStatus * status, const TcExtra ex) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char * smem = (unsigned char *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    constexpr int HALF = BN / 2;
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = HALF * TC_BK * 2, KB_BYTES = A_BYTES + B_BYTES, STAGE_BYTES = KPS * KB_BYTES;
    constexpr unsigned TMEM_COLS = 2 * BN;
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_s;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_cta_rank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    // a stage holds KPS blocks of 64 along K and is handed over with one barrier phase and one commit: the tensor
    // pipe idles for a fixed time at every hand-over, so longer stages keep it busier.  Blocks past the end of K
    // are filled with zeros by TMA.
    const int num_kb = ((K + TC_BK - 1) / TC_BK + KPS - 1) / KPS;
    const int m_tiles = (T + 2 * TC_BM - 1) / (2 * TC_BM), n_tiles = (N + BN - 1) / BN;
    const int num_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(smem_addr(&full_bar[s]), 1); mbar_init(smem_addr(&empty_bar[s]), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(smem_addr(&acc_full[b]), 1); mbar_init(smem_addr(&acc_empty[b]), 8); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {          // the same warp of both CTAs allocates: the two tensor memories get the same columns
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();       // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const unsigned tmem_base = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---- producer (both CTAs): its half of the pair's operands, completion on CTA 0's barrier ----------
        int it = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs) {
            const int m0 = (tile % m_tiles) * (2 * TC_BM) + (int) rank * TC_BM, n0 = (tile / m_tiles) * BN + (int) rank * HALF;
            for (int kb = 0; kb < num_kb; kb++, it++) {
                const int s = it % STAGES;
                const unsigned phase = (it / STAGES) & 1;
                if (!mbar_wait(smem_addr(&empty_bar[s]), phase ^ 1)) { status->code = 1; status->where = it; failed = 1; goto done; }
                const unsigned bar = map_to_cta(smem_addr(&full_bar[s]), 0);
                if (rank == 0) mbar_expect_tx(smem_addr(&full_bar[s]), 2 * STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < KPS; j++) {
                    tma_load_2d_pair(smem_addr(smem + s * STAGE_BYTES + j * KB_BYTES), &map_a, (kb * KPS + j) * TC_BK, m0, bar);
                    tma_load_2d_pair(smem_addr(smem + s * STAGE_BYTES + j * KB_BYTES + A_BYTES), &map_b, (kb * KPS + j) * TC_BK, n0, bar);
                }
            }
        }
        // the last commits still arrive on this CTA's barriers: take them before the CTA may leave
        for (int i = 0; i < STAGES; i++, it++)
            if (!mbar_wait(smem_addr(&empty_bar[it % STAGES]), ((it / STAGES) & 1) ^ 1)) { status->code = 5; status->where = it; failed = 1; break; }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---- MMA issuer (CTA 0 only) -------------------------------------------------------------------
        constexpr unsigned idesc = instr_desc_bf16(2 * TC_BM, BN);
        int it = 0, use = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, use++) {
            const int buf = use & 1;
            const unsigned acc_phase = (use >> 1) & 1;
            if (!mbar_wait(smem_addr(&acc_empty[buf]), acc_phase ^ 1)) { status->code = 4; status->where = use; failed = 1; goto done; }
            tc_fence_after();
            const unsigned d_tmem = tmem_base + (unsigned) (buf * BN);
            for (int kb = 0; kb < num_kb; kb++, it++) {
                const int s = it % STAGES;
                const unsigned phase = (it / STAGES) & 1;
                if (!mbar_wait(smem_addr(&full_bar[s]), phase)) { status->code = 2; status->where = it; failed = 1; goto done; }
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < KPS; j++) {
                    const unsigned long long da = smem_desc_sw128(smem_addr(smem + s * STAGE_BYTES + j * KB_BYTES));
                    const unsigned long long db = smem_desc_sw128(smem_addr(smem + s * STAGE_BYTES + j * KB_BYTES + A_BYTES));
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; k++)
                        tc_mma_pair(d_tmem, da + (unsigned long long) (k * 2), db + (unsigned long long) (k * 2), idesc, (kb > 0 || j > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit_pair(smem_addr(&empty_bar[s]));
            }
            tc_commit_pair(smem_addr(&acc_full[buf]));
        }
    } else if (warp >= 2) {
        // ---- epilogue (both CTAs): this CTA's 128 rows of the pair's tile ----------------------------------
        const int q = warp & 3;
        int use = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, use++) {
            const int buf = use & 1;
            const unsigned acc_phase = (use >> 1) & 1;
            const int m0 = (tile % m_tiles) * (2 * TC_BM) + (int) rank * TC_BM, n0 = (tile / m_tiles) * BN;
            if (!mbar_wait(smem_addr(&acc_full[buf]), acc_phase)) {
                if (lane == 0) { status->code = 3; status->where = use; }
                failed = 1;
                break;
            }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            float rs = 1.0f;
            if (ex.in_partial != nullptr && row < T) {
                float a = 0.0f;
                for (int i = 0; i < ex.in_tiles; i++) a += ex.in_partial[(size_t) row * ex.in_tiles + i];
                rs = rsqrtf(a * ex.inv_width + ex.eps);
            }
            float sq = 0.0f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned r[32];
                tc_ld32(tmem_base + ((unsigned) (q * 32) << 16) + (unsigned) (buf * BN + c0), r);
                tc_wait_ld();
                if (row < T) {
                    if constexpr (EPI == EPI_RESNORM)
                        sq += epilogue_resnorm32(r, reinterpret_cast<__nv_bfloat16 *>(out), ex.res, ex.norm_w, row, n0 + c0, N, rs);
                    else
                        epilogue_store32<EPI, OutT>(r, out, row, n0 + c0, N, ldo, rs);
                }
            }
            if constexpr (EPI == EPI_RESNORM) {
                if (row < T) ex.out_partial[(size_t) row * n_tiles + tile / m_tiles] = sq;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_addr(&acc_empty[buf]), 0));     // eight arrivals free the accumulator
        }
    }
done:
    // ---- common exit: both CTAs arrive here, also after a wait that gave up; neither frees tensor memory or
    // leaves while the other may still read its shared memory or write its tensor memory
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn) p;
    }
    return fn;
}

// a [rows, K] bf16 row-major matrix, boxes of [box_rows, 64], 128-byte swizzle, zero fill outside
static int make_map(CUtensorMap * map, const void * base, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return IIAN_ERR_LIMIT;
    cuuint64_t dims[2] = {(cuuint64_t) K, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) K * 2};
    cuuint32_t box[2] = {(cuuint32_t) TC_BK, (cuuint32_t) box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? IIAN_OK : 2000 + (int) r;
}

template <int BN, int STAGES, int EPI, typename OutT>
static int launch_tc(const CUtensorMap & ma, const CUtensorMap & mb, void * out, int T, int N, int K, int ldo, TcStatus * status,
                     const TcExtra & ex, cudaStream_t stream) {
    constexpr size_t smem = (size_t) STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return 1000 + (int) e;
        configured = true;
    }
    const int tiles = ((T + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    dim3 grid(tiles < sms ? tiles : sms);
    gemm_tcgen05_kernel<BN, STAGES, EPI, OutT><<<grid, TC_THREADS, smem, stream>>>(ma, mb, (OutT *) out, T, N, K, ldo, status, ex);
    return iian_launch_status();
}

template <int BN, int STAGES, int KPS, int EPI, typename OutT>
static int launch_tc_pair(const CUtensorMap & ma, const CUtensorMap & mb, void * out, int T, int N, int K, int ldo, TcStatus * status,
                          const TcExtra & ex, cudaStream_t stream) {
    constexpr size_t smem = (size_t) STAGES * KPS * (TC_BM * TC_BK * 2 + (BN / 2) * TC_BK * 2) + 1024;
    auto kernel = gemm_tcgen05_pair_kernel<BN, STAGES, KPS, EPI, OutT>;
    static int pairs = 0;
    if (pairs == 0) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return 1000 + (int) e;
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned) (sms & ~1));
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sms / 2; }
        pairs = n < sms / 2 ? n : sms / 2;
    }
    const int tiles = ((T + 2 * TC_BM - 1) / (2 * TC_BM)) * ((N + BN - 1) / BN);
    dim3 grid((unsigned) (2 * (tiles < pairs ? tiles : pairs)));
    kernel<<<grid, TC_THREADS, smem, stream>>>(ma, mb, (OutT *) out, T, N, K, ldo, status, ex);
    return iian_launch_status();
}

}  // namespace iian

using namespace iian;

// bn: 128 or 256 columns per tile on one SM; 512: tiles of 256 x 256 on pairs of SMs
static int tc_entry(const void * x, const void * w, void * out, int out_dtype, int T, int N, int K, int epilogue,
                    int bn, int * status, const TcExtra & ex, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return IIAN_OK;
    if (K <= 0 || K % 8 != 0) return IIAN_ERR_SHAPE;
    if (((uintptr_t) x & 15) || ((uintptr_t) w & 15)) return IIAN_ERR_ALIGN;
    if (epilogue == EPI_SWIGLU8 && N % 16 != 0) return IIAN_ERR_SHAPE;
    if (status == nullptr) return IIAN_ERR_SHAPE;
    if (bn != 128 && bn != 256 && bn != 512) return IIAN_ERR_SHAPE;
    if (ex.in_partial != nullptr && ex.in_tiles <= 0) return IIAN_ERR_SHAPE;
    const bool pair = bn == 512;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, x, T, K, TC_BM);
    if (rc != IIAN_OK) return rc;
    rc = make_map(&mb, w, N, K, pair ? 128 : bn);
    if (rc != IIAN_OK) return rc;
    TcStatus * st = (TcStatus *) status;
    const int ldo = epilogue == EPI_SWIGLU8 ? N / 2 : N;
    if (pair) {
        if (epilogue == EPI_RESNORM) {
            if (out_dtype != IIAN_BF16 || ex.res == nullptr || ex.norm_w == nullptr || ex.out_partial == nullptr) return IIAN_ERR_SHAPE;
            return launch_tc_pair<256, 3, 2, EPI_RESNORM, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream);
        }
        if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU8) return IIAN_ERR_SHAPE;
        if (out_dtype == IIAN_BF16)
            return epilogue == EPI_STORE ? launch_tc_pair<256, 3, 2, EPI_STORE, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream)
                                         : launch_tc_pair<256, 3, 2, EPI_SWIGLU8, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream);
        if (out_dtype == IIAN_F32 && epilogue == EPI_STORE)
            return launch_tc_pair<256, 3, 2, EPI_STORE, float>(ma, mb, out, T, N, K, ldo, st, ex, stream);
        return IIAN_ERR_DTYPE;
    }
    if (epilogue == EPI_RESNORM) {
        if (out_dtype != IIAN_BF16 || ex.res == nullptr || ex.norm_w == nullptr || ex.out_partial == nullptr) return IIAN_ERR_SHAPE;
        if (bn == 256) return launch_tc<256, 4, EPI_RESNORM, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream);
        return launch_tc<128, 6, EPI_RESNORM, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream);
    }
    if (epilogue != EPI_STORE && epilogue != EPI_SWIGLU8) return IIAN_ERR_SHAPE;
    if (out_dtype == IIAN_BF16) {
        if (bn == 256) return epilogue == EPI_STORE ? launch_tc<256, 4, EPI_STORE, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream)
                                                    : launch_tc<256, 4, EPI_SWIGLU8, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream);
        return epilogue == EPI_STORE ? launch_tc<128, 6, EPI_STORE, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream)
                                     : launch_tc<128, 6, EPI_SWIGLU8, __nv_bfloat16>(ma, mb, out, T, N, K, ldo, st, ex, stream);
    }
    if (out_dtype == IIAN_F32) {
        if (epilogue != EPI_STORE) return IIAN_ERR_DTYPE;
        if (bn == 256) return launch_tc<256, 4, EPI_STORE, float>(ma, mb, out, T, N, K, ldo, st, ex, stream);
        return launch_tc<128, 6, EPI_STORE, float>(ma, mb, out, T, N, K, ldo, st, ex, stream);
    }
    return IIAN_ERR_DTYPE;
}

// x: [T, K] bf16, w: [N, K] bf16; out: [T, N] (epilogue 0) or [T, N / 2] (epilogue 1: SiLU(gate) * up over
// rows interleaved in groups of 8), bf16 or f32.  K must be a multiple of 8 (16-byte rows for TMA), x and w
// 16-byte aligned.  status: two ints on the device, zero before the launch; non-zero afterwards means a
// wait gave up (code 1 producer, 2 and 4 MMA, 3 epilogue, 5 producer's tail) and the output is not valid.  bn: columns
// of a tile, 128 or 256; 512 runs tiles of 256 x 256 on pairs of SMs (tcgen05 cta_group::2).
IIAN_API int iian_gemm_tcgen05(const void * x, const void * w, void * out, int out_dtype, int T, int N, int K, int epilogue,
                               int bn, int * status, cudaStream_t stream) {
    if (epilogue == EPI_RESNORM) return IIAN_ERR_SHAPE;
    const TcExtra none = {nullptr, 0, 0.0f, 0.0f, nullptr, nullptr, nullptr};
    return tc_entry(x, w, out, out_dtype, T, N, K, epilogue, bn, status, none, stream);
}

// The product with its fused forms.  in_partial [T, in_tiles] (or null): the rows' sums of squares in parts; the
// result's row t is multiplied by rsqrt(sum / width + eps) with inv_width = 1 / width.  epilogue 2: out = bf16(res *
// norm_w) after res [T, N] float32 += bf16(product), and out_partial [T, ceil(N / bn)] receives the sums of squares
// of res per tile of bn columns.
IIAN_API int iian_gemm_tcgen05_fused(const void * x, const void * w, void * out, int out_dtype, int T, int N, int K, int epilogue,
                                     int bn, int * status, const float * in_partial, int in_tiles, float inv_width, float eps,
                                     float * res, const float * norm_w, float * out_partial, cudaStream_t stream) {
    const TcExtra ex = {in_partial, in_tiles, inv_width, eps, res, norm_w, out_partial};
    return tc_entry(x, w, out, out_dtype, T, N, K, epilogue, bn, status, ex, stream);
}
