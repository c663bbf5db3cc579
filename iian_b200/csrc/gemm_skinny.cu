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

// NT: 8-column tiles of the batch; MT: 16-row tiles of weights per block (they share the activation
// fragments); WARPS: how many warps split K; UNROLL: 32-wide k chunks whose weight loads are issued
// before the first of them is used.
// EPI 0: store the products.  EPI 1: the weight rows hold gate and up projections interleaved in groups of
// 8 (rows 16j..16j+7 gate, 16j+8..16j+15 up, same 8 features); the kernel stores silu(gate) * up, half as
// many columns (src/iian/graph.cpp:135).
template <int NT, int MT, int WARPS, int UNROLL, int EPI, typename OutT>
__global__ void __launch_bounds__(WARPS * 32) gemm_skinny_kernel(
    const __nv_bfloat16 * __restrict__ x, const __nv_bfloat16 * __restrict__ w, OutT * __restrict__ out,
    int B, int M, int K, float * __restrict__ part, int * __restrict__ counters) {
    extern __shared__ float red_raw[];
    __shared__ int s_last;
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
    const bool first_round = c + (UNROLL - 1) * WARPS < c_end;
    if (first_round) load_round(c);
    pdl_wait();
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
            out[(size_t) n * (M / 2) + (m0 / 2 + f)] = from_f32<OutT>(g / (1.0f + expf(-g)) * u);
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
                      int * counters, cudaStream_t stream) {
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
                       (const __nv_bfloat16 *) x, (const __nv_bfloat16 *) w, (OutT *) out, B, M, K, part, counters);
}

// cfg = MT * 100 + WARPS * 10 + UNROLL; 0 = the default for this (B, M)
template <int NT, int EPI, typename OutT>
static int launch_nt(const void * x, const void * w, void * out, int B, int M, int K, int cfg, int ksplit, float * part,
                     int * counters, cudaStream_t stream) {
    if (cfg == 0) {
        if (NT == 1) cfg = M >= 65536 ? 144 : (K >= 8192 ? 188 : 184);
        else if (NT == 2) cfg = 284;
        else cfg = 282;
    }
    if (NT == 1) {
        switch (cfg) {
            case 184: return launch_cfg<1, 1, 8, 4, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, stream);
            case 188: return launch_cfg<1, 1, 8, 8, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, stream);
            case 144: return launch_cfg<1, 1, 4, 4, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, stream);
            case 148: return launch_cfg<1, 1, 4, 8, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, stream);
        }
        return IIAN_ERR_SHAPE;
    }
    switch (cfg) {
        case 284: return launch_cfg<NT, 2, 8, 4, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, stream);
        case 282: return launch_cfg<NT, 2, 8, 2, EPI, OutT>(x, w, out, B, M, K, ksplit, part, counters, stream);
    }
    return IIAN_ERR_SHAPE;
}

template <int EPI, typename OutT>
static int launch_skinny(const void * x, const void * w, void * out, int B, int M, int K, int cfg, int ksplit, float * part,
                         int * counters, cudaStream_t stream) {
    if (B <= 8) return launch_nt<1, EPI, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, stream);
    if (EPI != 0) return IIAN_ERR_LIMIT;          // the fused epilogue is built for up to 8 rows
    if (B <= 16) return launch_nt<2, 0, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, stream);
    if (B <= 32) return launch_nt<4, 0, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, stream);
    return launch_nt<8, 0, OutT>(x, w, out, B, M, K, cfg, ksplit, part, counters, stream);
}


// ---- the same product with the work cut evenly over the SMs ------------------------------------------
// A grid of row tiles leaves SMs idle whenever the number of tiles is not a multiple of what the GPU
// holds at once (256 tiles of the output projection on 148 SMs: the slowest SM carries two, the mean is
// 1.7).  Here the grid is exactly what the GPU holds, and the work, counted in steps (one step = every
// warp of the CTA takes one 32-wide chunk of k of one 16-row tile), is cut into equal contiguous ranges:
// a CTA takes the rest of one tile, some whole tiles, and the start of another.  A tile that is shared
// leaves its parts in scratch memory; whichever CTA completes the tile's step count adds the parts in the
// order of their position (not of their arrival) and writes the result, so there is no waiting between
// CTAs and the sum does not depend on timing.  The cut depends on (M, K) and the device only, never on the
// batch.
template <int NT, int WARPS, int UNROLL, int EPI, typename OutT>
__global__ void __launch_bounds__(WARPS * 32, UNROLL >= 8 ? 2 : 3) gemm_stream_kernel(
    const __nv_bfloat16 * __restrict__ x, const __nv_bfloat16 * __restrict__ w, OutT * __restrict__ out,
    int B, int M, int K, float * __restrict__ part, int * __restrict__ counters, int max_parts) {
    __shared__ float red[WARPS][16][NT * 8 + 1];
    __shared__ int s_last;
    constexpr int CELLS = 16 * NT * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int spt = K / (32 * WARPS);                 // steps per tile
    const int tiles = (M + 15) / 16;
    const long long total = (long long) tiles * spt;
    const long long P = min((long long) gridDim.x, total);      // every CTA that works has at least one step
    if (blockIdx.x >= P) return;
    long long u = total * blockIdx.x / P;
    const long long u_end = total * (blockIdx.x + 1) / P;

    const uint4 * xr[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int n = min(nt * 8 + g, B - 1);
        xr[nt] = reinterpret_cast<const uint4 *>(x + (size_t) n * K) + t;
    }
    bool waited = false;
    while (u < u_end) {
        const int tile = (int) (u / spt), s_begin = (int) (u % spt);
        const int s_end = (int) min((long long) spt, s_begin + (u_end - u));
        const int m0 = tile * 16;
        const uint4 * w0 = reinterpret_cast<const uint4 *>(w + (size_t) min(m0 + g, M - 1) * K) + t;
        const uint4 * w1 = reinterpret_cast<const uint4 *>(w + (size_t) min(m0 + g + 8, M - 1) * K) + t;
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
        {
            const size_t off = ((size_t) s_begin * WARPS + warp) * 4;   // in 16-byte units; a step is WARPS * 4 of them
            const uint4 * p0 = w0 + off;
            const uint4 * p1 = w1 + off;
            const uint4 * px[NT];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) px[nt] = xr[nt] + off;
            for (int s = s_begin; s < s_end; s += UNROLL) {
                uint4 a0[UNROLL], a1[UNROLL];
#pragma unroll
                for (int q = 0; q < UNROLL; q++)
                    if (s + q < s_end) {
                        a0[q] = ld_stream(p0 + q * WARPS * 4);
                        a1[q] = ld_stream(p1 + q * WARPS * 4);
                    }
                // The weights do not depend on the kernel before this one: the first loads are in flight
                // before this kernel waits for its activations.
                if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
                for (int q = 0; q < UNROLL; q++)
                    if (s + q < s_end) {
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            const uint4 b = __ldg(px[nt] + q * WARPS * 4);
                            mma_bf16_16816(acc[nt], a0[q].x, a1[q].x, a0[q].y, a1[q].y, b.x, b.y);
                            mma_bf16_16816(acc[nt], a0[q].z, a1[q].z, a0[q].w, a1[q].w, b.z, b.w);
                        }
                    }
                p0 += UNROLL * WARPS * 4;
                p1 += UNROLL * WARPS * 4;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) px[nt] += UNROLL * WARPS * 4;
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
        // cell idx = n * 16 + r; the warps' sums are added in a fixed order
        float mine[(CELLS + WARPS * 32 - 1) / (WARPS * 32)];
#pragma unroll
        for (int j = 0; j < (CELLS + WARPS * 32 - 1) / (WARPS * 32); j++) {
            const int idx = threadIdx.x + j * WARPS * 32;
            float v = 0.0f;
            if (idx < CELLS) {
#pragma unroll
                for (int wv = 0; wv < WARPS; wv++) v += red[wv][idx % 16][idx / 16];
            }
            mine[j] = v;
        }
        __syncthreads();
        bool finish = true;
        if (s_begin != 0 || s_end != spt) {
            // position of this CTA among those that share the tile: CTA i starts at floor(total * i / P), so
            // the CTA that holds step v is floor(((v + 1) * P - 1) / total)
            const long long first = (((long long) tile * spt + 1) * P - 1) / total;
            const long long last = (((long long) (tile + 1) * spt) * P - 1) / total;
            const int slot = (int) (blockIdx.x - first), n_parts = (int) (last - first + 1);
            float * dst = part + ((size_t) tile * max_parts + slot) * CELLS;
#pragma unroll
            for (int j = 0; j < (CELLS + WARPS * 32 - 1) / (WARPS * 32); j++) {
                const int idx = threadIdx.x + j * WARPS * 32;
                if (idx < CELLS) dst[idx] = mine[j];
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) s_last = (atomicAdd(counters + tile, s_end - s_begin) + (s_end - s_begin) == spt);
            __syncthreads();
            finish = s_last != 0;
            if (finish) {
                __threadfence();
                const float * all = part + (size_t) tile * max_parts * CELLS;
#pragma unroll
                for (int j = 0; j < (CELLS + WARPS * 32 - 1) / (WARPS * 32); j++) {
                    const int idx = threadIdx.x + j * WARPS * 32;
                    float v = 0.0f;
                    if (idx < CELLS)
                        for (int i = 0; i < n_parts; i++) v += __ldcg(all + (size_t) i * CELLS + idx);
                    mine[j] = v;
                }
                if (threadIdx.x == 0) counters[tile] = 0;
            }
        }
        if (finish) {
            if (EPI == 1) {
                // rows 0..7 of the tile are gate, 8..15 up, of the same 8 features (src/iian/graph.cpp:135)
#pragma unroll
                for (int j = 0; j < (CELLS + WARPS * 32 - 1) / (WARPS * 32); j++) {
                    const int idx = threadIdx.x + j * WARPS * 32;
                    if (idx < CELLS) red[0][idx % 16][idx / 16] = mine[j];
                }
                __syncthreads();
                for (int idx = threadIdx.x; idx < CELLS / 2; idx += WARPS * 32) {
                    const int n = idx / 8, f = idx % 8;
                    if (n < B && m0 + 15 < M) {
                        const float gv = red[0][f][n], uv = red[0][f + 8][n];
                        out[(size_t) n * (M / 2) + (m0 / 2 + f)] = from_f32<OutT>(gv / (1.0f + expf(-gv)) * uv);
                    }
                }
                __syncthreads();
            } else {
#pragma unroll
                for (int j = 0; j < (CELLS + WARPS * 32 - 1) / (WARPS * 32); j++) {
                    const int idx = threadIdx.x + j * WARPS * 32;
                    const int n = idx / 16, m = m0 + idx % 16;
                    if (idx < CELLS && n < B && m < M) out[(size_t) n * M + m] = from_f32<OutT>(mine[j]);
                }
            }
        }
        u += s_end - s_begin;
    }
    pdl_launch_dependents();
}

// CTAs the device holds at once for this instantiation (SMs x CTAs per SM), per device
template <int NT, int WARPS, int UNROLL, int EPI, typename OutT>
static int stream_grid(int * grid) {
    static int cached[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return 1000 + (int) e;
    if (dev < 0 || dev >= 64) return IIAN_ERR_LIMIT;
    if (cached[dev] == 0) {
        int sms = 0, per_sm = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return 1000 + (int) e;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_stream_kernel<NT, WARPS, UNROLL, EPI, OutT>, WARPS * 32, 0);
        if (e != cudaSuccess) return 1000 + (int) e;
        if (per_sm < 1) return IIAN_ERR_LIMIT;
        cached[dev] = sms * per_sm;
    }
    *grid = cached[dev];
    return IIAN_OK;
}

static int stream_max_parts(int M, int K, int warps, int grid) {
    // a tile's parts are consecutive CTAs; all but the first and the last lie wholly inside the tile
    const long long spt = K / (32 * warps), tiles = (M + 15) / 16, total = tiles * spt;
    const long long P = grid < total ? grid : total;
    const long long mp = (spt + 1) * P / total + 2;
    return (int) (mp < spt ? mp : spt);
}

template <int NT, int WARPS, int UNROLL, int EPI, typename OutT>
static int launch_stream(const void * x, const void * w, void * out, int B, int M, int K, float * part, size_t part_floats,
                         int * counters, size_t counter_ints, size_t * need_floats, size_t * need_ints, cudaStream_t stream) {
    int grid = 0;
    const int rc = stream_grid<NT, WARPS, UNROLL, EPI, OutT>(&grid);
    if (rc != IIAN_OK) return rc;
    const int max_parts = stream_max_parts(M, K, WARPS, grid);
    const size_t tiles = (size_t) (M + 15) / 16;
    const size_t nf = tiles * max_parts * 16 * NT * 8;
    if (need_floats != nullptr) { *need_floats = nf; *need_ints = tiles; return IIAN_OK; }
    if (part == nullptr || counters == nullptr || part_floats < nf || counter_ints < tiles) return IIAN_ERR_LIMIT;
    return iian_launch(gemm_stream_kernel<NT, WARPS, UNROLL, EPI, OutT>, dim3(grid), dim3(WARPS * 32), 0, stream,
                       (const __nv_bfloat16 *) x, (const __nv_bfloat16 *) w, (OutT *) out, B, M, K, part, counters, max_parts);
}

template <int EPI, typename OutT>
static int launch_stream_k(const void * x, const void * w, void * out, int B, int M, int K, float * part, size_t pf, int * counters,
                           size_t ci, size_t * nf, size_t * ni, cudaStream_t stream) {
    if (K >= 8192) return launch_stream<1, 8, 8, EPI, OutT>(x, w, out, B, M, K, part, pf, counters, ci, nf, ni, stream);
    return launch_stream<1, 8, 4, EPI, OutT>(x, w, out, B, M, K, part, pf, counters, ci, nf, ni, stream);
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
IIAN_API int iian_gemm_skinny_cfg(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K,
                                  int cfg, int ksplit, float * part, int * counters, int epilogue, cudaStream_t stream) {
    if (B <= 0 || M <= 0) return IIAN_OK;
    if (B > 64) return IIAN_ERR_LIMIT;
    if (K <= 0 || K % 32 != 0) return IIAN_ERR_SHAPE;
    if (((uintptr_t) x & 15) || ((uintptr_t) w & 15)) return IIAN_ERR_ALIGN;
    if (ksplit < 1 || ksplit > 64 || ksplit > K / 32) return IIAN_ERR_SHAPE;
    if (ksplit > 1 && (part == nullptr || counters == nullptr)) return IIAN_ERR_SHAPE;
    if (epilogue == 1) {
        if (M % 16 != 0 || ksplit != 1 || out_dtype != IIAN_BF16) return IIAN_ERR_SHAPE;
        return launch_skinny<1, __nv_bfloat16>(x, w, out, B, M, K, cfg, 1, nullptr, nullptr, stream);
    }
    if (epilogue != 0) return IIAN_ERR_SHAPE;
    if (out_dtype == IIAN_BF16) return launch_skinny<0, __nv_bfloat16>(x, w, out, B, M, K, cfg, ksplit, part, counters, stream);
    if (out_dtype == IIAN_F32) return launch_skinny<0, float>(x, w, out, B, M, K, cfg, ksplit, part, counters, stream);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_gemm_skinny(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K,
                              cudaStream_t stream) {
    return iian_gemm_skinny_cfg(x, w, out, out_dtype, B, M, K, 0, 1, nullptr, nullptr, 0, stream);
}

// The evenly cut form (up to 8 rows, K a multiple of 256).  part and counters are scratch of at least the
// sizes that iian_gemm_stream_scratch reports; counters are zero before the first launch and left zero.
IIAN_API int iian_gemm_stream(const void * x, const void * w, void * out, int out_dtype, int B, int M, int K, float * part,
                              size_t part_floats, int * counters, size_t counter_ints, int epilogue, cudaStream_t stream) {
    if (B <= 0 || M <= 0) return IIAN_OK;
    if (B > 8) return IIAN_ERR_LIMIT;
    if (K <= 0 || K % 256 != 0) return IIAN_ERR_SHAPE;
    if (((uintptr_t) x & 15) || ((uintptr_t) w & 15)) return IIAN_ERR_ALIGN;
    if (epilogue == 1) {
        if (M % 16 != 0 || out_dtype != IIAN_BF16) return IIAN_ERR_SHAPE;
        return launch_stream_k<1, __nv_bfloat16>(x, w, out, B, M, K, part, part_floats, counters, counter_ints, nullptr, nullptr, stream);
    }
    if (epilogue != 0) return IIAN_ERR_SHAPE;
    if (out_dtype == IIAN_BF16)
        return launch_stream_k<0, __nv_bfloat16>(x, w, out, B, M, K, part, part_floats, counters, counter_ints, nullptr, nullptr, stream);
    if (out_dtype == IIAN_F32)
        return launch_stream_k<0, float>(x, w, out, B, M, K, part, part_floats, counters, counter_ints, nullptr, nullptr, stream);
    return IIAN_ERR_DTYPE;
}

IIAN_API int iian_gemm_stream_scratch(int out_dtype, int M, int K, int epilogue, size_t * part_floats, size_t * counter_ints) {
    if (M <= 0 || K <= 0 || K % 256 != 0 || part_floats == nullptr || counter_ints == nullptr) return IIAN_ERR_SHAPE;
    if (epilogue == 1) return launch_stream_k<1, __nv_bfloat16>(nullptr, nullptr, nullptr, 1, M, K, nullptr, 0, nullptr, 0, part_floats, counter_ints, nullptr);
    if (out_dtype == IIAN_F32) return launch_stream_k<0, float>(nullptr, nullptr, nullptr, 1, M, K, nullptr, 0, nullptr, 0, part_floats, counter_ints, nullptr);
    return launch_stream_k<0, __nv_bfloat16>(nullptr, nullptr, nullptr, 1, M, K, nullptr, 0, nullptr, 0, part_floats, counter_ints, nullptr);
}
