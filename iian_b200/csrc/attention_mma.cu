// Paged flash attention on tensor cores (bf16 in, float32 softmax and accumulation) for prefill
// portions and for decode, over block tables.
//
// One CTA works on a tile of rows of one (sequence, KV head): the rows are the (token, head) pairs of
// the query heads that share this KV head ("GQA packing": row r = token r / G, head kvh * G + r % G),
// so a K/V tile fetched once serves all G heads -- in decode, where a sequence has one token, the G
// heads are the rows.  Keys are walked in tiles of 64; K and V tiles are gathered page by page through
// the block table with 16-byte cp.async into swizzled shared memory (two stages), read back with
// ldmatrix, multiplied with mma.sync m16n8k16.  With n_split > 1 the key range is cut into n_split
// parts handled by different CTAs that write (normalised partial output, log-sum-exp) to scratch
// memory, and a second kernel merges them: this is how a single long sequence fills the GPU in decode.
//
// Formula (reference, src/iian/paged_attn.cpp:112-145): scores q.k * scale; key j visible to the token
// at position p iff j <= p and (window == 0 or p - j < window); softmax in float32; o = sum p_j v_j; a
// row that sees no key yields zeros.  The reference's GPU path reaches the same result by gathering
// each sequence's cells into a contiguous buffer and calling a dense flash-attention kernel
// (src/iian/graph.cpp:474-518); here the gather happens inside the kernel.
#include <cuda.h>

#include "common.cuh"
#include <cooperative_groups.h>
#include <mutex>

namespace iian {

namespace cg = cooperative_groups;

constexpr int BN = 64;   // keys per tile

struct AttnParams {
    const __nv_bfloat16 * q;        // [N, nh, HD]
    const __nv_bfloat16 * k_cache;  // [pages, nkv, page_size, HD]
    const __nv_bfloat16 * v_cache;
    __nv_bfloat16 * out;            // [N, nh * HD]
    float * part_o;                 // [N * nh, n_split, HD]   (n_split > 1)
    float * part_lse;               // [N * nh, n_split]
    int * counters;                 // [S * nkv * row tiles], zero between launches (decode form, n_split > 1)
    const int * cu_q;               // [S + 1]
    const int * ctx_len;            // [S]
    const int * block_table;        // [S, max_blocks]
    int max_blocks, nh, nkv, page_size, num_pages, window, n_split;
    float scale_log2;               // scale * log2(e)
    // fused form of the decode kernel: Q, K and V of the step's tokens come straight from the projection
    __nv_bfloat16 * k_cache_w;      // the caches again, writable
    __nv_bfloat16 * v_cache_w;
    const __nv_bfloat16 * qkv;      // [N, (nh + 2 nkv) * HD]
    const float * q_weight;         // [HD] or null: per-head RMSNorm weights
    const float * k_weight;
    const float2 * table;           // [N, HD / 2] (cos, sin) of the tokens' angles, or null: no rotation
    const int * slots;              // [N] cache cell of each token (page * page_size + offset), < 0: not stored
    float eps;
    int write_kv;
    int * status;                   // TMA form of the decode kernel: {code, where}, zero before the launch
};

// Tensor maps of the K and V caches for the TMA form of the decode kernel (unused by the other forms).
struct KvMaps {
    CUtensorMap k, v;
};

__device__ __forceinline__ unsigned smem_u32(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(unsigned dst, const void * src, bool valid) {
    const int n = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned & r0, unsigned & r1, unsigned & r2, unsigned & r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned & r0, unsigned & r1, unsigned & r2, unsigned & r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float * c, const unsigned * a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x in one MUFU instruction (about 2 ulp; -inf gives 0).  The probabilities are rounded to bfloat16 next.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}

// byte offset of 16-byte chunk `chunk` of row `row` in a tile with rows of HD bf16, XOR-swizzled so that
// the 8 rows an ldmatrix touches fall into different banks
template <int HD> __device__ __forceinline__ unsigned swz(int row, int chunk) {
    return (unsigned) (row * HD * 2 + ((chunk ^ (row & 7)) << 4));
}

// The same for a tile that TMA wrote with its 128-byte swizzle (head size 128): two planes of 128-byte rows,
// one per half of the head, chunks XOR-swizzled within a row by the row's low three bits.
template <int HD, bool TMA> __device__ __forceinline__ unsigned kv_off(int row, int chunk) {
    if (TMA) return (unsigned) ((chunk >> 3) * (BN * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
    return swz<HD>(row, chunk);
}

constexpr unsigned kDecodeSpinLimit = 4u * 1000u * 1000u;
__device__ __forceinline__ void dk_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void dk_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool dk_wait(unsigned bar, unsigned parity) {          // bounded: false when it gave up
    for (unsigned spin = 0; spin < kDecodeSpinLimit; spin++) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void dk_tma_4d(unsigned dst, const CUtensorMap * map, int x, int y, int z, int w, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar) : "memory");
}

template <int HD, int NW>
__global__ void __launch_bounds__(NW * 32, 3) attention_mma_kernel(const AttnParams p) {
    constexpr int BM = 16 * NW;
    constexpr int CH = HD / 8;                 // 16-byte chunks per row
    constexpr int KS = HD / 16;                // k-steps of QK^T
    constexpr int DT = HD / 8;                 // d-tiles of the output
    static_assert(BM <= BN, "the Q tile borrows the second V stage");
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char * sK = smem;                             // [2][BN][HD]
    unsigned char * sV = sK + 2 * BN * HD * 2;             // [2][BN][HD]
    // Q lives in shared memory only until its fragments are in registers: it borrows the second V stage, which
    // is first filled after that (three CTAs of 64 KB fit an SM, two of 80 KB did).
    unsigned char * sQ = sV + BN * HD * 2;
    __shared__ long long s_cell[2][BN];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g_ = lane >> 2, t_ = lane & 3;
    const int kvh = blockIdx.y;
    const int s = blockIdx.z / p.n_split, split = blockIdx.z % p.n_split;
    const int G = p.nh / p.nkv;
    const int q0 = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - q0;
    const int ctx = p.ctx_len[s];
    const int pos0 = ctx - q_len;
    const int rows_total = q_len * G;
    const int row0 = (gridDim.x - 1 - blockIdx.x) * BM;   // late rows see the most keys: they start first
    if (row0 >= rows_total) return;

    const int tok_min = row0 / G;
    const int tok_max = min(rows_total - 1, row0 + BM - 1) / G;
    const int k_hi = pos0 + tok_max;
    const int k_lo = p.window > 0 ? max(0, pos0 + tok_min - p.window + 1) : 0;
    const int tile_lo = k_lo / BN, tile_hi = k_hi / BN;
    const int n_tiles = tile_hi - tile_lo + 1;
    const int per = (n_tiles + p.n_split - 1) / p.n_split;
    const int tile_begin = tile_lo + split * per;
    const int tile_end = min(tile_hi + 1, tile_begin + per);

    const int * bt = p.block_table + (size_t) s * p.max_blocks;

    // ---- loaders ---------------------------------------------------------------------------
    auto load_q = [&]() {
        for (int c = tid; c < BM * CH; c += NW * 32) {
            const int r = c / CH, ch = c % CH;
            const int R = row0 + r;
            const bool valid = R < rows_total;
            const int tok = valid ? R / G : 0, head = kvh * G + (valid ? R % G : 0);
            const __nv_bfloat16 * src = p.q + ((size_t) (q0 + tok) * p.nh + head) * HD + ch * 8;
            cp_async16(smem_u32(sQ + swz<HD>(r, ch)), src, valid);
        }
    };
    // Row bases (element offset of a key's row in the cache, -1: nothing to load) are looked up once per
    // row into shared memory; the copies then run over consecutive 16-byte chunks, so that a warp's
    // request covers whole contiguous rows.
    auto lookup_rows = [&](int tile, int slot) {
        if (tid < BN) {
            const int j = tile * BN + tid;
            long long cell = -1;
            if (tile < tile_end && j <= k_hi) {
                const int page = bt[j / p.page_size];
                if (page >= 0 && page < p.num_pages)
                    cell = (((long long) page * p.nkv + kvh) * p.page_size + (j % p.page_size)) * HD;
            }
            s_cell[slot][tid] = cell;
        }
    };
    auto load_kv = [&](int stage, int slot) {
        unsigned char * dK = sK + stage * BN * HD * 2;
        unsigned char * dV = sV + stage * BN * HD * 2;
#pragma unroll
        for (int c = tid; c < BN * CH; c += NW * 32) {
            const int r = c / CH, ch = c % CH;
            const long long cell = s_cell[slot][r];
            const bool valid = cell >= 0;
            const size_t off = valid ? (size_t) cell + ch * 8 : 0;
            cp_async16(smem_u32(dK + swz<HD>(r, ch)), p.k_cache + off, valid);
            cp_async16(smem_u32(dV + swz<HD>(r, ch)), p.v_cache + off, valid);
        }
    };

    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    // rows of this thread: warp * 16 + g_ and + 8
    int row_tok[2], row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int R = row0 + warp * 16 + g_ + 8 * h;
        row_ok[h] = R < rows_total;
        row_tok[h] = pos0 + (row_ok[h] ? R / G : 0);       // position of the row's token
    }
    // bounds over the 16 rows of this warp: tiles wholly below every row's diagonal need no mask
    const int wr0 = row0 + warp * 16, wr1 = min(rows_total - 1, wr0 + 15);
    const bool warp_rows_ok = wr0 + 15 < rows_total;
    const int warp_pos_min = pos0 + min(wr0, rows_total - 1) / G, warp_pos_max = pos0 + max(wr1, 0) / G;

    if (tile_begin < tile_end) {
        lookup_rows(tile_begin, 0);
        lookup_rows(tile_begin + 1, 1);
        __syncthreads();
        load_q();
        cp_async_commit();
        load_kv(0, 0);
        cp_async_commit();

        unsigned qf[KS][4];
        cp_async_wait<1>();                         // Q has landed (the first K/V tile may still be in flight)
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const int r = warp * 16 + (lane & 15);
            const int ch = ks * 2 + (lane >> 4);
            ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], smem_u32(sQ + swz<HD>(r, ch)));
        }
        __syncthreads();                            // the borrowed stage may be overwritten from here on

        for (int tile = tile_begin; tile < tile_end; tile++) {
            const int stage = (tile - tile_begin) & 1;
            if (tile + 1 < tile_end) {
                load_kv(stage ^ 1, stage ^ 1);      // rows of tile + 1 were looked up an iteration ago
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            lookup_rows(tile + 2, stage);           // slot `stage` held this tile's rows; its copies are issued
            const unsigned char * tK = sK + stage * BN * HD * 2;
            const unsigned char * tV = sV + stage * BN * HD * 2;

            // ---- S = Q K^T -------------------------------------------------------------------
            float sc[BN / 8][4];
#pragma unroll
            for (int i = 0; i < BN / 8; i++) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
#pragma unroll
                for (int np = 0; np < BN / 16; np++) {
                    unsigned b0, b1, b2, b3;
                    const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                    const int ch = ks * 2 + ((lane >> 3) & 1);
                    ldmatrix_x4(b0, b1, b2, b3, smem_u32(tK + swz<HD>(r, ch)));
                    mma16816(sc[2 * np], qf[ks], b0, b1);
                    mma16816(sc[2 * np + 1], qf[ks], b2, b3);
                }
            }
            // ---- mask (only on tiles that touch a row's causal or window edge), online softmax ----
            const int key0 = tile * BN;
            const bool need_mask = key0 + BN - 1 > warp_pos_min || !warp_rows_ok ||
                                   (p.window > 0 && warp_pos_max - key0 >= p.window);
            if (need_mask) {
#pragma unroll
                for (int nt = 0; nt < BN / 8; nt++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int h = e >> 1;
                        const int j = key0 + nt * 8 + 2 * t_ + (e & 1);
                        const bool vis = row_ok[h] && j <= row_tok[h] && (p.window == 0 || row_tok[h] - j < p.window);
                        if (!vis) sc[nt][e] = -INFINITY;
                    }
                }
            }
            float m_new[2] = {m_run[0], m_run[1]};          // maxima of the raw scores (the scale is positive)
#pragma unroll
            for (int nt = 0; nt < BN / 8; nt++) {
                m_new[0] = fmaxf(m_new[0], fmaxf(sc[nt][0], sc[nt][1]));
                m_new[1] = fmaxf(m_new[1], fmaxf(sc[nt][2], sc[nt][3]));
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
                m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
            }
            float corr[2], neg[2], sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                corr[h] = (m_new[h] == -INFINITY) ? 1.0f : exp2f((m_run[h] - m_new[h]) * p.scale_log2);   // m_run = -inf gives 0
                neg[h] = (m_new[h] == -INFINITY) ? 0.0f : m_new[h] * p.scale_log2;
            }
#pragma unroll
            for (int nt = 0; nt < BN / 8; nt++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int h = e >> 1;
                    const float pv = fast_exp2(fmaf(sc[nt][e], p.scale_log2, -neg[h]));   // 2^-inf = 0 for masked keys
                    sc[nt][e] = pv;
                    sum[h] += pv;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                l_run[h] = l_run[h] * corr[h] + sum[h];     // per-thread partial; reduced over the quad at the end
                m_run[h] = m_new[h];
            }
            if (corr[0] != 1.0f || corr[1] != 1.0f) {       // the maximum of long rows settles early
#pragma unroll
                for (int dt = 0; dt < DT; dt++) {
                    o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
                    o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
                }
            }
            // ---- O += P V ------------------------------------------------------------------------
#pragma unroll
            for (int kk = 0; kk < BN / 16; kk++) {
                unsigned a[4];
                a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
                a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
                a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < DT / 2; dp++) {
                    unsigned b0, b1, b2, b3;
                    const int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    const int ch = dp * 2 + (lane >> 4);
                    ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(tV + swz<HD>(r, ch)));
                    mma16816(o[2 * dp], a, b0, b1);
                    mma16816(o[2 * dp + 1], a, b2, b3);
                }
            }
            __syncthreads();      // everyone is done with this stage before it is refilled
        }
    }

    // ---- finish --------------------------------------------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int R = row0 + warp * 16 + g_ + 8 * h;
        if (R >= rows_total) continue;
        const int tok = R / G, head = kvh * G + R % G;
        const float inv = l_run[h] > 0.0f ? 1.0f / l_run[h] : 0.0f;
        const size_t row_idx = (size_t) (q0 + tok) * p.nh + head;
        if (p.n_split == 1) {
            __nv_bfloat16 * dst = p.out + row_idx * HD;
#pragma unroll
            for (int dt = 0; dt < DT; dt++) {
                const int d = dt * 8 + 2 * t_;
                *reinterpret_cast<__nv_bfloat162 *>(dst + d) = __floats2bfloat162_rn(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
            }
        } else {
            float * dst = p.part_o + (row_idx * p.n_split + split) * HD;
#pragma unroll
            for (int dt = 0; dt < DT; dt++) {
                const int d = dt * 8 + 2 * t_;
                *reinterpret_cast<float2 *>(dst + d) = make_float2(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
            }
            if (t_ == 0)    // log-sum-exp in base 2; -inf marks a part that saw no key
                p.part_lse[row_idx * p.n_split + split] = l_run[h] > 0.0f ? m_run[h] * p.scale_log2 + log2f(l_run[h]) : -INFINITY;
        }
    }
}

// Decode form: few rows (the G heads of one token, up to 16 rows per CTA), many keys.  The four warps
// of a CTA share the rows and split the KEYS of every 64-key tile (16 each); each warp keeps a running
// (max, sum, output) of its own, and the four are merged through shared memory at the end.  Three
// cp.async stages keep two tiles in flight while one is consumed.  Every thread fetches one half row of
// K and of V per tile, so a tile costs it one block-table lookup, and that lookup is issued a tile ahead
// of its use.  With n_split > 1 the CTA that finishes last for its rows (a counter per row tile, bumped
// after the partial results are fenced out) merges the parts and writes the output, so there is no
// second launch; it leaves the counter at zero for the next launch.
// CLUSTER: the n_split (2 to 8) CTAs of a row tile are one thread-block cluster.  Each leaves its
// (max, sum, unnormalised output) in its own shared memory; after a cluster barrier every CTA merges a
// slice of the head's columns, reading the others' shared memory directly, and writes it out.  No scratch
// memory, no fence, no counter: the merge costs two cluster barriers instead of three trips through L2.
// FUSED (steps in which every sequence has one token): the kernel takes the output of the Q|K|V projection
// instead of prepared heads.  Every CTA normalises and rotates the query heads of its KV head itself
// (src/iian/arch/qwen3.cpp:80-87: RMSNorm over the head, then NEOX rotation), with the arithmetic of
// rope_kv.cu in the same order, so both routes give the same bits.  The CTA whose key range holds the
// token's own position also normalises and rotates the new key, writes it and the new value to the cache for
// later steps, and puts both from shared memory into the tile they belong to after that tile's copy has landed:
// no fence and no reading back lie on the path.  This saves a launch and a round trip of Q through memory.
// STAGES: tiles of shared memory per CTA.  Three keep two tiles in flight; two leave room for a third CTA
// on the SM, which pays when a step's CTAs then fit the GPU at once with fewer tiles each.
// TMA: the K and V tiles come by cp.async.bulk.tensor through the block table (a box per page and half head,
// 128-byte swizzle, as in the tcgen05 prefill kernel) and are awaited on an mbarrier per stage, instead of 16-byte
// cp.async copies with a looked-up address per row: the copies of a tile are sixteen instructions of one warp rather
// than sixteen of every thread, and they do not pass through the load/store units that bound the cp.async form at
// three quarters of the memory bandwidth.  Head size 128, pages of 8 to 64 tokens.
template <int HD, bool CLUSTER, bool FUSED, int STAGES, bool TMA>
__global__ void __launch_bounds__(128, STAGES == 2 ? 3 : 2) attention_decode_kernel(const AttnParams p, const __grid_constant__ KvMaps maps) {
    constexpr int NW = 4, BM = 16;
    constexpr int CH = HD / 8, KS = HD / 16, DT = HD / 8;
    constexpr int TILE_BYTES = BN * HD * 2;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // (the swizzle of a TMA tile is a function of the address: tiles start on 1024-byte boundaries)
    unsigned char * smem = TMA ? (unsigned char *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023) : smem_raw;
    unsigned char * sQ = smem;                               // [16][HD]
    unsigned char * sK = sQ + BM * HD * 2;                   // [STAGES][BN][HD]
    unsigned char * sV = sK + STAGES * TILE_BYTES;           // [STAGES][BN][HD]
    __shared__ int s_last;
    __shared__ long long s_cell[TMA ? 1 : STAGES][BN];
    __shared__ __align__(8) unsigned long long full_bar[STAGES];     // TMA: a tile's bytes have landed

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g_ = lane >> 2, t_ = lane & 3;
    const int kvh = blockIdx.y;
    const int s = blockIdx.z / p.n_split, split = blockIdx.z % p.n_split;
    const int G = p.nh / p.nkv;
    const int q0 = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - q0;
    const int ctx = p.ctx_len[s];
    const int pos0 = ctx - q_len;
    const int rows_total = q_len * G;
    const int row0 = blockIdx.x * BM;
    if (row0 >= rows_total) return;

    const int tok_min = row0 / G;
    const int tok_max = min(rows_total - 1, row0 + BM - 1) / G;
    const int k_hi = pos0 + tok_max;
    const int k_lo = p.window > 0 ? max(0, pos0 + tok_min - p.window + 1) : 0;
    const int tile_lo = k_lo / BN, tile_hi = k_hi / BN;
    const int n_tiles = tile_hi - tile_lo + 1;
    const int per = (n_tiles + p.n_split - 1) / p.n_split;
    const int tile_begin = tile_lo + split * per;
    const int tile_end = min(tile_hi + 1, tile_begin + per);
    const int n_my = max(0, tile_end - tile_begin);
    const int * bt = p.block_table + (size_t) s * p.max_blocks;

    // Row bases (element offset of a key's row in the cache, -1: nothing to load) are looked up once per
    // row into a ring of shared-memory slots, a tile ahead of the copies that use them; the copies run
    // over consecutive 16-byte chunks, so that a warp's request covers whole contiguous rows.
    const int page_shift = (p.page_size & (p.page_size - 1)) == 0 ? __ffs(p.page_size) - 1 : -1;
    auto lookup_rows = [&](int tile, int slot) {
        if (tid < BN) {
            const int j = tile * BN + tid;
            long long cell = -1;
            if (tile < tile_end && j <= k_hi) {
                const int blk = page_shift >= 0 ? j >> page_shift : j / p.page_size;
                const int page = bt[blk];
                if (page >= 0 && page < p.num_pages)
                    cell = (((long long) page * p.nkv + kvh) * p.page_size + (j - blk * p.page_size)) * HD;
            }
            s_cell[slot][tid] = cell;
        }
    };
    // A thread copies the same 16-byte column of rows tid / CH, tid / CH + ROWS_PER_PASS, ...: the swizzled
    // column is the same in every pass (ROWS_PER_PASS is a multiple of 8), so only the row base changes.
    constexpr int ROWS_PER_PASS = NW * 32 / CH;
    const int ld_row = tid / CH, ld_ch = tid % CH;
    const unsigned ld_dst = swz<HD>(ld_row, ld_ch);
    auto load_kv = [&](int stage) {                          // the slot of a tile is its stage
        const unsigned dK = smem_u32(sK + stage * TILE_BYTES) + ld_dst;
        const unsigned dV = smem_u32(sV + stage * TILE_BYTES) + ld_dst;
#pragma unroll
        for (int i = 0; i < BN / ROWS_PER_PASS; i++) {
            const long long cell = s_cell[stage][ld_row + i * ROWS_PER_PASS];
            const bool valid = cell >= 0;
            const size_t off = valid ? (size_t) cell + ld_ch * 8 : 0;
            cp_async16(dK + i * ROWS_PER_PASS * HD * 2, p.k_cache + off, valid);
            cp_async16(dV + i * ROWS_PER_PASS * HD * 2, p.v_cache + off, valid);
        }
    };

    // TMA form: lane l of warp 0 fetches one box of a tile: half l & 1 of the head, K or V by bit 1, page l >> 2 of
    // the tile.  The page numbers are read a tile before the copies that use them are issued.
    const int ld_half = lane & 1, ld_which = (lane >> 1) & 1, ld_pg = lane >> 2;
    const bool ld_lane = TMA && warp == 0 && ld_pg * p.page_size < BN;
    auto tma_page = [&](int tile) -> int {
        int page = p.num_pages;                              // out of range: the box is filled with zeros
        if (ld_lane && tile < tile_end) {
            const int j0 = tile * BN + ld_pg * p.page_size;
            if (j0 <= k_hi) {
                const int pg = bt[page_shift >= 0 ? j0 >> page_shift : j0 / p.page_size];
                if (pg >= 0 && pg < p.num_pages) page = pg;
            }
        }
        return page;
    };
    auto tma_issue = [&](int stage, int page) {              // warp 0, all lanes
        const unsigned bar = smem_u32(&full_bar[stage]);
        if (lane == 0) dk_expect_tx(bar, 2 * TILE_BYTES);
        __syncwarp();
        if (ld_lane) {
            unsigned char * base = (ld_which == 0 ? sK : sV) + stage * TILE_BYTES + ld_half * (BN * 128) + ld_pg * p.page_size * 128;
            dk_tma_4d(smem_u32(base), ld_which == 0 ? &maps.k : &maps.v, ld_half * 64, 0, kvh, page, bar);
        }
    };
    int pg_q[STAGES];
    if (TMA) {
        if (tid == 0) {
#pragma unroll
            for (int st = 0; st < STAGES; st++) dk_mbar_init(smem_u32(&full_bar[st]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
#pragma unroll
        for (int st = 0; st < STAGES; st++) pg_q[st] = tma_page(tile_begin + st);
    }

    auto load_ahead = [&]() {                                // the first STAGES - 1 tiles, one copy group each
#pragma unroll
        for (int st = 0; st < STAGES - 1; st++) {
            if (TMA) {
                if (st < n_my && warp == 0) tma_issue(st, pg_q[st]);
            } else {
                if (st < n_my) load_kv(st);
                cp_async_commit();
            }
        }
    };

    float o[DT][4];
#pragma unroll
    for (int i = 0; i < DT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    int row_tok[2], row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int R = row0 + g_ + 8 * h;
        row_ok[h] = R < rows_total;
        row_tok[h] = pos0 + (row_ok[h] ? R / G : 0);
    }
    const int pos_min = pos0 + tok_min, pos_max = pos0 + tok_max;
    const bool rows_full = row0 + BM <= rows_total;

    // Everything up to here reads only the step's integer buffers, which were uploaded before the first
    // kernel of the step; Q and the newest K/V rows come from the kernel before this one.
    if (n_my > 0 && !TMA) {
#pragma unroll
        for (int st = 0; st < STAGES; st++) lookup_rows(tile_begin + st, st);
    }
    pdl_wait();
    __shared__ __align__(16) __nv_bfloat16 s_new[2][HD];      // FUSED: the new key and value of the token (owner CTA)
    const int new_tile = k_hi / BN - tile_begin;              // FUSED: which of this CTA's tiles holds the token's own position
    const bool owner = FUSED && new_tile >= 0 && new_tile < n_my;
    bool patch = false;
    if (n_my > 0) {
        __syncthreads();
        if (!FUSED) {
            for (int c = tid; c < BM * CH; c += NW * 32) {          // Q rows
                const int r = c / CH, ch = c % CH;
                const int R = row0 + r;
                const bool valid = R < rows_total;
                const int tok = valid ? R / G : 0, head = kvh * G + (valid ? R % G : 0);
                cp_async16(smem_u32(sQ + swz<HD>(r, ch)), p.q + ((size_t) (q0 + tok) * p.nh + head) * HD + ch * 8, valid);
            }
            load_ahead();
        } else {
            // (one token per sequence: q_len 1, rows_total G <= 16, row0 0, k_hi the token's position)
            // The CTA whose keys include the token's own position makes the new key and value itself: they go to the
            // cache for later steps and, through shared memory, straight into the tile they belong to once that tile's
            // copy has landed (the copy brings whatever the cell held before) -- no fence, no reading back.
            load_ahead();
            constexpr int half = HD / 2;
            const int heads_total = p.nh + 2 * p.nkv;
            const __nv_bfloat16 * tok_in = p.qkv + (size_t) q0 * heads_total * HD;
            const float2 * tab = p.table != nullptr ? p.table + (size_t) q0 * half : nullptr;
            const int p0 = 2 * lane;                                  // a lane owns pairs p0 and p0 + 1 (HD <= 128)
            // normalise and rotate one head; dst0/dst1 receive elements (p0, p0 + 1) and (half + p0, half + p0 + 1)
            auto norm_rope = [&](const __nv_bfloat16 * src, const float * w, bool rotate, __nv_bfloat16 * dst0, __nv_bfloat16 * dst1) {
                float2 a = make_float2(0.0f, 0.0f), c = make_float2(0.0f, 0.0f);
                float ss = 0.0f;
                if (p0 < half) {
                    a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(src + p0));
                    c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(src + half + p0));
                    ss += a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
                }
                float inv = 1.0f;
                if (w != nullptr) {
                    ss = warp_sum(ss);
                    inv = rsqrtf(ss / (float) HD + p.eps);
                }
                if (p0 < half) {
                    if (w != nullptr) {
                        const float2 wl = *reinterpret_cast<const float2 *>(w + p0), wh = *reinterpret_cast<const float2 *>(w + half + p0);
                        a.x = a.x * inv * wl.x; a.y = a.y * inv * wl.y;
                        c.x = c.x * inv * wh.x; c.y = c.y * inv * wh.y;
                    }
                    if (rotate) {
                        const float4 cssn = *reinterpret_cast<const float4 *>(tab + p0);      // cos0 sin0 cos1 sin1
                        const float2 r0 = make_float2(rot_lo(a.x, c.x, cssn.x, cssn.y), rot_lo(a.y, c.y, cssn.z, cssn.w));
                        const float2 r1 = make_float2(rot_hi(a.x, c.x, cssn.x, cssn.y), rot_hi(a.y, c.y, cssn.z, cssn.w));
                        a = r0; c = r1;
                    }
                    *reinterpret_cast<__nv_bfloat162 *>(dst0) = __floats2bfloat162_rn(a.x, a.y);
                    *reinterpret_cast<__nv_bfloat162 *>(dst1) = __floats2bfloat162_rn(c.x, c.y);
                }
            };
            for (int c = tid; c < BM * CH; c += NW * 32) {              // rows beyond the G heads are zero
                const int r = c / CH, ch = c % CH;
                if (r >= rows_total) *reinterpret_cast<uint4 *>(sQ + swz<HD>(r, ch)) = make_uint4(0u, 0u, 0u, 0u);
            }
            for (int r = warp; r < rows_total; r += NW) {
                const __nv_bfloat16 * src = tok_in + (size_t) (kvh * G + r) * HD;
                __nv_bfloat16 * d0 = reinterpret_cast<__nv_bfloat16 *>(sQ + swz<HD>(r, p0 >> 3)) + (p0 & 7);
                __nv_bfloat16 * d1 = reinterpret_cast<__nv_bfloat16 *>(sQ + swz<HD>(r, (half + p0) >> 3)) + (p0 & 7);
                norm_rope(src, p.q_weight, tab != nullptr, d0, d1);
            }
            if (owner && p.write_kv) {
                const int slot = p.slots[q0];
                if (slot >= 0 && slot < p.num_pages * p.page_size) {
                    patch = true;
                    if (warp == 0) {
                        const __nv_bfloat16 * src = tok_in + (size_t) (p.nh + kvh) * HD;
                        norm_rope(src, p.k_weight, tab != nullptr, s_new[0] + p0, s_new[0] + half + p0);
                    } else if (warp == 1) {
                        const __nv_bfloat16 * src = tok_in + (size_t) (p.nh + p.nkv + kvh) * HD;
                        if (lane < CH) *reinterpret_cast<uint4 *>(s_new[1] + lane * 8) = *reinterpret_cast<const uint4 *>(src + lane * 8);
                    }
                }
            }
            __syncthreads();
            if (patch && tid < 2 * CH) {                     // the new rows into the cache, 16 bytes a thread
                const int slot = p.slots[q0];
                const int page = slot / p.page_size, off = slot - page * p.page_size;
                const size_t cell = (((size_t) page * p.nkv + kvh) * p.page_size + off) * HD;
                const int which = tid / CH, ch = tid % CH;
                __nv_bfloat16 * dst = (which == 0 ? p.k_cache_w : p.v_cache_w) + cell + ch * 8;
                *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(s_new[which] + ch * 8);
            }
        }

        unsigned qf[KS][4];
        int pg_next = TMA ? pg_q[STAGES - 1] : 0;
        bool failed = false;
        for (int i = 0; i < n_my; i++) {
            if (TMA) {
                if (i + STAGES - 1 < n_my && warp == 0) tma_issue((i + STAGES - 1) % STAGES, pg_next);
                pg_next = tma_page(tile_begin + i + STAGES);
                if (!dk_wait(smem_u32(&full_bar[i % STAGES]), (unsigned) (i / STAGES) & 1u)) failed = true;
                if (i == 0 && !FUSED) {                          // the Q rows came by cp.async
                    cp_async_commit();
                    cp_async_wait<0>();
                    __syncthreads();
                }
            } else {
                if (i + STAGES - 1 < n_my) load_kv((i + STAGES - 1) % STAGES);
                cp_async_commit();
                cp_async_wait<STAGES - 1>();
                __syncthreads();
            }
            if (FUSED && patch && i == new_tile) {               // the token's own key and value replace what the copy brought
                if (tid < 2 * CH) {
                    const int which = tid / CH, ch = tid % CH;
                    unsigned char * tile = (which == 0 ? sK : sV) + (i % STAGES) * TILE_BYTES;
                    *reinterpret_cast<uint4 *>(tile + kv_off<HD, TMA>(k_hi % BN, ch)) = *reinterpret_cast<const uint4 *>(s_new[which] + ch * 8);
                    if (TMA) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // a later copy overwrites the row
                }
                __syncthreads();
            }
            if (!TMA) lookup_rows(tile_begin + i + STAGES, i % STAGES);    // this tile's copies were issued earlier
            if (i == 0) {
#pragma unroll
                for (int ks = 0; ks < KS; ks++)
                    ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                                smem_u32(sQ + swz<HD>(lane & 15, ks * 2 + (lane >> 4))));
            }
            const unsigned char * tK = sK + (i % STAGES) * TILE_BYTES;
            const unsigned char * tV = sV + (i % STAGES) * TILE_BYTES;
            float sc[2][4];
#pragma unroll
            for (int n = 0; n < 2; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                unsigned b0, b1, b2, b3;
                const int r = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
                ldmatrix_x4(b0, b1, b2, b3, smem_u32(tK + kv_off<HD, TMA>(r, ks * 2 + ((lane >> 3) & 1))));
                mma16816(sc[0], qf[ks], b0, b1);
                mma16816(sc[1], qf[ks], b2, b3);
            }
            const int key0 = (tile_begin + i) * BN + warp * 16;
            const bool need_mask = key0 + 15 > pos_min || !rows_full || (p.window > 0 && pos_max - key0 >= p.window);
            if (need_mask) {
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int h = e >> 1;
                        const int j = key0 + nt * 8 + 2 * t_ + (e & 1);
                        const bool vis = row_ok[h] && j <= row_tok[h] && (p.window == 0 || row_tok[h] - j < p.window);
                        if (!vis) sc[nt][e] = -INFINITY;
                    }
                }
            }
            float m_new[2];
            m_new[0] = fmaxf(m_run[0], fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1])));
            m_new[1] = fmaxf(m_run[1], fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3])));
#pragma unroll
            for (int h = 0; h < 2; h++) {
                m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
                m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
            }
            float corr[2], neg[2], sum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                corr[h] = (m_new[h] == -INFINITY) ? 1.0f : exp2f((m_run[h] - m_new[h]) * p.scale_log2);
                neg[h] = (m_new[h] == -INFINITY) ? 0.0f : m_new[h] * p.scale_log2;
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int h = e >> 1;
                    const float pv = fast_exp2(fmaf(sc[nt][e], p.scale_log2, -neg[h]));
                    sc[nt][e] = pv;
                    sum[h] += pv;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                l_run[h] = l_run[h] * corr[h] + sum[h];
                m_run[h] = m_new[h];
            }
            if (corr[0] != 1.0f || corr[1] != 1.0f) {
#pragma unroll
                for (int dt = 0; dt < DT; dt++) {
                    o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
                    o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
                }
            }
            unsigned a[4];
            a[0] = pack_bf16(sc[0][0], sc[0][1]);
            a[1] = pack_bf16(sc[0][2], sc[0][3]);
            a[2] = pack_bf16(sc[1][0], sc[1][1]);
            a[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
            for (int dp = 0; dp < DT / 2; dp++) {
                unsigned b0, b1, b2, b3;
                const int r = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(tV + kv_off<HD, TMA>(r, dp * 2 + (lane >> 4))));
                mma16816(o[2 * dp], a, b0, b1);
                mma16816(o[2 * dp + 1], a, b2, b3);
            }
            if (TMA) {
                // A wait that gave up (its copy never landed) ends the walk for the whole CTA: the result is not
                // valid, and the host finds out from the status words.
                if (__syncthreads_or(failed ? 1 : 0)) {
                    if (tid == 0 && p.status != nullptr) { p.status[0] = 11; p.status[1] = i; }
                    break;
                }
            } else {
                __syncthreads();
            }
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();        // the keys are read: the next kernel may start fetching its weights

    // ---- merge the four warps ------------------------------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float * mo = reinterpret_cast<float *>(sK);              // [NW][16][HD]   (stage memory is free now)
    float * ml = mo + NW * BM * HD;                          // [NW][16][2]
    __syncthreads();
#pragma unroll
    for (int dt = 0; dt < DT; dt++) {
        const int d = dt * 8 + 2 * t_;
        *reinterpret_cast<float2 *>(mo + ((size_t) warp * BM + g_) * HD + d) = make_float2(o[dt][0], o[dt][1]);
        *reinterpret_cast<float2 *>(mo + ((size_t) warp * BM + g_ + 8) * HD + d) = make_float2(o[dt][2], o[dt][3]);
    }
    if (t_ == 0) {
        ml[(warp * BM + g_) * 2] = m_run[0];         ml[(warp * BM + g_) * 2 + 1] = l_run[0];
        ml[(warp * BM + g_ + 8) * 2] = m_run[1];     ml[(warp * BM + g_ + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    const int mr = tid >> 3, mpart = tid & 7;                // 8 threads per row, HD / 8 columns each
    const int mR = row0 + mr;
    const bool m_ok = mR < rows_total;
    const size_t row_idx = m_ok ? (size_t) (q0 + mR / G) * p.nh + kvh * G + mR % G : 0;
    float * cO = ml + NW * BM * 2;                           // [16][HD] unnormalised output of this CTA (cluster form)
    float * cML = cO + BM * HD;                              // [16][2]  its max and sum
    if (m_ok) {
        float mw[NW], m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) { mw[w] = ml[(w * BM + mr) * 2]; m = fmaxf(m, mw[w]); }
        float sw[NW], l = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            sw[w] = (mw[w] == -INFINITY) ? 0.0f : exp2f((mw[w] - m) * p.scale_log2);
            l += sw[w] * ml[(w * BM + mr) * 2 + 1];
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
        for (int c = 0; c < HD / 8; c += 2) {
            const int d = mpart * (HD / 8) + c;
            float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; w++) {
                const float2 x = *reinterpret_cast<const float2 *>(mo + ((size_t) w * BM + mr) * HD + d);
                v0 += sw[w] * x.x;
                v1 += sw[w] * x.y;
            }
            if (CLUSTER)
                *reinterpret_cast<float2 *>(cO + mr * HD + d) = make_float2(v0, v1);
            else if (p.n_split == 1)
                *reinterpret_cast<__nv_bfloat162 *>(p.out + row_idx * HD + d) = __floats2bfloat162_rn(v0 * inv, v1 * inv);
            else
                *reinterpret_cast<float2 *>(p.part_o + (row_idx * p.n_split + split) * HD + d) = make_float2(v0 * inv, v1 * inv);
        }
        if (CLUSTER) {
            if (mpart == 0) { cML[mr * 2] = m; cML[mr * 2 + 1] = l; }
        } else if (p.n_split > 1 && mpart == 0)        // log-sum-exp in base 2; -inf marks a part that saw no key
            p.part_lse[row_idx * p.n_split + split] = l > 0.0f ? m * p.scale_log2 + log2f(l) : -INFINITY;
    }
    if (CLUSTER) {
        // Every CTA of the cluster gets here (none returns early: they share the row tile), so the barriers
        // are complete.  CTA `rank` merges columns [rank, rank + 1) * ceil(HD / n_split) of every row.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int ns = p.n_split, rank = (int) cluster.block_rank();
        const int cols = (HD + ns - 1) / ns;
        const int n_rows = min(BM, rows_total - row0);
        for (int idx = tid; idx < n_rows * cols; idx += NW * 32) {
            const int r = idx / cols, d = rank * cols + idx % cols;
            if (d >= HD) continue;
            float mc[16], m = -INFINITY;
            for (int c = 0; c < ns; c++) {
                mc[c] = cluster.map_shared_rank(cML, c)[r * 2];
                m = fmaxf(m, mc[c]);
            }
            float l = 0.0f, v = 0.0f;
            for (int c = 0; c < ns; c++) {                   // in the order of the parts, whatever their timing
                if (mc[c] == -INFINITY) continue;
                const float f = exp2f((mc[c] - m) * p.scale_log2);
                l += f * cluster.map_shared_rank(cML, c)[r * 2 + 1];
                v += f * cluster.map_shared_rank(cO, c)[r * HD + d];
            }
            const int R = row0 + r;
            const size_t ri = (size_t) (q0 + R / G) * p.nh + kvh * G + R % G;
            p.out[ri * HD + d] = __float2bfloat16_rn(l > 0.0f ? v / l : 0.0f);
        }
        cluster.sync();                                      // nobody leaves while its shared memory is being read
        return;
    }
    if (p.n_split == 1) return;

    // ---- the last CTA of these rows merges the parts -------------------------------------------
    __threadfence();
    __syncthreads();
    int * counter = p.counters + ((size_t) s * p.nkv + kvh) * gridDim.x + blockIdx.x;
    if (tid == 0) s_last = (atomicAdd(counter, 1) == p.n_split - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (m_ok) {
        const float * lse = p.part_lse + row_idx * p.n_split;
        float mx = -INFINITY;
        for (int i = 0; i < p.n_split; i++) mx = fmaxf(mx, __ldcg(lse + i));
        float acc[HD / 8];
#pragma unroll
        for (int c = 0; c < HD / 8; c++) acc[c] = 0.0f;
        float wsum = 0.0f;
        if (mx != -INFINITY) {
            for (int i = 0; i < p.n_split; i++) {
                const float w = exp2f(__ldcg(lse + i) - mx);
                if (w == 0.0f) continue;
                wsum += w;
                const float * po = p.part_o + (row_idx * p.n_split + i) * HD + mpart * (HD / 8);
#pragma unroll
                for (int c = 0; c < HD / 8; c += 4) {
                    const float4 x = __ldcg(reinterpret_cast<const float4 *>(po + c));
                    acc[c] += w * x.x; acc[c + 1] += w * x.y; acc[c + 2] += w * x.z; acc[c + 3] += w * x.w;
                }
            }
        }
        const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
        __nv_bfloat16 * dst = p.out + row_idx * HD + mpart * (HD / 8);
#pragma unroll
        for (int c = 0; c < HD / 8; c += 2)
            *reinterpret_cast<__nv_bfloat162 *>(dst + c) = __floats2bfloat162_rn(acc[c] * inv, acc[c + 1] * inv);
    }
    if (tid == 0) *counter = 0;
}

typedef CUresult (*KvEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of a cache [num_pages, nkv, page_size, 128] bf16 with boxes of one page and half a head
// ([page_size rows, 64 values], 128-byte swizzle).  The maps of the caches seen so far are kept (a cache keeps its
// address for the life of an engine), so that a launch costs no call into the driver.
static int kv_map_for(const void * base, int num_pages, int nkv, int page_size, CUtensorMap * out) {
    struct Entry { const void * base; int num_pages, nkv, page_size; CUtensorMap map; };
    static Entry cache[256];
    static int n_cached = 0, next = 0;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < n_cached; i++) {
        const Entry & e = cache[i];
        if (e.base == base && e.num_pages == num_pages && e.nkv == nkv && e.page_size == page_size) { *out = e.map; return IIAN_OK; }
    }
    static KvEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void * f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            return IIAN_ERR_LIMIT;
        fn = (KvEncodeFn) f;
    }
    cuuint64_t dims[4] = {128, (cuuint64_t) page_size, (cuuint64_t) nkv, (cuuint64_t) num_pages};
    cuuint64_t strides[3] = {256, (cuuint64_t) page_size * 256, (cuuint64_t) nkv * page_size * 256};
    cuuint32_t box[4] = {64, (cuuint32_t) page_size, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap map;
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 2000 + (int) r;
    Entry & e = cache[next];
    e.base = base; e.num_pages = num_pages; e.nkv = nkv; e.page_size = page_size; e.map = map;
    next = (next + 1) % 256;
    if (n_cached < 256) n_cached++;
    *out = map;
    return IIAN_OK;
}

template <int HD, bool CLUSTER, bool FUSED, int STAGES, bool TMA>
static int launch_decode_st(const AttnParams & p, const KvMaps & maps, int S, int max_rows, cudaStream_t stream) {
    const size_t smem = (size_t) 16 * HD * 2 + 2 * STAGES * BN * HD * 2 + (TMA ? 1024 : 0);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, CLUSTER, FUSED, STAGES, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return 1000 + (int) e;
        configured = true;
    }
    dim3 grid((max_rows + 15) / 16, p.nkv, S * p.n_split);
    if (!CLUSTER) return iian_launch(attention_decode_kernel<HD, CLUSTER, FUSED, STAGES, TMA>, grid, dim3(128), smem, stream, p, maps);
    if (p.n_split > 8) {                                   // clusters of 9 to 16 CTAs have to be asked for
        static bool allowed = false;
        if (!allowed) {
            cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, CLUSTER, FUSED, STAGES, TMA>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return 1000 + (int) e;
            allowed = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = (unsigned) p.n_split;       // the parts of one row tile are consecutive in z
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_kernel<HD, CLUSTER, FUSED, STAGES, TMA>, p, maps);
    return e == cudaSuccess ? IIAN_OK : 1000 + (int) e;
}

static int decode_sm_count() {
    static int n[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (n[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n[dev] = v;
    }
    return n[dev];
}

static int g_decode_stages = 2;
static int g_unsplit_stages = 0;        // 0: the rule below; 2 or 3: that many for unsplit keys
template <int HD, bool CLUSTER, bool FUSED = false>
static int launch_decode(const AttnParams & p, int S, int max_rows, cudaStream_t stream) {
    // unsplit keys mean many sequences, each CTA walking a whole context: the deeper pipeline pays there
    bool deep = g_decode_stages == 3;
    if (p.n_split == 1) {
        // Unsplit keys: two CTAs per SM with three stages each stream faster than three CTAs with two (a wave of the
        // former takes about 0.87 of a wave of the latter), unless the former need a wave more: 320 (sequence, KV
        // head) pairs of 2048 keys take 99.7 us as two waves of 296 and 59.6 us as one wave of 444; 512 pairs 103.9
        // against 118.4 us (two waves either way); 640 pairs 150.3 against 122.9 us (three waves against two).
        const int sms = decode_sm_count();
        const long long ctas = (long long) ((max_rows + 15) / 16) * p.nkv * S;
        const long long waves3 = (ctas + 2 * sms - 1) / (2 * sms), waves2 = (ctas + 3 * sms - 1) / (3 * sms);
        deep = g_unsplit_stages != 0 ? g_unsplit_stages == 3 : waves3 * 100 <= waves2 * 115;
    }
    KvMaps maps = {};
    if constexpr (HD == 128) {
        // the TMA form: a status buffer to report to, pages that divide a tile and hold whole swizzle atoms
        const int ps = p.page_size;
        // (measured, one launch: with one or two sequences, whose CTAs have few tiles each and wait for the first of them,
        // the cp.async form is 2 to 7 % faster -- 26.4 against 28.2 us at batch 1 and 8k of context; from 8 sequences
        // on the TMA form is as fast or up to 4 % faster)
        if (p.status != nullptr && (ps == 8 || ps == 16 || ps == 32 || ps == 64) && S * p.nkv >= 32) {
            int rc = kv_map_for(p.k_cache, p.num_pages, p.nkv, ps, &maps.k);
            if (rc == IIAN_OK) rc = kv_map_for(p.v_cache, p.num_pages, p.nkv, ps, &maps.v);
            if (rc != IIAN_OK) return rc;
            if (deep) return launch_decode_st<HD, CLUSTER, FUSED, 3, true>(p, maps, S, max_rows, stream);
            return launch_decode_st<HD, CLUSTER, FUSED, 2, true>(p, maps, S, max_rows, stream);
        }
    }
    if (deep) return launch_decode_st<HD, CLUSTER, FUSED, 3, false>(p, maps, S, max_rows, stream);
    return launch_decode_st<HD, CLUSTER, FUSED, 2, false>(p, maps, S, max_rows, stream);
}

// merge the n_split partial results of every (token, head): one warp per row
template <int HD>
__global__ void attention_combine_kernel(const float * __restrict__ part_o, const float * __restrict__ part_lse,
                                         __nv_bfloat16 * __restrict__ out, int rows, int n_split) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float * lse = part_lse + (size_t) row * n_split;
    float mx = -INFINITY;
    for (int i = 0; i < n_split; i++) mx = fmaxf(mx, lse[i]);
    float acc[HD / 32];
#pragma unroll
    for (int i = 0; i < HD / 32; i++) acc[i] = 0.0f;
    float wsum = 0.0f;
    if (mx != -INFINITY) {
        for (int i = 0; i < n_split; i++) {
            const float w = exp2f(lse[i] - mx);      // 0 for a part that saw no key
            if (w == 0.0f) continue;
            wsum += w;
            const float * po = part_o + ((size_t) row * n_split + i) * HD;
#pragma unroll
            for (int k = 0; k < HD / 32; k++) acc[k] += w * po[lane + 32 * k];
        }
    }
    const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
#pragma unroll
    for (int k = 0; k < HD / 32; k++) out[(size_t) row * HD + lane + 32 * k] = __float2bfloat16_rn(acc[k] * inv);
}

template <int HD, int NW>
static int launch_attention(const AttnParams & p, int S, int max_rows, cudaStream_t stream) {
    constexpr int BM = 16 * NW;
    const size_t smem = (size_t) 4 * BN * HD * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<HD, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return 1000 + (int) e;
        configured = true;
    }
    dim3 grid((max_rows + BM - 1) / BM, p.nkv, S * p.n_split);
    attention_mma_kernel<HD, NW><<<grid, NW * 32, smem, stream>>>(p);
    return iian_launch_status();
}

}  // namespace iian

using namespace iian;

// Scratch needed for n_split > 1: part_o = N * nh * n_split * hd floats, part_lse = N * nh * n_split floats,
// and for the decode form (small_tiles 1) counters = S * nkv * ceil(max_q_len * nh / nkv / 16) ints that are
// zero before the first launch (the kernel leaves them zero).  small_tiles 2 is the decode form with the parts
// of a row tile merged inside a thread-block cluster: n_split 2 to 16, no scratch at all.
// Tiles of shared memory per CTA of the decode form: 2 (three CTAs per SM) or 3 (two CTAs, two tiles in flight).
// status: two ints on the device, zero before the launch, or null.  With a status buffer the decode form fetches
// its K/V tiles by TMA where it can (head size 128, pages of 8 to 64 tokens); a wait that gave up leaves {11, tile}
// there and the output is not valid.  Without one it copies with cp.async as before.
// iian_attention_decode_stages(3) gives every decode launch three stages; by default launches with split keys have two,
// and launches with unsplit keys the number that needs fewer waves of CTAs (iian_attention_unsplit_stages(2 | 3)
// fixes it for a measurement, 0 gives the choice back).
IIAN_API int iian_attention_unsplit_stages(int stages) {
    if (stages != 0 && stages != 2 && stages != 3) return IIAN_ERR_SHAPE;
    g_unsplit_stages = stages;
    return IIAN_OK;
}

IIAN_API int iian_attention_decode_stages(int stages) {
    if (stages != 2 && stages != 3) return IIAN_ERR_SHAPE;
    g_decode_stages = stages;
    return IIAN_OK;
}

IIAN_API int iian_attention_mma(
    const void * q, const void * k_cache, const void * v_cache, void * out, float * part_o, float * part_lse,
    int * counters, const int * cu_q, const int * ctx_len, const int * block_table, int max_blocks,
    int N, int S, int max_q_len, int nh, int nkv, int hd, int page_size, int num_pages,
    float scale, int window, int n_split, int small_tiles, int * status, cudaStream_t stream) {
    if (N <= 0 || S <= 0) return IIAN_OK;
    if (nkv <= 0 || nh % nkv != 0 || page_size <= 0 || n_split < 1) return IIAN_ERR_SHAPE;
    if (hd != 64 && hd != 128) return IIAN_ERR_SHAPE;
    const bool cluster = small_tiles == 2 && n_split > 1;   // decode form, parts merged inside a thread-block cluster
    if (cluster && n_split > 16) return IIAN_ERR_SHAPE;
    if (n_split > 1 && !cluster && (part_o == nullptr || part_lse == nullptr)) return IIAN_ERR_SHAPE;
    if (n_split > 1 && !cluster && small_tiles && counters == nullptr) return IIAN_ERR_SHAPE;
    if ((long long) S * n_split > 65535 || nkv > 65535) return IIAN_ERR_LIMIT;
    AttnParams p;
    p.q = (const __nv_bfloat16 *) q; p.k_cache = (const __nv_bfloat16 *) k_cache; p.v_cache = (const __nv_bfloat16 *) v_cache;
    p.out = (__nv_bfloat16 *) out; p.part_o = part_o; p.part_lse = part_lse; p.counters = counters;
    p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table; p.max_blocks = max_blocks;
    p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.n_split = n_split;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.k_cache_w = nullptr; p.v_cache_w = nullptr; p.qkv = nullptr; p.q_weight = nullptr; p.k_weight = nullptr;
    p.table = nullptr; p.slots = nullptr; p.eps = 0.0f; p.write_kv = 0;
    p.status = ((uintptr_t) k_cache & 15) || ((uintptr_t) v_cache & 15) ? nullptr : status;
    const int max_rows = max_q_len * (nh / nkv);
    int rc;
    if (cluster) rc = hd == 128 ? launch_decode<128, true>(p, S, max_rows, stream) : launch_decode<64, true>(p, S, max_rows, stream);
    else if (hd == 128) rc = small_tiles ? launch_decode<128, false>(p, S, max_rows, stream) : launch_attention<128, 4>(p, S, max_rows, stream);
    else rc = small_tiles ? launch_decode<64, false>(p, S, max_rows, stream) : launch_attention<64, 4>(p, S, max_rows, stream);
    if (rc != IIAN_OK || n_split == 1 || small_tiles) return rc;      // the decode form merges its parts itself
    const int rows = N * nh;
    const int warps = 4;
    if (hd == 128) attention_combine_kernel<128><<<(rows + warps - 1) / warps, warps * 32, 0, stream>>>(part_o, part_lse, (__nv_bfloat16 *) out, rows, n_split);
    else attention_combine_kernel<64><<<(rows + warps - 1) / warps, warps * 32, 0, stream>>>(part_o, part_lse, (__nv_bfloat16 *) out, rows, n_split);
    return iian_launch_status();
}

// Decode attention straight from the Q|K|V projection, for steps in which every sequence has exactly one
// token (token i belongs to sequence i, N == S): per-head RMSNorm (weights may be null: no norm), NEOX
// rotation over the whole head with the (cos, sin) table [N, hd / 2] (null: no rotation), the write of the
// new key and value to cache cell slots[i] (write_kv; a negative slot stores nothing), and attention over
// the cache, in one launch.  Scratch as for iian_attention_mma's decode form; cluster != 0 (n_split 2..16)
// needs none.  Up to 16 query heads per KV head.
IIAN_API int iian_attention_decode_fused(
    const void * qkv, void * k_cache, void * v_cache, void * out, float * part_o, float * part_lse, int * counters,
    const int * cu_q, const int * ctx_len, const int * block_table, int max_blocks,
    int S, int nh, int nkv, int hd, int page_size, int num_pages, float scale, int window, int n_split, int cluster,
    const float * q_weight, const float * k_weight, const float * table, const int * slots, float eps, int write_kv,
    int * status, cudaStream_t stream) {
    if (S <= 0) return IIAN_OK;
    if (nkv <= 0 || nh % nkv != 0 || nh / nkv > 16 || page_size <= 0 || n_split < 1) return IIAN_ERR_SHAPE;
    if (hd != 64 && hd != 128) return IIAN_ERR_SHAPE;
    const bool cl = cluster != 0 && n_split > 1;
    if (cl && n_split > 16) return IIAN_ERR_SHAPE;
    if (n_split > 1 && !cl && (part_o == nullptr || part_lse == nullptr || counters == nullptr)) return IIAN_ERR_SHAPE;
    if (write_kv && slots == nullptr) return IIAN_ERR_SHAPE;
    if ((long long) S * n_split > 65535 || nkv > 65535) return IIAN_ERR_LIMIT;
    if (((uintptr_t) qkv & 15) || ((uintptr_t) k_cache & 15) || ((uintptr_t) v_cache & 15) || ((uintptr_t) table & 15) ||
        ((uintptr_t) q_weight & 7) || ((uintptr_t) k_weight & 7)) return IIAN_ERR_ALIGN;
    AttnParams p;
    p.q = nullptr; p.k_cache = (const __nv_bfloat16 *) k_cache; p.v_cache = (const __nv_bfloat16 *) v_cache;
    p.out = (__nv_bfloat16 *) out; p.part_o = part_o; p.part_lse = part_lse; p.counters = counters;
    p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table; p.max_blocks = max_blocks;
    p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.n_split = n_split;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.k_cache_w = (__nv_bfloat16 *) k_cache; p.v_cache_w = (__nv_bfloat16 *) v_cache;
    p.qkv = (const __nv_bfloat16 *) qkv; p.q_weight = q_weight; p.k_weight = k_weight;
    p.table = (const float2 *) table; p.slots = slots; p.eps = eps; p.write_kv = write_kv;
    p.status = status;
    const int max_rows = nh / nkv;
    if (cl) return hd == 128 ? launch_decode<128, true, true>(p, S, max_rows, stream) : launch_decode<64, true, true>(p, S, max_rows, stream);
    return hd == 128 ? launch_decode<128, false, true>(p, S, max_rows, stream) : launch_decode<64, false, true>(p, S, max_rows, stream);
}

// ---------------------------------------------------------------------------------------------------
// Split-KV attention for callers that must not allocate.  Declared in attention_mma.h.
//
// The split path above needs scratch memory for the partial results, and the regular entry point
// expects the caller to bring it.  Some callers cannot: a program that has already handed the whole
// device to a memory pool of its own (a cudaMalloc would fail, or take memory the pool believes it
// owns), or a latency-critical loop that cannot afford cudaMalloc's device-wide synchronisation.  For
// them the scratch lives in a fixed array inside this library.
//
//  * The array has kNoAllocScratchFloats floats (8 MiB) for partial results, after a fixed region of
//    kNoAllocCounters ints for the per-row-tile arrival counters.  Every GPU on which this library is
//    loaded holds both until the process exits.
//  * A call with n_split > 1 needs N * nh * n_split * (hd + 1) floats and, in the decode form, S * nkv *
//    ceil(max_q_len * nh / nkv / 16) counters; a larger request is refused with IIAN_ERR_LIMIT and nothing
//    is launched.  The form that merges inside a thread-block cluster (small_tiles == 2) and unsplit calls
//    use nothing of the array and are not limited by it.
//    iian_attention_mma_noalloc_capacity() returns the limit in floats.
//  * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
//    device current) and remembers it per device.  Make that first call before any stream capture.
//  * No cudaMalloc, cudaFree or allocating library routine is called, on the first call or later.
//  * All calls share the one array, and it keeps what the last call left in it.  The partial results
//    need no clearing: each (row, split) cell is fully written by the CTA that owns it before the merging
//    CTA of the same call reads it.  The counters must be zero when a launch starts; they live in a
//    region of their own that nothing else is ever written to, start at zero (static storage) and are
//    put back to zero by the kernel itself.  Two calls whose kernels overlap on the GPU (different
//    streams without an ordering between them) race on the array; order them.
// ---------------------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchFloats = (size_t) 2 * 1024 * 1024;
constexpr size_t kNoAllocCounters = (size_t) 64 * 1024;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocCounters + kNoAllocScratchFloats];

namespace {
constexpr int kMaxDevices = 64;
float * g_noalloc_ptr[kMaxDevices] = {};     // device address of the array, per device; host code must not
                                             // pass g_noalloc_scratch itself to a kernel
}

IIAN_API long long iian_attention_mma_noalloc_capacity() { return (long long) kNoAllocScratchFloats; }

IIAN_API int iian_attention_mma_noalloc(
    const void * q, const void * k_cache, const void * v_cache, void * out,
    const int * cu_q, const int * ctx_len, const int * block_table, int max_blocks,
    int N, int S, int max_q_len, int nh, int nkv, int hd, int page_size, int num_pages,
    float scale, int window, int n_split, int small_tiles, cudaStream_t stream) {
    if (N <= 0 || S <= 0) return IIAN_OK;
    if (n_split < 1 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || (hd != 64 && hd != 128)) return IIAN_ERR_SHAPE;
    // which form runs decides what it needs of the array: the cluster form (small_tiles == 2, n_split 2..16)
    // merges in shared memory and needs nothing; the prefill form (small_tiles == 0) needs the partial results
    // but no counters; an unsplit call needs neither
    const bool uses_scratch = n_split > 1 && small_tiles != 2;
    const bool uses_counters = uses_scratch && small_tiles != 0;
    const unsigned long long need = (unsigned long long) N * nh * n_split * (unsigned long long) (hd + 1);
    if (uses_scratch && need > kNoAllocScratchFloats) return IIAN_ERR_LIMIT;
    const unsigned long long n_counters = (unsigned long long) S * nkv * (((unsigned long long) max_q_len * (nh / nkv) + 15) / 16);
    if (uses_counters && n_counters > kNoAllocCounters) return IIAN_ERR_LIMIT;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return 1000 + (int) e;
    if (dev < 0 || dev >= kMaxDevices) return IIAN_ERR_LIMIT;
    float * base = __atomic_load_n(&g_noalloc_ptr[dev], __ATOMIC_ACQUIRE);
    if (base == nullptr) {          // set-up, once per device, with that device current (two threads that race
        float * ptr = nullptr;      // here both look the same address up and store the same value)
        e = cudaGetSymbolAddress((void **) &ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return 1000 + (int) e;
        if (ptr == nullptr) return IIAN_ERR_NOSYMBOL;
        __atomic_store_n(&g_noalloc_ptr[dev], ptr, __ATOMIC_RELEASE);
        base = ptr;
    }
    int * counters = reinterpret_cast<int *>(base);                     // an int region of its own, zero at rest
    float * part_o = base + kNoAllocCounters;
    float * part_lse = part_o + (size_t) N * nh * n_split * hd;
    return iian_attention_mma(q, k_cache, v_cache, out, part_o, part_lse, counters, cu_q, ctx_len, block_table, max_blocks,
                              N, S, max_q_len, nh, nkv, hd, page_size, num_pages, scale, window, n_split, small_tiles,
                              nullptr, stream);
}
