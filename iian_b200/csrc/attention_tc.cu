// Paged causal attention for prefill portions on the fifth-generation tensor cores (head size 128, bf16).
//
// One CTA owns 256 rows of one (sequence, KV head), as two groups of 128: the rows are the (token, head) pairs
// of the query heads that share the KV head, so a K/V tile fetched once serves all of them.  Keys are walked in
// tiles of 128.  Per tile and group: S = Q K^T by tcgen05.mma into tensor memory (128 lanes x 128 columns of
// float32); the group's four softmax warps read S with tcgen05.ld -- thread i owns row i, so maxima and sums
// need no shuffles --, and write P = exp2(S * scale - max) as bf16 pairs back into the first 64 of those
// columns with tcgen05.st; O += P V is a second tcgen05.mma whose A operand is P in tensor memory (no shared
// memory traffic for P, which matters: a 128 x 128 x 16 MMA with both operands in shared memory reads 8 KB per
// 64 cycles, all the shared-memory bandwidth there is) and whose B operand is the V tile as TMA left it
// (MN-major: a key's row holds 64 values of the head).  Tensor memory: S/P and O of both groups, 512 columns.
// K and V tiles come through the block table by TMA, one box per page and half head (page_size rows x 64
// values, 128-byte swizzle), two stages each; pages past the context are asked for at an out-of-range
// coordinate, which TMA fills with zeros.
//
// Roles: warp 0 issues the TMA loads (a lane per page); warp 1 allocates tensor memory and its lane 0 issues the
// MMAs; warps 2..5 and 6..9 are the softmax of group A and B and, at the end, write O / sum.  A group's chain
// is Q K^T -> softmax -> P V -> next Q K^T (S and P share columns, and the tensor pipe runs one thread's MMAs in
// order); while one group's softmax runs, the tensor cores work for the other.  O is rescaled in tensor memory
// only when a row's maximum grew by more than 2^8 since the last rescale (the sums and P carry the stale
// maximum until then; the result is exact, P merely ranges up to 256).
//
// Formula (reference, src/iian/paged_attn.cpp:112-145): scores q.k * scale; key j visible to the token at
// position p iff j <= p and (window == 0 or p - j < window); softmax in float32; o = sum p_j v_j; a row that
// sees no key yields zeros.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records where it gave up in
// `status`, and every role falls through to the common exit, where tensor memory is freed.
#include <cuda.h>

#include "common.cuh"

namespace iian {

constexpr int AT_BM = 128, AT_BN = 128, AT_HD = 128;
constexpr int AT_ROWS = 2 * AT_BM;              // rows of a CTA: two groups of 128
constexpr int AT_THREADS = 320;
constexpr unsigned kAtSpinLimit = 4u * 1000u * 1000u;
constexpr int AT_HALF_BYTES = 128 * 128;          // 128 rows x 64 bf16: one 128-byte-swizzled half tile
constexpr int AT_TILE_BYTES = 2 * AT_HALF_BYTES;  // a 128 x 128 bf16 tile

struct TcAttnParams {
    const __nv_bfloat16 * q;        // [N, nh, 128]
    __nv_bfloat16 * out;            // [N, nh * 128]
    const int * cu_q;               // [S + 1]
    const int * ctx_len;            // [S]
    const int * block_table;        // [S, max_blocks]
    int max_blocks, nh, nkv, page_size, num_pages, window;
    float scale_log2;               // scale * log2(e)
    int * status;                   // {code, where}; zero before the launch
};

__device__ __forceinline__ unsigned at_smem(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool at_wait(unsigned bar, unsigned parity) {
    for (unsigned spin = 0; spin < kAtSpinLimit; spin++) {
        unsigned done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void at_tma_4d(unsigned dst, const CUtensorMap * map, int x, int y, int z, int w, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar) : "memory");
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void at_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void at_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (lane = row, 32-bit column = two consecutive bf16 along K)
__device__ __forceinline__ void at_mma_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc, unsigned idesc,
                                          unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void at_ld32(unsigned taddr, unsigned * r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void at_st32(unsigned taddr, const unsigned * r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void at_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void at_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// packed pairs of float32 (one instruction for two values) and the maximum of three
__device__ __forceinline__ unsigned long long at_pack2(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void at_unpack2(unsigned long long v, float & a, float & b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long at_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long at_add2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory matrix descriptor with 128-byte swizzle.  K-major operand (rows of 128 bytes along K, groups of
// 8 rows 1024 bytes apart): lbo unused, sbo = 1024.  MN-major operand (V: a key's row holds 64 values of the
// head, 8 keys make a 1024-byte swizzle atom): lbo = distance between the two halves of the head, sbo = 1024
// = the next 8 keys.  Addresses and offsets in units of 16 bytes.
__device__ __forceinline__ unsigned long long at_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long) ((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long) ((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (unsigned long long) ((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (unsigned long long) 1 << 46;
    d |= (unsigned long long) 2 << 61;
    return d;
}
// bf16 x bf16 -> f32, M x N tile; b_mn: the B operand is MN-major (else both are K-major)
__host__ __device__ constexpr unsigned at_idesc(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((unsigned) (n >> 3) << 17) | ((unsigned) (m >> 4) << 24);
}

__global__ void __launch_bounds__(AT_THREADS, 1) attention_tc_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const TcAttnParams p) {
    extern __shared__ __align__(1024) unsigned char at_smem_raw[];
    unsigned char * smem = (unsigned char *) (((uintptr_t) at_smem_raw + 1023) & ~(uintptr_t) 1023);
    unsigned char * sQ = smem;                               // [2 groups][2 halves][128 rows][128 B]
    unsigned char * sK = sQ + 2 * AT_TILE_BYTES;             // [2 stages][2 halves][128 keys][128 B]
    unsigned char * sV = sK + 2 * AT_TILE_BYTES;             // [2 stages][2 halves][128 keys][128 B]
    __shared__ __align__(8) unsigned long long k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2], q_full;
    __shared__ unsigned tmem_base_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = blockIdx.y, s = blockIdx.z;
    const int G = p.nh / p.nkv;
    const int q0 = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - q0;
    const int ctx = p.ctx_len[s];
    const int pos0 = ctx - q_len;
    const int rows_total = q_len * G;
    const int row0 = ((int) gridDim.x - 1 - (int) blockIdx.x) * AT_ROWS;    // late rows see the most keys: they start first
    if (row0 >= rows_total) return;

    // two groups of 128 rows (A, B) share every K/V tile; B may be empty, and A may need a tile less than B
    const bool has_b = row0 + AT_BM < rows_total;
    const int tok_min = row0 / G;
    const int k_hi_a = pos0 + min(rows_total - 1, row0 + AT_BM - 1) / G;
    const int k_hi = pos0 + min(rows_total - 1, row0 + AT_ROWS - 1) / G;
    const int k_lo = p.window > 0 ? max(0, pos0 + tok_min - p.window + 1) : 0;
    const int tile_lo = k_lo / AT_BN, tile_hi = k_hi / AT_BN;
    const int n_tiles = tile_hi - tile_lo + 1;
    const int n_grp[2] = {k_hi_a / AT_BN - tile_lo + 1, has_b ? n_tiles : 0};
    const int * bt = p.block_table + (size_t) s * p.max_blocks;
    int * status = p.status;

    if (threadIdx.x == 0) {
        for (int g = 0; g < 2; g++) {
            at_mbar_init(at_smem(&s_full[g]), 1);
            at_mbar_init(at_smem(&k_full[g]), 1); at_mbar_init(at_smem(&k_empty[g]), 1);
            at_mbar_init(at_smem(&v_full[g]), 1); at_mbar_init(at_smem(&v_empty[g]), 1);
            at_mbar_init(at_smem(&p_full[g]), 4); at_mbar_init(at_smem(&pv_done[g]), 1);
        }
        at_mbar_init(at_smem(&q_full), AT_THREADS / 32 - 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {          // the producer's first reads: the descriptors and the block table's first entries
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        }
        const int j0 = tile_lo * AT_BN + lane * p.page_size;
        if (lane < AT_BN / p.page_size && j0 <= k_hi) asm volatile("prefetch.global.L1 [%0];" ::"l"(bt + j0 / p.page_size));
    }
    if (warp == 1) {          // tensor memory: S of both groups (2 x 128 columns), O of both groups (2 x 128 columns)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(&tmem_base_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const unsigned tmem_base = tmem_base_s;

    if (warp > 0) {
        // Q rows into the swizzled K-major layout: row r, 16-byte chunk c of half h at h * 16 KB + r * 128 + ((c ^ (r & 7)) << 4).
        // Every warp but the producer takes part, meanwhile the producer's first K and V tiles are on their way; the
        // loads of a pass are all issued before the first is stored, so that a pass costs one trip to memory.
        constexpr int kLoaders = AT_THREADS - 32, kPass = 8;
        const int t = threadIdx.x - 32;
        for (int base = 0; base < AT_ROWS * 16; base += kLoaders * kPass) {
            uint4 buf[kPass];
#pragma unroll
            for (int u = 0; u < kPass; u++) {
                const int idx = base + u * kLoaders + t;
                const int rr = idx >> 4, c = idx & 15;
                const int R = row0 + rr;
                buf[u] = make_uint4(0u, 0u, 0u, 0u);
                if (idx < AT_ROWS * 16 && R < rows_total) {
                    const int tok = R / G, head = kvh * G + R % G;
                    buf[u] = *reinterpret_cast<const uint4 *>(p.q + ((size_t) (q0 + tok) * p.nh + head) * AT_HD + c * 8);
                }
            }
#pragma unroll
            for (int u = 0; u < kPass; u++) {
                const int idx = base + u * kLoaders + t;
                if (idx < AT_ROWS * 16) {
                    const int rr = idx >> 4, c = idx & 15;
                    const int g = rr >> 7, r = rr & 127;
                    *reinterpret_cast<uint4 *>(sQ + g * AT_TILE_BYTES + (c >> 3) * AT_HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = buf[u];
                }
            }
        }
        at_fence_async_smem();
        __syncwarp();
        if (lane == 0) at_arrive(at_smem(&q_full));
    }

    if (warp == 0) {
        // ---- producer: per step the K tile of the next key tile (lanes 0..15, a lane per page) and the V tile of this
        // one (lanes 16..31), each page as two boxes (the halves of the head); lanes 0 and 16 wait for the stage to
        // be free and post the byte counts.  Two stages each for K and V; K runs a tile ahead of V.  The block table
        // is read three steps ahead, so that a step costs no trip to memory.
        const int ps = p.page_size, pages_per_tile = AT_BN / ps;
        const int lp = lane & 15;
        const bool k_lane = lane < 16;
        auto page_of = [&](int i) -> int {
            int page = p.num_pages;                          // out of range: the box is filled with zeros
            if (i < n_tiles && lp < pages_per_tile) {
                const int j0 = (tile_lo + i) * AT_BN + lp * ps;
                if (j0 <= k_hi) {
                    const int pg = bt[j0 / ps];
                    if (pg >= 0 && pg < p.num_pages) page = pg;
                }
            }
            return page;
        };
        int pg_v = p.num_pages, pg_k = page_of(0), pg_k1 = page_of(1);
        for (int i = -1; i < n_tiles; i++) {
            const int pg_k2 = page_of(i + 3);
            const bool do_k = i + 1 < n_tiles, do_v = i >= 0;
            int ok = 1;
            if (lane == 0 && do_k) {
                const int t = i + 1;
                ok = at_wait(at_smem(&k_empty[t & 1]), ((unsigned) (t >> 1) & 1u) ^ 1u) ? 1 : 0;
                if (!ok) { status[0] = 1; status[1] = t; }
                else at_expect_tx(at_smem(&k_full[t & 1]), AT_TILE_BYTES);
            }
            if (lane == 16 && do_v) {
                ok = at_wait(at_smem(&v_empty[i & 1]), ((unsigned) (i >> 1) & 1u) ^ 1u) ? 1 : 0;
                if (!ok) { status[0] = 2; status[1] = i; }
                else at_expect_tx(at_smem(&v_full[i & 1]), AT_TILE_BYTES);
            }
            if (!__all_sync(0xffffffffu, ok)) break;
            if (lp < pages_per_tile) {
                if (k_lane && do_k) {
                    const int st = (i + 1) & 1;
                    unsigned char * base = sK + st * AT_TILE_BYTES + lp * ps * 128;
                    at_tma_4d(at_smem(base), &map_k, 0, 0, kvh, pg_k, at_smem(&k_full[st]));
                    at_tma_4d(at_smem(base + AT_HALF_BYTES), &map_k, 64, 0, kvh, pg_k, at_smem(&k_full[st]));
                } else if (!k_lane && do_v) {
                    const int st = i & 1;
                    unsigned char * base = sV + st * AT_TILE_BYTES + lp * ps * 128;
                    at_tma_4d(at_smem(base), &map_v, 0, 0, kvh, pg_v, at_smem(&v_full[st]));
                    at_tma_4d(at_smem(base + AT_HALF_BYTES), &map_v, 64, 0, kvh, pg_v, at_smem(&v_full[st]));
                }
            }
            pg_v = pg_k; pg_k = pg_k1; pg_k1 = pg_k2;
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer -----------------------------------------------------------------------------------
        constexpr unsigned idesc_qk = at_idesc(AT_BM, AT_BN, false);
        constexpr unsigned idesc_pv = at_idesc(AT_BM, AT_HD, true);
        constexpr int kHalf16 = AT_HALF_BYTES >> 4;
        // descriptors are built once; a step along K adds a constant (in units of 16 bytes) to the start address
        const unsigned long long dq[2] = {at_desc(at_smem(sQ), 16, 1024), at_desc(at_smem(sQ + AT_TILE_BYTES), 16, 1024)};
        const unsigned long long dk[2] = {at_desc(at_smem(sK), 16, 1024), at_desc(at_smem(sK + AT_TILE_BYTES), 16, 1024)};
        const unsigned long long dv[2] = {at_desc(at_smem(sV), AT_HALF_BYTES, 1024), at_desc(at_smem(sV + AT_TILE_BYTES), AT_HALF_BYTES, 1024)};
        // S = Q K^T of tile i for group g.  S and P of a group share tensor memory, so this must follow the group's
        // P V of the tile before in program order (the tensor pipe runs a thread's MMAs in order).
        auto issue_qk = [&](int g, int i) {
            const int st = i & 1;
#pragma unroll
            for (int k = 0; k < 8; k++) {             // 16 values of the head per step: 32 bytes inside the atom, halves 16 KB apart
                const unsigned long long off = (unsigned long long) ((k >> 2) * kHalf16 + (k & 3) * 2);
                at_mma(tmem_base + (unsigned) (g * 128), dq[g] + off, dk[st] + off, idesc_qk, k > 0 ? 1u : 0u);
            }
            at_commit(at_smem(&s_full[g]));
        };
        if (!at_wait(at_smem(&q_full), 0u)) { status[0] = 4; status[1] = 0; goto done; }
        if (!at_wait(at_smem(&k_full[0]), 0u)) { status[0] = 3; status[1] = 0; goto done; }
        at_fence_after();
        for (int g = 0; g < 2; g++)
            if (n_grp[g] > 0) issue_qk(g, 0);
        at_commit(at_smem(&k_empty[0]));
        for (int i = 0; i < n_tiles; i++) {
            const int st = i & 1;
            const unsigned ph = (unsigned) (i >> 1) & 1u;
            if (!at_wait(at_smem(&v_full[st]), ph)) { status[0] = 6; status[1] = i; goto done; }
            if (i + 1 < n_tiles && !at_wait(at_smem(&k_full[(i + 1) & 1]), (unsigned) ((i + 1) >> 1) & 1u)) { status[0] = 3; status[1] = i + 1; goto done; }
            for (int g = 0; g < 2; g++) {
                if (i >= n_grp[g]) continue;
                if (!at_wait(at_smem(&p_full[g]), (unsigned) i & 1u)) { status[0] = 5; status[1] = i; goto done; }
                at_fence_after();
#pragma unroll
                for (int k = 0; k < 8; k++)           // 16 keys per step: 8 columns of packed P, 16 key rows of V
                    at_mma_ts(tmem_base + 256u + (unsigned) (g * 128), tmem_base + (unsigned) (g * 128 + k * 8),
                              dv[st] + (unsigned long long) (k * 16 * 128 / 16), idesc_pv, (i > 0 || k > 0) ? 1u : 0u);
                at_commit(at_smem(&pv_done[g]));
                if (i + 1 < n_grp[g]) issue_qk(g, i + 1);
            }
            at_commit(at_smem(&v_empty[st]));
            if (i + 1 < n_tiles) at_commit(at_smem(&k_empty[(i + 1) & 1]));
        }
    } else if (warp >= 2) {
        // ---- softmax: warps 2..5 are group A, 6..9 group B; thread = row ---------------------------------------
        const int g = (warp - 2) >> 2;
        const int qd = warp & 3;
        const int r = qd * 32 + lane;
        const int R = row0 + g * AT_BM + r;
        const bool row_ok = R < rows_total;
        const int row_pos = pos0 + (row_ok ? R / G : 0);
        const unsigned lane_addr = (unsigned) (qd * 32) << 16;
        const unsigned tS = tmem_base + (unsigned) (g * 128), tO = tmem_base + 256u + (unsigned) (g * 128);
        const int n_mine = n_grp[g];
        float m_run = -INFINITY, l_run = 0.0f;
        const float sl = p.scale_log2;
        bool failed = false;
        for (int i = 0; i < n_mine; i++) {
            const unsigned ph = (unsigned) i & 1u;
            const int key0 = (tile_lo + i) * AT_BN;
            if (!at_wait(at_smem(&s_full[g]), ph)) { if (lane == 0) { status[0] = 7; status[1] = i; } failed = true; break; }
            at_fence_after();
            // the whole row of S into registers; tensor memory is then free for the next tile's Q K^T
            unsigned v[AT_BN];
#pragma unroll
            for (int c0 = 0; c0 < AT_BN; c0 += 32) at_ld32(tS + lane_addr + (unsigned) c0, v + c0);
            at_wait_ld();
            // visible keys of this row in this tile: columns [lo, hi]; most tiles lie wholly below the diagonal
            const int hi = row_ok ? min(AT_BN - 1, row_pos - key0) : -1;
            const int lo = p.window > 0 ? max(0, row_pos - p.window + 1 - key0) : 0;
            if (!__all_sync(0xffffffffu, lo <= 0 && hi >= AT_BN - 1)) {
                if (p.window > 0) {
#pragma unroll
                    for (int j = 0; j < AT_BN; j++)
                        if (j < lo || j > hi) v[j] = 0xff800000u;        // -inf
                } else {
#pragma unroll
                    for (int j = 0; j < AT_BN; j++)
                        if (j > hi) v[j] = 0xff800000u;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < AT_BN; j += 8) {      // maxima of three: half the instructions
                mx4[0] = at_max3(mx4[0], __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                mx4[1] = at_max3(mx4[1], __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                mx4[2] = at_max3(mx4[2], __uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                mx4[3] = at_max3(mx4[3], __uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the maximum the sums are taken against moves only when it grew by more than 2^8 (or was unset)
            float corr = 1.0f;
            bool moved = false;
            if (mx > m_run && (m_run == -INFINITY || (mx - m_run) * sl > 8.0f)) {
                corr = m_run == -INFINITY ? 0.0f : at_exp2((m_run - mx) * sl);
                m_run = mx;
                moved = true;
            }
            const float neg = m_run == -INFINITY ? 0.0f : m_run * sl;
            // s * scale - max for two keys per instruction (packed float32 pairs), the exponentials one by one, the
            // sums in pairs again; the pair of probabilities is rounded to bfloat16 at once, into a register whose
            // values have been used already
            const unsigned long long sl2 = at_pack2(sl, sl), neg2 = at_pack2(-neg, -neg);
            unsigned long long sum2[2] = {0ull, 0ull};
#pragma unroll
            for (int j = 0; j < AT_BN; j += 4) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const unsigned long long t = at_fma2(at_pack2(__uint_as_float(v[j + 2 * e]), __uint_as_float(v[j + 2 * e + 1])), sl2, neg2);
                    float t0, t1;
                    at_unpack2(t, t0, t1);
                    const float p0 = at_exp2(t0), p1 = at_exp2(t1);                // 2^-inf = 0 for masked keys
                    sum2[e] = at_add2(sum2[e], at_pack2(p0, p1));
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    v[(j >> 1) + e] = *reinterpret_cast<unsigned *>(&h);
                }
            }
            float s0, s1, s2, s3;
            at_unpack2(sum2[0], s0, s1);
            at_unpack2(sum2[1], s2, s3);
            l_run = l_run * corr + ((s0 + s1) + (s2 + s3));
            if (i > 0) {        // P (and O, if it has to be rescaled) are free once the product of the tile before is complete
                if (!at_wait(at_smem(&pv_done[g]), ph ^ 1u)) { if (lane == 0) { status[0] = 8; status[1] = i; } failed = true; break; }
                at_fence_after();
                if (__any_sync(0xffffffffu, moved)) {
#pragma unroll 1
                    for (int c0 = 0; c0 < AT_HD; c0 += 32) {
                        unsigned o[32];
                        at_ld32(tO + lane_addr + (unsigned) c0, o);
                        at_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
                        at_st32(tO + lane_addr + (unsigned) c0, o);
                    }
                    at_wait_st();
                }
            }
            // P as bf16 pairs into the tensor-memory columns S came from (64 of its 128)
            at_st32(tS + lane_addr, v);
            at_st32(tS + lane_addr + 32u, v + 32);
            at_wait_st();
            at_fence_before();
            __syncwarp();
            if (lane == 0) at_arrive(at_smem(&p_full[g]));
        }
        // ---- O / sum -> out ---------------------------------------------------------------------------
        if (n_mine > 0 && !failed) {
            if (at_wait(at_smem(&pv_done[g]), (unsigned) (n_mine - 1) & 1u)) {
                at_fence_after();
                const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
                __nv_bfloat16 * dst = nullptr;
                if (row_ok) {
                    const int tok = R / G, head = kvh * G + R % G;
                    dst = p.out + ((size_t) (q0 + tok) * p.nh + head) * AT_HD;
                }
                unsigned o[AT_HD];                  // the whole row at once: one wait for four loads
#pragma unroll
                for (int c0 = 0; c0 < AT_HD; c0 += 32) at_ld32(tO + lane_addr + (unsigned) c0, o + c0);
                at_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int q8 = 0; q8 < AT_HD / 8; q8++) {
                        uint4 pk;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(o[8 * q8 + 0]) * inv, __uint_as_float(o[8 * q8 + 1]) * inv);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(o[8 * q8 + 2]) * inv, __uint_as_float(o[8 * q8 + 3]) * inv);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[8 * q8 + 4]) * inv, __uint_as_float(o[8 * q8 + 5]) * inv);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(o[8 * q8 + 6]) * inv, __uint_as_float(o[8 * q8 + 7]) * inv);
                        pk.x = *reinterpret_cast<unsigned *>(&h0); pk.y = *reinterpret_cast<unsigned *>(&h1);
                        pk.z = *reinterpret_cast<unsigned *>(&h2); pk.w = *reinterpret_cast<unsigned *>(&h3);
                        *reinterpret_cast<uint4 *>(dst + 8 * q8) = pk;
                    }
                }
            } else if (lane == 0) {
                status[0] = 9; status[1] = n_mine;
            }
        }
    }
done:
    at_fence_before();
    __syncthreads();
    if (warp == 1) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

typedef CUresult (*AtEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AtEncodeFn at_encode_fn() {
    static AtEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void * p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (AtEncodeFn) p;
    }
    return fn;
}

// a cache [num_pages, nkv, page_size, 128] bf16; boxes of one page and half a head: [page_size rows, 64 values]
static int at_make_map(CUtensorMap * map, const void * base, int num_pages, int nkv, int page_size) {
    AtEncodeFn fn = at_encode_fn();
    if (fn == nullptr) return IIAN_ERR_LIMIT;
    cuuint64_t dims[4] = {(cuuint64_t) AT_HD, (cuuint64_t) page_size, (cuuint64_t) nkv, (cuuint64_t) num_pages};
    cuuint64_t strides[3] = {(cuuint64_t) AT_HD * 2, (cuuint64_t) page_size * AT_HD * 2, (cuuint64_t) nkv * page_size * AT_HD * 2};
    cuuint32_t box[4] = {64, (cuuint32_t) page_size, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? IIAN_OK : 2000 + (int) r;
}

}  // namespace iian

using namespace iian;

// Prefill attention on tcgen05: head size 128, bf16, page sizes 8, 16, 32, 64 or 128 (a page is one TMA box; 8 rows
// are one swizzle atom).  q [N, nh, 128], caches [num_pages, nkv, page_size, 128], out [N, nh * 128].  status: two
// ints on the device, zero before the launch; non-zero afterwards means a wait gave up and the output is not valid.
IIAN_API int iian_attention_tc(const void * q, const void * k_cache, const void * v_cache, void * out,
                               const int * cu_q, const int * ctx_len, const int * block_table, int max_blocks,
                               int N, int S, int max_q_len, int nh, int nkv, int hd, int page_size, int num_pages,
                               float scale, int window, int * status, cudaStream_t stream) {
    if (N <= 0 || S <= 0) return IIAN_OK;
    if (hd != AT_HD || nkv <= 0 || nh % nkv != 0) return IIAN_ERR_SHAPE;
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) return IIAN_ERR_SHAPE;
    if (status == nullptr) return IIAN_ERR_SHAPE;
    if (((uintptr_t) q & 15) || ((uintptr_t) k_cache & 15) || ((uintptr_t) v_cache & 15) || ((uintptr_t) out & 15)) return IIAN_ERR_ALIGN;
    if (S > 65535 || nkv > 65535) return IIAN_ERR_LIMIT;
    CUtensorMap mk, mv;
    int rc = at_make_map(&mk, k_cache, num_pages, nkv, page_size);
    if (rc != IIAN_OK) return rc;
    rc = at_make_map(&mv, v_cache, num_pages, nkv, page_size);
    if (rc != IIAN_OK) return rc;
    TcAttnParams p;
    p.q = (const __nv_bfloat16 *) q; p.out = (__nv_bfloat16 *) out; p.cu_q = cu_q; p.ctx_len = ctx_len; p.block_table = block_table;
    p.max_blocks = max_blocks; p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.num_pages = num_pages; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    const size_t smem = (size_t) 6 * AT_TILE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return 1000 + (int) e;
        configured = true;
    }
    const int max_rows = max_q_len * (nh / nkv);
    dim3 grid((max_rows + AT_ROWS - 1) / AT_ROWS, nkv, S);
    attention_tc_kernel<<<grid, AT_THREADS, smem, stream>>>(mk, mv, p);
    return iian_launch_status();
}
