/* C declarations of the entry points of attention_mma.cu. */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Paged flash attention on tensor cores; the caller brings scratch memory for n_split > 1:
 * part_o = N * nh * n_split * hd floats, part_lse = N * nh * n_split floats, and (decode form) counters =
 * S * nkv * ceil(max_q_len * nh / nkv / 16) ints that are zero before the first launch.  status: two ints on
 * the device, zero before the launch, or null; with it the decode form (small_tiles != 0) fetches its K/V tiles
 * by TMA where it can and reports a wait that gave up there ({11, tile}: the output is not valid).  Returns 0
 * when launched. */
int iian_attention_mma(const void * q, const void * k_cache, const void * v_cache, void * out, float * part_o,
                       float * part_lse, int * counters, const int * cu_q, const int * ctx_len, const int * block_table,
                       int max_blocks, int N, int S, int max_q_len, int nh, int nkv, int hd, int page_size,
                       int num_pages, float scale, int window, int n_split, int small_tiles, int * status,
                       cudaStream_t stream);

/* The same computation for callers that cannot allocate device memory (their process has given the
 * whole GPU to its own pool, or they run where cudaMalloc's synchronisation is not acceptable).  It has
 * no counterpart in the reference engine.  The partial results and arrival counters go to a fixed array (8.25 MiB) inside
 * the library instead of caller memory: a call that needs more than
 * iian_attention_mma_noalloc_capacity() floats (N * nh * n_split * (hd + 1)) returns 4 (limit) and
 * launches nothing.  The first call on a device resolves the array's address; make it before any stream
 * capture.  Calls share the array: calls that overlap on the GPU race, so keep them ordered.  Neither
 * the first nor later calls allocate or free device memory. */
int iian_attention_mma_noalloc(const void * q, const void * k_cache, const void * v_cache, void * out,
                               const int * cu_q, const int * ctx_len, const int * block_table, int max_blocks,
                               int N, int S, int max_q_len, int nh, int nkv, int hd, int page_size, int num_pages,
                               float scale, int window, int n_split, int small_tiles, cudaStream_t stream);
long long iian_attention_mma_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
