// Shared helpers for the engine's CUDA kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IIAN_API extern "C" __attribute__((visibility("default")))

// dtype codes used across the C entry points
enum { IIAN_F32 = 0, IIAN_BF16 = 1 };

// error codes returned by entry points (0 = launched; CUDA launch errors are returned as 1000 + cudaError)
enum {
    IIAN_OK = 0,
    IIAN_ERR_DTYPE = 1,      // combination of element types not built
    IIAN_ERR_SHAPE = 2,      // a size the kernel refuses
    IIAN_ERR_ALIGN = 3,      // a pointer or stride is not aligned as required
    IIAN_ERR_LIMIT = 4,      // beyond a stated maximum
    IIAN_ERR_NOSYMBOL = 5,   // the address of a device array inside the library could not be resolved
};

static inline int iian_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? IIAN_OK : 1000 + (int) e;
}

namespace iian {

// ---- programmatic dependent launch --------------------------------------------------------------
// A decode step is a chain of short kernels; with the usual stream order each one starts only after the
// one before it has drained.  Launched with the programmatic-serialization attribute, a kernel may begin
// while its predecessor is still running: it announces that its own successor may be launched
// (pdl_launch_dependents), does what does not depend on the predecessor (index arithmetic, fetching
// weights), and calls pdl_wait() before it first reads what the predecessor wrote or writes anything
// itself.  pdl_wait() returns once the predecessor grid has completed and its writes are visible; without
// the launch attribute both calls do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace iian

// Host side: set by iian_set_pdl (every library has its own copy; the Python layer sets them all).
static int g_iian_pdl = 0;
IIAN_API void iian_set_pdl(int on) { g_iian_pdl = on ? 1 : 0; }

template <typename... KArgs, typename... Args>
static inline int iian_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_iian_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    return e == cudaSuccess ? IIAN_OK : 1000 + (int) e;
}

namespace iian {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed combination order (deterministic for a given block size).
// `scratch` must hold 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float * scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < nwarps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

// Rotation of a pair by an angle: x cos - y sin and x sin + y cos, each as one rounded product and one fused
// multiply-add, spelled out so that every kernel that rotates (the rotation kernel's forms, the fused decode
// kernels) gives the same bits whatever the compiler would have contracted.
__device__ __forceinline__ float rot_lo(float x, float y, float cs, float sn) { return __fmaf_rn(x, cs, -__fmul_rn(y, sn)); }
__device__ __forceinline__ float rot_hi(float x, float y, float cs, float sn) { return __fmaf_rn(x, sn, __fmul_rn(y, cs)); }

// 8 bf16 (16 bytes) -> 8 floats
__device__ __forceinline__ void unpack8(const uint4 & raw, float * f) {
    const __nv_bfloat162 * p = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

}  // namespace iian
