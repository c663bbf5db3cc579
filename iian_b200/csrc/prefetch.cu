// Pulls a range of global memory into L2 without using it.
//
// A decode step at small batch is a chain of short kernels, and between two weight-streaming matrix
// products (norms, rotary, attention over a short context, kernel boundaries) HBM sits idle for about
// as long as it is busy.  The engine therefore runs this kernel on a side stream inside the captured
// decode graph: while the main stream works through the small kernels, the weights of the NEXT matrix
// products are already travelling from HBM into the 126 MB L2, and the product then reads them from
// there.  It changes no result: it only touches cache lines.
#include "common.cuh"

namespace iian {

__global__ void prefetch_l2_kernel(const char * __restrict__ base, size_t bytes) {
    const size_t stride = (size_t) gridDim.x * blockDim.x * 128;
    for (size_t off = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * 128; off < bytes; off += stride)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}

}  // namespace iian

using namespace iian;

IIAN_API int iian_prefetch_l2(const void * ptr, long long bytes, cudaStream_t stream) {
    if (ptr == nullptr || bytes <= 0) return IIAN_OK;
    const long long lines = (bytes + 127) / 128;
    const int threads = 256;
    long long blocks = (lines + threads - 1) / threads;
    static int sms = 0;           // four blocks per SM are enough to keep the requests flowing
    if (sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms = n;
    }
    if (blocks > (long long) sms * 4) blocks = (long long) sms * 4;
    prefetch_l2_kernel<<<(unsigned) blocks, threads, 0, stream>>>((const char *) ptr, (size_t) bytes);
    return iian_launch_status();
}
