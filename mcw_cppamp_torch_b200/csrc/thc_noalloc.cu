// Sum of a contiguous float array for callers that must not allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits -- inside a region being recorded
// for later replay, inside a latency-critical serving loop whose memory budget was fixed at start-up,
// or inside a host framework that owns every device byte and forbids libraries from taking more.
// The regular THGPUTensor_sumall grows a per-thread scratch block with cudaMalloc on first use and
// stages its result through pinned host memory; this entry point does neither.  Its only working
// memory is the fixed array below, which every GPU that loads this library holds (about 33 KB) until
// the process exits.
#include <mutex>

#include "thc_internal.h"

namespace {

constexpr int kChunk = 32768;        // floats folded by one block (512 threads x 64)
constexpr int kMaxBlocks = 4096;     // partial sums the scratch can hold
constexpr long kMaxElements = (long)kChunk * kMaxBlocks;  // 134,217,728 floats = 512 MiB

struct NoAllocScratch {
  double partial[kMaxBlocks];
  unsigned int ticket;               // blocks finished so far in the running call; must start at 0
  unsigned int pad[63];
};

// Device-side working memory.  In host code this name is only a stand-in for the symbol: the device
// address is obtained with cudaGetSymbolAddress (below) and handed to the kernel as a parameter.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

constexpr int kMaxDevices = 64;
void *g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

__global__ void __launch_bounds__(512) sum_noalloc_kernel(const float *__restrict__ x, long n, NoAllocScratch *s,
                                                          float *__restrict__ result) {
  __shared__ double warp_sums[16];
  __shared__ bool is_last;
  const long begin = (long)blockIdx.x * kChunk;
  long end = begin + kChunk;
  if (end > n) end = n;
  double acc = 0.0;
  for (long i = begin + threadIdx.x; i < end; i += blockDim.x) acc += (double)x[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double b = 0.0;
    for (int w = 0; w < 16; w++) b += warp_sums[w];
    s->partial[blockIdx.x] = b;
    __threadfence();
    is_last = atomicAdd(&s->ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (is_last) {  // the last block to finish folds the partials in index order: deterministic, no waiting
    __threadfence();
    double v = 0.0;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) v += ((volatile double *)s->partial)[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      double t = 0.0;
      for (int w = 0; w < 16; w++) t += warp_sums[w];
      result[0] = (float)t;
    }
  }
}

}  // namespace

// Sums `n` contiguous floats at DEVICE pointer `device_x` into `device_result[0]` (also a DEVICE
// pointer), asynchronously on `cuda_stream` (a cudaStream_t; NULL means the legacy default stream).
// The value is the float cast of a double-precision sum, the same as THGPUTensor_sumall returns.
//
//  * Allocates nothing: no cudaMalloc / cudaFree / pool or host allocation on the success path.
//  * n must be in [1, 134217728]; anything else is refused with an error, nothing is launched.
//  * The first call on each device looks up the address of the library's fixed scratch array (with
//    that device current).  Make that first call before starting any stream capture.
//  * All calls on a device share that one scratch array, which keeps the previous call's contents;
//    the progress counter in it is cleared on the stream at the start of every call.  Two calls that
//    overlap on the GPU (different streams, or different host threads without ordering) race on it:
//    serialise them.
// Returns 0 on success, 1 after recording an error (see THGPUGetLastError).
THC_API int THGPUTensor_sumall_noalloc(const float *device_x, long n, float *device_result, void *cuda_stream) {
  THC_BEGIN
  THC_CHECK(device_x != nullptr && device_result != nullptr, "sumall_noalloc: null device pointer");
  THC_CHECK(n >= 1, "sumall_noalloc: n must be at least 1 (got %ld)", n);
  THC_CHECK(n <= kMaxElements,
            "sumall_noalloc: n = %ld exceeds the fixed scratch capacity of %ld elements; use THGPUTensor_sumall",
            n, kMaxElements);
  int dev = -1;
  THC_CUDA(cudaGetDevice(&dev));
  THC_CHECK(dev >= 0 && dev < kMaxDevices, "sumall_noalloc: device index %d not supported", dev);
  void *scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
      void *p = nullptr;
      THC_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));  // device address of the array on `dev`
      g_scratch_addr[dev] = p;
    }
    scratch = g_scratch_addr[dev];
  }
  NoAllocScratch *s = static_cast<NoAllocScratch *>(scratch);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  THC_CUDA(cudaMemsetAsync(&s->ticket, 0, sizeof(unsigned int), stream));
  const int blocks = (int)((n + kChunk - 1) / kChunk);
  sum_noalloc_kernel<<<blocks, 512, 0, stream>>>(device_x, n, s, device_result);
  cudaError_t e = cudaGetLastError();
  THC_CHECK(e == cudaSuccess, "sumall_noalloc: launch failed: %s", cudaGetErrorString(e));
  return 0;
  THC_END(1)
}
