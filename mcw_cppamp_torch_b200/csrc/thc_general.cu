// Library state: per-thread device context, stream, error reporting, stream-ordered allocation.
// Replaces gputorch/lib/THC/THCGeneral.cpp:7-56 (empty init/shutdown, THError-on-failure) and the
// empty device stubs of gputorch/init.cpp:10-66 with real CUDA device management.
#include "thc_internal.h"

#include <cstring>
#include <map>
#include <mutex>

namespace thc {

namespace {
thread_local Context g_ctx;
thread_local std::string g_last_error;
thread_local bool g_has_error = false;
void (*g_handler)(const char *, void *) = nullptr;
void *g_handler_data = nullptr;

std::mutex g_pool_mutex;
std::map<int, bool> g_pool_ready;
}  // namespace

void fail(const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  throw Error(buf);
}

void record_error(const char *msg) {
  g_last_error = msg;
  g_has_error = true;
  if (g_handler) g_handler(msg, g_handler_data);
}

static void init_device(Context &c, int device) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    fail("libTHC: no CUDA device available (%s); this library has no CPU path",
         e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
  }
  THC_CHECK(device >= 0 && device < n, "libTHC: device %d out of range (have %d)", device, n);
  THC_CUDA(cudaSetDevice(device));
  if (c.owns_stream && c.stream) {
    cudaStreamSynchronize(c.stream);
    cudaStreamDestroy(c.stream);
  }
  if (c.scratch) { cudaFree(c.scratch); c.scratch = nullptr; c.scratch_bytes = 0; }
  if (c.stall_dev) { cudaFree(c.stall_dev); c.stall_dev = nullptr; }
  if (c.sched_counters) { cudaFree(c.sched_counters); c.sched_counters = nullptr; c.sched_stream = nullptr; }
  if (c.ws_base) { cudaFree(c.ws_base); c.ws_base = nullptr; c.ws_cap = c.ws_used = 0; c.ws_epoch++; }
  c.device = device;
  THC_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
  c.owns_stream = true;
  cudaDeviceProp prop;
  THC_CUDA(cudaGetDeviceProperties(&prop, device));
  c.sm_count = prop.multiProcessorCount;
  {
    // Keep freed blocks cached in the driver's pool: frees are stream-ordered and reuse is cheap.
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    if (!g_pool_ready[device]) {
      cudaMemPool_t pool;
      THC_CUDA(cudaDeviceGetDefaultMemPool(&pool, device));
      uint64_t threshold = UINT64_MAX;
      THC_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
      g_pool_ready[device] = true;
    }
  }
  if (!c.host_pinned) THC_CUDA(cudaMallocHost((void **)&c.host_pinned, 64));
  if (!c.stall_host) {
    THC_CUDA(cudaHostAlloc((void **)&c.stall_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
    *c.stall_host = 0;
  }
  THC_CUDA(cudaHostGetDevicePointer((void **)&c.stall_host_dev, c.stall_host, 0));
  THC_CUDA(cudaMalloc((void **)&c.stall_dev, sizeof(int)));
  THC_CUDA(cudaMemset(c.stall_dev, 0, sizeof(int)));
}

Context &ctx() {
  if (g_ctx.device < 0) init_device(g_ctx, 0);
  return g_ctx;
}

cudaStream_t stream() { return ctx().stream; }

mm::StallCtl stall_ctl() {
  Context &c = ctx();
  return mm::StallCtl{c.stall_dev, c.stall_host_dev, c.stall_limit};
}

unsigned *sched_counter() {
  Context &c = ctx();
  constexpr int kBlock = 4096;
  if (!c.sched_counters) {
    THC_CUDA(cudaMalloc((void **)&c.sched_counters, sizeof(unsigned) * kBlock));
    c.sched_next = kBlock;
  }
  if (c.sched_stream != c.stream) {
    // the caller moved to another stream: launches of the old one may still be reading their counters
    if (c.sched_stream) THC_CUDA(cudaDeviceSynchronize());
    c.sched_stream = c.stream;
    c.sched_next = kBlock;
  }
  if (c.sched_next == kBlock) {
    THC_CUDA(cudaMemsetAsync(c.sched_counters, 0, sizeof(unsigned) * kBlock, c.stream));
    c.sched_next = 0;
  }
  return c.sched_counters + c.sched_next++;
}

// Names of the wait codes of mm_tc.cuh (kWait*), for the error message.
static const char *wait_name(int code) {
  switch (code) {
    case 2: return "a splitter warp waiting for a TMA tile to land";
    case 3: return "a splitter warp waiting for a free lo slot";
    case 4: return "an MMA thread waiting for a drained accumulator buffer";
    case 5: return "an MMA thread waiting for a split tile";
    case 6: return "the TMA thread waiting for a free hi slot";
    case 7: return "a drain warp waiting for an accumulator";
    case 8: return "a role waiting for its next item number";
    case 9: return "the item thread waiting for the TMA thread to start the current item";
    case 10: return "the item thread waiting for a free ring slot";
    case 11: return "the stall probe";
    case 254: return "a kernel that found the stall flag already set";
    case 255: return "the peer CTA of a cluster";
    default: return "a pipeline wait";
  }
}

void check_stall() {
  Context &c = g_ctx;
  if (!c.stall_host) return;
  const int code = *(volatile int *)c.stall_host;
  if (!code) return;
  // The stream is idle (the caller has just synchronised it): clear both words so that later kernels run again.
  *(volatile int *)c.stall_host = 0;
  cudaMemset(c.stall_dev, 0, sizeof(int));
  fail("a tensor-core kernel gave up waiting on an mbarrier (pipeline stall; first report: %s, code %d); it and every "
       "kernel queued behind it on this stream left without writing results", wait_name(code), code);
}

void sync_stream() {
  THC_CUDA(cudaStreamSynchronize(stream()));
  check_stall();
}
int device_if_initialised() { return g_ctx.device; }

void *scratch(size_t bytes) {
  Context &c = ctx();
  if (bytes > c.scratch_bytes) {
    if (c.scratch) {
      THC_CUDA(cudaStreamSynchronize(c.stream));
      THC_CUDA(cudaFree(c.scratch));
    }
    size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
    THC_CUDA(cudaMalloc(&c.scratch, want));
    THC_CUDA(cudaMemsetAsync(c.scratch, 0, want, c.stream));
    c.scratch_bytes = want;
  }
  return c.scratch;
}

void *dev_alloc(size_t bytes) {
  if (bytes == 0) return nullptr;
  void *p = nullptr;
  THC_CUDA(cudaMallocAsync(&p, bytes, stream()));
  g_ctx.allocs++;
  return p;
}

void *ws_alloc(size_t bytes) {
  Context &c = ctx();
  THC_CHECK(c.ws_depth > 0, "internal: workspace request outside an entry point's scope");
  bytes = (bytes + 255) & ~(size_t)255;
  if (bytes == 0) bytes = 256;
  if (c.ws_used + bytes > c.ws_cap) {
    // Replace the arena by one that holds what this call has taken so far plus the request, with headroom.
    // Pointers handed out earlier in this call stay valid: the old arena is only freed when the call returns.
    THC_CHECK(c.ws_nretired < 8, "internal: workspace arena outgrown too often inside one call");
    size_t want = c.ws_used + bytes;
    if (want < c.ws_cap + c.ws_cap / 2) want = c.ws_cap + c.ws_cap / 2;
    want = (want + ((size_t)64 << 20) - 1) & ~(((size_t)64 << 20) - 1);
    char *nb = (char *)dev_alloc(want);
    if (c.ws_base) c.ws_retired[c.ws_nretired++] = c.ws_base;
    c.ws_base = nb; c.ws_cap = want; c.ws_used = 0; c.ws_epoch++;
  }
  void *p = c.ws_base + c.ws_used;
  c.ws_used += bytes;
  return p;
}
WsScope::WsScope() {
  Context &c = ctx();
  mark = c.ws_used; epoch = c.ws_epoch;
  c.ws_depth++;
}
WsScope::~WsScope() {
  Context &c = g_ctx;
  c.ws_used = epoch == c.ws_epoch ? mark : 0;
  if (--c.ws_depth == 0) {
    for (int i = 0; i < c.ws_nretired; i++) dev_free(c.ws_retired[i]);
    c.ws_nretired = 0;
    c.ws_used = 0;
  }
}

void dev_free(void *p) {
  if (!p) return;
  // Stream-ordered: kernels already queued that still read p finish first.
  cudaError_t e = cudaFreeAsync(p, stream());
  if (e != cudaSuccess) cudaGetLastError();
}

void check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) fail("CUDA launch of %s failed: %s", what, cudaGetErrorString(e));
  count_launch();
}

}  // namespace thc

using namespace thc;

THC_API void THGPUInit(void) { THC_BEGIN ctx(); THC_END() }

THC_API void THGPUShutdown(void) {
  THC_BEGIN
  ctx();
  sync_stream();
  THC_END()
}

THC_API int THGPUGetDeviceCount(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

THC_API void THGPUSetDevice(int device) {
  THC_BEGIN
  if (g_ctx.device == device) return;
  init_device(g_ctx, device);
  THC_END()
}

THC_API int THGPUGetDevice(void) { THC_BEGIN return ctx().device; THC_END(-1) }

THC_API void THGPUSynchronize(void) { THC_BEGIN sync_stream(); THC_END() }

THC_API void *THGPUGetStream(void) { THC_BEGIN return (void *)stream(); THC_END(nullptr) }

THC_API void THGPUSetStream(void *s) {
  THC_BEGIN
  Context &c = ctx();
  sync_stream();
  if (c.owns_stream && c.stream) cudaStreamDestroy(c.stream);
  if (s) {
    c.stream = (cudaStream_t)s;
    c.owns_stream = false;
  } else {
    THC_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    c.owns_stream = true;
  }
  THC_END()
}

THC_API const char *THGPUGetLastError(void) { return g_has_error ? g_last_error.c_str() : nullptr; }
THC_API void THGPUClearError(void) { g_has_error = false; }
THC_API void THGPUSetErrorHandler(void (*handler)(const char *, void *), void *data) {
  g_handler = handler;
  g_handler_data = data;
}

THC_API void THGPUBlas_setMathMode(int mode) {
  THC_BEGIN
  THC_CHECK(mode >= 0 && mode <= 2, "math mode must be 0 (fp32x3), 1 (simt) or 2 (bf16)");
  ctx().math_mode = mode;
  THC_END()
}
THC_API int THGPUBlas_getMathMode(void) { THC_BEGIN return ctx().math_mode; THC_END(-1) }
THC_API long THGPUKernelLaunchCount(void) { return g_ctx.launches; }
THC_API long THGPUDeviceAllocCount(void) { return g_ctx.allocs; }
