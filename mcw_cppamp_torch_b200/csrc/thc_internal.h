// Shared internals of libTHC (B200): error plumbing, per-thread device context, launch helpers.
#ifndef THC_INTERNAL_H
#define THC_INTERNAL_H

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "THC.h"

namespace thc {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

[[noreturn]] void fail(const char *fmt, ...);
void record_error(const char *msg);  // thread-local message + user handler

#define THC_CHECK(cond, ...) \
  do { if (!(cond)) ::thc::fail(__VA_ARGS__); } while (0)
// Mirrors THArgCheck(condition, argNumber, msg) of TH.
#define THC_ARG(cond, argn, msg) \
  do { if (!(cond)) ::thc::fail("Invalid argument %d: %s", (argn), (msg)); } while (0)
#define THC_CUDA(expr) \
  do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) \
    ::thc::fail("CUDA error %s at %s:%d: %s", cudaGetErrorName(e__), __FILE__, __LINE__, cudaGetErrorString(e__)); } while (0)

// Every extern "C" entry point body sits between these: C++ exceptions never cross the C ABI.
#define THC_BEGIN try {
#define THC_END(...) } catch (const std::exception &e__) { ::thc::record_error(e__.what()); return __VA_ARGS__; } \
                     catch (...) { ::thc::record_error("unknown error"); return __VA_ARGS__; }

// What the tensor-core kernels get to report a pipeline stall (a bounded mbarrier wait that ran out).
namespace mm {
struct StallCtl {
  int *dev_flag;     // device memory; a kernel that finds it set on entry does no work
  int *host_flag;    // mapped pinned host memory (device alias); the host reads it after a synchronisation
  long long limit;   // SM cycles one wait may take
};
}  // namespace mm

struct Context {
  int device = -1;            // current device of this host thread, -1 = not yet initialised
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  int sm_count = 0;
  int math_mode = 0;          // 0 fp32x3, 1 simt, 2 bf16
  long launches = 0;
  // small device scratch reused by reductions and the GEMM error flag (lazy, per device)
  void *scratch = nullptr;
  size_t scratch_bytes = 0;
  float *host_pinned = nullptr;  // 64 B pinned staging for scalar results
  // stall flags of the tensor-core kernels (see mm::StallCtl)
  int *stall_host = nullptr;      // mapped pinned host word
  int *stall_host_dev = nullptr;  // its device alias
  int *stall_dev = nullptr;       // device word
  long long stall_limit = 1ll << 27;
  // workspace arena of the entry points' temporaries (see ws_alloc)
  char *ws_base = nullptr;
  size_t ws_cap = 0, ws_used = 0;
  int ws_depth = 0;
  long ws_epoch = 0;             // bumped whenever the arena is replaced by a larger one
  void *ws_retired[8] = {};      // arenas outgrown inside the running entry point, freed when it returns
  int ws_nretired = 0;
  long allocs = 0;               // stream-ordered allocations requested from the driver (storages + arena growth)
  // item counters of the persistent matrix-multiply launches (see sched_counter)
  unsigned *sched_counters = nullptr;
  int sched_next = 0;
  cudaStream_t sched_stream = nullptr;
};

Context &ctx();                   // initialises device 0 on first use; fails loudly without CUDA
cudaStream_t stream();
// Waits for the stream, then turns a stall raised by any kernel since the last check into an Error (clearing it).
// Every entry point that hands results to the host synchronises through this.
void sync_stream();
void check_stall();               // the check alone, for callers that have just synchronised themselves
mm::StallCtl stall_ctl();         // kernel parameter of the tensor-core kernels
// A zeroed device word for one persistent launch to hand out its work items from.  The words come from a block of
// 4096 that is cleared on the stream each time it has been used up (the launches that used it are ahead of the
// clearing in the same stream).
unsigned *sched_counter();
int device_if_initialised();       // -1 before the first CUDA use on this thread; never initialises
void *scratch(size_t bytes);      // grow-only device scratch of the reductions, zero-filled when (re)allocated
void *dev_alloc(size_t bytes);    // stream-ordered allocation (caching pool): storages
void dev_free(void *p);
// Temporaries of one entry-point call (operand planes, split-K partials, repacked weights ...) come from a
// per-context arena instead of the driver: ws_alloc bumps a pointer, and the WsScope the entry point opened
// gives everything back when it is left.  Work on the context's stream is ordered, so the next call may reuse
// the bytes while this call's kernels are still queued.  The arena grows (a larger one replaces it; the old one
// is freed in stream order once the entry point returns) until it fits the largest call, then no entry point
// asks the driver for memory at all.
void *ws_alloc(size_t bytes);
struct WsScope {
  size_t mark;
  long epoch;
  WsScope();
  ~WsScope();
  WsScope(const WsScope &) = delete;
  WsScope &operator=(const WsScope &) = delete;
};
inline void count_launch() { ctx().launches++; }
void check_launch(const char *what);  // cudaGetLastError -> fail

inline int ceil_div(long a, long b) { return (int)((a + b - 1) / b); }

// ---- tensor helpers shared by the math / nn files ----
long nelem(const THGPUTensor *t);
bool is_contiguous(const THGPUTensor *t);
inline float *data_ptr(const THGPUTensor *t) { return t->storage ? t->storage->data + t->storageOffset : nullptr; }
void resize_nd(THGPUTensor *t, int nd, const long *size, const long *stride /*nullable*/);
THGPUStorage *storage_new();
void storage_free(THGPUStorage *s);
void storage_resize(THGPUStorage *s, long size);
// points `self` at `storage` (retained; may be null) with the given view; null size / stride keep / derive them
void tensor_raw_set(THGPUTensor *self, THGPUStorage *storage, long offset, int nd, const long *size, const long *stride);
// throwing internals behind the C ABI of the same names
THGPUTensor *tensor_new();
void tensor_free(THGPUTensor *t);
void tensor_copy(THGPUTensor *dst, THGPUTensor *src);
THGPUTensor *tensor_new_contiguous(THGPUTensor *t);   // retains t when it already is contiguous
THGPUTensor *tensor_new_sized(int nd, const long *size);
void tensor_resize_as(THGPUTensor *r, const THGPUTensor *t);

// Scope guard: one reference to a tensor, released when the scope is left by any route, so that a THC_CHECK that
// throws between THC_BEGIN and THC_END does not leak it.
struct TensorRef {
  THGPUTensor *t;
  explicit TensorRef(THGPUTensor *t_ = nullptr) : t(t_) {}
  TensorRef(const TensorRef &) = delete;
  TensorRef &operator=(const TensorRef &) = delete;
  ~TensorRef() { if (t) tensor_free(t); }
  void reset(THGPUTensor *t_ = nullptr) { if (t) tensor_free(t); t = t_; }
  operator THGPUTensor *() const { return t; }
  THGPUTensor *operator->() const { return t; }
};

// Collapsed strided description of up to 3 operands over one index space (used by the generic
// elementwise / copy kernels).  dims are merged wherever every operand allows it.
constexpr int kMaxDims = 8;
struct Strided {
  int nd;
  long size[kMaxDims];
  long stride[3][kMaxDims];
};
// Builds the description for operands that all have nelem equal; returns false if more than
// kMaxDims dims remain after collapsing.
bool collapse(int nops, const THGPUTensor *const *ops, Strided &out);

// SGD (with momentum when v is given) over flat buffers on an explicit stream
void sgd_update_async(float *w, const float *g, float *v, long n, float lr, float momentum, cudaStream_t s);

// device-side GEMM front (col-major BLAS semantics) shared by addmm / conv / Linear
void gemm(char transa, char transb, long m, long n, long k, float alpha, const float *a, long lda,
          const float *b, long ldb, float beta, float *c, long ldc);

}  // namespace thc

#endif
