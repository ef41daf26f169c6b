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
};

Context &ctx();                   // initialises device 0 on first use; fails loudly without CUDA
cudaStream_t stream();
int device_if_initialised();       // -1 before the first CUDA use on this thread; never initialises
void *scratch(size_t bytes);      // grow-only device scratch of the reductions, zero-filled when (re)allocated
void *dev_alloc(size_t bytes);    // stream-ordered allocation (caching pool)
void dev_free(void *p);
inline void count_launch() { ctx().launches++; }
void check_launch(const char *what);  // cudaGetLastError -> fail

inline int ceil_div(long a, long b) { return (int)((a + b - 1) / b); }

// ---- tensor helpers shared by the math / nn files ----
long nelem(const THGPUTensor *t);
bool is_contiguous(const THGPUTensor *t);
inline float *data_ptr(const THGPUTensor *t) { return t->storage ? t->storage->data + t->storageOffset : nullptr; }
void resize_nd(THGPUTensor *t, int nd, const long *size, const long *stride /*nullable*/);
// throwing internals behind the C ABI of the same names
THGPUTensor *tensor_new();
void tensor_free(THGPUTensor *t);
void tensor_copy(THGPUTensor *dst, THGPUTensor *src);
THGPUTensor *tensor_new_contiguous(THGPUTensor *t);   // retains t when it already is contiguous
THGPUTensor *tensor_new_sized(int nd, const long *size);
void tensor_resize_as(THGPUTensor *r, const THGPUTensor *t);

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

// device-side GEMM front (col-major BLAS semantics) shared by addmm / conv / Linear
void gemm(char transa, char transb, long m, long n, long k, float alpha, const float *a, long lda,
          const float *b, long ldb, float beta, float *c, long ldc);

}  // namespace thc

#endif
