// Copies between torch.GPUTensor / torch.GPUStorage (FP32 on the device) and the host tensor and storage types
// of TH: Byte, Char, Short, Int, Long, Float, Double, in both directions.
//
// The reference converts on the host: every non-Float copy goes through a temporary FloatTensor / FloatStorage
// of the full size (gputorch/lib/THC/THCTensorCopy.cpp:39-58, :83-102; THCStorageCopy.cpp:12-28, :37-53) and
// every transfer blocks.  Here the host data crosses the bus in its own type (a Byte image costs one byte per
// element, a Double tensor is not narrowed by a host loop first) and the conversion is a device kernel that
// reads the staged elements and writes the FP32 destination, or the reverse.  Values follow the C casts TH
// performs (`(float)x` to the device; `(type)x`, i.e. truncation toward zero, back to the host; the narrow
// integer types take the low bits of the `int` conversion, which is what the host's cast instruction does).
//
// A non-contiguous host tensor is gathered / scattered on the host in logical order; a non-contiguous device
// tensor goes through a contiguous device temporary and the strided copy kernel.
#include "thc_internal.h"

#include <type_traits>
#include <vector>

namespace thc {
namespace {

// Every TH<Type>Storage / TH<Type>Tensor has this layout (mcw_torch7_core/lib/TH/generic/THStorage.h:22-30,
// generic/THTensor.h); only the element type differs.
template <class T> struct HostStorage { T *data; long size; int refcount; char flag; void *allocator; void *allocatorContext; };
template <class T> struct HostTensor {
  long *size; long *stride; int nDimension; HostStorage<T> *storage; long storageOffset; int refcount; char flag;
};

template <class T> long host_nelem(const HostTensor<T> *t) {
  if (t->nDimension == 0) return 0;
  long n = 1;
  for (int d = 0; d < t->nDimension; d++) n *= t->size[d];
  return n;
}
template <class T> bool host_contiguous(const HostTensor<T> *t) {
  long z = 1;
  for (int d = t->nDimension - 1; d >= 0; d--) {
    if (t->size[d] != 1) {
      if (t->stride[d] == z) z *= t->size[d];
      else return false;
    }
  }
  return true;
}
// Walks a host tensor in logical (row-major) order into / out of a dense buffer.
template <class T> void host_walk(const HostTensor<T> *t, T *dense, bool to_dense) {
  const int nd = t->nDimension;
  const long n = host_nelem(t);
  std::vector<long> idx(nd, 0);
  T *base = t->storage->data + t->storageOffset;
  for (long i = 0; i < n; i++) {
    long off = 0;
    for (int d = 0; d < nd; d++) off += idx[d] * t->stride[d];
    if (to_dense) dense[i] = base[off];
    else base[off] = dense[i];
    for (int d = nd - 1; d >= 0; d--) {
      if (++idx[d] < t->size[d]) break;
      idx[d] = 0;
    }
  }
}

template <class T> __device__ __forceinline__ T from_float(float x) { return (T)(int)x; }   // narrow integers: low bits of the int
template <> __device__ __forceinline__ int from_float<int>(float x) { return (int)x; }
template <> __device__ __forceinline__ long from_float<long>(float x) { return (long)x; }
template <> __device__ __forceinline__ double from_float<double>(float x) { return (double)x; }
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }

// Four consecutive elements per thread and step: the FP32 side moves 16 bytes per access.
template <class T>
__global__ void __launch_bounds__(256) widen_kernel(const T *__restrict__ src, float *__restrict__ dst, long n) {
  const long nthreads = (long)gridDim.x * blockDim.x;
  const long n4 = n / 4;
  const bool vec = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
  for (long q = (long)blockIdx.x * blockDim.x + threadIdx.x; q < n4; q += nthreads) {
    const T a = src[4 * q], b = src[4 * q + 1], c = src[4 * q + 2], d = src[4 * q + 3];
    if (vec) reinterpret_cast<float4 *>(dst)[q] = make_float4((float)a, (float)b, (float)c, (float)d);
    else { dst[4 * q] = (float)a; dst[4 * q + 1] = (float)b; dst[4 * q + 2] = (float)c; dst[4 * q + 3] = (float)d; }
  }
  for (long i = n4 * 4 + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nthreads) dst[i] = (float)src[i];
}
template <class T>
__global__ void __launch_bounds__(256) narrow_kernel(const float *__restrict__ src, T *__restrict__ dst, long n) {
  const long nthreads = (long)gridDim.x * blockDim.x;
  const long n4 = n / 4;
  const bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  for (long q = (long)blockIdx.x * blockDim.x + threadIdx.x; q < n4; q += nthreads) {
    float4 v;
    if (vec) v = reinterpret_cast<const float4 *>(src)[q];
    else v = make_float4(src[4 * q], src[4 * q + 1], src[4 * q + 2], src[4 * q + 3]);
    dst[4 * q] = from_float<T>(v.x); dst[4 * q + 1] = from_float<T>(v.y);
    dst[4 * q + 2] = from_float<T>(v.z); dst[4 * q + 3] = from_float<T>(v.w);
  }
  for (long i = n4 * 4 + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nthreads) dst[i] = from_float<T>(src[i]);
}
int convert_blocks(long n) {
  long b = (n / 4 + 255) / 256;
  const long cap = (long)ctx().sm_count * 8;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

// n host elements of type T at `hsrc` -> n floats at the device pointer `dst`
template <class T> void upload(float *dst, const T *hsrc, long n) {
  if constexpr (std::is_same<T, float>::value) {
    THC_CUDA(cudaMemcpyAsync(dst, hsrc, sizeof(float) * n, cudaMemcpyHostToDevice, stream()));
    return;
  }
  else {
  T *stage = (T *)ws_alloc(sizeof(T) * n);
  THC_CUDA(cudaMemcpyAsync(stage, hsrc, sizeof(T) * n, cudaMemcpyHostToDevice, stream()));
  widen_kernel<T><<<convert_blocks(n), 256, 0, stream()>>>(stage, dst, n);
  check_launch("widen");
  }
}
// n floats at the device pointer `src` -> n host elements of type T at `hdst`
template <class T> void download(T *hdst, const float *src, long n) {
  if constexpr (std::is_same<T, float>::value) {
    THC_CUDA(cudaMemcpyAsync(hdst, src, sizeof(float) * n, cudaMemcpyDeviceToHost, stream()));
    return;
  }
  else {
  T *stage = (T *)ws_alloc(sizeof(T) * n);
  narrow_kernel<T><<<convert_blocks(n), 256, 0, stream()>>>(src, stage, n);
  check_launch("narrow");
  THC_CUDA(cudaMemcpyAsync(hdst, stage, sizeof(T) * n, cudaMemcpyDeviceToHost, stream()));
  }
}

template <class T> void tensor_from_host(THGPUTensor *self, const void *src_) {
  const HostTensor<T> *src = static_cast<const HostTensor<T> *>(src_);
  const long n = nelem(self);
  THC_ARG(n == host_nelem(src), 2, "sizes do not match");
  if (n == 0) return;
  WsScope ws_scope;
  std::vector<T> dense;
  const T *hsrc;
  if (host_contiguous(src)) hsrc = src->storage->data + src->storageOffset;
  else { dense.resize(n); host_walk(src, dense.data(), true); hsrc = dense.data(); }
  if (is_contiguous(self)) {
    upload<T>(data_ptr(self), hsrc, n);
    sync_stream();   // the host buffer may be pageable or freed by the caller right away
  } else {
    TensorRef tmp(tensor_new_sized(self->nDimension, self->size));
    upload<T>(data_ptr(tmp), hsrc, n);
    tensor_copy(self, tmp);
    sync_stream();
  }
}
template <class T> void tensor_to_host(void *self_, THGPUTensor *src) {
  HostTensor<T> *self = static_cast<HostTensor<T> *>(self_);
  const long n = nelem(src);
  THC_ARG(n == host_nelem(self), 2, "sizes do not match");
  if (n == 0) return;
  WsScope ws_scope;
  TensorRef c(tensor_new_contiguous(src));
  if (host_contiguous(self)) {
    download<T>(self->storage->data + self->storageOffset, data_ptr(c), n);
    sync_stream();
  } else {
    std::vector<T> dense(n);
    download<T>(dense.data(), data_ptr(c), n);
    sync_stream();
    host_walk(self, dense.data(), false);
  }
}
template <class T> void storage_from_host(THGPUStorage *self, const void *src_) {
  const HostStorage<T> *src = static_cast<const HostStorage<T> *>(src_);
  THC_ARG(self->size == src->size, 2, "size does not match");
  if (self->size == 0) return;
  WsScope ws_scope;
  upload<T>(self->data, src->data, self->size);
  sync_stream();
}
template <class T> void storage_to_host(void *self_, THGPUStorage *src) {
  HostStorage<T> *self = static_cast<HostStorage<T> *>(self_);
  THC_ARG(self->size == src->size, 2, "size does not match");
  if (self->size == 0) return;
  WsScope ws_scope;
  download<T>(self->data, src->data, self->size);
  sync_stream();
}

}  // namespace
}  // namespace thc

using namespace thc;

#define THC_IMPLEMENT_HOST_COPIES(NAME, T)                                                                        \
  THC_API void THGPUTensor_copy##NAME(THGPUTensor *self, TH##NAME##Tensor *src) {                                \
    THC_BEGIN tensor_from_host<T>(self, src); THC_END()                                                           \
  }                                                                                                               \
  THC_API void TH##NAME##Tensor_copyGPU(TH##NAME##Tensor *self, THGPUTensor *src) {                              \
    THC_BEGIN tensor_to_host<T>(self, src); THC_END()                                                             \
  }                                                                                                               \
  THC_API void THGPUStorage_copy##NAME(THGPUStorage *self, TH##NAME##Storage *src) {                             \
    THC_BEGIN storage_from_host<T>(self, src); THC_END()                                                          \
  }                                                                                                               \
  THC_API void TH##NAME##Storage_copyGPU(TH##NAME##Storage *self, THGPUStorage *src) {                           \
    THC_BEGIN storage_to_host<T>(self, src); THC_END()                                                            \
  }

THC_IMPLEMENT_HOST_COPIES(Byte, unsigned char)
THC_IMPLEMENT_HOST_COPIES(Char, char)
THC_IMPLEMENT_HOST_COPIES(Short, short)
THC_IMPLEMENT_HOST_COPIES(Int, int)
THC_IMPLEMENT_HOST_COPIES(Long, long)
THC_IMPLEMENT_HOST_COPIES(Float, float)
THC_IMPLEMENT_HOST_COPIES(Double, double)
