// torch.GPUStorage / torch.GPUTensor object model and copies.
//
// Semantics follow gputorch/lib/THC/THCStorage.cpp:7-198 (refcounted storage, flags),
// THCTensor.cpp (views, rawResize growing the storage only, isContiguous ignoring size-1 dims
// :510-525, newContiguous :186-195, freeCopyTo :578-584) and THCTensorCopy.cpp (contiguous D2D
// fast path :238-247, strided copy otherwise).  Storage memory is CUDA device memory from a
// stream-ordered pool; metadata lives on the host.
#include <cstdlib>
#include <cstring>
#include <vector>

#include "thc_apply.cuh"

namespace thc {

long nelem(const THGPUTensor *t) {
  if (t->nDimension == 0) return 0;
  long n = 1;
  for (int d = 0; d < t->nDimension; d++) n *= t->size[d];
  return n;
}

bool is_contiguous(const THGPUTensor *t) {
  long z = 1;
  for (int d = t->nDimension - 1; d >= 0; d--) {
    if (t->size[d] != 1) {
      if (t->stride[d] == z) z *= t->size[d];
      else return false;
    }
  }
  return true;
}

bool collapse(int nops, const THGPUTensor *const *ops, Strided &out) {
  const THGPUTensor *ref = ops[0];
  out.nd = 0;
  for (int d = 0; d < ref->nDimension; d++) {
    const long sz = ref->size[d];
    if (sz == 1) continue;
    bool merged = false;
    if (out.nd > 0) {
      merged = true;
      for (int k = 0; k < nops; k++)
        if (out.stride[k][out.nd - 1] != ops[k]->stride[d] * sz) merged = false;
      if (merged) {
        out.size[out.nd - 1] *= sz;
        for (int k = 0; k < nops; k++) out.stride[k][out.nd - 1] = ops[k]->stride[d];
      }
    }
    if (!merged) {
      if (out.nd == kMaxDims) return false;
      out.size[out.nd] = sz;
      for (int k = 0; k < nops; k++) out.stride[k][out.nd] = ops[k]->stride[d];
      out.nd++;
    }
  }
  if (out.nd == 0) {  // all dims of size 1
    out.nd = 1;
    out.size[0] = 1;
    for (int k = 0; k < nops; k++) out.stride[k][0] = 1;
  }
  return true;
}

static int owning_device_tag() { return device_if_initialised() + 1; }  // 0: no device memory yet

THGPUStorage *storage_new() {
  THGPUStorage *s = (THGPUStorage *)std::calloc(1, sizeof(THGPUStorage));
  THC_CHECK(s, "out of host memory");
  s->refcount = 1;
  s->flag = TH_STORAGE_REFCOUNTED | TH_STORAGE_RESIZABLE | TH_STORAGE_FREEMEM;
  s->allocatorContext = (void *)(intptr_t)owning_device_tag();
  return s;
}

static THGPUStorage *storage_new_with_size(long size) {
  THC_ARG(size >= 0, 2, "invalid size");
  THGPUStorage *s = storage_new();
  if (size > 0) {
    s->data = (float *)dev_alloc(sizeof(float) * size);
    s->size = size;
    s->allocatorContext = (void *)(intptr_t)owning_device_tag();
  }
  return s;
}

void storage_free(THGPUStorage *s) {
  if (!s) return;
  if ((s->flag & TH_STORAGE_REFCOUNTED) && s->refcount > 0) {
    if (--s->refcount == 0) {
      if (s->flag & TH_STORAGE_FREEMEM) dev_free(s->data);
      std::free(s);
    }
  }
}

void storage_resize(THGPUStorage *s, long size) {
  THC_ARG(size >= 0, 2, "invalid size");
  THC_CHECK(s->flag & TH_STORAGE_RESIZABLE, "Trying to resize storage that is not resizable");
  if (size == s->size) return;
  if (size == 0) {
    if (s->flag & TH_STORAGE_FREEMEM) dev_free(s->data);
    s->data = nullptr;
    s->size = 0;
    return;
  }
  float *nd = (float *)dev_alloc(sizeof(float) * size);
  if (s->data) {
    const long keep = size < s->size ? size : s->size;
    THC_CUDA(cudaMemcpyAsync(nd, s->data, sizeof(float) * keep, cudaMemcpyDeviceToDevice, stream()));
    if (s->flag & TH_STORAGE_FREEMEM) dev_free(s->data);
  }
  s->data = nd;
  s->size = size;
  s->flag |= TH_STORAGE_FREEMEM;
  s->allocatorContext = (void *)(intptr_t)owning_device_tag();
}

// ---- tensor metadata ----
THGPUTensor *tensor_new() {
  THGPUTensor *t = (THGPUTensor *)std::calloc(1, sizeof(THGPUTensor));
  THC_CHECK(t, "out of host memory");
  t->refcount = 1;
  t->flag = TH_TENSOR_REFCOUNTED;
  return t;
}

void resize_nd(THGPUTensor *self, int nDimension, const long *size, const long *stride) {
  int nd = 0;
  bool same = true;
  for (int d = 0; d < nDimension; d++) {
    if (size[d] > 0) {
      nd++;
      if (self->nDimension > d && size[d] != self->size[d]) same = false;
      if (self->nDimension > d && stride && stride[d] >= 0 && stride[d] != self->stride[d]) same = false;
    } else
      break;
  }
  nDimension = nd;
  if (nDimension != self->nDimension) same = false;
  if (same) return;
  if (nDimension > 0) {
    if (nDimension != self->nDimension) {
      self->size = (long *)std::realloc(self->size, sizeof(long) * nDimension);
      self->stride = (long *)std::realloc(self->stride, sizeof(long) * nDimension);
      self->nDimension = nDimension;
    }
    long total = 1;
    for (int d = nDimension - 1; d >= 0; d--) {
      self->size[d] = size[d];
      if (stride && stride[d] >= 0) self->stride[d] = stride[d];
      else self->stride[d] = (d == nDimension - 1) ? 1 : self->size[d + 1] * self->stride[d + 1];
      total += (self->size[d] - 1) * self->stride[d];
    }
    if (total + self->storageOffset > 0) {
      if (!self->storage) self->storage = storage_new();
      if (total + self->storageOffset > self->storage->size) storage_resize(self->storage, total + self->storageOffset);
    }
  } else
    self->nDimension = 0;
}

void tensor_raw_set(THGPUTensor *self, THGPUStorage *storage, long offset, int nd, const long *size,
                           const long *stride) {
  if (self->storage != storage) {
    if (self->storage) storage_free(self->storage);
    if (storage) {
      self->storage = storage;
      storage->refcount++;
    } else
      self->storage = nullptr;
  }
  THC_CHECK(offset >= 0, "Tensor: invalid storage offset");
  self->storageOffset = offset;
  resize_nd(self, nd, size, stride);
}

void tensor_free(THGPUTensor *self) {
  if (!self) return;
  if (self->flag & TH_TENSOR_REFCOUNTED) {
    if (--self->refcount == 0) {
      std::free(self->size);
      std::free(self->stride);
      if (self->storage) storage_free(self->storage);
      std::free(self);
    }
  }
}

static THGPUTensor *tensor_new_with(THGPUTensor *src) {
  THGPUTensor *t = tensor_new();
  tensor_raw_set(t, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  return t;
}

struct CopyOp {
  __device__ float operator()(const float *a) const { return a[0]; }
};

void tensor_copy(THGPUTensor *self, THGPUTensor *src) {
  if (self == src) return;
  const long n = nelem(self);
  THC_ARG(n == nelem(src), 2, "sizes do not match");
  if (n == 0) return;
  if (is_contiguous(self) && is_contiguous(src)) {
    THC_CUDA(cudaMemcpyAsync(data_ptr(self), data_ptr(src), sizeof(float) * n, cudaMemcpyDeviceToDevice, stream()));
    return;
  }
  bool same_shape = self->nDimension == src->nDimension;
  for (int d = 0; same_shape && d < self->nDimension; d++) same_shape = self->size[d] == src->size[d];
  if (same_shape) {
    apply<1>(self, src, nullptr, CopyOp(), "copy");
    return;
  }
  // Different shapes, equal element counts: TH copies in each side's logical order.  Stage the
  // side that is not contiguous through a contiguous buffer viewed with the other side's shape.
  if (!is_contiguous(src)) {
    THGPUTensor *tmp = tensor_new();
    resize_nd(tmp, src->nDimension, src->size, nullptr);
    apply<1>(tmp, src, nullptr, CopyOp(), "copy");
    tensor_copy(self, tmp);
    tensor_free(tmp);
  } else {
    THGPUTensor *view = tensor_new();
    tensor_raw_set(view, src->storage, src->storageOffset, self->nDimension, self->size, nullptr);
    apply<1>(self, view, nullptr, CopyOp(), "copy");
    tensor_free(view);
  }
}

THGPUTensor *tensor_new_contiguous(THGPUTensor *t) {
  if (is_contiguous(t)) {
    t->refcount++;
    return t;
  }
  THGPUTensor *c = tensor_new();
  resize_nd(c, t->nDimension, t->size, nullptr);
  tensor_copy(c, t);
  return c;
}

THGPUTensor *tensor_new_sized(int nd, const long *size) {
  THGPUTensor *t = tensor_new();
  resize_nd(t, nd, size, nullptr);
  return t;
}

void tensor_resize_as(THGPUTensor *r, const THGPUTensor *t) {
  bool same = r->nDimension == t->nDimension;
  for (int d = 0; same && d < r->nDimension; d++) same = r->size[d] == t->size[d];
  if (!same) resize_nd(r, t->nDimension, t->size, nullptr);
}

}  // namespace thc

using namespace thc;

// ---------------------------------------------------------------- storage C ABI
THC_API float *THGPUStorage_data(const THGPUStorage *self) { return self->data; }
THC_API long THGPUStorage_size(const THGPUStorage *self) { return self->size; }

THC_API void THGPUStorage_set(THGPUStorage *self, long index, float value) {
  THC_BEGIN
  THC_ARG(index >= 0 && index < self->size, 2, "index out of bounds");
  THC_CUDA(cudaMemcpyAsync(self->data + index, &value, sizeof(float), cudaMemcpyHostToDevice, stream()));
  sync_stream();
  THC_END()
}

THC_API float THGPUStorage_get(const THGPUStorage *self, long index) {
  THC_BEGIN
  THC_ARG(index >= 0 && index < self->size, 2, "index out of bounds");
  float v;
  THC_CUDA(cudaMemcpyAsync(&v, self->data + index, sizeof(float), cudaMemcpyDeviceToHost, stream()));
  sync_stream();
  return v;
  THC_END(0.f)
}

THC_API THGPUStorage *THGPUStorage_new(void) { THC_BEGIN return storage_new(); THC_END(nullptr) }
THC_API THGPUStorage *THGPUStorage_newWithSize(long size) { THC_BEGIN return storage_new_with_size(size); THC_END(nullptr) }

THC_API THGPUStorage *THGPUStorage_newWithData(float *device_data, long size) {
  THC_BEGIN
  THGPUStorage *s = storage_new();
  s->flag = TH_STORAGE_REFCOUNTED;  // borrowed memory: neither resized nor freed here
  s->data = device_data;
  s->size = size;
  return s;
  THC_END(nullptr)
}

THC_API void THGPUStorage_retain(THGPUStorage *self) {
  if (self && (self->flag & TH_STORAGE_REFCOUNTED)) ++self->refcount;
}
THC_API void THGPUStorage_free(THGPUStorage *self) { THC_BEGIN storage_free(self); THC_END() }
THC_API void THGPUStorage_resize(THGPUStorage *self, long size) { THC_BEGIN storage_resize(self, size); THC_END() }

struct FillOp {
  float v;
  __device__ float operator()(const float *) const { return v; }
};

THC_API void THGPUStorage_fill(THGPUStorage *self, float value) {
  THC_BEGIN
  if (self->size == 0) return;
  THGPUTensor view;
  long size = self->size, stride = 1;
  std::memset(&view, 0, sizeof(view));
  view.size = &size; view.stride = &stride; view.nDimension = 1; view.storage = self;
  apply<0>(&view, nullptr, nullptr, FillOp{value}, "fill");
  THC_END()
}

THC_API void THGPUStorage_rawCopy(THGPUStorage *self, float *host_src) {
  THC_BEGIN
  THC_CUDA(cudaMemcpyAsync(self->data, host_src, sizeof(float) * self->size, cudaMemcpyHostToDevice, stream()));
  sync_stream();
  THC_END()
}

THC_API void THGPUStorage_copy(THGPUStorage *self, THGPUStorage *src) {
  THC_BEGIN
  THC_ARG(self->size == src->size, 2, "size does not match");
  THC_CUDA(cudaMemcpyAsync(self->data, src->data, sizeof(float) * self->size, cudaMemcpyDeviceToDevice, stream()));
  THC_END()
}
THC_API void THGPUStorage_copyGPU(THGPUStorage *self, THGPUStorage *src) { THGPUStorage_copy(self, src); }


// ---------------------------------------------------------------- tensor C ABI
THC_API THGPUStorage *THGPUTensor_storage(const THGPUTensor *self) { return self->storage; }
THC_API long THGPUTensor_storageOffset(const THGPUTensor *self) { return self->storageOffset; }
THC_API int THGPUTensor_nDimension(const THGPUTensor *self) { return self->nDimension; }
THC_API long THGPUTensor_size(const THGPUTensor *self, int dim) {
  THC_BEGIN
  THC_ARG(dim >= 0 && dim < self->nDimension, 2, "out of range");
  return self->size[dim];
  THC_END(0)
}
THC_API long THGPUTensor_stride(const THGPUTensor *self, int dim) {
  THC_BEGIN
  THC_ARG(dim >= 0 && dim < self->nDimension, 2, "out of range");
  return self->stride[dim];
  THC_END(0)
}
THC_API float *THGPUTensor_data(const THGPUTensor *self) { return data_ptr(self); }

THC_API THGPUTensor *THGPUTensor_new(void) { THC_BEGIN return tensor_new(); THC_END(nullptr) }
THC_API THGPUTensor *THGPUTensor_newWithTensor(THGPUTensor *tensor) { THC_BEGIN return tensor_new_with(tensor); THC_END(nullptr) }

THC_API THGPUTensor *THGPUTensor_newWithStorage(THGPUStorage *storage, long offset, THLongStorage *size, THLongStorage *stride) {
  THC_BEGIN
  if (size && stride) THC_ARG(size->size == stride->size, 4, "inconsistent size");
  THGPUTensor *t = tensor_new();
  tensor_raw_set(t, storage, offset, size ? (int)size->size : (stride ? (int)stride->size : 0),
                 size ? size->data : nullptr, stride ? stride->data : nullptr);
  return t;
  THC_END(nullptr)
}
THC_API THGPUTensor *THGPUTensor_newWithStorage1d(THGPUStorage *storage, long offset, long size0, long stride0) {
  THC_BEGIN
  long size[1] = {size0}, stride[1] = {stride0};
  THGPUTensor *t = tensor_new();
  tensor_raw_set(t, storage, offset, 1, size, stride);
  return t;
  THC_END(nullptr)
}
THC_API THGPUTensor *THGPUTensor_newWithStorage2d(THGPUStorage *storage, long offset, long size0, long stride0, long size1, long stride1) {
  THC_BEGIN
  long size[2] = {size0, size1}, stride[2] = {stride0, stride1};
  THGPUTensor *t = tensor_new();
  tensor_raw_set(t, storage, offset, 2, size, stride);
  return t;
  THC_END(nullptr)
}
THC_API THGPUTensor *THGPUTensor_newWithSize(THLongStorage *size, THLongStorage *stride) {
  return THGPUTensor_newWithStorage(nullptr, 0, size, stride);
}
static THGPUTensor *new_with_size_nd(int nd, long s0, long s1, long s2, long s3) {
  long size[4] = {s0, s1, s2, s3};
  THGPUTensor *t = tensor_new();
  resize_nd(t, nd, size, nullptr);
  return t;
}
THC_API THGPUTensor *THGPUTensor_newWithSize1d(long s0) { THC_BEGIN return new_with_size_nd(1, s0, -1, -1, -1); THC_END(nullptr) }
THC_API THGPUTensor *THGPUTensor_newWithSize2d(long s0, long s1) { THC_BEGIN return new_with_size_nd(2, s0, s1, -1, -1); THC_END(nullptr) }
THC_API THGPUTensor *THGPUTensor_newWithSize3d(long s0, long s1, long s2) { THC_BEGIN return new_with_size_nd(3, s0, s1, s2, -1); THC_END(nullptr) }
THC_API THGPUTensor *THGPUTensor_newWithSize4d(long s0, long s1, long s2, long s3) { THC_BEGIN return new_with_size_nd(4, s0, s1, s2, s3); THC_END(nullptr) }

THC_API THGPUTensor *THGPUTensor_newClone(THGPUTensor *self) {
  THC_BEGIN
  THGPUTensor *t = tensor_new();
  resize_nd(t, self->nDimension, self->size, nullptr);
  tensor_copy(t, self);
  return t;
  THC_END(nullptr)
}
THC_API THGPUTensor *THGPUTensor_newContiguous(THGPUTensor *tensor) { THC_BEGIN return tensor_new_contiguous(tensor); THC_END(nullptr) }

THC_API void THGPUTensor_narrow(THGPUTensor *self, THGPUTensor *src, int dimension, long firstIndex, long size) {
  THC_BEGIN
  if (!src) src = self;
  THC_ARG(dimension >= 0 && dimension < src->nDimension, 3, "out of range");
  THC_ARG(firstIndex >= 0 && firstIndex < src->size[dimension], 4, "out of range");
  THC_ARG(size > 0 && firstIndex + size <= src->size[dimension], 5, "out of range");
  if (self != src) tensor_raw_set(self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  if (firstIndex > 0) self->storageOffset += firstIndex * self->stride[dimension];
  self->size[dimension] = size;
  THC_END()
}
THC_API void THGPUTensor_select(THGPUTensor *self, THGPUTensor *src, int dimension, long sliceIndex) {
  THC_BEGIN
  if (!src) src = self;
  THC_ARG(src->nDimension > 1, 1, "cannot select on a vector");
  THC_ARG(dimension >= 0 && dimension < src->nDimension, 3, "out of range");
  THC_ARG(sliceIndex >= 0 && sliceIndex < src->size[dimension], 4, "out of range");
  if (self != src) tensor_raw_set(self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  self->storageOffset += sliceIndex * self->stride[dimension];
  for (int d = dimension; d < self->nDimension - 1; d++) {
    self->size[d] = self->size[d + 1];
    self->stride[d] = self->stride[d + 1];
  }
  self->nDimension--;
  THC_END()
}
THC_API void THGPUTensor_transpose(THGPUTensor *self, THGPUTensor *src, int d1, int d2) {
  THC_BEGIN
  if (!src) src = self;
  THC_ARG(d1 >= 0 && d1 < src->nDimension, 1, "out of range");
  THC_ARG(d2 >= 0 && d2 < src->nDimension, 2, "out of range");
  if (self != src) tensor_raw_set(self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  if (d1 == d2) return;
  long z = self->stride[d1]; self->stride[d1] = self->stride[d2]; self->stride[d2] = z;
  z = self->size[d1]; self->size[d1] = self->size[d2]; self->size[d2] = z;
  THC_END()
}
THC_API void THGPUTensor_squeeze(THGPUTensor *self, THGPUTensor *src) {
  THC_BEGIN
  if (!src) src = self;
  if (self != src) tensor_raw_set(self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  int nd = 0;
  for (int d = 0; d < src->nDimension; d++) {
    if (src->size[d] != 1) {
      if (d != nd) { self->size[nd] = src->size[d]; self->stride[nd] = src->stride[d]; }
      nd++;
    }
  }
  if (nd == 0 && src->nDimension > 0) { self->size[0] = 1; self->stride[0] = 1; nd = 1; }
  self->nDimension = nd;
  THC_END()
}
THC_API THGPUTensor *THGPUTensor_newSelect(THGPUTensor *tensor, int dimension, long sliceIndex) {
  THGPUTensor *t = THGPUTensor_newWithTensor(tensor);
  if (t) THGPUTensor_select(t, nullptr, dimension, sliceIndex);
  return t;
}
THC_API THGPUTensor *THGPUTensor_newNarrow(THGPUTensor *tensor, int dimension, long firstIndex, long size) {
  THGPUTensor *t = THGPUTensor_newWithTensor(tensor);
  if (t) THGPUTensor_narrow(t, nullptr, dimension, firstIndex, size);
  return t;
}
THC_API THGPUTensor *THGPUTensor_newTranspose(THGPUTensor *tensor, int d1, int d2) {
  THGPUTensor *t = THGPUTensor_newWithTensor(tensor);
  if (t) THGPUTensor_transpose(t, nullptr, d1, d2);
  return t;
}

THC_API void THGPUTensor_resize(THGPUTensor *tensor, THLongStorage *size, THLongStorage *stride) {
  THC_BEGIN
  THC_ARG(size != nullptr, 2, "invalid size");
  if (stride) THC_ARG(stride->size == size->size, 3, "invalid stride");
  resize_nd(tensor, (int)size->size, size->data, stride ? stride->data : nullptr);
  THC_END()
}
THC_API void THGPUTensor_resizeAs(THGPUTensor *tensor, THGPUTensor *src) {
  THC_BEGIN
  bool same = tensor->nDimension == src->nDimension;
  for (int d = 0; same && d < tensor->nDimension; d++) same = tensor->size[d] == src->size[d];
  if (!same) resize_nd(tensor, src->nDimension, src->size, nullptr);
  THC_END()
}
THC_API void THGPUTensor_resize1d(THGPUTensor *t, long s0) { THC_BEGIN long s[1] = {s0}; resize_nd(t, 1, s, nullptr); THC_END() }
THC_API void THGPUTensor_resize2d(THGPUTensor *t, long s0, long s1) { THC_BEGIN long s[2] = {s0, s1}; resize_nd(t, 2, s, nullptr); THC_END() }
THC_API void THGPUTensor_resize3d(THGPUTensor *t, long s0, long s1, long s2) { THC_BEGIN long s[3] = {s0, s1, s2}; resize_nd(t, 3, s, nullptr); THC_END() }
THC_API void THGPUTensor_resize4d(THGPUTensor *t, long s0, long s1, long s2, long s3) { THC_BEGIN long s[4] = {s0, s1, s2, s3}; resize_nd(t, 4, s, nullptr); THC_END() }
THC_API void THGPUTensor_resize5d(THGPUTensor *t, long s0, long s1, long s2, long s3, long s4) { THC_BEGIN long s[5] = {s0, s1, s2, s3, s4}; resize_nd(t, 5, s, nullptr); THC_END() }

THC_API void THGPUTensor_set(THGPUTensor *self, THGPUTensor *src) {
  THC_BEGIN
  if (self != src) tensor_raw_set(self, src->storage, src->storageOffset, src->nDimension, src->size, src->stride);
  THC_END()
}
THC_API void THGPUTensor_setStorage(THGPUTensor *self, THGPUStorage *storage, long offset, THLongStorage *size, THLongStorage *stride) {
  THC_BEGIN
  if (size && stride) THC_ARG(size->size == stride->size, 5, "inconsistent size/stride sizes");
  tensor_raw_set(self, storage, offset, size ? (int)size->size : (stride ? (int)stride->size : 0),
                 size ? size->data : nullptr, stride ? stride->data : nullptr);
  THC_END()
}

THC_API int THGPUTensor_isContiguous(const THGPUTensor *self) { return is_contiguous(self) ? 1 : 0; }
THC_API int THGPUTensor_isSameSizeAs(const THGPUTensor *self, const THGPUTensor *src) {
  if (self->nDimension != src->nDimension) return 0;
  for (int d = 0; d < self->nDimension; d++)
    if (self->size[d] != src->size[d]) return 0;
  return 1;
}
THC_API long THGPUTensor_nElement(const THGPUTensor *self) { return nelem(self); }
THC_API long THGPUTensor_numel(THGPUTensor *t) { return nelem(t); }
THC_API void THGPUTensor_retain(THGPUTensor *self) {
  if (self->flag & TH_TENSOR_REFCOUNTED) ++self->refcount;
}
THC_API void THGPUTensor_free(THGPUTensor *self) { THC_BEGIN tensor_free(self); THC_END() }
THC_API void THGPUTensor_freeCopyTo(THGPUTensor *self, THGPUTensor *dst) {
  THC_BEGIN
  if (self != dst) tensor_copy(dst, self);
  tensor_free(self);
  THC_END()
}

THC_API void THGPUTensor_set1d(THGPUTensor *t, long x0, float value) {
  THC_BEGIN
  THC_ARG(t->nDimension == 1, 1, "tensor must have one dimension");
  THC_ARG(x0 >= 0 && x0 < t->size[0], 2, "out of range");
  THGPUStorage_set(t->storage, t->storageOffset + x0 * t->stride[0], value);
  THC_END()
}
THC_API void THGPUTensor_set2d(THGPUTensor *t, long x0, long x1, float value) {
  THC_BEGIN
  THC_ARG(t->nDimension == 2, 1, "tensor must have two dimensions");
  THC_ARG(x0 >= 0 && x0 < t->size[0] && x1 >= 0 && x1 < t->size[1], 2, "out of range");
  THGPUStorage_set(t->storage, t->storageOffset + x0 * t->stride[0] + x1 * t->stride[1], value);
  THC_END()
}
THC_API float THGPUTensor_get1d(const THGPUTensor *t, long x0) {
  THC_BEGIN
  THC_ARG(t->nDimension == 1, 1, "tensor must have one dimension");
  THC_ARG(x0 >= 0 && x0 < t->size[0], 2, "out of range");
  return THGPUStorage_get(t->storage, t->storageOffset + x0 * t->stride[0]);
  THC_END(0.f)
}
THC_API float THGPUTensor_get2d(const THGPUTensor *t, long x0, long x1) {
  THC_BEGIN
  THC_ARG(t->nDimension == 2, 1, "tensor must have two dimensions");
  THC_ARG(x0 >= 0 && x0 < t->size[0] && x1 >= 0 && x1 < t->size[1], 2, "out of range");
  return THGPUStorage_get(t->storage, t->storageOffset + x0 * t->stride[0] + x1 * t->stride[1]);
  THC_END(0.f)
}

// ---------------------------------------------------------------- copies
THC_API void THGPUTensor_copy(THGPUTensor *self, THGPUTensor *src) { THC_BEGIN tensor_copy(self, src); THC_END() }
THC_API void THGPUTensor_copyGPU(THGPUTensor *self, THGPUTensor *src) { THGPUTensor_copy(self, src); }

THC_API void THGPUTensor_fill(THGPUTensor *self, float value) {
  THC_BEGIN
  apply<0>(self, nullptr, nullptr, FillOp{value}, "fill");
  THC_END()
}
THC_API void THGPUTensor_zero(THGPUTensor *self) {
  THC_BEGIN
  if (is_contiguous(self) && nelem(self) > 0)
    THC_CUDA(cudaMemsetAsync(data_ptr(self), 0, sizeof(float) * nelem(self), stream()));
  else
    apply<0>(self, nullptr, nullptr, FillOp{0.f}, "zero");
  THC_END()
}
