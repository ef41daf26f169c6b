// Serialisation of torch.GPUStorage / torch.GPUTensor: the records `torch.save`, `torch.load` and
// `nn.Module:clone()` (which writes the module into a memory file and reads it back,
// mcw_nn/Module.lua:104-114) produce for GPU objects.
//
// Record layout = what the reference's C code emits into a binary-mode THFile:
//   storage (gputorch/torch/generic/Storage.c:180-200 with the raw IO of gputorch/Storage.cpp:15-31):
//       long size; float data[size]
//   tensor header (gputorch/torch/generic/Tensor.c:1150-1199):
//       int nDimension; long size[nDimension]; long stride[nDimension]; long storageOffset + 1
// In the reference the tensor's storage follows its header through Lua's `file:writeObject`; a Lua binding of
// this library calls THGPUTensor_writeHeader / THGPUStorage_write in the same two places.  Hosts without Lua
// use THGPUTensor_write / _read, which put a `long` flag (1: a storage record follows, 0: the tensor has none)
// between the two.
//
// The reference stages the whole storage through one host allocation of its full size; here the data moves
// in chunks of at most 16 MiB through one bounce buffer.  The file is a pair of callbacks (the binding passes
// THFile_writeByteRaw / THFile_readByteRaw wrappers, a Python host passes closures over a file object).
#include "thc_internal.h"

#include <vector>

namespace thc {
namespace {

constexpr long kChunkFloats = 4l << 20;

void put(const THGPUFile *f, const void *p, long n) {
  THC_CHECK(f && f->write, "file is not writable");
  THC_CHECK(f->write(f->ctx, p, n) == n, "write error: wrote fewer than %ld bytes", n);
}
void get(const THGPUFile *f, void *p, long n) {
  THC_CHECK(f && f->read, "file is not readable");
  THC_CHECK(f->read(f->ctx, p, n) == n, "read error: fewer than %ld bytes left in the file", n);
}

void storage_write(const THGPUStorage *s, const THGPUFile *f) {
  const long size = s->size;
  put(f, &size, sizeof(long));
  std::vector<float> chunk((size_t)(size < kChunkFloats ? size : kChunkFloats));
  for (long o = 0; o < size; o += kChunkFloats) {
    const long n = size - o < kChunkFloats ? size - o : kChunkFloats;
    THC_CUDA(cudaMemcpyAsync(chunk.data(), s->data + o, sizeof(float) * n, cudaMemcpyDeviceToHost, stream()));
    sync_stream();
    put(f, chunk.data(), sizeof(float) * n);
  }
}
void storage_read(THGPUStorage *s, const THGPUFile *f) {
  long size = 0;
  get(f, &size, sizeof(long));
  THC_CHECK(size >= 0, "corrupt storage record (size %ld)", size);
  storage_resize(s, size);
  std::vector<float> chunk((size_t)(size < kChunkFloats ? size : kChunkFloats));
  for (long o = 0; o < size; o += kChunkFloats) {
    const long n = size - o < kChunkFloats ? size - o : kChunkFloats;
    get(f, chunk.data(), sizeof(float) * n);
    THC_CUDA(cudaMemcpyAsync(s->data + o, chunk.data(), sizeof(float) * n, cudaMemcpyHostToDevice, stream()));
    sync_stream();   // the bounce buffer is reused by the next chunk
  }
}
void header_write(const THGPUTensor *t, const THGPUFile *f) {
  const int nd = t->nDimension;
  put(f, &nd, sizeof(int));
  put(f, t->size, sizeof(long) * nd);
  put(f, t->stride, sizeof(long) * nd);
  const long off1 = t->storageOffset + 1;   // Lua convention, as the reference writes it
  put(f, &off1, sizeof(long));
}
// Reads a header into plain arrays; the caller applies it once the storage is known.
struct Header { int nd; long size[kMaxDims], stride[kMaxDims], offset; };
Header header_read(const THGPUFile *f) {
  Header h;
  get(f, &h.nd, sizeof(int));
  THC_CHECK(h.nd >= 0 && h.nd <= kMaxDims, "corrupt tensor record (%d dimensions)", h.nd);
  get(f, h.size, sizeof(long) * h.nd);
  get(f, h.stride, sizeof(long) * h.nd);
  get(f, &h.offset, sizeof(long));
  h.offset -= 1;
  for (int d = 0; d < h.nd; d++) THC_CHECK(h.size[d] >= 0 && h.stride[d] >= 0, "corrupt tensor record (negative extent)");
  THC_CHECK(h.offset >= 0, "corrupt tensor record (offset %ld)", h.offset);
  return h;
}
// The highest storage index a view reaches, + 1.
long header_span(const Header &h) {
  if (h.nd == 0) return 0;
  long last = h.offset;
  for (int d = 0; d < h.nd; d++) {
    if (h.size[d] == 0) return 0;
    last += (h.size[d] - 1) * h.stride[d];
  }
  return last + 1;
}

}  // namespace
}  // namespace thc

using namespace thc;

THC_API int THGPUStorage_write(const THGPUStorage *self, const THGPUFile *file) {
  THC_BEGIN
  storage_write(self, file);
  return 0;
  THC_END(1)
}
THC_API int THGPUStorage_read(THGPUStorage *self, const THGPUFile *file) {
  THC_BEGIN
  storage_read(self, file);
  return 0;
  THC_END(1)
}
THC_API int THGPUTensor_writeHeader(const THGPUTensor *self, const THGPUFile *file) {
  THC_BEGIN
  header_write(self, file);
  return 0;
  THC_END(1)
}
THC_API int THGPUTensor_readHeader(THGPUTensor *self, THGPUStorage *storage, const THGPUFile *file) {
  THC_BEGIN
  const Header h = header_read(file);
  THC_CHECK(h.nd == 0 || (storage && header_span(h) <= storage->size), "tensor record reaches beyond its storage");
  tensor_raw_set(self, h.nd ? storage : nullptr, h.nd ? h.offset : 0, h.nd, h.size, h.stride);
  return 0;
  THC_END(1)
}
THC_API int THGPUTensor_write(const THGPUTensor *self, const THGPUFile *file) {
  THC_BEGIN
  header_write(self, file);
  const long has = self->storage ? 1 : 0;
  put(file, &has, sizeof(long));
  if (has) storage_write(self->storage, file);
  return 0;
  THC_END(1)
}
THC_API int THGPUTensor_read(THGPUTensor *self, const THGPUFile *file) {
  THC_BEGIN
  const Header h = header_read(file);
  long has = 0;
  get(file, &has, sizeof(long));
  THC_CHECK(has == 0 || has == 1, "corrupt tensor record (storage flag %ld)", has);
  if (!has) {
    THC_CHECK(header_span(h) == 0, "tensor record with elements but no storage");
    tensor_raw_set(self, nullptr, 0, h.nd, h.size, h.stride);
    return 0;
  }
  THGPUStorage *st = storage_new();
  struct Release { THGPUStorage *s; ~Release() { storage_free(s); } } release{st};   // the tensor keeps its own reference
  storage_read(st, file);
  THC_CHECK(header_span(h) <= st->size, "tensor record reaches beyond its storage");
  tensor_raw_set(self, st, h.offset, h.nd, h.size, h.stride);
  return 0;
  THC_END(1)
}
