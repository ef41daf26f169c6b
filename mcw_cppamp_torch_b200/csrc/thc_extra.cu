// The rest of the torch.GPUTensor math surface: zeros / ones / reshape, prodall / prod(dim), renorm and the
// index operations.
//   reference GPU bodies  gputorch/lib/THC/THCTensorMath.cpp: zeros :44-48, ones :50-54, reshape :56-60,
//                         prodall :316-322, prod :607-610, renorm :1195-1222, indexCopy :1331-1359,
//                         indexFill :1361-1381, indexSelect :1434-1465
//   values follow the CPU  mcw_torch7_core/lib/TH/generic/THTensorMath.c: indexSelect :69-108, indexCopy :110-147,
//                         indexFill :149-172, prodall :219-224, prod :693-711, renorm :1447-1496
// Products accumulate in double (TH's accreal) and are folded in a fixed order; index vectors are host
// LongTensors of 1-based positions, checked against the indexed dimension on the host before anything is
// launched (the reference kernels index out of bounds instead).
#include "thc_internal.h"

#include <vector>

namespace thc {
namespace {

// ---- products ------------------------------------------------------------------------------------
constexpr int kProdBlocks = 512;
__global__ void __launch_bounds__(256) prod_partial_kernel(const float *__restrict__ x, long n, double *__restrict__ partial) {
  __shared__ double sm[8];
  double acc = 1.0;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) acc *= (double)x[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc *= __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++) acc *= sm[w];
    partial[blockIdx.x] = acc;
  }
}
__global__ void prod_finish_kernel(const double *__restrict__ partial, int n, double *result) {
  double acc = 1.0;
  for (int i = 0; i < n; i++) acc *= partial[i];
  *result = acc;
}
// src viewed as [outer][R][inner] (contiguous): out[o][i] = prod_r src[o][r][i].  inner > 1: one thread per output,
// neighbouring threads read neighbouring addresses.
__global__ void __launch_bounds__(256) prod_dim_kernel(const float *__restrict__ src, long outer, long R, long inner,
                                                       float *__restrict__ out) {
  const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= outer * inner) return;
  const long o = t / inner, i = t - o * inner;
  const float *p = src + o * R * inner + i;
  double acc = 1.0;
  for (long r = 0; r < R; r++) acc *= (double)p[r * inner];
  out[t] = (float)acc;
}
// inner == 1: one warp per row, lanes stride the row, partial products folded in lane order.
__global__ void __launch_bounds__(256) prod_rows_kernel(const float *__restrict__ src, long rows, long R, float *__restrict__ out) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const float *p = src + row * R;
  double acc = 1.0;
  for (long r = lane; r < R; r += 32) acc *= (double)p[r];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc *= __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[row] = (float)acc;
}

// ---- renorm: one block per row of a contiguous [rows][size] matrix, in place -----------------------
__global__ void __launch_bounds__(256) renorm_rows_kernel(float *__restrict__ data, long size, float value, float maxnorm) {
  __shared__ double sm[8];
  __shared__ float factor;
  float *row = data + (long)blockIdx.x * size;
  double acc = 0.0;
  for (long i = threadIdx.x; i < size; i += blockDim.x) {
    const double a = fabs((double)row[i]);
    acc += value == 1.f ? a : (value == 2.f ? a * a : pow(a, (double)value));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++) acc += sm[w];
    const float norm = (float)pow(acc, 1.0 / (double)value);
    // the CPU computes maxnorm / (norm + 1e-7) in double and stores it in a float (THTensorMath.c:1479-1482)
    factor = norm > maxnorm ? (float)((double)maxnorm / ((double)norm + 1e-7)) : 1.f;
  }
  __syncthreads();
  const float f = factor;
  if (f != 1.f)
    for (long i = threadIdx.x; i < size; i += blockDim.x) row[i] = row[i] * f;
}

// ---- index operations over contiguous [outer][D][inner] / [outer][nidx][inner] blocks ---------------
// MODE 0 select: dst[o][k][i] = src[o][idx[k]][i];  1 copy: dst[o][idx[k]][i] = src[o][k][i];  2 fill: dst[o][idx[k]][i] = val
template <int MODE>
__global__ void __launch_bounds__(256) index_kernel(float *__restrict__ dst, const float *__restrict__ src,
                                                    const long *__restrict__ idx, long outer, long D, long nidx, long inner,
                                                    float val) {
  const long total = outer * nidx * inner;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long)gridDim.x * blockDim.x) {
    const long i = t % inner, q = t / inner, k = q % nidx, o = q / nidx;
    const long at = (o * D + (idx[k] - 1)) * inner + i;
    if (MODE == 0) dst[t] = src[at];
    else if (MODE == 1) dst[at] = src[t];
    else dst[at] = val;
  }
}

struct Block3 { long outer, D, inner; };
Block3 split_at(const THGPUTensor *t, int dim) {
  Block3 b{1, t->size[dim], 1};
  for (int d = 0; d < dim; d++) b.outer *= t->size[d];
  for (int d = dim + 1; d < t->nDimension; d++) b.inner *= t->size[d];
  return b;
}
// Host index vector -> device, after checking every entry against [1, D].
long *upload_indices(const THLongTensor *index, long D, long &n) {
  THC_ARG(index && index->nDimension == 1, 3, "expecting vector of indices");
  n = index->size[0];
  THC_ARG(n > 0, 3, "empty index vector");
  std::vector<long> host((size_t)n);
  const long *base = index->storage->data + index->storageOffset;
  for (long k = 0; k < n; k++) {
    host[k] = base[k * index->stride[0]];
    THC_ARG(host[k] >= 1 && host[k] <= D, 3, "index out of range");
  }
  long *dev = (long *)ws_alloc(sizeof(long) * n);
  THC_CUDA(cudaMemcpyAsync(dev, host.data(), sizeof(long) * n, cudaMemcpyHostToDevice, stream()));
  sync_stream();   // `host` goes out of scope with this function
  return dev;
}
int grid_for(long total) {
  long b = (total + 255) / 256;
  const long cap = (long)ctx().sm_count * 8;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

}  // namespace
}  // namespace thc

using namespace thc;

THC_API void THGPUTensor_zeros(THGPUTensor *r_, THLongStorage *size) {
  THC_BEGIN
  THC_ARG(size && size->size > 0, 2, "size expected");
  resize_nd(r_, (int)size->size, size->data, nullptr);
  THGPUTensor_zero(r_);
  THC_END()
}
THC_API void THGPUTensor_ones(THGPUTensor *r_, THLongStorage *size) {
  THC_BEGIN
  THC_ARG(size && size->size > 0, 2, "size expected");
  resize_nd(r_, (int)size->size, size->data, nullptr);
  THGPUTensor_fill(r_, 1.f);
  THC_END()
}
THC_API void THGPUTensor_reshape(THGPUTensor *r_, THGPUTensor *t, THLongStorage *size) {
  THC_BEGIN
  THC_ARG(size && size->size > 0, 3, "size expected");
  long n = 1;
  for (long d = 0; d < size->size; d++) n *= size->data[d];
  THC_ARG(n == nelem(t), 3, "sizes do not match");
  if (r_ == t) {   // reshaping in place: the elements already lie in logical order once made contiguous
    TensorRef c(tensor_new_contiguous(t));
    TensorRef tmp(tensor_new_sized((int)size->size, size->data));
    tensor_copy(tmp, c);
    resize_nd(r_, (int)size->size, size->data, nullptr);
    tensor_copy(r_, tmp);
    return;
  }
  resize_nd(r_, (int)size->size, size->data, nullptr);
  tensor_copy(r_, t);
  THC_END()
}

THC_API float THGPUTensor_prodall(THGPUTensor *self) {
  THC_BEGIN
  const long n = nelem(self);
  THC_ARG(n > 0, 1, "empty tensor");
  WsScope ws_scope;
  TensorRef c(tensor_new_contiguous(self));
  double *partial = (double *)ws_alloc(sizeof(double) * (kProdBlocks + 1));
  int blocks = (int)((n + 255) / 256);
  if (blocks > kProdBlocks) blocks = kProdBlocks;
  prod_partial_kernel<<<blocks, 256, 0, stream()>>>(data_ptr(c), n, partial);
  check_launch("prod_partial");
  prod_finish_kernel<<<1, 1, 0, stream()>>>(partial, blocks, partial + kProdBlocks);
  check_launch("prod_finish");
  double *host = (double *)ctx().host_pinned;
  THC_CUDA(cudaMemcpyAsync(host, partial + kProdBlocks, sizeof(double), cudaMemcpyDeviceToHost, stream()));
  sync_stream();
  return (float)*host;
  THC_END(0.f)
}

THC_API void THGPUTensor_prod(THGPUTensor *self, THGPUTensor *src, long dimension) {
  THC_BEGIN
  THC_ARG(dimension >= 0 && dimension < src->nDimension, 3, "dimension out of range");
  TensorRef c(tensor_new_contiguous(src));
  const Block3 b = split_at(c, (int)dimension);
  long osize[kMaxDims * 4];
  THC_CHECK(src->nDimension <= kMaxDims * 4, "too many dimensions");
  for (int d = 0; d < src->nDimension; d++) osize[d] = src->size[d];
  osize[dimension] = 1;
  const int nd = src->nDimension;
  TensorRef out(tensor_new_sized(nd, osize));   // src may alias self: compute aside, then hand over
  if (b.outer * b.inner > 0) {
    if (b.inner == 1) {
      prod_rows_kernel<<<(unsigned)((b.outer + 7) / 8), 256, 0, stream()>>>(data_ptr(c), b.outer, b.D, data_ptr(out));
      check_launch("prod_rows");
    } else {
      prod_dim_kernel<<<(unsigned)((b.outer * b.inner + 255) / 256), 256, 0, stream()>>>(data_ptr(c), b.outer, b.D, b.inner,
                                                                                         data_ptr(out));
      check_launch("prod_dim");
    }
  }
  resize_nd(self, nd, osize, nullptr);
  tensor_copy(self, out);
  THC_END()
}

THC_API void THGPUTensor_renorm(THGPUTensor *self, THGPUTensor *src, float value, long dimension, float maxnorm) {
  THC_BEGIN
  THC_ARG(dimension >= 0 && dimension < src->nDimension, 3, "invalid dimension");
  THC_ARG(value > 0, 2, "non-positive-norm not supported");
  THC_ARG(src->nDimension > 1, 1, "need at least 2 dimensions");
  // rows = slices along `dimension`: a contiguous copy of src with that dimension first
  TensorRef srct(THGPUTensor_newTranspose(src, (int)dimension, 0));
  THC_CHECK(srct.t != nullptr, "could not transpose");
  TensorRef data(tensor_new_sized(srct->nDimension, srct->size));
  tensor_copy(data, srct);
  const long rows = data->size[0], size = rows ? nelem(data) / rows : 0;
  if (rows > 0 && size > 0) {
    renorm_rows_kernel<<<(unsigned)rows, 256, 0, stream()>>>(data_ptr(data), size, value, maxnorm);
    check_launch("renorm_rows");
  }
  TensorRef back(THGPUTensor_newTranspose(data, (int)dimension, 0));
  THC_CHECK(back.t != nullptr, "could not transpose");
  tensor_resize_as(self, back);
  tensor_copy(self, back);
  THC_END()
}

THC_API void THGPUTensor_indexSelect(THGPUTensor *res_, THGPUTensor *src, int dim, THLongTensor *indices) {
  THC_BEGIN
  THC_ARG(src->nDimension > 0, 2, "Source tensor is empty");
  THC_ARG(dim >= 0 && dim < src->nDimension, 4, "Indexing dim is out of bounds");
  WsScope ws_scope;
  long nidx;
  const long *idx = upload_indices(indices, src->size[dim], nidx);
  TensorRef c(tensor_new_contiguous(src));
  const Block3 b = split_at(c, dim);
  long osize[kMaxDims * 4];
  THC_CHECK(src->nDimension <= kMaxDims * 4, "too many dimensions");
  for (int d = 0; d < src->nDimension; d++) osize[d] = src->size[d];
  osize[dim] = nidx;
  const int nd = src->nDimension;
  TensorRef out(tensor_new_sized(nd, osize));
  const long total = b.outer * nidx * b.inner;
  if (total > 0) {
    index_kernel<0><<<grid_for(total), 256, 0, stream()>>>(data_ptr(out), data_ptr(c), idx, b.outer, b.D, nidx, b.inner, 0.f);
    check_launch("indexSelect");
  }
  resize_nd(res_, nd, osize, nullptr);
  tensor_copy(res_, out);
  THC_END()
}

THC_API void THGPUTensor_indexCopy(THGPUTensor *res_, int dim, THLongTensor *indices, THGPUTensor *src) {
  THC_BEGIN
  THC_ARG(src->nDimension > 0, 2, "Source tensor is empty");
  THC_ARG(dim >= 0 && dim < src->nDimension && dim < res_->nDimension, 4, "Indexing dim is out of bounds");
  WsScope ws_scope;
  long nidx;
  const long *idx = upload_indices(indices, res_->size[dim], nidx);
  THC_ARG(nidx == src->size[dim], 4, "length of src.size[dim] is not equal to length of indices");
  THC_ARG(src->nDimension == res_->nDimension, 4, "source and destination must have the same number of dimensions");
  for (int d = 0; d < src->nDimension; d++)
    THC_ARG(d == dim || src->size[d] == res_->size[d], 4, "source and destination sizes differ outside the indexed dimension");
  TensorRef c(tensor_new_contiguous(src));
  TensorRef rc(tensor_new_contiguous(res_));   // res_ itself when it is contiguous
  const Block3 b = split_at(rc, dim);
  const long total = b.outer * nidx * b.inner;
  if (total > 0) {
    index_kernel<1><<<grid_for(total), 256, 0, stream()>>>(data_ptr(rc), data_ptr(c), idx, b.outer, b.D, nidx, b.inner, 0.f);
    check_launch("indexCopy");
  }
  if (rc.t != res_) tensor_copy(res_, rc);
  THC_END()
}

THC_API void THGPUTensor_indexFill(THGPUTensor *res_, int dim, THLongTensor *indices, float val) {
  THC_BEGIN
  THC_ARG(res_->nDimension > 0, 2, "Source tensor is empty");
  THC_ARG(dim >= 0 && dim < res_->nDimension, 4, "Indexing dim is out of bounds");
  WsScope ws_scope;
  long nidx;
  const long *idx = upload_indices(indices, res_->size[dim], nidx);
  TensorRef rc(tensor_new_contiguous(res_));
  const Block3 b = split_at(rc, dim);
  const long total = b.outer * nidx * b.inner;
  if (total > 0) {
    index_kernel<2><<<grid_for(total), 256, 0, stream()>>>(data_ptr(rc), nullptr, idx, b.outer, b.D, nidx, b.inner, val);
    check_launch("indexFill");
  }
  if (rc.t != res_) tensor_copy(res_, rc);
  THC_END()
}
