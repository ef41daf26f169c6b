// torch.GPUTensor math: elementwise, full reductions, dim-wise reductions, BLAS-backed products.
//
// Reference: gputorch/lib/THC/THCTensorMath.cpp (line ranges per function in include/THC.h) and its
// Bolt wrappers gputorch/lib/THC/THCBolt.cpp:96-412.  Numerics follow the CPU TH semantics the
// results are checked against (mcw_torch7_core/lib/TH/generic/THTensorMath.c): sums accumulate in
// double (TH's accreal), max/min use strict comparisons so the first extremum wins.
#include <cfloat>

#include "thc_apply.cuh"

namespace thc {

// ------------------------------------------------------------------ elementwise functors
struct ConstOp { float v; __device__ float operator()(const float *) const { return v; } };
struct AddScalarOp { float v; __device__ float operator()(const float *a) const { return a[0] + v; } };
struct MulScalarOp { float v; __device__ float operator()(const float *a) const { return a[0] * v; } };
struct DivScalarOp { float v; __device__ float operator()(const float *a) const { return a[0] / v; } };
// t + value*src with the product rounded before the sum, like the C expression on the CPU
struct CaddOp { float v; __device__ float operator()(const float *a) const { return __fadd_rn(a[0], __fmul_rn(v, a[1])); } };
struct CmulOp { __device__ float operator()(const float *a) const { return a[0] * a[1]; } };
struct CdivOp { __device__ float operator()(const float *a) const { return a[0] / a[1]; } };

static void resize_as(THGPUTensor *r, const THGPUTensor *t) { tensor_resize_as(r, t); }

// ------------------------------------------------------------------ full reductions
// Pass 1: every block reduces a grid-strided slice (fp32 runs of 4 folded into a double
// accumulator per thread), writes one partial; the last block to finish (atomic ticket) folds the
// partials in fixed order, so the result is deterministic.  No block ever waits on another.
enum { RED_SUM = 0, RED_MAX = 1, RED_MIN = 2, RED_DOT = 3 };

struct RedScratch {
  double partial[1024];
  unsigned int ticket;
  unsigned int pad;
  double result;
};

template <int MODE> struct RedTraits;
template <> struct RedTraits<RED_SUM> {
  __device__ static double init(float) { return 0.0; }
  __device__ static double fold4(float4 v) { return (double)((v.x + v.y) + (v.z + v.w)); }
  __device__ static double one(float v) { return (double)v; }
  __device__ static double comb(double a, double b) { return a + b; }
};
template <> struct RedTraits<RED_MAX> {
  __device__ static double init(float first) { return (double)first; }
  __device__ static double fold4(float4 v) { return (double)fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)); }
  __device__ static double one(float v) { return (double)v; }
  __device__ static double comb(double a, double b) { return a > b ? a : b; }
};
template <> struct RedTraits<RED_MIN> {
  __device__ static double init(float first) { return (double)first; }
  __device__ static double fold4(float4 v) { return (double)fminf(fminf(v.x, v.y), fminf(v.z, v.w)); }
  __device__ static double one(float v) { return (double)v; }
  __device__ static double comb(double a, double b) { return a < b ? a : b; }
};

template <int MODE>
__device__ __forceinline__ double block_reduce(double v, double *smem) {
  typedef RedTraits<MODE> T;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = T::comb(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    // lanes beyond the warp count re-use entry 0 for max/min (idempotent) and contribute 0 to sums
    v = lane < nwarps ? smem[lane] : (MODE == RED_SUM ? 0.0 : smem[0]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = T::comb(v, __shfl_xor_sync(0xffffffffu, v, o));
  }
  __syncthreads();
  return v;  // valid in warp 0
}

template <int MODE>
__global__ void __launch_bounds__(512) reduce_all_kernel(const float *__restrict__ x, const float *__restrict__ y,
                                                         long n, bool vec, RedScratch *s) {
  typedef RedTraits<MODE == RED_DOT ? RED_SUM : MODE> T;
  __shared__ double smem[32];
  __shared__ bool is_last;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long)gridDim.x * blockDim.x;
  double acc = T::init(x[0]);
  long done = 0;
  if (vec) {
    const long nvec = n >> 2;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *y4 = reinterpret_cast<const float4 *>(y);
    long i = tid;
    if (MODE != RED_DOT) {  // four independent 16-byte loads per thread in flight
      for (; i + 3 * nthreads < nvec; i += 4 * nthreads) {
        const float4 v0 = x4[i], v1 = x4[i + nthreads], v2 = x4[i + 2 * nthreads], v3 = x4[i + 3 * nthreads];
        acc = T::comb(acc, T::comb(T::comb(T::fold4(v0), T::fold4(v1)), T::comb(T::fold4(v2), T::fold4(v3))));
      }
    }
    for (; i < nvec; i += nthreads) {
      float4 v = x4[i];
      if (MODE == RED_DOT) {
        const float4 w = y4[i];
        // products are exact in double; keeps the dot product faithful to a double accumulator
        acc += (double)v.x * w.x + (double)v.y * w.y + (double)v.z * w.z + (double)v.w * w.w;
      } else
        acc = T::comb(acc, T::fold4(v));
    }
    done = nvec << 2;
  }
  for (long i = done + tid; i < n; i += nthreads) {
    if (MODE == RED_DOT) acc += (double)x[i] * y[i];
    else acc = T::comb(acc, T::one(x[i]));
  }
  acc = block_reduce<(MODE == RED_DOT ? RED_SUM : MODE)>(acc, smem);
  if (threadIdx.x == 0) {
    s->partial[blockIdx.x] = acc;
    __threadfence();
    const unsigned int t = atomicAdd(&s->ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    double v = T::init(x[0]);
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) v = T::comb(v, ((volatile double *)s->partial)[i]);
    v = block_reduce<(MODE == RED_DOT ? RED_SUM : MODE)>(v, smem);
    if (threadIdx.x == 0) {
      s->result = v;
      s->ticket = 0;  // ready for the next launch on this stream
    }
  }
}

// A tensor whose elements occupy one gap-free block of memory in some dim order (contiguous, or a
// transposed / permuted view of a contiguous block): order-free reductions can run over the block.
static bool is_dense_block(const THGPUTensor *t) {
  int order[kMaxDims * 4];
  int nd = 0;
  for (int d = 0; d < t->nDimension; d++)
    if (t->size[d] != 1) { if (nd >= kMaxDims * 4) return false; order[nd++] = d; }
  for (int i = 1; i < nd; i++)
    for (int j = i; j > 0 && t->stride[order[j]] < t->stride[order[j - 1]]; j--) {
      int z = order[j]; order[j] = order[j - 1]; order[j - 1] = z;
    }
  long z = 1;
  for (int i = 0; i < nd; i++) {
    if (t->stride[order[i]] != z) return false;
    z *= t->size[order[i]];
  }
  return true;
}

static bool same_layout(const THGPUTensor *a, const THGPUTensor *b) {
  if (a->nDimension != b->nDimension) return false;
  for (int d = 0; d < a->nDimension; d++)
    if (a->size[d] != b->size[d] || (a->size[d] != 1 && a->stride[d] != b->stride[d])) return false;
  return true;
}

template <int MODE>
static double reduce_all(THGPUTensor *t, THGPUTensor *u) {
  const long n = nelem(t);
  THC_ARG(n > 0, 1, "tensor must have one dimension");
  THGPUTensor *tc = nullptr, *uc = nullptr;
  const float *x, *y = nullptr;
  if (MODE == RED_DOT) {
    THC_ARG(nelem(u) == n, 2, "sizes do not match");
    if (is_dense_block(t) && same_layout(t, u)) { x = data_ptr(t); y = data_ptr(u); }
    else { tc = tensor_new_contiguous(t); uc = tensor_new_contiguous(u); x = data_ptr(tc); y = data_ptr(uc); }
  } else {
    if (is_dense_block(t)) x = data_ptr(t);
    else { tc = tensor_new_contiguous(t); x = data_ptr(tc); }
  }
  Context &c = ctx();
  RedScratch *s = (RedScratch *)scratch(sizeof(RedScratch));
  // the ticket starts at 0 (scratch is zero-filled when allocated); each launch resets it
  const bool vec = aligned16(x) && (MODE != RED_DOT || aligned16(y));
  long work = vec ? (n + 3) / 4 : n;
  int blocks = (int)((work + 511) / 512);
  int cap = c.sm_count * 4;   // 4 blocks of 512 threads per SM = full occupancy
  if (cap > 1024) cap = 1024;
  if (blocks > cap) blocks = cap;
  reduce_all_kernel<MODE><<<blocks, 512, 0, stream()>>>(x, y, n, vec, s);
  check_launch("reduce_all");
  double *host = (double *)c.host_pinned;
  THC_CUDA(cudaMemcpyAsync(host, &s->result, sizeof(double), cudaMemcpyDeviceToHost, stream()));
  sync_stream();
  if (tc) tensor_free(tc);
  if (uc) tensor_free(uc);
  return *host;
}

// ------------------------------------------------------------------ dim-wise reductions
// The source is described as out(o, j) <- reduce_r src[base + o*so + j*sj + r*sr].
//   row kernel   : sr == 1 (reduced dim is the unit-stride one).  One block per output.
//   column kernel: sj == 1 (outputs are unit-stride neighbours).  Threads own 1 column each, the
//                  reduced dim is additionally split over threadIdx.y and blockIdx.y; a second tiny
//                  kernel folds the blockIdx.y partials in ascending order.
template <int MODE, class I = long> __device__ __forceinline__ bool better(float a, I ia, float b, I ib) {
  // true when (a, ia) should replace (b, ib): strictly better value, or equal value at a lower index
  if (MODE == RED_MAX) return a > b || (a == b && ia < ib);
  return a < b || (a == b && ia < ib);
}

template <int MODE>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const float *__restrict__ src, long so, long R,
                                                          float *__restrict__ out, float *__restrict__ idx,
                                                          float scale, bool vec) {
  __shared__ double sd[32];
  __shared__ float sv[32];
  __shared__ long si[32];
  const float *row = src + (long)blockIdx.x * so;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (MODE == RED_SUM) {
    double acc = 0;
    long done = 0;
    if (vec) {
      const float4 *r4 = reinterpret_cast<const float4 *>(row);
      const long n4 = R >> 2, bd = blockDim.x;
      long i = threadIdx.x;
      // four 16-byte loads in flight per thread before the first add (a row of 8192 floats is two such rounds)
      for (; i + 3 * bd < n4; i += 4 * bd) {
        const float4 v0 = r4[i], v1 = r4[i + bd], v2 = r4[i + 2 * bd], v3 = r4[i + 3 * bd];
        acc += (double)v0.x + (double)v0.y + (double)v0.z + (double)v0.w;
        acc += (double)v1.x + (double)v1.y + (double)v1.z + (double)v1.w;
        acc += (double)v2.x + (double)v2.y + (double)v2.z + (double)v2.w;
        acc += (double)v3.x + (double)v3.y + (double)v3.z + (double)v3.w;
      }
      for (; i < n4; i += bd) {
        const float4 v = r4[i];
        acc += (double)v.x + (double)v.y + (double)v.z + (double)v.w;
      }
      done = n4 << 2;
    }
    for (long i = done + threadIdx.x; i < R; i += blockDim.x) acc += (double)row[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) sd[warp] = acc;
    __syncthreads();
    if (warp == 0) {
      acc = lane < nwarps ? sd[lane] : 0.0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) out[blockIdx.x] = (float)(acc * (double)scale);
    }
  } else {
    // positions fit 32 bits (checked by the launcher): half the integer work of 64-bit indices per element
    float bv = row[0];
    int bi = 0;
    long done = 0;
    if (vec) {
      const float4 *r4 = reinterpret_cast<const float4 *>(row);
      const long n4 = R >> 2, bd = blockDim.x;
      // the best of the four first (ties keep the lower position), then one comparison against the running best
      auto take = [&](const float4 &v, long i) {
        const int b = (int)(i << 2);
        float m = v.x; int mi = b;
        if (MODE == RED_MAX ? v.y > m : v.y < m) { m = v.y; mi = b + 1; }
        if (MODE == RED_MAX ? v.z > m : v.z < m) { m = v.z; mi = b + 2; }
        if (MODE == RED_MAX ? v.w > m : v.w < m) { m = v.w; mi = b + 3; }
        if (better<MODE, int>(m, mi, bv, bi)) { bv = m; bi = mi; }
      };
      long i = threadIdx.x;
      for (; i + 3 * bd < n4; i += 4 * bd) {   // four 16-byte loads in flight per thread
        const float4 v0 = r4[i], v1 = r4[i + bd], v2 = r4[i + 2 * bd], v3 = r4[i + 3 * bd];
        take(v0, i); take(v1, i + bd); take(v2, i + 2 * bd); take(v3, i + 3 * bd);
      }
      for (; i < n4; i += bd) take(r4[i], i);
      done = n4 << 2;
    }
    for (long i = done + threadIdx.x; i < R; i += blockDim.x)
      if (better<MODE, int>(row[i], (int)i, bv, bi)) { bv = row[i]; bi = (int)i; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better<MODE, int>(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < nwarps ? sv[lane] : sv[0];
      bi = lane < nwarps ? (int)si[lane] : (int)si[0];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better<MODE, int>(ov, oi, bv, bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0) {
        out[blockIdx.x] = bv;
        if (idx) idx[blockIdx.x] = (float)(bi + 1);
      }
    }
  }
}

// grid (ceil(J/32), splits, O); block (32, 8).  Partials: [O][splits][J].
template <int MODE>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const float *__restrict__ src, long so, long sr, long J,
                                                          long R, long rows_per_split, double *__restrict__ psum,
                                                          float *__restrict__ pval, long *__restrict__ pidx) {
  __shared__ double sd[8][33];
  __shared__ float sv[8][33];
  __shared__ long si[8][33];
  const long j = (long)blockIdx.x * 32 + threadIdx.x;
  const long r0 = (long)blockIdx.y * rows_per_split;
  long r1 = r0 + rows_per_split;
  if (r1 > R) r1 = R;
  const float *base = src + (long)blockIdx.z * so + j;
  double acc = 0;
  float bv = 0;
  long bi = -1;
  if (j < J) {
    long r = r0 + threadIdx.y;
    for (; r + 24 < r1; r += 32) {  // four independent loads in flight per thread
      const float v0 = base[r * sr], v1 = base[(r + 8) * sr], v2 = base[(r + 16) * sr], v3 = base[(r + 24) * sr];
      if (MODE == RED_SUM) acc += ((double)v0 + (double)v1) + ((double)v2 + (double)v3);
      else {
        if (bi < 0 || better<MODE>(v0, r, bv, bi)) { bv = v0; bi = r; }
        if (better<MODE>(v1, r + 8, bv, bi)) { bv = v1; bi = r + 8; }
        if (better<MODE>(v2, r + 16, bv, bi)) { bv = v2; bi = r + 16; }
        if (better<MODE>(v3, r + 24, bv, bi)) { bv = v3; bi = r + 24; }
      }
    }
    for (; r < r1; r += 8) {
      const float v = base[r * sr];
      if (MODE == RED_SUM) acc += (double)v;
      else if (bi < 0 || better<MODE>(v, r, bv, bi)) { bv = v; bi = r; }
    }
  }
  if (MODE == RED_SUM) sd[threadIdx.y][threadIdx.x] = acc;
  else { sv[threadIdx.y][threadIdx.x] = bv; si[threadIdx.y][threadIdx.x] = bi; }
  __syncthreads();
  if (threadIdx.y == 0 && j < J) {
    const long o = ((long)blockIdx.z * gridDim.y + blockIdx.y) * J + j;
    if (MODE == RED_SUM) {
      for (int k = 1; k < 8; k++) acc += sd[k][threadIdx.x];
      psum[o] = acc;
    } else {
      for (int k = 1; k < 8; k++) {
        const float ov = sv[k][threadIdx.x];
        const long oi = si[k][threadIdx.x];
        if (oi >= 0 && (bi < 0 || better<MODE>(ov, oi, bv, bi))) { bv = ov; bi = oi; }
      }
      pval[o] = bv;
      pidx[o] = bi;
    }
  }
}

// The same with four adjacent columns per thread (16-byte loads: a warp fetches 512 contiguous bytes per row, and
// eight rows are requested before the first is used).  J % 4 == 0, 16-byte aligned rows.  grid (ceil(J/128), splits, O).
template <int MODE>
__global__ void __launch_bounds__(256) reduce_cols4_kernel(const float *__restrict__ src, long so, long sr, long J, long R,
                                                           long rows_per_split, double *__restrict__ psum,
                                                           float *__restrict__ pval, long *__restrict__ pidx) {
  __shared__ double sd[8][129];
  __shared__ float sv[8][129];
  __shared__ long si[8][129];
  const long j = ((long)blockIdx.x * 32 + threadIdx.x) * 4;
  const long r0 = (long)blockIdx.y * rows_per_split;
  long r1 = r0 + rows_per_split;
  if (r1 > R) r1 = R;
  const float *base = src + (long)blockIdx.z * so + j;
  double acc[4] = {0, 0, 0, 0};
  float bv[4] = {0, 0, 0, 0};
  long bi[4] = {-1, -1, -1, -1};
  auto take = [&](const float4 &v, long r) {
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int c = 0; c < 4; c++) {
      if (MODE == RED_SUM) acc[c] += (double)e[c];
      else if (bi[c] < 0 || better<MODE>(e[c], r, bv[c], bi[c])) { bv[c] = e[c]; bi[c] = r; }
    }
  };
  if (j < J) {
    long r = r0 + threadIdx.y;
    for (; r + 56 < r1; r += 64) {
      float4 v[8];
#pragma unroll
      for (int u = 0; u < 8; u++) v[u] = *reinterpret_cast<const float4 *>(base + (r + 8 * u) * sr);
#pragma unroll
      for (int u = 0; u < 8; u++) take(v[u], r + 8 * u);
    }
    for (; r < r1; r += 8) take(*reinterpret_cast<const float4 *>(base + r * sr), r);
  }
#pragma unroll
  for (int c = 0; c < 4; c++) {
    if (MODE == RED_SUM) sd[threadIdx.y][threadIdx.x * 4 + c] = acc[c];
    else { sv[threadIdx.y][threadIdx.x * 4 + c] = bv[c]; si[threadIdx.y][threadIdx.x * 4 + c] = bi[c]; }
  }
  __syncthreads();
  // 128 columns of the block, folded over the eight row slices in slice order
  const int col = threadIdx.y * 32 + threadIdx.x;
  if (col < 128) {
    const long jc = (long)blockIdx.x * 128 + col;
    if (jc < J) {
      const long o = ((long)blockIdx.z * gridDim.y + blockIdx.y) * J + jc;
      if (MODE == RED_SUM) {
        double a = sd[0][col];
        for (int k = 1; k < 8; k++) a += sd[k][col];
        psum[o] = a;
      } else {
        float v = sv[0][col];
        long i = si[0][col];
        for (int k = 1; k < 8; k++) {
          const float ov = sv[k][col];
          const long oi = si[k][col];
          if (oi >= 0 && (i < 0 || better<MODE>(ov, oi, v, i))) { v = ov; i = oi; }
        }
        pval[o] = v;
        pidx[o] = i;
      }
    }
  }
}

template <int MODE>
__global__ void reduce_cols_finish_kernel(const double *__restrict__ psum, const float *__restrict__ pval,
                                          const long *__restrict__ pidx, int splits, long J, long O,
                                          float *__restrict__ out, float *__restrict__ idx, float scale) {
  const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= O * J) return;
  const long o = t / J, j = t - o * J;
  if (MODE == RED_SUM) {
    double acc = 0;
    for (int s = 0; s < splits; s++) acc += psum[(o * splits + s) * J + j];
    out[t] = (float)(acc * (double)scale);
  } else {
    float bv = 0;
    long bi = -1;
    for (int s = 0; s < splits; s++) {
      const float ov = pval[(o * splits + s) * J + j];
      const long oi = pidx[(o * splits + s) * J + j];
      if (oi >= 0 && (bi < 0 || better<MODE>(ov, oi, bv, bi))) { bv = ov; bi = oi; }
    }
    out[t] = bv;
    if (idx) idx[t] = (float)(bi + 1);
  }
}

template <int MODE>
static void reduce_dim(THGPUTensor *values, THGPUTensor *indices, THGPUTensor *src, long dim, float scale) {
  THC_ARG(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  // output shape = src shape with size[dim] = 1 (kept), computed into a contiguous result
  long osize[kMaxDims * 4];
  THC_CHECK(src->nDimension <= kMaxDims * 4, "too many dimensions");
  for (int d = 0; d < src->nDimension; d++) osize[d] = src->size[d];
  osize[dim] = 1;
  const long R = src->size[dim];
  // The result is produced into contiguous temporaries when the destinations alias the source or
  // are not contiguous after resizing.
  THGPUTensor *src_keep = nullptr;
  long O, J, so, sj, sr;
  const float *base;
  auto describe = [&](THGPUTensor *t) -> bool {
    // contiguous: [outer, R, inner]
    if (is_contiguous(t)) {
      O = 1; J = 1;
      for (int d = 0; d < dim; d++) O *= t->size[d];
      for (int d = (int)dim + 1; d < t->nDimension; d++) J *= t->size[d];
      so = R * J; sj = 1; sr = J;
      if (J == 1) { J = O; O = 1; sj = R; sr = 1; so = 0; }  // innermost dim: rows
      return true;
    }
    if (t->nDimension == 2) {  // strided 2-D view (e.g. a transpose): use its strides directly
      const int od = dim == 0 ? 1 : 0;
      O = 1; so = 0; J = t->size[od]; sj = t->stride[od]; sr = t->stride[dim];
      return sr == 1 || sj == 1;
    }
    return false;
  };
  THC_ARG(nelem(src) > 0, 3, "empty tensor");
  if (R == 1) {  // nothing to reduce: values = src, every index is 1
    THGPUTensor *c = tensor_new_contiguous(src);
    THGPUTensor *v = tensor_new_sized(src->nDimension, osize);
    tensor_copy(v, c);
    if (MODE == RED_SUM && scale != 1.f) apply<1>(v, v, nullptr, MulScalarOp{scale}, "mean");
    tensor_free(c);
    resize_nd(values, src->nDimension, osize, nullptr);
    tensor_copy(values, v);
    tensor_free(v);
    if (indices) {
      resize_nd(indices, src->nDimension, osize, nullptr);
      apply<0>(indices, nullptr, nullptr, ConstOp{1.f}, "ones");
    }
    return;
  }
  if (!describe(src)) {
    src_keep = tensor_new_contiguous(src);
    src = src_keep;
    describe(src);
  }
  THC_CHECK(O <= 65535, "outer dimension too large for the column reducer");
  base = data_ptr(src);
  THGPUTensor *vtmp = tensor_new_sized(src->nDimension, osize);
  THGPUTensor *itmp = indices ? tensor_new_sized(src->nDimension, osize) : nullptr;
  float *out = data_ptr(vtmp), *idx = itmp ? data_ptr(itmp) : nullptr;
  if (sr == 1) {
    THC_CHECK(O == 1, "internal: row reduce with outer dim");
    THC_CHECK(R < (1l << 31), "reduced dimension too long");
    const bool vec = aligned16(base) && (sj % 4 == 0);
    int threads = R >= 4096 ? 256 : (R >= 512 ? 128 : 32);
    reduce_rows_kernel<MODE><<<(unsigned)J, threads, 0, stream()>>>(base, sj, R, out, idx, scale, vec);
    check_launch("reduce_rows");
  } else {
    THC_CHECK(sj == 1, "internal: column reduce needs unit stride");
    const bool vec4 = J % 4 == 0 && sr % 4 == 0 && so % 4 == 0 && aligned16(base) && J >= 128;
    const long colblocks = vec4 ? (J + 127) / 128 : (J + 31) / 32;
    long want = (long)ctx().sm_count * 8;
    long splits = want / (colblocks * O);
    if (splits < 1) splits = 1;
    if (splits > (R + 63) / 64) splits = (R + 63) / 64;
    if (splits > 512) splits = 512;
    long rows_per_split = (R + splits - 1) / splits;
    splits = (R + rows_per_split - 1) / rows_per_split;
    const size_t nparts = (size_t)O * splits * J;
    WsScope ws_scope;
    char *scr = (char *)ws_alloc(nparts * (MODE == RED_SUM ? sizeof(double) : sizeof(float) + sizeof(long)));
    double *psum = (double *)scr;
    long *pidx = (long *)scr;
    float *pval = (float *)(scr + (MODE == RED_SUM ? 0 : nparts * sizeof(long)));
    dim3 grid((unsigned)colblocks, (unsigned)splits, (unsigned)O), block(32, 8);
    if (vec4) reduce_cols4_kernel<MODE><<<grid, block, 0, stream()>>>(base, so, sr, J, R, rows_per_split, psum, pval, pidx);
    else reduce_cols_kernel<MODE><<<grid, block, 0, stream()>>>(base, so, sr, J, R, rows_per_split, psum, pval, pidx);
    check_launch("reduce_cols");
    const long total = O * J;
    reduce_cols_finish_kernel<MODE><<<ceil_div(total, 256), 256, 0, stream()>>>(psum, pval, pidx, (int)splits, J, O, out, idx, scale);
    check_launch("reduce_cols_finish");
  }
  const int ond = src->nDimension;
  if (src_keep) tensor_free(src_keep);
  resize_nd(values, ond, osize, nullptr);
  tensor_copy(values, vtmp);
  tensor_free(vtmp);
  if (indices) {
    resize_nd(indices, ond, osize, nullptr);
    tensor_copy(indices, itmp);
    tensor_free(itmp);
  }
}

}  // namespace thc

using namespace thc;

THC_API void THGPUTensor_add(THGPUTensor *self, THGPUTensor *src, float value) {
  THC_BEGIN resize_as(self, src); apply<1>(self, src, nullptr, AddScalarOp{value}, "add"); THC_END()
}
THC_API void THGPUTensor_mul(THGPUTensor *self, THGPUTensor *src, float value) {
  THC_BEGIN resize_as(self, src); apply<1>(self, src, nullptr, MulScalarOp{value}, "mul"); THC_END()
}
THC_API void THGPUTensor_div(THGPUTensor *self, THGPUTensor *src, float value) {
  THC_BEGIN resize_as(self, src); apply<1>(self, src, nullptr, DivScalarOp{value}, "div"); THC_END()
}
THC_API void THGPUTensor_cadd(THGPUTensor *self, THGPUTensor *src1, float value, THGPUTensor *src2) {
  THC_BEGIN
  THC_ARG(nelem(src1) == nelem(src2), 3, "size do not match");
  resize_as(self, src1);
  THC_ARG(THGPUTensor_isSameSizeAs(src1, src2), 3, "shapes do not match");
  apply<2>(self, src1, src2, CaddOp{value}, "cadd");
  THC_END()
}
THC_API void THGPUTensor_cmul(THGPUTensor *self, THGPUTensor *src1, THGPUTensor *src2) {
  THC_BEGIN
  THC_ARG(nelem(src1) == nelem(src2), 3, "size do not match");
  resize_as(self, src1);
  THC_ARG(THGPUTensor_isSameSizeAs(src1, src2), 3, "shapes do not match");
  apply<2>(self, src1, src2, CmulOp(), "cmul");
  THC_END()
}
THC_API void THGPUTensor_cdiv(THGPUTensor *self, THGPUTensor *src1, THGPUTensor *src2) {
  THC_BEGIN
  THC_ARG(nelem(src1) == nelem(src2), 3, "size do not match");
  resize_as(self, src1);
  THC_ARG(THGPUTensor_isSameSizeAs(src1, src2), 3, "shapes do not match");
  apply<2>(self, src1, src2, CdivOp(), "cdiv");
  THC_END()
}

THC_API float THGPUTensor_dot(THGPUTensor *self, THGPUTensor *src) { THC_BEGIN return (float)reduce_all<RED_DOT>(self, src); THC_END(0.f) }
THC_API float THGPUTensor_minall(THGPUTensor *self) { THC_BEGIN return (float)reduce_all<RED_MIN>(self, nullptr); THC_END(0.f) }
THC_API float THGPUTensor_maxall(THGPUTensor *self) { THC_BEGIN return (float)reduce_all<RED_MAX>(self, nullptr); THC_END(0.f) }
THC_API float THGPUTensor_sumall(THGPUTensor *self) { THC_BEGIN return (float)reduce_all<RED_SUM>(self, nullptr); THC_END(0.f) }
THC_API float THGPUTensor_meanall(THGPUTensor *self) {
  THC_BEGIN
  return (float)(reduce_all<RED_SUM>(self, nullptr) / (double)nelem(self));
  THC_END(0.f)
}

THC_API void THGPUTensor_sum(THGPUTensor *self, THGPUTensor *src, long dim) {
  THC_BEGIN reduce_dim<RED_SUM>(self, nullptr, src, dim, 1.f); THC_END()
}
THC_API void THGPUTensor_mean(THGPUTensor *self, THGPUTensor *src, long dim) {
  THC_BEGIN
  THC_ARG(dim >= 0 && dim < src->nDimension, 3, "dimension out of range");
  reduce_dim<RED_SUM>(self, nullptr, src, dim, 1.f / (float)src->size[dim]);
  THC_END()
}
THC_API void THGPUTensor_max(THGPUTensor *values, THGPUTensor *indices, THGPUTensor *src, long dim) {
  THC_BEGIN reduce_dim<RED_MAX>(values, indices, src, dim, 1.f); THC_END()
}
THC_API void THGPUTensor_min(THGPUTensor *values, THGPUTensor *indices, THGPUTensor *src, long dim) {
  THC_BEGIN reduce_dim<RED_MIN>(values, indices, src, dim, 1.f); THC_END()
}

// ------------------------------------------------------------------ BLAS-backed products
// addmv (THCTensorMath.cpp:624-695): r = beta*t + alpha*mat*vec
THC_API void THGPUTensor_addmv(THGPUTensor *r_, float beta, THGPUTensor *t, float alpha, THGPUTensor *mat, THGPUTensor *vec) {
  THC_BEGIN
  THC_CHECK(mat->nDimension == 2 && vec->nDimension == 1, "matrix and vector expected");
  THC_CHECK(mat->size[1] == vec->size[0], "size mismatch");
  THC_CHECK(t->nDimension == 1 && t->size[0] == mat->size[0], "size mismatch");
  if (r_ != t) { resize_as(r_, t); tensor_copy(r_, t); }
  THGPUTensor *m = nullptr;
  if (mat->stride[0] == 1) {
    THGPUBlas_gemv('n', mat->size[0], mat->size[1], alpha, data_ptr(mat), mat->stride[1], data_ptr(vec), vec->stride[0],
                   beta, data_ptr(r_), r_->stride[0]);
  } else if (mat->stride[1] == 1) {
    THGPUBlas_gemv('t', mat->size[1], mat->size[0], alpha, data_ptr(mat), mat->stride[0], data_ptr(vec), vec->stride[0],
                   beta, data_ptr(r_), r_->stride[0]);
  } else {
    m = tensor_new_contiguous(mat);
    THGPUBlas_gemv('t', mat->size[1], mat->size[0], alpha, data_ptr(m), m->stride[0], data_ptr(vec), vec->stride[0],
                   beta, data_ptr(r_), r_->stride[0]);
    tensor_free(m);
  }
  THC_END()
}

// addr (THCTensorMath.cpp:809-860): r = beta*t + alpha * vec1 (x) vec2
THC_API void THGPUTensor_addr(THGPUTensor *r_, float beta, THGPUTensor *t, float alpha, THGPUTensor *vec1, THGPUTensor *vec2) {
  THC_BEGIN
  THC_CHECK(vec1->nDimension == 1 && vec2->nDimension == 1, "vector and vector expected");
  THC_CHECK(t->nDimension == 2, "size mismatch");
  THC_CHECK(t->size[0] == vec1->size[0] && t->size[1] == vec2->size[0], "size mismatch");
  if (r_ != t) { resize_as(r_, t); tensor_copy(r_, t); }
  if (beta != 1.f) apply<1>(r_, r_, nullptr, MulScalarOp{beta}, "mul");
  if (r_->stride[0] == 1) {
    THGPUBlas_ger(vec1->size[0], vec2->size[0], alpha, data_ptr(vec1), vec1->stride[0], data_ptr(vec2), vec2->stride[0],
                  data_ptr(r_), r_->stride[1]);
  } else if (r_->stride[1] == 1) {
    THGPUBlas_ger(vec2->size[0], vec1->size[0], alpha, data_ptr(vec2), vec2->stride[0], data_ptr(vec1), vec1->stride[0],
                  data_ptr(r_), r_->stride[0]);
  } else {
    THGPUTensor *c = tensor_new_sized(r_->nDimension, r_->size);
    tensor_copy(c, r_);
    THGPUBlas_ger(vec2->size[0], vec1->size[0], alpha, data_ptr(vec2), vec2->stride[0], data_ptr(vec1), vec1->stride[0],
                  data_ptr(c), c->stride[0]);
    tensor_copy(r_, c);
    tensor_free(c);
  }
  THC_END()
}

// addmm (THCTensorMath.cpp:697-807; CPU semantics mcw_torch7_core/lib/TH/generic/THTensorMath.c:458-561):
// r = beta*t + alpha*m1*m2.  Row-major results are computed as the transposed column-major product;
// transpose flags come from the operands' strides, so transposed views cost nothing.  A result with
// neither stride equal to 1 goes through a contiguous temporary and is copied back (the CPU
// behaviour; the reference GPU code wrote into the wrong buffer there).
THC_API void THGPUTensor_addmm(THGPUTensor *r_, float beta, THGPUTensor *t, float alpha, THGPUTensor *m1, THGPUTensor *m2) {
  THC_BEGIN
  THC_CHECK(m1->nDimension == 2 && m2->nDimension == 2, "matrix and matrix expected");
  THC_CHECK(t->nDimension == 2, "size mismatch");
  THC_CHECK(t->size[0] == m1->size[0] && t->size[1] == m2->size[1] && m1->size[1] == m2->size[0], "size mismatch");
  if (t != r_) { resize_as(r_, t); tensor_copy(r_, t); }
  char transpose_r, transpose_m1, transpose_m2;
  THGPUTensor *r__, *m1_, *m2_;
  if (r_->stride[0] == 1 && r_->stride[1] != 0) { transpose_r = 'n'; r__ = r_; }
  else if (r_->stride[1] == 1 && r_->stride[0] != 0) { THGPUTensor *sw = m2; m2 = m1; m1 = sw; transpose_r = 't'; r__ = r_; }
  else {
    transpose_r = 'n';
    const long tsize[2] = {r_->size[1], r_->size[0]};
    r__ = tensor_new_sized(2, tsize);
    { long z = r__->size[0]; r__->size[0] = r__->size[1]; r__->size[1] = z;
      z = r__->stride[0]; r__->stride[0] = r__->stride[1]; r__->stride[1] = z; }
    tensor_copy(r__, r_);
  }
  const int i0 = transpose_r == 'n' ? 0 : 1, i1 = transpose_r == 'n' ? 1 : 0;
  if (m1->stride[i0] == 1 && m1->stride[i1] != 0) { transpose_m1 = 'n'; m1_ = m1; }
  else if (m1->stride[i1] == 1 && m1->stride[i0] != 0) { transpose_m1 = 't'; m1_ = m1; }
  else { transpose_m1 = transpose_r == 'n' ? 't' : 'n'; m1_ = tensor_new_contiguous(m1); }
  if (m2->stride[i0] == 1 && m2->stride[i1] != 0) { transpose_m2 = 'n'; m2_ = m2; }
  else if (m2->stride[i1] == 1 && m2->stride[i0] != 0) { transpose_m2 = 't'; m2_ = m2; }
  else { transpose_m2 = transpose_r == 'n' ? 't' : 'n'; m2_ = tensor_new_contiguous(m2); }
  gemm(transpose_m1, transpose_m2, r__->size[i0], r__->size[i1], m1_->size[i1], alpha, data_ptr(m1_),
       transpose_m1 == 'n' ? m1_->stride[i1] : m1_->stride[i0], data_ptr(m2_),
       transpose_m2 == 'n' ? m2_->stride[i1] : m2_->stride[i0], beta, data_ptr(r__), r__->stride[i1]);
  if (m1_ != m1) tensor_free(m1_);
  if (m2_ != m2) tensor_free(m2_);
  if (r__ != r_) { tensor_copy(r_, r__); tensor_free(r__); }
  THC_END()
}
