// BLAS front-ends on raw device pointers (column-major Fortran convention), the layer the
// reference implemented in gputorch/lib/THC/THCBlas.cpp: gemm dispatch :249-288 over four 16x16
// tile kernels :10-246 (three of which ignored the leading dimensions), gemv :291-467, axpy
// :470-483, ger :486-502.  Here gemm maps onto the shared matrix-multiply engines (tcgen05 3xTF32
// by default), all leading dimensions are honoured and C is not read when beta == 0.
#include "mm_launch.cuh"

namespace thc {

struct ScaleOp { float v; __device__ float operator()(const float *a) const { return a[0] * v; } };

static __global__ void scale_matrix_kernel(float *c, long m, long n, long ldc, float beta) {
  const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= m * n) return;
  const long j = t / m, i = t - j * m;
  c[i + j * ldc] = beta == 0.f ? 0.f : beta * c[i + j * ldc];
}

// Tensor-core path: both operands are first rounded into K-major hi / lo planes (one pass over each,
// which also absorbs all four transpose layouts), then one engine instance serves every gemm.
static void gemm_split(bool ta, bool tb, long m, long n, long k, float alpha, const float *a, long lda, const float *b,
                       long ldb, float beta, float *c, long ldc) {
  using namespace mm;
  SplitPlanes pa = make_split_planes(a, ta ? lda : 1, ta ? 1 : lda, m, k);   // A(i,l): 'n' a[i + l*lda], 't' a[l + i*lda]
  SplitPlanes pb = make_split_planes(b, tb ? 1 : ldb, tb ? ldb : 1, n, k);   // B(j,l): 'n' b[l + j*ldb], 't' b[j + l*ldb]
  Problem<SplitOperand, SplitOperand> p;
  p.a = split_operand(pa, m);
  p.b = split_operand(pb, n);
  p.epi = Epilogue{c, nullptr, alpha, beta, LONG_MAX, 0, ldc};
  p.M = m; p.N = n; p.K = k;
  launch_planes(p);
}

// Tensor-core path over the matrices as they lie in memory (raw-operand engine): TMA reads either layout of
// either operand, so no pass over the operands precedes the product.
template <bool TA, bool TB>
static void gemm_raw_t(long m, long n, long k, float alpha, const float *a, long lda, const float *b, long ldb, float beta,
                       float *c, long ldc) {
  using namespace mm;
  // A(i,l): 'n' a[i + l*lda] runs along the rows (MN-major), 't' a[l + i*lda] along k.  B(j,l): 'n' b[l + j*ldb]
  // runs along k, 't' b[j + l*ldb] along the rows.
  typedef RawOperand<!TA> OpA;
  typedef RawOperand<TB> OpB;
  Problem<OpA, OpB> p;
  p.epi = Epilogue{c, nullptr, alpha, beta, LONG_MAX, 0, ldc};
  p.M = m; p.N = n; p.K = k;
  launch_raw(p, [&](Problem<OpA, OpB> &q, int bn2) {
    attach_raw_map(q.a, a, m, k, lda, TC_BM);
    attach_raw_map(q.b, b, n, k, ldb, bn2 / 2);
  });
}
static bool gemm_raw_ok(long m, long n, const float *a, long lda, const float *b, long ldb) {
  return mm::tc2_tile_width(m, n) != 0 && mm::raw_matrix_ok(a, lda) && mm::raw_matrix_ok(b, ldb);
}

// BF16 math mode: one BF16 plane per operand, the BF16 two-SM engine; products too small for it run FP32-accurate.
static void gemm_half(bool ta, bool tb, long m, long n, long k, float alpha, const float *a, long lda, const float *b,
                      long ldb, float beta, float *c, long ldc) {
  using namespace mm;
  HalfPlane pa = make_half_plane(a, ta ? lda : 1, ta ? 1 : lda, m, k);
  HalfPlane pb = make_half_plane(b, tb ? 1 : ldb, tb ? ldb : 1, n, k);
  Problem<SplitOperand, SplitOperand> p;
  p.a = half_operand(pa.p, m, pa.ld);
  p.b = half_operand(pb.p, n, pb.ld);
  p.epi = Epilogue{c, nullptr, alpha, beta, LONG_MAX, 0, ldc};
  p.M = m; p.N = n; p.K = pa.ld / 2;
  launch_planes_half(p);
}

template <bool TA, bool TB>
static void gemm_t(long m, long n, long k, float alpha, const float *a, long lda, const float *b, long ldb,
                   float beta, float *c, long ldc) {
  using namespace mm;
  typedef Operand<LinearMap, LinearMap, 0, TA> OpA;     // 't': memory runs along k
  typedef Operand<LinearMap, LinearMap, 0, !TB> OpB;    // 'n': b[l + j*ldb] runs along k
  Problem<OpA, OpB> p;
  p.a.base = a;
  p.a.rows = LinearMap{m, TA ? lda : 1};
  p.a.ks = LinearMap{k, TA ? 1 : lda};
  p.b.base = b;
  p.b.rows = LinearMap{n, TB ? 1 : ldb};
  p.b.ks = LinearMap{k, TB ? ldb : 1};
  auto vec_ok = [](const float *base, long row_stride, long k_stride) {
    return (int)(((uintptr_t)base & 15) == 0 && row_stride % 4 == 0 && k_stride == 1);
  };
  p.a.vec4 = vec_ok(a, p.a.rows.stride, p.a.ks.stride);
  p.b.vec4 = vec_ok(b, p.b.rows.stride, p.b.ks.stride);
  p.a.H = p.a.W = p.b.H = p.b.W = 0;
  p.a.dH = p.a.dW = p.b.dH = p.b.dW = 1;
  p.epi = Epilogue{c, nullptr, alpha, beta, LONG_MAX, 0, ldc};
  p.M = m; p.N = n; p.K = k;
  launch(p);
}

void gemm(char transa, char transb, long m, long n, long k, float alpha, const float *a, long lda,
          const float *b, long ldb, float beta, float *c, long ldc) {
  const bool ta = transa == 't' || transa == 'T', tb = transb == 't' || transb == 'T';
  if (m <= 0 || n <= 0) return;
  WsScope ws_scope;
  if (k <= 0 || alpha == 0.f) {
    if (beta == 1.f) return;
    scale_matrix_kernel<<<ceil_div(m * n, 256), 256, 0, stream()>>>(c, m, n, ldc, beta);
    check_launch("scale_matrix");
    return;
  }
  if (ctx().math_mode == 2 && mm::tc2h_tile_width(m, n, false)) {
    gemm_half(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    return;
  }
  if (ctx().math_mode != 1 && gemm_raw_ok(m, n, a, lda, b, ldb)) {
    if (!ta && !tb) gemm_raw_t<false, false>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    else if (ta && !tb) gemm_raw_t<true, false>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    else if (!ta && tb) gemm_raw_t<false, true>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    else gemm_raw_t<true, true>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    return;
  }
  if (ctx().math_mode != 1) { gemm_split(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc); return; }
  if (!ta && !tb) gemm_t<false, false>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
  else if (ta && !tb) gemm_t<true, false>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
  else if (!ta && tb) gemm_t<false, true>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
  else gemm_t<true, true>(m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

// y = beta*y + alpha*op(A)*x.  'n': A is m x n column-major, y has m entries: threads own rows
// (coalesced across the column).  't': y has n entries, one warp per column of A.
// block = 32 rows x 32 column slices; the slices' partial sums are folded in slice order (deterministic)
static __global__ void __launch_bounds__(1024) gemv_n_kernel(long m, long n, float alpha, const float *__restrict__ a, long lda,
                                                             const float *__restrict__ x, long incx, float beta, float *y,
                                                             long incy) {
  __shared__ float part[32][33];
  const long i = (long)blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (i < m)
    for (long j = threadIdx.y; j < n; j += 32) acc = fmaf(a[i + j * lda], x[j * incx], acc);
  part[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && i < m) {
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < 32; s++) sum += part[s][threadIdx.x];
    y[i * incy] = (beta == 0.f ? 0.f : beta * y[i * incy]) + alpha * sum;
  }
}
static __global__ void gemv_t_kernel(long m, long n, float alpha, const float *__restrict__ a, long lda,
                                     const float *__restrict__ x, long incx, float beta, float *y, long incy) {
  const long j = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (j >= n) return;
  const int lane = threadIdx.x & 31;
  float acc = 0.f;
  for (long i = lane; i < m; i += 32) acc = fmaf(a[i + j * lda], x[i * incx], acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) y[j * incy] = (beta == 0.f ? 0.f : beta * y[j * incy]) + alpha * acc;
}
static __global__ void axpy_kernel(long n, float a, const float *__restrict__ x, long incx, float *y, long incy) {
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nthreads)
    y[i * incy] = __fadd_rn(y[i * incy], __fmul_rn(a, x[i * incx]));
}
static __global__ void ger_kernel(long m, long n, float alpha, const float *__restrict__ x, long incx,
                                  const float *__restrict__ y, long incy, float *a, long lda) {
  const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= m * n) return;
  const long j = t / m, i = t - j * m;
  a[i + j * lda] += alpha * x[i * incx] * y[j * incy];
}

}  // namespace thc

using namespace thc;

THC_API void THGPUBlas_gemm(char transa, char transb, long m, long n, long k, float alpha, const float *a, long lda,
                            const float *b, long ldb, float beta, float *c, long ldc) {
  THC_BEGIN
  gemm(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
  THC_END()
}

THC_API void THGPUBlas_gemv(char trans, long m, long n, float alpha, const float *a, long lda, const float *x,
                            long incx, float beta, float *y, long incy) {
  THC_BEGIN
  if (m <= 0 || n <= 0) return;
  if (trans == 't' || trans == 'T') {
    gemv_t_kernel<<<ceil_div(n, 8), 256, 0, stream()>>>(m, n, alpha, a, lda, x, incx, beta, y, incy);
    check_launch("gemv_t");
  } else {
    gemv_n_kernel<<<ceil_div(m, 32), dim3(32, 32), 0, stream()>>>(m, n, alpha, a, lda, x, incx, beta, y, incy);
    check_launch("gemv_n");
  }
  THC_END()
}

THC_API void THGPUBlas_axpy(long n, float a, const float *x, long incx, float *y, long incy) {
  THC_BEGIN
  if (n <= 0) return;
  int blocks = ceil_div(n, 256);
  const int cap = ctx().sm_count * 8;
  if (blocks > cap) blocks = cap;
  axpy_kernel<<<blocks, 256, 0, stream()>>>(n, a, x, incx, y, incy);
  check_launch("axpy");
  THC_END()
}

THC_API void THGPUBlas_ger(long m, long n, float alpha, const float *x, long incx, const float *y, long incy,
                           float *a, long lda) {
  THC_BEGIN
  if (m <= 0 || n <= 0) return;
  ger_kernel<<<ceil_div(m * n, 256), 256, 0, stream()>>>(m, n, alpha, x, incx, y, incy, a, lda);
  check_launch("ger");
  THC_END()
}

// ---- stall reporting of the tensor-core kernels ---------------------------------------------------------------
// One warp waits, with the engines' own bounded wait, on an mbarrier that nobody arrives on, and on expiry does
// what an engine CTA does: raises the stall flags and returns.  It faults nothing and waits no longer than
// `limit` SM cycles (plus one polling interval of a few tens of microseconds).
static __global__ void stall_probe_kernel(const mm::StallCtl ctl) {
  __shared__ uint64_t bar;
  __shared__ mm::WaitCtl w;
  if (threadIdx.x == 0) {
    mm::mbar_init(mm::smem_u32(&bar), 1);
    mm::wait_ctl_init(&w, ctl);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (w.abort) return;   // a stall is already on record
  const bool ok = mm::mbar_wait(mm::smem_u32(&bar), 0, &w, mm::kWaitProbe);
  if (!ok && threadIdx.x == 0) mm::stall_raise(ctl, w.abort);
}

THC_API void THGPUSetWaitLimit(long cycles) {
  THC_BEGIN
  THC_CHECK(cycles >= 1024 && cycles <= (1l << 34), "wait limit must lie in [2^10, 2^34] SM cycles");
  ctx().stall_limit = cycles;
  THC_END()
}
THC_API long THGPUGetWaitLimit(void) { THC_BEGIN return (long)ctx().stall_limit; THC_END(-1) }

THC_API int THGPUStallProbe(long limit_cycles) {
  THC_BEGIN
  Context &c = ctx();
  if (limit_cycles < 0) {   // host only: what the host sees after a kernel has raised the flag
    *(volatile int *)c.stall_host = 1;
    return 0;
  }
  THC_CHECK(limit_cycles >= 1024 && limit_cycles <= (1l << 27), "probe limit must lie in [2^10, 2^27] SM cycles");
  mm::StallCtl ctl = stall_ctl();
  ctl.limit = limit_cycles;
  stall_probe_kernel<<<1, 32, 0, stream()>>>(ctl);
  check_launch("stall_probe");
  return 0;
  THC_END(1)
}
