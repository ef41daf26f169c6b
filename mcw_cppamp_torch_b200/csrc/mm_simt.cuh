// FP32 FMA engine for mm::Problem ("simt" math mode): 64x64 output tile per 256-thread block, 4x4
// micro-tile per thread, operands gathered through the same row / k maps as the tensor-core engine.
// It is the exact-FP32 alternative to the 3xTF32 path and the on-device cross-check for it; it
// stands where the reference had its 16x16-tile one-output-per-thread SGEMM kernels
// (gputorch/lib/THC/THCBlas.cpp:10-246).
#ifndef THC_MM_SIMT_CUH
#define THC_MM_SIMT_CUH

#include "mm_problem.cuh"

namespace thc {
namespace mm {

constexpr int SIMT_BM = 64, SIMT_BN = 64, SIMT_BK = 16;

template <class P>
__global__ void __launch_bounds__(256) simt_kernel(const P p) {
  __shared__ float As[SIMT_BK][SIMT_BM + 4];
  __shared__ float Bs[SIMT_BK][SIMT_BN + 4];
  __shared__ Info kiA[SIMT_BK], kiB[SIMT_BK];
  const int t = threadIdx.x;
  const long m0 = (long)blockIdx.x * SIMT_BM, n0 = (long)blockIdx.y * SIMT_BN;
  long k_begin = 0, k_end = p.K;
  if (p.ws) {
    k_begin = (long)blockIdx.z * p.k_per_split;
    k_end = k_begin + p.k_per_split;
    if (k_end > p.K) k_end = p.K;
  }
  // loader role: row (t % 64) of A and of B, k slots (t / 64) + 4*i
  const int lrow = t & 63, lk = t >> 6;
  const Info ra = p.a.rows(m0 + lrow), rb = p.b.rows(n0 + lrow);
  // compute role: 4x4 micro tile
  const int tm = (t & 15) * 4, tn = (t >> 4) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (long k0 = k_begin; k0 < k_end; k0 += SIMT_BK) {
    if (t < SIMT_BK) {
      const long k = k0 + t;
      Info ka = p.a.ks(k), kb = p.b.ks(k);
      if (k >= k_end) { ka.y = kInvalid; kb.y = kInvalid; }
      kiA[t] = ka;
      kiB[t] = kb;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int kk = lk + 4 * i;
      As[kk][lrow] = p.a.fetch(ra, kiA[kk]);
      Bs[kk][lrow] = p.b.fetch(rb, kiB[kk]);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SIMT_BK; kk++) {
      const float4 a = *reinterpret_cast<const float4 *>(&As[kk][tm]);
      const float4 b = *reinterpret_cast<const float4 *>(&Bs[kk][tn]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const long m = m0 + tm + i;
    if (m >= p.M) continue;
    const long mo = p.ws ? 0 : p.epi.template moff<P::PAIR>(m);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const long n = n0 + tn + j;
      if (n >= p.N) continue;
      if (p.ws) p.ws[((long)blockIdx.z * p.N + n) * p.M + m] = acc[i][j];
      else p.epi.template store<P::PAIR>(mo, n, acc[i][j]);
    }
  }
}

}  // namespace mm
}  // namespace thc

#endif
