// Operand / epilogue descriptions shared by the matrix-multiply engines.
//
// Every GEMM-shaped operation of the library (BLAS gemm behind addmm / Linear, and the three
// SpatialConvolutionMM passes) is stated once as
//
//     D(m, n) = sum_k  A(m, k) * B(n, k)          m < M, n < N, k < K
//
// where an operand element is found by adding a per-row and a per-k memory offset and passing a
// small box test that realises zero padding.  That is the implicit-GEMM form of what the reference
// does by materialising a column matrix per image and calling a generic SGEMM on it
// (gputorch/lib/THC/gpunn-impl/SpatialConvolutionMM.cpp:10-92 im2col / col2im, :185-217 host loop;
// operand mapping in the table of the gemm call sites :194-216, :289-300, :404-417).  The engines
// (mm_simt.cuh: FP32 FMA; mm_tc.cuh: tcgen05 tensor cores with a 3xTF32 split) only see these
// descriptions, so the index rules are written, and tested, exactly once.
#ifndef THC_MM_PROBLEM_CUH
#define THC_MM_PROBLEM_CUH

#include "thc_internal.h"

namespace thc {
namespace mm {

struct Info {
  long off;  // memory offset contribution (floats)
  int y, x;  // box-test coordinates contribution
};
constexpr int kInvalid = -(1 << 29);

// Division of a non-negative 31-bit integer by a runtime constant as multiply-high + shift.
struct FastDiv {
  unsigned d, mul, shr;
  __host__ static FastDiv make(long divisor) {
    FastDiv f;
    f.d = (unsigned)divisor;
    if (divisor <= 1) { f.mul = 0; f.shr = 0; return f; }
    int lg = 0;
    while ((1l << lg) < divisor) lg++;          // ceil(log2 d)
    const int p = 31 + lg;
    f.mul = (unsigned)(((1ull << p) + (unsigned long long)divisor - 1) / (unsigned long long)divisor);
    f.shr = (unsigned)(p - 32);
    return f;
  }
  __device__ __forceinline__ void divmod(unsigned n, unsigned &q, unsigned &r) const {
    q = d > 1 ? (__umulhi(n, mul) >> shr) : n;
    r = n - q * d;
  }
};

// idx -> idx * stride
struct LinearMap {
  static constexpr bool kLinear = true;   // cheap enough to evaluate inline, no staging needed
  long count, stride;
  __device__ __forceinline__ Info operator()(long idx) const {
    Info r;
    r.off = idx * stride;
    r.y = idx < count ? 0 : kInvalid;
    r.x = 0;
    return r;
  }
};

// idx = (img, y, x) over a [count/PP, PP/XW, XW] grid of pixels
struct PixelMap {
  static constexpr bool kLinear = false;
  long count;            // < 2^31 (checked by set())
  FastDiv PP, XW;
  unsigned p_valid;      // pixels of a plane that exist; indices in [p_valid, PP) are padding (zeros)
  long img_stride, y_stride, x_stride, off0;
  int sy, y0, sx, x0;
  void set(long count_, long pp, long xw, long pp_valid = -1) {
    THC_CHECK(count_ < (1l << 31) && pp > 0 && xw > 0, "problem too large for 32-bit pixel indices");
    count = count_; PP = FastDiv::make(pp); XW = FastDiv::make(xw);
    p_valid = (unsigned)(pp_valid < 0 ? pp : pp_valid);
  }
  __device__ __forceinline__ Info operator()(long idx) const {
    Info r;
    if (idx >= count) { r.off = 0; r.y = kInvalid; r.x = 0; return r; }
    unsigned img, p, y, x;
    PP.divmod((unsigned)idx, img, p);
    if (p >= p_valid) { r.off = 0; r.y = kInvalid; r.x = 0; return r; }
    XW.divmod(p, y, x);
    r.off = (long)img * img_stride + (long)y * y_stride + (long)x * x_stride + off0;
    r.y = (int)y * sy + y0;
    r.x = (int)x * sx + x0;
    return r;
  }
};

// idx = (c, i, j) over [count/kHW, kHW/kW, kW] filter taps
struct TapMap {
  static constexpr bool kLinear = false;
  long count;            // < 2^31 (checked by set())
  FastDiv kHW, kW;
  long c_stride, i_stride, j_stride;
  int si, sj;
  void set(long count_, long khw, long kw) {
    THC_CHECK(count_ < (1l << 31) && khw > 0 && kw > 0, "problem too large for 32-bit tap indices");
    count = count_; kHW = FastDiv::make(khw); kW = FastDiv::make(kw);
  }
  __device__ __forceinline__ Info operator()(long idx) const {
    Info r;
    if (idx >= count) { r.off = 0; r.y = kInvalid; r.x = 0; return r; }
    unsigned c, t, i, j;
    kHW.divmod((unsigned)idx, c, t);
    kW.divmod(t, i, j);
    r.off = (long)c * c_stride + (long)i * i_stride + (long)j * j_stride;
    r.y = (int)i * si;
    r.x = (int)j * sj;
    return r;
  }
};

// BOX 0: valid rows/ks only.  BOX 1: additionally 0 <= y < H and 0 <= x < W (zero padding).
// BOX 2: the summed coordinates must be non-negative multiples of (dH, dW) and the quotients index
//        an H x W plane (gradInput of a strided convolution).
template <class RowMap_, class KMap_, int BOX_, bool ALONG_K_>
struct Operand {
  typedef RowMap_ RowMap;
  typedef KMap_ KMap;
  static constexpr int BOX = BOX_;
  static constexpr bool ALONG_K = ALONG_K_;  // memory is contiguous along k (else along rows)
  // plain matrices whose k runs are contiguous can be read 16 bytes at a time when vec4 is set
  static constexpr bool VECTORIZABLE = ALONG_K_ && BOX_ == 0 && RowMap_::kLinear && KMap_::kLinear;
  static constexpr bool PRESPLIT = false;
  const float *base;
  RowMap rows;
  KMap ks;
  int H, W, dH, dW;
  int vec4;  // host promise: base 16-byte aligned, row stride a multiple of 4 floats, k stride 1
  // Where element (r, k) lives, or nullptr when it is a structural zero (padding / out of range).
  __device__ __forceinline__ const float *locate(const Info &r, const Info &k) const {
    const int ty = r.y + k.y, tx = r.x + k.x;
    if (BOX == 0) return ty >= 0 ? base + (r.off + k.off) : nullptr;
    if (BOX == 1)
      return ((unsigned)ty < (unsigned)H && (unsigned)tx < (unsigned)W) ? base + (r.off + k.off) : nullptr;
    if (ty < 0 || tx < 0) return nullptr;
    const int y = ty / dH, x = tx / dW;
    if (y * dH != ty || x * dW != tx || y >= H || x >= W) return nullptr;
    return base + (r.off + k.off + (long)y * W + x);
  }
  __device__ __forceinline__ float fetch(const Info &r, const Info &k) const {
    const int ty = r.y + k.y, tx = r.x + k.x;
    if (BOX == 0) return ty >= 0 ? base[r.off + k.off] : 0.f;
    if (BOX == 1)
      return ((unsigned)ty < (unsigned)H && (unsigned)tx < (unsigned)W) ? base[r.off + k.off] : 0.f;
    if (ty < 0 || tx < 0) return 0.f;
    const int y = ty / dH, x = tx / dW;
    if (y * dH != ty || x * dW != tx || y >= H || x >= W) return 0.f;
    return base[r.off + k.off + (long)y * W + x];
  }
};

// A plain matrix that a preparation pass (split_planes_kernel) has already rounded into two K-major
// planes of TF32 values, hi and lo = tf32(x - hi), each [rows][ld] with ld a multiple of 32 floats
// and zeros beyond the real K.  The tensor-core engine copies both planes straight into their tiles
// (16-byte cp.async, no per-element work in the main loop).
struct SplitOperand {
  typedef LinearMap RowMap;
  typedef LinearMap KMap;
  static constexpr int BOX = 0;
  static constexpr bool ALONG_K = true;
  static constexpr bool VECTORIZABLE = true;
  static constexpr bool PRESPLIT = true;
  const float *base;  // hi plane
  const float *lo;    // lo plane
  RowMap rows;        // {row count, ld}
  KMap ks;            // {ld, 1}
  int H, W, dH, dW, vec4;
  // optional second level along k: k = outer * k_inner + inner lives at outer * k_outer_stride + inner
  // (k_inner a multiple of 32, so a k tile never straddles two outer blocks); k_inner.d == 0: plain
  FastDiv k_inner;
  long k_outer_stride;
  __device__ __forceinline__ long ktile_off(long k0) const {
    if (k_inner.d == 0) return k0;
    unsigned q, r;
    k_inner.divmod((unsigned)k0, q, r);
    return (long)q * k_outer_stride + r;
  }
  __device__ __forceinline__ float fetch(const Info &r, const Info &k) const {
    return (r.y | k.y) >= 0 ? base[r.off + k.off] + lo[r.off + k.off] : 0.f;
  }
  __device__ __forceinline__ const float *locate(const Info &r, const Info &k) const {
    return (r.y | k.y) >= 0 ? base + (r.off + k.off) : nullptr;
  }
};

// hi/lo planes of a strided matrix: element (r, k) at src[r*rs + k*ks]; out planes [rows][ld], zero for k >= K.
// 32x32 tiles through shared memory so that reads are coalesced along whichever source dimension is
// contiguous and writes are coalesced along k.
static __global__ void __launch_bounds__(256) split_planes_kernel(const float *__restrict__ src, long rs, long ks, long rows,
                                                                  long K, float *__restrict__ hi, float *__restrict__ lo,
                                                                  long ld) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long tiles_k = ld / 32;
  const long ntiles = ((rows + 31) / 32) * tiles_k;
  for (long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long r0 = (t / tiles_k) * 32, k0 = (t % tiles_k) * 32;
    if (rs == 1 && ks != 1) {  // contiguous along rows: read transposed
#pragma unroll
      for (int j = ty; j < 32; j += 8) {
        const long r = r0 + tx, k = k0 + j;
        tile[tx][j] = (r < rows && k < K) ? src[r + k * ks] : 0.f;
      }
    } else {
#pragma unroll
      for (int j = ty; j < 32; j += 8) {
        const long r = r0 + j, k = k0 + tx;
        tile[j][tx] = (r < rows && k < K) ? src[r * rs + k * ks] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
      const long r = r0 + j;
      if (r < rows) {
        const float x = tile[j][tx];
        unsigned h;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
        const float xl = x - __uint_as_float(h);
        unsigned l;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(xl));
        hi[r * ld + k0 + tx] = __uint_as_float(h);
        lo[r * ld + k0 + tx] = __uint_as_float(l);
      }
    }
    __syncthreads();
  }
}

// out[(m / mdiv) * mouter + (m % mdiv) + n * nstride] = alpha*acc (+ bias[n]) (+ beta*old)
struct Epilogue {
  float *out;
  const float *bias;
  float alpha, beta;
  long mdiv, mouter, nstride;
  __device__ __forceinline__ long moff(long m) const {
    const long q = m / mdiv;
    return q * mouter + (m - q * mdiv);
  }
  __device__ __forceinline__ void store(long mo, long n, float acc) const {
    const long o = mo + n * nstride;
    float v = alpha * acc;
    if (bias) v += bias[n];
    if (beta != 0.f) v += beta * out[o];
    out[o] = v;
  }
};

template <class OpA_, class OpB_>
struct Problem {
  typedef OpA_ OpA;
  typedef OpB_ OpB;
  OpA a;
  OpB b;
  Epilogue epi;
  long M, N, K;
  // split-K: gridDim.z slices of k_per_split (a multiple of the engine's k tile); partial sums go
  // to ws[z][n][m] and a second kernel folds them in slice order and applies the epilogue.
  long k_per_split;
  float *ws;
};

// Folds split-K partials (fixed order -> deterministic) and applies the epilogue.
static __global__ void __launch_bounds__(256) splitk_finish_kernel(const float *__restrict__ ws, int splits, long M, long N,
                                                            Epilogue epi) {
  const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= M * N) return;
  const long n = t / M, m = t - n * M;
  float acc = 0.f;
  for (int z = 0; z < splits; z++) acc += ws[((long)z * N + n) * M + m];
  epi.store(epi.moff(m), n, acc);
}

}  // namespace mm
}  // namespace thc

#endif
