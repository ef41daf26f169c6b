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

#include <cuda.h>
#include <cuda_bf16.h>

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
  static constexpr bool MN_MAJOR = false;
  static constexpr bool TMA_CAPABLE = false;
  static constexpr bool TMA_IM2COL = false;
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
  static constexpr bool MN_MAJOR = false;
  static constexpr bool TMA_CAPABLE = false;
  static constexpr bool TMA_IM2COL = false;
  const float *base;  // hi plane (BF16 mode: one plane of BF16 values, offsets then count 4-byte units)
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
  // what 16-byte chunk `chunk` of the 32-k tile starting at k0 adds to a row's offset / box coordinates
  __device__ __forceinline__ Info ktile(long k0, int chunk) const {
    Info t;
    t.off = ktile_off(k0) + chunk * 4; t.y = 0; t.x = 0;
    return t;
  }
  __device__ __forceinline__ bool valid(const Info &r, const Info &) const { return r.y >= 0; }
  __device__ __forceinline__ float fetch(const Info &r, const Info &k) const {
    return (r.y | k.y) >= 0 ? base[r.off + k.off] + lo[r.off + k.off] : 0.f;
  }
  __device__ __forceinline__ const float *locate(const Info &r, const Info &k) const {
    return (r.y | k.y) >= 0 ? base + (r.off + k.off) : nullptr;
  }
};


// ---------------------------------------------------------------------------------------------
// Channels-last hi / lo planes of an activation tensor: P[img][y][x][c], c contiguous and padded with zero
// planes to a multiple of 4, every value already rounded to TF32 (hi) and tf32(x - hi) (lo) by
// nchw_to_planes_kernel.  With channels innermost, a 16-byte chunk of the implicit column matrix is ONE
// filter tap and 4 consecutive channels, so the tensor-core engine fills its tiles with 16-byte copies
// and one box test per (pixel, chunk) instead of per element; with 32 or more channels a whole 32-k tile
// (128 contiguous bytes per pixel) belongs to one tap.  Tensor-core engine only (no fetch()).
//
// Window view (K-major): row = pixel (img, y, x) of the product's output grid, k = (i, j, c); K is
// taps * C rounded up to 32, the tail reads as zero.
struct PlanesWindowOperand {
  typedef PixelMap RowMap;
  typedef LinearMap KMap;   // unused; k chunks are decoded by ktile()
  static constexpr int BOX = 1;
  static constexpr bool ALONG_K = true;
  static constexpr bool VECTORIZABLE = true;
  static constexpr bool PRESPLIT = true;
  static constexpr bool MN_MAJOR = false;
  static constexpr bool TMA_CAPABLE = true;
  static constexpr bool TMA_IM2COL = true;
  // When use_tma is set (one FP32 plane, raw-operand engine), tmap is an im2col tensor map over the plane seen
  // as a channels-last tensor {C, W, H, n_img}: 32 channels of 128 consecutive windows per load, the 128-byte
  // swizzle of the operand tiles, padding read as zeros: one TMA load per k tile (one tap, 32 channels).
  CUtensorMap tmap;
  int use_tma;
  int n_img;                // images per plane
  int n_planes;             // 2: hi / lo planes; 1: one plane of FP32 values (raw-operand engine)
  FastDiv ctiles;           // C / 32 (TMA form only)
  const float *base, *lo;
  RowMap rows;              // off = plane offset of the window's top-left pixel, (y, x) = its coordinates
  KMap ks;
  int H, W, dH, dW, vec4;   // H x W: the plane's pixel grid (box test)
  FastDiv cquads;           // C / 4
  FastDiv kW;
  unsigned taps;            // kH * kW
  long i_stride, j_stride;  // W*C, C
  // Window corner (x, y) and image of row m, the start coordinates of an im2col load; rows past the end map
  // beyond the last image, where every read is out of bounds (zeros).
  __device__ __forceinline__ void tile_origin(long m, int &x, int &y, int &img) const {
    if (m >= rows.count) { x = rows.x0; y = rows.y0; img = n_planes * n_img; return; }
    unsigned im, px, yy, xx;
    rows.PP.divmod((unsigned)m, im, px);
    rows.XW.divmod(px, yy, xx);
    x = (int)xx * rows.sx + rows.x0;
    y = (int)yy * rows.sy + rows.y0;
    img = (int)im;
  }
  // Tap (i, j) and first channel of the k tile starting at k0.
  __device__ __forceinline__ void tile_tap(long k0, int &i, int &j, int &c0) const {
    unsigned tap, cb, ii, jj;
    ctiles.divmod((unsigned)(k0 >> 5), tap, cb);
    kW.divmod(tap, ii, jj);
    i = (int)ii; j = (int)jj; c0 = (int)cb * 32;
  }
  __device__ __forceinline__ Info ktile(long k0, int chunk) const {
    unsigned tap, cq, i, j;
    cquads.divmod((unsigned)(k0 >> 2) + (unsigned)chunk, tap, cq);
    kW.divmod(tap, i, j);
    Info t;
    t.off = (long)i * i_stride + (long)j * j_stride + (long)cq * 4;
    t.y = tap < taps ? (int)i : kInvalid;
    t.x = (int)j;
    return t;
  }
  __device__ __forceinline__ bool valid(const Info &r, const Info &t) const {
    return (unsigned)(r.y + t.y) < (unsigned)H && (unsigned)(r.x + t.x) < (unsigned)W;
  }
};

// A plain FP32 matrix read by TMA alone (raw-operand engine, mm_tc2r.cuh): K-major (memory runs along k) or
// MN-major (memory runs along the rows).  tmap: K-major {K, rows} with a {32 k, tile rows} box and the 128-byte
// swizzle; MN-major {rows, K} with a {32 rows, 32 k} box per 32-row block and the 32-byte-granule swizzle.
// Elements beyond either extent read as zeros.
template <bool MN_>
struct RawOperand {
  static constexpr bool PRESPLIT = true;
  static constexpr bool MN_MAJOR = MN_;
  static constexpr bool TMA_CAPABLE = true;
  static constexpr bool TMA_IM2COL = false;
  CUtensorMap tmap;
  int use_tma;
};

// Input windows of a convolution as the MN-major operand of the weight-gradient product, read by TMA alone
// (raw-operand engine): rows = (tap, c) of one channels-last FP32 plane [n_img][H][W][C], C % 32 == 0,
// k = output pixels.  tmap: im2col map {C, W, H, n_img}, 32 channels of 32 consecutive windows per load (one
// 32-row block of a k tile), the 32-byte-granule swizzle.
struct WindowRowsOperand {
  static constexpr bool PRESPLIT = true;
  static constexpr bool MN_MAJOR = true;
  static constexpr bool TMA_CAPABLE = true;
  static constexpr bool TMA_IM2COL = false;
  CUtensorMap tmap;
  int use_tma;
  int n_img;
  PixelMap ks;              // output pixel -> window corner
  FastDiv C, kW;
  __device__ __forceinline__ void pixel_origin(long k, int &x, int &y, int &img) const {
    if (k >= ks.count) { x = ks.x0; y = ks.y0; img = n_img; return; }
    unsigned im, px, yy, xx;
    ks.PP.divmod((unsigned)k, im, px);
    ks.XW.divmod(px, yy, xx);
    x = (int)xx * ks.sx + ks.x0;
    y = (int)yy * ks.sy + ks.y0;
    img = (int)im;
  }
  __device__ __forceinline__ void row_tap(long r, int &i, int &j, int &c0) const {
    unsigned tap, c, ii, jj;
    C.divmod((unsigned)r, tap, c);
    kW.divmod(tap, ii, jj);
    i = (int)ii; j = (int)jj; c0 = (int)c;
  }
};

// A pixel map cheap enough for every thread to evaluate for itself once per stage.
struct InlinePixelMap : PixelMap {
  static constexpr bool kLinear = true;
};

// Pixel view (MN-major): k = pixel (img, y, x) of the reduction grid, row = (tap, c) (TAPS) or just c.
// Memory runs along the rows, which tcgen05 reads as an "MN-major" operand: the tile is stored as
// [32-channel block][32 pixels][128 bytes] and the instruction descriptor carries the transpose bit.
// This is the weight-gradient form: both gradOutput and the input windows are reduced over pixels.
template <bool TAPS_>
struct PlanesPixelOperand {
  typedef LinearMap RowMap;
  typedef InlinePixelMap KMap;
  static constexpr int BOX = 1;
  static constexpr bool ALONG_K = false;
  static constexpr bool VECTORIZABLE = true;
  static constexpr bool PRESPLIT = true;
  static constexpr bool MN_MAJOR = true;
  static constexpr bool TMA_CAPABLE = false;
  static constexpr bool TMA_IM2COL = false;
  static constexpr bool TAPS = TAPS_;
  const float *base, *lo;
  RowMap rows;              // {row count, 1}
  KMap ks;                  // pixel -> plane offset of the window's top-left pixel + its coordinates
  int H, W, dH, dW, vec4;
  FastDiv C;                // channels per tap (rows = taps * C)
  FastDiv kW;
  long i_stride, j_stride;
  __device__ __forceinline__ Info rowblock(long r0) const {   // 4-row chunk starting at r0 (never straddles a tap)
    Info t;
    if (!TAPS) { t.off = r0; t.y = 0; t.x = 0; return t; }
    unsigned tap, c, i, j;
    C.divmod((unsigned)r0, tap, c);
    kW.divmod(tap, i, j);
    t.off = (long)i * i_stride + (long)j * j_stride + (long)c;
    t.y = (int)i; t.x = (int)j;
    return t;
  }
  __device__ __forceinline__ bool valid(const Info &px, const Info &t) const {
    return (unsigned)(px.y + t.y) < (unsigned)H && (unsigned)(px.x + t.x) < (unsigned)W;
  }
};

// NCHW fp32 -> channels-last hi / lo planes.  One 32-channel x 32-pixel tile per step through shared
// memory: reads coalesced along pixels, writes coalesced along channels.  C % 32 == 0.
// `chan_partial` (optional): [gridDim.x][C] sums over the pixels this block transposed, per channel -- the gradBias
// reduction of a convolution rides on the transposition of gradOutput instead of reading the tensor a second time.
// A channel of a tile belongs to one warp, tiles are taken in a fixed order, so the sums are reproducible.
static __global__ void __launch_bounds__(256) nchw_to_planes_kernel(const float *__restrict__ src, long N, long C, long HW,
                                                                    float *__restrict__ hi, float *__restrict__ lo,
                                                                    float *__restrict__ chan_partial) {
  // 32 channels x 128 pixels per pass: sixteen loads per thread in flight before the barrier (32 x 32 tiles with
  // four left the kernel at half the HBM rate)
  constexpr int PT = 128;
  __shared__ float tile[32][PT + 1];
  extern __shared__ float chan_sum[];   // [C] when chan_partial is given
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long ptiles = (HW + PT - 1) / PT, ctiles = C / 32;
  const long ntiles = N * ptiles * ctiles;
  if (chan_partial) {
    for (long c = threadIdx.x; c < C; c += blockDim.x) chan_sum[c] = 0.f;
    __syncthreads();
  }
  for (long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long pt = t % ptiles, q = t / ptiles, ct = q % ctiles, img = q / ctiles;
    const long p0 = pt * PT, c0 = ct * 32;
    const float *s = src + (img * C + c0) * HW + p0;
    const int np = HW - p0 < PT ? (int)(HW - p0) : PT;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
      float part = 0.f;
#pragma unroll
      for (int g = 0; g < PT; g += 32) {
        const float v = (g + tx < np) ? s[(long)j * HW + g + tx] : 0.f;
        tile[j][g + tx] = v;
        part += v;
      }
      if (chan_partial) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (tx == 0) chan_sum[c0 + j] += part;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int j = ty; j < np; j += 8) {
      const float x = tile[tx][j];
      const long o = (img * HW + p0 + j) * C + c0 + tx;
      if (lo) {
        unsigned h, l;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
        const float xl = x - __uint_as_float(h);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(xl));
        hi[o] = __uint_as_float(h); lo[o] = __uint_as_float(l);
      } else {
        hi[o] = x;   // one plane of plain FP32 values (raw-operand engine)
      }
    }
    __syncthreads();
  }
  if (chan_partial)
    for (long c = threadIdx.x; c < C; c += blockDim.x) chan_partial[(long)blockIdx.x * C + c] = chan_sum[c];
}
// out[c] += scale * sum_b partial[b][c]: 32 row slices per channel (one warp each, eight loads in flight per
// thread), folded in a fixed order.  The partials are a few MB at most; what this kernel costs is the chain of
// dependent loads per thread, hence the wide block.
static __global__ void __launch_bounds__(1024) chan_partial_finish_kernel(const float *__restrict__ partial, int nblocks, long C,
                                                                          float *out, float scale) {
  __shared__ float sm[32][33];
  const int lane = threadIdx.x & 31, s = threadIdx.x >> 5;
  const long c = (long)blockIdx.x * 32 + lane;
  float a[8];
#pragma unroll
  for (int i = 0; i < 8; i++) a[i] = 0.f;
  if (c < C) {
    int b = s;
    for (; b + 7 * 32 < nblocks; b += 8 * 32) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = partial[(long)(b + 32 * i) * C + c];
#pragma unroll
      for (int i = 0; i < 8; i++) a[i] += v[i];
    }
    for (; b < nblocks; b += 32) a[0] += partial[(long)b * C + c];
  }
  const float a0 = a[0] + a[4], a1 = a[1] + a[5], a2 = a[2] + a[6], a3 = a[3] + a[7];
  sm[s][lane] = (a0 + a1) + (a2 + a3);
  __syncthreads();
  if (s == 0 && c < C) {
    float acc = 0.f;
    for (int k = 0; k < 32; k++) acc += sm[k][lane];
    out[c] += scale * acc;
  }
}

// The same for channel counts that are not multiples of 32: one thread per pixel walks the planes (reads
// coalesced across threads) and writes its pixel's Cp = round_up(C, 4) channels 16 bytes at a time.
static __global__ void __launch_bounds__(256) nchw_to_planes_any_kernel(const float *__restrict__ src, long N, long C, long HW,
                                                                        long Cp, float *__restrict__ hi, float *__restrict__ lo) {
  const long total = N * HW;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const long img = t / HW, px = t - img * HW;
    const float *s = src + img * C * HW + px;
    for (long c0 = 0; c0 < Cp; c0 += 4) {
      float h[4], l[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float x = c0 + e < C ? s[(c0 + e) * HW] : 0.f;
        unsigned hh, ll;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hh) : "f"(x));
        const float xl = x - __uint_as_float(hh);
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(ll) : "f"(xl));
        h[e] = lo ? __uint_as_float(hh) : x; l[e] = __uint_as_float(ll);
      }
      *reinterpret_cast<float4 *>(hi + t * Cp + c0) = make_float4(h[0], h[1], h[2], h[3]);
      if (lo) *reinterpret_cast<float4 *>(lo + t * Cp + c0) = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
}

// Weight matrix W[ko][(c, tap)] -> hi / lo planes in the k order of the planes operands, channel counts
// padded to multiples of 4 (Cp, Kp) and rows to `ld` floats (a multiple of 32); padding is zero.
//   flip == 0: out[ko][(tap, c)],          rows = K, row length taps * Cp   (forward: k = (i, j, c))
//   flip == 1: out[c][(kHW-1-tap, ko)],    rows = C, row length taps * Kp   (gradInput as a forward pass over
//              gradOutput with the filter rotated by 180 degrees: k = (i', j', ko))
// pair_shift > 0 (pixel-pair mode, see Epilogue): the filter is widened to kWe = kW + pair_shift columns and
// stored twice, rows [0, rows) as it is (output parity 0) and rows [rows, 2 rows) shifted right by pair_shift
// columns (parity 1, whose window starts one stride later); the new columns are zero.
static __global__ void __launch_bounds__(256) repack_weight_planes_kernel(const float *__restrict__ w, long K, long C, long kHW,
                                                                          long Cp, long Kp, long ld, int flip, int kW,
                                                                          int pair_shift, float *__restrict__ hi,
                                                                          float *__restrict__ lo) {
  const long rows = flip ? C : K;
  const long total = (pair_shift ? 2 : 1) * rows * ld;
  const long nthreads = (long)gridDim.x * blockDim.x;
  const long chans = flip ? Kp : Cp;
  const long kWe = kW + pair_shift, kH = kHW / kW;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    long r = t / ld;
    const long k = t - r * ld;
    const long par = r >= rows ? 1 : 0;
    r -= par * rows;
    const long tape = k / chans, ch = k - tape * chans;       // tap in the widened filter
    const long i = tape / kWe, j = tape - i * kWe - par * pair_shift;
    float x = 0.f;
    if (i < kH && j >= 0 && j < kW) {
      const long tap = i * kW + j;
      if (!flip) { if (ch < C) x = w[(r * C + ch) * kHW + tap]; }
      else if (ch < K) x = w[(ch * C + r) * kHW + (kHW - 1 - tap)];
    }
    unsigned h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    const float xl = x - __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(xl));
    if (lo) { hi[t] = __uint_as_float(h); lo[t] = __uint_as_float(l); }
    else hi[t] = x;
  }
}

// gradW[ko][(c, tap)] += scale * tmp[ko][(tap, c)], tmp rows of length kHW * Cp (channels padded to Cp)
static __global__ void __launch_bounds__(256) unpack_grad_weight_kernel(const float *__restrict__ tmp, float *__restrict__ gw,
                                                                        long K, long C, long kHW, long Cp, float scale) {
  const long total = K * C * kHW;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const long tap = t % kHW, q = t / kHW, c = q % C, ko = q / C;
    gw[t] += scale * tmp[(ko * kHW + tap) * Cp + c];
  }
}


// ---------------------------------------------------------------------------------------------
// BF16 planes (math mode 2): the same layouts with one plane of BF16 values; rows are padded so that a row
// is a whole number of 16-byte chunks (8 values), k extents to 64 values.
//
// NCHW fp32 -> channels-last BF16 plane [N * HW][Cp], Cp a multiple of 8.  One thread per pixel.
static __global__ void __launch_bounds__(256) nchw_to_planes_bf16_kernel(const float *__restrict__ src, long N, long C, long HW,
                                                                         long Cp, __nv_bfloat16 *__restrict__ out) {
  const long total = N * HW;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const long img = t / HW, px = t - img * HW;
    const float *s = src + img * C * HW + px;
    for (long c0 = 0; c0 < Cp; c0 += 8) {
      __align__(16) __nv_bfloat16 v[8];
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] = __float2bfloat16(c0 + e < C ? s[(c0 + e) * HW] : 0.f);
      *reinterpret_cast<uint4 *>(out + t * Cp + c0) = *reinterpret_cast<const uint4 *>(v);
    }
  }
}
// The same for C % 32 == 0 through 32 x 32 shared-memory tiles (reads coalesced along pixels, writes along channels).
static __global__ void __launch_bounds__(256) nchw_to_planes_bf16_tiled_kernel(const float *__restrict__ src, long N, long C,
                                                                               long HW, __nv_bfloat16 *__restrict__ out) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long ptiles = (HW + 31) / 32, ctiles = C / 32;
  const long ntiles = N * ptiles * ctiles;
  for (long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long pt = t % ptiles, q = t / ptiles, ct = q % ctiles, img = q / ctiles;
    const long p0 = pt * 32, c0 = ct * 32;
    const float *s = src + (img * C + c0) * HW + p0;
#pragma unroll
    for (int j = ty; j < 32; j += 8) tile[j][tx] = (p0 + tx < HW) ? s[(long)j * HW + tx] : 0.f;
    __syncthreads();
    // thread (pixel row j, channel pair tx % 16): two passes of 16 pixel rows
#pragma unroll
    for (int j = ty * 2 + (tx >> 4); j < 32; j += 16) {
      if (p0 + j < HW) {
        const int cp = (tx & 15) * 2;
        const __nv_bfloat162 v = __floats2bfloat162_rn(tile[cp][j], tile[cp + 1][j]);
        *reinterpret_cast<__nv_bfloat162 *>(out + (img * HW + p0 + j) * C + c0 + cp) = v;
      }
    }
    __syncthreads();
  }
}
// BF16 plane of a strided matrix: element (r, k) at src[r*rs + k*ks]; out [rows][ld], zero for k >= K.
static __global__ void __launch_bounds__(256) bf16_rows_kernel(const float *__restrict__ src, long rs, long ks, long rows, long K,
                                                               __nv_bfloat16 *__restrict__ out, long ld) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long tiles_k = ld / 32;
  const long ntiles = ((rows + 31) / 32) * tiles_k;
  for (long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long r0 = (t / tiles_k) * 32, k0 = (t % tiles_k) * 32;
    if (rs == 1 && ks != 1) {
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
      if (r < rows) out[r * ld + k0 + tx] = __float2bfloat16(tile[j][tx]);
    }
    __syncthreads();
  }
}
// Weight matrix -> one BF16 plane in the k order of the planes operands (see repack_weight_planes_kernel).
static __global__ void __launch_bounds__(256) repack_weight_bf16_kernel(const float *__restrict__ w, long K, long C, long kHW,
                                                                        long Cp, long Kp, long ld, int flip,
                                                                        __nv_bfloat16 *__restrict__ out) {
  const long rows = flip ? C : K;
  const long total = rows * ld;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const long r = t / ld, k = t - r * ld;
    float x = 0.f;
    if (!flip) {
      const long tap = k / Cp, c = k - tap * Cp;
      if (tap < kHW && c < C) x = w[(r * C + c) * kHW + tap];
    } else {
      const long tapf = k / Kp, ko = k - tapf * Kp;
      if (tapf < kHW && ko < K) x = w[(ko * C + r) * kHW + (kHW - 1 - tapf)];
    }
    out[t] = __float2bfloat16(x);
  }
}
// gradW[ko][(c, tap)] += scale * tmp[...] is shared with the FP32 path (tmp is FP32 in both modes).

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
  // Pixel-pair mode (pair_K > 0, beta == 0): a convolution with few output planes computes two horizontally
  // adjacent output pixels per row so that its tile is twice as wide.  Row m = (img, y, x2), column
  // n = (parity, plane): out[img * pair_img + plane * nstride + y * pair_oW + 2 * x2 + parity]; with an odd
  // output width the last pair of a row has no parity-1 pixel.
  long pair_K = 0, pair_oH = 1, pair_oW2 = 1, pair_oW = 0, pair_img = 0;
  static constexpr long kLastOdd = 1l << 62;
  // PAIR is a compile-time property of the problem: the common path carries none of the pair arithmetic
  template <bool PAIR = false>
  __device__ __forceinline__ long moff(long m) const {
    if (PAIR) {
      const long r = m / pair_oW2, x2 = m - r * pair_oW2, img = r / pair_oH, y = r - img * pair_oH;
      return (img * pair_img + y * pair_oW + 2 * x2) | (2 * x2 + 1 >= pair_oW ? kLastOdd : 0);
    }
    const long q = m / mdiv;
    return q * mouter + (m - q * mdiv);
  }
  // the same with the destination's previous value already in a register (never in pixel-pair mode)
  __device__ __forceinline__ void store_with(long mo, long n, float acc, float old) const {
    float v = alpha * acc;
    if (bias) v += bias[n];
    v += beta * old;
    out[mo + n * nstride] = v;
  }
  // beta == 0 with the bias fetched by the caller (several columns' bias values at once, ahead of the stores: a
  // load per column between the stores would serialise them, the compiler cannot move it across a store)
  template <bool PAIR = false>
  __device__ __forceinline__ float bias_of(long n) const {
    if (!bias) return 0.f;
    return __ldg(bias + (PAIR && n >= pair_K ? n - pair_K : n));
  }
  template <bool PAIR = false>
  __device__ __forceinline__ void store_biased(long mo, long n, float acc, float b) const {
    const float v = alpha * acc + b;
    if (PAIR) {
      const long par = n >= pair_K ? 1 : 0, plane = n - par * pair_K;
      if (par && (mo & kLastOdd)) return;
      out[(mo & ~kLastOdd) + plane * nstride + par] = v;
      return;
    }
    out[mo + n * nstride] = v;
  }
  template <bool PAIR = false>
  __device__ __forceinline__ void store(long mo, long n, float acc) const {
    if (PAIR) {
      const long par = n >= pair_K ? 1 : 0, plane = n - par * pair_K;
      if (par && (mo & kLastOdd)) return;
      float v = alpha * acc;
      if (bias) v += bias[plane];
      out[(mo & ~kLastOdd) + plane * nstride + par] = v;
      return;
    }
    const long o = mo + n * nstride;
    float v = alpha * acc;
    if (bias) v += bias[n];
    if (beta != 0.f) v += beta * out[o];
    out[o] = v;
  }
};

template <class OpA_, class OpB_, bool PAIR_ = false>
struct Problem {
  typedef OpA_ OpA;
  typedef OpB_ OpB;
  static constexpr bool PAIR = PAIR_;   // pixel-pair epilogue (see Epilogue)
  OpA a;
  OpB b;
  Epilogue epi;
  long M, N, K;
  // split-K: gridDim.z slices of k_per_split (a multiple of the engine's k tile); partial sums go
  // to ws[z][n][m] and a second kernel folds them in slice order and applies the epilogue.
  long k_per_split;
  float *ws;
  // The persistent raw-operand engine splits only the tiles of its last, partly filled round: tiles (m fastest)
  // from tail_first on are cut into tail_splits slices of k_per_split, whose partial sums go to
  // ws[(tile - tail_first) * tail_splits + z][column of the tile][row of the tile] (256 rows); tail_finish_kernel
  // folds them.  Tiles before tail_first run over the whole reduction and store their results themselves.
  long tail_first = 0;
  int tail_splits = 1;
};

// Epilogue of one drain thread: its row m of the tile, NCOL columns from nb on (split-K partials go to the
// workspace instead).
template <class P, int NCOL>
__device__ __forceinline__ void tc2_store_rows(const P &p, const float (&acc)[NCOL], long m, long nb, long z = -1,
                                               bool direct = false) {
  if constexpr (!P::PAIR) {
    // Plain accumulation into a destination whose ROWS are neighbours in memory (column-major gradWeight of a Linear
    // layer: out[m + n * nstride]): 16-byte reductions at the L2.  A thread holds one row and NCOL columns, a 16-byte
    // reduction wants four consecutive rows of one column, so the four lanes of a quad transpose each 4 x 4 block
    // through two rounds of shuffles (every lane of the warp takes part, also those whose row lies past M).  A
    // quarter of the memory-side operations of the per-element form below, which is what bounds a weight gradient
    // with a short reduction.
    const bool to_out = !(p.ws && !direct);
    if (to_out && p.epi.beta == 1.f && !p.epi.bias && p.epi.mdiv >= p.M && (p.epi.nstride & 3) == 0 &&
        nb + NCOL <= p.N && (reinterpret_cast<uintptr_t>(p.epi.out) & 15) == 0) {
      const unsigned full = 0xffffffffu;
      const int i = threadIdx.x & 3;
      const bool b0 = i & 1, b1 = i & 2;
      const long m0 = m - i;                       // first row of this quad; the warp's first row is a multiple of 32
      const bool whole = m0 + 3 < p.M;
      const float alpha = p.epi.alpha;
      const long st = p.epi.nstride;
      float *quad = p.epi.out + m0 + (nb + i) * st;   // (row m0, column nb + i); moff(m) = m since mdiv >= M
#pragma unroll
      for (int c0 = 0; c0 < NCOL; c0 += 4) {
        float a0 = alpha * acc[c0], a1 = alpha * acc[c0 + 1], a2 = alpha * acc[c0 + 2], a3 = alpha * acc[c0 + 3];
        float s0 = b0 ? a0 : a1, s1 = b0 ? a2 : a3;
        float r0 = __shfl_xor_sync(full, s0, 1), r1 = __shfl_xor_sync(full, s1, 1);
        if (b0) { a0 = r0; a2 = r1; } else { a1 = r0; a3 = r1; }
        s0 = b1 ? a0 : a2; s1 = b1 ? a1 : a3;
        r0 = __shfl_xor_sync(full, s0, 2); r1 = __shfl_xor_sync(full, s1, 2);
        if (b1) { a0 = r0; a1 = r1; } else { a2 = r0; a3 = r1; }
        // a_r = alpha * D(row m0 + r, column nb + c0 + i)
        float *dst = quad + (long)c0 * st;
        if (whole) {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a0), "f"(a1), "f"(a2), "f"(a3) : "memory");
        } else {
          if (m0 < p.M) atomicAdd(dst, a0);
          if (m0 + 1 < p.M) atomicAdd(dst + 1, a1);
          if (m0 + 2 < p.M) atomicAdd(dst + 2, a2);
        }
      }
      return;
    }
  }
  if (m >= p.M) return;
  if (z < 0) z = blockIdx.z;   // split-K slice: the launch's z index unless the (persistent) caller names it
  const bool to_ws = p.ws && !direct;   // `direct`: a whole-reduction tile of a launch that splits only its tail
  const long mo = to_ws ? 0 : p.epi.template moff<P::PAIR>(m);
  if (to_ws) {
#pragma unroll
    for (int j = 0; j < NCOL; j++)
      if (nb + j < p.N) p.ws[(z * p.N + nb + j) * p.M + m] = acc[j];
  } else if (!P::PAIR && p.epi.nstride == 1 && nb + NCOL <= p.N &&
             ((reinterpret_cast<uintptr_t>(p.epi.out + mo + nb) & 15) == 0)) {
    // Row-major destination (the columns of a row are neighbours in memory) and this thread's NCOL columns start on
    // a 16-byte boundary: 16-byte loads and stores.  Neighbouring lanes are a whole row apart, so every access of a
    // warp touches 32 lines whatever its width; four columns per access instead of one cuts the number of those
    // accesses by four, which is what a product with a short reduction (an outer-product-like weight gradient)
    // spends its time on.
    float4 *o = reinterpret_cast<float4 *>(p.epi.out + mo + nb);
    const float alpha = p.epi.alpha, beta = p.epi.beta;
    const float *bias = p.epi.bias;
#pragma unroll
    for (int j0 = 0; j0 < NCOL; j0 += 16) {
      float4 old[4];
      float b[16];
      if (beta != 0.f) {
#pragma unroll
        for (int q = 0; q < 4; q++) old[q] = o[j0 / 4 + q];
      }
#pragma unroll
      for (int j = 0; j < 16; j++) b[j] = bias ? __ldg(bias + nb + j0 + j) : 0.f;
#pragma unroll
      for (int q = 0; q < 4; q++) {
        float4 v;
        v.x = alpha * acc[j0 + 4 * q + 0] + b[4 * q + 0];
        v.y = alpha * acc[j0 + 4 * q + 1] + b[4 * q + 1];
        v.z = alpha * acc[j0 + 4 * q + 2] + b[4 * q + 2];
        v.w = alpha * acc[j0 + 4 * q + 3] + b[4 * q + 3];
        if (beta != 0.f) {
          v.x += beta * old[q].x; v.y += beta * old[q].y; v.z += beta * old[q].z; v.w += beta * old[q].w;
        }
        o[j0 / 4 + q] = v;
      }
    }
  } else if (p.epi.beta == 0.f) {
    // Measured on the two-SM GEMM: this plain form (one pointer, a constant stride, bias values fetched ahead of
    // the stores) takes 4.7 k cycles for a 128 x 256 tile where a per-column call of Epilogue::store took 23 k.
    const float alpha = p.epi.alpha;
    if (!P::PAIR && nb + NCOL <= p.N) {
      float *o = p.epi.out + mo + nb * p.epi.nstride;
      const long st = p.epi.nstride;
      const float *bias = p.epi.bias;
#pragma unroll
      for (int j0 = 0; j0 < NCOL; j0 += 16) {
        float b[16];
#pragma unroll
        for (int j = 0; j < 16; j++) b[j] = bias ? __ldg(bias + nb + j0 + j) : 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++) o[(j0 + j) * st] = alpha * acc[j0 + j] + b[j];
      }
      return;
    }
    if constexpr (P::PAIR) {
      // Pixel-pair mode in 32-bit arithmetic (N = 2 * pair_K <= 128 columns): one base pointer per thread, a
      // 32 x 64-bit product per column.  The general form below spent about 280 cycles per column here.
      float *o0 = p.epi.out + (mo & ~Epilogue::kLastOdd);
      const bool has_odd = !(mo & Epilogue::kLastOdd);
      const int pk = (int)p.epi.pair_K, n_end = (int)p.N, n0 = (int)nb;
      const long st = p.epi.nstride;
      const float *bias = p.epi.bias;
#pragma unroll
      for (int j0 = 0; j0 < NCOL; j0 += 16) {
        float b[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int n = n0 + j0 + j, plane = n >= pk ? n - pk : n;
          b[j] = (bias && n < n_end) ? __ldg(bias + plane) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int n = n0 + j0 + j, par = n >= pk ? 1 : 0, plane = n - par * pk;
          if (n < n_end && (has_odd || !par)) o0[(long)plane * st + par] = alpha * acc[j0 + j] + b[j];
        }
      }
      return;
    }
#pragma unroll
    for (int j0 = 0; j0 < NCOL; j0 += 16) {
      float b[16];
#pragma unroll
      for (int j = 0; j < 16; j++) b[j] = nb + j0 + j < p.N ? p.epi.template bias_of<P::PAIR>(nb + j0 + j) : 0.f;
#pragma unroll
      for (int j = 0; j < 16; j++)
        if (nb + j0 + j < p.N) p.epi.template store_biased<P::PAIR>(mo, nb + j0 + j, acc[j0 + j], b[j]);
    }
  } else if (p.epi.beta == 1.f && !p.epi.bias) {
    // Plain accumulation (gradWeight += ...): a reduction performed at the L2 cache per element, with no value
    // coming back, so the thread never waits for the old contents (a product with a short reduction is nothing
    // but this epilogue: fetching 16 old values at a time left it at a fifth of the HBM rate).  Every element is
    // touched once per launch, so the result does not depend on any order; it is the same FP32 add, except that
    // the memory-side adder flushes subnormal operands and results to zero.
    float *o = p.epi.out + mo + nb * p.epi.nstride;
    const long st = p.epi.nstride;
    const float alpha = p.epi.alpha;
#pragma unroll
    for (int j = 0; j < NCOL; j++)
      if (nb + j < p.N) atomicAdd(o + j * st, alpha * acc[j]);
  } else {
    // beta != 0: fetch the old values 16 at a time before any store, so that the loads overlap
#pragma unroll
    for (int j0 = 0; j0 < NCOL; j0 += 16) {
      float old[16];
#pragma unroll
      for (int j = 0; j < 16; j++) old[j] = nb + j0 + j < p.N ? p.epi.out[mo + (nb + j0 + j) * p.epi.nstride] : 0.f;
#pragma unroll
      for (int j = 0; j < 16; j++)
        if (nb + j0 + j < p.N) p.epi.store_with(mo, nb + j0 + j, acc[j0 + j], old[j]);
    }
  }
}


// Pixel-pair epilogue with whole-line stores (pair_K == 64 planes, 128-column tile, no split-K, beta == 0).  The warp
// owns 32 planes in BOTH parities: acc[j] = (parity 0, plane plane0 + j), acc[32 + j] = (parity 1, same plane).  A row
// of the product is a pair of horizontally adjacent output pixels, so a lane's two values of a plane are neighbours
// in memory while neighbouring lanes are two floats apart: stored as they lie, every store instruction would fill
// half of each sector.  Instead the warp transposes through shuffles: in pass k lane l stores parity l & 1 of the
// row that lane 16 k + l / 2 holds, so that the 32 lanes write 32 consecutive floats wherever their rows are
// consecutive pairs of one output row.  Every lane of the warp must call this (rows past M carry m >= p.M).
template <class P>
__device__ __forceinline__ void tc2_store_pair_rows(const P &p, const float (&acc)[64], long m, int plane0) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31, par = lane & 1;
  const long long kNone = -1;
  const long long mo = m < p.M ? (long long)p.epi.template moff<true>(m) : kNone;
  const float alpha = p.epi.alpha;
  const long st = p.epi.nstride;
  const float *bias = p.epi.bias;
  float *base[2];
  bool live[2];
#pragma unroll
  for (int k = 0; k < 2; k++) {
    const long long smo = __shfl_sync(full, mo, 16 * k + (lane >> 1));
    live[k] = smo != kNone && !(par && (smo & Epilogue::kLastOdd));
    base[k] = p.epi.out + (smo & ~Epilogue::kLastOdd) + par + (long)plane0 * st;
  }
#pragma unroll
  for (int j0 = 0; j0 < 32; j0 += 8) {
    float b[8];
#pragma unroll
    for (int j = 0; j < 8; j++) b[j] = bias ? __ldg(bias + plane0 + j0 + j) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int k = 0; k < 2; k++) {
        const int src = 16 * k + (lane >> 1);
        const float v0 = __shfl_sync(full, acc[j0 + j], src), v1 = __shfl_sync(full, acc[32 + j0 + j], src);
        if (live[k]) base[k][(long)(j0 + j) * st] = alpha * (par ? v1 : v0) + b[j];
      }
    }
  }
}

// Folds split-K partials (fixed order -> deterministic) and applies the epilogue.  grid.y walks n, threads walk
// m, which is contiguous in the workspace.
static __global__ void __launch_bounds__(256) splitk_finish_kernel(const float *__restrict__ ws, int splits, long M, long N,
                                                            Epilogue epi) {
  const long m = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const bool pair = epi.pair_K != 0;
  const long mo = pair ? epi.moff<true>(m) : epi.moff<false>(m);
  for (long n = blockIdx.y; n < N; n += gridDim.y) {
    float acc = 0.f;
    for (int z = 0; z < splits; z++) acc += ws[((long)z * N + n) * M + m];
    if (pair) epi.store<true>(mo, n, acc);
    else epi.store<false>(mo, n, acc);
  }
}

// The same for the tile-local partials of the raw-operand engine (Problem::tail_first): block (t, y) folds columns
// y, y + gridDim.y, ... of tail tile t; a thread owns one of the tile's 256 rows, which are contiguous in the
// workspace.
static __global__ void __launch_bounds__(256) tail_finish_kernel(const float *__restrict__ ws, int splits, int bn2, long tail_first,
                                                          long gm, long M, long N, Epilogue epi) {
  const long tile = tail_first + blockIdx.x;
  const long nt = tile / gm, mt = tile - nt * gm;
  const long m = mt * 256 + threadIdx.x;
  if (m >= M) return;
  const bool pair = epi.pair_K != 0;
  const long mo = pair ? epi.moff<true>(m) : epi.moff<false>(m);
  const float *base = ws + (long)blockIdx.x * splits * bn2 * 256 + threadIdx.x;
  for (int c = blockIdx.y; c < bn2; c += gridDim.y) {
    const long n = nt * bn2 + c;
    if (n >= N) break;
    float acc = 0.f;
    for (int z = 0; z < splits; z++) acc += base[((long)z * bn2 + c) * 256];
    if (pair) epi.store<true>(mo, n, acc);
    else epi.store<false>(mo, n, acc);
  }
}

}  // namespace mm
}  // namespace thc

#endif
