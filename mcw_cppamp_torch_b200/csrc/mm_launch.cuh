// Host-side dispatch of an mm::Problem onto an engine: picks the tile width, decides split-K,
// owns the split-K workspace, launches, and folds the partials.
#ifndef THC_MM_LAUNCH_CUH
#define THC_MM_LAUNCH_CUH

#include <algorithm>
#include <climits>

#include "mm_simt.cuh"
#include "mm_tc.cuh"
#include "mm_tc2.cuh"
#include "mm_tc2h.cuh"
#include "mm_tc2r.cuh"

namespace thc {
namespace mm {

// hi / lo planes of a strided matrix for the tensor-core engine (workspace of the running entry point).
// Element (r, k) of the source lives at src[r*rs + k*ks].
struct SplitPlanes {
  float *hi = nullptr, *lo = nullptr;
  long ld = 0;
};
static SplitPlanes make_split_planes(const float *src, long rs, long ks, long rows, long K) {
  SplitPlanes sp;
  sp.ld = (K + 31) / 32 * 32;
  sp.hi = (float *)ws_alloc(sizeof(float) * 2 * rows * sp.ld);
  sp.lo = sp.hi + rows * sp.ld;
  const long ntiles = ((rows + 31) / 32) * (sp.ld / 32);
  long blocks = ntiles;
  const long cap = (long)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap;
  split_planes_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(src, rs, ks, rows, K, sp.hi, sp.lo, sp.ld);
  check_launch("split_planes");
  return sp;
}
static SplitOperand split_operand(const SplitPlanes &sp, long rows) {
  SplitOperand o;
  o.base = sp.hi; o.lo = sp.lo;
  o.rows = LinearMap{rows, sp.ld};
  o.ks = LinearMap{sp.ld, 1};
  o.H = o.W = 0; o.dH = o.dW = 1; o.vec4 = 1;
  o.k_inner.d = 0; o.k_inner.mul = 0; o.k_inner.shr = 0; o.k_outer_stride = 0;
  return o;
}

template <class P, int BN>
static void launch_tc(const P &p, dim3 grid) {
  typedef TcCfg<BN> Cfg;
  static bool configured = false;
  if (!configured) {
    THC_CUDA(cudaFuncSetAttribute(tc_kernel<P, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured = true;
  }
  tc_kernel<P, BN><<<grid, TC_THREADS, Cfg::SMEM_BYTES, stream()>>>(p, stall_ctl());
  check_launch("tc_kernel");
}

// How many k slices to cut a product into so that tiles * slices fills whole waves of `slots` concurrent tiles.
// Slicing costs a workspace round trip (slices * M * N floats written and read back), so it needs a clear
// gain: one slice unless the fill of the last wave rises by a quarter; every slice keeps at least 16 k tiles.
static long choose_splits(long tiles, long ktiles, int slots) {
  if (tiles >= 4l * slots || ktiles < 32) return 1;
  auto fill = [&](long s) {
    const long ctas = tiles * s, waves = (ctas + slots - 1) / slots;
    return (double)ctas / (double)(waves * slots);
  };
  long best = 1, max_s = ktiles / 16;
  if (max_s > 256) max_s = 256;
  const double base = fill(1);
  double best_fill = base;
  for (long s = 2; s <= max_s; s++) {
    const double f = fill(s);
    if (f > base * 1.25 && f > best_fill + 0.04) { best = s; best_fill = f; }
  }
  return best;
}

// Slices for the `tail` tiles a persistent launch has left after its whole rounds over `slots` clusters.  A model in
// microseconds: a 32-k tile step of a two-SM tile takes about 1.2 us; a partial-sum block (256 x BN2 floats) costs
// about 0.17 us of device-wide write + read-back; the folding kernel about 5 us to launch.  Every slice keeps at
// least six k tiles (the pipeline fill of an item is two to three).
static int choose_tail_splits(long tail, long ktiles, int slots) {
  int best = 1;
  double best_us = 1.2 * (double)ktiles;
  const long max_s = std::min<long>(ktiles / 6, 4l * slots);
  for (long s = 2; s <= max_s; s++) {
    const long rounds = (tail * s + slots - 1) / slots, per = (ktiles + s - 1) / s;
    const double us = 1.2 * (double)(rounds * per) + 0.17 * (double)(tail * s) + 5.0;
    if (us < best_us * 0.9) { best = (int)s; best_us = us; }
  }
  return best;
}

// `allow_split` lets long-K problems with few output tiles spread over the SMs.  TC_ONLY problems
// (operands that only the tensor-core engine can read) never instantiate the FP32 FMA engine.
template <class P, bool TC_ONLY>
static void launch_impl(P p, bool allow_split) {
  if (p.M <= 0 || p.N <= 0) return;
  THC_CHECK(p.K > 0, "internal: matrix product with empty reduction");
  const int mode = ctx().math_mode;
  THC_CHECK(mode == 0 || mode == 2 || (mode == 1 && !TC_ONLY), "math mode %d cannot run this product", mode);
  const int sms = ctx().sm_count;
  const bool tc = mode != 1;   // the BF16 mode runs what its own engine does not take in the FP32-accurate one
  const int bm = tc ? TC_BM : SIMT_BM;
  const int bn = tc ? (p.N > 64 ? 128 : 64) : SIMT_BN;
  const long gm = (p.M + bm - 1) / bm, gn = (p.N + bn - 1) / bn, tiles = gm * gn;
  THC_CHECK(gn <= 65535, "matrix too wide for one launch");
  const long ktiles = (p.K + TC_BK - 1) / TC_BK;
  long splits = allow_split ? choose_splits(tiles, ktiles, sms) : 1;
  p.ws = nullptr;
  p.k_per_split = p.K;
  if (splits > 1) {
    const long per = (ktiles + splits - 1) / splits;
    p.k_per_split = per * TC_BK;
    splits = (p.K + p.k_per_split - 1) / p.k_per_split;
  }
  if (splits > 1) p.ws = (float *)ws_alloc(sizeof(float) * splits * p.M * p.N);
  dim3 grid((unsigned)gm, (unsigned)gn, (unsigned)splits);
  if (tc) {
    if (bn == 128) launch_tc<P, 128>(p, grid);
    else launch_tc<P, 64>(p, grid);
  } else if constexpr (!TC_ONLY) {
    simt_kernel<P><<<grid, 256, 0, stream()>>>(p);
    check_launch("simt_kernel");
  }
  if (splits > 1) {
    splitk_finish_kernel<<<dim3((unsigned)ceil_div(p.M, 256), (unsigned)(p.N < 32768 ? p.N : 32768)), 256, 0, stream()>>>(
        p.ws, (int)splits, p.M, p.N, p.epi);
    check_launch("splitk_finish");
  }
}
template <class P> static void launch(const P &p, bool allow_split = true) { launch_impl<P, false>(p, allow_split); }
template <class P> static void launch_tc_only(const P &p, bool allow_split = true) { launch_impl<P, true>(p, allow_split); }

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
    else
      cudaGetLastError();
  }
  return fn;
}
typedef CUresult (*EncodeIm2colFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const int *, const int *, cuuint32_t, cuuint32_t, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeIm2colFn encode_im2col_fn() {
  static EncodeIm2colFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeIm2colFn)ptr;
    else
      cudaGetLastError();
  }
  return fn;
}
// Describes the windows of one channels-last FP32 plane [N][H][W][C] to TMA's im2col mode (raw-operand engine):
// windows of an [oH, oW] output grid at strides (dH, dW) under padding (padH, padW); one load brings 32 channels
// of 128 consecutive windows at one filter tap.  hi / lo plane pairs (n_planes == 2) belong to the plane engine,
// whose threads copy the tiles themselves: use_tma stays 0 for them, and whenever the plane cannot be described.
static void attach_window_map(PlanesWindowOperand &op, long N, long H, long W, long C, long oH, long oW, int dH, int dW,
                              int padH, int padW, int n_planes) {
  op.use_tma = 0;
  op.n_img = (int)N;
  op.n_planes = n_planes;
  op.ctiles = FastDiv::make(C >= 32 ? C / 32 : 1);
  EncodeIm2colFn enc = encode_im2col_fn();
  const int lower[2] = {-padW, -padH};
  const long up_w = -(long)padW + (oW - 1) * dW - (W - 1), up_h = -(long)padH + (oH - 1) * dH - (H - 1);
  if (n_planes != 1 || !enc || C % 32 != 0 || ((uintptr_t)op.base & 15) != 0 ||
      2 * N >= (1l << 31) ||
      padW > 128 || padH > 128 || up_w < -128 || up_w > 127 || up_h < -128 || up_h > 127 || dW < 1 || dW > 8 || dH < 1 ||
      dH > 8 || W >= (1l << 31) || H >= (1l << 31))
    return;
  const int upper[2] = {(int)up_w, (int)up_h};
  const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)(n_planes * N)};
  const cuuint64_t strides[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
  const cuuint32_t estr[4] = {1, (cuuint32_t)dW, (cuuint32_t)dH, 1};
  const CUresult r = enc(&op.tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)op.base, dims, strides, lower, upper, 32, TC_BM,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) op.use_tma = 1;
}

template <class P, int BN2>
static void launch_tc2_kernel(P &p, dim3 grid) {
  typedef Tc2Cfg<BN2> Cfg;
  static bool configured = false;
  if (!configured) {
    THC_CUDA(cudaFuncSetAttribute(tc2_kernel<P, BN2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured = true;
  }
  tc2_kernel<P, BN2><<<grid, T2_THREADS, Cfg::SMEM_BYTES, stream()>>>(p, stall_ctl());
  check_launch("tc2_kernel");
}

// Describes a plain FP32 matrix (element (r, k) at base[r * row_stride + k * k_stride], one stride being 1) to the
// raw-operand engine.  False when TMA cannot address it (alignment, pitch).
static bool raw_matrix_ok(const float *base, long ld) {
  return encode_tiled_fn() && ((uintptr_t)base & 15) == 0 && ld % 4 == 0 && ld > 0;
}
template <bool MN>
static void attach_raw_map(RawOperand<MN> &op, const float *base, long rows, long K, long ld, int tile_rows) {
  op.use_tma = 0;
  EncodeTiledFn enc = encode_tiled_fn();
  THC_CHECK(enc && raw_matrix_ok(base, ld), "internal: matrix not addressable by TMA");
  const cuuint64_t dims[2] = {(cuuint64_t)(MN ? rows : K), (cuuint64_t)(MN ? K : rows)};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  const cuuint32_t box[2] = {32, (cuuint32_t)(MN ? 32 : tile_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(&op.tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, MN ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  THC_CHECK(r == CUDA_SUCCESS, "internal: cuTensorMapEncodeTiled failed");
  op.use_tma = 1;
}

// Corners of the im2col bounding box of windows of an [oH, oW] output grid over an H x W plane; false when TMA
// cannot express them.
static bool window_corners(long H, long W, long oH, long oW, int dH, int dW, int padH, int padW, int lower[2], int upper[2]) {
  const long up_w = -(long)padW + (oW - 1) * dW - (W - 1), up_h = -(long)padH + (oH - 1) * dH - (H - 1);
  if (padW > 128 || padH > 128 || padW < -127 || padH < -127 || up_w < -128 || up_w > 127 || up_h < -128 || up_h > 127 ||
      dW < 1 || dW > 8 || dH < 1 || dH > 8 || W >= (1l << 31) || H >= (1l << 31))
    return false;
  lower[0] = -padW; lower[1] = -padH; upper[0] = (int)up_w; upper[1] = (int)up_h;
  return true;
}
static bool raw_windows_ok(long N, long H, long W, long C, long oH, long oW, int dH, int dW, int padH, int padW) {
  int lo[2], up[2];
  return encode_im2col_fn() && encode_tiled_fn() && C % 32 == 0 && N < (1l << 30) &&
         window_corners(H, W, oH, oW, dH, dW, padH, padW, lo, up);
}
// The input windows of a weight-gradient product (WindowRowsOperand) over one FP32 plane [N][H][W][C].
static void attach_window_rows_map(WindowRowsOperand &op, const float *base, long N, long H, long W, long C, long oH, long oW,
                                   int dH, int dW, int padH, int padW) {
  op.use_tma = 0;
  op.n_img = (int)N;
  EncodeIm2colFn enc = encode_im2col_fn();
  int lower[2], upper[2];
  THC_CHECK(enc && C % 32 == 0 && ((uintptr_t)base & 15) == 0 && window_corners(H, W, oH, oW, dH, dW, padH, padW, lower, upper),
            "internal: windows not addressable by TMA");
  const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  const cuuint64_t strides[3] = {(cuuint64_t)C * 4, (cuuint64_t)W * C * 4, (cuuint64_t)H * W * C * 4};
  const cuuint32_t estr[4] = {1, (cuuint32_t)dW, (cuuint32_t)dH, 1};
  const CUresult r = enc(&op.tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)base, dims, strides, lower, upper, 32, 32, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  THC_CHECK(r == CUDA_SUCCESS, "internal: cuTensorMapEncodeIm2col failed");
  op.use_tma = 1;
}

// Clusters of the raw-operand kernel that the device runs at once (the kernel is persistent: a launch has no more).
template <class P, int BN2>
static int tc2r_resident_clusters() {
  typedef Tc2rCfg<BN2> Cfg;
  static int n = 0;
  if (n) return n;
  THC_CUDA(cudaFuncSetAttribute(tc2r_kernel<P, BN2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ctx().sm_count, 1, 1);
  cfg.blockDim = dim3(T2_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  int c = 0;
  if (cudaOccupancyMaxActiveClusters(&c, tc2r_kernel<P, BN2>, &cfg) != cudaSuccess || c < 1) {
    cudaGetLastError();
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&c, tc2r_kernel<P, BN2>, &cfg) != cudaSuccess || c < 1) {
      cudaGetLastError();
      c = ctx().sm_count / 2;
    }
  }
  if (c > ctx().sm_count / 2) c = ctx().sm_count / 2;
  n = c;
  return n;
}
template <class P, int BN2>
static void launch_tc2r_kernel(const P &p, long items) {
  typedef Tc2rCfg<BN2> Cfg;
  const long clusters = std::min<long>(items, tc2r_resident_clusters<P, BN2>());
  tc2r_kernel<P, BN2><<<dim3((unsigned)(2 * clusters), 1, 1), T2_THREADS, Cfg::SMEM_BYTES, stream()>>>(p, stall_ctl(),
                                                                                                                sched_counter());
  check_launch("tc2r_kernel");
}

// Width of the two-SM tile that pads N least (wider wins ties); 0 when the product is too small for it.
static int tc2_tile_width(long M, long N) {
  if (M <= 128 || N <= 32) return 0;
  int best = 0;
  long best_pad = 0;
  const int widths[4] = {256, 192, 128, 64};
  for (int w : widths) {
    const long pad = (N + w - 1) / w * w;
    if (!best || pad < best_pad) { best = w; best_pad = pad; }
  }
  return best;
}

// Products over plain FP32 operands that TMA can fetch (raw-operand engine).  `attach(p, bn2)` writes the
// operands' tensor maps for the chosen tile width.  The caller has checked tc2_tile_width(M, N) != 0.
template <class P, class Attach>
static void launch_raw(P p, Attach attach, bool allow_split = true) {
  if (p.M <= 0 || p.N <= 0) return;
  THC_CHECK(p.K > 0, "internal: matrix product with empty reduction");
  const int bn2 = tc2_tile_width(p.M, p.N);
  THC_CHECK(bn2 != 0 && ctx().math_mode != 1, "internal: raw-operand engine on a product it does not serve");
  attach(p, bn2);
  const long gm = (p.M + 255) / 256, gn = (p.N + bn2 - 1) / bn2, tiles = gm * gn;
  const int slots = bn2 == 256 ? tc2r_resident_clusters<P, 256>() : bn2 == 192 ? tc2r_resident_clusters<P, 192>()
                  : bn2 == 128 ? tc2r_resident_clusters<P, 128>() : tc2r_resident_clusters<P, 64>();
  const long ktiles = (p.K + TC_BK - 1) / TC_BK;
  // Every cluster first runs tiles / slots whole tiles; the remaining `tail` tiles (all of them when there are fewer
  // tiles than clusters) are cut along k so that they fill the clusters once more instead of leaving most idle.
  const long tail = tiles % slots;
  const int splits = allow_split && tail ? choose_tail_splits(tail, ktiles, slots) : 1;
  p.ws = nullptr;
  p.k_per_split = p.K;
  p.tail_first = tiles;
  p.tail_splits = 1;
  if (splits > 1) {
    const long per = (ktiles + splits - 1) / splits;
    p.k_per_split = per * TC_BK;
    p.tail_splits = (int)((p.K + p.k_per_split - 1) / p.k_per_split);
  }
  if (p.tail_splits > 1) {
    p.tail_first = tiles - tail;
    p.ws = (float *)ws_alloc(sizeof(float) * tail * p.tail_splits * bn2 * 256);
  }
  const long items = p.tail_first + (tiles - p.tail_first) * p.tail_splits;
  THC_CHECK(items < (1l << 31) - 4096, "matrix product with too many tiles for one launch");
  if (bn2 == 256) launch_tc2r_kernel<P, 256>(p, items);
  else if (bn2 == 192) launch_tc2r_kernel<P, 192>(p, items);
  else if (bn2 == 128) launch_tc2r_kernel<P, 128>(p, items);
  else launch_tc2r_kernel<P, 64>(p, items);
  if (p.ws) {
    // a few thousand blocks whatever the number of tail tiles: a lone tile cut into many slices gets a block per column
    const long by = std::min<long>(bn2, std::max<long>(32, ceil_div(8l * ctx().sm_count, tail)));
    tail_finish_kernel<<<dim3((unsigned)tail, (unsigned)by), 256, 0, stream()>>>(
        p.ws, p.tail_splits, bn2, p.tail_first, gm, p.M, p.N, p.epi);
    check_launch("tail_finish");
  }
}

// Products over ready-made planes: the two-SM engine when the tile fits the problem, else the one-SM engine.
template <class P>
static void launch_planes(P p, bool allow_split = true) {
  if (p.M <= 0 || p.N <= 0) return;
  THC_CHECK(p.K > 0, "internal: matrix product with empty reduction");
  const int bn2 = tc2_tile_width(p.M, p.N);
  if (!bn2) { launch_tc_only(p, allow_split); return; }
  THC_CHECK(ctx().math_mode != 1, "internal: plane operands need a tensor-core math mode");
  const int sms = ctx().sm_count;
  const long gm = (p.M + 255) / 256, gn = (p.N + bn2 - 1) / bn2, tiles = gm * gn;
  THC_CHECK(gn <= 65535, "matrix too wide for one launch");
  const long ktiles = (p.K + TC_BK - 1) / TC_BK;
  long splits = allow_split ? choose_splits(tiles, ktiles, sms / 2) : 1;
  p.ws = nullptr;
  p.k_per_split = p.K;
  if (splits > 1) {
    const long per = (ktiles + splits - 1) / splits;
    p.k_per_split = per * TC_BK;
    splits = (p.K + p.k_per_split - 1) / p.k_per_split;
  }
  if (splits > 1) p.ws = (float *)ws_alloc(sizeof(float) * splits * p.M * p.N);
  dim3 grid((unsigned)(2 * gm), (unsigned)gn, (unsigned)splits);
  if (bn2 == 256) launch_tc2_kernel<P, 256>(p, grid);
  else if (bn2 == 192) launch_tc2_kernel<P, 192>(p, grid);
  else if (bn2 == 128) launch_tc2_kernel<P, 128>(p, grid);
  else launch_tc2_kernel<P, 64>(p, grid);
  if (splits > 1) {
    splitk_finish_kernel<<<dim3((unsigned)ceil_div(p.M, 256), (unsigned)(p.N < 32768 ? p.N : 32768)), 256, 0, stream()>>>(
        p.ws, (int)splits, p.M, p.N, p.epi);
    check_launch("splitk_finish");
  }
}

// Channels-last hi / lo planes of an NCHW activation tensor, channels padded with zeros to Cp = a multiple
// of 4 (in a caller's tensor or in the workspace of the running entry point).
struct ActPlanes {
  float *hi = nullptr, *lo = nullptr;
  long Cp = 0;
  // per-channel sums of the transposed tensor, when asked for: [chan_blocks][C] partials (see nchw_to_planes_kernel)
  float *chan_partial = nullptr;
  int chan_blocks = 0;
};
inline long planes_channels(long C) { return (C + 3) / 4 * 4; }
// `dst`: room for 2 * N * HW * planes_channels(C) floats, or null for workspace.  raw: one plane
// of the FP32 values themselves (half the room), lo stays null: the form the raw-operand engine reads.
static ActPlanes make_act_planes(const float *src, long N, long C, long HW, float *dst = nullptr, bool raw = false,
                                 bool want_chan_sums = false) {
  ActPlanes ap;
  ap.Cp = planes_channels(C);
  const long total = N * ap.Cp * HW;
  ap.hi = dst ? dst : (float *)ws_alloc(sizeof(float) * (raw ? 1 : 2) * total);
  ap.lo = raw ? nullptr : ap.hi + total;
  const long cap = (long)ctx().sm_count * 16;
  if (C % 32 == 0) {
    long blocks = N * ((HW + 127) / 128) * (C / 32);
    if (blocks > cap) blocks = cap;
    size_t smem = 0;
    if (want_chan_sums && C <= 4096) {
      // every block leaves a row of per-channel sums for a second kernel to fold.  On a small tensor (a few tiles per
      // block) that fold costs as much as the transposition: a quarter of the blocks keeps it short (measured at
      // 128 images: fold 83 -> 33 us, transposition unchanged); on a large one the transposition wants all its
      // blocks (at 1024 images the same cut cost it 3 %, more than the fold gained)
      const long needed = N * ((HW + 127) / 128) * (C / 32);
      if (needed <= 4 * cap && blocks > cap / 4) blocks = cap / 4;
      ap.chan_blocks = (int)blocks;
      ap.chan_partial = (float *)ws_alloc(sizeof(float) * blocks * C);
      smem = sizeof(float) * C;
    }
    nchw_to_planes_kernel<<<(unsigned)blocks, 256, smem, stream()>>>(src, N, C, HW, ap.hi, ap.lo, ap.chan_partial);
  } else {
    long blocks = (N * HW + 255) / 256;
    if (blocks > cap) blocks = cap;
    nchw_to_planes_any_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(src, N, C, HW, ap.Cp, ap.hi, ap.lo);
  }
  check_launch("nchw_to_planes");
  return ap;
}


// ---- BF16 math mode ---------------------------------------------------------------------------------------
// One BF16 plane of a strided matrix (rows padded to 64 values), addressed in 4-byte units by the operands.
struct HalfPlane {
  __nv_bfloat16 *p = nullptr;
  long ld = 0;   // values per row
};
static HalfPlane make_half_plane(const float *src, long rs, long ks, long rows, long K) {
  HalfPlane hp;
  hp.ld = (K + 63) / 64 * 64;
  hp.p = (__nv_bfloat16 *)ws_alloc(sizeof(__nv_bfloat16) * rows * hp.ld);
  long blocks = ((rows + 31) / 32) * (hp.ld / 32);
  const long cap = (long)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap;
  bf16_rows_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(src, rs, ks, rows, K, hp.p, hp.ld);
  check_launch("bf16_rows");
  return hp;
}
static SplitOperand half_operand(const __nv_bfloat16 *plane, long rows, long ld) {
  SplitOperand o;
  o.base = reinterpret_cast<const float *>(plane); o.lo = nullptr;
  o.rows = LinearMap{rows, ld / 2};
  o.ks = LinearMap{ld / 2, 1};
  o.H = o.W = 0; o.dH = o.dW = 1; o.vec4 = 1;
  o.k_inner.d = 0; o.k_inner.mul = 0; o.k_inner.shr = 0; o.k_outer_stride = 0;
  return o;
}
// Tile width of the BF16 engine for an M x N product; MN-major operands need whole 64-channel blocks per CTA.
static int tc2h_tile_width(long M, long N, bool mn_major) {
  if (mn_major) {
    if (M <= 128 || N <= 64) return 0;
    return (N + 255) / 256 * 256 <= (N + 127) / 128 * 128 ? 256 : 128;
  }
  return tc2_tile_width(M, N);
}
template <class P, int BN2>
static void launch_tc2h_kernel(P &p, dim3 grid) {
  typedef Tc2hCfg<BN2> Cfg;
  static bool configured = false;
  if (!configured) {
    THC_CUDA(cudaFuncSetAttribute(tc2h_kernel<P, BN2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    configured = true;
  }
  tc2h_kernel<P, BN2><<<grid, T2_THREADS, Cfg::SMEM_BYTES, stream()>>>(p, stall_ctl());
  check_launch("tc2h_kernel");
}
// Products over BF16 planes.  p.K counts the operands' own k index (4-byte units for K-major operands,
// pixels for MN-major ones); the caller has checked tc2h_tile_width(M, N) != 0.
template <class P>
static void launch_planes_half(P p, bool allow_split = true) {
  constexpr bool MN = P::OpA::MN_MAJOR;
  constexpr int KT = MN ? 64 : 32;
  const int bn2 = tc2h_tile_width(p.M, p.N, MN);
  THC_CHECK(bn2 != 0 && p.K > 0, "internal: product too small for the BF16 engine");
  const int sms = ctx().sm_count;
  const long gm = (p.M + 255) / 256, gn = (p.N + bn2 - 1) / bn2, tiles = gm * gn;
  THC_CHECK(gn <= 65535, "matrix too wide for one launch");
  const long ktiles = (p.K + KT - 1) / KT;
  long splits = allow_split ? choose_splits(tiles, ktiles, sms / 2) : 1;
  p.ws = nullptr;
  p.k_per_split = p.K;
  if (splits > 1) {
    const long per = (ktiles + splits - 1) / splits;
    p.k_per_split = per * KT;
    splits = (p.K + p.k_per_split - 1) / p.k_per_split;
  }
  if (splits > 1) p.ws = (float *)ws_alloc(sizeof(float) * splits * p.M * p.N);
  dim3 grid((unsigned)(2 * gm), (unsigned)gn, (unsigned)splits);
  if (bn2 == 256) launch_tc2h_kernel<P, 256>(p, grid);
  else if (bn2 == 128) launch_tc2h_kernel<P, 128>(p, grid);
  else if constexpr (!MN) {
    if (bn2 == 192) launch_tc2h_kernel<P, 192>(p, grid);
    else launch_tc2h_kernel<P, 64>(p, grid);
  }
  if (splits > 1) {
    splitk_finish_kernel<<<dim3((unsigned)ceil_div(p.M, 256), (unsigned)(p.N < 32768 ? p.N : 32768)), 256, 0, stream()>>>(
        p.ws, (int)splits, p.M, p.N, p.epi);
    check_launch("splitk_finish");
  }
}

// Channels-last BF16 plane of an NCHW activation tensor, channels padded with zeros to a multiple of 8.
struct HalfActPlane {
  __nv_bfloat16 *p = nullptr;
  long Cp = 0;
};
static HalfActPlane make_half_act_plane(const float *src, long N, long C, long HW) {
  HalfActPlane ap;
  ap.Cp = (C + 7) / 8 * 8;
  ap.p = (__nv_bfloat16 *)ws_alloc(sizeof(__nv_bfloat16) * N * HW * ap.Cp);
  const long cap = (long)ctx().sm_count * 16;
  if (C % 32 == 0) {
    long blocks = N * ((HW + 31) / 32) * (C / 32);
    if (blocks > cap) blocks = cap;
    nchw_to_planes_bf16_tiled_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(src, N, C, HW, ap.p);
  } else {
    long blocks = (N * HW + 255) / 256;
    if (blocks > cap) blocks = cap;
    nchw_to_planes_bf16_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(src, N, C, HW, ap.Cp, ap.p);
  }
  check_launch("nchw_to_planes_bf16");
  return ap;
}

}  // namespace mm
}  // namespace thc

#endif
