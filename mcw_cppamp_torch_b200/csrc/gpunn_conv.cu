// nn.SpatialConvolutionMM on torch.GPUTensor: forward, gradInput, gradParameters.
//
// The reference (gputorch/lib/THC/gpunn-impl/SpatialConvolutionMM.cpp: updateOutput :110-225,
// updateGradInput :227-311, accGradParameters :313-429) loops over the images of a batch on the
// host and, per image, launches im2col / col2im and a 16x16-tile SGEMM.  Here each pass is ONE
// implicit-GEMM launch over the whole batch: the operand maps below state where element (row, k) of
// the would-be column matrix lives in the NCHW tensor, and the matrix-multiply engine gathers it on
// the fly.  Results follow the CPU nn semantics (mcw_nn/generic/SpatialConvolutionMM.c) and also
// cover dW/dH > 1, which the CPU MM path rejects (:148-149) and the reference GPU path supports.
#include "mm_launch.cuh"

#include <unordered_map>

namespace thc {

// What the planes kept in a module's `finput` were made from.  accGradParameters reuses them only when it is
// handed the very input (same device memory, same math mode) that the forward pass transposed; a forward pass
// that does not write `finput` forgets the entry, so planes of an earlier pass are never taken for fresh ones.
// Keyed by the address of finput's data; one table per host thread, as the rest of the library's state.
namespace {
struct PlaneStamp { const float *input; int mode; };
thread_local std::unordered_map<const float *, PlaneStamp> g_plane_stamps;
void stamp_planes(const THGPUTensor *finput, const float *input) {
  if (!finput || !finput->storage) return;
  if (g_plane_stamps.size() > 4096) g_plane_stamps.clear();
  g_plane_stamps[data_ptr(finput)] = PlaneStamp{input, ctx().math_mode};
}
void forget_planes(const THGPUTensor *finput) {
  if (finput && finput->storage) g_plane_stamps.erase(data_ptr(finput));
}
bool planes_made_from(const THGPUTensor *finput, const float *input) {
  if (!finput || !finput->storage) return false;
  auto it = g_plane_stamps.find(data_ptr(finput));
  return it != g_plane_stamps.end() && it->second.input == input && it->second.mode == ctx().math_mode;
}
}  // namespace

struct ConvGeom {
  long N, C, H, W, K, oH, oW, P, R;
  int kH, kW, dH, dW, pad;
  bool batch;
};

static ConvGeom conv_geom(const THGPUTensor *input, const THGPUTensor *weight, int kW, int kH, int dW, int dH, int padding) {
  THC_ARG(input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D (batch mode) tensor is expected");
  THC_ARG(kW > 0 && kH > 0 && dW > 0 && dH > 0 && padding >= 0, 1, "invalid kernel / stride / padding");
  THC_ARG(weight->nDimension == 2, 1, "weight must be 2D (nOutputPlane x nInputPlane*kH*kW)");
  ConvGeom g;
  g.batch = input->nDimension == 4;
  const int o = g.batch ? 1 : 0;
  g.N = g.batch ? input->size[0] : 1;
  g.C = input->size[o];
  g.H = input->size[o + 1];
  g.W = input->size[o + 2];
  g.K = weight->size[0];
  g.kH = kH; g.kW = kW; g.dH = dH; g.dW = dW; g.pad = padding;
  g.R = g.C * kH * kW;
  THC_ARG(weight->size[1] == g.R, 2, "input channels and nInputPlane dont match");
  THC_ARG(g.H + 2 * padding >= kH && g.W + 2 * padding >= kW, 2, "input image smaller than kernel size");
  g.oH = (g.H + 2 * padding - kH) / dH + 1;
  g.oW = (g.W + 2 * padding - kW) / dW + 1;
  g.P = g.oH * g.oW;
  THC_CHECK(g.C * g.H * g.W < (1l << 31) && g.K * g.P < (1l << 31), "image too large");
  return g;
}

static mm::PixelMap input_windows(const ConvGeom &g) {  // (img, y, x) -> top-left corner of its window
  mm::PixelMap m;
  m.set(g.N * g.P, g.P, g.oW);
  m.img_stride = g.C * g.H * g.W; m.y_stride = g.dH * g.W; m.x_stride = g.dW;
  m.off0 = -(long)g.pad * g.W - g.pad;
  m.sy = g.dH; m.y0 = -g.pad; m.sx = g.dW; m.x0 = -g.pad;
  return m;
}
static mm::TapMap input_taps(const ConvGeom &g) {  // (c, i, j) -> offset inside the window
  mm::TapMap m;
  m.set(g.R, g.kH * g.kW, g.kW);
  m.c_stride = g.H * g.W; m.i_stride = g.W; m.j_stride = 1;
  m.si = 1; m.sj = 1;
  return m;
}

// ------------------------------------------------------------------------------------------------
// Tensor-core passes over channels-last hi / lo planes (layers whose channel counts are multiples of 32;
// first layers with 3 input planes keep the element gathers above).  The activation tensor is rounded
// and transposed once per call (12 bytes per element, a small fraction of the pass), after which
// every operand tile of the product is filled with 16-byte asynchronous copies.

// windows of the plane grid [N, H, W, C] seen from the output grid [N, oH, oW]
static void set_window_map(mm::PixelMap &m, long N, long oH, long oW, long H, long W, long C, int dH, int dW, int padH,
                           int padW) {
  m.set(N * oH * oW, oH * oW, oW);
  m.img_stride = H * W * C; m.y_stride = dH * W * C; m.x_stride = dW * C;
  m.off0 = -((long)padH * W + padW) * C;
  m.sy = dH; m.y0 = -padH; m.sx = dW; m.x0 = -padW;
}

struct WeightPlanes {
  float *hi = nullptr, *lo = nullptr;
  long ld = 0;
};
// flip 0: rows = output planes, k = (tap, input plane padded to Cp); flip 1: rows = input planes,
// k = (rotated tap, output plane padded to Kp).  Rows are padded with zeros to a multiple of 32 floats.
static WeightPlanes make_weight_planes(const float *w, long K, long C, int kH, int kW, long Cp, long Kp, int flip,
                                       int pair_shift = 0, bool raw = false) {
  WeightPlanes wp;
  const long rows = (flip ? C : K) * (pair_shift ? 2 : 1);
  wp.ld = ((long)kH * (kW + pair_shift) * (flip ? Kp : Cp) + 31) / 32 * 32;
  const long total = rows * wp.ld;
  wp.hi = (float *)ws_alloc(sizeof(float) * (raw ? 1 : 2) * total);
  wp.lo = raw ? nullptr : wp.hi + total;   // raw: the FP32 values themselves, for the raw-operand engine
  int blocks = ceil_div(total, 256);
  if (blocks > ctx().sm_count * 8) blocks = ctx().sm_count * 8;
  mm::repack_weight_planes_kernel<<<blocks, 256, 0, stream()>>>(w, K, C, (long)kH * kW, Cp, Kp, wp.ld, flip, kW, pair_shift,
                                                                wp.hi, wp.lo);
  check_launch("repack_weight_planes");
  return wp;
}
static mm::SplitOperand weight_operand(const WeightPlanes &wp, long rows) {
  mm::SplitOperand o;
  o.base = wp.hi; o.lo = wp.lo;
  o.rows = mm::LinearMap{rows, wp.ld};
  o.ks = mm::LinearMap{wp.ld, 1};
  o.H = o.W = 0; o.dH = o.dW = 1; o.vec4 = 1;
  o.k_inner.d = 0; o.k_inner.mul = 0; o.k_inner.shr = 0; o.k_outer_stride = 0;
  return o;
}

// out[n, ko, y, x] = bias[ko] + sum_{i,j,c} planes[n, y*dH-pad+i, x*dW-pad+j, c] * W'[ko][(i,j,c)]
// `Cp` (padded) channels per pixel of the planes, plane grid H x W, output grid oH x oW.  `w` is the weight
// matrix [K][C*kH*kW]; flip: the gradInput form (rows = C, filter rotated).  A tcgen05.mma occupies the tensor
// pipe about 80 cycles however narrow it is, so with up to 64 output planes two horizontally adjacent output
// pixels share a row of the product (pixel-pair mode): half the rows, twice the columns, a window one stride wider.
template <bool PAIR>
static void conv_window_product_t(const mm::ActPlanes &act, const float *w, long Kw, long Cw, int flip, long N, long H, long W,
                                  long Kout, long oH, long oW, int kH, int kW, int dH, int dW, int padH, int padW,
                                  const float *bias, float *out) {
  using namespace mm;
  const bool raw = act.lo == nullptr;                    // one FP32 plane: the raw-operand engine
  const long Cp = act.Cp;
  const long oWr = PAIR ? (oW + 1) / 2 : oW;             // rows of the product per output row
  const int dWr = PAIR ? 2 * dW : dW, kWe = PAIR ? kW + dW : kW;
  WeightPlanes wp = make_weight_planes(w, Kw, Cw, kH, kW, flip ? 0 : Cp, flip ? Cp : 0, flip, PAIR ? dW : 0, raw);
  auto describe = [&](auto &p) {
    p.a.base = act.hi; p.a.lo = act.lo;
    set_window_map(p.a.rows, N, oH, oWr, H, W, Cp, dH, dWr, padH, padW);
    p.a.ks = LinearMap{wp.ld, 1};
    p.a.H = (int)H; p.a.W = (int)W; p.a.dH = p.a.dW = 1; p.a.vec4 = 1;
    p.a.cquads = FastDiv::make(Cp / 4);
    p.a.kW = FastDiv::make(kWe);
    p.a.taps = (unsigned)(kH * kWe);
    p.a.i_stride = W * Cp; p.a.j_stride = Cp;
    attach_window_map(p.a, N, H, W, Cp, oH, oWr, dH, dWr, padH, padW, raw ? 1 : 2);
    p.epi = Epilogue{out, bias, 1.f, 0.f, oH * oW, Kout * oH * oW, oH * oW};
    if (PAIR) {
      p.epi.pair_K = Kout; p.epi.pair_oH = oH; p.epi.pair_oW2 = oWr; p.epi.pair_oW = oW; p.epi.pair_img = Kout * oH * oW;
    }
    p.M = N * oH * oWr; p.N = PAIR ? 2 * Kout : Kout; p.K = wp.ld;
  };
  if (raw) {
    Problem<PlanesWindowOperand, RawOperand<false>, PAIR> p;
    describe(p);
    THC_CHECK(p.a.use_tma, "internal: windows not addressable by TMA");
    launch_raw(p, [&](Problem<PlanesWindowOperand, RawOperand<false>, PAIR> &q, int bn2) {
      attach_raw_map(q.b, wp.hi, q.N, wp.ld, wp.ld, bn2 / 2);
    });
  } else {
    Problem<PlanesWindowOperand, SplitOperand, PAIR> p;
    describe(p);
    p.b = weight_operand(wp, PAIR ? 2 * Kout : Kout);
    launch_planes(p);
  }
}
static bool conv_pair_mode(long N, long Kout, long oH, long oW) {
  return Kout <= 64 && Kout > 16 && oW >= 2 && N * oH * ((oW + 1) / 2) > 128;
}
static void conv_window_product(const mm::ActPlanes &act, const float *w, long Kw, long Cw, int flip, long N, long H, long W,
                                long Kout, long oH, long oW, int kH, int kW, int dH, int dW, int padH, int padW,
                                const float *bias, float *out) {
  const bool pair = conv_pair_mode(N, Kout, oH, oW);
  if (pair) conv_window_product_t<true>(act, w, Kw, Cw, flip, N, H, W, Kout, oH, oW, kH, kW, dH, dW, padH, padW, bias, out);
  else conv_window_product_t<false>(act, w, Kw, Cw, flip, N, H, W, Kout, oH, oW, kH, kW, dH, dW, padH, padW, bias, out);
}

// The planes passes serve every layer in the tensor-core math mode; the element gathers remain for the
// FP32 FMA mode and for gradInput of strided convolutions.
static bool planes_forward_ok(const ConvGeom &g) { return ctx().math_mode != 1 && g.H < 16000 && g.W < 16000; }
static bool planes_grad_input_ok(const ConvGeom &g) {
  return planes_forward_ok(g) && g.dH == 1 && g.dW == 1 && g.pad <= g.kH - 1 && g.pad <= g.kW - 1;
}
static bool planes_acc_grad_ok(const ConvGeom &g) { return planes_forward_ok(g); }
// The raw-operand engine serves a layer when all three of its products can read plain FP32 planes by TMA (32-channel
// k tiles on both sides, two-SM tiles, expressible window boxes): then the input and gradOutput are transposed
// into ONE channels-last plane each, with no hi / lo copies.
static bool raw_window_product_ok(long N, long H, long W, long Cin, long Kout, long oH, long oW, int dH, int dW, int padH,
                                  int padW) {
  const bool pair = conv_pair_mode(N, Kout, oH, oW);
  const long oWr = pair ? (oW + 1) / 2 : oW;
  return mm::tc2_tile_width(N * oH * oWr, pair ? 2 * Kout : Kout) != 0 &&
         mm::raw_windows_ok(N, H, W, Cin, oH, oWr, dH, pair ? 2 * dW : dW, padH, padW);
}
static bool raw_layer_ok(const ConvGeom &g) {
  if (ctx().math_mode != 0 || !planes_forward_ok(g) || g.C % 32 != 0 || g.K % 32 != 0) return false;
  if (!raw_window_product_ok(g.N, g.H, g.W, g.C, g.K, g.oH, g.oW, g.dH, g.dW, g.pad, g.pad)) return false;
  if (planes_grad_input_ok(g) &&
      !raw_window_product_ok(g.N, g.oH, g.oW, g.K, g.C, g.H, g.W, 1, 1, g.kH - 1 - g.pad, g.kW - 1 - g.pad))
    return false;
  const long Rp = (long)g.kH * g.kW * g.C;
  return (mm::tc2_tile_width(g.K, Rp) != 0 || mm::tc2_tile_width(Rp, g.K) != 0) &&
         mm::raw_windows_ok(g.N, g.H, g.W, g.C, g.oH, g.oW, g.dH, g.dW, g.pad, g.pad);
}

// `finput`: when given, receives the input's planes (sized here), the counterpart of the column matrix the
// reference keeps there; accGradParameters reads them back instead of transposing the input again.
// A planes tensor is [2, N, H, W, Cp] (TF32 hi and lo planes) or [1, N, H, W, Cp] (the FP32 values, raw layers).
static mm::ActPlanes input_planes_into(const ConvGeom &g, const float *in, THGPUTensor *finput, bool raw) {
  float *dst = nullptr;
  if (finput) {
    const long s[5] = {raw ? 1 : 2, g.N, g.H, g.W, mm::planes_channels(g.C)};
    resize_nd(finput, 5, s, nullptr);
    if (is_contiguous(finput)) { dst = data_ptr(finput); stamp_planes(finput, in); }
  }
  return mm::make_act_planes(in, g.N, g.C, g.H * g.W, dst, raw);
}
// The planes the forward pass over this very input left in `finput`, if it holds any of the wanted kind.
static bool input_planes_from(const ConvGeom &g, const float *in, const THGPUTensor *finput, mm::ActPlanes &ap, bool raw) {
  if (!finput || finput->nDimension != 5 || !finput->storage || !is_contiguous(finput)) return false;
  if (!planes_made_from(finput, in)) return false;
  const long Cp = mm::planes_channels(g.C);
  if (finput->size[0] != (raw ? 1 : 2) || finput->size[1] != g.N || finput->size[2] != g.H || finput->size[3] != g.W ||
      finput->size[4] != Cp)
    return false;
  ap.hi = data_ptr(finput); ap.lo = raw ? nullptr : ap.hi + g.N * g.H * g.W * Cp; ap.Cp = Cp;
  return true;
}

static bool fold_layer_ok(const ConvGeom &g);
static void conv_forward_folded(const ConvGeom &g, const float *in, const float *w, const float *bias, float *out,
                                THGPUTensor *finput);
static void conv_forward_planes(const ConvGeom &g, const float *in, const float *w, const float *bias, float *out,
                                THGPUTensor *finput) {
  if (fold_layer_ok(g)) { conv_forward_folded(g, in, w, bias, out, finput); return; }
  mm::ActPlanes act = input_planes_into(g, in, finput, raw_layer_ok(g));
  conv_window_product(act, w, g.K, g.C, 0, g.N, g.H, g.W, g.K, g.oH, g.oW, g.kH, g.kW, g.dH, g.dW, g.pad, g.pad, bias, out);
}

// Stride 1: gradInput is the forward pass of gradOutput (K planes, oH x oW grid, padding k-1-pad) under the
// filter rotated by 180 degrees with its plane roles swapped.  `pgo`: planes of gradOutput.
static void conv_grad_input_planes(const ConvGeom &g, const mm::ActPlanes &pgo, const float *w, float *gin) {
  conv_window_product(pgo, w, g.K, g.C, 1, g.N, g.oH, g.oW, g.C, g.H, g.W, g.kH, g.kW, 1, 1, g.kH - 1 - g.pad,
                      g.kW - 1 - g.pad, nullptr, gin);
}

// gradW[ko][(c,i,j)] += scale * sum_{n,y,x} gradOut[n,ko,y,x] * in[n,c,y*dH-pad+i,x*dW-pad+j]: the reduction runs
// over pixels, along which neither tensor is contiguous in channels-last form, so both enter as MN-major
// operands.  The product lands in tmp[ko][(i,j,c)] and is folded into gradWeight's (c,i,j) order afterwards.
static void conv_acc_grad_planes(const ConvGeom &g, const mm::ActPlanes &pin, const mm::ActPlanes &pgo, float *gw,
                                 float scale) {
  using namespace mm;
  const long kHW = (long)g.kH * g.kW;
  const long Cp = pin.Cp, Kp = pgo.Cp, Rp = kHW * Cp;
  float *tmp = (float *)ws_alloc(sizeof(float) * g.K * Rp);
  if (!pin.lo) {
    // Raw layer: gradOutput's plane is a plain [pixels][Kp] matrix read along its rows; the input windows come by
    // im2col loads.  Either tensor may take the 256-row side of the product, whichever pads less.
    THC_CHECK(!pgo.lo, "internal: mixed plane kinds");
    WindowRowsOperand oi;
    set_window_map(oi.ks, g.N, g.oH, g.oW, g.H, g.W, Cp, g.dH, g.dW, g.pad, g.pad);
    oi.C = FastDiv::make(Cp); oi.kW = FastDiv::make(g.kW);
    attach_window_rows_map(oi, pin.hi, g.N, g.H, g.W, Cp, g.oH, g.oW, g.dH, g.dW, g.pad, g.pad);
    auto fill = [](long M, long N) {
      const int w = tc2_tile_width(M, N);
      if (!w) return 0.0;
      return (double)(M * N) / (double)(((M + 255) / 256 * 256) * ((N + w - 1) / w * w));
    };
    if (fill(g.K, Rp) >= fill(Rp, g.K)) {
      Problem<RawOperand<true>, WindowRowsOperand> p;
      p.b = oi;
      p.epi = Epilogue{tmp, nullptr, 1.f, 0.f, 1, Rp, 1};                 // tmp[m * Rp + n]
      p.M = g.K; p.N = Rp; p.K = g.N * g.P;
      launch_raw(p, [&](Problem<RawOperand<true>, WindowRowsOperand> &q, int) {
        attach_raw_map(q.a, pgo.hi, Kp, g.N * g.P, Kp, TC_BM);
      });
    } else {
      Problem<WindowRowsOperand, RawOperand<true>> p;
      p.a = oi;
      p.epi = Epilogue{tmp, nullptr, 1.f, 0.f, LONG_MAX, 0, Rp};          // tmp[n * Rp + m]
      p.M = Rp; p.N = g.K; p.K = g.N * g.P;
      launch_raw(p, [&](Problem<WindowRowsOperand, RawOperand<true>> &q, int bn2) {
        attach_raw_map(q.b, pgo.hi, Kp, g.N * g.P, Kp, bn2 / 2);
      });
    }
    int blocks = ceil_div(g.K * g.R, 256);
    if (blocks > ctx().sm_count * 8) blocks = ctx().sm_count * 8;
    unpack_grad_weight_kernel<<<blocks, 256, 0, stream()>>>(tmp, gw, g.K, g.C, kHW, Cp, scale);
    check_launch("unpack_grad_weight");
    return;
  }
  PlanesPixelOperand<false> og;   // gradOutput: rows = output planes, k = output pixels
  og.base = pgo.hi; og.lo = pgo.lo;
  og.rows = LinearMap{Kp, 1};
  og.ks.set(g.N * g.P, g.P, g.oW);
  og.ks.img_stride = g.P * Kp; og.ks.y_stride = g.oW * Kp; og.ks.x_stride = Kp; og.ks.off0 = 0;
  og.ks.sy = 0; og.ks.y0 = 0; og.ks.sx = 0; og.ks.x0 = 0;
  og.H = 1; og.W = 1; og.dH = og.dW = 1; og.vec4 = 1;
  og.C = FastDiv::make(Kp); og.kW = FastDiv::make(1); og.i_stride = og.j_stride = 0;
  PlanesPixelOperand<true> oi;    // input windows: rows = (tap, input plane), k = output pixels
  oi.base = pin.hi; oi.lo = pin.lo;
  oi.rows = LinearMap{Rp, 1};
  set_window_map(oi.ks, g.N, g.oH, g.oW, g.H, g.W, Cp, g.dH, g.dW, g.pad, g.pad);
  oi.H = (int)g.H; oi.W = (int)g.W; oi.dH = oi.dW = 1; oi.vec4 = 1;
  oi.C = FastDiv::make(Cp); oi.kW = FastDiv::make(g.kW);
  oi.i_stride = g.W * Cp; oi.j_stride = Cp;
  // Either tensor may take the M side (256-row tiles) of the product; pick the orientation that pads less.
  auto fill = [](long M, long N) {
    const int w = tc2_tile_width(M, N);
    const long bm = w ? 256 : 128, bn = w ? w : (N > 64 ? 128 : 64);
    return (double)(M * N) / (double)(((M + bm - 1) / bm * bm) * ((N + bn - 1) / bn * bn));
  };
  if (fill(g.K, Rp) >= fill(Rp, g.K)) {
    Problem<PlanesPixelOperand<false>, PlanesPixelOperand<true>> p;
    p.a = og; p.b = oi;
    p.epi = Epilogue{tmp, nullptr, 1.f, 0.f, 1, Rp, 1};                 // tmp[m * Rp + n]
    p.M = g.K; p.N = Rp; p.K = g.N * g.P;
    launch_planes(p);
  } else {
    Problem<PlanesPixelOperand<true>, PlanesPixelOperand<false>> p;
    p.a = oi; p.b = og;
    p.epi = Epilogue{tmp, nullptr, 1.f, 0.f, LONG_MAX, 0, Rp};          // tmp[n * Rp + m]
    p.M = Rp; p.N = g.K; p.K = g.N * g.P;
    launch_planes(p);
  }
  int blocks = ceil_div(g.K * g.R, 256);
  if (blocks > ctx().sm_count * 8) blocks = ctx().sm_count * 8;
  unpack_grad_weight_kernel<<<blocks, 256, 0, stream()>>>(tmp, gw, g.K, g.C, kHW, Cp, scale);
  check_launch("unpack_grad_weight");
}

// ------------------------------------------------------------------------------------------------
// Stride folding (tensor-core math mode): a strided layer with few input planes -- the 11x11 / stride 4 layer
// over 3 planes -- is restated as a stride-1 layer over "folded" pixels.  The dH x dW pixels of a stride cell
// become channels: S[n][Y][X][(dy, dx, c)] = in[n][c][Y*dH + dy - pad][X*dW + dx - pad], with c padded to a
// multiple of 4 so that a folded pixel holds Cs = dH*dW*Cq channels (64 for stride 4 over 3 planes).  Filter
// tap (i, j) becomes tap (i / dH, j / dW) of a ceil(kH/dH) x ceil(kW/dW) filter over channel (i % dH, j % dW, c),
// taps beyond the filter being zero weights.  The restated layer has 32-multiple channel counts and no
// stride, so its forward and weight-gradient products run on the raw-operand engine with im2col TMA loads
// instead of per-tap 16-byte thread copies (which left the 3-plane layer bound by L2 -> SM traffic).
struct FoldGeom {
  long Cq, Cs, Hs, Ws;
  int kHs, kWs;
};
static FoldGeom fold_geom(const ConvGeom &g) {
  FoldGeom f;
  f.Cq = mm::planes_channels(g.C);
  f.Cs = (long)g.dH * g.dW * f.Cq;
  f.kHs = (g.kH + g.dH - 1) / g.dH; f.kWs = (g.kW + g.dW - 1) / g.dW;
  f.Hs = g.oH + f.kHs - 1; f.Ws = g.oW + f.kWs - 1;
  return f;
}
// The restated layer: N, K and the output grid are those of the layer itself.
static ConvGeom folded_layer(const ConvGeom &g, const FoldGeom &f) {
  ConvGeom e = g;
  e.C = f.Cs; e.H = f.Hs; e.W = f.Ws; e.kH = f.kHs; e.kW = f.kWs; e.dH = e.dW = 1; e.pad = 0;
  e.R = f.Cs * f.kHs * f.kWs;
  return e;
}
static bool fold_layer_ok(const ConvGeom &g) {
  if (ctx().math_mode != 0 || !planes_forward_ok(g) || (g.dH == 1 && g.dW == 1) || g.K % 32 != 0) return false;
  if (raw_layer_ok(g)) return false;
  const FoldGeom f = fold_geom(g);
  if (f.Cs % 32 != 0 || f.Cs > 256) return false;
  if (g.N * f.Hs >= (1l << 31)) return false;
  // zero weights must not outnumber the real ones
  if (2 * g.R < f.Cs * f.kHs * f.kWs) return false;
  const long Rp = (long)f.kHs * f.kWs * f.Cs;
  return raw_window_product_ok(g.N, f.Hs, f.Ws, f.Cs, g.K, g.oH, g.oW, 1, 1, 0, 0) &&
         (mm::tc2_tile_width(g.K, Rp) != 0 || mm::tc2_tile_width(Rp, g.K) != 0);
}
// Planes of gradOutput come as one FP32 plane for raw and folded layers alike.
static bool raw_or_folded(const ConvGeom &g) { return raw_layer_ok(g) || fold_layer_ok(g); }

// One block per (image, folded row).  A thread produces one 16-byte chunk of a folded pixel: four planes at one
// (dy, dx) of stride cell X.  Neighbouring threads hold neighbouring dx, so for every plane a warp reads whole
// 32-byte runs of a few input rows (every sector it touches is used in full) and writes whole folded pixels.
static __global__ void __launch_bounds__(256) fold_input_kernel(const float *__restrict__ in, float *__restrict__ S, int C, int H,
                                                                int W, int dH, int dW, int pad, int Cq, int Hs, int Ws) {
  const long n = blockIdx.x / Hs;
  const int Y = (int)(blockIdx.x - n * Hs);
  const int cq4 = Cq / 4, q = dH * dW * cq4;   // 16-byte chunks per folded pixel
  const int quads = Ws * q;
  float4 *dst = reinterpret_cast<float4 *>(S + ((n * Hs + Y) * Ws) * (long)(4 * q));
  const float *img = in + n * C * (long)H * W;
  for (int o = threadIdx.x; o < quads; o += blockDim.x) {
    const int X = o / q, cp4 = o - X * q, c4 = cp4 % cq4, dxy = cp4 / cq4, dy = dxy / dW, dx = dxy - dy * dW;
    const int r = Y * dH + dy - pad, xx = X * dW + dx - pad;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (r >= 0 && r < H && xx >= 0 && xx < W) {
      const float *p = img + ((long)(4 * c4) * H + r) * W + xx;
#pragma unroll
      for (int e = 0; e < 4; e++)
        if (4 * c4 + e < C) v[e] = __ldg(p + (long)e * H * W);
    }
    dst[o] = make_float4(v[0], v[1], v[2], v[3]);
  }
}
// weff[ko][(c', bi, bj)] = w[ko][(c, bi*dH + dy, bj*dW + dx)], c' = (dy*dW + dx)*Cq + c: the folded layer's weight
// matrix in the layout of a SpatialConvolutionMM weight; taps and planes that do not exist are zero.
static __global__ void __launch_bounds__(256) fold_weight_kernel(const float *__restrict__ w, float *__restrict__ weff, long K, int C,
                                                                 int kH, int kW, int dH, int dW, int Cq, int kHs, int kWs) {
  const int Cs = dH * dW * Cq;
  const long total = K * Cs * kHs * kWs;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    long q = t;
    const int bj = (int)(q % kWs); q /= kWs;
    const int bi = (int)(q % kHs); q /= kHs;
    const int cp = (int)(q % Cs);
    const long ko = q / Cs;
    const int c = cp % Cq, dxy = cp / Cq, dx = dxy % dW, dy = dxy / dW, i = bi * dH + dy, j = bj * dW + dx;
    weff[t] = (c < C && i < kH && j < kW) ? w[((ko * C + c) * kH + i) * kW + j] : 0.f;
  }
}
// gw[ko][(c, i, j)] += gweff[ko][(c', i / dH, j / dW)]: the folded layer's weight gradient back in the layer's own order.
static __global__ void __launch_bounds__(256) unfold_grad_weight_kernel(const float *__restrict__ gweff, float *__restrict__ gw, long K,
                                                                        int C, int kH, int kW, int dH, int dW, int Cq, int kHs,
                                                                        int kWs) {
  const int Cs = dH * dW * Cq;
  const long total = K * C * kH * kW;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    long q = t;
    const int j = (int)(q % kW); q /= kW;
    const int i = (int)(q % kH); q /= kH;
    const int c = (int)(q % C);
    const long ko = q / C;
    const int cp = ((i % dH) * dW + (j % dW)) * Cq + c;
    gw[t] += gweff[((ko * Cs + cp) * kHs + i / dH) * kWs + j / dW];
  }
}

// gin[n][c][h][w] = gS[n][(dy, dx, c)][Y][X] with h + pad = Y*dH + dy, w + pad = X*dW + dx: the inverse of the fold,
// applied to the gradient of the folded input (NCHW over the folded grid).  Folding is a bijection between the
// padded input pixels and the (Y, X, dy, dx) cells, so every input pixel reads exactly one value; pixels below the
// last stride cell that any window reaches get zero.
static __global__ void __launch_bounds__(256) unfold_grad_input_kernel(const float *__restrict__ gS, float *__restrict__ gin, long N,
                                                                       int C, int H, int W, int dH, int dW, int pad, int Cq, int Hs,
                                                                       int Ws) {
  const long total = N * C * H * W;
  const long nthreads = (long)gridDim.x * blockDim.x;
  const int Cs = dH * dW * Cq;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const int w = (int)(t % W);
    long q = t / W;
    const int h = (int)(q % H); q /= H;
    const int c = (int)(q % C);
    const long n = q / C;
    const int Y = (h + pad) / dH, dy = (h + pad) - Y * dH, X = (w + pad) / dW, dx = (w + pad) - X * dW;
    float v = 0.f;
    if (Y < Hs && X < Ws) v = gS[((n * Cs + (dy * dW + dx) * Cq + c) * Hs + Y) * Ws + X];
    gin[t] = v;
  }
}

// The folded input of a layer, written into `finput` ([1, N, Hs, Ws, Cs]) when given.
static mm::ActPlanes folded_input_into(const ConvGeom &g, const FoldGeom &f, const float *in, THGPUTensor *finput) {
  mm::ActPlanes ap;
  ap.Cp = f.Cs; ap.lo = nullptr;
  float *dst = nullptr;
  if (finput) {
    const long s[5] = {1, g.N, f.Hs, f.Ws, f.Cs};
    resize_nd(finput, 5, s, nullptr);
    if (is_contiguous(finput)) { dst = data_ptr(finput); stamp_planes(finput, in); }
  }
  ap.hi = dst ? dst : (float *)ws_alloc(sizeof(float) * g.N * f.Hs * f.Ws * f.Cs);
  fold_input_kernel<<<(unsigned)(g.N * f.Hs), 256, 0, stream()>>>(in, ap.hi, (int)g.C, (int)g.H, (int)g.W, g.dH, g.dW, g.pad,
                                                                     (int)f.Cq, (int)f.Hs, (int)f.Ws);
  check_launch("fold_input");
  return ap;
}
static bool folded_input_from(const ConvGeom &g, const FoldGeom &f, const float *in, const THGPUTensor *finput,
                              mm::ActPlanes &ap) {
  if (!finput || finput->nDimension != 5 || !finput->storage || !is_contiguous(finput)) return false;
  if (!planes_made_from(finput, in)) return false;
  if (finput->size[0] != 1 || finput->size[1] != g.N || finput->size[2] != f.Hs || finput->size[3] != f.Ws ||
      finput->size[4] != f.Cs)
    return false;
  ap.hi = data_ptr(finput); ap.lo = nullptr; ap.Cp = f.Cs;
  return true;
}
static void conv_forward_folded(const ConvGeom &g, const float *in, const float *w, const float *bias, float *out,
                                THGPUTensor *finput) {
  const FoldGeom f = fold_geom(g);
  mm::ActPlanes act = folded_input_into(g, f, in, finput);
  const long wn = g.K * f.Cs * f.kHs * f.kWs;
  float *weff = (float *)ws_alloc(sizeof(float) * wn);
  fold_weight_kernel<<<ceil_div(wn, 256), 256, 0, stream()>>>(w, weff, g.K, (int)g.C, g.kH, g.kW, g.dH, g.dW, (int)f.Cq, f.kHs,
                                                             f.kWs);
  check_launch("fold_weight");
  conv_window_product(act, weff, g.K, f.Cs, 0, g.N, f.Hs, f.Ws, g.K, g.oH, g.oW, f.kHs, f.kWs, 1, 1, 0, 0, bias, out);
}
// gradInput of a folded layer = stride-1 gradInput of the folded filter over gradOutput (raw-operand engine, no
// masked taps, no 3 -> 64 plane padding) followed by the unfold.  `pgo`: gradOutput as one FP32 channels-last plane.
static bool fold_grad_input_ok(const ConvGeom &g) {
  if (!fold_layer_ok(g)) return false;
  const FoldGeom f = fold_geom(g);
  return raw_window_product_ok(g.N, g.oH, g.oW, g.K, f.Cs, f.Hs, f.Ws, 1, 1, f.kHs - 1, f.kWs - 1) &&
         g.N * f.Cs * f.Hs * f.Ws < (1l << 40);
}
static void conv_grad_input_folded(const ConvGeom &g, const mm::ActPlanes &pgo, const float *w, float *gin) {
  const FoldGeom f = fold_geom(g);
  const ConvGeom e = folded_layer(g, f);
  const long wn = g.K * e.R;
  float *weff = (float *)ws_alloc(sizeof(float) * wn);
  fold_weight_kernel<<<ceil_div(wn, 256), 256, 0, stream()>>>(w, weff, g.K, (int)g.C, g.kH, g.kW, g.dH, g.dW, (int)f.Cq, f.kHs,
                                                             f.kWs);
  check_launch("fold_weight");
  float *gS = (float *)ws_alloc(sizeof(float) * g.N * f.Cs * f.Hs * f.Ws);
  conv_grad_input_planes(e, pgo, weff, gS);
  const long total = g.N * g.C * g.H * g.W;
  long blocks = (total + 255) / 256;
  if (blocks > (long)ctx().sm_count * 16) blocks = (long)ctx().sm_count * 16;
  unfold_grad_input_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(gS, gin, g.N, (int)g.C, (int)g.H, (int)g.W, g.dH, g.dW, g.pad,
                                                                  (int)f.Cq, (int)f.Hs, (int)f.Ws);
  check_launch("unfold_grad_input");
}

// `pin`: the folded input; `pgo`: gradOutput as one FP32 channels-last plane.
// gw[ko][(c, i, j)] += scale * T[(i / dH, c')][(kWs - 1 - j / dW, ko)], c' = ((i % dH) * dW + j % dW) * Cq + c: the result of
// the shifted-columns product below back in the layer's own order.
static __global__ void __launch_bounds__(256) unfold_grad_weight_shifted_kernel(const float *__restrict__ T, float *__restrict__ gw,
                                                                                long K, int C, int kH, int kW, int dH, int dW,
                                                                                int Cq, int kWs, long Kp, float scale) {
  const int Cs = dH * dW * Cq;
  const long total = K * C * kH * kW, ncols = (long)kWs * Kp;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    long q = t;
    const int j = (int)(q % kW); q /= kW;
    const int i = (int)(q % kH); q /= kH;
    const int c = (int)(q % C);
    const long ko = q / C;
    const int cp = ((i % dH) * dW + (j % dW)) * Cq + c;
    gw[t] += scale * T[((long)(i / dH) * Cs + cp) * ncols + (long)(kWs - 1 - j / dW) * Kp + ko];
  }
}

// Weight gradient of a folded layer.  The folded filter has few output planes (64 for the 11 x 11 / 4 layer), which as
// the N side of the product means 64-wide tiles at half the tensor-pipe rate, and 576 rows that pad to 768.  So the
// filter's COLUMNS move to the N side instead: with the reduction running over the full folded width Ws,
//   T[(bi, c')][(j', ko)] = sum_{n, y, x'} S[n][y + bi][x'][c'] * gradOut[n][y][x' - (kWs - 1 - j')][ko]
// is the gradient of folded tap (bi, bj = kWs - 1 - j'): the column shift is a zero-padded window of the gradOutput
// plane, which TMA's im2col mode reads like any other.  A kHs * Cs x kWs * K product (192 x 192 for that layer): one
// full-rate tile, split along the reduction over all SM pairs.
static bool fold_acc_grad_shifted_ok(const ConvGeom &g, const FoldGeom &f, long Kp) {
  const long M = (long)f.kHs * f.Cs, N = (long)f.kWs * Kp;
  return Kp == g.K && mm::tc2_tile_width(M, N) != 0 && f.kWs - 1 <= 128 && g.N * g.oH * f.Ws < (1l << 31) &&
         mm::raw_windows_ok(g.N, f.Hs, f.Ws, f.Cs, g.oH, f.Ws, 1, 1, 0, 0) &&
         mm::raw_windows_ok(g.N, g.oH, g.oW, Kp, g.oH, f.Ws, 1, 1, 0, f.kWs - 1);
}
static void conv_acc_grad_folded_shifted(const ConvGeom &g, const FoldGeom &f, const mm::ActPlanes &pin, const mm::ActPlanes &pgo,
                                         float *gw, float scale) {
  using namespace mm;
  const long Kp = pgo.Cp, M = (long)f.kHs * f.Cs, Nc = (long)f.kWs * Kp;
  float *T = (float *)ws_alloc(sizeof(float) * M * Nc);
  Problem<WindowRowsOperand, WindowRowsOperand> p;
  // A: rows (bi, c') of the folded input, one column of taps; reduction grid [N, oH, Ws]
  set_window_map(p.a.ks, g.N, g.oH, f.Ws, f.Hs, f.Ws, f.Cs, 1, 1, 0, 0);
  p.a.C = FastDiv::make(f.Cs); p.a.kW = FastDiv::make(1);
  attach_window_rows_map(p.a, pin.hi, g.N, f.Hs, f.Ws, f.Cs, g.oH, f.Ws, 1, 1, 0, 0);
  // B: rows (j', ko) of gradOutput seen through a 1 x kWs window with kWs - 1 columns of zero padding on the left
  set_window_map(p.b.ks, g.N, g.oH, f.Ws, g.oH, g.oW, Kp, 1, 1, 0, f.kWs - 1);
  p.b.C = FastDiv::make(Kp); p.b.kW = FastDiv::make(f.kWs);
  attach_window_rows_map(p.b, pgo.hi, g.N, g.oH, g.oW, Kp, g.oH, f.Ws, 1, 1, 0, f.kWs - 1);
  p.epi = Epilogue{T, nullptr, 1.f, 0.f, 1, Nc, 1};                     // T[m * Nc + n]
  p.M = M; p.N = Nc; p.K = g.N * g.oH * f.Ws;
  launch_raw(p, [](Problem<WindowRowsOperand, WindowRowsOperand> &, int) {});
  unfold_grad_weight_shifted_kernel<<<ceil_div(g.K * g.R, 256), 256, 0, stream()>>>(T, gw, g.K, (int)g.C, g.kH, g.kW, g.dH, g.dW,
                                                                                   (int)f.Cq, f.kWs, Kp, scale);
  check_launch("unfold_grad_weight_shifted");
}

static void conv_acc_grad_folded(const ConvGeom &g, const mm::ActPlanes &pin, const mm::ActPlanes &pgo, float *gw, float scale) {
  const FoldGeom f = fold_geom(g);
  if (fold_acc_grad_shifted_ok(g, f, pgo.Cp)) { conv_acc_grad_folded_shifted(g, f, pin, pgo, gw, scale); return; }
  const ConvGeom e = folded_layer(g, f);
  const long wn = g.K * e.R;
  float *gweff = (float *)ws_alloc(sizeof(float) * wn);
  THC_CUDA(cudaMemsetAsync(gweff, 0, sizeof(float) * wn, stream()));
  conv_acc_grad_planes(e, pin, pgo, gweff, scale);
  unfold_grad_weight_kernel<<<ceil_div(g.K * g.R, 256), 256, 0, stream()>>>(gweff, gw, g.K, (int)g.C, g.kH, g.kW, g.dH, g.dW,
                                                                           (int)f.Cq, f.kHs, f.kWs);
  check_launch("unfold_grad_weight");
}

// ------------------------------------------------------------------------------------------------
// BF16 math mode (opt-in): the same three passes over one BF16 plane per tensor on the BF16 engine.  Offsets
// of the operands count 4-byte units (pairs of BF16 values).  Products too small for the two-SM tile run
// on the FP32-accurate paths above.
static __nv_bfloat16 *make_weight_half(const float *w, long K, long C, long kHW, long Cp, long Kp, int flip, long *ld_out) {
  const long rows = flip ? C : K;
  const long ld = (kHW * (flip ? Kp : Cp) + 63) / 64 * 64;
  __nv_bfloat16 *out = (__nv_bfloat16 *)ws_alloc(sizeof(__nv_bfloat16) * rows * ld);
  int blocks = ceil_div(rows * ld, 256);
  if (blocks > ctx().sm_count * 8) blocks = ctx().sm_count * 8;
  mm::repack_weight_bf16_kernel<<<blocks, 256, 0, stream()>>>(w, K, C, kHW, Cp, Kp, ld, flip, out);
  check_launch("repack_weight_bf16");
  *ld_out = ld;
  return out;
}
// windows of a BF16 plane [N, H, W, Cp] seen from the output grid, offsets in 4-byte units
static void set_window_map_half(mm::PixelMap &m, long N, long oH, long oW, long H, long W, long Cu, int dH, int dW, int padH,
                                int padW) {
  m.set(N * oH * oW, oH * oW, oW);
  m.img_stride = H * W * Cu; m.y_stride = dH * W * Cu; m.x_stride = dW * Cu;
  m.off0 = -((long)padH * W + padW) * Cu;
  m.sy = dH; m.y0 = -padH; m.sx = dW; m.x0 = -padW;
}
static void conv_window_product_half(const mm::HalfActPlane &act, const __nv_bfloat16 *wp, long wld, long N, long H, long W,
                                     long Kout, long oH, long oW, int kH, int kW, int dH, int dW, int padH, int padW,
                                     const float *bias, float *out) {
  using namespace mm;
  Problem<PlanesWindowOperand, SplitOperand> p;
  const long Cu = act.Cp / 2;
  p.a.base = reinterpret_cast<const float *>(act.p); p.a.lo = nullptr;
  p.a.use_tma = 0; p.a.n_img = 0; p.a.n_planes = 1; p.a.ctiles = FastDiv::make(1);
  set_window_map_half(p.a.rows, N, oH, oW, H, W, Cu, dH, dW, padH, padW);
  p.a.ks = LinearMap{wld / 2, 1};
  p.a.H = (int)H; p.a.W = (int)W; p.a.dH = p.a.dW = 1; p.a.vec4 = 1;
  p.a.cquads = FastDiv::make(Cu / 4);
  p.a.kW = FastDiv::make(kW);
  p.a.taps = (unsigned)(kH * kW);
  p.a.i_stride = W * Cu; p.a.j_stride = Cu;
  p.b = half_operand(wp, Kout, wld);
  p.epi = Epilogue{out, bias, 1.f, 0.f, oH * oW, Kout * oH * oW, oH * oW};
  p.M = N * oH * oW; p.N = Kout; p.K = wld / 2;
  launch_planes_half(p);
}
static bool half_forward_ok(const ConvGeom &g) {
  return ctx().math_mode == 2 && planes_forward_ok(g) && mm::tc2h_tile_width(g.N * g.P, g.K, false);
}
static bool half_grad_input_ok(const ConvGeom &g) {
  return ctx().math_mode == 2 && planes_grad_input_ok(g) && mm::tc2h_tile_width(g.N * g.H * g.W, g.C, false);
}
// the weight gradient needs whole 64-channel blocks on its N side; which tensor goes there is free
static int half_acc_grad_orientation(const ConvGeom &g) {
  if (ctx().math_mode != 2 || !planes_acc_grad_ok(g)) return 0;
  const long Kp = (g.K + 7) / 8 * 8, Rp = (long)g.kH * g.kW * ((g.C + 7) / 8 * 8);
  auto fill = [](long M, long N) {
    const int w = mm::tc2h_tile_width(M, N, true);
    if (!w) return 0.0;
    return (double)(M * N) / (double)(((M + 255) / 256 * 256) * ((N + w - 1) / w * w));
  };
  const double f1 = fill(Kp, Rp), f2 = fill(Rp, Kp);
  if (f1 == 0.0 && f2 == 0.0) return 0;
  return f1 >= f2 ? 1 : 2;
}
static void conv_forward_half(const ConvGeom &g, const float *in, const float *w, const float *bias, float *out) {
  mm::HalfActPlane act = mm::make_half_act_plane(in, g.N, g.C, g.H * g.W);
  long wld;
  __nv_bfloat16 *wp = make_weight_half(w, g.K, g.C, (long)g.kH * g.kW, act.Cp, 0, 0, &wld);
  conv_window_product_half(act, wp, wld, g.N, g.H, g.W, g.K, g.oH, g.oW, g.kH, g.kW, g.dH, g.dW, g.pad, g.pad, bias, out);
}
static void conv_grad_input_half(const ConvGeom &g, const float *gout, const float *w, float *gin) {
  mm::HalfActPlane act = mm::make_half_act_plane(gout, g.N, g.K, g.P);
  long wld;
  __nv_bfloat16 *wp = make_weight_half(w, g.K, g.C, (long)g.kH * g.kW, 0, act.Cp, 1, &wld);
  conv_window_product_half(act, wp, wld, g.N, g.oH, g.oW, g.C, g.H, g.W, g.kH, g.kW, 1, 1, g.kH - 1 - g.pad,
                           g.kW - 1 - g.pad, nullptr, gin);
}
static void conv_acc_grad_half(const ConvGeom &g, const float *in, const float *gout, float *gw, float scale, int orient) {
  using namespace mm;
  const long kHW = (long)g.kH * g.kW;
  HalfActPlane pin = make_half_act_plane(in, g.N, g.C, g.H * g.W);
  HalfActPlane pgo = make_half_act_plane(gout, g.N, g.K, g.P);
  const long Cp = pin.Cp, Kp = pgo.Cp, Rp = kHW * Cp, Cu = Cp / 2, Ku = Kp / 2;
  float *tmp = (float *)ws_alloc(sizeof(float) * g.K * Rp);
  PlanesPixelOperand<false> og;   // gradOutput: rows = output planes (in pairs), k = output pixels
  og.base = reinterpret_cast<const float *>(pgo.p); og.lo = nullptr;
  og.rows = LinearMap{Ku, 1};
  og.ks.set(g.N * g.P, g.P, g.oW);
  og.ks.img_stride = g.P * Ku; og.ks.y_stride = g.oW * Ku; og.ks.x_stride = Ku; og.ks.off0 = 0;
  og.ks.sy = 0; og.ks.y0 = 0; og.ks.sx = 0; og.ks.x0 = 0;
  og.H = 1; og.W = 1; og.dH = og.dW = 1; og.vec4 = 1;
  og.C = FastDiv::make(Ku); og.kW = FastDiv::make(1); og.i_stride = og.j_stride = 0;
  PlanesPixelOperand<true> oi;    // input windows: rows = (tap, input plane pairs), k = output pixels
  oi.base = reinterpret_cast<const float *>(pin.p); oi.lo = nullptr;
  oi.rows = LinearMap{kHW * Cu, 1};
  set_window_map_half(oi.ks, g.N, g.oH, g.oW, g.H, g.W, Cu, g.dH, g.dW, g.pad, g.pad);
  oi.H = (int)g.H; oi.W = (int)g.W; oi.dH = oi.dW = 1; oi.vec4 = 1;
  oi.C = FastDiv::make(Cu); oi.kW = FastDiv::make(g.kW);
  oi.i_stride = g.W * Cu; oi.j_stride = Cu;
  if (orient == 1) {
    Problem<PlanesPixelOperand<false>, PlanesPixelOperand<true>> p;
    p.a = og; p.b = oi;
    p.epi = Epilogue{tmp, nullptr, 1.f, 0.f, 1, Rp, 1};                 // tmp[m * Rp + n]
    p.M = g.K; p.N = Rp; p.K = g.N * g.P;
    launch_planes_half(p);
  } else {
    Problem<PlanesPixelOperand<true>, PlanesPixelOperand<false>> p;
    p.a = oi; p.b = og;
    p.epi = Epilogue{tmp, nullptr, 1.f, 0.f, LONG_MAX, 0, Rp};          // tmp[n * Rp + m]
    p.M = Rp; p.N = g.K; p.K = g.N * g.P;
    launch_planes_half(p);
  }
  int blocks = ceil_div(g.K * g.R, 256);
  if (blocks > ctx().sm_count * 8) blocks = ctx().sm_count * 8;
  unpack_grad_weight_kernel<<<blocks, 256, 0, stream()>>>(tmp, gw, g.K, g.C, kHW, Cp, scale);
  check_launch("unpack_grad_weight");
}

template <class OpB>
static void conv_forward_with(const ConvGeom &g, const float *in, const OpB &b, const float *bias, float *out) {
  using namespace mm;
  typedef Operand<PixelMap, TapMap, 1, false> OpA;     // im2col rows: output pixels, contiguous along x
  Problem<OpA, OpB> p;
  p.a.base = in; p.a.rows = input_windows(g); p.a.ks = input_taps(g);
  p.a.H = (int)g.H; p.a.W = (int)g.W; p.a.dH = p.a.dW = 1; p.a.vec4 = 0;
  p.b = b;
  p.epi = Epilogue{out, bias, 1.f, 0.f, g.P, g.K * g.P, g.P};
  p.M = g.N * g.P; p.N = g.K; p.K = g.R;
  launch(p);
}

static void conv_forward(const ConvGeom &g, const float *in, const float *w, const float *bias, float *out,
                         THGPUTensor *finput) {
  using namespace mm;
  if (planes_forward_ok(g) && !half_forward_ok(g)) { conv_forward_planes(g, in, w, bias, out, finput); return; }
  forget_planes(finput);   // the passes below leave finput alone: what it holds belongs to an earlier input
  if (half_forward_ok(g)) { conv_forward_half(g, in, w, bias, out); return; }
  if (ctx().math_mode != 1) {  // tensor cores: the weight matrix is rounded into hi / lo planes once per call
    SplitPlanes pw = make_split_planes(w, g.R, 1, g.K, g.R);
    conv_forward_with(g, in, split_operand(pw, g.K), bias, out);
    return;
  }
  typedef Operand<LinearMap, LinearMap, 0, true> OpB;  // weight [K, R], contiguous along k
  OpB b;
  b.base = w; b.rows = LinearMap{g.K, g.R}; b.ks = LinearMap{g.R, 1};
  b.H = b.W = 0; b.dH = b.dW = 1;
  b.vec4 = (((uintptr_t)w & 15) == 0 && g.R % 4 == 0) ? 1 : 0;
  conv_forward_with(g, in, b, bias, out);
}

// Wt[c][(ko, i, j)] = W[ko][(c, i, j)]: the weight matrix as the gradInput product reads it, so that its
// k runs are contiguous (16-byte copies) instead of a tap gather.
static __global__ void __launch_bounds__(256) repack_weight_kernel(const float *__restrict__ w, float *__restrict__ wt,
                                                                   long K, long C, long kHW) {
  const long total = K * C * kHW;
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const long tap = t % kHW, q = t / kHW, ko = q % K, c = q / K;
    wt[t] = w[(ko * C + c) * kHW + tap];
  }
}

template <class OpB>
static void conv_grad_input_with(const ConvGeom &g, const float *gout, const OpB &b, float *gin) {
  using namespace mm;
  const long kHW = (long)g.kH * g.kW, Kd = g.K * kHW;
  PixelMap rows;  // (img, h, w) input pixels
  rows.set(g.N * g.H * g.W, g.H * g.W, g.W);
  rows.img_stride = g.K * g.P;
  rows.sy = 1; rows.y0 = g.pad; rows.sx = 1; rows.x0 = g.pad;
  TapMap ks;  // (ko, i, j)
  ks.set(Kd, kHW, g.kW); ks.c_stride = g.P; ks.si = -1; ks.sj = -1;
  Epilogue epi{gin, nullptr, 1.f, 0.f, g.H * g.W, g.C * g.H * g.W, g.H * g.W};
  if (g.dH == 1 && g.dW == 1) {
    // y = h + pad - i, x = w + pad - j are linear in the maps: fold them into the offsets
    typedef Operand<PixelMap, TapMap, 1, false> OpA;
    Problem<OpA, OpB> p;
    rows.y_stride = g.oW; rows.x_stride = 1; rows.off0 = (long)g.pad * g.oW + g.pad;
    ks.i_stride = -g.oW; ks.j_stride = -1;
    p.a.base = gout; p.a.rows = rows; p.a.ks = ks; p.a.H = (int)g.oH; p.a.W = (int)g.oW; p.a.dH = p.a.dW = 1; p.a.vec4 = 0;
    p.b = b; p.epi = epi; p.M = rows.count; p.N = g.C; p.K = Kd;
    launch(p);
  } else {
    typedef Operand<PixelMap, TapMap, 2, false> OpA;  // only taps with (h+pad-i) % dH == 0 contribute
    Problem<OpA, OpB> p;
    rows.y_stride = 0; rows.x_stride = 0; rows.off0 = 0;
    ks.i_stride = 0; ks.j_stride = 0;
    p.a.base = gout; p.a.rows = rows; p.a.ks = ks; p.a.H = (int)g.oH; p.a.W = (int)g.oW; p.a.dH = g.dH; p.a.dW = g.dW; p.a.vec4 = 0;
    p.b = b; p.epi = epi; p.M = rows.count; p.N = g.C; p.K = Kd;
    launch(p);
  }
}

static void conv_grad_input(const ConvGeom &g, const float *gout, const float *w, float *gin,
                            const mm::ActPlanes *pgo_ready = nullptr) {
  using namespace mm;
  if (half_grad_input_ok(g)) { conv_grad_input_half(g, gout, w, gin); return; }
  if (fold_grad_input_ok(g)) {
    ActPlanes pgo = pgo_ready ? *pgo_ready : make_act_planes(gout, g.N, g.K, g.P, nullptr, true);
    conv_grad_input_folded(g, pgo, w, gin);
    return;
  }
  if (planes_grad_input_ok(g)) {
    ActPlanes pgo = pgo_ready ? *pgo_ready : make_act_planes(gout, g.N, g.K, g.P, nullptr, raw_layer_ok(g));
    conv_grad_input_planes(g, pgo, w, gin);
    return;
  }
  const long kHW = (long)g.kH * g.kW, Kd = g.K * kHW;
  float *wt = (float *)ws_alloc(sizeof(float) * g.C * Kd);
  {
    int blocks = ceil_div(g.C * Kd, 256);
    if (blocks > ctx().sm_count * 8) blocks = ctx().sm_count * 8;
    repack_weight_kernel<<<blocks, 256, 0, stream()>>>(w, wt, g.K, g.C, kHW);
    check_launch("repack_weight");
  }
  if (ctx().math_mode != 1) {
    SplitPlanes pw = make_split_planes(wt, Kd, 1, g.C, Kd);
    conv_grad_input_with(g, gout, split_operand(pw, g.C), gin);
  } else {
    typedef Operand<LinearMap, LinearMap, 0, true> OpB;  // B(c, (ko,i,j)) = Wt[c][(ko,i,j)]
    OpB b;
    b.base = wt; b.rows = LinearMap{g.C, Kd}; b.ks = LinearMap{Kd, 1};
    b.H = b.W = 0; b.dH = b.dW = 1;
    b.vec4 = (((uintptr_t)wt & 15) == 0 && Kd % 4 == 0) ? 1 : 0;
    conv_grad_input_with(g, gout, b, gin);
  }
}

// gradBias[k] += scale * sum_{img, p} gradOut[img, k, p].  Pass 1: block (k, s) sums the images
// s, s+S, ... of plane k into partial[k][s]; pass 2 folds the S partials in order (deterministic).
static __global__ void __launch_bounds__(256) conv_grad_bias_partial_kernel(const float *__restrict__ gout,
                                                                            float *__restrict__ partial, long N, long K,
                                                                            long P) {
  __shared__ float sm[8];
  const long k = blockIdx.x;
  // One image per warp at a time (eight images in flight per block), four independent partial sums per lane:
  // with one dependent load chain per thread, or one image per block, small planes (13 x 13) left the kernel
  // waiting on memory latency.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (long img = blockIdx.y + (long)warp * gridDim.y; img < N; img += 8l * gridDim.y) {
    const float *g = gout + (img * K + k) * P;
    long p = lane;
    for (; p + 96 < P; p += 128) { a0 += g[p]; a1 += g[p + 32]; a2 += g[p + 64]; a3 += g[p + 96]; }
    for (; p < P; p += 32) a0 += g[p];
  }
  float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < 8 ? sm[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) partial[k * gridDim.y + blockIdx.y] = acc;
  }
}
static __global__ void conv_grad_bias_finish_kernel(const float *__restrict__ partial, float *gbias, long K, int S,
                                                    float scale) {
  const long k = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  float acc = 0.f;
  for (int s = 0; s < S; s++) acc += partial[k * S + s];
  gbias[k] += scale * acc;
}

static void conv_acc_grad(const ConvGeom &g, const float *in, const float *gout, float *gw, float *gb, float scale,
                          const THGPUTensor *finput, const mm::ActPlanes *pgo_ready = nullptr) {
  using namespace mm;
  typedef Operand<TapMap, PixelMap, 1, true> OpA;     // A(r, (img,y,x)) = input under tap r of window (img,y,x)
  const Epilogue epi{gw, nullptr, scale, 1.f, LONG_MAX, 0, g.R};
  if (const int orient = half_acc_grad_orientation(g)) {
    conv_acc_grad_half(g, in, gout, gw, scale, orient);
  } else if (planes_acc_grad_ok(g)) {
    // the input's planes: those the forward pass left in finput (as the CPU nn path reuses its finput,
    // mcw_nn/generic/SpatialConvolutionMM.c:284-346), else made here
    const bool folded = fold_layer_ok(g), raw = folded || raw_layer_ok(g);
    ActPlanes pin;
    if (folded) {
      const FoldGeom f = fold_geom(g);
      if (!folded_input_from(g, f, in, finput, pin)) pin = folded_input_into(g, f, in, nullptr);
    } else if (!input_planes_from(g, in, finput, pin, raw)) {
      pin = make_act_planes(in, g.N, g.C, g.H * g.W, nullptr, raw);
    }
    ActPlanes pgo = pgo_ready ? *pgo_ready : make_act_planes(gout, g.N, g.K, g.P, nullptr, raw, true);
    if (folded) conv_acc_grad_folded(g, pin, pgo, gw, scale);
    else conv_acc_grad_planes(g, pin, pgo, gw, scale);
    if (pgo.chan_partial) {
      // gradBias came along with the transposition of gradOutput
      chan_partial_finish_kernel<<<ceil_div(g.K, 32), 1024, 0, stream()>>>(pgo.chan_partial, pgo.chan_blocks, g.K, gb, scale);
      check_launch("conv_grad_bias_finish");
      return;
    }
  } else if (ctx().math_mode != 1) {
    // gradOut becomes hi / lo planes [img][ko][Ppad] (Ppad = P rounded up to 32, zeros in the padding), so
    // the reduction index is k = img * Ppad + p and a k tile never straddles two images; the gathered
    // operand uses the same padded indexing (its padding pixels read as zero).
    SplitPlanes pg = make_split_planes(gout, g.P, 1, g.N * g.K, g.P);
    const long Ppad = pg.ld;
    Problem<OpA, SplitOperand> p;
    p.a.base = in; p.a.rows = input_taps(g); p.a.ks = input_windows(g);
    p.a.ks.set(g.N * Ppad, Ppad, g.oW, g.P);
    p.a.H = (int)g.H; p.a.W = (int)g.W; p.a.dH = p.a.dW = 1; p.a.vec4 = 0;
    p.b = split_operand(pg, g.K);
    p.b.k_inner = FastDiv::make(Ppad);
    p.b.k_outer_stride = g.K * Ppad;
    p.epi = epi;
    p.M = g.R; p.N = g.K; p.K = g.N * Ppad;
    launch(p);
  } else {
    typedef Operand<LinearMap, PixelMap, 0, true> OpB;  // B(ko, (img,p)) = gradOut[img, ko, p]
    Problem<OpA, OpB> p;
    p.a.base = in; p.a.rows = input_taps(g); p.a.ks = input_windows(g);
    p.a.H = (int)g.H; p.a.W = (int)g.W; p.a.dH = p.a.dW = 1;
    p.b.base = gout; p.b.rows = LinearMap{g.K, g.P};
    p.b.ks.set(g.N * g.P, g.P, g.P);
    p.b.ks.img_stride = g.K * g.P; p.b.ks.y_stride = 0; p.b.ks.x_stride = 1; p.b.ks.off0 = 0;
    p.b.ks.sy = 0; p.b.ks.y0 = 0; p.b.ks.sx = 0; p.b.ks.x0 = 0;
    p.b.H = p.b.W = 0; p.b.dH = p.b.dW = 1;
    p.a.vec4 = 0; p.b.vec4 = 0;
    p.epi = epi;
    p.M = g.R; p.N = g.K; p.K = g.N * g.P;
    launch(p);
  }
  long S = (long)ctx().sm_count * 8 / g.K;
  if (S > g.N) S = g.N;
  if (S < 1) S = 1;
  float *partial = (float *)ws_alloc(sizeof(float) * g.K * S);
  conv_grad_bias_partial_kernel<<<dim3((unsigned)g.K, (unsigned)S), 256, 0, stream()>>>(gout, partial, g.N, g.K, g.P);
  check_launch("conv_grad_bias_partial");
  conv_grad_bias_finish_kernel<<<ceil_div(g.K, 128), 128, 0, stream()>>>(partial, gb, g.K, (int)S, scale);
  check_launch("conv_grad_bias_finish");
}

static void check_grad_output(const ConvGeom &g, const THGPUTensor *gradOutput) {
  const int o = g.batch ? 1 : 0;
  THC_ARG(gradOutput->nDimension == (g.batch ? 4 : 3), 3, "gradOutput must have the rank of the output");
  THC_ARG(gradOutput->size[o] == g.K, 1, "Number of output features is not equal to nOutputPlane");
  THC_ARG(gradOutput->size[o + 1] == g.oH && gradOutput->size[o + 2] == g.oW && (!g.batch || gradOutput->size[0] == g.N), 3,
          "gradOutput has the wrong size");
}

}  // namespace thc

using namespace thc;

THC_API int THGPUNN_SpatialConvolutionMM_updateOutput(THGPUTensor *input, THGPUTensor *output, THGPUTensor *weight,
    THGPUTensor *bias, THGPUTensor *finput, THGPUTensor *fgradInput, int kW, int kH, int dW, int dH, int padding) {
  (void)fgradInput;
  THC_BEGIN
  WsScope ws_scope;
  const ConvGeom g = conv_geom(input, weight, kW, kH, dW, dH, padding);
  THC_ARG(bias->nDimension == 1 && bias->size[0] == g.K, 1, "bias must have nOutputPlane entries");
  TensorRef in(tensor_new_contiguous(input)); TensorRef w(tensor_new_contiguous(weight)); TensorRef b(tensor_new_contiguous(bias));
  if (g.batch) { const long s[4] = {g.N, g.K, g.oH, g.oW}; resize_nd(output, 4, s, nullptr); }
  else { const long s[3] = {g.K, g.oH, g.oW}; resize_nd(output, 3, s, nullptr); }
  THC_CHECK(is_contiguous(output), "output must be contiguous");
  conv_forward(g, data_ptr(in), data_ptr(w), data_ptr(b), data_ptr(output), finput);
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SpatialConvolutionMM_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradInput,
    THGPUTensor *weight, THGPUTensor *finput, THGPUTensor *fgradInput, int kW, int kH, int dW, int dH, int padding) {
  (void)finput; (void)fgradInput;
  THC_BEGIN
  WsScope ws_scope;
  const ConvGeom g = conv_geom(input, weight, kW, kH, dW, dH, padding);
  check_grad_output(g, gradOutput);
  TensorRef go(tensor_new_contiguous(gradOutput)); TensorRef w(tensor_new_contiguous(weight));
  tensor_resize_as(gradInput, input);
  THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
  conv_grad_input(g, data_ptr(go), data_ptr(w), data_ptr(gradInput));
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SpatialConvolutionMM_accGradParameters(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradWeight,
    THGPUTensor *gradBias, THGPUTensor *finput, THGPUTensor *fgradInput, int kW, int kH, int dW, int dH, int padding, float scale) {
  (void)fgradInput;
  THC_BEGIN
  WsScope ws_scope;
  const ConvGeom g = conv_geom(input, gradWeight, kW, kH, dW, dH, padding);
  check_grad_output(g, gradOutput);
  THC_ARG(gradBias->nDimension == 1 && gradBias->size[0] == g.K, 1, "gradBias must have nOutputPlane entries");
  THC_CHECK(is_contiguous(gradWeight) && is_contiguous(gradBias), "gradWeight / gradBias must be contiguous");
  TensorRef in(tensor_new_contiguous(input)); TensorRef go(tensor_new_contiguous(gradOutput));
  conv_acc_grad(g, data_ptr(in), data_ptr(go), data_ptr(gradWeight), data_ptr(gradBias), scale, finput);
  return 0;
  THC_END(1)
}

// updateGradInput (skipped when gradInput is null) followed by accGradParameters, sharing one transposition of
// gradOutput.  The reference has no such entry: nn.Module:backward calls the two methods one after the other
// (mcw_nn/Module.lua), and a GPU module may override backward with this.
THC_API int THGPUNN_SpatialConvolutionMM_backward(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradInput,
    THGPUTensor *weight, THGPUTensor *gradWeight, THGPUTensor *gradBias, THGPUTensor *finput, THGPUTensor *fgradInput,
    int kW, int kH, int dW, int dH, int padding, float scale) {
  (void)fgradInput;
  THC_BEGIN
  WsScope ws_scope;
  const ConvGeom g = conv_geom(input, weight, kW, kH, dW, dH, padding);
  check_grad_output(g, gradOutput);
  THC_ARG(gradWeight->nDimension == 2 && gradWeight->size[0] == g.K && gradWeight->size[1] == g.R, 1,
          "gradWeight must have the shape of weight");
  THC_ARG(gradBias->nDimension == 1 && gradBias->size[0] == g.K, 1, "gradBias must have nOutputPlane entries");
  THC_CHECK(is_contiguous(gradWeight) && is_contiguous(gradBias), "gradWeight / gradBias must be contiguous");
  TensorRef in(tensor_new_contiguous(input)); TensorRef go(tensor_new_contiguous(gradOutput)); TensorRef w(tensor_new_contiguous(weight));
  mm::ActPlanes pgo;
  const bool share = planes_acc_grad_ok(g) && ctx().math_mode == 0;
  if (share) pgo = mm::make_act_planes(data_ptr(go), g.N, g.K, g.P, nullptr, raw_or_folded(g), true);
  if (gradInput) {
    tensor_resize_as(gradInput, input);
    THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
    conv_grad_input(g, data_ptr(go), data_ptr(w), data_ptr(gradInput), share ? &pgo : nullptr);
  }
  conv_acc_grad(g, data_ptr(in), data_ptr(go), data_ptr(gradWeight), data_ptr(gradBias), scale, finput, share ? &pgo : nullptr);
  return 0;
  THC_END(1)
}
