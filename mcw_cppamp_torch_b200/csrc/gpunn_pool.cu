// nn.SpatialMaxPooling on torch.GPUTensor.
//
// Forward follows gputorch/lib/THC/gpunn-impl/SpatialMaxPooling.cpp:9-81,205-281 and the CPU
// kernel mcw_nn/generic/SpatialMaxPooling.c:5-56: window scanned rows-then-columns with a strict
// '>' so the first maximum wins; `indices` is a float tensor [2, (N,) C, oH, oW] holding the 1-based
// window-local row (plane 0) and column (plane 1) of the maximum.
// Backward: the reference GPU code only handled non-overlapping windows (:293-294) with a scatter;
// here every INPUT pixel gathers from the (at most ceil(kH/dH)*ceil(kW/dW)) windows that cover it,
// visiting them in ascending (y, x) order, which is the order in which the CPU loop
// (mcw_nn/generic/SpatialMaxPooling.c:147-176) adds them: no atomics, deterministic, and bit-equal
// to the CPU result for overlapping windows too.
#include <cfloat>

#include "thc_internal.h"

namespace thc {

// 31-bit division by a runtime constant (multiply-high + shift): the kernels below decompose flat
// indices on every element, which 64-bit hardware division made the dominant cost.
struct Div32 {
  unsigned d, mul, shr;
  static Div32 make(long divisor) {
    Div32 f;
    f.d = (unsigned)divisor;
    if (divisor <= 1) { f.mul = 0; f.shr = 0; return f; }
    int lg = 0;
    while ((1l << lg) < divisor) lg++;
    const int p = 31 + lg;
    f.mul = (unsigned)(((1ull << p) + (unsigned long long)divisor - 1) / (unsigned long long)divisor);
    f.shr = (unsigned)(p - 32);
    return f;
  }
  __device__ __forceinline__ unsigned div(unsigned n) const { return d > 1 ? (__umulhi(n, mul) >> shr) : n; }
};

// grid.y strides over planes, grid.x * block over the plane's outputs: no division by the plane size.
// KH, KW, DH, DW: compile-time window and stride (0 = use the runtime arguments); the common 3x3 / 2 and
// 2x2 / 2 windows get fully unrolled scans and shifts instead of divisions.
template <int KH, int KW, int DH, int DW>
static __global__ void __launch_bounds__(256) maxpool_forward_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                                     float *__restrict__ indy, float *__restrict__ indx,
                                                                     long planes, int H, int W, int oH, int oW, Div32 doW,
                                                                     int kH_, int kW_, int dH_, int dW_) {
  const int kH = KH ? KH : kH_, kW = KW ? KW : kW_, dH = DH ? DH : dH_, dW = DW ? DW : dW_;
  const unsigned P = (unsigned)(oH * oW);
  for (long plane = blockIdx.y; plane < planes; plane += gridDim.y) {
    const float *ip0 = in + plane * H * W;
    const long ob = plane * P;
    for (unsigned t = blockIdx.x * blockDim.x + threadIdx.x; t < P; t += gridDim.x * blockDim.x) {
      const unsigned y = doW.div(t), x = t - y * oW;
      const float *ip = ip0 + (y * dH) * W + x * dW;
      float best = -INFINITY;  // the CPU starts from (float)(-DBL_MAX) = -inf
      int bi = -1, cnt = 0;
#pragma unroll
      for (int i = 0; i < kH; i++)
#pragma unroll
        for (int j = 0; j < kW; j++) {
          const float v = ip[i * W + j];
          if (v > best) { best = v; bi = cnt; }
          cnt++;
        }
      out[ob + t] = best;
      // bi == -1 (all NaN / -inf) reproduces the CPU's (int)(-1 / kW) + 1 and (-1 % kW) + 1
      indy[ob + t] = (float)(bi / kW + 1);
      indx[ob + t] = (float)(bi % kW + 1);
    }
  }
}

// One work item = G consecutive planes (small planes) or one band of input rows of one plane (large planes).
// Phase 1 turns every window that can reach the item's pixels into (flat position of its maximum, gradOutput
// value) in shared memory, reading indices and gradOutput exactly once and coalesced; phase 2 lets every input
// pixel scan the windows covering it.  Global traffic is the algorithmic minimum.
static __device__ __forceinline__ float *gi_plane(float *gin, long plane, int HW) { return gin + plane * HW; }

template <int KH, int KW, int DH, int DW>
static __global__ void __launch_bounds__(256) maxpool_backward_kernel(const float *__restrict__ gout,
                                                                      const float *__restrict__ indy,
                                                                      const float *__restrict__ indx, float *__restrict__ gin,
                                                                      long planes, int H, int W, Div32 dW_in, int oH, int oW,
                                                                      Div32 doW, int kH_, int kW_, int dH_, int dW_, Div32 ddH,
                                                                      Div32 ddW, int G, int band_rows, int bands) {
  extern __shared__ int pool_sm[];
  const int kH = KH ? KH : kH_, kW = KW ? KW : kW_, dH = DH ? DH : dH_, dW = DW ? DW : dW_;
  auto div_dH = [&](unsigned v) { return DH ? (int)(v / (unsigned)(DH ? DH : 1)) : (int)ddH.div(v); };
  auto div_dW = [&](unsigned v) { return DW ? (int)(v / (unsigned)(DW ? DW : 1)) : (int)ddW.div(v); };
  const int HW = H * W, oHW = oH * oW;
  const long groups = (planes + G - 1) / G;
  const long items = groups * bands;
  for (long item = blockIdx.x; item < items; item += gridDim.x) {
    const long grp = item / bands;
    const int band = (int)(item - grp * bands);
    const long p0 = grp * G;
    const int np = (int)(planes - p0 < G ? planes - p0 : G);
    const int h0 = band * band_rows, h1 = h0 + band_rows < H ? h0 + band_rows : H;
    // window rows that can cover input rows [h0, h1)
    int ylo = h0 - kH + 1;
    ylo = ylo <= 0 ? 0 : div_dH((unsigned)(ylo + dH - 1));
    int yhi = div_dH((unsigned)(h1 - 1));
    if (yhi > oH - 1) yhi = oH - 1;
    const int nwy = yhi >= ylo ? yhi - ylo + 1 : 0;
    const int nwin = nwy * oW;                 // per plane
    int *tgt = pool_sm;
    float *val = reinterpret_cast<float *>(pool_sm + np * nwin);
    for (int t = threadIdx.x; t < np * nwin; t += blockDim.x) {
      int pl = 0, r = t;
      if (np > 1) { pl = t / nwin; r = t - pl * nwin; }
      const int yy = (int)doW.div((unsigned)r), x = r - yy * oW, y = ylo + yy;
      const long o = (p0 + pl) * oHW + (long)y * oW + x;
      tgt[t] = ((int)indy[o] - 1 + y * dH) * W + ((int)indx[o] - 1 + x * dW);
      val[t] = gout[o];
    }
    __syncthreads();
    if (KH && KW && DH && DW) {
      // Fixed window shape: a thread owns one stride cell of DH x DW pixels.  The windows that can reach the
      // cell are those of the cells up to NY-1 rows / NX-1 columns before it; each is fetched once and tested
      // against every pixel of the cell, in ascending (y, x) order, which keeps the CPU's order of additions.
      constexpr int cDH = DH ? DH : 1, cDW = DW ? DW : 1;
      constexpr int NY = (KH + cDH - 1) / cDH, NX = (KW + cDW - 1) / cDW;
      const int cW = (W + cDW - 1) / cDW, cH = (h1 - h0 + cDH - 1) / cDH, cells = cH * cW;
      const int a0 = h0 / cDH;                       // band_rows is a multiple of dH
      for (int t = threadIdx.x; t < np * cells; t += blockDim.x) {
        int pl = 0, r = t;
        if (np > 1) { pl = t / cells; r = t - pl * cells; }
        const int ca = r / cW, b = r - ca * cW, a = a0 + ca;
        const int *tp = tgt + pl * nwin;
        const float *vp = val + pl * nwin;
        float acc[cDH][cDW];
#pragma unroll
        for (int rr = 0; rr < cDH; rr++)
#pragma unroll
          for (int ss = 0; ss < cDW; ss++) acc[rr][ss] = 0.f;
        const int me0 = a * cDH * W + b * cDW;       // flat position of the cell's first pixel
#pragma unroll
        for (int dy = 0; dy < NY; dy++) {
          const int y = a - (NY - 1) + dy;
#pragma unroll
          for (int dx = 0; dx < NX; dx++) {
            const int x = b - (NX - 1) + dx;
            const bool in = y >= ylo && y <= yhi && x >= 0 && x < oW;
            const int i = in ? (y - ylo) * oW + x : 0;
            const int tg = in ? tp[i] : -1;
            const float v = vp[i];
#pragma unroll
            for (int rr = 0; rr < cDH; rr++)
#pragma unroll
              for (int ss = 0; ss < cDW; ss++) acc[rr][ss] = tg == me0 + rr * W + ss ? acc[rr][ss] + v : acc[rr][ss];
          }
        }
        float *gp = gi_plane(gin, p0 + pl, HW) + (long)a * cDH * W + b * cDW;
#pragma unroll
        for (int rr = 0; rr < cDH; rr++)
#pragma unroll
          for (int ss = 0; ss < cDW; ss++)
            if (a * cDH + rr < h1 && b * cDW + ss < W) gp[rr * W + ss] = acc[rr][ss];
      }
    } else {
    const int npix = (h1 - h0) * W;            // per plane
    for (int t = threadIdx.x; t < np * npix; t += blockDim.x) {
      int pl = 0, r = t;
      if (np > 1) { pl = t / npix; r = t - pl * npix; }
      const int hh = (int)dW_in.div((unsigned)r), w = r - hh * W, h = h0 + hh;
      // windows y with y*dH <= h <= y*dH + kH - 1, clipped to the output
      int y0 = h - kH + 1;
      y0 = y0 <= 0 ? 0 : div_dH((unsigned)(y0 + dH - 1));
      int y1 = div_dH((unsigned)h);
      if (y1 > oH - 1) y1 = oH - 1;
      int x0 = w - kW + 1;
      x0 = x0 <= 0 ? 0 : div_dW((unsigned)(x0 + dW - 1));
      int x1 = div_dW((unsigned)w);
      if (x1 > oW - 1) x1 = oW - 1;
      const int me = h * W + w;
      const int *tp = tgt + pl * nwin;
      const float *vp = val + pl * nwin;
      float acc = 0.f;
      for (int y = y0; y <= y1; y++)
        for (int x = x0; x <= x1; x++) {
          const int i = (y - ylo) * oW + x;
          if (tp[i] == me) acc += vp[i];
        }
      gin[(p0 + pl) * HW + (long)h0 * W + r] = acc;
    }
    }
    __syncthreads();
  }
}

// Backward for planes of at most 32 stride cells per row (the 55 / 27 / 13-wide planes of the AlexNet-style net, the
// 56-wide and smaller ones of the VGG-style net), stride 2, windows of 2 or 3.  A group of LP lanes walks one plane
// from the top, one row of windows per step; lane b holds window (y, b), read from global memory exactly once,
// coalesced, with the next rows' loads already in flight.  Every window has ONE target pixel, so instead of testing
// each pixel against each window that covers it, the window adds its value to its target in a three-row buffer in
// shared memory (input rows 2y, 2y+1, 2y+2).  Two windows of a row can share a target only when they are
// neighbours; then the right-hand lane adds both, left one first.  Together with the top-to-bottom walk this is the
// CPU's order of additions (ascending window row, then column), so the result is bit-equal to it.  After a step
// rows 2y and 2y+1 are final and leave as whole lines; row 2y+2 carries over as the next step's first row.
template <int KH, int KW, int LP>
static __global__ void __launch_bounds__(256, 8) maxpool_backward_rows_kernel(const float *__restrict__ gout,
                                                                              const float *__restrict__ indy,
                                                                              const float *__restrict__ indx,
                                                                              float *__restrict__ gin, long planes, int H, int W,
                                                                              int oH, int oW) {
  static_assert(KH <= 3 && KW <= 3, "a window reaches at most one stride cell further");
  constexpr int PPW = 32 / LP, RW = 2 * LP;          // planes per warp, floats per buffered row of one plane
  __shared__ float rows_sm[8][3][64];
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31, sub = lane % LP, seg = lane / LP, wib = threadIdx.x >> 5;
  const long warps = ((long)gridDim.x * blockDim.x) >> 5, warp0 = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int oHW = oH * oW;
  const long groups = (planes + PPW - 1) / PPW;
  const int i0 = seg * RW + sub, i1 = i0 + LP;       // this lane's two elements of a buffered row
  for (long grp = warp0; grp < groups; grp += warps) {
    const long plane = grp * PPW + seg;
    const bool live = plane < planes;
    const bool mine = live && sub < oW, st0 = live && sub < W, st1 = live && LP + sub < W;
    const float *go = gout + plane * oHW + sub, *iy = indy + plane * oHW + sub, *ix = indx + plane * oHW + sub;
    float *outp = gin + plane * (long)H * W + sub;   // this lane's first element of the row being written
    float *r0 = rows_sm[wib][0], *r1 = rows_sm[wib][1], *r2 = rows_sm[wib][2];
    r0[lane] = 0.f; r0[lane + 32] = 0.f; r1[lane] = 0.f; r1[lane + 32] = 0.f; r2[lane] = 0.f; r2[lane + 32] = 0.f;
    __syncwarp();
    // (target row - 2y) * 128 + target column, or -1 for "no window here"; value
    auto load = [&](int y, int &t, float &v) {
      t = -1; v = 0.f;
      if (mine && y < oH) {
        const int o = y * oW;
        t = ((int)iy[o] - 1) * 128 + ((int)ix[o] - 1 + 2 * sub);
        v = go[o];
      }
    };
    int ct, qt[3], nt;
    float cv, qv[3], nv;
    load(0, ct, cv);
#pragma unroll
    for (int d = 0; d < 3; d++) load(1 + d, qt[d], qv[d]);
    // A finished row leaves as a line (lane `sub` writes elements sub and LP + sub) and its buffer is cleared by the
    // lanes that read it: only columns below W can ever be targets.
    auto flush = [&](float *row) {
      if (st0) { outp[0] = row[i0]; row[i0] = 0.f; }
      if (st1) { outp[LP] = row[i1]; row[i1] = 0.f; }
      outp += W;
    };
    for (int y = 0; y < oH; y++) {
      load(y + 4, nt, nv);
      const int lt = __shfl_up_sync(full, ct, 1, LP), rt = __shfl_down_sync(full, ct, 1, LP);
      const float lv = __shfl_up_sync(full, cv, 1, LP);
      const bool with_left = sub > 0 && lt == ct;
      const bool right_takes_it = sub < LP - 1 && rt == ct;
      if (ct >= 0 && !right_takes_it) {
        float *row = (ct >> 7) == 0 ? r0 : ((ct >> 7) == 1 ? r1 : r2);
        float x = row[seg * RW + (ct & 127)];
        if (with_left) x += lv;
        row[seg * RW + (ct & 127)] = x + cv;
      }
      __syncwarp();
      flush(r0);                                      // rows 2y and 2y + 1 are final (H >= 2 oH: both exist)
      flush(r1);
      __syncwarp();
      float *z = r0; r0 = r2; r2 = r1; r1 = z;      // row 2y+2 becomes the next step's row 0; two cleared rows follow
      ct = qt[0]; cv = qv[0];
      qt[0] = qt[1]; qv[0] = qv[1]; qt[1] = qt[2]; qv[1] = qv[2]; qt[2] = nt; qv[2] = nv;
    }
    // what lies below the last window row: the carried row, then rows no window reaches (zeros)
    for (int h = 2 * oH; h < H; h++) flush(r0);
    __syncwarp();
  }
}

static dim3 plane_grid(long planes, long per_plane) {
  long gx = (per_plane + 255) / 256;
  if (gx > 64) gx = 64;
  long gy = planes;
  const long cap = (long)ctx().sm_count * 32;
  if (gx * gy > cap) gy = cap / gx > 0 ? cap / gx : 1;
  if (gy > 65535) gy = 65535;
  return dim3((unsigned)gx, (unsigned)gy, 1);
}

// ---- SpatialAveragePooling (gputorch/lib/THC/gpunn-impl/SpatialAveragePooling.cpp:9-62 forward, :130-182
// backward; CPU mcw_nn/generic/SpatialAveragePooling.c:5-80, :84-150).  In this code base the module writes the
// window SUM, neither path divides by the window size.  Forward: one thread per output, the window summed in
// FP32 row by row as the CPU does.  Backward: one thread per INPUT pixel adds the gradOutput of every window that
// covers it in ascending (y, x) order, the order in which the CPU's scatter reaches that pixel, so the result is
// bit-equal to the CPU's and overlapping windows work (the reference GPU path refuses dW != kW, :194-195).
static __global__ void __launch_bounds__(256) sumpool_forward_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                                     long planes, int H, int W, int oH, int oW, int kH, int kW,
                                                                     int dH, int dW) {
  const long total = planes * oH * oW;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long)gridDim.x * blockDim.x) {
    const int x = (int)(t % oW);
    const long q = t / oW;
    const int y = (int)(q % oH);
    const long pl = q / oH;
    const float *p = in + (pl * H + (long)y * dH) * W + (long)x * dW;
    float sum = 0.f;
    for (int ky = 0; ky < kH; ky++, p += W)
      for (int kx = 0; kx < kW; kx++) sum += p[kx];
    out[t] = sum;
  }
}
static __global__ void __launch_bounds__(256) sumpool_backward_kernel(const float *__restrict__ gout, float *__restrict__ gin,
                                                                      long planes, int H, int W, int oH, int oW, int kH, int kW,
                                                                      int dH, int dW) {
  const long total = planes * H * W;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long)gridDim.x * blockDim.x) {
    const int w = (int)(t % W);
    const long q = t / W;
    const int h = (int)(q % H);
    const long pl = q / H;
    // windows (y, x) with y*dH <= h < y*dH + kH
    int y0 = h - kH + 1; y0 = y0 <= 0 ? 0 : (y0 + dH - 1) / dH;
    int x0 = w - kW + 1; x0 = x0 <= 0 ? 0 : (x0 + dW - 1) / dW;
    int y1 = h / dH; if (y1 > oH - 1) y1 = oH - 1;
    int x1 = w / dW; if (x1 > oW - 1) x1 = oW - 1;
    const float *g = gout + pl * oH * oW;
    float sum = 0.f;
    for (int y = y0; y <= y1; y++)
      for (int x = x0; x <= x1; x++) sum += g[y * oW + x];
    gin[t] = sum;
  }
}

}  // namespace thc

using namespace thc;

THC_API int THGPUNN_SpatialMaxPooling_updateOutput(THGPUTensor *input, THGPUTensor *output, THGPUTensor *indices,
                                                   int kW, int kH, int dW, int dH) {
  THC_BEGIN
  THC_ARG(input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D (batch) tensor expected");
  THC_ARG(kW > 0 && kH > 0 && dW > 0 && dH > 0, 1, "invalid kernel / stride");
  const bool batch = input->nDimension == 4;
  const int o = batch ? 1 : 0;
  const long N = batch ? input->size[0] : 1, C = input->size[o], H = input->size[o + 1], W = input->size[o + 2];
  THC_ARG(W >= kW && H >= kH, 2, "input image smaller than kernel size");
  const long oH = (H - kH) / dH + 1, oW = (W - kW) / dW + 1;
  TensorRef in(tensor_new_contiguous(input));
  if (batch) {
    const long s[4] = {N, C, oH, oW}, si[5] = {2, N, C, oH, oW};
    resize_nd(output, 4, s, nullptr);
    resize_nd(indices, 5, si, nullptr);
  } else {
    const long s[3] = {C, oH, oW}, si[4] = {2, C, oH, oW};
    resize_nd(output, 3, s, nullptr);
    resize_nd(indices, 4, si, nullptr);
  }
  THC_CHECK(is_contiguous(output) && is_contiguous(indices), "output / indices must be contiguous");
  const long total = N * C * oH * oW;
  THC_CHECK(H * W < (1l << 31), "image plane too large");
  if (total > 0) {
    const dim3 grid = plane_grid(N * C, oH * oW);
#define THC_POOL_FWD(KH, KW, DH, DW)                                                                               \
  maxpool_forward_kernel<KH, KW, DH, DW><<<grid, 256, 0, stream()>>>(                                              \
      data_ptr(in), data_ptr(output), data_ptr(indices), data_ptr(indices) + total, N * C, (int)H, (int)W, (int)oH, \
      (int)oW, Div32::make(oW), kH, kW, dH, dW)
    if (kH == 3 && kW == 3 && dH == 2 && dW == 2) THC_POOL_FWD(3, 3, 2, 2);
    else if (kH == 2 && kW == 2 && dH == 2 && dW == 2) THC_POOL_FWD(2, 2, 2, 2);
    else THC_POOL_FWD(0, 0, 0, 0);
#undef THC_POOL_FWD
    check_launch("maxpool_forward");
  }
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SpatialMaxPooling_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradInput,
                                                      THGPUTensor *indices, int kW, int kH, int dW, int dH) {
  THC_BEGIN
  THC_ARG(input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D (batch) tensor expected");
  const bool batch = input->nDimension == 4;
  const int o = batch ? 1 : 0;
  const long N = batch ? input->size[0] : 1, C = input->size[o], H = input->size[o + 1], W = input->size[o + 2];
  THC_ARG(W >= kW && H >= kH, 2, "input image smaller than kernel size");
  const long oH = (H - kH) / dH + 1, oW = (W - kW) / dW + 1;
  THC_ARG(gradOutput->nDimension == input->nDimension && gradOutput->size[o] == C && gradOutput->size[o + 1] == oH &&
              gradOutput->size[o + 2] == oW && (!batch || gradOutput->size[0] == N), 3, "gradOutput has the wrong size");
  THC_ARG(nelem(indices) == 2 * N * C * oH * oW, 1, "indices do not belong to this input");
  TensorRef go(tensor_new_contiguous(gradOutput)); TensorRef ind(tensor_new_contiguous(indices));
  tensor_resize_as(gradInput, input);
  THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
  const long total = N * C * H * W, ototal = N * C * oH * oW;
  THC_CHECK(H * W < (1l << 31), "image plane too large");
  if (total > 0) {
    // shared memory holds (position, value) of up to kMaxWin windows per work item
    const int kMaxWin = 5120;
    int G = 1, band_rows = (int)H, bands = 1;
    if (oH * oW <= kMaxWin) {
      // whole planes; several per block when they are small, so that a block has ~8 K pixels between barriers
      G = (int)(8192 / (H * W));
      if (G < 1) G = 1;
      if (G * oH * oW > kMaxWin) G = (int)(kMaxWin / (oH * oW));
      if (G > N * C) G = (int)(N * C);
    } else {
      long wrows = kMaxWin / oW;            // window rows that fit
      THC_CHECK(wrows >= 2 + (kH + dH - 1) / dH, "pooling window row too wide for the backward kernel");
      band_rows = (int)((wrows - 1 - (kH + dH - 1) / dH) * dH);
      if (band_rows < 1) band_rows = 1;
      bands = (int)((H + band_rows - 1) / band_rows);
    }
    // narrow planes with the common windows: the row-buffer kernel
    const long cW = (W + dW - 1) / dW;
    const bool k33 = kH == 3 && kW == 3 && dH == 2 && dW == 2, k22 = kH == 2 && kW == 2 && dH == 2 && dW == 2;
    if ((k33 || k22) && cW <= 32) {
      const int LP = cW <= 8 ? 8 : (cW <= 16 ? 16 : 32);
      const long groups = (N * C + 32 / LP - 1) / (32 / LP);
      long blocks = (groups + 7) / 8;
      const long cap = (long)ctx().sm_count * 8;
      if (blocks > cap) blocks = cap;
#define THC_POOL_BWD_WARP(KH, KW, LPV)                                                                                \
  maxpool_backward_rows_kernel<KH, KW, LPV><<<(unsigned)blocks, 256, 0, stream()>>>(                                  \
      data_ptr(go), data_ptr(ind), data_ptr(ind) + ototal, data_ptr(gradInput), N * C, (int)H, (int)W, (int)oH, (int)oW)
      if (k33) { if (LP == 8) THC_POOL_BWD_WARP(3, 3, 8); else if (LP == 16) THC_POOL_BWD_WARP(3, 3, 16); else THC_POOL_BWD_WARP(3, 3, 32); }
      else { if (LP == 8) THC_POOL_BWD_WARP(2, 2, 8); else if (LP == 16) THC_POOL_BWD_WARP(2, 2, 16); else THC_POOL_BWD_WARP(2, 2, 32); }
#undef THC_POOL_BWD_WARP
      check_launch("maxpool_backward");
      return 0;
    }
    const long items = ((N * C + G - 1) / G) * bands;
    // shared memory actually needed per work item: (position, value) per window
    const size_t smem = bands > 1 ? (size_t)kMaxWin * 8 : (size_t)G * oH * oW * 8;
    long blocks = items;
    const long cap = (long)ctx().sm_count * 8;
    if (blocks > cap) blocks = cap;
#define THC_POOL_BWD(KH, KW, DH, DW)                                                                                \
  maxpool_backward_kernel<KH, KW, DH, DW><<<(unsigned)blocks, 256, smem, stream()>>>(                         \
      data_ptr(go), data_ptr(ind), data_ptr(ind) + ototal, data_ptr(gradInput), N * C, (int)H, (int)W, Div32::make(W), \
      (int)oH, (int)oW, Div32::make(oW), kH, kW, dH, dW, Div32::make(dH), Div32::make(dW), G, band_rows, bands)
    if (kH == 3 && kW == 3 && dH == 2 && dW == 2) THC_POOL_BWD(3, 3, 2, 2);
    else if (kH == 2 && kW == 2 && dH == 2 && dW == 2) THC_POOL_BWD(2, 2, 2, 2);
    else THC_POOL_BWD(0, 0, 0, 0);
#undef THC_POOL_BWD
    check_launch("maxpool_backward");
  }
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SpatialAveragePooling_updateOutput(THGPUTensor *input, THGPUTensor *output, int kW, int kH, int dW, int dH) {
  THC_BEGIN
  THC_ARG(input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D(batch mode) tensor expected");
  THC_ARG(kW > 0 && kH > 0 && dW > 0 && dH > 0, 1, "invalid kernel / stride");
  const bool batch = input->nDimension == 4;
  const int o = batch ? 1 : 0;
  const long N = batch ? input->size[0] : 1, C = input->size[o], H = input->size[o + 1], W = input->size[o + 2];
  THC_ARG(W >= kW && H >= kH, 2, "input image smaller than kernel size");
  const long oH = (H - kH) / dH + 1, oW = (W - kW) / dW + 1;
  TensorRef in(tensor_new_contiguous(input));
  if (batch) { const long s[4] = {N, C, oH, oW}; resize_nd(output, 4, s, nullptr); }
  else { const long s[3] = {C, oH, oW}; resize_nd(output, 3, s, nullptr); }
  THC_CHECK(is_contiguous(output), "output must be contiguous");
  const long total = N * C * oH * oW;
  if (total > 0) {
    long blocks = (total + 255) / 256;
    if (blocks > (long)ctx().sm_count * 16) blocks = (long)ctx().sm_count * 16;
    sumpool_forward_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(data_ptr(in), data_ptr(output), N * C, (int)H, (int)W, (int)oH,
                                                                  (int)oW, kH, kW, dH, dW);
    check_launch("SpatialAveragePooling_updateOutput");
  }
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SpatialAveragePooling_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradInput,
                                                          int kW, int kH, int dW, int dH) {
  THC_BEGIN
  THC_ARG(input->nDimension == 3 || input->nDimension == 4, 2, "3D or 4D(batch mode) tensor expected");
  THC_ARG(kW > 0 && kH > 0 && dW > 0 && dH > 0, 1, "invalid kernel / stride");
  const bool batch = input->nDimension == 4;
  const int o = batch ? 1 : 0;
  const long N = batch ? input->size[0] : 1, C = input->size[o], H = input->size[o + 1], W = input->size[o + 2];
  THC_ARG(W >= kW && H >= kH, 2, "input image smaller than kernel size");
  const long oH = (H - kH) / dH + 1, oW = (W - kW) / dW + 1;
  THC_ARG(gradOutput->nDimension == input->nDimension && gradOutput->size[o] == C && gradOutput->size[o + 1] == oH &&
              gradOutput->size[o + 2] == oW && (!batch || gradOutput->size[0] == N), 3, "gradOutput has the wrong size");
  TensorRef go(tensor_new_contiguous(gradOutput));
  tensor_resize_as(gradInput, input);
  THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
  const long total = N * C * H * W;
  if (total > 0) {
    long blocks = (total + 255) / 256;
    if (blocks > (long)ctx().sm_count * 16) blocks = (long)ctx().sm_count * 16;
    sumpool_backward_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(data_ptr(go), data_ptr(gradInput), N * C, (int)H, (int)W, (int)oH,
                                                                   (int)oW, kH, kW, dH, dW);
    check_launch("SpatialAveragePooling_updateGradInput");
  }
  return 0;
  THC_END(1)
}
