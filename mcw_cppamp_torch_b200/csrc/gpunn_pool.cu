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

static __global__ void __launch_bounds__(256) maxpool_forward_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                                     float *__restrict__ indy, float *__restrict__ indx,
                                                                     long total, int H, int W, int oH, int oW, int kH,
                                                                     int kW, int dH, int dW) {
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const int x = (int)(t % oW);
    const long q = t / oW;
    const int y = (int)(q % oH);
    const long plane = q / oH;
    const float *ip = in + plane * H * W + (long)y * dH * W + (long)x * dW;
    float best = -INFINITY;  // the CPU starts from (float)(-DBL_MAX) = -inf
    int bi = -1, cnt = 0;
    for (int i = 0; i < kH; i++)
      for (int j = 0; j < kW; j++) {
        const float v = ip[i * W + j];
        if (v > best) { best = v; bi = cnt; }
        cnt++;
      }
    out[t] = best;
    // bi == -1 (all NaN / -inf) reproduces the CPU's (int)(-1 / kW) + 1 and (-1 % kW) + 1
    indy[t] = (float)(bi / kW + 1);
    indx[t] = (float)(bi % kW + 1);
  }
}

static __global__ void __launch_bounds__(256) maxpool_backward_kernel(const float *__restrict__ gout,
                                                                      const float *__restrict__ indy,
                                                                      const float *__restrict__ indx, float *__restrict__ gin,
                                                                      long total, int H, int W, int oH, int oW, int kH,
                                                                      int kW, int dH, int dW) {
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long t = (long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += nthreads) {
    const int w = (int)(t % W);
    const long q = t / W;
    const int h = (int)(q % H);
    const long plane = q / H;
    int y0 = h - kH + 1;
    y0 = y0 <= 0 ? 0 : (y0 + dH - 1) / dH;
    int y1 = h / dH;
    if (y1 > oH - 1) y1 = oH - 1;
    int x0 = w - kW + 1;
    x0 = x0 <= 0 ? 0 : (x0 + dW - 1) / dW;
    int x1 = w / dW;
    if (x1 > oW - 1) x1 = oW - 1;
    const long ob = plane * oH * oW;
    float acc = 0.f;
    for (int y = y0; y <= y1; y++)
      for (int x = x0; x <= x1; x++) {
        const long o = ob + (long)y * oW + x;
        const int my = (int)indy[o] - 1 + y * dH, mx = (int)indx[o] - 1 + x * dW;
        if (my == h && mx == w) acc += gout[o];
      }
    gin[t] = acc;
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
  THGPUTensor *in = tensor_new_contiguous(input);
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
  if (total > 0) {
    int blocks = ceil_div(total, 256);
    const int cap = ctx().sm_count * 16;
    if (blocks > cap) blocks = cap;
    maxpool_forward_kernel<<<blocks, 256, 0, stream()>>>(data_ptr(in), data_ptr(output), data_ptr(indices),
                                                         data_ptr(indices) + total, total, (int)H, (int)W, (int)oH,
                                                         (int)oW, kH, kW, dH, dW);
    check_launch("maxpool_forward");
  }
  tensor_free(in);
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
  THGPUTensor *go = tensor_new_contiguous(gradOutput), *ind = tensor_new_contiguous(indices);
  tensor_resize_as(gradInput, input);
  THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
  const long total = N * C * H * W, ototal = N * C * oH * oW;
  if (total > 0) {
    int blocks = ceil_div(total, 256);
    const int cap = ctx().sm_count * 16;
    if (blocks > cap) blocks = cap;
    maxpool_backward_kernel<<<blocks, 256, 0, stream()>>>(data_ptr(go), data_ptr(ind), data_ptr(ind) + ototal,
                                                          data_ptr(gradInput), total, (int)H, (int)W, (int)oH, (int)oW,
                                                          kH, kW, dH, dW);
    check_launch("maxpool_backward");
  }
  tensor_free(go); tensor_free(ind);
  return 0;
  THC_END(1)
}
