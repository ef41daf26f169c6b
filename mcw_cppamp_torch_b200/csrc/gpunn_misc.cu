// Threshold / ReLU, LogSoftMax, ClassNLLCriterion and the parameter update on torch.GPUTensor.
//   Threshold         gputorch/lib/THC/gpunn-impl/Threshold.cpp:16-38,53-81; CPU mcw_nn/generic/Threshold.c:5-32
//   LogSoftMax        gpunn-impl/LogSoftMax.cpp:5-194;                       CPU mcw_nn/generic/LogSoftMax.c:5-103
//   ClassNLLCriterion gpunn-impl/ClassNLLCriterion.cpp:9-198;                CPU mcw_nn/ClassNLLCriterion.lua:13-70
//   SGD               Module:updateParameters, mcw_nn/Module.lua:75-82 (momentum is an addition)
#include "thc_apply.cuh"

namespace thc {

// threshold and val are compared / stored as floats, as the CPU kernel does (Threshold.c:8-9)
struct ThresholdFwdOp { float th, val; __device__ float operator()(const float *a) const { return a[0] > th ? a[0] : val; } };
// a[0] = input, a[1] = gradOutput
struct ThresholdBwdOp { float th; __device__ float operator()(const float *a) const { return a[0] > th ? a[1] : 0.f; } };

static __device__ __forceinline__ float block_max(float v, float *sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  v = sm[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); i++) v = fmaxf(v, sm[i]);
  __syncthreads();
  return v;
}
static __device__ __forceinline__ double block_sum(double v, double *sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  v = sm[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); i++) v += sm[i];
  __syncthreads();
  return v;
}

// exp(-x) for x >= 0 exactly as the CPU kernel evaluates it (THExpMinusApprox,
// mcw_torch7_core/lib/TH/THLogAdd.c:56-86): (1 + x/8 + x^2/128 + ...)^-8 in double, 0 beyond 13.
// Using the same polynomial keeps the classifier loss bit-close to the CPU nn path; the exact
// exponential differs from it by up to ~2e-3 in the log-sum.
static __device__ __forceinline__ double exp_minus_approx(double x) {
  if (x < 13.0) {
    double y = 1.0 + x * (0.125 + x * (0.0078125 + x * (0.00032552083 + x * 1.0172526e-5)));
    y *= y; y *= y; y *= y;
    return 1.0 / y;
  }
  return 0.0;
}

// one block per row: out = x - (max + log(sum exp(x - max)))
static __global__ void __launch_bounds__(256) logsoftmax_forward_kernel(const float *__restrict__ in, float *__restrict__ out, long dim) {
  __shared__ float smf[8];
  __shared__ double smd[8];
  const float *x = in + (long)blockIdx.x * dim;
  float *o = out + (long)blockIdx.x * dim;
  float m = -INFINITY;
  for (long d = threadIdx.x; d < dim; d += blockDim.x) m = fmaxf(m, x[d]);
  m = block_max(m, smf);
  double s = 0;
  for (long d = threadIdx.x; d < dim; d += blockDim.x) s += exp_minus_approx((double)(m - x[d]));
  s = block_sum(s, smd);
  const double logsum = (double)m + log(s);
  for (long d = threadIdx.x; d < dim; d += blockDim.x) o[d] = (float)((double)x[d] - logsum);
}
// gradIn = gradOut - exp(out) * sum(gradOut)
static __global__ void __launch_bounds__(256) logsoftmax_backward_kernel(const float *__restrict__ gout, const float *__restrict__ out,
                                                                         float *__restrict__ gin, long dim) {
  __shared__ double smd[8];
  const long b = (long)blockIdx.x * dim;
  double s = 0;
  for (long d = threadIdx.x; d < dim; d += blockDim.x) s += (double)gout[b + d];
  s = block_sum(s, smd);
  for (long d = threadIdx.x; d < dim; d += blockDim.x) gin[b + d] = (float)((double)gout[b + d] - exp((double)out[b + d]) * s);
}

// SoftMax (gputorch/lib/THC/gpunn-impl/SoftMax.cpp; CPU mcw_nn/generic/SoftMax.c:5-60, :62-110): one block per row.
// Forward as the CPU evaluates it: z_d = expminus(max - x_d) with the same polynomial, stored as a float, their sum
// in double, out_d = z_d * (float)(1 / sum).  Backward: gradIn_d = out_d * (gradOut_d - sum_e gradOut_e * out_e),
// the sum in double.
static __global__ void __launch_bounds__(256) softmax_forward_kernel(const float *__restrict__ in, float *__restrict__ out, long dim) {
  __shared__ float smf[8];
  __shared__ double smd[8];
  const float *x = in + (long)blockIdx.x * dim;
  float *o = out + (long)blockIdx.x * dim;
  float m = -INFINITY;
  for (long d = threadIdx.x; d < dim; d += blockDim.x) m = fmaxf(m, x[d]);
  m = block_max(m, smf);
  double s = 0;
  for (long d = threadIdx.x; d < dim; d += blockDim.x) {
    const float z = (float)exp_minus_approx((double)(m - x[d]));
    o[d] = z;
    s += (double)z;
  }
  s = block_sum(s, smd);
  const double inv = 1.0 / s;
  for (long d = threadIdx.x; d < dim; d += blockDim.x) o[d] = (float)((double)o[d] * inv);
}
static __global__ void __launch_bounds__(256) softmax_backward_kernel(const float *__restrict__ gout, const float *__restrict__ out,
                                                                      float *__restrict__ gin, long dim) {
  __shared__ double smd[8];
  const long b = (long)blockIdx.x * dim;
  double s = 0;
  for (long d = threadIdx.x; d < dim; d += blockDim.x) s += (double)gout[b + d] * (double)out[b + d];
  s = block_sum(s, smd);
  for (long d = threadIdx.x; d < dim; d += blockDim.x) gin[b + d] = (float)((double)out[b + d] * ((double)gout[b + d] - s));
}

// loss = -sum_i in[i][target_i - 1] (/ nframe)
static __global__ void __launch_bounds__(256) classnll_forward_kernel(const float *__restrict__ in, const float *__restrict__ target,
                                                                      float *out, long nframe, long dim, int size_average) {
  __shared__ double smd[8];
  double s = 0;
  for (long i = threadIdx.x; i < nframe; i += blockDim.x) {
    const long t = (long)target[i] - 1;
    if (t >= 0 && t < dim) s -= (double)in[i * dim + t];
  }
  s = block_sum(s, smd);
  if (threadIdx.x == 0) out[0] = (float)(size_average ? s / (double)nframe : s);
}
static __global__ void classnll_backward_kernel(const float *__restrict__ target, float *gin, long nframe, long dim, float z) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nframe) return;
  const long t = (long)target[i] - 1;
  if (t >= 0 && t < dim) gin[i * dim + t] = z;
}

static __global__ void __launch_bounds__(256) sgd_kernel(float *__restrict__ w, const float *__restrict__ g, float *__restrict__ v,
                                                         long n, float lr, float momentum) {
  const long nthreads = (long)gridDim.x * blockDim.x;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long nvec = (((uintptr_t)w | (uintptr_t)g | (uintptr_t)v) & 15) == 0 ? n >> 2 : 0;
  for (long i = tid; i < nvec; i += nthreads) {
    float4 ww = reinterpret_cast<float4 *>(w)[i];
    const float4 gg = reinterpret_cast<const float4 *>(g)[i];
    if (v) {
      float4 vv = reinterpret_cast<float4 *>(v)[i];
      vv.x = momentum * vv.x + gg.x; vv.y = momentum * vv.y + gg.y; vv.z = momentum * vv.z + gg.z; vv.w = momentum * vv.w + gg.w;
      reinterpret_cast<float4 *>(v)[i] = vv;
      ww.x -= lr * vv.x; ww.y -= lr * vv.y; ww.z -= lr * vv.z; ww.w -= lr * vv.w;
    } else {
      ww.x -= lr * gg.x; ww.y -= lr * gg.y; ww.z -= lr * gg.z; ww.w -= lr * gg.w;
    }
    reinterpret_cast<float4 *>(w)[i] = ww;
  }
  for (long i = (nvec << 2) + tid; i < n; i += nthreads) {
    float gv = g[i];
    if (v) { gv = momentum * v[i] + gv; v[i] = gv; }
    w[i] -= lr * gv;
  }
}

// w -= lr * (v = momentum * v + g) over n floats on stream `s` (v null: plain SGD).  Also the consumer the
// communicator runs behind each gradient bucket's all-reduce.
void sgd_update_async(float *w, const float *g, float *v, long n, float lr, float momentum, cudaStream_t s) {
  if (n <= 0) return;
  int blocks = ceil_div((n + 3) / 4, 256);
  const int cap = ctx().sm_count * 8;
  if (blocks > cap) blocks = cap;
  sgd_kernel<<<blocks, 256, 0, s>>>(w, g, v, n, lr, momentum);
  check_launch("sgd");
}

static void rows_of(const THGPUTensor *t, long &nframe, long &dim) {
  THC_ARG(t->nDimension == 1 || t->nDimension == 2, 2, "vector or matrix expected");
  nframe = t->nDimension == 1 ? 1 : t->size[0];
  dim = t->nDimension == 1 ? t->size[0] : t->size[1];
}

}  // namespace thc

using namespace thc;

THC_API int THGPUNN_Threshold_updateOutput(THGPUTensor *input, THGPUTensor *output, double threshold, double val) {
  THC_BEGIN
  tensor_resize_as(output, input);
  apply<1>(output, input, nullptr, ThresholdFwdOp{(float)threshold, (float)val}, "Threshold_updateOutput");
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_Threshold_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradInput, double threshold) {
  THC_BEGIN
  THC_ARG(nelem(input) == nelem(gradOutput) && THGPUTensor_isSameSizeAs(input, gradOutput), 3, "gradOutput has the wrong size");
  tensor_resize_as(gradInput, input);
  apply<2>(gradInput, input, gradOutput, ThresholdBwdOp{(float)threshold}, "Threshold_updateGradInput");
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_LogSoftMax_updateOutput(THGPUTensor *input, THGPUTensor *output) {
  THC_BEGIN
  long nframe, dim;
  rows_of(input, nframe, dim);
  TensorRef in(tensor_new_contiguous(input));
  tensor_resize_as(output, input);
  THC_CHECK(is_contiguous(output), "output must be contiguous");
  if (nframe > 0 && dim > 0) {
    logsoftmax_forward_kernel<<<(unsigned)nframe, 256, 0, stream()>>>(data_ptr(in), data_ptr(output), dim);
    check_launch("logsoftmax_forward");
  }
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_LogSoftMax_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradInput, THGPUTensor *output) {
  (void)input;
  THC_BEGIN
  long nframe, dim;
  rows_of(output, nframe, dim);
  THC_ARG(nelem(gradOutput) == nelem(output), 3, "gradOutput has the wrong size");
  TensorRef go(tensor_new_contiguous(gradOutput)); TensorRef out(tensor_new_contiguous(output));
  tensor_resize_as(gradInput, output);
  THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
  if (nframe > 0 && dim > 0) {
    logsoftmax_backward_kernel<<<(unsigned)nframe, 256, 0, stream()>>>(data_ptr(go), data_ptr(out), data_ptr(gradInput), dim);
    check_launch("logsoftmax_backward");
  }
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_ClassNLLCriterion_updateOutput(THGPUTensor *input, THGPUTensor *target, THGPUTensor *outputTensor, int sizeAverage) {
  THC_BEGIN
  long nframe, dim;
  rows_of(input, nframe, dim);
  THC_ARG(nelem(target) == nframe, 3, "one target per input row expected");
  TensorRef in(tensor_new_contiguous(input)); TensorRef tg(tensor_new_contiguous(target));
  const long one[1] = {1};
  resize_nd(outputTensor, 1, one, nullptr);
  classnll_forward_kernel<<<1, 256, 0, stream()>>>(data_ptr(in), data_ptr(tg), data_ptr(outputTensor), nframe, dim, sizeAverage);
  check_launch("classnll_forward");
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_ClassNLLCriterion_updateGradInput(THGPUTensor *input, THGPUTensor *target, THGPUTensor *gradInput, int sizeAverage) {
  THC_BEGIN
  long nframe, dim;
  rows_of(input, nframe, dim);
  THC_ARG(nelem(target) == nframe, 3, "one target per input row expected");
  TensorRef tg(tensor_new_contiguous(target));
  tensor_resize_as(gradInput, input);
  THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
  THC_CUDA(cudaMemsetAsync(data_ptr(gradInput), 0, sizeof(float) * nframe * dim, stream()));
  const float z = sizeAverage ? -1.f / (float)nframe : -1.f;
  classnll_backward_kernel<<<ceil_div(nframe, 128), 128, 0, stream()>>>(data_ptr(tg), data_ptr(gradInput), nframe, dim, z);
  check_launch("classnll_backward");
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SGD_update(THGPUTensor *weight, THGPUTensor *grad, THGPUTensor *velocity, float lr, float momentum) {
  THC_BEGIN
  const long n = nelem(weight);
  THC_ARG(nelem(grad) == n, 2, "grad has the wrong size");
  THC_CHECK(is_contiguous(weight) && is_contiguous(grad), "flat contiguous parameter buffers expected");
  float *v = nullptr;
  if (momentum != 0.f) {
    THC_ARG(velocity && nelem(velocity) == n && is_contiguous(velocity), 3, "velocity buffer of the weight's size expected");
    v = data_ptr(velocity);
  }
  sgd_update_async(data_ptr(weight), data_ptr(grad), v, n, lr, momentum, stream());
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SoftMax_updateOutput(THGPUTensor *input, THGPUTensor *output) {
  THC_BEGIN
  long nframe, dim;
  rows_of(input, nframe, dim);
  TensorRef in(tensor_new_contiguous(input));
  tensor_resize_as(output, input);
  THC_CHECK(is_contiguous(output), "output must be contiguous");
  if (nframe > 0 && dim > 0) {
    softmax_forward_kernel<<<(unsigned)nframe, 256, 0, stream()>>>(data_ptr(in), data_ptr(output), dim);
    check_launch("SoftMax_updateOutput");
  }
  return 0;
  THC_END(1)
}

THC_API int THGPUNN_SoftMax_updateGradInput(THGPUTensor *input, THGPUTensor *gradOutput, THGPUTensor *gradInput,
                                            THGPUTensor *output) {
  (void)input;
  THC_BEGIN
  long nframe, dim;
  rows_of(output, nframe, dim);
  THC_ARG(nelem(gradOutput) == nelem(output), 3, "gradOutput has the wrong size");
  TensorRef go(tensor_new_contiguous(gradOutput)); TensorRef out(tensor_new_contiguous(output));
  tensor_resize_as(gradInput, output);
  THC_CHECK(is_contiguous(gradInput), "gradInput must be contiguous");
  if (nframe > 0 && dim > 0) {
    softmax_backward_kernel<<<(unsigned)nframe, 256, 0, stream()>>>(data_ptr(go), data_ptr(out), data_ptr(gradInput), dim);
    check_launch("SoftMax_updateGradInput");
  }
  return 0;
  THC_END(1)
}
