// torch.GPUTensor pointwise math beyond add / cadd / cmul: unary functions, pow, clamp, sign, atan2, the
// comparison operators, addcmul / addcdiv, and the whole-tensor norms built on them.
//
// Reference: gputorch/lib/THC/THCTensorMath.h:39-88 (signatures), bodies gputorch/lib/THC/THCTensorMath.cpp
// :165-267 (addcmul / addcdiv) and :862-1465 (unary functions, comparisons, norms).  Values follow the CPU
// TH functions they are checked against, mcw_torch7_core/lib/TH/generic/THTensorMath.c: a unary function is
// the C function of the element (:1236-1241, :1277-1294; within rel 1e-4 / abs 1e-5 here), comparisons write 1 / 0 as
// floats (:1198-1234), sign is -1 / 0 / 1 (:746-760), addcmul is r = t + (value * src1) * src2 with every
// product rounded to float (:346-355).  All of them run through the shared elementwise kernels
// (thc_apply.cuh): contiguous float4 streaming, tiled transposes, generic strides.
#include <cmath>

#include "thc_apply.cuh"

namespace thc {

// Single-precision CUDA math functions (no fast-math): at most 1-2 ulp from the CPU's (float) f((double) x), well
// inside the rel 1e-4 / abs 1e-5 bound, and the kernels stay HBM-bound (in double precision exp ran at 58 % and
// tanh at 33 % of the HBM rate).
#define THC_UNARY_F(NAME, EXPR) \
  struct NAME { __device__ float operator()(const float *a) const { const float x = a[0]; return EXPR; } };
THC_UNARY_F(LogOp, logf(x))
THC_UNARY_F(Log1pOp, log1pf(x))
THC_UNARY_F(ExpOp, expf(x))
THC_UNARY_F(CosOp, cosf(x))
THC_UNARY_F(AcosOp, acosf(x))
THC_UNARY_F(CoshOp, coshf(x))
THC_UNARY_F(SinOp, sinf(x))
THC_UNARY_F(AsinOp, asinf(x))
THC_UNARY_F(SinhOp, sinhf(x))
THC_UNARY_F(TanOp, tanf(x))
THC_UNARY_F(AtanOp, atanf(x))
THC_UNARY_F(TanhOp, tanhf(x))
#undef THC_UNARY_F
// exact: these give the CPU's result bit for bit
struct SqrtOp { __device__ float operator()(const float *a) const { return sqrtf(a[0]); } };
struct CeilOp { __device__ float operator()(const float *a) const { return ceilf(a[0]); } };
struct FloorOp { __device__ float operator()(const float *a) const { return floorf(a[0]); } };
struct RoundOp { __device__ float operator()(const float *a) const { return roundf(a[0]); } };   // halves away from zero, like C round()
struct AbsOp { __device__ float operator()(const float *a) const { return fabsf(a[0]); } };
struct SignOp { __device__ float operator()(const float *a) const { return a[0] > 0.f ? 1.f : (a[0] < 0.f ? -1.f : 0.f); } };
struct PowOp { float v; __device__ float operator()(const float *a) const { return powf(a[0], v); } };
// TH's clamp: (x < min) ? min : (x > max ? max : x)
struct ClampOp { float lo, hi; __device__ float operator()(const float *a) const { return a[0] < lo ? lo : (a[0] > hi ? hi : a[0]); } };
struct Atan2Op { __device__ float operator()(const float *a) const { return atan2f(a[0], a[1]); } };

enum { CMP_LT, CMP_GT, CMP_LE, CMP_GE, CMP_EQ, CMP_NE };
template <int C> __device__ __forceinline__ bool cmp(float a, float b) {
  return C == CMP_LT ? a < b : C == CMP_GT ? a > b : C == CMP_LE ? a <= b : C == CMP_GE ? a >= b : C == CMP_EQ ? a == b : a != b;
}
template <int C> struct CmpValueOp { float v; __device__ float operator()(const float *a) const { return cmp<C>(a[0], v) ? 1.f : 0.f; } };
template <int C> struct CmpTensorOp { __device__ float operator()(const float *a) const { return cmp<C>(a[0], a[1]) ? 1.f : 0.f; } };

// (value * src1) * src2 and (value * src1) / src2, each step rounded to float as in the C expression
struct ScaledMulOp { float v; __device__ float operator()(const float *a) const { return __fmul_rn(__fmul_rn(v, a[0]), a[1]); } };
struct ScaledDivOp { float v; __device__ float operator()(const float *a) const { return __fdiv_rn(__fmul_rn(v, a[0]), a[1]); } };
struct SumOp { __device__ float operator()(const float *a) const { return __fadd_rn(a[0], a[1]); } };

// terms of the whole-tensor norms
struct NonZeroOp { __device__ float operator()(const float *a) const { return a[0] != 0.f ? 1.f : 0.f; } };
struct SquareOp { __device__ float operator()(const float *a) const { const double z = (double)a[0]; return (float)(z * z); } };
struct AbsPowOp { float v; __device__ float operator()(const float *a) const { return powf(fabsf(a[0]), v); } };
struct AbsDiffPowOp { float v; __device__ float operator()(const float *a) const { return powf(fabsf(a[0] - a[1]), v); } };
struct CenteredSquareOp { double mean; __device__ float operator()(const float *a) const { const double d = (double)a[0] - mean; return (float)(d * d); } };

template <typename Op>
static void unary(THGPUTensor *self, THGPUTensor *src, Op op, const char *name) {
  tensor_resize_as(self, src);
  apply<1>(self, src, nullptr, op, name);
}
template <typename Op>
static void binary(THGPUTensor *self, THGPUTensor *a, THGPUTensor *b, Op op, const char *name) {
  THC_ARG(nelem(a) == nelem(b), 3, "sizes do not match");
  tensor_resize_as(self, a);
  apply<2>(self, a, b, op, name);
}
// sum over all elements of op(a) or op(a, b), through a temporary of a's shape
template <typename Op>
static double sum_of(THGPUTensor *a, THGPUTensor *b, Op op, const char *name) {
  THGPUTensor *tmp = tensor_new();
  tensor_resize_as(tmp, a);
  if (b) apply<2>(tmp, a, b, op, name);
  else apply<1>(tmp, a, nullptr, op, name);
  const double s = (double)THGPUTensor_sumall(tmp);
  tensor_free(tmp);
  return s;
}
// r = t + op(src1, src2).  TH walks the three tensors element by element in memory order, so operands of another
// shape with the same number of elements are taken as contiguous copies seen under t's sizes.
template <typename Op>
static void add_scaled(THGPUTensor *self, THGPUTensor *t, THGPUTensor *src1, THGPUTensor *src2, Op op, const char *name) {
  THC_ARG(nelem(src1) == nelem(t) && nelem(src2) == nelem(t), 3, "sizes do not match");
  THGPUTensor *v1 = nullptr, *v2 = nullptr;
  if (!THGPUTensor_isSameSizeAs(src1, t)) { v1 = THGPUTensor_newClone(src1); tensor_resize_as(v1, t); }
  if (!THGPUTensor_isSameSizeAs(src2, t)) { v2 = THGPUTensor_newClone(src2); tensor_resize_as(v2, t); }
  THGPUTensor *tmp = tensor_new();
  tensor_resize_as(tmp, t);
  apply<2>(tmp, v1 ? v1 : src1, v2 ? v2 : src2, op, name);
  if (self != t) tensor_resize_as(self, t);
  apply<2>(self, t, tmp, SumOp(), name);
  if (v1) tensor_free(v1);
  if (v2) tensor_free(v2);
  tensor_free(tmp);
}

}  // namespace thc

using namespace thc;

#define THC_DEFINE_UNARY(NAME, OP) \
  THC_API void THGPUTensor_##NAME(THGPUTensor *self, THGPUTensor *src) { THC_BEGIN unary(self, src, OP(), #NAME); THC_END() }
THC_DEFINE_UNARY(log, LogOp)
THC_DEFINE_UNARY(log1p, Log1pOp)
THC_DEFINE_UNARY(exp, ExpOp)
THC_DEFINE_UNARY(cos, CosOp)
THC_DEFINE_UNARY(acos, AcosOp)
THC_DEFINE_UNARY(cosh, CoshOp)
THC_DEFINE_UNARY(sin, SinOp)
THC_DEFINE_UNARY(asin, AsinOp)
THC_DEFINE_UNARY(sinh, SinhOp)
THC_DEFINE_UNARY(tan, TanOp)
THC_DEFINE_UNARY(atan, AtanOp)
THC_DEFINE_UNARY(tanh, TanhOp)
THC_DEFINE_UNARY(sqrt, SqrtOp)
THC_DEFINE_UNARY(ceil, CeilOp)
THC_DEFINE_UNARY(floor, FloorOp)
THC_DEFINE_UNARY(abs, AbsOp)
THC_DEFINE_UNARY(sign, SignOp)
THC_DEFINE_UNARY(round, RoundOp)
#undef THC_DEFINE_UNARY

THC_API void THGPUTensor_pow(THGPUTensor *self, THGPUTensor *src, float value) {
  THC_BEGIN unary(self, src, PowOp{value}, "pow"); THC_END()
}
THC_API void THGPUTensor_clamp(THGPUTensor *self, THGPUTensor *src, float min_value, float max_value) {
  THC_BEGIN unary(self, src, ClampOp{min_value, max_value}, "clamp"); THC_END()
}
THC_API void THGPUTensor_atan2(THGPUTensor *r_, THGPUTensor *tx, THGPUTensor *ty) {
  THC_BEGIN binary(r_, tx, ty, Atan2Op(), "atan2"); THC_END()
}

#define THC_DEFINE_CMP(NAME, C) \
  THC_API void THGPUTensor_##NAME##Value(THGPUTensor *self_, THGPUTensor *src, float value) { \
    THC_BEGIN unary(self_, src, CmpValueOp<C>{value}, #NAME "Value"); THC_END() } \
  THC_API void THGPUTensor_##NAME##Tensor(THGPUTensor *self_, THGPUTensor *src1, THGPUTensor *src2) { \
    THC_BEGIN binary(self_, src1, src2, CmpTensorOp<C>(), #NAME "Tensor"); THC_END() }
THC_DEFINE_CMP(lt, CMP_LT)
THC_DEFINE_CMP(gt, CMP_GT)
THC_DEFINE_CMP(le, CMP_LE)
THC_DEFINE_CMP(ge, CMP_GE)
THC_DEFINE_CMP(eq, CMP_EQ)
THC_DEFINE_CMP(ne, CMP_NE)
#undef THC_DEFINE_CMP

THC_API void THGPUTensor_addcmul(THGPUTensor *self, THGPUTensor *t, float value, THGPUTensor *src1, THGPUTensor *src2) {
  THC_BEGIN add_scaled(self, t, src1, src2, ScaledMulOp{value}, "addcmul"); THC_END()
}
THC_API void THGPUTensor_addcdiv(THGPUTensor *self, THGPUTensor *t, float value, THGPUTensor *src1, THGPUTensor *src2) {
  THC_BEGIN add_scaled(self, t, src1, src2, ScaledDivOp{value}, "addcdiv"); THC_END()
}

THC_API float THGPUTensor_normall(THGPUTensor *self, float value) {
  THC_BEGIN
  if (nelem(self) == 0) return 0.f;
  if (value == 0.f) return (float)sum_of(self, nullptr, NonZeroOp(), "normall");
  if (value == 1.f) return (float)sum_of(self, nullptr, AbsOp(), "normall");
  if (value == 2.f) return (float)sqrt(sum_of(self, nullptr, SquareOp(), "normall"));
  return (float)pow(sum_of(self, nullptr, AbsPowOp{value}, "normall"), 1.0 / (double)value);
  THC_END(0.f)
}
THC_API float THGPUTensor_dist(THGPUTensor *self, THGPUTensor *src, float value) {
  THC_BEGIN
  THC_ARG(nelem(self) == nelem(src), 2, "sizes do not match");
  if (nelem(self) == 0) return 0.f;
  return (float)pow(sum_of(self, src, AbsDiffPowOp{value}, "dist"), 1.0 / (double)value);
  THC_END(0.f)
}
THC_API float THGPUTensor_varall(THGPUTensor *self) {
  THC_BEGIN
  const long n = nelem(self);
  THC_ARG(n > 0, 1, "empty Tensor");
  const double mean = (double)THGPUTensor_sumall(self) / (double)n;
  return (float)(sum_of(self, nullptr, CenteredSquareOp{mean}, "varall") / (double)(n - 1));
  THC_END(0.f)
}
THC_API float THGPUTensor_stdall(THGPUTensor *self) {
  THC_BEGIN
  const long n = nelem(self);
  THC_ARG(n > 0, 1, "empty Tensor");
  const double mean = (double)THGPUTensor_sumall(self) / (double)n;
  return (float)sqrt(sum_of(self, nullptr, CenteredSquareOp{mean}, "stdall") / (double)(n - 1));
  THC_END(0.f)
}
// norm along a dimension (mcw_torch7_core/lib/TH/generic/THTensorMath.c:1401-1427): the terms |x|^value (or
// x != 0 for value 0) go through the dim-wise sum, whose accumulator is a double like TH's, then the root.
THC_API void THGPUTensor_norm(THGPUTensor *self, THGPUTensor *src, float value, long dimension) {
  THC_BEGIN
  THC_ARG(dimension >= 0 && dimension < src->nDimension, 3, "invalid dimension");
  THGPUTensor *terms = tensor_new();
  tensor_resize_as(terms, src);
  if (value == 0.f) apply<1>(terms, src, nullptr, NonZeroOp(), "norm");
  else apply<1>(terms, src, nullptr, AbsPowOp{value}, "norm");
  THGPUTensor_sum(self, terms, dimension);
  tensor_free(terms);
  if (value != 0.f && value != 1.f) apply<1>(self, self, nullptr, PowOp{1.f / value}, "norm");
  THC_END()
}

