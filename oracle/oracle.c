/* TEST INFRASTRUCTURE ONLY -- the checker for tests, the smoke run and the bench's CPU
 * baseline leg.  Nothing in the product (the package, its CUDA library) links, imports or
 * executes this file.
 *
 * A plain-C restatement of the reference's CPU path (Torch7 TH + nn "generic" kernels) for the
 * conv / pool / threshold / tensor-math hot path.  Every function cites the reference code it
 * follows (paths relative to the reference project).  The arithmetic ORDER per output element is
 * kept exactly as in the reference (sequential fp32 dot products, double accumulators where TH
 * uses `accreal`), so on the stride-1 cases the reference can run, this port reproduces the
 * reference's own compiled code bit for bit; loops are only interchanged in ways that do not
 * alter any element's sequence of floating-point operations.
 *
 * Parity pin: tests compare this port with the reference's own sources compiled by the Makefile
 * beside this file (the `ref` target) and with golden vectors generated from that build. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>

/* ------------------------------------------------------------------------------------------
 * RNG: TH's Mersenne Twister (mcw_torch7_core/lib/TH/THRandom.c:96-118 seeding, :130-149
 * state refresh, :151-184 tempering / [0,1) double, :192-220 uniform and Box-Muller normal).
 * ---------------------------------------------------------------------------------------- */
#define ORC_MT_N 624
#define ORC_MT_M 397

typedef struct orc_rng {
  uint64_t state[ORC_MT_N];
  int left, next;
  int normal_is_valid;
  double normal_x, normal_y, normal_rho;
} orc_rng;

orc_rng *orc_rng_new(unsigned long seed)
{
  orc_rng *g = (orc_rng *)calloc(1, sizeof(orc_rng));
  int j;
  g->state[0] = seed & 0xffffffffUL;
  for (j = 1; j < ORC_MT_N; j++) {
    g->state[j] = (1812433253UL * (g->state[j - 1] ^ (g->state[j - 1] >> 30)) + j);
    g->state[j] &= 0xffffffffUL;
  }
  g->left = 1;
  return g;
}
void orc_rng_free(orc_rng *g) { free(g); }

static void orc_rng_next_state(orc_rng *g)
{
#define ORC_MIX(u, v) (((u) & 0x80000000UL) | ((v) & 0x7fffffffUL))
#define ORC_TWIST(u, v) ((ORC_MIX(u, v) >> 1) ^ (((v) & 1UL) ? 0x9908b0dfUL : 0UL))
  uint64_t *p = g->state;
  int j;
  g->left = ORC_MT_N;
  g->next = 0;
  for (j = ORC_MT_N - ORC_MT_M + 1; --j; p++) *p = p[ORC_MT_M] ^ ORC_TWIST(p[0], p[1]);
  for (j = ORC_MT_M; --j; p++) *p = p[ORC_MT_M - ORC_MT_N] ^ ORC_TWIST(p[0], p[1]);
  *p = p[ORC_MT_M - ORC_MT_N] ^ ORC_TWIST(p[0], g->state[0]);
}

static double orc_rng_u01(orc_rng *g)
{
  uint64_t y;
  if (--g->left == 0) orc_rng_next_state(g);
  y = g->state[g->next++];
  y ^= (y >> 11);
  y ^= (y << 7) & 0x9d2c5680UL;
  y ^= (y << 15) & 0xefc60000UL;
  y ^= (y >> 18);
  return (double)y * (1.0 / 4294967296.0);
}

/* THFloatTensor_uniform: one double draw per element, cast to float, in logical order
 * (mcw_torch7_core/lib/TH/generic/THTensorRandom.c:38-41). */
void orc_rng_uniform(orc_rng *g, float *out, long n, double a, double b)
{
  long i;
  for (i = 0; i < n; i++) out[i] = (float)(orc_rng_u01(g) * (b - a) + a);
}

/* THFloatTensor_normal (generic/THTensorRandom.c:43-46 over THRandom.c:201-220): pairs of
 * draws, cosine branch first, sine branch from the cached pair second. */
void orc_rng_normal(orc_rng *g, float *out, long n, double mean, double stdv)
{
  long i;
  for (i = 0; i < n; i++) {
    double v;
    if (!g->normal_is_valid) {
      g->normal_x = orc_rng_u01(g);
      g->normal_y = orc_rng_u01(g);
      g->normal_rho = sqrt(-2. * log(1.0 - g->normal_y));
      g->normal_is_valid = 1;
    } else
      g->normal_is_valid = 0;
    if (g->normal_is_valid) v = g->normal_rho * cos(2. * M_PI * g->normal_x) * stdv + mean;
    else v = g->normal_rho * sin(2. * M_PI * g->normal_x) * stdv + mean;
    out[i] = (float)v;
  }
}

/* ------------------------------------------------------------------------------------------
 * Column unfolding.  Stride 1: mcw_nn/generic/SpatialConvolutionMM.c:52-96 (unfolded_copy).
 * General stride/pad: the reference GPU kernel's index rule
 * (gputorch/lib/THC/gpunn-impl/SpatialConvolutionMM.cpp:10-52): row r = c*kH*kW + kh*kW + kw,
 * column p = y*oW + x reads in[c, y*dH - pad + kh, x*dW - pad + kw] or 0 outside the image.
 * For dH = dW = 1 both give the same matrix.
 * ---------------------------------------------------------------------------------------- */
static void orc_unfold(const float *in, float *col, long C, long H, long W, long kH, long kW,
                       long dH, long dW, long pad, long oH, long oW)
{
  long r;
  for (r = 0; r < C * kH * kW; r++) {
    long c = r / (kH * kW), rest = r % (kH * kW), kh = rest / kW, kw = rest % kW, y, x;
    float *dst = col + r * oH * oW;
    const float *src = in + c * H * W;
    for (y = 0; y < oH; y++) {
      long iy = y * dH - pad + kh;
      for (x = 0; x < oW; x++) {
        long ix = x * dW - pad + kw;
        dst[y * oW + x] = (iy >= 0 && iy < H && ix >= 0 && ix < W) ? src[iy * W + ix] : 0.f;
      }
    }
  }
}

/* nn.SpatialConvolutionMM forward, batch mode
 * (mcw_nn/generic/SpatialConvolutionMM.c:98-118 frame, :186-201 batch loop).
 * Per image: out[k,:] = bias[k]; then addmm(out2d, 1, out2d, 1, weight, finput), which lands in
 * THBlas gemm('n','n', P, K, R, ...) (mcw_torch7_core/lib/TH/generic/THBlas.c:319-336):
 *   sum = 0; for l in 0..R-1: sum += col[l][p] * W[k][l];  out = 1*out + 1*sum   (all fp32). */
void orc_conv_mm_forward(const float *in, const float *weight, const float *bias, float *out,
                         long N, long C, long H, long W, long K, long kH, long kW, long dH,
                         long dW, long pad)
{
  long oH = (H + 2 * pad - kH) / dH + 1, oW = (W + 2 * pad - kW) / dW + 1;
  long R = C * kH * kW, P = oH * oW, n;
#pragma omp parallel for
  for (n = 0; n < N; n++) {
    float *col = (float *)malloc(sizeof(float) * R * P);
    float *acc = (float *)malloc(sizeof(float) * P);
    long k, r, p;
    orc_unfold(in + n * C * H * W, col, C, H, W, kH, kW, dH, dW, pad, oH, oW);
    for (k = 0; k < K; k++) {
      float *o = out + (n * K + k) * P;
      for (p = 0; p < P; p++) acc[p] = 0.f;
      for (r = 0; r < R; r++) {
        const float w = weight[k * R + r];
        const float *cr = col + r * P;
        for (p = 0; p < P; p++) acc[p] += cr[p] * w;
      }
      for (p = 0; p < P; p++) o[p] = 1.f * bias[k] + 1.f * acc[p];
    }
    free(col);
    free(acc);
  }
}

/* nn.SpatialConvolutionMM gradInput (SpatialConvolutionMM.c:211-223 frame, :243-279 batch).
 * gradCol[r][p] = 0*old + sum_k gradOut[k][p] * W[k][r] (gemm('n','t'), THBlas.c:354-370, sequential
 * over k), then unfolded_acc (:6-50): gradIn zeroed, and for c, kh ascending, kw ascending, each
 * column block is added onto the image rows it was copied from.  The stride-aware form visits the
 * same (kh, kw) order and adds gradCol[(c,kh,kw), (y,x)] to gradIn[c, y*dH-pad+kh, x*dW-pad+kw]. */
void orc_conv_mm_grad_input(const float *gradOut, const float *weight, float *gradIn, long N,
                            long C, long H, long W, long K, long kH, long kW, long dH, long dW,
                            long pad)
{
  long oH = (H + 2 * pad - kH) / dH + 1, oW = (W + 2 * pad - kW) / dW + 1;
  long R = C * kH * kW, P = oH * oW, n;
#pragma omp parallel for
  for (n = 0; n < N; n++) {
    float *gcol = (float *)malloc(sizeof(float) * R * P);
    const float *go = gradOut + n * K * P;
    float *gi = gradIn + n * C * H * W;
    long r, k, p;
    for (r = 0; r < R; r++) {
      float *g = gcol + r * P;
      for (p = 0; p < P; p++) g[p] = 0.f;
      for (k = 0; k < K; k++) {
        const float w = weight[k * R + r];
        const float *gk = go + k * P;
        for (p = 0; p < P; p++) g[p] += gk[p] * w;
      }
      for (p = 0; p < P; p++) g[p] = 1.f * g[p]; /* beta = 0 on a zeroed buffer, alpha = 1 */
    }
    memset(gi, 0, sizeof(float) * C * H * W);
    for (r = 0; r < R; r++) {
      long c = r / (kH * kW), rest = r % (kH * kW), kh = rest / kW, kw = rest % kW, y, x;
      const float *g = gcol + r * P;
      for (y = 0; y < oH; y++) {
        long iy = y * dH - pad + kh;
        if (iy < 0 || iy >= H) continue;
        for (x = 0; x < oW; x++) {
          long ix = x * dW - pad + kw;
          if (ix < 0 || ix >= W) continue;
          gi[(c * H + iy) * W + ix] += g[y * oW + x];
        }
      }
    }
    free(gcol);
  }
}

/* nn.SpatialConvolutionMM accGradParameters (SpatialConvolutionMM.c:284-309 frame, :324-343
 * serial batch loop).  Per image, in batch order:
 *   gradW[k][r] = 1*gradW[k][r] + scale * (sum_p col[r][p]*gradOut[k][p])   gemm('t','n'), THBlas.c:337-353
 *   gradBias[k] += scale * (float sum_p gradOut[k][p])                      (:297-305)          */
void orc_conv_mm_acc_grad(const float *in, const float *gradOut, float *gradW, float *gradBias,
                          float scale, long N, long C, long H, long W, long K, long kH, long kW,
                          long dH, long dW, long pad)
{
  long oH = (H + 2 * pad - kH) / dH + 1, oW = (W + 2 * pad - kW) / dW + 1;
  long R = C * kH * kW, P = oH * oW, n;
  float *col = (float *)malloc(sizeof(float) * R * P);
  for (n = 0; n < N; n++) {
    const float *go = gradOut + n * K * P;
    long k;
    orc_unfold(in + n * C * H * W, col, C, H, W, kH, kW, dH, dW, pad, oH, oW);
#pragma omp parallel for
    for (k = 0; k < K; k++) {
      const float *gk = go + k * P;
      long r, p;
      float bsum = 0;
      for (r = 0; r < R; r++) {
        const float *cr = col + r * P;
        float sum = 0;
        for (p = 0; p < P; p++) sum += cr[p] * gk[p];
        gradW[k * R + r] = 1.f * gradW[k * R + r] + scale * sum;
      }
      for (p = 0; p < P; p++) bsum += gk[p];
      gradBias[k] += scale * bsum;
    }
  }
  free(col);
}

/* ------------------------------------------------------------------------------------------
 * nn.SpatialMaxPooling (mcw_nn/generic/SpatialMaxPooling.c:5-56 frame, :82-140 driver).
 * indices is [2, N*C, oH, oW] as floats: plane 0 = 1-based window row, plane 1 = 1-based window
 * column; scan rows then columns, strict '>' from -DBL_MAX so the first maximum wins.
 * ---------------------------------------------------------------------------------------- */
void orc_maxpool_forward(const float *in, float *out, float *indices, long NC, long H, long W,
                         long kH, long kW, long dH, long dW)
{
  long oH = (H - kH) / dH + 1, oW = (W - kW) / dW + 1, k;
  float *indy = indices, *indx = indices + NC * oH * oW;
#pragma omp parallel for
  for (k = 0; k < NC; k++) {
    long i, j;
    for (i = 0; i < oH; i++)
      for (j = 0; j < oW; j++) {
        const float *ip = in + k * W * H + i * W * dH + j * dW;
        long maxindex = -1, tcntr = 0, x, y;
        float maxval = (float)(-DBL_MAX); /* reference: real maxval = -THInf, THInf = DBL_MAX */
        for (y = 0; y < kH; y++)
          for (x = 0; x < kW; x++) {
            float val = ip[y * W + x];
            if (val > maxval) { maxval = val; maxindex = tcntr; }
            tcntr++;
          }
        out[k * oW * oH + i * oW + j] = maxval;
        indy[k * oW * oH + i * oW + j] = (float)((int)(maxindex / kW) + 1);
        indx[k * oW * oH + i * oW + j] = (float)((maxindex % kW) + 1);
      }
  }
}

/* SpatialMaxPooling.c:147-176 frame, :200-248 driver: gradIn = 0, then outputs visited in
 * row-major order each add their gradOut onto the argmax pixel (fp32 adds, that order). */
void orc_maxpool_backward(const float *gradOut, const float *indices, float *gradIn, long NC,
                          long H, long W, long oH, long oW, long dH, long dW)
{
  const float *indy = indices, *indx = indices + NC * oH * oW;
  long k;
  memset(gradIn, 0, sizeof(float) * NC * H * W);
#pragma omp parallel for
  for (k = 0; k < NC; k++) {
    long i, j;
    for (i = 0; i < oH; i++)
      for (j = 0; j < oW; j++) {
        long maxi = (long)indy[k * oH * oW + i * oW + j] - 1 + i * dH;
        long maxj = (long)indx[k * oH * oW + i * oW + j] - 1 + j * dW;
        gradIn[k * H * W + maxi * W + maxj] += gradOut[k * oH * oW + i * oW + j];
      }
  }
}

/* ------------------------------------------------------------------------------------------
 * nn.Threshold (mcw_nn/generic/Threshold.c:5-32); th/val are cast to float first (:8-9).
 * ---------------------------------------------------------------------------------------- */
void orc_threshold_forward(const float *in, float *out, long n, double threshold, double val)
{
  float th = (float)threshold, v = (float)val;
  long i;
#pragma omp parallel for
  for (i = 0; i < n; i++) out[i] = (in[i] > th) ? in[i] : v;
}
void orc_threshold_backward(const float *in, const float *gradOut, float *gradIn, long n,
                            double threshold)
{
  float th = (float)threshold;
  long i;
#pragma omp parallel for
  for (i = 0; i < n; i++) gradIn[i] = (in[i] > th) ? gradOut[i] : 0.f;
}

/* ------------------------------------------------------------------------------------------
 * Tensor math (mcw_torch7_core/lib/TH/generic/THTensorMath.c).  2-D operands are described by
 * (pointer, stride0, stride1) so transposed views are first-class, as in TH.
 * ---------------------------------------------------------------------------------------- */
/* add: :226-240   r = t + value */
void orc_add(float *r, long rs0, long rs1, const float *t, long ts0, long ts1, float value,
             long n0, long n1)
{
  long i, j;
#pragma omp parallel for private(j)
  for (i = 0; i < n0; i++)
    for (j = 0; j < n1; j++) r[i * rs0 + j * rs1] = t[i * ts0 + j * ts1] + value;
}
/* cadd: :291-310   r = t + value * src (product rounded, then the sum rounded) */
void orc_cadd(float *r, long rs0, long rs1, const float *t, long ts0, long ts1, float value,
              const float *s, long ss0, long ss1, long n0, long n1)
{
  long i, j;
#pragma omp parallel for private(j)
  for (i = 0; i < n0; i++)
    for (j = 0; j < n1; j++)
      r[i * rs0 + j * rs1] = t[i * ts0 + j * ts1] + value * s[i * ss0 + j * ss1];
}
/* cmul: :312-327 */
void orc_cmul(float *r, long rs0, long rs1, const float *t, long ts0, long ts1, const float *s,
              long ss0, long ss1, long n0, long n1)
{
  long i, j;
#pragma omp parallel for private(j)
  for (i = 0; i < n0; i++)
    for (j = 0; j < n1; j++)
      r[i * rs0 + j * rs1] = t[i * ts0 + j * ts1] * s[i * ss0 + j * ss1];
}
/* sumall: :212-217, double accumulator over logical order */
double orc_sumall(const float *t, long ts0, long ts1, long n0, long n1)
{
  double sum = 0;
  long i, j;
  for (i = 0; i < n0; i++)
    for (j = 0; j < n1; j++) sum += t[i * ts0 + j * ts1];
  return sum;
}
/* maxall: :203-210, starts from element 0, strict '>' */
float orc_maxall(const float *t, long ts0, long ts1, long n0, long n1)
{
  float m = t[0];
  long i, j;
  for (i = 0; i < n0; i++)
    for (j = 0; j < n1; j++)
      if (t[i * ts0 + j * ts1] > m) m = t[i * ts0 + j * ts1];
  return m;
}
/* sum(dim): :674-691, double accumulator, cast to float at the end.  dim is 0-based. */
void orc_sum_dim(float *r, const float *t, long ts0, long ts1, long n0, long n1, int dim)
{
  long o, i, no = dim == 0 ? n1 : n0, ni = dim == 0 ? n0 : n1;
  long so = dim == 0 ? ts1 : ts0, si = dim == 0 ? ts0 : ts1;
#pragma omp parallel for private(i)
  for (o = 0; o < no; o++) {
    double sum = 0;
    for (i = 0; i < ni; i++) sum += t[o * so + i * si];
    r[o] = (float)sum;
  }
}
/* max(dim): :615-642, values + 0-based index of the first maximum (strict '>'). */
void orc_max_dim(float *values, long *indices, const float *t, long ts0, long ts1, long n0,
                 long n1, int dim)
{
  long o, i, no = dim == 0 ? n1 : n0, ni = dim == 0 ? n0 : n1;
  long so = dim == 0 ? ts1 : ts0, si = dim == 0 ? ts0 : ts1;
#pragma omp parallel for private(i)
  for (o = 0; o < no; o++) {
    long idx = 0;
    float m = t[o * so];
    for (i = 1; i < ni; i++)
      if (t[o * so + i * si] > m) { idx = i; m = t[o * so + i * si]; }
    indices[o] = idx;
    values[o] = m;
  }
}
/* addmm: :458-561 over THBlas gemm (generic/THBlas.c:319-390).  Whatever transpose flags the
 * strides select, every variant computes, per element,
 *   sum = 0; for l ascending: sum += m1[i][l]*m2[l][j];   r[i][j] = beta*t[i][j] + alpha*sum
 * in fp32.  r may alias t. */
void orc_addmm(float *r, long rs0, long rs1, float beta, const float *t, long ts0, long ts1,
               float alpha, const float *m1, long as0, long as1, const float *m2, long bs0,
               long bs1, long M, long N, long K)
{
  long i;
#pragma omp parallel for
  for (i = 0; i < M; i++) {
    float *acc = (float *)malloc(sizeof(float) * N);
    long j, l;
    for (j = 0; j < N; j++) acc[j] = 0.f;
    for (l = 0; l < K; l++) {
      const float a = m1[i * as0 + l * as1];
      const float *b = m2 + l * bs0;
      if (bs1 == 1) for (j = 0; j < N; j++) acc[j] += a * b[j];
      else for (j = 0; j < N; j++) acc[j] += a * b[j * bs1];
    }
    for (j = 0; j < N; j++) r[i * rs0 + j * rs1] = beta * t[i * ts0 + j * ts1] + alpha * acc[j];
    free(acc);
  }
}

/* ------------------------------------------------------------------------------------------
 * Classifier tail.  LogSoftMax: mcw_nn/generic/LogSoftMax.c:5-55 (fwd, uses the polynomial
 * exp(-x) of mcw_torch7_core/lib/TH/THLogAdd.c:56-86), :57-103 (bwd).
 * ---------------------------------------------------------------------------------------- */
static double orc_exp_minus_approx(double x)
{
  if (x < 13.0) {
    double y = 1.0 + x * (0.125 + x * (0.0078125 + x * (0.00032552083 + x * 1.0172526e-5)));
    y *= y; y *= y; y *= y;
    return 1 / y;
  }
  return 0;
}
void orc_logsoftmax_forward(const float *in, float *out, long nframe, long dim)
{
  long t;
#pragma omp parallel for
  for (t = 0; t < nframe; t++) {
    const float *x = in + dim * t;
    float *o = out + dim * t;
    double logsum = 0;
    float maxInput = (float)(-DBL_MAX);
    long d;
    for (d = 0; d < dim; d++) maxInput = maxInput > x[d] ? maxInput : x[d];
    for (d = 0; d < dim; d++) logsum += orc_exp_minus_approx(maxInput - x[d]);
    logsum = maxInput + log(logsum);
    for (d = 0; d < dim; d++) o[d] = x[d] - logsum;
  }
}
void orc_logsoftmax_backward(const float *gradOut, const float *out, float *gradIn, long nframe,
                             long dim)
{
  long t;
#pragma omp parallel for
  for (t = 0; t < nframe; t++) {
    double sum = 0;
    long d;
    for (d = 0; d < dim; d++) sum += gradOut[dim * t + d];
    for (d = 0; d < dim; d++)
      gradIn[dim * t + d] = gradOut[dim * t + d] - exp(out[dim * t + d]) * sum;
  }
}
/* nn.ClassNLLCriterion (mcw_nn/ClassNLLCriterion.lua:13-40 fwd, :42-70 bwd), sizeAverage = true,
 * no class weights; targets are 1-based.  Lua numbers are doubles. */
double orc_classnll_forward(const float *in, const float *target, long nframe, long dim)
{
  double output = 0;
  long i;
  for (i = 0; i < nframe; i++) output = output - in[i * dim + ((long)target[i] - 1)];
  return output / nframe;
}
void orc_classnll_backward(const float *target, float *gradIn, long nframe, long dim)
{
  long i;
  double z = -1.0 / nframe;
  memset(gradIn, 0, sizeof(float) * nframe * dim);
  for (i = 0; i < nframe; i++) gradIn[i * dim + ((long)target[i] - 1)] = (float)z;
}

/* ------------------------------------------------------------------------------------------
 * Pointwise functions and whole-tensor norms (mcw_torch7_core/lib/TH/generic/THTensorMath.c),
 * contiguous operands of n elements.  Operation codes follow ORC_POINTWISE_NAMES in
 * oracle/__init__.py.
 *   unary functions  :1236-1241 (macro), :1277-1294   r = (float) cfunc((double) t)
 *   pow              :1243-1249, :1289                r = (float) pow(t, value)
 *   clamp            :274-290                         r = t < min ? min : (t > max ? max : t)
 *   sign             :746-760                         1 / -1 / 0
 *   atan2            :1296-1300                       r = (float) atan2(tx, ty)
 *   comparisons      :1198-1234 (ValueT / TensorT)    r = 1 where t OP value (or t OP tb), else 0
 *   addcmul, addcdiv :346-367                         r = t + value * s1 * s2,  t + value * s1 / s2,
 *                                                     every step rounded to float
 * ---------------------------------------------------------------------------------------- */
void orc_pointwise(int op, float *r, const float *a, const float *b, const float *c, long n, float v1, float v2)
{
  long i;
  for (i = 0; i < n; i++) {
    const float x = a[i];
    float y = 0.f;
    switch (op) {
      case 0: y = log(x); break;
      case 1: y = log1p(x); break;
      case 2: y = exp(x); break;
      case 3: y = cos(x); break;
      case 4: y = acos(x); break;
      case 5: y = cosh(x); break;
      case 6: y = sin(x); break;
      case 7: y = asin(x); break;
      case 8: y = sinh(x); break;
      case 9: y = tan(x); break;
      case 10: y = atan(x); break;
      case 11: y = tanh(x); break;
      case 12: y = sqrt(x); break;
      case 13: y = ceil(x); break;
      case 14: y = floor(x); break;
      case 15: y = fabs(x); break;
      case 16: y = x > 0 ? 1.f : (x < 0 ? -1.f : 0.f); break;
      case 17: y = round(x); break;
      case 18: y = pow(x, v1); break;
      case 19: y = x < v1 ? v1 : (x > v2 ? v2 : x); break;
      case 20: y = atan2(x, b[i]); break;
      case 21: y = x < v1; break;
      case 22: y = x > v1; break;
      case 23: y = x <= v1; break;
      case 24: y = x >= v1; break;
      case 25: y = x == v1; break;
      case 26: y = x != v1; break;
      case 27: y = x < b[i]; break;
      case 28: y = x > b[i]; break;
      case 29: y = x <= b[i]; break;
      case 30: y = x >= b[i]; break;
      case 31: y = x == b[i]; break;
      case 32: y = x != b[i]; break;
      case 33: { float p = v1 * b[i]; p = p * c[i]; y = x + p; } break;
      case 34: { float p = v1 * b[i]; p = p / c[i]; y = x + p; } break;
    }
    r[i] = y;
  }
}
/* normall: :1429-1446 (double accumulator) */
double orc_normall(const float *t, long n, float value)
{
  double sum = 0;
  long i;
  if (value == 0) { for (i = 0; i < n; i++) sum += t[i] != 0.0; return sum; }
  if (value == 1) { for (i = 0; i < n; i++) sum += fabs(t[i]); return sum; }
  if (value == 2) { for (i = 0; i < n; i++) { double z = t[i]; sum += z * z; } return sqrt(sum); }
  for (i = 0; i < n; i++) sum += pow(fabs(t[i]), value);
  return pow(sum, 1.0 / value);
}
/* dist: :1495-1501 (the accumulator is a float there) */
double orc_dist(const float *a, const float *b, long n, float value)
{
  float sum = 0;
  long i;
  for (i = 0; i < n; i++) sum += pow(fabs(a[i] - b[i]), value);
  return pow(sum, 1.0 / value);
}
/* varall: :1509-1516 (mean = sumall / n in double); stdall is its square root (:1518-1521) */
double orc_varall(const float *t, long n)
{
  double mean = 0, sum = 0;
  long i;
  for (i = 0; i < n; i++) mean += t[i];
  mean /= n;
  for (i = 0; i < n; i++) sum += (t[i] - mean) * (t[i] - mean);
  return sum / (n - 1);
}
/* norm along a dimension of a contiguous n0 x n1 matrix: :1401-1427 (double accumulator per output) */
void orc_norm_dim(float *r, const float *t, long n0, long n1, float value, int dim)
{
  long i, j, outer = dim == 0 ? n1 : n0, inner = dim == 0 ? n0 : n1;
  for (i = 0; i < outer; i++) {
    double sum = 0;
    for (j = 0; j < inner; j++) {
      const float x = dim == 0 ? t[j * n1 + i] : t[i * n1 + j];
      if (value == 0) sum += x != 0.0;
      else sum += pow(fabs(x), value);
    }
    r[i] = value == 0 ? sum : pow(sum, 1.0 / value);
  }
}


/* ---- the rest of the tensor-math surface and two more nn operators ---------------------------------
 * All on contiguous blocks viewed as [outer][D][inner], D the dimension worked on. */

/* prodall: THTensorMath.c:219-224 (accreal = double) */
double orc_prodall(const float *t, long n)
{
  double prod = 1;
  long i;
  for (i = 0; i < n; i++) prod *= t[i];
  return prod;
}
/* prod along D: THTensorMath.c:693-711 (double accumulator per output, cast to float) */
void orc_prod_dim(float *r, const float *t, long outer, long D, long inner)
{
  long o, i, d;
  for (o = 0; o < outer; o++)
    for (i = 0; i < inner; i++) {
      double prod = 1;
      for (d = 0; d < D; d++) prod *= t[(o * D + d) * inner + i];
      r[o * inner + i] = (float)prod;
    }
}
/* renorm of every slice d along D: THTensorMath.c:1447-1496.  The norm accumulates in a FLOAT (`real norm`), the
 * terms are doubles for value == 2 and pow() results otherwise; new_norm = maxnorm / (norm + 1e-7) is evaluated in
 * double and stored in a float. */
void orc_renorm(float *r, const float *t, long outer, long D, long inner, float value, float maxnorm)
{
  long o, i, d;
  for (d = 0; d < D; d++) {
    float norm = 0, new_norm;
    for (o = 0; o < outer; o++)
      for (i = 0; i < inner; i++) {
        const float x = t[(o * D + d) * inner + i];
        if (value == 1) norm += fabs(x);
        else if (value == 2) { double z = x; norm += z * z; }
        else norm += pow(fabs(x), value);
      }
    norm = pow(norm, 1 / value);
    if (norm > maxnorm) {
      new_norm = maxnorm / (norm + 1e-7);
      for (o = 0; o < outer; o++)
        for (i = 0; i < inner; i++) r[(o * D + d) * inner + i] = t[(o * D + d) * inner + i] * new_norm;
    } else {
      for (o = 0; o < outer; o++)
        for (i = 0; i < inner; i++) r[(o * D + d) * inner + i] = t[(o * D + d) * inner + i];
    }
  }
}
/* indexSelect :69-108, indexCopy :110-147, indexFill :149-172; idx holds 1-based positions */
void orc_index_select(float *r, const float *t, const long *idx, long outer, long D, long nidx, long inner)
{
  long o, k, i;
  for (o = 0; o < outer; o++)
    for (k = 0; k < nidx; k++)
      for (i = 0; i < inner; i++) r[(o * nidx + k) * inner + i] = t[(o * D + idx[k] - 1) * inner + i];
}
void orc_index_copy(float *r, const float *src, const long *idx, long outer, long D, long nidx, long inner)
{
  long o, k, i;
  for (k = 0; k < nidx; k++)   /* slice by slice, in index order: a repeated index keeps the last copy */
    for (o = 0; o < outer; o++)
      for (i = 0; i < inner; i++) r[(o * D + idx[k] - 1) * inner + i] = src[(o * nidx + k) * inner + i];
}
void orc_index_fill(float *r, const long *idx, long outer, long D, long nidx, long inner, float val)
{
  long o, k, i;
  for (k = 0; k < nidx; k++)
    for (o = 0; o < outer; o++)
      for (i = 0; i < inner; i++) r[(o * D + idx[k] - 1) * inner + i] = val;
}
/* nn.SoftMax: mcw_nn/generic/SoftMax.c:5-60 forward (z stored as float, sum in double, out *= 1/sum),
 * :62-110 backward (sum of gradOut * out in double) */
void orc_softmax_forward(const float *in, float *out, long nframe, long dim)
{
  long t, d;
  for (t = 0; t < nframe; t++) {
    const float *x = in + dim * t;
    float *o = out + dim * t;
    float inputMax = -HUGE_VALF;
    double sum = 0;
    for (d = 0; d < dim; d++) if (x[d] >= inputMax) inputMax = x[d];
    for (d = 0; d < dim; d++) {
      float z = orc_exp_minus_approx(inputMax - x[d]);
      o[d] = z;
      sum += z;
    }
    for (d = 0; d < dim; d++) o[d] *= 1 / sum;
  }
}
void orc_softmax_backward(const float *gradOut, const float *out, float *gradIn, long nframe, long dim)
{
  long t, d;
  for (t = 0; t < nframe; t++) {
    double sum = 0;
    for (d = 0; d < dim; d++) sum += (double)gradOut[dim * t + d] * out[dim * t + d];
    for (d = 0; d < dim; d++) gradIn[dim * t + d] = out[dim * t + d] * (gradOut[dim * t + d] - sum);
  }
}
/* nn.SpatialAveragePooling: mcw_nn/generic/SpatialAveragePooling.c:5-80 forward (window SUM in a float, no
 * division), :84-150 backward (gradInput zeroed, then every window adds its gradOutput to the pixels it covers,
 * windows visited in ascending (y, x) order) */
void orc_sumpool_forward(const float *in, float *out, long planes, long H, long W, int kH, int kW, int dH, int dW)
{
  const long oH = (H - kH) / dH + 1, oW = (W - kW) / dW + 1;
  long p, y, x;
  int ky, kx;
  for (p = 0; p < planes; p++)
    for (y = 0; y < oH; y++)
      for (x = 0; x < oW; x++) {
        const float *q = in + (p * H + y * dH) * W + x * dW;
        float sum = 0;
        for (ky = 0; ky < kH; ky++, q += W)
          for (kx = 0; kx < kW; kx++) sum += q[kx];
        out[(p * oH + y) * oW + x] = sum;
      }
}
void orc_sumpool_backward(const float *gradOut, float *gradIn, long planes, long H, long W, int kH, int kW, int dH, int dW)
{
  const long oH = (H - kH) / dH + 1, oW = (W - kW) / dW + 1;
  long p, y, x, i;
  int ky, kx;
  for (i = 0; i < planes * H * W; i++) gradIn[i] = 0;
  for (p = 0; p < planes; p++)
    for (y = 0; y < oH; y++)
      for (x = 0; x < oW; x++) {
        float *q = gradIn + (p * H + y * dH) * W + x * dW;
        const float z = gradOut[(p * oH + y) * oW + x];
        for (ky = 0; ky < kH; ky++, q += W)
          for (kx = 0; kx < kW; kx++) q[kx] += z;
      }
}
