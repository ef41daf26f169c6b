// Host-side dispatch of an mm::Problem onto an engine: picks the tile width, decides split-K,
// owns the split-K workspace, launches, and folds the partials.
#ifndef THC_MM_LAUNCH_CUH
#define THC_MM_LAUNCH_CUH

#include <climits>

#include "mm_simt.cuh"
#include "mm_tc.cuh"

namespace thc {
namespace mm {

int *tc_error_flag();        // device-visible int the tensor-core kernels raise on a timed-out wait
void tc_check_error_flag();  // throws if a previous kernel raised it (call after a stream sync)

// hi / lo planes of a strided matrix for the tensor-core engine (stream-ordered scratch; free with
// release()).  Element (r, k) of the source lives at src[r*rs + k*ks].
struct SplitPlanes {
  float *hi = nullptr, *lo = nullptr;
  long ld = 0;
  void release() { dev_free(hi); hi = lo = nullptr; }  // one allocation holds both planes
};
static SplitPlanes make_split_planes(const float *src, long rs, long ks, long rows, long K) {
  SplitPlanes sp;
  sp.ld = (K + 31) / 32 * 32;
  sp.hi = (float *)dev_alloc(sizeof(float) * 2 * rows * sp.ld);
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
  tc_kernel<P, BN><<<grid, TC_THREADS, Cfg::SMEM_BYTES, stream()>>>(p, tc_error_flag());
  check_launch("tc_kernel");
}

// How many k slices to cut a product into so that tiles * slices fills whole waves of SMs.  One slice
// unless that raises the fill of the last wave noticeably; every slice keeps at least 16 k tiles.
static long choose_splits(long tiles, long ktiles, int sms) {
  if (tiles >= 4l * sms || ktiles < 32) return 1;
  auto fill = [&](long s) {
    const long ctas = tiles * s, waves = (ctas + sms - 1) / sms;
    return (double)ctas / (double)(waves * sms);
  };
  long best = 1, max_s = ktiles / 16;
  if (max_s > 64) max_s = 64;
  double best_fill = fill(1);
  for (long s = 2; s <= max_s; s++) {
    const double f = fill(s);
    if (f > best_fill + 0.04) { best = s; best_fill = f; }
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
  THC_CHECK(mode == 0 || (mode == 1 && !TC_ONLY), "math mode %d is not available in this build (0 = fp32x3, 1 = simt)", mode);
  const int sms = ctx().sm_count;
  const bool tc = mode == 0;
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
  if (splits > 1) p.ws = (float *)dev_alloc(sizeof(float) * splits * p.M * p.N);
  dim3 grid((unsigned)gm, (unsigned)gn, (unsigned)splits);
  if (tc) {
    if (bn == 128) launch_tc<P, 128>(p, grid);
    else launch_tc<P, 64>(p, grid);
  } else if constexpr (!TC_ONLY) {
    simt_kernel<P><<<grid, 256, 0, stream()>>>(p);
    check_launch("simt_kernel");
  }
  if (splits > 1) {
    const long total = p.M * p.N;
    splitk_finish_kernel<<<ceil_div(total, 256), 256, 0, stream()>>>(p.ws, (int)splits, p.M, p.N, p.epi);
    check_launch("splitk_finish");
    dev_free(p.ws);
  }
}
template <class P> static void launch(const P &p, bool allow_split = true) { launch_impl<P, false>(p, allow_split); }
template <class P> static void launch_tc_only(const P &p, bool allow_split = true) { launch_impl<P, true>(p, allow_split); }

// Channels-last hi / lo planes of an NCHW activation tensor (stream-ordered scratch; one allocation).
struct ActPlanes {
  float *hi = nullptr, *lo = nullptr;
  void release() { dev_free(hi); hi = lo = nullptr; }
};
static ActPlanes make_act_planes(const float *src, long N, long C, long HW) {
  ActPlanes ap;
  const long total = N * C * HW;
  ap.hi = (float *)dev_alloc(sizeof(float) * 2 * total);
  ap.lo = ap.hi + total;
  long blocks = N * ((HW + 31) / 32) * (C / 32);
  const long cap = (long)ctx().sm_count * 16;
  if (blocks > cap) blocks = cap;
  nchw_to_planes_kernel<<<(unsigned)blocks, 256, 0, stream()>>>(src, N, C, HW, ap.hi, ap.lo);
  check_launch("nchw_to_planes");
  return ap;
}

}  // namespace mm
}  // namespace thc

#endif
