// Elementwise kernel family shared by copy, tensor math and Threshold.
//
// One functor, three data paths, picked on the host from the operands' strides:
//   contiguous : float4 grid-stride streaming (the HBM-bound fast path)
//   tiled 2-D  : operands whose unit-stride dimension differs from the output's (transposed views)
//                are staged through 32x33 shared-memory tiles so that every global access stays
//                coalesced; counts the same algorithmic bytes as the contiguous case
//   strided    : anything else, collapsed dims + div/mod indexing (correct, not fast)
// This replaces the reference pattern "newContiguous every operand, run, freeCopyTo the result"
// (gputorch/lib/THC/THCTensorMath.cpp:67-163) and its per-element div/mod copy kernel
// (gputorch/lib/THC/THCTensorCopy.cpp:170-218).
#ifndef THC_APPLY_CUH
#define THC_APPLY_CUH

#include "thc_internal.h"

namespace thc {

template <int NIN>
struct Operands {
  float *out;
  const float *in[NIN > 0 ? NIN : 1];
};

template <typename Op, int NIN>
__global__ void __launch_bounds__(256) apply_contig_kernel(Operands<NIN> p, long n, bool vec, Op op) {
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long nthreads = (long)gridDim.x * blockDim.x;
  long done = 0;
  if (vec) {
    const long nvec = n >> 2;
    long i = tid;
    // U independent 16-byte loads per operand in flight per thread before the first store: one load per thread left
    // the one-input operations at 0.86 of the copy rate the two-input ones reach with their two
    constexpr int U = NIN <= 1 ? 4 : 2;
    for (; i + (U - 1) * nthreads < nvec; i += U * nthreads) {
      float4 v[U][NIN > 0 ? NIN : 1];
#pragma unroll
      for (int u = 0; u < U; u++)
#pragma unroll
        for (int k = 0; k < NIN; k++) v[u][k] = reinterpret_cast<const float4 *>(p.in[k])[i + u * nthreads];
#pragma unroll
      for (int u = 0; u < U; u++) {
        float a[NIN > 0 ? NIN : 1];
        float4 r;
#pragma unroll
        for (int k = 0; k < NIN; k++) a[k] = v[u][k].x;
        r.x = op(a);
#pragma unroll
        for (int k = 0; k < NIN; k++) a[k] = v[u][k].y;
        r.y = op(a);
#pragma unroll
        for (int k = 0; k < NIN; k++) a[k] = v[u][k].z;
        r.z = op(a);
#pragma unroll
        for (int k = 0; k < NIN; k++) a[k] = v[u][k].w;
        r.w = op(a);
        reinterpret_cast<float4 *>(p.out)[i + u * nthreads] = r;
      }
    }
    for (; i < nvec; i += nthreads) {
      float4 v[NIN > 0 ? NIN : 1];
#pragma unroll
      for (int k = 0; k < NIN; k++) v[k] = reinterpret_cast<const float4 *>(p.in[k])[i];
      float a[NIN > 0 ? NIN : 1];
      float4 r;
#pragma unroll
      for (int k = 0; k < NIN; k++) a[k] = v[k].x;
      r.x = op(a);
#pragma unroll
      for (int k = 0; k < NIN; k++) a[k] = v[k].y;
      r.y = op(a);
#pragma unroll
      for (int k = 0; k < NIN; k++) a[k] = v[k].z;
      r.z = op(a);
#pragma unroll
      for (int k = 0; k < NIN; k++) a[k] = v[k].w;
      r.w = op(a);
      reinterpret_cast<float4 *>(p.out)[i] = r;
    }
    done = nvec << 2;
  }
  for (long i = done + tid; i < n; i += nthreads) {
    float a[NIN > 0 ? NIN : 1];
#pragma unroll
    for (int k = 0; k < NIN; k++) a[k] = p.in[k][i];
    p.out[i] = op(a);
  }
}

struct StridedArgs {
  int nd;
  long size[kMaxDims];
  long stride[3][kMaxDims];
};

template <typename Op, int NIN>
__global__ void __launch_bounds__(256) apply_strided_kernel(Operands<NIN> p, StridedArgs s, long n, Op op) {
  const long nthreads = (long)gridDim.x * blockDim.x;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nthreads) {
    long rem = i, off[NIN + 1];
#pragma unroll
    for (int k = 0; k <= NIN; k++) off[k] = 0;
    for (int d = s.nd - 1; d >= 0; d--) {
      const long q = rem / s.size[d], r = rem - q * s.size[d];
#pragma unroll
      for (int k = 0; k <= NIN; k++) off[k] += r * s.stride[k][d];
      rem = q;
    }
    float a[NIN > 0 ? NIN : 1];
#pragma unroll
    for (int k = 0; k < NIN; k++) a[k] = p.in[k][off[k + 1]];
    p.out[off[0]] = op(a);
  }
}

// 2-D index space (n0, n1); the output has unit stride along dim 1.  Inputs flagged in `via_smem`
// have unit stride along dim 0 and are transposed through shared memory.  kTile2d x kTile2d tiles (32 or 64, chosen
// by the caller): every global access of a warp is one contiguous 128-byte segment and a thread has
// kTile2d * kTile2d / 256 independent loads per operand in flight.
template <typename Op, int NIN, int kTile2d>
__global__ void __launch_bounds__(256) apply_tiled2d_kernel(Operands<NIN> p, long n0, long n1,
                                                            long os0, long is0_0, long is1_0,
                                                            long is0_1, long is1_1, unsigned via_smem,
                                                            long tiles1, long ntiles, Op op) {
  extern __shared__ float tile2d_smem[];   // [NIN][kTile2d][kTile2d + 1]
  const long is0[2] = {is0_0, is0_1}, is1[2] = {is1_0, is1_1};
  constexpr int TY = 256 / kTile2d;
  const int tx = threadIdx.x % kTile2d, ty = threadIdx.x / kTile2d;
  for (long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long b0 = (t / tiles1) * kTile2d, b1 = (t % tiles1) * kTile2d;
#pragma unroll
    for (int k = 0; k < NIN; k++) {
      if (via_smem & (1u << k)) {
        float *tile = tile2d_smem + k * kTile2d * (kTile2d + 1);
        const long i0 = b0 + tx;
#pragma unroll
        for (int j = ty; j < kTile2d; j += TY) {
          const long i1 = b1 + j;
          if (i0 < n0 && i1 < n1) tile[j * (kTile2d + 1) + tx] = p.in[k][i0 * is0[k] + i1 * is1[k]];
        }
      }
    }
    // operands that need no transposition are fetched into registers BEFORE the barrier, so that their loads fly
    // together with the staged ones instead of starting after them
    const long i1 = b1 + tx;
    float direct[NIN > 1 ? NIN : 1][NIN > 1 ? kTile2d / TY : 1];   // a single input is always the staged one
#pragma unroll
    for (int k = 0; k < (NIN > 1 ? NIN : 0); k++) {
      if (!(via_smem & (1u << k))) {
#pragma unroll
        for (int jj = 0; jj < kTile2d / TY; jj++) {
          const long i0 = b0 + ty + jj * TY;
          direct[k][jj] = (i0 < n0 && i1 < n1) ? p.in[k][i0 * is0[k] + i1 * is1[k]] : 0.f;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int jj = 0; jj < kTile2d / TY; jj++) {
      const int j = ty + jj * TY;
      const long i0 = b0 + j;
      if (i0 < n0 && i1 < n1) {
        float a[NIN > 0 ? NIN : 1];
#pragma unroll
        for (int k = 0; k < NIN; k++)
          a[k] = (NIN == 1 || (via_smem & (1u << k))) ? tile2d_smem[k * kTile2d * (kTile2d + 1) + tx * (kTile2d + 1) + j]
                                                      : direct[NIN > 1 ? k : 0][NIN > 1 ? jj : 0];
        p.out[i0 * os0 + i1] = op(a);
      }
    }
    __syncthreads();
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// out = op(in...) over tensors of equal shape (already resized by the caller); out may alias an input.
template <int NIN, typename Op>
void apply(THGPUTensor *out, const THGPUTensor *in0, const THGPUTensor *in1, Op op, const char *name) {
  const long n = nelem(out);
  if (n == 0) return;
  const THGPUTensor *ops[3] = {out, in0, in1};
  Operands<NIN> p;
  p.out = data_ptr(out);
  if (NIN > 0) p.in[0] = data_ptr(in0);
  if (NIN > 1) p.in[1] = data_ptr(in1);
  const int max_blocks = ctx().sm_count * 8;
  bool all_contig = is_contiguous(out);
  for (int k = 0; k < NIN; k++) all_contig = all_contig && is_contiguous(ops[k + 1]);
  if (all_contig) {
    bool vec = aligned16(p.out);
    for (int k = 0; k < NIN; k++) vec = vec && aligned16(p.in[k]);
    long work = vec ? (n + 3) / 4 : n;
    int blocks = (int)((work + 255) / 256);
    if (blocks > max_blocks) blocks = max_blocks;
    apply_contig_kernel<Op, NIN><<<blocks, 256, 0, stream()>>>(p, n, vec, op);
    check_launch(name);
    return;
  }
  Strided s;
  THC_CHECK(collapse(NIN + 1, ops, s), "%s: too many non-collapsible dimensions", name);
  if (s.nd == 2 && NIN > 0) {
    // normalise so that the output's unit-stride dim is dim 1
    int a = 0, b = 1;
    if (s.stride[0][1] != 1 && s.stride[0][0] == 1) { a = 1; b = 0; }
    if (s.stride[0][b] == 1) {
      unsigned via = 0;
      for (int k = 0; k < NIN; k++)
        if (s.stride[k + 1][a] == 1 && s.stride[k + 1][b] != 1) via |= 1u << k;
      if (via) {
        const long n0 = s.size[a], n1 = s.size[b];
        constexpr int kTile2d = 64;   // 32 x 32 tiles measured the same for one input (0.63 / 0.64 of the HBM rate) and worse for two
        const long tiles0 = (n0 + kTile2d - 1) / kTile2d, tiles1 = (n1 + kTile2d - 1) / kTile2d, ntiles = tiles0 * tiles1;
        int blocks = (int)(ntiles < max_blocks ? ntiles : max_blocks);
        const size_t smem = (NIN > 0 ? NIN : 1) * kTile2d * (kTile2d + 1) * sizeof(float);
        apply_tiled2d_kernel<Op, NIN, kTile2d><<<blocks, 256, smem, stream()>>>(
            p, n0, n1, s.stride[0][a], s.stride[1][a], s.stride[1][b], NIN > 1 ? s.stride[2][a] : 0,
            NIN > 1 ? s.stride[2][b] : 0, via, tiles1, ntiles, op);
        check_launch(name);
        return;
      }
    }
  }
  StridedArgs sa;
  sa.nd = s.nd;
  for (int d = 0; d < kMaxDims; d++) {
    sa.size[d] = d < s.nd ? s.size[d] : 1;
    for (int k = 0; k < 3; k++) sa.stride[k][d] = d < s.nd ? s.stride[k][d] : 0;
  }
  int blocks = (int)((n + 255) / 256);
  if (blocks > max_blocks) blocks = max_blocks;
  apply_strided_kernel<Op, NIN><<<blocks, 256, 0, stream()>>>(p, sa, n, op);
  check_launch(name);
}

}  // namespace thc

#endif
