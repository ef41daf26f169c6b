// BF16 variant of the two-SM tcgen05 engine (opt-in math mode 2): the same pipeline as mm_tc2.cuh over
// single planes of BF16 values, one tcgen05.mma.kind::f16 per 16 k instead of three kind::tf32 per 8 k.
//
// Operands are the descriptions of mm_problem.cuh with every offset counted in 4-byte units (pairs of BF16
// values), so a tile row is still 128 bytes: 64 k of a K-major operand, or 64 channels of one pixel of an
// MN-major one (whose k tile holds 64 pixels and uses the plain 128-byte swizzle).  Products are exact in
// FP32 and the tolerance of this mode is BF16's, so four k tiles (16 MMAs) chain in one TMEM accumulator
// before the drain warps fold it into their FP32 registers.
#ifndef THC_MM_TC2H_CUH
#define THC_MM_TC2H_CUH

#include "mm_tc2.cuh"

namespace thc {
namespace mm {

constexpr int T2H_CHAIN = 4;

template <int BN2> struct Tc2hCfg {
  static constexpr int BH = BN2 / 2;
  static constexpr int A_BYTES = TC_BM * 128;
  static constexpr int B_BYTES = BH * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 192 * 1024 / STAGE_BYTES > 8 ? 8 : 192 * 1024 / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN2 > 256 ? 512 : 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 512 + 1024;
};

// BF16 operand tiles: K-major as for TF32; MN-major [64-channel block][64 pixels][128 B], plain 128-byte
// swizzle, blocks 8192 B apart (leading offset), 8-pixel groups 1024 B apart (stride offset).
template <bool MN_MAJOR>
__device__ __forceinline__ uint64_t umma_desc_half(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(MN_MAJOR ? (8192 >> 4) : 1) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}
// bytes between the operand slices of consecutive MMAs (16 k each)
template <bool MN_MAJOR> __host__ __device__ constexpr int umma_kstep_bytes_half() { return MN_MAJOR ? 2048 : 32; }
// kind::f16 with BF16 operands, FP32 accumulate, M = 256 over the CTA pair
__host__ __device__ constexpr uint32_t umma2_idesc_bf16(int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <class P, int BN2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T2_THREADS, 1) tc2h_kernel(const __grid_constant__ P p, const StallCtl ctl) {
  typedef Tc2hCfg<BN2> Cfg;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BH = Cfg::BH;
  constexpr bool A_MN = P::OpA::MN_MAJOR, B_MN = P::OpB::MN_MAJOR;
  static_assert(A_MN == B_MN, "the k index is pixels for MN-major operands and 4-byte units otherwise: no mixing");
  constexpr int KT = A_MN ? 64 : 32;            // k per tile in the operands' own k index
  // rows of the fills in the operands' own row index (MN-major rows are 4-byte units = channel pairs)
  constexpr int A_ROWS = A_MN ? TC_BM / 2 : TC_BM, B_ROWS = B_MN ? BH / 2 : BH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t *aux = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(aux);   // full[S], empty[S], acc_full[2], acc_empty[2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile WaitCtl *abort_flag = reinterpret_cast<volatile WaitCtl *>(tmem_slot + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  const long m0 = (long)(blockIdx.x >> 1) * 256 + (long)rank * TC_BM;
  const long n_tile0 = (long)blockIdx.y * BN2;
  const long n0 = n_tile0 + (long)rank * BH;
  long k_begin = 0, k_end = p.K;
  if (p.ws) {
    k_begin = (long)blockIdx.z * p.k_per_split;
    k_end = k_begin + p.k_per_split;
    if (k_end > p.K) k_end = p.K;
  }
  const int num_k_tiles = (int)((k_end - k_begin + KT - 1) / KT);
  const int num_groups = (num_k_tiles + T2H_CHAIN - 1) / T2H_CHAIN;

  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const uint32_t bar_acc_full = smem_u32(bars + 2 * STAGES), bar_acc_empty = smem_u32(bars + 2 * STAGES + 2);
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(bar_full + 8 * s, 2 * T2_PRODUCERS / 32);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 2 * T2_DRAIN_WARPS);
    }
    wait_ctl_init(abort_flag, ctl, mapa_shared(smem_u32(const_cast<int *>(&abort_flag->abort)), rank ^ 1u));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == T2_MMA_WARP) tmem_alloc2(smem_u32(tmem_slot), Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = abort_flag->abort == 0;   // set on entry: an earlier kernel of this stream stalled, do no work

  if (!ok) {
    if (tid == 0) wait_ctl_give_up(abort_flag, kWaitEntry);   // the peer may have read the flag before it was set: tell it
  } else if (warp < T2_MMA_WARP) {
    // ------------------------------------------------------------ producers
    setmaxnreg_dec<72>();
    TileFill2<typename P::OpA, A_ROWS, true> fa;
    TileFill2<typename P::OpB, B_ROWS, true> fb;
    fa.init(p.a, A_MN ? m0 / 2 : m0, tid);
    fb.init(p.b, B_MN ? n0 / 2 : n0, tid);
    const uint32_t full_leader = mapa_shared(bar_full, 0);
    auto issue_tile = [&](int t) {
      if (t < num_k_tiles) {
        const long k0 = k_begin + (long)t * KT;
        const uint32_t stage = smem_u32(smem + (t % STAGES) * Cfg::STAGE_BYTES);
        fa.issue(p.a, k0, k_end, tid, stage);
        fb.issue(p.b, k0, k_end, tid, stage + Cfg::A_BYTES);
      }
      cp_async_commit();
    };
    constexpr int LA = STAGES - 1;
    for (int t = 0; t < LA; t++) issue_tile(t);
    for (int it = 0; it < num_k_tiles; it++) {
      cp_async_wait<LA - 1>();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(full_leader + 8 * (it % STAGES));
      const int t = it + LA;
      if (t < num_k_tiles && t >= STAGES) {
        const uint32_t phase = (uint32_t)(t / STAGES) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * (t % STAGES), phase ^ 1u, abort_flag));
        if (!ok) break;
      }
      issue_tile(t);
    }
    cp_async_wait<0>();
  } else if (warp < T2_DRAIN_WARP0) {
    // ------------------------------------------------------------ MMA issuer (one thread of the leader CTA)
    setmaxnreg_dec<40>();
    if (warp == T2_MMA_WARP && lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma2_idesc_bf16(BN2, A_MN, B_MN);
      for (int it = 0; it < num_k_tiles; it++) {
        const int s = it % STAGES, grp = it / T2H_CHAIN, buf = grp & 1;
        const bool first = it % T2H_CHAIN == 0, last = it % T2H_CHAIN == T2H_CHAIN - 1 || it == num_k_tiles - 1;
        const uint32_t phase = (uint32_t)(it / STAGES) & 1u, acc_phase = (uint32_t)(grp >> 1) & 1u;
        if (first) ok = mbar_wait_spin(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag);
        ok = ok && mbar_wait_spin(bar_full + 8 * s, phase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t a_d = umma_desc_half<A_MN>(st), b_d = umma_desc_half<B_MN>(st + Cfg::A_BYTES);
        const uint32_t d = tmem_base + (uint32_t)(buf * BN2);
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {   // 16 k per MMA
          const uint64_t adv_a = (uint64_t)((kk * umma_kstep_bytes_half<A_MN>()) >> 4);
          const uint64_t adv_b = (uint64_t)((kk * umma_kstep_bytes_half<B_MN>()) >> 4);
          umma2_bf16(d, a_d + adv_a, b_d + adv_b, idesc, (kk || !first) ? 1u : 0u);
        }
        umma2_commit_both(bar_empty + 8 * s);
        if (last) umma2_commit_both(bar_acc_full + 8 * buf);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ drain + epilogue warps
    setmaxnreg_inc<192>();   // 128 x 72 + 128 x 40 + 256 x 192 <= the 512 x 128 registers the CTA was launched with
    const int q = warp & 3;
    const int h = (warp - T2_DRAIN_WARP0) >> 2;
    constexpr int NCOL = BN2 / 2;
    const uint32_t acc_empty_leader = mapa_shared(bar_acc_empty, 0);
    float acc[NCOL];
#pragma unroll
    for (int j = 0; j < NCOL; j++) acc[j] = 0.f;
    for (int it = 0; it < num_groups; it++) {
      const int buf = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      ok = mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN2 + h * NCOL);
#pragma unroll
      for (int c0 = 0; c0 < NCOL; c0 += 32) {
        uint32_t v[32];
        tmem_ld32_nowait(t0 + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j++) acc[c0 + j] += __uint_as_float(v[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8 * buf);
    }
    if (ok) {
      const long m = m0 + q * 32 + lane;
      tc2_store_rows<P, NCOL>(p, acc, m, n_tile0 + h * NCOL);
    }
  }
  if (abort_flag->abort && tid == 0) stall_raise(ctl, abort_flag->abort);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == T2_MMA_WARP) tmem_dealloc2(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace mm
}  // namespace thc

#endif
