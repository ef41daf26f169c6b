// Two-SM tcgen05 engine (cta_group::2) for products whose operands are ready-made TF32 hi / lo planes.
//
// A cluster of two CTAs on neighbouring SMs computes one 256 x BN2 tile of D (BN2 = 64, 128, 192 or 256):
// CTA r of the pair stages rows [128 r, 128 r + 128) of the A tile and rows [BN2/2 r, BN2/2 (r+1)) of the
// B tile in its own shared memory; the MMAs, issued by one thread of CTA 0, read both CTAs' shared
// memory and leave rows [128 r, +128) of the result in CTA r's tensor memory.  Compared with the
// one-SM engine (mm_tc.cuh) every byte fetched from L2 feeds twice the arithmetic and every barrier
// round trip covers twice the MMA time, which is what that engine is short of.
//
// Roles (512 threads per CTA):
//   warps 0-3   producers: 16-byte cp.async of both planes of both operands straight into the swizzled
//               tiles (K-major or MN-major, as in mm_tc.cuh), two k tiles ahead; they arrive on CTA 0's
//               `full` barrier (remote arrive from CTA 1).
//   warp 4      (CTA 0 only) one thread issues the 12 tcgen05.mma.cta_group::2.kind::tf32 of a k tile
//               (Alo*Bhi, Ahi*Blo, Ahi*Bhi over four 8-k steps) into one of two TMEM accumulator buffers,
//               then commits to the `empty` and `acc_full` barriers of BOTH CTAs.  Warps 5-7 only give
//               their registers away.
//   warps 8-15  drain: tcgen05.ld every finished 32-k partial tile and add it into FP32 registers with
//               round-to-nearest (the tensor core's own accumulation truncates, so chains stay 12 MMAs
//               long), arrive on CTA 0's `acc_empty`; finally the epilogue (TMEM lane = row m).
// Registers are rebalanced with setmaxnreg: the drain warps hold BN2/2 accumulators per thread.
//
// Every mbarrier wait is bounded; on expiry the CTA tells its peer, raises the stall flags (see StallCtl in
// mm_tc.cuh), skips its stores, and still joins the final cluster barrier, so that neither CTA of a pair can
// leave while the other may still touch its shared or tensor memory.  All operand tiles of this engine are
// copied by threads; TMA serves the raw-operand engine (mm_tc2r.cuh) only.
#ifndef THC_MM_TC2_CUH
#define THC_MM_TC2_CUH

#include "mm_tc.cuh"

namespace thc {
namespace mm {

constexpr int T2_PRODUCERS = 128;
constexpr int T2_MMA_WARP = 4;
constexpr int T2_DRAIN_WARP0 = 8;
constexpr int T2_DRAIN_WARPS = 8;
constexpr int T2_THREADS = 512;
constexpr int T2_STAGES = 3;
constexpr int T2_CHAIN = 1;   // k tiles accumulated in tensor memory before the drain warps fold them into FP32 registers

template <int BN2> struct Tc2Cfg {
  static constexpr int BH = BN2 / 2;                 // B rows staged per CTA
  static constexpr int A_BYTES = TC_BM * 128;        // one precision plane of this CTA's A rows
  static constexpr int B_BYTES = BH * 128;
  static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);
  static constexpr int TMEM_COLS = 2 * BN2 > 256 ? 512 : 256;   // two accumulator buffers, power of two
  static constexpr int SMEM_BYTES = T2_STAGES * STAGE_BYTES + 256 + 1024;
};

// ---------------------------------------------------------------- cluster / cta_group::2 PTX
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier of any CTA of the cluster (address from mapa_shared).  Default (CTA-scope release)
// semantics on purpose: a cluster-scope release costs the arriving thread one to two thousand cycles here,
// and nothing these arrivals hand over travels through the generic proxy between the CTAs: shared-memory
// tiles are published to the async proxy by the producer's own fence.proxy.async, tensor memory by
// tcgen05.fence / tcgen05.wait::ld.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded busy wait for the single MMA-issuing thread: polling without suspension answers within a few
// cycles of the arrival, which is what keeps the tensor pipe fed; one spinning thread costs nothing.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, volatile WaitCtl *w, int code = kWaitOther) {
  long long t0 = 0;
  for (int polls = 0;; polls++) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((polls & 255) == 255) {
      if (w->abort) return false;
      if (t0 == 0) t0 = clock64();
      else if (clock64() - t0 > w->limit) { wait_ctl_give_up(w, code); return false; }
    }
  }
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// completion of all MMAs issued so far -> one arrival on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// kind::tf32, FP32 accumulate, M = 256 over the CTA pair
__host__ __device__ constexpr uint32_t umma2_idesc_tf32(int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// im2col TMA load of 32 channels of 128 consecutive windows (tensor {C, W, H, images}) starting at window
// corner (x, y) of image `img`, at tap offset (j, i); completion as above.
__device__ __forceinline__ void tma_load_windows(uint32_t dst, const void *tmap, int c, int x, int y, int img, int j, int i,
                                                 uint32_t mbar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
      ::"r"(dst), "l"((unsigned long long)tmap), "r"(mbar), "r"(c), "r"(x), "r"(y), "r"(img), "h"((unsigned short)j),
        "h"((unsigned short)i)
      : "memory");
}
template <int N> __device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t *v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One producer thread's share of an operand tile (ROWS rows of this CTA x one k tile) with T2_PRODUCERS threads.
// Row state is kept compact (offset in 16-byte units + packed box coordinates) so that the producers
// run in a small register budget.  All offsets are in 4-byte units: FP32 planes count floats, BF16 planes
// (HALF) count pairs of values, so one row of a tile is 128 bytes = 32 units in both.
//   K-major : thread = (16-byte chunk tid % 8, rows tid / 8 + PASS c)
//   MN-major: thread = (16-byte column tid % 8 of every 32-unit block, pixels tid / 8 + PASS ps of the k tile);
//             the k tile holds KPIX pixels: 32 for TF32 (128-byte swizzle with 32-byte atoms), 64 for BF16
//             (plain 128-byte swizzle), the layouts tcgen05 reads MN-major operands of those widths in.
// HALF tiles have one plane; FP32 tiles a hi and a lo plane, the lo tile following the hi tile.
template <class Op, int ROWS, bool HALF = false>
struct TileFill2 {
  static_assert(Op::PRESPLIT, "the two-SM engine only reads ready-made planes");
  static constexpr int PASS = T2_PRODUCERS / 8;       // rows (K-major) or k (MN-major) covered by one pass of the threads
  static_assert(ROWS % 32 == 0 && 32 % PASS == 0, "thread mapping");
  static constexpr int KPIX = HALF ? 64 : 32;
  static constexpr int NR = Op::MN_MAJOR ? ROWS / 32 : ROWS / PASS;
  int off16[NR];   // offset in units of 16 bytes
  int yx[NR];      // (y + 16384) << 16 | (x + 16384); 0 = invalid row
  static __device__ __forceinline__ int pack(const Info &r) {
    if (r.y <= -16384) return 0;
    return ((r.y + 16384) << 16) | ((r.x + 16384) & 0xffff);
  }
  static __device__ __forceinline__ Info unpack(int o16, int p) {
    Info r;
    r.off = (long)o16 * 4;
    r.y = (int)((unsigned)p >> 16) - 16384;
    r.x = (int)((unsigned)p & 0xffffu) - 16384;
    return r;
  }
  __device__ __forceinline__ void init(const Op &op, long row0, int tid) {
    if constexpr (Op::MN_MAJOR) {
#pragma unroll
      for (int a = 0; a < NR; a++) {
        const long r0 = row0 + 32 * a + (tid & 7) * 4;
        Info r = op.rowblock(r0);
        if (r0 >= op.rows.count) r.y = kInvalid;
        off16[a] = (int)(r.off >> 2);
        yx[a] = pack(r);
      }
    } else {
#pragma unroll
      for (int c = 0; c < NR; c++) {
        const Info r = op.rows(row0 + (tid >> 3) + PASS * c);
        off16[c] = (int)(r.off >> 2);   // arithmetic shift: window corners may sit before the plane
        yx[c] = pack(r);
      }
    }
  }
  __device__ __forceinline__ void issue(const Op &op, long k0, long k_end, int tid, uint32_t hi_tile) const {
    if constexpr (Op::MN_MAJOR) {
      const int q0 = tid & 7;
#pragma unroll
      for (int ps = 0; ps < KPIX / PASS; ps++) {
        const int kk = (tid >> 3) + PASS * ps;
        Info px = op.ks(k0 + kk);
        if (k0 + kk >= k_end) px.y = kInvalid;
#pragma unroll
        for (int a = 0; a < NR; a++) {
          const Info rb = unpack(off16[a], yx[a]);
          const bool okay = op.valid(px, rb);
          const long o = okay ? px.off + rb.off : 0;
          const uint32_t sw = HALF ? (uint32_t)((q0 ^ (kk & 7)) << 4)
                                   : (uint32_t)((((q0 >> 1) ^ (kk & 3)) << 5) | ((q0 & 1) << 4));
          const uint32_t dst = hi_tile + (uint32_t)(a * KPIX * 128 + kk * 128) + sw;
          cp_async16(dst, op.base + o, okay);
          if constexpr (!HALF) cp_async16(dst + ROWS * 128, op.lo + o, okay);
        }
      }
    } else {
      const int chunk = tid & 7;
      const Info kt = op.ktile(k0, chunk);   // this thread's 16-byte chunk of the k tile
#pragma unroll
      for (int c = 0; c < NR; c++) {
        const int row = (tid >> 3) + PASS * c;
        const Info r = unpack(off16[c], yx[c]);
        const bool okay = op.valid(r, kt);
        const long o = okay ? r.off + kt.off : 0;
        const uint32_t dst = hi_tile + (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
        cp_async16(dst, op.base + o, okay);
        if constexpr (!HALF) cp_async16(dst + ROWS * 128, op.lo + o, okay);
      }
    }
  }
};

template <class P, int BN2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T2_THREADS, 1) tc2_kernel(const __grid_constant__ P p, const StallCtl ctl) {
  typedef Tc2Cfg<BN2> Cfg;
  constexpr int STAGES = T2_STAGES;
  constexpr int BH = Cfg::BH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t *aux = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(aux);   // full[S], empty[S], acc_full[2], acc_empty[2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile WaitCtl *abort_flag = reinterpret_cast<volatile WaitCtl *>(tmem_slot + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();              // 0 = leader (issues the MMAs)
  const long m0 = (long)(blockIdx.x >> 1) * 256 + (long)rank * TC_BM;   // this CTA's 128 rows of A and D
  const long n_tile0 = (long)blockIdx.y * BN2;
  const long n0 = n_tile0 + (long)rank * BH;            // this CTA's rows of B
  long k_begin = 0, k_end = p.K;
  if (p.ws) {
    k_begin = (long)blockIdx.z * p.k_per_split;
    k_end = k_begin + p.k_per_split;
    if (k_end > p.K) k_end = p.K;
  }
  const int num_k_tiles = (int)((k_end - k_begin + TC_BK - 1) / TC_BK);

  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const uint32_t bar_acc_full = smem_u32(bars + 2 * STAGES), bar_acc_empty = smem_u32(bars + 2 * STAGES + 2);
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(bar_full + 8 * s, 2 * T2_PRODUCERS / 32);   // both CTAs' producer warps (used in CTA 0)
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 2 * T2_DRAIN_WARPS);  // drain warps of both CTAs (used in CTA 0)
    }
    wait_ctl_init(abort_flag, ctl, mapa_shared(smem_u32(const_cast<int *>(&abort_flag->abort)), rank ^ 1u));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == T2_MMA_WARP) tmem_alloc2(smem_u32(tmem_slot), Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anyone arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = abort_flag->abort == 0;   // set on entry: an earlier kernel of this stream stalled, do no work

  if (!ok) {
    if (tid == 0) wait_ctl_give_up(abort_flag, kWaitEntry);   // the peer may have read the flag before it was set: tell it
  } else if (warp < T2_MMA_WARP) {
    // ------------------------------------------------------------ producers
    setmaxnreg_dec<72>();
    TileFill2<typename P::OpA, TC_BM> fa;
    TileFill2<typename P::OpB, BH> fb;
    fa.init(p.a, m0, tid);
    fb.init(p.b, n0, tid);
    const uint32_t full_leader = mapa_shared(bar_full, 0);
    auto issue_tile = [&](int t) {
      if (t < num_k_tiles) {
        const long k0 = k_begin + (long)t * TC_BK;
        const uint32_t stage = smem_u32(smem + (t % STAGES) * Cfg::STAGE_BYTES);
        fa.issue(p.a, k0, k_end, tid, stage);
        fb.issue(p.b, k0, k_end, tid, stage + 2 * Cfg::A_BYTES);
      }
      cp_async_commit();
    };
    constexpr int LA = STAGES - 1;
    for (int t = 0; t < LA; t++) issue_tile(t);
    for (int it = 0; it < num_k_tiles; it++) {
      cp_async_wait<LA - 1>();     // tile `it` has landed in this CTA's stage
      fence_proxy_async_smem();    // visible to the tensor cores' async proxy
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
      constexpr bool A_MN = P::OpA::MN_MAJOR, B_MN = P::OpB::MN_MAJOR;
      constexpr uint32_t idesc = umma2_idesc_tf32(BN2, A_MN, B_MN);
      for (int it = 0; it < num_k_tiles; it++) {
        const int s = it % STAGES, grp = it / T2_CHAIN, buf = grp & 1;
        const bool first = it % T2_CHAIN == 0, last = it % T2_CHAIN == T2_CHAIN - 1 || it == num_k_tiles - 1;
        const uint32_t phase = (uint32_t)(it / STAGES) & 1u, acc_phase = (uint32_t)(grp >> 1) & 1u;
        if (first) ok = mbar_wait_spin(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag);
        ok = ok && mbar_wait_spin(bar_full + 8 * s, phase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t a_hi = umma_desc_sw128<A_MN>(st), a_lo = umma_desc_sw128<A_MN>(st + Cfg::A_BYTES);
        const uint64_t b_hi = umma_desc_sw128<B_MN>(st + 2 * Cfg::A_BYTES),
                       b_lo = umma_desc_sw128<B_MN>(st + 2 * Cfg::A_BYTES + Cfg::B_BYTES);
        const uint32_t d = tmem_base + (uint32_t)(buf * BN2);
#pragma unroll
        for (int kk = 0; kk < TC_BK / 8; kk++) {
          const uint64_t adv_a = (uint64_t)((kk * umma_kstep_bytes<A_MN>()) >> 4);
          const uint64_t adv_b = (uint64_t)((kk * umma_kstep_bytes<B_MN>()) >> 4);
          umma2_tf32(d, a_lo + adv_a, b_hi + adv_b, idesc, (kk || !first) ? 1u : 0u);
          umma2_tf32(d, a_hi + adv_a, b_lo + adv_b, idesc, 1u);
        }
#pragma unroll
        for (int kk = 0; kk < TC_BK / 8; kk++) {
          const uint64_t adv_a = (uint64_t)((kk * umma_kstep_bytes<A_MN>()) >> 4);
          const uint64_t adv_b = (uint64_t)((kk * umma_kstep_bytes<B_MN>()) >> 4);
          umma2_tf32(d, a_hi + adv_a, b_hi + adv_b, idesc, 1u);
        }
        umma2_commit_both(bar_empty + 8 * s);       // both CTAs may refill the stage once these MMAs have read it
        if (last) umma2_commit_both(bar_acc_full + 8 * buf);  // and both halves of the accumulator are complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ drain + epilogue warps
    setmaxnreg_inc<192>();   // 128 x 72 + 128 x 40 + 256 x 192 <= the 512 x 128 registers the CTA was launched with
    const int q = warp & 3;                           // TMEM lane quarter this warp may access
    const int h = (warp - T2_DRAIN_WARP0) >> 2;       // column half
    constexpr int NCOL = BN2 / 2;
    const uint32_t acc_empty_leader = mapa_shared(bar_acc_empty, 0);
    float acc[NCOL];
#pragma unroll
    for (int j = 0; j < NCOL; j++) acc[j] = 0.f;
    const int num_groups = (num_k_tiles + T2_CHAIN - 1) / T2_CHAIN;
    for (int it = 0; it < num_groups; it++) {
      const int buf = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      ok = mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective
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
    if (ok) tc2_store_rows<P, NCOL>(p, acc, m0 + q * 32 + lane, n_tile0 + h * NCOL);
  }
  if (abort_flag->abort && tid == 0) stall_raise(ctl, abort_flag->abort);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // nobody frees tensor memory or exits while the peer's MMAs / arrivals may still touch it
  if (warp == T2_MMA_WARP) tmem_dealloc2(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace mm
}  // namespace thc

#endif
