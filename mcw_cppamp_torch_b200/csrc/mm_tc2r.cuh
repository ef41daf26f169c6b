// Two-SM tcgen05 engine over plain FP32 operands: the 3xTF32 split happens inside the SM.
//
// The plane engine (mm_tc2.cuh) reads a TF32 hi and a TF32 lo copy of every operand element, eight bytes per
// element and k tile, and its main loop runs at the pace of L2 -> SM traffic, not of the tensor pipe.  Here
// TMA brings the FP32 values themselves (four bytes per element) straight into the `hi` slot of a stage, in
// the swizzled layout the MMAs read; kind::tf32 ignores the low 13 mantissa bits of its operands, so that
// slot already is the hi operand, hi = trunc_tf32(x).  Four splitter warps per CTA read the slot back and
// write lo = tf32(x - hi) into the `lo` slot at the same offsets (both slots share one layout, K-major or
// MN-major alike).  Products Alo*Bhi + Ahi*Blo + Ahi*Bhi and the drain into FP32 registers are those of
// the plane engine.
//
// Rings: R `hi` slots (loads in flight, tiles being split, tiles being multiplied) and L <= R `lo` slots
// (only tiles being split or multiplied), so that the load queue can be deep although shared memory holds
// no more than the plane engine's.
//
// Roles (512 threads per CTA, cluster of two CTAs as in mm_tc2.cuh):
//   warps 0-3   splitters, two groups of two warps taking alternate k tiles: wait for the tile's TMA bytes
//               (`raw_full`, CTA-local) and for its lo slot to be free, split, publish to the async proxy,
//               arrive on CTA 0's `full`.
//   warps 4, 6  (CTA 0) one MMA-issuing thread each, for the even and the odd k tiles.
//   warp 5      one thread per CTA issues the TMA loads of this CTA's A rows and B rows, R - 1 tiles ahead,
//               as soon as the MMAs that read a slot have completed (`empty`).
//   warps 8-15  drain + epilogue, as in the plane engine.
// The kernel is persistent: see tc2r_kernel.
// Every wait is bounded; on expiry the CTA tells its peer, raises the stall flags (StallCtl, mm_tc.cuh), skips
// its stores and still joins the final cluster barrier.
#ifndef THC_MM_TC2R_CUH
#define THC_MM_TC2R_CUH

#include "mm_tc2.cuh"

namespace thc {
namespace mm {

constexpr int T2R_TMA_WARP = 5;
constexpr int T2R_MMA_WARP2 = 6;

template <int BN2> struct Tc2rCfg {
  static constexpr int BH = BN2 / 2;
  static constexpr int A_BYTES = TC_BM * 128;
  static constexpr int B_BYTES = BH * 128;
  static constexpr int SLOT_BYTES = A_BYTES + B_BYTES;          // one precision of this CTA's A rows and B rows
  static constexpr int LO_SLOTS = 3;
  static constexpr int HI_MAX = (227 * 1024 - 1024 - 512) / SLOT_BYTES - LO_SLOTS;
  static constexpr int HI_SLOTS = HI_MAX > 6 ? 6 : HI_MAX;
  static constexpr int TMEM_COLS = 2 * BN2 > 256 ? 512 : 256;
  static constexpr int SMEM_BYTES = (HI_SLOTS + LO_SLOTS) * SLOT_BYTES + 512 + 1024;
  static_assert(HI_SLOTS >= LO_SLOTS, "ring sizes");
  static_assert(HI_SLOTS % 2 == 0 || HI_SLOTS <= LO_SLOTS + 2, "an odd hi ring must not be longer than the lo ring + 2 (parity waits of the two MMA threads)");
};

// lo = tf32(x - trunc_tf32(x)) of four values
__device__ __forceinline__ uint4 tf32_lo4(const uint4 &v) {
  uint4 l;
  l.x = to_tf32(__uint_as_float(v.x) - __uint_as_float(v.x & 0xffffe000u));
  l.y = to_tf32(__uint_as_float(v.y) - __uint_as_float(v.y & 0xffffe000u));
  l.z = to_tf32(__uint_as_float(v.z) - __uint_as_float(v.z & 0xffffe000u));
  l.w = to_tf32(__uint_as_float(v.w) - __uint_as_float(v.w & 0xffffe000u));
  return l;
}
// Volatile without a memory clobber: these keep their order among themselves and against the (volatile) barrier
// waits and fences around them, which is all the splitter needs, and leave the compiler free to keep values
// in registers across them.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w));
}

// Tiled TMA loads of one CTA's share of a plain matrix operand: K-major, one {32 k, ROWS} box; MN-major, one
// {32 rows, 32 k} box per 32-row block (4096 bytes each).  Completion in bytes on this CTA's `mbar`.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int x, int y, uint32_t mbar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"((unsigned long long)tmap), "r"(mbar), "r"(x), "r"(y)
      : "memory");
}
// One non-blocking poll of a barrier phase.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
template <int ROWS, bool MN>
__device__ __forceinline__ void tma_issue(const RawOperand<MN> &op, uint32_t dst, long row0, long k0, uint32_t mbar) {
  if constexpr (MN) {
#pragma unroll
    for (int a = 0; a < ROWS / 32; a++) tma_load_2d(dst + a * 4096, &op.tmap, (int)row0 + 32 * a, (int)k0, mbar);
  } else {
    tma_load_2d(dst, &op.tmap, (int)k0, (int)row0, mbar);
  }
}
// Convolution windows as rows (K-major): one im2col load of 32 channels of ROWS = 128 consecutive windows.
template <int ROWS>
__device__ __forceinline__ void tma_issue(const PlanesWindowOperand &op, uint32_t dst, long row0, long k0, uint32_t mbar) {
  static_assert(ROWS == TC_BM, "the window map loads 128 windows");
  int x, y, img, i, j, c0;
  op.tile_origin(row0, x, y, img);
  op.tile_tap(k0, i, j, c0);
  tma_load_windows(dst, &op.tmap, c0, x, y, img, j, i, mbar);
}
// Convolution windows as the reduction (MN-major): per 32-row block, 32 channels of 32 consecutive windows.
template <int ROWS>
__device__ __forceinline__ void tma_issue(const WindowRowsOperand &op, uint32_t dst, long row0, long k0, uint32_t mbar) {
  int x, y, img;
  op.pixel_origin(k0, x, y, img);
#pragma unroll
  for (int a = 0; a < ROWS / 32; a++) {
    int i, j, c0;
    op.row_tap(row0 + 32 * a, i, j, c0);
    tma_load_windows(dst + a * 4096, &op.tmap, c0, x, y, img, j, i, mbar);
  }
}

// ---- item hand-out ------------------------------------------------------------------------------------------
// The clusters of a launch take their work items from a counter in device memory, first come first served, so a
// cluster that starts late (its SMs were still busy with another stream's kernel: a collective, a parameter
// update) simply takes fewer items instead of leaving its fixed share to run alone at the end.  One thread of the
// leader CTA fetches the next item number when the leader's TMA thread, the role that runs furthest ahead, starts on
// the current one (`go` barrier): one item of look-ahead hides the counter's round trip, and a cluster never holds
// claims on work it is not about to do.  The numbers go into a ring of T2R_SCHED slots that exists in both CTAs;
// every role of both CTAs reads the ring in the same order.  Slot protocol: `full` (one per CTA, count 1) completes
// when the number is there; `empty` (leader CTA only) collects one arrival per reading role of either CTA.  The
// peer's copy travels as st.async, whose completion is counted in bytes on the peer's `full` barrier: the peer
// sees the number when it sees the phase.
constexpr int T2R_SCHED = 8;
constexpr int T2R_SCHED_WARP = 7;
constexpr uint32_t T2R_NO_ITEM = 0xffffffffu;
constexpr int T2R_ITEM_WAIT_SHIFT = 6;   // item-level waits may take 64 k-tile limits (see mbar_wait)
// readers per slot: TMA thread, 4 splitter warps, 8 drain warps in each CTA, the two MMA threads in the leader
constexpr int T2R_SCHED_READERS = 2 * (1 + 4 + T2_DRAIN_WARPS) + 2;

__device__ __forceinline__ void mbar_arrive_local(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void sched_publish_peer(uint32_t peer_item, uint32_t peer_full, uint32_t w) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(peer_full), "r"(4u) : "memory");
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];"
               ::"r"(peer_item), "r"(w), "r"(peer_full) : "memory");
}
struct Tc2rSched {
  uint32_t full, empty_leader, ring;   // shared-memory addresses: this CTA's `full` barriers and ring, the leader's `empty`
  // The n-th item number of this cluster (T2R_NO_ITEM: no more work), or false when the wait ran out.  A warp calls
  // this with all lanes; its lane 0 (or the single calling thread) then reports the slot read with done().
  __device__ __forceinline__ bool next(uint32_t n, uint32_t &w, volatile WaitCtl *ctl) const {
    const uint32_t slot = n % T2R_SCHED;
    if (!mbar_wait(full + 8 * slot, (n / T2R_SCHED) & 1u, ctl, kWaitItemNumber, T2R_ITEM_WAIT_SHIFT)) return false;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(ring + 4 * slot) : "memory");
    return true;
  }
  __device__ __forceinline__ void done(uint32_t n) const { mbar_arrive_cluster(empty_leader + 8 * (n % T2R_SCHED)); }
};

// One work item of a launch: a 256 x BN2 tile of the product over one split-K slice.
struct Tc2rItem {
  long m_tile0, n_tile0, k_begin;
  long z;      // k slice of a tail tile, -1 for a whole-reduction tile
  long slot;   // partial-sum block of the workspace (tail items only)
  int num_k_tiles;
};

// Persistent: the launch has as many clusters as the device runs at once; cluster c starts with item c and takes
// further items from `sched_counter` (zero at launch) as it finishes (m tiles fastest, so that clusters running
// side by side share their B rows in L2).  All
// rings, barrier phases and accumulator buffers run on with a k-tile count `g` that spans the items, so the
// loads, splits and first MMAs of an item run under the previous item's epilogue stores, and the barrier and
// tensor-memory set-up is paid once per launch.
template <class P, int BN2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T2_THREADS, 1) tc2r_kernel(const __grid_constant__ P p, const StallCtl ctl,
                                                                                                unsigned *sched_counter) {
  typedef Tc2rCfg<BN2> Cfg;
  constexpr int R = Cfg::HI_SLOTS, L = Cfg::LO_SLOTS;
  constexpr int BH = Cfg::BH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t *lo_ring = smem + R * Cfg::SLOT_BYTES;
  uint8_t *aux = lo_ring + L * Cfg::SLOT_BYTES;
  // full[R], empty[R], raw_full[R], acc_full[2], acc_empty[2], lo_empty[L], sched_full[T2R_SCHED], sched_empty[T2R_SCHED], sched_go
  uint64_t *bars = reinterpret_cast<uint64_t *>(aux);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * R + 4 + L + 2 * T2R_SCHED + 1);
  volatile WaitCtl *abort_flag = reinterpret_cast<volatile WaitCtl *>(tmem_slot + 2);
  uint32_t *sched_ring = tmem_slot + 2 + sizeof(WaitCtl) / 4;
  static_assert((3 * 6 + 4 + Cfg::LO_SLOTS + 2 * T2R_SCHED + 1) * 8 + 8 + sizeof(WaitCtl) + 4 * T2R_SCHED <= 512, "auxiliary shared memory");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  // item counts fit 32 bits (checked by the launcher): the decode below runs once per item in every role
  const uint32_t gm = (uint32_t)((p.M + 255) / 256), gn = (uint32_t)((p.N + BN2 - 1) / BN2);
  const uint32_t tiles = gm * gn, tail_first = p.ws ? (uint32_t)p.tail_first : tiles;
  const uint32_t tail_tiles = tiles - tail_first;
  const uint32_t items = tail_first + tail_tiles * (uint32_t)p.tail_splits, cluster_id = blockIdx.x >> 1, clusters = gridDim.x >> 1;
  // Items 0 .. tail_first - 1 are whole tiles; the rest are the k slices of the tail tiles, slice-major (clusters
  // running side by side then work on neighbouring tiles of one k range and share its B rows in L2).
  auto item_at = [&](uint32_t w) {
    Tc2rItem t;
    uint32_t tile = w;
    t.z = -1;
    t.k_begin = 0;
    long k_end = p.K;
    if (w >= tail_first) {
      const uint32_t r = w - tail_first, z = r / tail_tiles;
      tile = tail_first + (r - z * tail_tiles);
      t.z = z;
      t.slot = (long)(tile - tail_first) * p.tail_splits + z;
      t.k_begin = (long)z * p.k_per_split;
      k_end = t.k_begin + p.k_per_split;
      if (k_end > p.K) k_end = p.K;
    }
    const uint32_t nt = tile / gm, mt = tile - nt * gm;
    t.m_tile0 = (long)mt * 256; t.n_tile0 = (long)nt * BN2;
    t.num_k_tiles = (int)((k_end - t.k_begin + TC_BK - 1) / TC_BK);
    return t;
  };

  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + R), bar_raw = smem_u32(bars + 2 * R);
  const uint32_t bar_acc_full = smem_u32(bars + 3 * R), bar_acc_empty = smem_u32(bars + 3 * R + 2);
  const uint32_t bar_lo_empty = smem_u32(bars + 3 * R + 4);
  const uint32_t bar_sched_full = smem_u32(bars + 3 * R + 4 + L), bar_sched_empty = bar_sched_full + 8 * T2R_SCHED;
  const uint32_t bar_sched_go = bar_sched_empty + 8 * T2R_SCHED;
  Tc2rSched sched;
  sched.full = bar_sched_full;
  sched.empty_leader = mapa_shared(bar_sched_empty, 0);
  sched.ring = smem_u32(sched_ring);
  if (tid == 0) {
    for (int s = 0; s < R; s++) {
      mbar_init(bar_full + 8 * s, 2 * T2_PRODUCERS / 64);   // one group of two splitter warps in each CTA (used in CTA 0)
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_raw + 8 * s, 1);                        // this CTA's TMA thread + the bytes it announces
    }
    for (int l = 0; l < L; l++) mbar_init(bar_lo_empty + 8 * l, 1);
    for (int k = 0; k < T2R_SCHED; k++) {
      mbar_init(bar_sched_full + 8 * k, 1);
      mbar_init(bar_sched_empty + 8 * k, T2R_SCHED_READERS);   // used in CTA 0
    }
    mbar_init(bar_sched_go, 1);                                // used in CTA 0
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
    // ------------------------------------------------------------ splitters
    setmaxnreg_dec<72>();
    const uint32_t full_leader = mapa_shared(bar_full, 0);
    // Two groups of two warps take alternate k tiles, so that one group's barrier round trips and proxy fence
    // overlap the other group's copying: under the MMAs' own shared-memory traffic every access here waits
    // hundreds of cycles.
    const int grp = warp >> 1, gtid = tid & 63;
    int g0 = 0;
    for (uint32_t n = 0; ok; n++) {
      uint32_t w = T2R_NO_ITEM;
      ok = __all_sync(0xffffffffu, sched.next(n, w, abort_flag));
      if (!ok) break;
      if (lane == 0) sched.done(n);
      if (w == T2R_NO_ITEM) break;
      const int nk = item_at(w).num_k_tiles;
      for (int it = (g0 + grp) & 1; it < nk; it += 2) {
        const int g = g0 + it;
        const int s = g % R, ls = g % L;
        const uint32_t raw_bar = bar_raw + 8 * s, raw_par = (uint32_t)(g / R) & 1u;
        // The lo slot is free once the MMAs of tile g - L have read it.  It has a barrier of its own: the hi slots'
        // `empty` barriers can run two phases ahead of a splitter group that was slow to wake up (the other group and
        // the other MMA thread do not wait for it), and a parity wait cannot tell two completed phases from none.
        const uint32_t lo_bar = bar_lo_empty + 8 * ls, lo_par = (uint32_t)(g / L + 1) & 1u;
        const bool r1 = mbar_try_wait(raw_bar, raw_par), r2 = g < L || mbar_try_wait(lo_bar, lo_par);
        ok = (r1 || mbar_wait(raw_bar, raw_par, abort_flag, kWaitRawTile)) && (r2 || mbar_wait(lo_bar, lo_par, abort_flag, kWaitLoSlot));
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t src = smem_u32(smem + s * Cfg::SLOT_BYTES) + (uint32_t)gtid * 16u;
        const uint32_t dst = smem_u32(lo_ring + ls * Cfg::SLOT_BYTES) + (uint32_t)gtid * 16u;
        // a quarter of the group's 16-byte chunks per batch: all loads of a batch are in flight before its first store
        constexpr int GT = T2_PRODUCERS / 2, PASSES = Cfg::SLOT_BYTES / (GT * 16), BATCH = PASSES <= 24 ? PASSES / 2 : PASSES / 4;
        static_assert(Cfg::SLOT_BYTES % (GT * 16 * 4) == 0, "slot size");
#pragma unroll
        for (int i0 = 0; i0 < PASSES; i0 += BATCH) {
          uint4 v[BATCH];
#pragma unroll
          for (int i = 0; i < BATCH; i++) v[i] = lds128(src + (uint32_t)((i0 + i) * GT * 16));
#pragma unroll
          for (int i = 0; i < BATCH; i++) sts128(dst + (uint32_t)((i0 + i) * GT * 16), tf32_lo4(v[i]));
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(full_leader + 8 * s);
      }
      g0 += nk;
    }
  } else if (warp < T2_DRAIN_WARP0) {
    setmaxnreg_dec<40>();
    if ((warp == T2_MMA_WARP || warp == T2R_MMA_WARP2) && lane == 0 && rank == 0) {
      // ---------------------------------------------------------- MMA issuers
      // Two threads take alternate k tiles (and with them alternate accumulator buffers): while one is blocked on
      // the tensor pipe's queue the other sits through its barrier polls, each a shared-memory round trip of
      // hundreds of cycles under the MMAs' own traffic.
      // With an odd number of hi slots a thread meets a slot only every second time round, so its parity wait for
      // tile g sees the phase of tile g - 2R as "the previous one".  That is safe because the phase of tile g - R
      // is over by then: the thread has waited for tile g - 2, which was split only after the MMAs of tile g - 5
      // released its lo slot (three lo slots), and R = 5 is the only odd ring size in use (static_assert below).
      // A scheme in which a thread skips whole revolutions (alternate ITEMS instead of alternate tiles) loses that
      // guarantee and stalls.
      constexpr bool A_MN = P::OpA::MN_MAJOR, B_MN = P::OpB::MN_MAJOR;
      constexpr uint32_t idesc = umma2_idesc_tf32(BN2, A_MN, B_MN);
      const int buf = warp == T2_MMA_WARP ? 0 : 1;
      int g0 = 0;
      for (uint32_t n = 0; ok; n++) {
        uint32_t w = T2R_NO_ITEM;
        ok = sched.next(n, w, abort_flag);
        if (!ok) break;
        sched.done(n);
        if (w == T2R_NO_ITEM) break;
        const int nk = item_at(w).num_k_tiles;
        for (int it = (g0 + buf) & 1; it < nk; it += 2) {
          const int g = g0 + it;
          const int s = g % R, ls = g % L;
          const uint32_t phase = (uint32_t)(g / R) & 1u, acc_phase = (uint32_t)(g >> 1) & 1u;
          ok = mbar_wait_spin(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag, kWaitAccEmpty);
          ok = ok && mbar_wait_spin(bar_full + 8 * s, phase, abort_flag, kWaitTileFull);
          if (!ok) break;
          tc_fence_after();
          const uint32_t hs = smem_u32(smem + s * Cfg::SLOT_BYTES), lsl = smem_u32(lo_ring + ls * Cfg::SLOT_BYTES);
          const uint64_t a_hi = umma_desc_sw128<A_MN>(hs), a_lo = umma_desc_sw128<A_MN>(lsl);
          const uint64_t b_hi = umma_desc_sw128<B_MN>(hs + Cfg::A_BYTES), b_lo = umma_desc_sw128<B_MN>(lsl + Cfg::A_BYTES);
          const uint32_t d = tmem_base + (uint32_t)(buf * BN2);
#pragma unroll
          for (int kk = 0; kk < TC_BK / 8; kk++) {
            const uint64_t adv_a = (uint64_t)((kk * umma_kstep_bytes<A_MN>()) >> 4);
            const uint64_t adv_b = (uint64_t)((kk * umma_kstep_bytes<B_MN>()) >> 4);
            umma2_tf32(d, a_lo + adv_a, b_hi + adv_b, idesc, kk ? 1u : 0u);
            umma2_tf32(d, a_hi + adv_a, b_lo + adv_b, idesc, 1u);
          }
#pragma unroll
          for (int kk = 0; kk < TC_BK / 8; kk++) {
            const uint64_t adv_a = (uint64_t)((kk * umma_kstep_bytes<A_MN>()) >> 4);
            const uint64_t adv_b = (uint64_t)((kk * umma_kstep_bytes<B_MN>()) >> 4);
            umma2_tf32(d, a_hi + adv_a, b_hi + adv_b, idesc, 1u);
          }
          umma2_commit_both(bar_empty + 8 * s);
          umma2_commit_both(bar_lo_empty + 8 * ls);
          umma2_commit_both(bar_acc_full + 8 * buf);
        }
        g0 += nk;
      }
    } else if (warp == T2R_TMA_WARP && lane == 0) {
      // ---------------------------------------------------------- TMA issuer (one per CTA)
      int g0 = 0;
      for (uint32_t n = 0; ok; n++) {
        uint32_t w = T2R_NO_ITEM;
        ok = sched.next(n, w, abort_flag);
        if (!ok) break;
        sched.done(n);
        if (w == T2R_NO_ITEM) break;
        if (rank == 0) mbar_arrive_local(bar_sched_go);   // item n is under way: time to fetch the number of item n + 1
        const Tc2rItem item = item_at(w);
        const long m0 = item.m_tile0 + (long)rank * TC_BM, n0 = item.n_tile0 + (long)rank * BH;
        for (int t = 0; t < item.num_k_tiles; t++) {
          const int g = g0 + t;
          const int s = g % R;
          if (g >= R && !mbar_wait(bar_empty + 8 * s, (uint32_t)((g - R) / R) & 1u, abort_flag, kWaitSlotEmpty)) { ok = false; break; }
          const long k0 = item.k_begin + (long)t * TC_BK;
          const uint32_t slot = smem_u32(smem + s * Cfg::SLOT_BYTES);
          mbar_arrive_expect_tx(bar_raw + 8 * s, (uint32_t)Cfg::SLOT_BYTES);
          tma_issue<TC_BM>(p.a, slot, m0, k0, bar_raw + 8 * s);
          tma_issue<BH>(p.b, slot + Cfg::A_BYTES, n0, k0, bar_raw + 8 * s);
        }
        g0 += item.num_k_tiles;
      }
    } else if (warp == T2R_SCHED_WARP && lane == 0 && rank == 0) {
      // ---------------------------------------------------------- item hand-out (one thread per cluster)
      const uint32_t peer_ring = mapa_shared(sched.ring, 1), peer_full = mapa_shared(bar_sched_full, 1);
      for (uint32_t n = 0;; n++) {
        const uint32_t slot = n % T2R_SCHED;
        if (n >= 1 && !mbar_wait(bar_sched_go, (n - 1) & 1u, abort_flag, kWaitItemGo, T2R_ITEM_WAIT_SHIFT)) break;
        if (n >= T2R_SCHED && !mbar_wait(bar_sched_empty + 8 * slot, (n / T2R_SCHED - 1) & 1u, abort_flag, kWaitItemSlot, T2R_ITEM_WAIT_SHIFT)) break;
        uint32_t w = n == 0 ? cluster_id : clusters + atomicAdd(sched_counter, 1u);
        if (w >= items) w = T2R_NO_ITEM;
        sched_publish_peer(peer_ring + 4 * slot, peer_full + 8 * slot, w);
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(sched.ring + 4 * slot), "r"(w) : "memory");
        mbar_arrive_local(bar_sched_full + 8 * slot);
        if (w == T2R_NO_ITEM) break;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ drain + epilogue warps
    setmaxnreg_inc<192>();
    const int q = warp & 3;
    const int h = (warp - T2_DRAIN_WARP0) >> 2;
    constexpr int NCOL = BN2 / 2;
    const uint32_t acc_empty_leader = mapa_shared(bar_acc_empty, 0);
    // Pixel-pair products over 64 planes (a 128-column tile: parity 0 in columns 0-63, parity 1 in 64-127): this warp
    // takes 32 planes in both parities instead of 64 columns of one, for the whole-line epilogue
    const bool pair_capable = P::PAIR && BN2 == 128 && p.epi.pair_K == 64 && p.epi.beta == 0.f;
    int g0 = 0;
    for (uint32_t n = 0; ok; n++) {
      uint32_t w = T2R_NO_ITEM;
      ok = __all_sync(0xffffffffu, sched.next(n, w, abort_flag));
      if (!ok) break;
      if (lane == 0) sched.done(n);
      if (w == T2R_NO_ITEM) break;
      const Tc2rItem item = item_at(w);
      const bool pair_lines = pair_capable && item.z < 0;   // tail slices keep the plain column order for the workspace
      float acc[NCOL];
#pragma unroll
      for (int j = 0; j < NCOL; j++) acc[j] = 0.f;
      for (int it = 0; it < item.num_k_tiles; it++) {
        const int g = g0 + it;
        const int buf = g & 1;
        const uint32_t acc_phase = (uint32_t)(g >> 1) & 1u;
        ok = mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kWaitAccFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN2 + (pair_lines ? h * 32 : h * NCOL));
#pragma unroll
        for (int c0 = 0; c0 < NCOL; c0 += 32) {
          uint32_t v[32];
          tmem_ld32_nowait(t0 + (pair_lines ? 2 * c0 : c0), v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) acc[c0 + j] += __uint_as_float(v[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8 * buf);
      }
      g0 += item.num_k_tiles;
      if (ok) {
        const long m = item.m_tile0 + (long)rank * TC_BM + q * 32 + lane;
        if (item.z >= 0) {
          // partial sums of a tail slice: ws[slot][column][row], a warp's 32 rows side by side
          float *o = p.ws + (item.slot * BN2 + h * NCOL) * 256 + (rank * TC_BM + q * 32 + lane);
#pragma unroll
          for (int j = 0; j < NCOL; j++) o[j * 256] = acc[j];
        } else if constexpr (P::PAIR && BN2 == 128) {
          if (pair_lines) tc2_store_pair_rows<P>(p, acc, m, h * 32);
          else tc2_store_rows<P, NCOL>(p, acc, m, item.n_tile0 + h * NCOL, 0, true);
        } else {
          tc2_store_rows<P, NCOL>(p, acc, m, item.n_tile0 + h * NCOL, 0, true);
        }
      }
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
