// tcgen05 tensor-core engine for mm::Problem: FP32-accurate products through a 3xTF32 split.
//
// One CTA computes a 128 x BN tile of D (BN = 64 or 128) with the accumulator in tensor memory:
//
//   warps 0-7  producers: gather operand elements through the problem's row / k maps (this is the
//              implicit im2col: no column matrix ever exists in memory) with cp.async straight into
//              K-major, 128-byte-swizzled shared-memory tiles (the canonical tcgen05 operand layout,
//              32 k per stage, copies running STAGES-1 tiles ahead), then split every value x in
//              place into hi = tf32(x) and, in a second tile, lo = tf32(x - hi).
//   warp 8     one elected thread issues tcgen05.mma.kind::tf32, three per k-step:
//              Alo*Bhi + Ahi*Blo + Ahi*Bhi (lo*lo is below FP32 resolution).  Every 32-k tile goes
//              into one of two TMEM accumulator buffers; tcgen05.commit hands smem stages back to
//              the producers and finished accumulators to the drain warps through mbarriers.
//   warps 9-16 drain: tcgen05.ld each finished 32-k partial tile and add it into FP32 registers
//              (round-to-nearest; the tensor core's own accumulation truncates, so long chains are
//              kept out of TMEM), then the epilogue: TMEM lane = output row m, so consecutive
//              lanes store consecutive addresses; alpha / beta / bias applied on the way out.
//
// Every mbarrier wait is bounded (StallCtl::limit SM cycles); on expiry the CTA raises the stall flags
// (one in device memory that every later CTA of the stream reads on entry and then does no work, one in mapped
// host memory that the host reads at its next synchronisation point), skips its stores and exits normally.
#ifndef THC_MM_TC_CUH
#define THC_MM_TC_CUH

#include "mm_problem.cuh"

namespace thc {
namespace mm {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;  // floats per stage row = 128 bytes = one swizzle span
constexpr int TC_PRODUCERS = 256;
constexpr int TC_DRAINERS = 256;
constexpr int TC_THREADS = TC_PRODUCERS + 32 + TC_DRAINERS;

template <int BN> struct TcCfg {
  static constexpr int STAGES = BN == 128 ? 3 : 4;
  static constexpr int A_BYTES = TC_BM * 128;      // one precision plane of A
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);
  static constexpr int NACC = 512 / BN > 4 ? 4 : 512 / BN;  // TMEM accumulator buffers (NACC * BN columns)
  static constexpr int AUX_BYTES = (STAGES + 1) * 2 * TC_BK * (int)sizeof(Info) + 256   // k maps, mbarriers, flags
                                   + (TC_BM + BN) * (int)sizeof(Info);                   // row maps of the tile
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + 1024;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)  // suspend-time hint (ns): sleep in hardware instead of spinning
      : "memory");
  return ok != 0;
}
// Stall handling.  StallCtl (thc_internal.h) is a kernel parameter: `dev_flag` (device memory) is read by every
// CTA on entry, a CTA that finds it set does no work; `host_flag` (mapped pinned host memory) is what the host
// reads after it has synchronised the stream; `limit` is the number of SM cycles one wait may take.  WaitCtl is
// the per-CTA copy in shared memory that the waits poll: `abort` is set by the first wait of the CTA that runs
// out (and, in a cluster pair, in the peer CTA's copy too, through `peer_abort`), every other role leaves at its
// next poll.
struct WaitCtl {
  int abort;             // 0, or the code of the wait that gave up first (kWait*), or kWaitPeer / kWaitEntry
  uint32_t peer_abort;   // shared::cluster address of the peer CTA's `abort`, 0 outside a cluster
  long long limit;
};
// Which wait ran out: the code travels to the host flag and into the error message (names: thc_general.cu).
enum : int {
  kWaitOther = 1, kWaitRawTile = 2, kWaitLoSlot = 3, kWaitAccEmpty = 4, kWaitTileFull = 5, kWaitSlotEmpty = 6,
  kWaitAccFull = 7, kWaitItemNumber = 8, kWaitItemGo = 9, kWaitItemSlot = 10, kWaitProbe = 11,
  kWaitEntry = 254, kWaitPeer = 255
};
__device__ __forceinline__ void wait_ctl_init(volatile WaitCtl *w, const StallCtl &ctl, uint32_t peer_abort = 0) {
  w->abort = *reinterpret_cast<volatile int *>(ctl.dev_flag) != 0 ? kWaitEntry : 0;
  w->peer_abort = peer_abort;
  w->limit = ctl.limit;
}
__device__ __forceinline__ void wait_ctl_give_up(volatile WaitCtl *w, int code = kWaitOther) {
  if (w->abort == 0) w->abort = code;
  const uint32_t peer = w->peer_abort;
  if (peer) asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer), "r"((uint32_t)kWaitPeer) : "memory");
}
// What a CTA does before it leaves when any of its waits ran out (or it found the flag set on entry): `code` is its
// abort word.  The host flag keeps the code of a wait that ran out in preference to "the peer / an earlier kernel did".
__device__ __forceinline__ void stall_raise(const StallCtl &ctl, int code = kWaitOther) {
  atomicExch(ctl.dev_flag, 1);
  volatile int *host = reinterpret_cast<volatile int *>(ctl.host_flag);
  if ((code != kWaitEntry && code != kWaitPeer) || *host == 0) *host = code;
  __threadfence_system();
}
// Bounded wait.  Returns false when the phase did not complete within the limit (the CTA's abort word is then
// set to `code`) or another thread already gave up.
// `shift`: the wait may take 2^shift limits.  For waits that span a whole work item rather than one k tile (the item
// hand-out of the persistent engine): when the pipeline really stands still a k-tile wait runs out first and sets
// the abort word, which these waits poll too, so the longer allowance costs no detection time, and a long item
// (or a kernel slowed a few hundred times by a profiler's instrumentation) is not taken for a stall.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile WaitCtl *w, int code = kWaitOther,
                                          int shift = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 15) == 0) {
      if (w->abort) return false;
      if (clock64() - t0 > (w->limit << shift)) { wait_ctl_give_up(w, code); return false; }
    }
  }
  return true;
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Operand tile descriptors.
//   K-major : rows (m or n) of 128 B = 32 k, 128-byte swizzle (16-byte chunk index XOR row % 8); 8-row groups
//             1024 B apart (stride offset); leading offset unused.
//   MN-major: rows are k, each 128 B = 32 consecutive m (or n); the tile is [32-wide block][32 k][128 B].  For
//             32-bit elements the tensor core reads this form with the "128-byte swizzle, 32-byte atom" mode:
//             32-byte granule index XOR k % 4, blocks along m / n 4096 B apart (leading offset), 4-k groups
//             512 B apart (stride offset).
template <bool MN_MAJOR>
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);               // start address
  d |= (uint64_t)(MN_MAJOR ? (4096 >> 4) : 1) << 16;          // leading byte offset
  d |= (uint64_t)((MN_MAJOR ? 512 : 1024) >> 4) << 32;        // stride byte offset
  d |= (uint64_t)1 << 46;                                     // descriptor version (Blackwell)
  d |= (uint64_t)(MN_MAJOR ? 1 : 2) << 61;                    // SWIZZLE_128B_BASE32B : SWIZZLE_128B
  return d;
}
// bytes between the operand slices of consecutive MMAs (8 k each)
template <bool MN_MAJOR> __host__ __device__ constexpr int umma_kstep_bytes() { return MN_MAJOR ? 1024 : 32; }
// kind::tf32, FP32 accumulate, M = 128; bits 15 / 16 flag an MN-major A / B
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int n, bool a_mn = false, bool b_mn = false) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *v) {
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
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void cp_async4(uint32_t dst, const float *src, const float *any_valid) {
  // 4-byte asynchronous global -> shared copy; a null source zero-fills the destination (src-size 0:
  // nothing is read, `any_valid` only keeps the address operand well-formed)
  const unsigned n = src ? 4u : 0u;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"((const void *)(src ? src : any_valid)), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const float *src, bool valid) {
  const unsigned n = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"((const void *)src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One producer thread's share of an operand tile for one stage (32 k).
//   ALONG_K false: the thread owns one row and CPT 16-byte chunks of it (lanes run along rows).
//   ALONG_K true : the thread owns one chunk column and RPT rows (lanes run along k).
// issue() starts asynchronous copies of the raw FP32 elements straight into their final (swizzled)
// positions of the `hi` tile; split() later re-reads the thread's own chunks, rounds them to TF32 in
// place and writes the residuals to the `lo` tile.  Only the issuing thread touches its chunks, so
// cp.async.wait_group is all the synchronisation the two steps need.
template <class Op, int ROWS>
struct TileFill {
  static constexpr int NG = TC_PRODUCERS / ROWS;          // row mapping: thread groups per row
  static constexpr int CPT = 8 / NG;                      // chunks per thread (row mapping)
  static constexpr int RPT = ROWS / 32;                   // rows per thread (k mapping)
  static constexpr int NINFO = Op::MN_MAJOR ? ROWS / 32 : (Op::ALONG_K ? RPT : 1);
  static constexpr int NCH = Op::ALONG_K ? RPT : CPT;     // 16-byte chunks per thread per stage
  // Operands that cannot be copied 16 bytes at a time (gathers) go through registers instead of
  // cp.async: coalesced 4-byte loads one tile ahead, rounded in registers, one 16-byte shared store
  // per chunk.  (A 4-byte cp.async costs a shared-memory wavefront per 8 elements; this path one
  // per 32.)
  static constexpr bool REG = !Op::VECTORIZABLE;
  // Register-path operands whose memory runs along k use a third mapping: lane = k within the tile,
  // warp w owns rows [w*RPW, (w+1)*RPW).  One 128-byte load and two conflict-free 4-byte shared
  // stores per 32 elements, one k map per thread per stage; row maps come from a shared table.
  static constexpr bool KLANE = REG && Op::ALONG_K;
  static constexpr int RPW = ROWS / (TC_PRODUCERS / 32);
  static constexpr int NVAL = ROWS * TC_BK / TC_PRODUCERS;  // elements per thread per stage
  Info rows[NINFO];
  float v[REG ? NVAL : 1];
  __device__ __forceinline__ void init(const Op &op, long row0, int tid) {
    if constexpr (Op::MN_MAJOR) {
      // thread = (pixel tid / 8 of the stage, 16-byte column tid % 8 of every 32-row block)
#pragma unroll
      for (int a = 0; a < NINFO; a++) {
        const long r0 = row0 + 32 * a + (tid & 7) * 4;
        rows[a] = op.rowblock(r0);
        if (r0 >= op.rows.count) rows[a].y = kInvalid;
      }
    } else if (Op::ALONG_K) {
#pragma unroll
      for (int i = 0; i < NINFO; i++) rows[i] = op.rows(row0 + (tid >> 3) + 32 * i);
    } else
      rows[0] = op.rows(row0 + (tid % ROWS));
  }
  static __device__ __forceinline__ int chunk_of(int tid, int c) { return Op::ALONG_K ? (tid & 7) : ((tid / ROWS) * CPT + c); }
  static __device__ __forceinline__ int row_of(int tid, int c) { return Op::ALONG_K ? ((tid >> 3) + 32 * c) : (tid % ROWS); }
  static __device__ __forceinline__ int offset_of(int row, int chunk) {
    return (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4);
  }
  __device__ __forceinline__ Info kinfo(const Op &op, const Info *ki, long k0, long k_end, int kk) const {
    if (Op::KMap::kLinear) {
      Info k = op.ks(k0 + kk);
      if (k0 + kk >= k_end) k.y = kInvalid;
      return k;
    }
    return ki[kk];
  }
  __device__ __forceinline__ void issue(const Op &op, const Info *ki, long k0, long k_end, int tid, uint32_t hi_tile) const {
    if constexpr (Op::MN_MAJOR) {
      const int kk = tid >> 3, q0 = tid & 7;
      Info px = op.ks(k0 + kk);
      if (k0 + kk >= k_end) px.y = kInvalid;
#pragma unroll
      for (int a = 0; a < NINFO; a++) {
        const bool okay = op.valid(px, rows[a]);
        const long o = okay ? px.off + rows[a].off : 0;
        const uint32_t dst = hi_tile + (uint32_t)(a * 4096 + kk * 128 + ((((q0 >> 1) ^ (kk & 3)) << 5) | ((q0 & 1) << 4)));
        cp_async16(dst, op.base + o, okay);
        cp_async16(dst + ROWS * 128, op.lo + o, okay);  // the lo tile follows the hi tile
      }
      return;
    } else if constexpr (Op::PRESPLIT) {
      // both planes are padded to whole k tiles: no k tail, only the row / box test of the tile
      const Info kt = op.ktile(k0, tid & 7);   // this thread's 16-byte chunk of the k tile
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        const Info &r = rows[c];
        const uint32_t dst = hi_tile + (uint32_t)offset_of(row_of(tid, c), chunk_of(tid, c));
        const bool okay = op.valid(r, kt);
        const long o = okay ? r.off + kt.off : 0;
        cp_async16(dst, op.base + o, okay);
        cp_async16(dst + ROWS * 128, op.lo + o, okay);  // the lo tile follows the hi tile
      }
      return;
    } else {
#pragma unroll
      for (int c = 0; c < NCH; c++) {
        const int chunk = chunk_of(tid, c);
        const Info &r = rows[Op::ALONG_K ? c : 0];
        const uint32_t dst = hi_tile + (uint32_t)offset_of(row_of(tid, c), chunk);
        const long kc = k0 + chunk * 4;
        if (Op::VECTORIZABLE && op.vec4 && kc + 3 < k_end && kc + 3 < op.ks.count) {
          cp_async16(dst, op.base + (r.y >= 0 ? r.off + kc : 0), r.y >= 0);
        } else {
#pragma unroll
          for (int e = 0; e < 4; e++) cp_async4(dst + 4 * e, op.locate(r, kinfo(op, ki, k0, k_end, chunk * 4 + e)), op.base);
        }
      }
    }
  }
  __device__ __forceinline__ void load_regs(const Op &op, const Info *ki, const Info *rowtab, long k0, long k_end, int tid) {
    if (KLANE) {
      const int lane = tid & 31, w = tid >> 5;
      const Info k = kinfo(op, ki, k0, k_end, lane);
#pragma unroll
      for (int j = 0; j < RPW; j++) v[REG ? j : 0] = op.fetch(rowtab[w * RPW + j], k);
      return;
    }
#pragma unroll
    for (int c = 0; c < NCH; c++) {
      const int chunk = chunk_of(tid, c);
      const Info &r = rows[Op::ALONG_K ? c : 0];
#pragma unroll
      for (int e = 0; e < 4; e++) v[REG ? c * 4 + e : 0] = op.fetch(r, kinfo(op, ki, k0, k_end, chunk * 4 + e));
    }
  }
  __device__ __forceinline__ void store_regs(uint8_t *hi_tile, uint8_t *lo_tile, int tid) const {
    if (KLANE) {
      const int lane = tid & 31, w = tid >> 5;
#pragma unroll
      for (int j = 0; j < RPW; j++) {
        const int off = offset_of(w * RPW + j, lane >> 2) + (lane & 3) * 4;
        const float x = v[REG ? j : 0];
        const uint32_t h = to_tf32(x);
        *reinterpret_cast<uint32_t *>(hi_tile + off) = h;
        *reinterpret_cast<uint32_t *>(lo_tile + off) = to_tf32(x - __uint_as_float(h));
      }
      return;
    }
#pragma unroll
    for (int c = 0; c < NCH; c++) {
      const int off = offset_of(row_of(tid, c), chunk_of(tid, c));
      const float *x = &v[REG ? c * 4 : 0];
      uint4 h, l;
      h.x = to_tf32(x[0]); l.x = to_tf32(x[0] - __uint_as_float(h.x));
      h.y = to_tf32(x[1]); l.y = to_tf32(x[1] - __uint_as_float(h.y));
      h.z = to_tf32(x[2]); l.z = to_tf32(x[2] - __uint_as_float(h.z));
      h.w = to_tf32(x[3]); l.w = to_tf32(x[3] - __uint_as_float(h.w));
      *reinterpret_cast<uint4 *>(hi_tile + off) = h;
      *reinterpret_cast<uint4 *>(lo_tile + off) = l;
    }
  }
  __device__ __forceinline__ void split(uint8_t *hi_tile, uint8_t *lo_tile, int tid) const {
    if (Op::PRESPLIT) return;  // nothing to do: both planes arrived ready-made
#pragma unroll
    for (int c = 0; c < NCH; c++) {
      const int off = offset_of(row_of(tid, c), chunk_of(tid, c));
      const float4 v = *reinterpret_cast<const float4 *>(hi_tile + off);
      uint4 h, l;
      h.x = to_tf32(v.x); l.x = to_tf32(v.x - __uint_as_float(h.x));
      h.y = to_tf32(v.y); l.y = to_tf32(v.y - __uint_as_float(h.y));
      h.z = to_tf32(v.z); l.z = to_tf32(v.z - __uint_as_float(h.z));
      h.w = to_tf32(v.w); l.w = to_tf32(v.w - __uint_as_float(h.w));
      *reinterpret_cast<uint4 *>(hi_tile + off) = h;
      *reinterpret_cast<uint4 *>(lo_tile + off) = l;
    }
  }
};

template <class P, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) tc_kernel(const P p, const StallCtl ctl) {
  typedef TcCfg<BN> Cfg;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NACC = Cfg::NACC;               // TMEM accumulator buffers in flight
  constexpr int KRING = STAGES + 1;             // k-map staging buffers (maps are staged 3 tiles ahead)
  constexpr int MMA_WARP = TC_PRODUCERS / 32;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t *aux = smem + STAGES * Cfg::STAGE_BYTES;
  Info *kiA = reinterpret_cast<Info *>(aux);                 // [KRING][32]
  Info *kiB = kiA + KRING * TC_BK;                           // [KRING][32]
  uint64_t *bars = reinterpret_cast<uint64_t *>(kiB + KRING * TC_BK);  // full[S], empty[S], acc_full[NACC], acc_empty[NACC]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 2 * NACC);
  volatile int *cont = reinterpret_cast<volatile int *>(tmem_slot + 1);   // [2]
  volatile WaitCtl *abort_flag = reinterpret_cast<volatile WaitCtl *>(tmem_slot + 4);   // 16-byte aligned
  Info *rowtabA = reinterpret_cast<Info *>(aux + Cfg::AUX_BYTES - (TC_BM + BN) * (int)sizeof(Info));  // [128]
  Info *rowtabB = rowtabA + TC_BM;                                                                     // [BN]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long m0 = (long)blockIdx.x * TC_BM, n0 = (long)blockIdx.y * BN;
  long k_begin = 0, k_end = p.K;
  if (p.ws) {
    k_begin = (long)blockIdx.z * p.k_per_split;
    k_end = k_begin + p.k_per_split;
    if (k_end > p.K) k_end = p.K;
  }
  const int num_k_tiles = (int)((k_end - k_begin + TC_BK - 1) / TC_BK);

  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const uint32_t bar_acc_full = smem_u32(bars + 2 * STAGES), bar_acc_empty = smem_u32(bars + 2 * STAGES + NACC);
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(bar_full + 8 * s, TC_PRODUCERS / 32);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < NACC; b++) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, TC_DRAINERS / 32);
    }
    wait_ctl_init(abort_flag, ctl);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(smem_u32(tmem_slot), NACC * BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = abort_flag->abort == 0;   // set on entry: an earlier kernel of this stream stalled, do no work

  if (!ok) {
  } else if (warp < MMA_WARP) {
    // ------------------------------------------------------------ producers
    typedef TileFill<typename P::OpA, TC_BM> FillA;
    typedef TileFill<typename P::OpB, BN> FillB;
    constexpr bool NEED_KI = !(P::OpA::KMap::kLinear && P::OpB::KMap::kLinear);
    FillA fa;
    FillB fb;
    fa.init(p.a, m0, tid);
    fb.init(p.b, n0, tid);
    // k maps of tile t (gather problems only): two threads' worth of divisions per k, staged in a ring
    auto stage_kmaps = [&](int t) {
      if (!NEED_KI || t >= num_k_tiles) return;
      const long k0 = k_begin + (long)t * TC_BK;
      const int kb = (t % KRING) * TC_BK;
      if (tid < TC_BK) {
        Info ka = p.a.ks(k0 + tid);
        if (k0 + tid >= k_end) ka.y = kInvalid;
        kiA[kb + tid] = ka;
      } else if (tid < 2 * TC_BK) {
        Info kbi = p.b.ks(k0 + tid - TC_BK);
        if (k0 + tid - TC_BK >= k_end) kbi.y = kInvalid;
        kiB[kb + tid - TC_BK] = kbi;
      }
    };
    // starts the copies of tile t into its stage; one commit group per tile, even when t is past the end
    auto issue_tile = [&](int t) {
      if (t < num_k_tiles) {
        const int s = t % STAGES;
        const long k0 = k_begin + (long)t * TC_BK;
        const int kb = (t % KRING) * TC_BK;
        const uint32_t stage = smem_u32(smem + s * Cfg::STAGE_BYTES);
        if constexpr (!FillA::REG) fa.issue(p.a, kiA + kb, k0, k_end, tid, stage);
        if constexpr (!FillB::REG) fb.issue(p.b, kiB + kb, k0, k_end, tid, stage + 2 * Cfg::A_BYTES);
      }
      cp_async_commit();
    };
    // prologue: row maps of the tile, k maps of tiles 0..2, copies of tile 0 in flight, gathers of tile 0 loaded
    if (FillA::KLANE && tid < TC_BM) rowtabA[tid] = p.a.rows(m0 + tid);
    if (FillB::KLANE && tid < BN) rowtabB[tid] = p.b.rows(n0 + tid);
    for (int t = 0; t < 3; t++) stage_kmaps(t);
    if (NEED_KI || FillA::KLANE || FillB::KLANE) asm volatile("bar.sync 1, %0;" ::"n"(TC_PRODUCERS) : "memory");
    // register-path operands: loads of tile t into this thread's registers
    auto load_tile_regs = [&](int t) {
      if (t >= num_k_tiles) return;
      const long k0 = k_begin + (long)t * TC_BK;
      const int kb = (t % KRING) * TC_BK;
      if constexpr (FillA::REG) fa.load_regs(p.a, kiA + kb, rowtabA, k0, k_end, tid);
      if constexpr (FillB::REG) fb.load_regs(p.b, kiB + kb, rowtabB, k0, k_end, tid);
    };
    // asynchronous copies run LA tiles ahead of the tile being handed over
    constexpr int LA = STAGES - 1;
    for (int t = 0; t < LA; t++) issue_tile(t);
    load_tile_regs(0);
    for (int it = 0; it < num_k_tiles; it++) {
      const int s = it % STAGES;
      uint8_t *stage = smem + s * Cfg::STAGE_BYTES;
      // (1) gathered operands of tile `it`: round, store (the stage was awaited LA iterations ago, before tile
      //     `it`'s copies were issued), and start the loads of tile it+1 at once so that they fly during the rest
      if constexpr (FillA::REG) fa.store_regs(stage, stage + Cfg::A_BYTES, tid);
      if constexpr (FillB::REG) fb.store_regs(stage + 2 * Cfg::A_BYTES, stage + 2 * Cfg::A_BYTES + Cfg::B_BYTES, tid);
      load_tile_regs(it + 1);
      // (2) copies of tile `it` have landed (those of the next LA-1 tiles may still fly): split them in place
      //     where needed and hand the stage to the tensor core
      cp_async_wait<LA - 1>();
      if constexpr (!FillA::REG) fa.split(stage, stage + Cfg::A_BYTES, tid);
      if constexpr (!FillB::REG) fb.split(stage + 2 * Cfg::A_BYTES, stage + 2 * Cfg::A_BYTES + Cfg::B_BYTES, tid);
      fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_full + 8 * s);
      // (3) copies of tile it+LA into the stage that tile it-1 used, as soon as its MMAs have read it: the
      //     copy latency of a tile is hidden behind the MMAs of the LA tiles before it
      const int t = it + LA;
      bool mine = true;
      if (t < num_k_tiles && t >= STAGES) {
        const uint32_t phase = (uint32_t)(t / STAGES) & 1u;
        // warp-uniform, so that no lane leaves its warp behind at the next __syncwarp
        mine = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * (t % STAGES), phase ^ 1u, abort_flag));
      }
      if (!mine && !NEED_KI) { ok = false; break; }  // without a shared barrier a warp may leave on its own
      if (mine) issue_tile(t);
      else cp_async_commit();                          // keep the group count in step until the agreed stop
      // (4) publish the k maps of tile it+3; agree on whether to go on
      stage_kmaps(it + 3);
      if (NEED_KI) {
        if (tid == 0) cont[it & 1] = abort_flag->abort ? 0 : 1;
        asm volatile("bar.sync 1, %0;" ::"n"(TC_PRODUCERS) : "memory");
        if (!cont[it & 1]) { ok = false; break; }
      }
    }
    cp_async_wait<0>();
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      constexpr bool A_MN = P::OpA::MN_MAJOR, B_MN = P::OpB::MN_MAJOR;
      constexpr uint32_t idesc = umma_idesc_tf32(BN, A_MN, B_MN);
      for (int it = 0; it < num_k_tiles; it++) {
        const int s = it % STAGES, buf = it % NACC;
        const uint32_t phase = (uint32_t)(it / STAGES) & 1u, acc_phase = (uint32_t)(it / NACC) & 1u;
        ok = mbar_wait(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag) && mbar_wait(bar_full + 8 * s, phase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t a_hi = umma_desc_sw128<A_MN>(st), a_lo = umma_desc_sw128<A_MN>(st + Cfg::A_BYTES);
        const uint64_t b_hi = umma_desc_sw128<B_MN>(st + 2 * Cfg::A_BYTES),
                       b_lo = umma_desc_sw128<B_MN>(st + 2 * Cfg::A_BYTES + Cfg::B_BYTES);
        const uint32_t d = tmem_base + (uint32_t)(buf * BN);
        // Each k tile accumulates into a fresh TMEM buffer, small cross terms first; the drain warps
        // add the finished tile into FP32 registers with round-to-nearest.  The tensor core truncates
        // when it accumulates, so long chains in TMEM would drift; 12-MMA chains do not.
#pragma unroll
        for (int kk = 0; kk < TC_BK / 8; kk++) {  // 8 k per MMA: 32 bytes along a K-major row, 8 rows of an MN-major tile
          const uint64_t adv_a = (uint64_t)((kk * umma_kstep_bytes<A_MN>()) >> 4);
          const uint64_t adv_b = (uint64_t)((kk * umma_kstep_bytes<B_MN>()) >> 4);
          umma_tf32(d, a_lo + adv_a, b_hi + adv_b, idesc, kk ? 1u : 0u);
          umma_tf32(d, a_hi + adv_a, b_lo + adv_b, idesc, 1u);
        }
#pragma unroll
        for (int kk = 0; kk < TC_BK / 8; kk++) {
          const uint64_t adv_a = (uint64_t)((kk * umma_kstep_bytes<A_MN>()) >> 4);
          const uint64_t adv_b = (uint64_t)((kk * umma_kstep_bytes<B_MN>()) >> 4);
          umma_tf32(d, a_hi + adv_a, b_hi + adv_b, idesc, 1u);
        }
        umma_commit(bar_empty + 8 * s);       // the stage may be refilled once these MMAs have read it
        umma_commit(bar_acc_full + 8 * buf);  // and the tile's accumulator is complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ drain + epilogue warps
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int h = (warp - MMA_WARP - 1) >> 2;     // column half
    constexpr int NCOL = BN / 2;
    float acc[NCOL];
#pragma unroll
    for (int j = 0; j < NCOL; j++) acc[j] = 0.f;
    for (int it = 0; it < num_k_tiles; it++) {
      const int buf = it % NACC;
      const uint32_t acc_phase = (uint32_t)(it / NACC) & 1u;
      ok = mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < NCOL; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + h * NCOL + c0), v);
#pragma unroll
        for (int j = 0; j < 32; j++) acc[c0 + j] += __uint_as_float(v[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
    }
    if (ok) {
      const long m = m0 + q * 32 + lane;
      tc2_store_rows<P, NCOL>(p, acc, m, n0 + h * NCOL);
    }
  }
  if (abort_flag->abort && tid == 0) stall_raise(ctl, abort_flag->abort);
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, NACC * BN);
}

}  // namespace mm
}  // namespace thc

#endif
