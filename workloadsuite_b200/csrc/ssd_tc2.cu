// Two-head tensor-core SSD forward for sm_100a (the fast path when the heads of a
// group come in pairs).  One persistent CTA per SM walks work items (a run of
// 128-token tiles of one (batch, head pair) sequence) in order.
//
// The two heads of a pair read the same B and C (model_ref.py:97-99), so B, C and
// G = C.B^T (model_ref.py:143) are loaded/computed once per tile and shared.  The two
// heads' Xd tiles and 16-bit state copies lie one 64-column block apart in shared
// memory, so S = B^T.[Xd0|Xd1] and C.[H0|H1] are single N = 128 MMAs as well (an N = 64
// MMA occupies the tensor pipe as long as an N = 128 one).  Each head has its own
// compute warpgroup (one thread per tile row / TMEM lane).  Per head and tile k, in
// the order the warpgroup runs them inside one loop iteration:
//   a. H <- exp(cs_last) H + S(k)         (model_ref.py:150,156)   S = B^T.Xd from step c of the previous iteration
//   e. Y(k-1) -> global                    (:162)                   the P.X MMA of tile k-1 ran under step a
//   c. tile k+1: prefix sum (:135), Xd = exp(cs_last - cs_l) x~ (:144,148) -> smem -> S MMA; the rows of Xd are dealt
//      to the four warps unevenly (the row's scale goes through shared memory), the warps with fewer blocks of P in
//      step d taking more
//   d. P(k) = G o exp(segsum) o causal     (:139-145) -> TMEM as the A operand of Y += P.X
//   b. Y(k) <- exp(cs_l) * (C.H)           (:160-161) scaled in place in TMEM (the C.H MMA ran under steps c, d)
//      16-bit copy of H(k+1) -> smem for the next C.H MMA
// Warp 0 is the TMA producer, warp 1 issues the G MMAs, warp 2 the S and C.H MMAs,
// warp 3 the two heads' P.X MMAs (one thread each, blocking on the mbarriers in the
// order the warpgroups raise them); warps 4-7 and 8-11 are the compute warpgroups.
// tcgen05.mma holds its issuing thread for about as long as the MMA runs (77-160
// cycles per 128xNx16 step, depending on the operand layouts), which is why the three
// MMA streams have a thread each.  All waits are bounded.
#include <cuda.h>

#include <algorithm>
#include <type_traits>

#include "ssd_common.cuh"
#include "tc_common.cuh"
#include "tc_ptx.cuh"

namespace ssd {
namespace {

using namespace ptx;
using namespace tc;

constexpr int kThreads2 = 384;
constexpr int kSms = 148;
constexpr int kXStages = 3;   // X tiles in flight per head; a consumed stage doubles as the Y staging buffer

template <int N>
struct Layout2 {
  static constexpr int NB = N / 64;
  static constexpr int oB = 0;
  static constexpr int oC = oB + NB * kBlk;
  static constexpr int oX = oC + NB * kBlk;     // [head][stage], kXStages stages
  static constexpr int oXd = oX + 2 * kXStages * kBlk;   // [head]
  static constexpr int oH = oXd + 2 * kBlk;      // [head], N rows of 128 B
  static constexpr int oMisc = oH + 2 * N * 128;
  static constexpr int kBytes = oMisc + 3072;   // no slack: the dynamic segment must start 1024-byte aligned
};

// Work list of this CTA.
//  - Regular mode: items blockIdx.x, blockIdx.x + gridDim.x, ... of the (segment, sequence) grid.
//  - Chained mode (sp.chain == 1): all tiles of all sequences, laid end to end, are cut into gridDim.x equal
//    ranges, so every CTA gets the same number of tiles (+-1) whatever the number of sequences.  A range holds
//    the tail of one sequence, whole sequences and the head of another; they are walked in reverse, head first:
//    the head's state is what the next CTA's tail piece waits for, and a tail piece (walked last) then finds
//    the state it needs already there when there is at least one sequence per CTA.
//  - Look-back mode (sp.chain == 2), for fewer sequences than CTAs: the same even cut, but a piece cannot wait
//    for the full scan of the piece before it (the pieces of one sequence would run one after the other).
//    Instead every CTA first scans the LAST piece of its range from a zero state, state and log-decay sum only
//    (about 0.4 of the full work; item 0, skipped when that piece ends its sequence), and publishes the pair.
//    Then it walks its pieces like the chained mode; a piece that starts inside a sequence folds the published
//    pairs of the CTAs before it, back to the one that holds the sequence's first tile (the recurrence is linear:
//    H_in = sum_c exp(sum of the log-decays after c) F_c), and stops early once the decay factor has underflowed.
// Computed once per CTA (thread 0, into shared memory): the 64-bit divisions are bulky code.
struct Work {
  int count;
  int lo, hi, nt, pl;   // chained mode: global tile range, tiles per sequence, last sequence of the range
  int hp, hpg;          // head pairs per batch entry, heads per B/C group
  int pre;              // look-back mode: 1 when item 0 is the state-only scan of the range's last piece
  int ytot;             // tiles of all Y-producing items
};

struct Misc2 {
  Work work;
  uint64_t full_b, full_c, empty_b, empty_c;
  uint64_t full_x[2][kXStages], empty_x[2][kXStages];
  uint64_t bar_g;
  uint64_t bar_yo, bar_s, bar_y[2];   // tcgen05.commit arrivals (the S and C.H MMAs serve both heads at once)
  uint64_t bar_xd, bar_h, bar_e;      // one arrival per compute warp of either head (8)
  uint64_t bar_p[2];                  // one arrival per compute warp of the head (4)
  uint64_t bar_drain[3];              // give-up path: the MMAs of issuing warp 1 / 2 / 3 have all completed
  uint32_t tmem_base;
  long long wait_clocks;     // bound of every wait (SM clock cycles)
  volatile int abort_flag;   // 0, or the status code of the first wait that gave up (every role then leaves)
  float wsum[2][4];
  // Double-buffered by tile parity: step c writes the next tile's values while step d still reads this tile's.
  alignas(16) float cf[2][2][T];   // [head][parity][row]: exp(cs at the end of the row's 32-block - cs of the row)
  float cend[2][2][4];             // [head][parity][block]: cs * log2(e) at the end of each 32-row block
  uint16_t xs[2][T];               // [head][row]: the 16-bit scale exp(cs_last - cs_row) * dt of the row of X being turned into Xd
};

static_assert(sizeof(Misc2) <= 3072, "Misc2 outgrew its shared-memory slot");
static_assert(Layout2<128>::kBytes <= 232448, "shared memory budget of one SM exceeded");

struct Tc2Params {
  ScanParams sp;
  int nitems;   // (batch * nheads / 2) * nseg
  int upairs;   // batch * nheads / 2
};

// One work item: `ntiles` tiles of one (batch, head pair) sequence from token t_begin on.  in_slot / out_slot are
// the scratch slots the state is taken from / handed to when the item is an inner piece of a sequence that
// continues on a neighbouring CTA (-1: the sequence starts / ends here).
struct Item {
  int seg, bi, h0, gi, t_begin, ntiles, in_slot, out_slot;
  int yflag;      // this item produces Y (0: state and log-decay sum only)
  int fold_from;  // look-back mode: first CTA whose published pair enters the fold (-1: none), up to in_slot
  int ends_seq;   // the item holds the last tile of its sequence: it writes the caller's final state
};

__device__ __forceinline__ void work_list(const Tc2Params& prm, Work* out) {
  Work wk;
  wk.lo = wk.hi = wk.pl = 0;
  wk.nt = 1;
  wk.hp = prm.sp.nheads >> 1;
  wk.hpg = prm.sp.nheads / prm.sp.ngroups;
  if (prm.sp.chain) {
    wk.nt = prm.sp.seqlen / T;
    const long long total = (long long)prm.upairs * wk.nt;
    wk.lo = (int)((long long)blockIdx.x * total / gridDim.x);
    wk.hi = (int)((long long)(blockIdx.x + 1) * total / gridDim.x);
    wk.pl = wk.hi > wk.lo ? (wk.hi - 1) / wk.nt : 0;
    wk.count = wk.hi > wk.lo ? wk.pl - wk.lo / wk.nt + 1 : 0;
    wk.pre = (prm.sp.chain == 2 && wk.hi > wk.lo && wk.hi % wk.nt != 0) ? 1 : 0;
    wk.count += wk.pre;
  } else {
    wk.pre = 0;
    wk.count = (int)blockIdx.x < prm.nitems ? (prm.nitems - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  }
  wk.ytot = 0;
  *out = wk;
}

__device__ __forceinline__ Item work_item(const Tc2Params& prm, const Work& wk, int i) {
  const ScanParams& sp = prm.sp;
  Item it;
  int u2;
  it.yflag = sp.compute_y;
  it.fold_from = -1;
  it.ends_seq = 1;
  if (sp.chain) {
    const bool pre = wk.pre && i == 0;        // look-back mode: the state-only scan of the last piece
    u2 = wk.pl - (pre ? 0 : i - wk.pre);
    const int first = u2 * wk.nt, start = max(wk.lo, first), end = min(wk.hi, first + wk.nt);
    it.seg = 0;
    it.t_begin = (start - first) * T;
    it.ntiles = end - start;
    it.in_slot = start > first ? (int)blockIdx.x - 1 : -1;
    it.out_slot = end < first + wk.nt ? (int)blockIdx.x : -1;
    it.ends_seq = end == first + wk.nt;
    if (sp.chain == 2) {
      if (pre) {
        it.yflag = 0;
        it.in_slot = -1;                      // from a zero state
      } else {
        it.out_slot = -1;                     // only the state-only scan publishes
        if (it.in_slot >= 0) {
          // the CTA that holds the sequence's first tile: the largest c with lo(c) <= first
          const long long total = (long long)prm.upairs * wk.nt;
          int c = (int)((((long long)first + 1) * gridDim.x - 1) / total);
          while (c > 0 && (long long)c * total / gridDim.x > first) --c;
          while ((long long)(c + 1) * total / gridDim.x <= first) ++c;
          it.fold_from = c;
        }
      }
    }
  } else {
    const int item = blockIdx.x + i * gridDim.x;
    it.seg = item / prm.upairs;
    u2 = item - it.seg * prm.upairs;
    it.t_begin = it.seg * sp.seg_len;
    it.ntiles = (min(sp.seqlen, it.t_begin + sp.seg_len) - it.t_begin) / T;
    it.in_slot = it.out_slot = -1;
  }
  it.bi = u2 / wk.hp;
  it.h0 = 2 * (u2 - it.bi * wk.hp);
  it.gi = it.h0 / wk.hpg;
  return it;
}

// Bounded wait on an mbarrier phase; false when it gave up (or another role already had).
__device__ __forceinline__ bool wait2(uint64_t* bar, uint32_t parity, Misc2* m, int code, int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;   // the common case in steady state: no clock read, no sleep
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {   // (try_wait parks the thread for a short, hardware-chosen time by itself)
    if (m->abort_flag) return false;
    // (twice the bound of the wait for another CTA's hand-over: everything inside the CTA may be waiting behind
    //  that one, and the wait that is the cause should be the one that reports)
    if (clock64() - t0 > 2 * m->wait_clocks) {
      m->abort_flag = code;   // reported to the caller's status word at kernel end
      return false;
    }
  }
  return true;
}

// Last act of an MMA-issuing thread: tensor memory is freed at the end of the kernel, so the MMAs this thread
// has issued must have completed by then -- also when the roles that would have waited for them gave up
// (bounded, like every wait).
__device__ __forceinline__ void drain_mmas(Misc2* m, int which) {
  umma_commit(&m->bar_drain[which]);
  const long long t0 = clock64();
  while (!mbar_try_wait(&m->bar_drain[which], 0))
    if (clock64() - t0 > m->wait_clocks) break;
}


// EPI: apply the skip and gate of model_ref.py:116-118 to Y on its way out (sp.D / sp.Z; either may be null).
template <typename T16, int N, bool EPI>
__global__ void __launch_bounds__(kThreads2, 1)
ssd_tc2_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmY,
               const Tc2Params prm) {
  using L = Layout2<N>;
  constexpr int NB = L::NB;
  constexpr int KN = N / 16;
  constexpr int KT = T / 16;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  Misc2* m = reinterpret_cast<Misc2*>(smem + L::oMisc);
  const ScanParams& sp = prm.sp;
  if (smem_u32(smem) & 1023u) {   // the 128-byte swizzle needs 1024-byte aligned tiles; give up cleanly otherwise
    if (threadIdx.x == 0 && sp.status) atomicCAS(sp.status, 0, (int)STATUS_BAD_SMEM_ALIGNMENT);
    return;
  }
  // (fault injection for the tests of the give-up path: the first CTA of a chained launch never publishes its
  //  hand-over, so the CTA that continues its sequence runs into the bound of its wait)
  if (sp.inject_lost_handover && sp.chain && blockIdx.x == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool want_y = sp.compute_y != 0;
  int32_t* status = sp.status;

  if (tid == 0) {
    mbar_init(&m->full_b, 1); mbar_init(&m->full_c, 1);
    // B is released by the G MMA and the S MMA; C by the G MMA and the C.H MMA
    mbar_init(&m->empty_b, want_y ? 2 : 1); mbar_init(&m->empty_c, 2);   // (a state-only item inside a Y launch: the S issuer commits twice)
    mbar_init(&m->bar_g, 1);
    mbar_init(&m->bar_yo, 1); mbar_init(&m->bar_s, 1);
    mbar_init(&m->bar_xd, 8); mbar_init(&m->bar_h, 8); mbar_init(&m->bar_e, 8);
    for (int h = 0; h < 2; ++h) {
      // an X stage is handed back by the head's warpgroup once it is done with it (in Y mode: after the stage
      // has served as the source of the TMA store of Y)
      for (int s = 0; s < kXStages; ++s) {
        mbar_init(&m->full_x[h][s], 1);
        mbar_init(&m->empty_x[h][s], 4);   // Y items: the thread that issued the TMA store of Y arrives for all four
      }
      mbar_init(&m->bar_y[h], 1);
      mbar_init(&m->bar_p[h], 4);   // one arrival per compute warp (lane 0, after a warp barrier)
    }
    for (int i = 0; i < 3; ++i) mbar_init(&m->bar_drain[i], 1);
    m->abort_flag = 0;
    m->wait_clocks = sp.wait_clocks;
    work_list(prm, &m->work);
    for (int i = 0; i < m->work.count; ++i) {
      const Item wi = work_item(prm, m->work, i);
      if (wi.yflag) m->work.ytot += wi.ntiles;
    }
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&m->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = m->tmem_base;
  const uint32_t tG = tb;
  const uint32_t sB = smem_u32(smem + L::oB), sC = smem_u32(smem + L::oC), sX = smem_u32(smem + L::oX);
  const uint32_t sXd = smem_u32(smem + L::oXd), sH = smem_u32(smem + L::oH);

  if (warp < 4) {
    setmaxnreg_dec<72>();   // 128*72 + 256*216 = 384*168: the CTA can only re-divide its own allocation
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      prefetch_tmap(&tmX); prefetch_tmap(&tmB); prefetch_tmap(&tmC); prefetch_tmap(&tmY);
      bool ok = true;
      uint32_t it = 0;    // running tile ordinal of this CTA
      uint32_t ity = 0;   // ... counting the tiles of Y-producing items only (C is loaded for those)
      const Work wk = m->work;
      for (int wi = 0; wi < wk.count && ok; ++wi) {
        const Item w = work_item(prm, wk, wi);
        for (int j = 0; j < w.ntiles && ok; ++j, ++it) {
          const int t0 = w.t_begin + j * T;
          const uint32_t st = it % kXStages, use = it / kXStages;
          for (int h = 0; h < 2 && ok; ++h) {
            if (use > 0) ok = wait2(&m->empty_x[h][st], (use - 1) & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
            if (!ok) break;
            mbar_expect_tx(&m->full_x[h][st], kBlk);
            tma_load_4d(smem + L::oX + (kXStages * h + st) * kBlk, &tmX, &m->full_x[h][st], 0, w.h0 + h, t0, w.bi);
          }
          if (!ok) break;
          // B before C: the B tile is free as soon as the previous tile's G and S MMAs are done, the C tile only once
          // its C.H MMA is, which waits for the read-out of the tile before; the S MMA of this tile must not wait that long.
          if (it > 0) ok = wait2(&m->empty_b, (it - 1) & 1, m, STATUS_WAIT_TIMEOUT_MMA, status);
          if (!ok) break;
          mbar_expect_tx(&m->full_b, NB * kBlk);
#pragma unroll
          for (int kb = 0; kb < NB; ++kb)
            tma_load_4d(smem + L::oB + kb * kBlk, &tmB, &m->full_b, 64 * kb, w.gi, t0, w.bi);
          if (!ok) break;
          if (w.yflag) {
            if (ity > 0) ok = wait2(&m->empty_c, (ity - 1) & 1, m, STATUS_WAIT_TIMEOUT_MMA, status);
            if (!ok) break;
            mbar_expect_tx(&m->full_c, NB * kBlk);
#pragma unroll
            for (int kb = 0; kb < NB; ++kb)
              tma_load_4d(smem + L::oC + kb * kBlk, &tmC, &m->full_c, 64 * kb, w.gi, t0, w.bi);
            ++ity;
          }
        }
      }
      if (m->abort_flag && it > 0) {
        // let copies already in flight land before the CTA gives its shared memory back
        const uint32_t k = it - 1;
        const long long c0 = clock64();
        while (clock64() - c0 < 2000000LL) {
          const uint32_t xs = k % kXStages, xp = (k / kXStages) & 1;
          if (mbar_try_wait(&m->full_b, k & 1) && mbar_try_wait(&m->full_x[0][xs], xp) &&
              mbar_try_wait(&m->full_x[1][xs], xp) && (ity == 0 || mbar_try_wait(&m->full_c, (ity - 1) & 1)))
            break;
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer for G = C.B^T (shared by the heads)
      if (want_y) {
        constexpr int fmt = std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
        constexpr uint32_t idG = umma_idesc(128, 128, fmt, 0, 0);
        constexpr uint64_t dK = umma_desc_base(16, 1024);
        const Work wk = m->work;
        bool ok = true;
        uint32_t it = 0, k = 0;   // tile ordinal over all items / over the Y-producing ones
        for (int wi = 0; wi < wk.count && ok; ++wi) {
          const Item w = work_item(prm, wk, wi);
          if (!w.yflag) { it += w.ntiles; continue; }
        for (int j = 0; j < w.ntiles && ok; ++j, ++it, ++k) {
          // both heads are done reading G(k-1); B and C of tile k have landed
          if (k > 0)
            ok = wait2(&m->bar_p[0], (k - 1) & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status) &&
                 wait2(&m->bar_p[1], (k - 1) & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
          ok = ok && wait2(&m->full_c, k & 1, m, STATUS_WAIT_TIMEOUT_TMA, status) &&
               wait2(&m->full_b, it & 1, m, STATUS_WAIT_TIMEOUT_TMA, status);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < KN; ++kk) {
            const uint32_t off = (kk >> 2) * kBlk + (kk & 3) * 32;
            umma_ss(tG, umma_desc(dK, sC + off), umma_desc(dK, sB + off), idG, kk > 0);
          }
          umma_commit(&m->bar_g);
          umma_commit(&m->empty_c);
          umma_commit(&m->empty_b);
        }
        }
      }
      drain_mmas(m, 0);
    } else if (warp == 2 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer for S = B^T.[Xd0|Xd1] and Y = C.[H0|H1]
      // The two heads' Xd (and state copies) lie one 64-column block apart in shared memory, so one
      // N = 128 MMA serves both heads; it costs the tensor pipe what the N = 64 one does.
      constexpr int fmt = std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idKM = umma_idesc(128, 128, fmt, 0, 1);
      constexpr uint32_t idMM = umma_idesc(128, 128, fmt, 1, 1);
      constexpr uint64_t dK = umma_desc_base(16, 1024);
      constexpr uint64_t dMN = umma_desc_base(kBlk, 1024);       // B tile; [Xd0|Xd1]
      constexpr uint64_t dMNh = umma_desc_base(N * 128, 1024);   // [H0|H1]
      const uint32_t tS = tb + 128, tY = tb + 256;
      bool ok = true;
      uint32_t k0 = 0;   // running tile ordinal of the item's first tile
      uint32_t ky = 0;   // tile ordinal over the Y-producing items
      const Work wk = m->work;
      for (int wi = 0; wi < wk.count && ok; ++wi) {
        const Item w = work_item(prm, wk, wi);
        const int nt = w.ntiles;
#pragma unroll 1
        for (int j = 0; j < nt && ok; ++j) {
          const uint32_t k = k0 + j;
          // S <- B^T . Xd
          ok = wait2(&m->full_b, k & 1, m, STATUS_WAIT_TIMEOUT_TMA, status) &&
               wait2(&m->bar_xd, k & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < KT; ++kk)
            umma_ss(tS, umma_desc(dMN, sB + kk * 2048), umma_desc(dMN, sXd + kk * 2048), idMM, kk > 0);
          umma_commit(&m->bar_s);
          umma_commit(&m->empty_b);
          if (!w.yflag) {
            // (a state-only item inside a Y launch: no G MMA reads this B tile, its arrival is made here)
            if (want_y) umma_commit(&m->empty_b);
            continue;
          }
          // Y <- C . H
          ok = wait2(&m->full_c, ky & 1, m, STATUS_WAIT_TIMEOUT_TMA, status) &&
               wait2(&m->bar_h, ky & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
          if (ok && ky > 0) ok = wait2(&m->bar_e, (ky - 1) & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
          if (!ok) break;
          ++ky;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < KN; ++kk) {
            const uint32_t off = (kk >> 2) * kBlk + (kk & 3) * 32;
            umma_ss(tY, umma_desc(dK, sC + off), umma_desc(dMNh, sH + kk * 2048), idKM, kk > 0);
          }
          umma_commit(&m->bar_yo);
          umma_commit(&m->empty_c);
        }
        k0 += nt;
      }
      drain_mmas(m, 1);
    } else if (warp == 3 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer for Y_h += P_h . X_h, head 0 then head 1
      if (want_y) {
        constexpr int fmt = std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
        constexpr uint32_t idKM = umma_idesc(128, 64, fmt, 0, 1);
        constexpr uint64_t dMN = umma_desc_base(kBlk, 1024);
        const Work wk = m->work;
        bool ok = true;
        uint32_t it = 0, k = 0;   // tile ordinal over all items / over the Y-producing ones
        for (int wi = 0; wi < wk.count && ok; ++wi) {
          const Item w = work_item(prm, wk, wi);
          if (!w.yflag) { it += w.ntiles; continue; }
#pragma unroll 1
        for (int j = 0; j < w.ntiles && ok; ++j, ++it, ++k) {
          const uint32_t st = it % kXStages;
#pragma unroll 1
          for (int h = 0; h < 2 && ok; ++h) {
            ok = wait2(&m->bar_p[h], k & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status) &&
                 wait2(&m->full_x[h][st], (it / kXStages) & 1, m, STATUS_WAIT_TIMEOUT_TMA, status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tY = tb + 256 + 64 * h, tP = tb + 384 + 64 * h;
#pragma unroll
            for (int kk = 0; kk < KT; ++kk)
              umma_ts(tY, tP + 8 * kk, umma_desc(dMN, sX + (kXStages * h + st) * kBlk + kk * 2048), idKM, 1);
            umma_commit(&m->bar_y[h]);
          }
        }
        }
      }
      drain_mmas(m, 2);
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups (warps 4-7: head 0, 8-11: head 1)
    setmaxnreg_inc<216>();
    const int h = (warp - 4) >> 2;
    const int lane_base = (warp & 3) * 32;
    const int l = lane_base + lane;
    const int q = warp & 3;
    const uint32_t tlane = (uint32_t)lane_base << 16;
    const uint32_t swz = (uint32_t)(l & 7);
    const bool owns_state = lane_base < N;
    const uint32_t tS = tb + 128 + 64 * h, tY = tb + 256 + 64 * h, tP = tb + 384 + 64 * h;
    const uint32_t sHh = sH + h * (N * 128), sXdh = sXd + h * kBlk;
    const int bar_id = 1 + h;

    uint32_t it = 0;    // running tile ordinal of this CTA
    uint32_t ity = 0;   // ... counting the tiles of Y-producing items only
    bool ok = true;
    auto cwait = [&](uint64_t* bar, uint32_t parity, int code) {
      return __all_sync(0xffffffffu, wait2(bar, parity, m, code, status)) != 0;
    };
    // One arrival per warp: every lane has issued its fences, the warp barrier orders their writes before
    // lane 0's arrive (128 per-thread arrivals on one mbarrier cost several hundred cycles per hand-off).
    auto warp_arrive = [&](uint64_t* bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };

    float H[P];
    float cs = 0.f, tot = 0.f, cs2 = 0.f;   // of the tile whose P / Y is being produced
    // dt multiplies the columns of P instead of the rows of X (P.(dt o x) = (P o dt_s).x), so the X tile stays as
    // loaded: this row's value as a column of the diagonal mask block is cs2 - log2(dt) (clamped: dt == 0 must not
    // break the chain of per-token factors there; the clamped column then weighs 2^-60, i.e. nothing).
    float cs2c = 0.f;
    // log-decay / dt of this thread's row in the next tile to be scanned.  dt stays as loaded (16 bits) until the scan uses
    // it one iteration later: a conversion right behind the load would hold the warp for the whole memory latency.
    float a_next = 0.f;
    T16 dt_next = Cvt<T16>::from_f(1.f);
    bool next_prefetched = false;
    bool store_pending = false;    // (thread l == 0) a TMA store of Y is in flight from X stage store_stage
    uint32_t store_stage = 0;
    float asum = 0.f, acomp = 0.f;   // compensated (Kahan) sum of the tile totals; FP64 is slow on this part

    // prefix sum of the log-decay over the 128 rows (model_ref.py:135); publishes cs*log2(e) for the P step
    auto scan_tile = [&](float a, float dtv, uint32_t par, float& cs_o, float& tot_o, float& cs2_o,
                         float& cs2c_o) {
      float v = a;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += t;
      }
      if (lane == 31) m->wsum[h][q] = v;
      named_bar_sync(bar_id, 128);
      const float w0 = m->wsum[h][0], w1 = m->wsum[h][1], w2 = m->wsum[h][2], w3 = m->wsum[h][3];
      cs_o = v + ((q > 0 ? w0 : 0.f) + (q > 1 ? w1 : 0.f) + (q > 2 ? w2 : 0.f));
      tot_o = (w0 + w1 + w2) + w3;
      cs2_o = cs_o * kLog2e;
      // column factor of the factored decay mask: exp(cs at the end of this row's 32-token block - cs_row)
      // (times dt of the row: the factor belongs to the row as a column of P)
      m->cf[h][par][l] = ex2(__shfl_sync(0xffffffffu, cs2_o, 31) - cs2_o) * dtv;
      cs2c_o = cs2_o - fmaxf(__log2f(dtv), -60.f);
      if (lane == 31) m->cend[h][par][q] = cs2_o;
      // the row's scale for Xd (model_ref.py:144,148), for whichever thread turns that row of X into Xd
      m->xs[h][l] = (uint16_t)pack2<T16>(ex2((tot_o - cs_o) * kLog2e) * dtv, 0.f);
      named_bar_sync(bar_id, 128);
    };
    // Xd = exp(cs_last - cs_l) * dt * x (model_ref.py:144,148) from X stage `st` into this head's Xd buffer, in packed
    // 16-bit arithmetic as the reference does it.  The rows are not dealt out evenly: the mask step that follows gives
    // warp q (rows 32q..32q+31 of the causal P) q + 1 blocks of 32 columns to fill, and the four warps meet at the next
    // tile's prefix sum, so the warps with fewer mask blocks take more rows here.  Eight lanes share a row (one 16-byte
    // piece each), a warp moves four rows per instruction ("a quad": 32 quads per tile).
    auto make_xd = [&](uint32_t st, bool with_mask) {
      // first quad of warp 0..3 and the end, one byte each: 0 14 24 30 32 when all four warps also update and copy the
      // state (N = 128), 0 10 18 26 32 when only warps 0 and 1 do
      constexpr uint64_t kFirst = N == 128 ? 0x201E180E00ull : 0x201A120A00ull;
      const int qb = with_mask ? (int)((kFirst >> (8 * q)) & 0xff) : 8 * q;
      const int qe = with_mask ? (int)((kFirst >> (8 * q + 8)) & 0xff) : 8 * q + 8;
      const uint32_t xb = sX + (kXStages * h + st) * kBlk;
      const uint32_t sub = (uint32_t)lane >> 3, pc = (uint32_t)lane & 7u;
#pragma unroll 1
      for (int qd = qb; qd < qe; qd += 2) {   // (every share is an even number of quads)
        const uint32_t r0 = 4 * qd + sub, r1 = r0 + 4;
        const uint32_t o0 = r0 * 128 + ((pc ^ (r0 & 7u)) << 4), o1 = r1 * 128 + ((pc ^ (r1 & 7u)) << 4);
        const uint4 a0 = lds128(xb + o0), a1 = lds128(xb + o1);
        const uint32_t s0 = m->xs[h][r0], s1 = m->xs[h][r1];
        const uint32_t d0 = s0 | (s0 << 16), d1 = s1 | (s1 << 16);
        uint4 v;
        v.x = mul2<T16>(a0.x, d0); v.y = mul2<T16>(a0.y, d0); v.z = mul2<T16>(a0.z, d0); v.w = mul2<T16>(a0.w, d0);
        sts128(sXdh + o0, v);
        v.x = mul2<T16>(a1.x, d1); v.y = mul2<T16>(a1.y, d1); v.z = mul2<T16>(a1.z, d1); v.w = mul2<T16>(a1.w, d1);
        sts128(sXdh + o1, v);
      }
    };
    auto store_hb = [&]() {
      if (owns_state) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 v;
          v.x = pack2<T16>(H[8 * c + 0], H[8 * c + 1]); v.y = pack2<T16>(H[8 * c + 2], H[8 * c + 3]);
          v.z = pack2<T16>(H[8 * c + 4], H[8 * c + 5]); v.w = pack2<T16>(H[8 * c + 6], H[8 * c + 7]);
          sts128(sHh + l * 128 + ((c ^ swz) << 4), v);
        }
      }
    };

    // ---- e. Y -> global, for the tile whose P.X MMA was started one step earlier (its latency is spent in the
    //      next tile's state update).  Returns false when a wait gave up.
    bool y_pending = false;
    uint32_t y_it = 0, y_ity = 0;
    int y_hi = 0, y_t0 = 0, y_bi = 0;
    float y_dskip = 0.f;   // (EPI) D of the head whose tile is queued: loaded when the tile is queued, used a tile later
    auto finish_y = [&]() -> bool {
      // (EPI) the gate rows of this warp's 32 tokens, fetched ahead of the wait for the MMA.  Eight lanes read one
      // 128-byte row per load (whole lines), four rows per instruction; the rows reach their threads through the
      // staging buffer below.
      uint4 zr[8];
      if constexpr (EPI) {
        if (sp.Z) {
          const T16* zbase = static_cast<const T16*>(sp.Z) + y_bi * sp.zs[0] + y_hi * sp.zs[2] + 8 * (lane & 7);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int row = lane_base + 4 * i + (lane >> 3);
            zr[i] = __ldg(reinterpret_cast<const uint4*>(zbase + (int64_t)(y_t0 + row) * sp.zs[1]));
          }
          // the next tile's gate rows as far as L2 (one row per lane), so that the loads above find them there
          if (y_t0 + T + lane_base + lane < sp.seqlen)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const T16*>(sp.Z) + y_bi * sp.zs[0] + y_hi * sp.zs[2] +
                                                         (int64_t)(y_t0 + T + lane_base + lane) * sp.zs[1]));
        }
      }
      if (!cwait(&m->bar_y[h], y_ity & 1, STATUS_WAIT_TIMEOUT_MMA)) return false;
      tc_fence_after();
      // The X stage of that tile is dead (its P.X MMA is complete): stage the 16-bit Y rows there; one
      // thread then hands the whole tile to the TMA engine.
      const uint32_t xst = y_it % kXStages;
      const uint32_t ystage = sX + (kXStages * h + xst) * kBlk;
      {
        uint32_t y0[32], y1[32];
        tmem_ld32(tY + tlane, y0);
        tmem_ld32(tY + tlane + 32, y1);
        tmem_ld_wait();
        tc_fence_before();
        warp_arrive(&m->bar_e);   // the Y accumulator is read out: the next tile's C.H may overwrite it
        if constexpr (EPI) {
          // Y <- (Y + x * D) * silu(z) (model_ref.py:116-118) in fp32; x is this thread's row of the X tile, still in
          // the stage that the Y rows go to; silu(z) = z * (0.5 + 0.5 tanh(z / 2)), the tanh on 16-bit pairs.
          const bool gate = sp.Z != nullptr;
          if (sp.D) {
            const float dskip = y_dskip;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint4 xr = lds128(ystage + l * 128 + ((c ^ swz) << 4));
              const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint32_t* yy = (c < 4) ? &y0[8 * c + 2 * e] : &y1[8 * (c - 4) + 2 * e];
                const float2 xf = unpack2<T16>(xw[e]);
                yy[0] = __float_as_uint(fmaf(xf.x, dskip, __uint_as_float(yy[0])));
                yy[1] = __float_as_uint(fmaf(xf.y, dskip, __uint_as_float(yy[1])));
              }
            }
          }
          if (gate) {
            // x is consumed: the warp's gate rows go through its 32 rows of the stage to the threads that own them
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = lane_base + 4 * i + (lane >> 3);
              sts128(ystage + row * 128 + ((((uint32_t)lane & 7u) ^ ((uint32_t)row & 7u)) << 4), zr[i]);
            }
            __syncwarp();
            const uint32_t half2 = pack2<T16>(0.5f, 0.5f);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint4 zq = lds128(ystage + l * 128 + ((c ^ swz) << 4));
              const uint32_t zw[4] = {zq.x, zq.y, zq.z, zq.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint32_t* yy = (c < 4) ? &y0[8 * c + 2 * e] : &y1[8 * (c - 4) + 2 * e];
                // silu(z) = z * (0.5 + 0.5 tanh(z / 2)) on the packed 16-bit pair, as the reference forms it in
                // half precision (model_ref.py:118); the product with Y is taken in fp32
                const uint32_t sg = fma2<T16>(tanh2<T16>(mul2<T16>(zw[e], half2)), half2, half2);
                const float2 gf = unpack2<T16>(mul2<T16>(zw[e], sg));
                yy[0] = __float_as_uint(__uint_as_float(yy[0]) * gf.x);
                yy[1] = __float_as_uint(__uint_as_float(yy[1]) * gf.y);
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 o;
          o.x = pack2<T16>(__uint_as_float(y0[8 * c + 0]), __uint_as_float(y0[8 * c + 1]));
          o.y = pack2<T16>(__uint_as_float(y0[8 * c + 2]), __uint_as_float(y0[8 * c + 3]));
          o.z = pack2<T16>(__uint_as_float(y0[8 * c + 4]), __uint_as_float(y0[8 * c + 5]));
          o.w = pack2<T16>(__uint_as_float(y0[8 * c + 6]), __uint_as_float(y0[8 * c + 7]));
          sts128(ystage + l * 128 + ((c ^ swz) << 4), o);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 o;
          o.x = pack2<T16>(__uint_as_float(y1[8 * c + 0]), __uint_as_float(y1[8 * c + 1]));
          o.y = pack2<T16>(__uint_as_float(y1[8 * c + 2]), __uint_as_float(y1[8 * c + 3]));
          o.z = pack2<T16>(__uint_as_float(y1[8 * c + 4]), __uint_as_float(y1[8 * c + 5]));
          o.w = pack2<T16>(__uint_as_float(y1[8 * c + 6]), __uint_as_float(y1[8 * c + 7]));
          sts128(ystage + l * 128 + (((4 + c) ^ swz) << 4), o);
        }
      }
      fence_proxy_async();         // staged rows -> visible to the TMA engine
      named_bar_sync(bar_id, 128);
      if (l == 0) {
        // The previous store must be done reading its stage before the producer may refill it.
        if (store_pending) {
          bulk_wait_read_all();
          mbar_arrive_n(&m->empty_x[h][store_stage], 4);
        }
        tma_store_4d(&tmY, ystage, 0, y_hi, y_t0, y_bi);
        bulk_commit();
        store_pending = true;
        store_stage = xst;
      }
      y_pending = false;
      return true;
    };

    const Work wk = m->work;
    // (one pass more than there are items: an empty item whose only iteration reads out the last Y tile, so that
    //  the read-out code exists once)
    for (int wi = 0; wi <= wk.count && ok; ++wi) {
      Item w = {};
      if (wi < wk.count) w = work_item(prm, wk, wi);
      if (w.ntiles == 0 && wi < wk.count) continue;
      const int hi = w.h0 + h;
      const bool wy = w.yflag != 0;   // this item produces Y (a look-back launch starts with a state-only item)
      const int64_t unit = (int64_t)w.bi * sp.nheads + hi;
      const float* Ag = sp.A + w.bi * sp.as[0] + hi * sp.as[2];
      const T16* Dg = sp.dt ? static_cast<const T16*>(sp.dt) + w.bi * sp.dts[0] + hi * sp.dts[2] : nullptr;

      float asum0 = 0.f;   // log-decay summed over the earlier segments of a chained sequence
      asum = 0.f;
      acomp = 0.f;
      if (!next_prefetched && w.ntiles > 0) {   // (the first item of this CTA; later items were prefetched during their predecessor)
        a_next = Ag[(int64_t)(w.t_begin + l) * sp.as[1]];
        dt_next = Dg ? Dg[(int64_t)(w.t_begin + l) * sp.dts[1]] : Cvt<T16>::from_f(1.f);
      }
      next_prefetched = false;

      // Iteration j = -1 only prepares tile 0 (state copy, prefix sum, Xd); iteration j >= 0 finishes
      // tile j (steps a, b, d, e) and prepares tile j + 1 (step c) in between, so that the S MMA of the
      // next tile runs under steps d and e.  One copy of each step keeps the loop inside the
      // instruction cache.
#pragma unroll 1
      for (int j = -1; j < w.ntiles && ok; ++j) {
        const int t0 = w.t_begin + j * T;
        const bool have_next = (j + 1 < w.ntiles);
        if (j >= 0) {
          // ---- a. state: H <- exp(cs_last) H + S
          ok = cwait(&m->bar_s, it & 1, STATUS_WAIT_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          {
            const float yk = tot - acomp, tk = asum + yk;
            acomp = (tk - asum) - yk;
            asum = tk;
          }
          if (owns_state) {
            const float g = ex2(tot * kLog2e);
            uint32_t sv0[32], sv1[32];
            tmem_ld32(tS + tlane, sv0);
            tmem_ld32(tS + tlane + 32, sv1);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) H[e] = fmaf(H[e], g, __uint_as_float(sv0[e]));
#pragma unroll
            for (int e = 0; e < 32; ++e) H[32 + e] = fmaf(H[32 + e], g, __uint_as_float(sv1[e]));
          }
        }
        // ---- state leaving the item: it is final once the last tile's update (step a) is done, so it is
        //      handed over here, ahead of the rest of that tile; the next item's first log-decays are fetched too
        if (j >= 0 && !have_next) {
          const bool hand_over = w.out_slot >= 0;
          if (hand_over) {
            const int64_t slot = 2 * w.out_slot + h;
            if (owns_state) {
              float4* F = reinterpret_cast<float4*>(sp.chain_state + slot * (int64_t)(N * P) + (int64_t)l * P);
    #pragma unroll
              for (int j = 0; j < P / 4; ++j) F[j] = make_float4(H[4 * j], H[4 * j + 1], H[4 * j + 2], H[4 * j + 3]);
            }
            if (l == 0) sp.chain_ld[slot] = asum0 + asum;
            // Each warp publishes its own rows: a release-add by lane 0 after a warp barrier orders the
            // whole warp's stores before the count, and nobody has to wait for the stores to land.
            __syncwarp();
            if (lane == 0) {
              const int one = 1;
              asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(sp.chain_flag + slot), "r"(one) : "memory");
            }
          } else if (w.ends_seq) {
            // last (or only) segment of the sequence: the caller's outputs
            const int fseg = sp.chain ? 0 : w.seg;
            if (sp.fin && owns_state) {
              float4* F = reinterpret_cast<float4*>(sp.fin + unit * sp.fin_unit_stride + fseg * sp.fin_seg_stride +
                                                    (int64_t)l * P);
    #pragma unroll
              for (int j = 0; j < P / 4; ++j) F[j] = make_float4(H[4 * j], H[4 * j + 1], H[4 * j + 2], H[4 * j + 3]);
            }
            if (sp.fin_ld && l == 0)
              sp.fin_ld[unit * sp.finld_unit_stride + fseg * sp.finld_seg_stride] = asum0 + asum;
          }
          if (wi + 1 < wk.count) {
            const Item wn = work_item(prm, wk, wi + 1);
            if (wn.ntiles > 0) {
              const int hn = wn.h0 + h;
              a_next = sp.A[wn.bi * sp.as[0] + hn * sp.as[2] + (int64_t)(wn.t_begin + l) * sp.as[1]];
              if (sp.dt)
                dt_next = static_cast<const T16*>(sp.dt)[wn.bi * sp.dts[0] + hn * sp.dts[2] +
                                                          (int64_t)(wn.t_begin + l) * sp.dts[1]];
              next_prefetched = true;
            }
          }
        }
        if (y_pending) {   // (j == -1: the previous item's last tile)
          ok = finish_y();
          if (!ok) break;
        }
        // ---- c. next tile: prefix sum and Xd (the S MMA that read the Xd buffer was waited for in step a)
        float cs_n = 0.f, tot_n = 0.f, cs2_n = 0.f, cs2c_n = 0.f;
        if (have_next) {
          const uint32_t itn = (j >= 0) ? it + 1 : it;
          const float a = a_next, dtv = Cvt<T16>::to_f(dt_next);
          if (j + 2 < w.ntiles) {
            a_next = Ag[(int64_t)(t0 + 2 * T + l) * sp.as[1]];
            if (Dg) dt_next = Dg[(int64_t)(t0 + 2 * T + l) * sp.dts[1]];
          }
          scan_tile(a, dtv, itn & 1, cs_n, tot_n, cs2_n, cs2c_n);
          ok = cwait(&m->full_x[h][itn % kXStages], (itn / kXStages) & 1, STATUS_WAIT_TIMEOUT_TMA);
          if (!ok) break;
          make_xd(itn % kXStages, wy);
          fence_proxy_async();
          warp_arrive(&m->bar_xd);
          if (!wy) warp_arrive(&m->empty_x[h][itn % kXStages]);   // nothing else reads X of a state-only item
        }
        // ---- state entering the item (after the first tile's Xd is on its way to the S MMA: the wait for a
        //      chained predecessor and the state load then overlap that MMA)
        if (j == -1 && w.ntiles > 0) {
          if (w.in_slot >= 0 && sp.chain == 2) {
            // Look-back: fold the pairs (state from zero, log-decay sum) that the CTAs fold_from..in_slot published
            // for their pieces of this sequence, newest first: H_in = sum_c exp(log-decay after c) F_c (+ the same
            // for the caller's initial state).  Wait (bounded) until all of them are there.
            if (l == 0) {
              const long long c0 = clock64();
              for (int c = w.in_slot; c >= w.fold_from && !m->abort_flag; --c) {
                while (true) {
                  int f;
                  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(sp.chain_flag + 2 * c + h) : "memory");
                  if (f >= 4) break;   // all four warps of that CTA's warpgroup have published
                  if (m->abort_flag) break;
                  if (clock64() - c0 > m->wait_clocks) {
                    m->abort_flag = (int)STATUS_WAIT_TIMEOUT_CHAIN;
                    break;
                  }
                }
              }
            }
            named_bar_sync(bar_id, 128);
            if (m->abort_flag) { ok = false; break; }
#pragma unroll
            for (int e = 0; e < P; ++e) H[e] = 0.f;
            float dsum = 0.f;   // log-decay between the end of the piece being added and the start of this one
            for (int c = w.in_slot; c >= w.fold_from; --c) {
              const int64_t slot = 2 * c + h;
              const float wgt = ex2(dsum * kLog2e);
              if (owns_state && wgt != 0.f) {   // (a piece whose weight has underflowed adds nothing)
                const float4* I = reinterpret_cast<const float4*>(sp.chain_state + slot * (int64_t)(N * P) + (int64_t)l * P);
#pragma unroll
                for (int e = 0; e < P / 4; ++e) {
                  const float4 v = __ldcg(I + e);   // written by another SM: bypass L1
                  H[4 * e] = fmaf(wgt, v.x, H[4 * e]); H[4 * e + 1] = fmaf(wgt, v.y, H[4 * e + 1]);
                  H[4 * e + 2] = fmaf(wgt, v.z, H[4 * e + 2]); H[4 * e + 3] = fmaf(wgt, v.w, H[4 * e + 3]);
                }
              }
              dsum += __ldcg(sp.chain_ld + slot);
            }
            if (sp.init && owns_state) {
              const float wgt = ex2(dsum * kLog2e);
              const float4* I = reinterpret_cast<const float4*>(sp.init + unit * sp.init_unit_stride + (int64_t)l * P);
#pragma unroll
              for (int e = 0; e < P / 4; ++e) {
                const float4 v = I[e];
                H[4 * e] = fmaf(wgt, v.x, H[4 * e]); H[4 * e + 1] = fmaf(wgt, v.y, H[4 * e + 1]);
                H[4 * e + 2] = fmaf(wgt, v.z, H[4 * e + 2]); H[4 * e + 3] = fmaf(wgt, v.w, H[4 * e + 3]);
              }
            }
            asum0 = dsum;
          } else if (w.in_slot >= 0) {
            // wait (bounded) for the previous segment of this unit, which another CTA may still be finishing
            const int64_t slot = 2 * w.in_slot + h;
            if (l == 0) {
              const long long c0 = clock64();
              while (true) {
                int f;
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(sp.chain_flag + slot) : "memory");
                if (f >= 4) break;   // all four warps of the predecessor's warpgroup have published
                if (m->abort_flag) break;
                if (clock64() - c0 > m->wait_clocks) {
                  m->abort_flag = (int)STATUS_WAIT_TIMEOUT_CHAIN;
                  break;
                }
              }
            }
            named_bar_sync(bar_id, 128);
            if (m->abort_flag) { ok = false; break; }
            if (owns_state) {
              const float4* I = reinterpret_cast<const float4*>(sp.chain_state + slot * (int64_t)(N * P) + (int64_t)l * P);
    #pragma unroll
              for (int j = 0; j < P / 4; ++j) {
                const float4 v = __ldcg(I + j);   // written by another SM: bypass L1
                H[4 * j] = v.x; H[4 * j + 1] = v.y; H[4 * j + 2] = v.z; H[4 * j + 3] = v.w;
              }
            } else {
    #pragma unroll
              for (int j = 0; j < P; ++j) H[j] = 0.f;
            }
            asum0 = __ldcg(sp.chain_ld + slot);
          } else if (sp.init && owns_state && !(sp.chain == 2 && !wy)) {   // (the look-back scan starts from zero)
            const float4* I = reinterpret_cast<const float4*>(sp.init + unit * sp.init_unit_stride +
                                                              w.seg * sp.init_seg_stride + (int64_t)l * P);
    #pragma unroll
            for (int j = 0; j < P / 4; ++j) {
              const float4 v = I[j];
              H[4 * j] = v.x; H[4 * j + 1] = v.y; H[4 * j + 2] = v.z; H[4 * j + 3] = v.w;
            }
          } else {
    #pragma unroll
            for (int j = 0; j < P; ++j) H[j] = 0.f;
          }
        }
        if (l == 0 && store_pending) {
          // the Y store issued in the previous tile's step e has finished reading its stage by now: hand it back
          bulk_wait_read_all();
          mbar_arrive_n(&m->empty_x[h][store_stage], 4);
          store_pending = false;
        }
        if (j >= 0) {
          if (wy) {
            // ---- d. P = (C B^T) o exp(segsum), causal -> TMEM (A operand, 16-bit pairs)
            ok = cwait(&m->bar_g, ity & 1, STATUS_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            const uint32_t par = it & 1;
            // Decay mask per 32-token column block J of this warp's 32 rows (block q is the diagonal one):
            //   J == q: exp2(cs_l - cs_s), causal, one ex2 per element;
            //   J <  q: exp(cs_l - cs_s) = rf_J[l] * cf[s] with both factors <= 1 for non-positive
            //           log-decays (rf_J[l] = exp(cs_l - cs_end(J)), cf[s] = exp(cs_end(J) - cs_s)): two multiplies;
            //   J >  q: zero, written once (nothing else ever writes those TMEM columns).
            {
              // diagonal block first: its TMEM load is in flight while the factors are fetched
              uint32_t gd[32];
              tmem_ld32(tG + tlane + 32 * q, gd);
              tmem_ld_wait();
              // One ex2 per four columns: exp(cs_l - cs_{s+1}) = exp(cs_l - cs_s) * exp(-a_{s+1}), the per-token
              // factor exp(-a) coming from the lane that owns the row (clamped: an entry above the diagonal may
              // overflow, it is masked out by a select, never multiplied into anything that is kept).
              const float einv = ex2(fminf(__shfl_up_sync(0xffffffffu, cs2c, 1) - cs2c, 126.f));
              uint32_t pk[16];
#pragma unroll
              for (int e4 = 0; e4 < 8; ++e4) {
                const float c0 = __shfl_sync(0xffffffffu, cs2c, 4 * e4);   // the column's value: from the lane owning that row
                const float f1 = __shfl_sync(0xffffffffu, einv, 4 * e4 + 1), f2 = __shfl_sync(0xffffffffu, einv, 4 * e4 + 2);
                const float f3 = __shfl_sync(0xffffffffu, einv, 4 * e4 + 3);
                const float w0 = ex2(cs2 - c0), w1 = w0 * f1, w2 = w1 * f2, w3 = w2 * f3;
                const float v0 = __uint_as_float(gd[4 * e4]) * w0, v1 = __uint_as_float(gd[4 * e4 + 1]) * w1;
                const float v2 = __uint_as_float(gd[4 * e4 + 2]) * w2, v3 = __uint_as_float(gd[4 * e4 + 3]) * w3;
                pk[2 * e4] = pack2<T16>(4 * e4 <= lane ? v0 : 0.f, 4 * e4 + 1 <= lane ? v1 : 0.f);
                pk[2 * e4 + 1] = pack2<T16>(4 * e4 + 2 <= lane ? v2 : 0.f, 4 * e4 + 3 <= lane ? v3 : 0.f);
              }
              tmem_st16(tP + tlane + 16 * q, pk);
            }
#pragma unroll 1
            for (int J = 0; J < q; ++J) {   // strictly below the diagonal
              uint32_t gv[32];
              tmem_ld32(tG + tlane + 32 * J, gv);
              const float rf = ex2(cs2 - m->cend[h][par][J]);
              float4 fq[8];
              const float4* fv = reinterpret_cast<const float4*>(&m->cf[h][par][32 * J]);
#pragma unroll
              for (int e4 = 0; e4 < 8; ++e4) fq[e4] = fv[e4];
              tmem_ld_wait();
              uint32_t pk[16];
#pragma unroll
              for (int e4 = 0; e4 < 8; ++e4) {
                const float w0 = rf * fq[e4].x, w1 = rf * fq[e4].y, w2 = rf * fq[e4].z, w3 = rf * fq[e4].w;
                pk[2 * e4] = pack2<T16>(__uint_as_float(gv[4 * e4]) * w0, __uint_as_float(gv[4 * e4 + 1]) * w1);
                pk[2 * e4 + 1] = pack2<T16>(__uint_as_float(gv[4 * e4 + 2]) * w2, __uint_as_float(gv[4 * e4 + 3]) * w3);
              }
              tmem_st16(tP + tlane + 16 * J, pk);
            }
            if (ity == 0) {
              uint32_t pz[16];
#pragma unroll
              for (int e = 0; e < 16; ++e) pz[e] = 0u;
#pragma unroll 1
              for (int J = q + 1; J < 4; ++J) tmem_st16(tP + tlane + 16 * J, pz);
            }
            // ---- b. Y <- exp(cs_l) * (C.H) in place (after P: the C.H MMA could only start once the previous
            //      tile's Y had been read out, so it runs under step d); the P.X MMA accumulates on top
            ok = cwait(&m->bar_yo, ity & 1, STATUS_WAIT_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            const float el = ex2(cs2);
            {
              uint32_t y0[32], y1[32];
              tmem_ld32(tY + tlane, y0);
              tmem_ld32(tY + tlane + 32, y1);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 32; ++e) y0[e] = __float_as_uint(__uint_as_float(y0[e]) * el);
              tmem_st32(tY + tlane, y0);
#pragma unroll
              for (int e = 0; e < 32; ++e) y1[e] = __float_as_uint(__uint_as_float(y1[e]) * el);
              tmem_st32(tY + tlane + 32, y1);
            }
            tmem_st_wait();
            tc_fence_before();
            warp_arrive(&m->bar_p[h]);   // P is written and Y is scaled: the P.X MMA may run
          }
        }
        // (all C.H MMAs that read the state copy have been waited for: the previous item's in its step b)
        if (wy && have_next) {
          store_hb();
          fence_proxy_async();
          warp_arrive(&m->bar_h);
        }
        if (j >= 0) {
          if (wy) {
            y_pending = true;
            y_it = it; y_ity = ity; y_hi = hi; y_t0 = t0; y_bi = w.bi;
            if constexpr (EPI) {
              if (sp.D) y_dskip = sp.D[hi];
            }
            ++ity;
          }
          ++it;
        }
        cs = cs_n; tot = tot_n; cs2 = cs2_n; cs2c = cs2c_n;
      }
      if (!ok) break;

    }
    if (l == 0) bulk_wait_all();   // the Y tiles this thread stored must have landed before the CTA exits
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && m->abort_flag && status) atomicCAS(status, 0, (int)m->abort_flag);
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tb, 512);
  }
}

template <typename T16, int N, bool EPI>
int launch_typed2(const CUtensorMap& tx, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& ty,
                  const Tc2Params& prm, cudaStream_t stream) {
  auto kern = ssd_tc2_kernel<T16, N, EPI>;
  constexpr int smem = Layout2<N>::kBytes;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return SSD_ERR_CUDA;
  // chained mode: the tiles of all sequences are dealt out evenly, every CTA gets at least one
  const long long tiles = (long long)prm.upairs * (prm.sp.seqlen / T);
  const int grid = prm.sp.chain ? (int)std::min<long long>(tiles, kSms) : std::min(prm.nitems, kSms);
  kern<<<grid, kThreads2, smem, stream>>>(tx, tb, tc, ty, prm);
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

}  // namespace

bool tc2_supports(const SsdArgs& a) {
  if (!tc_supports(a)) return false;
  const int hpg = a.nheads / a.ngroups;
  return a.nheads % 2 == 0 && hpg % 2 == 0;
}

// Rounds of `items` equal work items over the persistent grid, as a fraction of the ideal.
static double round_efficiency(int64_t items) {
  const int64_t rounds = (items + kSms - 1) / kSms;
  return (double)items / (double)(rounds * kSms);
}

// How a sequence that is cut (nseg > 1) is scanned by this kernel:
//   1  with at least one sequence per SM the tiles of all sequences are dealt out evenly over the CTAs inside one
//      launch; a sequence cut that way hands its state from CTA to CTA through scratch ("chained");
//   2  with fewer sequences than SMs the same even deal, but each CTA first scans the last piece of its range
//      from zero and publishes (state, log-decay sum), and a piece folds what the CTAs before it published
//      ("look-back"), still one launch;
//   0  two passes and a fold (three launches): kept for the state-only run and the run that reuses its segment
//      states, which a sequence-sharded forward makes around its exchange.
int tc2_chain_mode(const SsdArgs& a, int nseg) {
  if (nseg <= 1) return 0;
  const int64_t upairs = (int64_t)a.batch * a.nheads / 2;
  if (upairs >= kSms) return 1;
  return (a.flags & (SSD_FLAG_STATE_ONLY | SSD_FLAG_REUSE_SEGMENTS)) ? 0 : 2;
}

int tc2_default_segments(const SsdArgs& a) {
  const int64_t upairs = (int64_t)a.batch * a.nheads / 2;
  const int tiles = a.seqlen / T;
  // whole sequences already fill the rounds of the persistent grid well: no cuts; else the even deal (any count
  // above one selects it, the cut points follow from the grid)
  if (upairs >= kSms) return (round_efficiency(upairs) >= 0.97 || tiles < 2) ? 1 : 2;
  const double whole = (double)tiles + 1.5;   // one CTA per sequence, in tile times
  if (!(a.flags & (SSD_FLAG_STATE_ONLY | SSD_FLAG_REUSE_SEGMENTS))) {
    // Look-back: every CTA gets total / SMs tiles plus the state-only scan of its last piece (0.4 of a full
    // tile, on most of its range) and two item start-ups.
    const double lookback = (double)upairs * tiles / kSms * 1.3 + 3.5;
    return (tiles >= 2 && lookback < 0.95 * whole) ? 2 : 1;
  }
  if (upairs >= 120) return 1;
  // Two passes: cutting the sequences into concurrently scanned segments costs a second pass
  // (about 0.4 of a full pass) and a per-item start-up (about 1.5 tile times).  Pick the count that
  // minimises the modelled time, in tile times, of the busiest CTA.
  double best_cost = whole;
  int best = 1;
  for (int nseg = 2; nseg <= 32 && nseg * 2 <= tiles; ++nseg) {
    const int64_t rounds = (upairs * nseg + kSms - 1) / kSms;
    const int per_item = (tiles + nseg - 1) / nseg;
    const double cost = (double)rounds * (per_item * 1.4 + 3.0);
    if (cost < best_cost * 0.97) {
      best_cost = cost;
      best = nseg;
    }
  }
  return best;
}

int launch_tc2(const SsdArgs& a, const ScanParams& sp, cudaStream_t stream) {
  if (sp.seg_len % T != 0) return SSD_ERR_UNSUPPORTED;
  Tc2Params prm;
  prm.sp = sp;
  prm.upairs = a.batch * (a.nheads / 2);
  prm.nitems = prm.upairs * sp.nseg;
  CUtensorMap tx, tb, tc, ty;
  if (!make_map(&tx, a.X, a.dtype, a.headdim, a.nheads, a.seqlen, a.batch, a.x_stride)) return SSD_ERR_CUDA;
  if (!make_map(&tb, a.B, a.dtype, a.dstate, a.ngroups, a.seqlen, a.batch, a.b_stride)) return SSD_ERR_CUDA;
  if (sp.compute_y) {
    if (!make_map(&tc, a.C, a.dtype, a.dstate, a.ngroups, a.seqlen, a.batch, a.c_stride)) return SSD_ERR_CUDA;
    if (!make_map(&ty, a.Y, a.dtype, a.headdim, a.nheads, a.seqlen, a.batch, a.y_stride)) return SSD_ERR_CUDA;
  } else {
    tc = tb;
    ty = tx;
  }
  const bool epi = sp.compute_y && (sp.D || sp.Z);
  if (epi) {
    // the gate rows are read with 16-byte loads
    if (sp.Z && ((reinterpret_cast<uintptr_t>(sp.Z) & 15) || sp.zs[0] % 8 || sp.zs[1] % 8 || sp.zs[2] % 8))
      return SSD_ERR_MISALIGNED;
    if (a.dtype == SSD_DTYPE_BF16)
      return a.dstate == 128 ? launch_typed2<__nv_bfloat16, 128, true>(tx, tb, tc, ty, prm, stream)
                             : launch_typed2<__nv_bfloat16, 64, true>(tx, tb, tc, ty, prm, stream);
    return a.dstate == 128 ? launch_typed2<__half, 128, true>(tx, tb, tc, ty, prm, stream)
                           : launch_typed2<__half, 64, true>(tx, tb, tc, ty, prm, stream);
  }
  if (a.dtype == SSD_DTYPE_BF16)
    return a.dstate == 128 ? launch_typed2<__nv_bfloat16, 128, false>(tx, tb, tc, ty, prm, stream)
                           : launch_typed2<__nv_bfloat16, 64, false>(tx, tb, tc, ty, prm, stream);
  return a.dstate == 128 ? launch_typed2<__half, 128, false>(tx, tb, tc, ty, prm, stream)
                         : launch_typed2<__half, 64, false>(tx, tb, tc, ty, prm, stream);
}

}  // namespace ssd
