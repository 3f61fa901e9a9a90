// Tensor-core SSD forward for sm_100a: tcgen05.mma with TMEM accumulators, TMA-staged
// operands, one CTA walking the 128-token tiles of one (batch, head[, segment]) in order.
//
// Per tile (tokens l, s in [0,128), state index n, head dim p), following the chunked
// form of the reference (model_ref.py:135-162) with the tile as the chunk:
//   cs        = inclusive prefix sum of the log-decay a           (:135)   warp-shuffle scan
//   G         = C . B^T                                            (:143)   UMMA 128x128xN
//   P[l,s]    = G[l,s] * exp(cs_l - cs_s) * [s <= l]   -> bf16     (:139-145) TMEM -> regs -> smem
//   Yd        = P . X                                              (:145)   UMMA 128x64x128
//   Xd[l,:]   = exp(cs_last - cs_l) * X[l,:]           -> bf16     (:148)
//   S         = B^T . Xd                                           (:149)   UMMA Nx64x128
//   Yo        = C . H (H = state entering the tile, bf16 copy)     (:155,161) UMMA 128x64xN
//   Y[l,:]    = Yd[l,:] + exp(cs_l) * Yo[l,:]                      (:160-162)
//   H         = exp(cs_last) * H + S   (fp32, registers)           (:150,156)
// L = exp(segsum) never exists in memory; the state never leaves the SM.
//
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = compute (one
// thread per tile row / TMEM lane).  All waits are bounded by a clock limit; a wait
// that runs out sets an abort flag, writes a status code and every role leaves.
#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "ssd_common.cuh"
#include "tc_common.cuh"
#include "tc_ptx.cuh"

namespace ssd {
namespace {

using namespace ptx;

using namespace tc;
constexpr int kThreads = 192;

template <int N>
struct Layout {
  static constexpr int NB = N / 64;
  static constexpr int oB = 0;
  static constexpr int oC = oB + NB * kBlk;
  static constexpr int oX = oC + NB * kBlk;   // two stages
  static constexpr int oXd = oX + 2 * kBlk;
  static constexpr int oP = oXd + kBlk;        // two blocks
  static constexpr int oH = oP + 2 * kBlk;     // N rows of 128 B
  static constexpr int oMisc = oH + N * 128;
  static constexpr int kBytes = oMisc + 4096 + 1024;  // misc + slack for 1024-byte alignment
};

struct Misc {
  uint64_t full_b, full_c, full_x[2], empty_b, empty_c, empty_x[2];
  uint64_t bar_g, bar_xd, bar_s, bar_p, bar_y, bar_h, bar_e[2];
  uint32_t tmem_base;
  long long wait_clocks;   // bound of every wait (SM clock cycles)
  volatile int abort_flag;
  float wsum[2][4];
  alignas(16) float cs2[2][T];   // prefix sums times log2(e), double-buffered by tile parity
};

struct TcParams {
  ScanParams sp;
  int fmt;  // 0 = f16, 1 = bf16
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Misc* m, int code, int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63) == 0) {
      if (m->abort_flag) return false;
      if (clock64() - t0 > m->wait_clocks) {
        m->abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

template <typename T16, int N>
__global__ void __launch_bounds__(kThreads, 1)
ssd_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmB,
              const __grid_constant__ CUtensorMap tmC, const TcParams prm) {
  using L = Layout<N>;
  constexpr int NB = L::NB;
  constexpr int KN = N / 16;   // k-steps over the state dimension
  constexpr int KT = T / 16;   // k-steps over the tile's tokens
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Misc* m = reinterpret_cast<Misc*>(smem + L::oMisc);
  const ScanParams& sp = prm.sp;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int unit = blockIdx.x, seg = blockIdx.y;
  const int bi = unit / sp.nheads, hi = unit - bi * sp.nheads;
  const int gi = hi / (sp.nheads / sp.ngroups);
  const int t_begin = seg * sp.seg_len;
  const int t_end = min(sp.seqlen, t_begin + sp.seg_len);
  const int ntiles = (t_end - t_begin) / T;
  const bool want_y = sp.compute_y != 0;
  int32_t* status = sp.status;

  if (tid == 0) {
    mbar_init(&m->full_b, 1); mbar_init(&m->full_c, 1); mbar_init(&m->full_x[0], 1); mbar_init(&m->full_x[1], 1);
    mbar_init(&m->empty_b, 1); mbar_init(&m->empty_c, 1); mbar_init(&m->empty_x[0], 1); mbar_init(&m->empty_x[1], 1);
    mbar_init(&m->bar_g, 1); mbar_init(&m->bar_s, 1); mbar_init(&m->bar_y, 1);
    mbar_init(&m->bar_xd, 128); mbar_init(&m->bar_p, 128); mbar_init(&m->bar_h, 128);
    mbar_init(&m->bar_e[0], 128); mbar_init(&m->bar_e[1], 128);
    m->abort_flag = 0;
    m->wait_clocks = prm.sp.wait_clocks;
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(&m->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = m->tmem_base;
  const uint32_t tG = tb, tS = tb + 128;
  const uint32_t tYo[2] = {tb + 192, tb + 256};
  const uint32_t tYd[2] = {tb + 320, tb + 384};

  const uint32_t sB = smem_u32(smem + L::oB), sC = smem_u32(smem + L::oC), sX = smem_u32(smem + L::oX);
  const uint32_t sXd = smem_u32(smem + L::oXd), sP = smem_u32(smem + L::oP), sH = smem_u32(smem + L::oH);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmX); prefetch_tmap(&tmB); prefetch_tmap(&tmC);
      bool ok = true;
      int armed = 0;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int t0 = t_begin + i * T;
        if (want_y) {
          if (i > 0) ok = wait_or_abort(&m->empty_c, (i - 1) & 1, m, STATUS_WAIT_TIMEOUT_MMA, status);
          if (!ok) break;
          mbar_expect_tx(&m->full_c, NB * kBlk);
#pragma unroll
          for (int kb = 0; kb < NB; ++kb) tma_load_4d(smem + L::oC + kb * kBlk, &tmC, &m->full_c, 64 * kb, gi, t0, bi);
        }
        if (i > 0) ok = wait_or_abort(&m->empty_b, (i - 1) & 1, m, STATUS_WAIT_TIMEOUT_MMA, status);
        if (!ok) break;
        mbar_expect_tx(&m->full_b, NB * kBlk);
#pragma unroll
        for (int kb = 0; kb < NB; ++kb) tma_load_4d(smem + L::oB + kb * kBlk, &tmB, &m->full_b, 64 * kb, gi, t0, bi);
        const int st = i & 1;
        if (i >= 2) ok = wait_or_abort(&m->empty_x[st], ((i - 2) >> 1) & 1, m, STATUS_WAIT_TIMEOUT_MMA, status);
        if (!ok) break;
        mbar_expect_tx(&m->full_x[st], kBlk);
        tma_load_4d(smem + L::oX + st * kBlk, &tmX, &m->full_x[st], 0, hi, t0, bi);
        armed = i + 1;
      }
      if (m->abort_flag && armed > 0) {
        // let copies already in flight land before the CTA gives its shared memory back
        const int i = armed - 1;
        const long long c0 = clock64();
        while (clock64() - c0 < 2000000LL) {
          if (mbar_try_wait(&m->full_b, i & 1) && mbar_try_wait(&m->full_x[i & 1], (i >> 1) & 1) &&
              (!want_y || mbar_try_wait(&m->full_c, i & 1)))
            break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr int fmt = sizeof(T16) == 2 && std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idG = umma_idesc(128, 128, fmt, 0, 0);   // C (K-major) x B (K-major)
      constexpr uint32_t idKM = umma_idesc(128, 64, fmt, 0, 1);   // A K-major, B MN-major
      constexpr uint32_t idMM = umma_idesc(128, 64, fmt, 1, 1);   // A MN-major, B MN-major
      constexpr uint64_t dK = umma_desc_base(16, 1024);
      constexpr uint64_t dMN = umma_desc_base(kBlk, 1024);
      bool ok = true;
      for (int i = 0; i < ntiles && ok; ++i) {
        const int st = i & 1, buf = i & 1;
        if (want_y) {
          ok = wait_or_abort(&m->full_c, i & 1, m, STATUS_WAIT_TIMEOUT_TMA, status) &&
               wait_or_abort(&m->full_b, i & 1, m, STATUS_WAIT_TIMEOUT_TMA, status) &&
               wait_or_abort(&m->bar_h, i & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
          if (ok && i >= 2) ok = wait_or_abort(&m->bar_e[buf], ((i - 2) >> 1) & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < KN; ++k) {
            const uint32_t off = (k >> 2) * kBlk + (k & 3) * 32;
            umma_ss(tG, umma_desc(dK, sC + off), umma_desc(dK, sB + off), idG, k > 0);
          }
#pragma unroll
          for (int k = 0; k < KN; ++k) {
            const uint32_t off = (k >> 2) * kBlk + (k & 3) * 32;
            umma_ss(tYo[buf], umma_desc(dK, sC + off), umma_desc(dMN, sH + k * 2048), idKM, k > 0);
          }
          umma_commit(&m->bar_g);
          umma_commit(&m->empty_c);
        } else {
          ok = wait_or_abort(&m->full_b, i & 1, m, STATUS_WAIT_TIMEOUT_TMA, status) &&
               wait_or_abort(&m->bar_h, i & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
          if (!ok) break;
        }
        ok = wait_or_abort(&m->bar_xd, i & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < KT; ++k)
          umma_ss(tS, umma_desc(dMN, sB + k * 2048), umma_desc(dMN, sXd + k * 2048), idMM, k > 0);
        umma_commit(&m->bar_s);
        umma_commit(&m->empty_b);
        if (want_y) {
          ok = wait_or_abort(&m->bar_p, i & 1, m, STATUS_WAIT_TIMEOUT_SYNC, status) &&
               wait_or_abort(&m->full_x[st], (i >> 1) & 1, m, STATUS_WAIT_TIMEOUT_TMA, status);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < KT; ++k) {
            const uint32_t off = (k >> 2) * kBlk + (k & 3) * 32;
            umma_ss(tYd[buf], umma_desc(dK, sP + off), umma_desc(dMN, sX + st * kBlk + k * 2048), idKM, k > 0);
          }
          umma_commit(&m->bar_y);
          umma_commit(&m->empty_x[st]);
        } else {
          mbar_arrive(&m->empty_x[st]);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps (one thread per row / TMEM lane)
    const int lane_base = (warp & 3) * 32;
    const int l = lane_base + lane;
    const uint32_t tlane = (uint32_t)lane_base << 16;
    const uint32_t swz = (uint32_t)(l & 7);
    const bool owns_state = lane_base < N;  // warp-uniform: rows of the n x p state live in lanes [0, N)

    float H[P];
    if (sp.init && owns_state) {
      const float4* I = reinterpret_cast<const float4*>(sp.init + unit * sp.init_unit_stride + seg * sp.init_seg_stride +
                                                        (int64_t)l * P);
#pragma unroll
      for (int j = 0; j < P / 4; ++j) {
        const float4 v = I[j];
        H[4 * j] = v.x; H[4 * j + 1] = v.y; H[4 * j + 2] = v.z; H[4 * j + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < P; ++j) H[j] = 0.f;
    }
    auto store_hb = [&]() {
      if (owns_state) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 v;
          v.x = pack2<T16>(H[8 * c + 0], H[8 * c + 1]); v.y = pack2<T16>(H[8 * c + 2], H[8 * c + 3]);
          v.z = pack2<T16>(H[8 * c + 4], H[8 * c + 5]); v.w = pack2<T16>(H[8 * c + 6], H[8 * c + 7]);
          sts128(sH + l * 128 + ((c ^ swz) << 4), v);
        }
      }
    };
    if (want_y) {
      store_hb();
      fence_proxy_async();
    }
    mbar_arrive(&m->bar_h);   // completion #0: state entering tile 0 is in place

    const float* Ag = sp.A + bi * sp.as[0] + hi * sp.as[2];
    const T16* Dg = sp.dt ? static_cast<const T16*>(sp.dt) + bi * sp.dts[0] + hi * sp.dts[2] : nullptr;
    T16* Yg = want_y ? static_cast<T16*>(sp.Y) + bi * sp.ys[0] + hi * sp.ys[2] : nullptr;
    float a_next = ntiles > 0 ? Ag[(int64_t)(t_begin + l) * sp.as[1]] : 0.f;
    // (dt stays as loaded until its use one iteration later: a conversion right behind the load would hold the warp
    //  for the memory latency)
    T16 dt_next = (Dg && ntiles > 0) ? Dg[(int64_t)(t_begin + l) * sp.dts[1]] : Cvt<T16>::from_f(1.f);
    double asum = 0.0;
    bool ok = true;
    // the outcome of a wait is made uniform over the warp: tcgen05.ld needs the whole warp
    auto cwait = [&](uint64_t* bar, uint32_t parity, int code) {
      return __all_sync(0xffffffffu, wait_or_abort(bar, parity, m, code, status)) != 0;
    };

    for (int i = 0; i < ntiles && ok; ++i) {
      const int t0 = t_begin + i * T;
      const int par = i & 1, st = i & 1, buf = i & 1;
      const float a = a_next, dtv = Cvt<T16>::to_f(dt_next);
      if (i + 1 < ntiles) {
        a_next = Ag[(int64_t)(t0 + T + l) * sp.as[1]];
        if (Dg) dt_next = Dg[(int64_t)(t0 + T + l) * sp.dts[1]];
      }
      // ---- in-tile inclusive prefix sum of the log-decay (model_ref.py:135)
      float v = a;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += t;
      }
      if (lane == 31) m->wsum[par][warp & 3] = v;
      named_bar_sync(1, 128);
      const float w0 = m->wsum[par][0], w1 = m->wsum[par][1], w2 = m->wsum[par][2], w3 = m->wsum[par][3];
      const int q = warp & 3;
      const float cs = v + ((q > 0 ? w0 : 0.f) + (q > 1 ? w1 : 0.f) + (q > 2 ? w2 : 0.f));
      const float tot = (w0 + w1 + w2) + w3;
      const float cs2 = cs * kLog2e;
      m->cs2[par][l] = cs2;
      named_bar_sync(1, 128);
      asum += (double)tot;

      // ---- Xd = exp(cs_last - cs_l) * x~   (model_ref.py:144,148)
      ok = cwait(&m->full_x[st], (i >> 1) & 1, STATUS_WAIT_TIMEOUT_TMA);
      if (!ok) break;
      {
        const float dl = ex2((tot - cs) * kLog2e);
        const uint32_t xrow = sX + st * kBlk + l * 128, xdrow = sXd + l * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t phys = (c ^ swz) << 4;
          uint4 raw = lds128(xrow + phys);
          float2 f0 = unpack2<T16>(raw.x), f1 = unpack2<T16>(raw.y), f2 = unpack2<T16>(raw.z), f3 = unpack2<T16>(raw.w);
          if (Dg) {
            f0.x *= dtv; f0.y *= dtv; f1.x *= dtv; f1.y *= dtv; f2.x *= dtv; f2.y *= dtv; f3.x *= dtv; f3.y *= dtv;
            raw.x = pack2<T16>(f0.x, f0.y); raw.y = pack2<T16>(f1.x, f1.y);
            raw.z = pack2<T16>(f2.x, f2.y); raw.w = pack2<T16>(f3.x, f3.y);
            sts128(xrow + phys, raw);   // x~ replaces x as the operand of P . X
          }
          uint4 o;
          o.x = pack2<T16>(f0.x * dl, f0.y * dl); o.y = pack2<T16>(f1.x * dl, f1.y * dl);
          o.z = pack2<T16>(f2.x * dl, f2.y * dl); o.w = pack2<T16>(f3.x * dl, f3.y * dl);
          sts128(xdrow + phys, o);
        }
      }
      fence_proxy_async();
      mbar_arrive(&m->bar_xd);

      if (want_y) {
        // ---- P = (C B^T) o exp(segsum), causal  (model_ref.py:139-145)
        ok = cwait(&m->bar_g, i & 1, STATUS_WAIT_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t prow = sP + (j >> 1) * kBlk + l * 128;
          const int cbase = (j & 1) * 4;
          if (j > q) {   // strictly above the diagonal for every row of this warp
#pragma unroll
            for (int c = 0; c < 4; ++c) sts128(prow + (((cbase + c) ^ swz) << 4), make_uint4(0, 0, 0, 0));
          } else {
            uint32_t gv[32];
            tmem_ld32(tG + tlane + 32 * j, gv);
            tmem_ld_wait();
            const float4* csv = reinterpret_cast<const float4*>(&m->cs2[par][32 * j]);
            float pv[32];
#pragma unroll
            for (int e4 = 0; e4 < 8; ++e4) {
              const float4 c4 = csv[e4];
              const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
              for (int r = 0; r < 4; ++r) {
                const int e = 4 * e4 + r;
                const float w = ex2(cs2 - cc[r]);
                const float val = __uint_as_float(gv[e]) * w;
                pv[e] = (j < q || 32 * j + e <= l) ? val : 0.f;
              }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 o;
              o.x = pack2<T16>(pv[8 * c + 0], pv[8 * c + 1]); o.y = pack2<T16>(pv[8 * c + 2], pv[8 * c + 3]);
              o.z = pack2<T16>(pv[8 * c + 4], pv[8 * c + 5]); o.w = pack2<T16>(pv[8 * c + 6], pv[8 * c + 7]);
              sts128(prow + (((cbase + c) ^ swz) << 4), o);
            }
          }
        }
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(&m->bar_p);
      }

      // ---- state: H <- exp(cs_last) H + S   (model_ref.py:150,156); bf16 copy for the next tile's C . H
      ok = cwait(&m->bar_s, i & 1, STATUS_WAIT_TIMEOUT_MMA);
      if (!ok) break;
      tc_fence_after();
      if (owns_state) {
        const float g = ex2(tot * kLog2e);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t sv[32];
          tmem_ld32(tS + tlane + 32 * hf, sv);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) H[32 * hf + e] = fmaf(H[32 * hf + e], g, __uint_as_float(sv[e]));
        }
        if (want_y && i + 1 < ntiles) store_hb();
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&m->bar_h);

      if (want_y) {
        // ---- Y = Yd + exp(cs_l) * Yo   (model_ref.py:160-162)
        ok = cwait(&m->bar_y, i & 1, STATUS_WAIT_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const float el = ex2(cs2);
        T16* yrow = Yg + (int64_t)(t0 + l) * sp.ys[1];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t vd[32], vo[32];
          tmem_ld32(tYd[buf] + tlane + 32 * hf, vd);
          tmem_ld32(tYo[buf] + tlane + 32 * hf, vo);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float y[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
              y[r] = fmaf(el, __uint_as_float(vo[8 * c + r]), __uint_as_float(vd[8 * c + r]));
            uint4 o;
            o.x = pack2<T16>(y[0], y[1]); o.y = pack2<T16>(y[2], y[3]);
            o.z = pack2<T16>(y[4], y[5]); o.w = pack2<T16>(y[6], y[7]);
            *reinterpret_cast<uint4*>(yrow + 32 * hf + 8 * c) = o;
          }
        }
        tc_fence_before();
        mbar_arrive(&m->bar_e[buf]);
      }
    }

    if (ok) {
      if (sp.fin && owns_state) {
        float4* F = reinterpret_cast<float4*>(sp.fin + unit * sp.fin_unit_stride + seg * sp.fin_seg_stride +
                                              (int64_t)l * P);
#pragma unroll
        for (int j = 0; j < P / 4; ++j) F[j] = make_float4(H[4 * j], H[4 * j + 1], H[4 * j + 2], H[4 * j + 3]);
      }
      if (sp.fin_ld && l == 0) sp.fin_ld[unit * sp.finld_unit_stride + seg * sp.finld_seg_stride] = (float)asum;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tb, 512);
  }
}

// ---------------------------------------------------------------------------- host side

template <typename T16, int N>
int launch_typed(const CUtensorMap& tx, const CUtensorMap& tb, const CUtensorMap& tc, const TcParams& prm,
                 cudaStream_t stream) {
  auto kern = ssd_tc_kernel<T16, N>;
  constexpr int smem = Layout<N>::kBytes;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return SSD_ERR_CUDA;
  dim3 grid((unsigned)(prm.sp.batch * prm.sp.nheads), (unsigned)prm.sp.nseg);
  kern<<<grid, kThreads, smem, stream>>>(tx, tb, tc, prm);
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

}  // namespace

bool tc_supports(const SsdArgs& a) {
  if (a.dtype != SSD_DTYPE_F16 && a.dtype != SSD_DTYPE_BF16) return false;
  if (a.headdim != P || (a.dstate != 64 && a.dstate != 128)) return false;
  if (a.seqlen % T != 0) return false;
  if (!ok16(a.X) || !ok16(a.B) || !stride_ok(a.x_stride) || !stride_ok(a.b_stride)) return false;
  const bool state_only = (a.flags & SSD_FLAG_STATE_ONLY) != 0;
  if (!state_only) {
    if (!a.C || !a.Y) return true;  // shape query without pointers (kernel_name / workspace_bytes)
    if (!ok16(a.C) || !ok16(a.Y) || !stride_ok(a.c_stride) || !stride_ok(a.y_stride)) return false;
  }
  return true;
}

int tc_default_segments(const SsdArgs& a) {
  const int64_t units = (int64_t)a.batch * a.nheads;
  if (units >= 120) return 1;
  const int tiles = a.seqlen / T;
  int want = (int)((2 * 148 + units - 1) / units);
  want = std::min(want, std::max(1, tiles / 4));   // at least four tiles per segment
  return std::max(1, want);
}

int launch_tc(const SsdArgs& a, const ScanParams& sp, cudaStream_t stream) {
  if (sp.seg_len % T != 0) return SSD_ERR_UNSUPPORTED;
  TcParams prm;
  prm.sp = sp;
  prm.fmt = a.dtype == SSD_DTYPE_BF16 ? 1 : 0;
  CUtensorMap tx, tb, tc;
  if (!make_map(&tx, a.X, a.dtype, a.headdim, a.nheads, a.seqlen, a.batch, a.x_stride)) return SSD_ERR_CUDA;
  if (!make_map(&tb, a.B, a.dtype, a.dstate, a.ngroups, a.seqlen, a.batch, a.b_stride)) return SSD_ERR_CUDA;
  if (sp.compute_y) {
    if (!make_map(&tc, a.C, a.dtype, a.dstate, a.ngroups, a.seqlen, a.batch, a.c_stride)) return SSD_ERR_CUDA;
  } else {
    tc = tb;
  }
  if (a.dtype == SSD_DTYPE_BF16)
    return a.dstate == 128 ? launch_typed<__nv_bfloat16, 128>(tx, tb, tc, prm, stream)
                           : launch_typed<__nv_bfloat16, 64>(tx, tb, tc, prm, stream);
  return a.dstate == 128 ? launch_typed<__half, 128>(tx, tb, tc, prm, stream)
                         : launch_typed<__half, 64>(tx, tb, tc, prm, stream);
}

}  // namespace ssd
