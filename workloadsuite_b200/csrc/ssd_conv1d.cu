// Causal depthwise conv1d + SiLU, the producer of the SSD core's X (model_ref.py:50-58, 83-86):
//   y[b,t,c] = silu(bias[c] + sum_{k<K} w[c,k] * x[b, t-(K-1)+k, c]),  x == 0 before the sequence start
// (nn.Conv1d(d, d, K, padding=K-1, groups=d) on [b,d,l], output truncated to the first l steps).
// The reference transposes to [b,d,l] and back; here x stays channel-innermost, read as a strided view of
// the projection output and written in the [b,l,h*p] layout the core reads.  HBM-bound: every x read once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "ssd_b200.h"
#include "ssd_common.cuh"

namespace ssd {
namespace {

constexpr int kTokensPerThread = 32;
constexpr int kMaxTaps = 8;

// 8 consecutive elements <-> 8 floats, through 16-byte vectors kept in registers when `vec`.
__device__ __forceinline__ float2 up2(const __half*, uint32_t v) { return __half22float2(*reinterpret_cast<const __half2*>(&v)); }
__device__ __forceinline__ float2 up2(const __nv_bfloat16*, uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ float2 up2(const float*, uint32_t) { return make_float2(0.f, 0.f); }   // (never taken)
__device__ __forceinline__ uint32_t pk2(const __half*, float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pk2(const __nv_bfloat16*, float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8], bool vec) {
  if (vec) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const float2 a = up2(p, q.x), b = up2(p, q.y), c = up2(p, q.z), d = up2(p, q.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = Cvt<T>::to_f(p[e]);
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8], bool vec) {
  if (vec) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = p[e];
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8], bool vec) {
  if (vec) {
    uint4 q;
    q.x = pk2(p, v[0], v[1]); q.y = pk2(p, v[2], v[3]); q.z = pk2(p, v[4], v[5]); q.w = pk2(p, v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = q;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) p[e] = Cvt<T>::from_f(v[e]);
  }
}
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8], bool vec) {
  if (vec) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) p[e] = v[e];
  }
}

// One thread: 8 consecutive channels (one 16-byte vector of a 16-bit row), kTokensPerThread consecutive tokens,
// the last K-1 rows kept in registers as a sliding window.
template <typename T, int K>
__global__ void __launch_bounds__(128, 4)
conv1d_silu_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                   int batch, int seqlen, int channels, int64_t xsb, int64_t xsl, int64_t ysb, int64_t ysl, int vec_ok) {
  const int cvecs = channels / 8;
  const int chunks = (seqlen + kTokensPerThread - 1) / kTokensPerThread;
  const int64_t total = (int64_t)batch * chunks * cvecs;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int cv = (int)(i % cvecs);          // consecutive threads: consecutive channel vectors (coalesced rows)
  const int64_t r = i / cvecs;
  const int ch = (int)(r % chunks);
  const int b = (int)(r / chunks);
  const int c0 = 8 * cv;
  const int t_begin = ch * kTokensPerThread, t_end = min(seqlen, t_begin + kTokensPerThread);

  float wk[K][8], bs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    bs[e] = bias ? Cvt<T>::to_f(bias[c0 + e]) : 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) wk[k][e] = Cvt<T>::to_f(w[(int64_t)(c0 + e) * K + k]);
  }
  const bool vec = vec_ok != 0;
  auto load_row = [&](int t, float (&v)[8]) {   // zeros outside the sequence
    if (t < 0 || t >= seqlen) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
    } else {
      load8<T>(x + b * xsb + (int64_t)t * xsl + c0, v, vec);
    }
  };
  auto emit = [&](int t, float (&win)[K][8]) {   // win holds rows t-(K-1) .. t
    float out[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float acc = bs[e];
#pragma unroll
      for (int k = 0; k < K; ++k) acc = fmaf(wk[k][e], win[k][e], acc);
      if (sizeof(T) == 2) {
        // silu(a) = a * (0.5 + 0.5 tanh(a / 2)): one MUFU operation; its 2^-11 error is below the 16-bit rounding
        float th;
        asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * acc));
        out[e] = acc * fmaf(0.5f, th, 0.5f);
      } else {
        out[e] = __fdividef(acc, 1.f + __expf(-acc));
      }
    }
    store8<T>(y + b * ysb + (int64_t)t * ysl + c0, out, vec);
  };

  float win[K][8];   // win[k] = row t-(K-1)+k
#pragma unroll
  for (int k = 0; k < K - 1; ++k) load_row(t_begin - (K - 1) + k, win[k + 1]);
  if (vec && sizeof(T) == 2) {
    // rows fetched four at a time as raw 16-byte vectors: several loads per thread in flight, few registers
    constexpr int kBatch = 4;
    const T* xrow = x + b * xsb + c0;
    for (int t0 = t_begin; t0 < t_end; t0 += kBatch) {
      uint4 raw[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        raw[u] = (t0 + u < t_end) ? *reinterpret_cast<const uint4*>(xrow + (int64_t)(t0 + u) * xsl) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (t0 + u < t_end) {
#pragma unroll
          for (int k = 0; k < K - 1; ++k) {
#pragma unroll
            for (int e = 0; e < 8; ++e) win[k][e] = win[k + 1][e];
          }
          const float2 a = up2(xrow, raw[u].x), bq = up2(xrow, raw[u].y), c = up2(xrow, raw[u].z), d = up2(xrow, raw[u].w);
          win[K - 1][0] = a.x; win[K - 1][1] = a.y; win[K - 1][2] = bq.x; win[K - 1][3] = bq.y;
          win[K - 1][4] = c.x; win[K - 1][5] = c.y; win[K - 1][6] = d.x; win[K - 1][7] = d.y;
          emit(t0 + u, win);
        }
      }
    }
  } else {
    for (int t = t_begin; t < t_end; ++t) {
#pragma unroll
      for (int k = 0; k < K - 1; ++k) {
#pragma unroll
        for (int e = 0; e < 8; ++e) win[k][e] = win[k + 1][e];
      }
      load_row(t, win[K - 1]);
      emit(t, win);
    }
  }
}

// ---- 16-bit rows staged through shared memory -----------------------------------------------------------
// The same arithmetic, arranged for the memory system: a thread streams its 16-byte column (8 channels) of a run of
// 64 tokens through a private ring of shared-memory slots filled by cp.async (three 8-row pieces in flight per thread,
// up to 147 KB per SM: enough outstanding bytes to cover the DRAM latency, which registers cannot hold); nobody else
// reads those slots, so cp.async.wait_group is the only synchronisation (no barrier, no spin-wait).  The taps run as
// packed fp32 pairs (fma.rn.f32x2), and the sliding window lives in a ring of eight register rows whose slots are
// compile-time constants: no row is ever moved.
constexpr int kRun = 64, kPiece = 8, kStages = 4, kStagedThreads = 128;
constexpr int kStagedSmem = kStages * kPiece * kStagedThreads * 16;

typedef unsigned long long f32x2;   // two packed floats
__device__ __forceinline__ f32x2 pack_f2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma_f2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 mul_f2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int K>
__global__ void __launch_bounds__(kStagedThreads, 3)
conv1d_silu_staged_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                          int batch, int seqlen, int channels, int64_t xsb, int64_t xsl, int64_t ysb, int64_t ysl) {
  extern __shared__ __align__(16) unsigned char ring_smem[];
  const int cvecs = channels / 8;
  const int runs = (seqlen + kRun - 1) / kRun;
  const int64_t total = (int64_t)batch * runs * cvecs;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int cv = (int)(i % cvecs);          // consecutive threads: consecutive channel vectors (coalesced rows)
  const int64_t r = i / cvecs;
  const int run = (int)(r % runs);
  const int b = (int)(r / runs);
  const int c0 = 8 * cv;
  const int t_begin = run * kRun, t_end = min(seqlen, t_begin + kRun);
  const int npieces = (t_end - t_begin + kPiece - 1) / kPiece;
  const T* xcol = x + b * xsb + c0;
  T* ycol = y + b * ysb + c0;
  // slot of (stage, row) for this thread; consecutive threads lie 16 bytes apart: no bank conflicts
  const uint32_t ring0 = (uint32_t)__cvta_generic_to_shared(ring_smem) + threadIdx.x * 16;
  auto slot_addr = [&](int stage, int row) { return ring0 + (uint32_t)((stage * kPiece + row) * kStagedThreads * 16); };
  auto issue = [&](int piece) {   // the rows of one piece that exist, one 16-byte copy each
    if (piece < npieces) {
      const int t0 = t_begin + piece * kPiece;
#pragma unroll
      for (int u = 0; u < kPiece; ++u)
        if (t0 + u < t_end) cp_async16(slot_addr(piece % kStages, u), xcol + (int64_t)(t0 + u) * xsl);
    }
    cp_async_commit();   // (an empty group when there is nothing left: keeps the group count in step)
  };
#pragma unroll
  for (int p = 0; p < kStages - 1; ++p) issue(p);

  f32x2 wk[K][4], bs[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    bs[j] = bias ? pack_f2(Cvt<T>::to_f(bias[c0 + 2 * j]), Cvt<T>::to_f(bias[c0 + 2 * j + 1])) : pack_f2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < K; ++k)
      wk[k][j] = pack_f2(Cvt<T>::to_f(w[(int64_t)(c0 + 2 * j) * K + k]), Cvt<T>::to_f(w[(int64_t)(c0 + 2 * j + 1) * K + k]));
  }
  auto widen = [&](const uint4& q, f32x2 (&row)[4]) {
    const float2 a = up2(xcol, q.x), bq = up2(xcol, q.y), c = up2(xcol, q.z), d = up2(xcol, q.w);
    row[0] = pack_f2(a.x, a.y); row[1] = pack_f2(bq.x, bq.y); row[2] = pack_f2(c.x, c.y); row[3] = pack_f2(d.x, d.y);
  };
  // window: row t_begin + j lives in register row (4 + j) & 7, j >= -(K - 1)
  f32x2 win[8][4];
#pragma unroll
  for (int k = 1; k < K; ++k) {
    const int t = t_begin - k;
    const uint4 q = t >= 0 ? *reinterpret_cast<const uint4*>(xcol + (int64_t)t * xsl) : make_uint4(0, 0, 0, 0);
    widen(q, win[(4 - k) & 7]);
  }
  const f32x2 half2 = pack_f2(0.5f, 0.5f);
  for (int piece = 0; piece < npieces; ++piece) {
    issue(piece + kStages - 1);
    cp_async_wait<kStages - 1>();   // this thread's copies of `piece` have landed (it is their only reader)
    const int t0 = t_begin + piece * kPiece, st = piece % kStages;
#pragma unroll
    for (int u = 0; u < kPiece; ++u) {
      if (t0 + u < t_end) {
        const int s = (4 + u) & 7;
        uint4 q;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(slot_addr(st, u)));
        widen(q, win[s]);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f32x2 acc = bs[j];
#pragma unroll
          for (int k = 0; k < K; ++k) acc = fma_f2(wk[k][j], win[(s + 8 - (K - 1) + k) & 7][j], acc);
          // silu(a) = a * (0.5 + 0.5 tanh(a / 2)): one MUFU operation per element; its 2^-11 error is below the 16-bit rounding
          float h0, h1, a0, a1;
          unpack_f2(mul_f2(acc, half2), h0, h1);
          asm("tanh.approx.f32 %0, %1;" : "=f"(h0) : "f"(h0));
          asm("tanh.approx.f32 %0, %1;" : "=f"(h1) : "f"(h1));
          unpack_f2(mul_f2(acc, fma_f2(pack_f2(h0, h1), half2, half2)), a0, a1);
          o[j] = pk2(xcol, a0, a1);
        }
        *reinterpret_cast<uint4*>(ycol + (int64_t)(t0 + u) * ysl) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  cp_async_wait<0>();
}

template <typename T>
int launch_conv(const void* x, const void* w, const void* bias, void* y, int batch, int seqlen, int channels, int taps,
                int64_t xsb, int64_t xsl, int64_t ysb, int64_t ysl, cudaStream_t stream) {
  const int chunks = (seqlen + kTokensPerThread - 1) / kTokensPerThread;
  const int64_t total = (int64_t)batch * chunks * (channels / 8);
  if ((total + 127) / 128 > 0x7fffffffLL) return SSD_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)((total + 127) / 128);
  const int per16 = 16 / (int)sizeof(T);
  const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 && xsb % per16 == 0 &&
                  xsl % per16 == 0 && ysb % per16 == 0 && ysl % per16 == 0;
  const T* xx = static_cast<const T*>(x);
  const T* ww = static_cast<const T*>(w);
  const T* bb = static_cast<const T*>(bias);
  T* yy = static_cast<T*>(y);
  if constexpr (sizeof(T) == 2) {
    if (al && taps >= 2 && taps <= 4) {
      const int runs = (seqlen + kRun - 1) / kRun;
      const int64_t tot = (int64_t)batch * runs * (channels / 8);
      if ((tot + kStagedThreads - 1) / kStagedThreads > 0x7fffffffLL) return SSD_ERR_TOO_LARGE;
      const unsigned g = (unsigned)((tot + kStagedThreads - 1) / kStagedThreads);
      auto go = [&](auto kern) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kStagedSmem) != cudaSuccess)
          return (int)SSD_ERR_CUDA;
        kern<<<g, kStagedThreads, kStagedSmem, stream>>>(xx, ww, bb, yy, batch, seqlen, channels, xsb, xsl, ysb, ysl);
        return cudaGetLastError() == cudaSuccess ? (int)SSD_OK : (int)SSD_ERR_CUDA;
      };
      if (taps == 2) return go(conv1d_silu_staged_kernel<T, 2>);
      if (taps == 3) return go(conv1d_silu_staged_kernel<T, 3>);
      return go(conv1d_silu_staged_kernel<T, 4>);
    }
  }
  switch (taps) {
    case 2: conv1d_silu_kernel<T, 2><<<grid, 128, 0, stream>>>(xx, ww, bb, yy, batch, seqlen, channels, xsb, xsl, ysb, ysl, al); break;
    case 3: conv1d_silu_kernel<T, 3><<<grid, 128, 0, stream>>>(xx, ww, bb, yy, batch, seqlen, channels, xsb, xsl, ysb, ysl, al); break;
    case 4: conv1d_silu_kernel<T, 4><<<grid, 128, 0, stream>>>(xx, ww, bb, yy, batch, seqlen, channels, xsb, xsl, ysb, ysl, al); break;
    default: return SSD_ERR_UNSUPPORTED;
  }
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

}  // namespace
}  // namespace ssd

extern "C" int ssd_b200_conv1d_silu(const void* x, const void* weight, const void* bias, void* y, int32_t batch,
                                    int32_t seqlen, int32_t channels, int32_t taps, int32_t dtype, int64_t x_stride_b,
                                    int64_t x_stride_l, int64_t y_stride_b, int64_t y_stride_l, void* stream) {
  if (!x || !weight || !y) return SSD_ERR_NULL_POINTER;
  if (batch <= 0 || seqlen <= 0 || channels <= 0 || taps <= 0 || taps > ssd::kMaxTaps) return SSD_ERR_BAD_SHAPE;
  if (channels % 8 != 0) return SSD_ERR_UNSUPPORTED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SSD_DTYPE_F32:
      return ssd::launch_conv<float>(x, weight, bias, y, batch, seqlen, channels, taps, x_stride_b, x_stride_l,
                                     y_stride_b, y_stride_l, s);
    case SSD_DTYPE_F16:
      return ssd::launch_conv<__half>(x, weight, bias, y, batch, seqlen, channels, taps, x_stride_b, x_stride_l,
                                      y_stride_b, y_stride_l, s);
    case SSD_DTYPE_BF16:
      return ssd::launch_conv<__nv_bfloat16>(x, weight, bias, y, batch, seqlen, channels, taps, x_stride_b,
                                             x_stride_l, y_stride_b, y_stride_l, s);
    default:
      return SSD_ERR_UNSUPPORTED;
  }
}
