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

// pairs of 16-bit elements <-> float2
__device__ __forceinline__ float2 up2(const __half*, uint32_t v) { return __half22float2(*reinterpret_cast<const __half2*>(&v)); }
__device__ __forceinline__ float2 up2(const __nv_bfloat16*, uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ uint32_t pk2(const __half*, float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pk2(const __nv_bfloat16*, float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// V consecutive elements (V = 8: one 16-byte vector of a 16-bit row; V = 4: half of it) <-> V floats.
template <typename T, int V>
__device__ __forceinline__ void loadv(const T* p, float (&v)[V], bool vec) {
  if constexpr (sizeof(T) == 2) {
    if (!vec) {
#pragma unroll
      for (int e = 0; e < V; ++e) v[e] = Cvt<T>::to_f(p[e]);
      return;
    }
    uint32_t q[V / 2];
    if (V == 8) {
      const uint4 r = *reinterpret_cast<const uint4*>(p);
      q[0] = r.x; q[1] = r.y; q[V / 2 - 2] = r.z; q[V / 2 - 1] = r.w;
    } else {
      const uint2 r = *reinterpret_cast<const uint2*>(p);
      q[0] = r.x; q[1] = r.y;
    }
#pragma unroll
    for (int e = 0; e < V / 2; ++e) {
      const float2 a = up2(p, q[e]);
      v[2 * e] = a.x; v[2 * e + 1] = a.y;
    }
    return;
  }
  if (vec) {
#pragma unroll
    for (int e = 0; e < V; e += 4) {
      const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + e);
      v[e] = a.x; v[e + 1] = a.y; v[e + 2] = a.z; v[e + 3] = a.w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) v[e] = Cvt<T>::to_f(p[e]);
  }
}
template <typename T, int V>
__device__ __forceinline__ void storev(T* p, const float (&v)[V], bool vec) {
  if constexpr (sizeof(T) == 2) {
    if (!vec) {
#pragma unroll
      for (int e = 0; e < V; ++e) p[e] = Cvt<T>::from_f(v[e]);
      return;
    }
    uint32_t q[V / 2];
#pragma unroll
    for (int e = 0; e < V / 2; ++e) q[e] = pk2(p, v[2 * e], v[2 * e + 1]);
    if (V == 8) *reinterpret_cast<uint4*>(p) = make_uint4(q[0], q[1], q[V / 2 - 2], q[V / 2 - 1]);
    else *reinterpret_cast<uint2*>(p) = make_uint2(q[0], q[1]);
    return;
  }
  if (vec) {
#pragma unroll
    for (int e = 0; e < V; e += 4)
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) p[e] = Cvt<T>::from_f(v[e]);
  }
}

// One thread: V consecutive channels, kTokensPerThread consecutive tokens, the last K-1 rows kept in registers as a
// sliding window.  V = 4 for 16-bit types (8-byte vectors: a warp still reads 256 contiguous bytes per row) keeps the
// thread's registers low enough for eight rows in flight per thread on 20 resident warps (40 KB of reads in flight
// per SM; bandwidth x latency asks for about 35 KB); V = 8 for fp32.
template <typename T, int K, int V>
__global__ void __launch_bounds__(128, (V == 4 ? 5 : 4))
conv1d_silu_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                   int batch, int seqlen, int channels, int64_t xsb, int64_t xsl, int64_t ysb, int64_t ysl, int vec_ok) {
  const int cvecs = channels / V;
  const int chunks = (seqlen + kTokensPerThread - 1) / kTokensPerThread;
  const int64_t total = (int64_t)batch * chunks * cvecs;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int cv = (int)(i % cvecs);          // consecutive threads: consecutive channel vectors (coalesced rows)
  const int64_t r = i / cvecs;
  const int ch = (int)(r % chunks);
  const int b = (int)(r / chunks);
  const int c0 = V * cv;
  const int t_begin = ch * kTokensPerThread, t_end = min(seqlen, t_begin + kTokensPerThread);

  float wk[K][V], bs[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    bs[e] = bias ? Cvt<T>::to_f(bias[c0 + e]) : 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) wk[k][e] = Cvt<T>::to_f(w[(int64_t)(c0 + e) * K + k]);
  }
  const bool vec = vec_ok != 0;
  const T* xrow = x + b * xsb + c0;
  auto emit = [&](int t, float (&win)[K][V]) {   // win holds rows t-(K-1) .. t
    float out[V];
#pragma unroll
    for (int e = 0; e < V; ++e) {
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
    storev<T, V>(y + b * ysb + (int64_t)t * ysl + c0, out, vec);
  };

  float win[K][V];   // win[k] = row t-(K-1)+k
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {   // the K-1 rows before the run: zeros before the sequence start
    const int t = t_begin - (K - 1) + k;
    if (t < 0) {
#pragma unroll
      for (int e = 0; e < V; ++e) win[k + 1][e] = 0.f;
    } else {
      loadv<T, V>(xrow + (int64_t)t * xsl, win[k + 1], vec);
    }
  }
  // rows fetched kBatch at a time: several loads per thread in flight before the first is used
  constexpr int kBatch = (V == 4 ? 8 : 4);
  for (int t0 = t_begin; t0 < t_end; t0 += kBatch) {
    float rows[kBatch][V];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (t0 + u < t_end) {
        loadv<T, V>(xrow + (int64_t)(t0 + u) * xsl, rows[u], vec);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) rows[u][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (t0 + u < t_end) {
#pragma unroll
        for (int k = 0; k < K - 1; ++k) {
#pragma unroll
          for (int e = 0; e < V; ++e) win[k][e] = win[k + 1][e];
        }
#pragma unroll
        for (int e = 0; e < V; ++e) win[K - 1][e] = rows[u][e];
        emit(t0 + u, win);
      }
    }
  }
}

template <typename T>
int launch_conv(const void* x, const void* w, const void* bias, void* y, int batch, int seqlen, int channels, int taps,
                int64_t xsb, int64_t xsl, int64_t ysb, int64_t ysl, cudaStream_t stream) {
  constexpr int V = sizeof(T) == 2 ? 4 : 8;
  const int chunks = (seqlen + kTokensPerThread - 1) / kTokensPerThread;
  const int64_t total = (int64_t)batch * chunks * (channels / V);
  if ((total + 127) / 128 > 0x7fffffffLL) return SSD_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)((total + 127) / 128);
  const int per16 = 16 / (int)sizeof(T);
  const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 && xsb % per16 == 0 &&
                  xsl % per16 == 0 && ysb % per16 == 0 && ysl % per16 == 0;
  const T* xx = static_cast<const T*>(x);
  const T* ww = static_cast<const T*>(w);
  const T* bb = static_cast<const T*>(bias);
  T* yy = static_cast<T*>(y);
  switch (taps) {
    case 2: conv1d_silu_kernel<T, 2, V><<<grid, 128, 0, stream>>>(xx, ww, bb, yy, batch, seqlen, channels, xsb, xsl, ysb, ysl, al); break;
    case 3: conv1d_silu_kernel<T, 3, V><<<grid, 128, 0, stream>>>(xx, ww, bb, yy, batch, seqlen, channels, xsb, xsl, ysb, ysl, al); break;
    case 4: conv1d_silu_kernel<T, 4, V><<<grid, 128, 0, stream>>>(xx, ww, bb, yy, batch, seqlen, channels, xsb, xsl, ysb, ysl, al); break;
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
