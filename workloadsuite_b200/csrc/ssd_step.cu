// One token of the SSD recurrence per call, the state carried in place: the decode-style use of the carry of
// model_ref.py:152-157 (the reference itself only has the chunked forward; one token of it reduces to this):
//   H[b,h] <- exp(a[b,h]) * H[b,h] + B[b,g] (x) (dt[b,h] * x[b,h])        H is [n, p] fp32
//   y[b,h] <- C[b,g] . H[b,h]   (+ x * D[h], then * silu(z), as model_ref.py:116-118, when given)
// HBM-bound: the fp32 state is read and written once (2 * n * p * 4 bytes per (b, h)); everything else is small.
// One CTA per (batch, head): thread (r, c) owns four state columns 4c..4c+3 of the rows r, r + 16, ... ; all of its
// state loads are issued before the first use (n / 16 sixteen-byte loads in flight per thread), y is reduced over
// the sixteen row groups through shared memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "ssd_b200.h"
#include "ssd_common.cuh"

namespace ssd {
namespace {

constexpr int kStepThreads = 256;
constexpr int kHeadDim = 64;    // four columns per thread, sixteen threads per state row
constexpr int kMaxRowsPerThread = 16;   // dstate <= 256

template <typename T, int ROWS>   // ROWS = dstate / 16
__global__ void __launch_bounds__(kStepThreads)
ssd_step_kernel(const T* __restrict__ x, const float* __restrict__ a, const T* __restrict__ B, const T* __restrict__ C,
                const T* __restrict__ dt, const float* __restrict__ D, const T* __restrict__ z, float* __restrict__ state,
                T* __restrict__ y, int nheads, int ngroups) {
  __shared__ float ypart[16][kHeadDim];
  __shared__ float bs[16 * ROWS], cs[16 * ROWS];
  const int n = 16 * ROWS;
  const int unit = blockIdx.x;               // b * nheads + h
  const int b = unit / nheads, h = unit - b * nheads;
  const int g = h / (nheads / ngroups);
  const int tid = threadIdx.x, r = tid >> 4, c = tid & 15;
  float4* S = reinterpret_cast<float4*>(state + (int64_t)unit * n * kHeadDim) + c;
  float4 hv[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) hv[i] = S[(int64_t)(i * 16 + r) * (kHeadDim / 4)];   // all loads first
  const T* Bg = B + ((int64_t)b * ngroups + g) * n;
  const T* Cg = C + ((int64_t)b * ngroups + g) * n;
  for (int i = tid; i < n; i += kStepThreads) {
    bs[i] = Cvt<T>::to_f(Bg[i]);
    cs[i] = Cvt<T>::to_f(Cg[i]);
  }
  const T* xr = x + (int64_t)unit * kHeadDim + 4 * c;
  float xv[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) xv[e] = Cvt<T>::to_f(xr[e]);
  // x * dt in the layer's precision, as the reference forms it (model_ref.py:144)
  float xd[4];
  const float dtv = dt ? Cvt<T>::to_f(dt[unit]) : 1.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) xd[e] = dt ? Cvt<T>::to_f(Cvt<T>::from_f(xv[e] * dtv)) : xv[e];
  const float decay = __expf(a[unit]);
  __syncthreads();
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int row = i * 16 + r;
    const float bn = bs[row], cn = cs[row];
    float4 v = hv[i];
    v.x = fmaf(decay, v.x, bn * xd[0]); v.y = fmaf(decay, v.y, bn * xd[1]);
    v.z = fmaf(decay, v.z, bn * xd[2]); v.w = fmaf(decay, v.w, bn * xd[3]);
    S[(int64_t)row * (kHeadDim / 4)] = v;
    acc[0] = fmaf(cn, v.x, acc[0]); acc[1] = fmaf(cn, v.y, acc[1]);
    acc[2] = fmaf(cn, v.z, acc[2]); acc[3] = fmaf(cn, v.w, acc[3]);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) ypart[r][4 * c + e] = acc[e];
  __syncthreads();
  if (tid < kHeadDim) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) s += ypart[k][tid];
    const int64_t o = (int64_t)unit * kHeadDim + tid;
    if (D) s = fmaf(Cvt<T>::to_f(x[o]), D[h], s);
    if (z) {
      const float zz = Cvt<T>::to_f(z[o]);
      s *= zz / (1.f + __expf(-zz));
    }
    y[o] = Cvt<T>::from_f(s);
  }
}

template <typename T>
int launch_step(const void* x, const float* a, const void* B, const void* C, const void* dt, const float* D,
                const void* z, float* state, void* y, int batch, int nheads, int dstate, int ngroups,
                cudaStream_t stream) {
  const int units = batch * nheads;
  auto go = [&](auto kern) {
    kern<<<units, kStepThreads, 0, stream>>>(static_cast<const T*>(x), a, static_cast<const T*>(B),
                                             static_cast<const T*>(C), static_cast<const T*>(dt), D,
                                             static_cast<const T*>(z), state, static_cast<T*>(y), nheads, ngroups);
    return cudaGetLastError() == cudaSuccess ? (int)SSD_OK : (int)SSD_ERR_CUDA;
  };
  switch (dstate / 16) {
    case 1: return go(ssd_step_kernel<T, 1>);
    case 2: return go(ssd_step_kernel<T, 2>);
    case 4: return go(ssd_step_kernel<T, 4>);
    case 8: return go(ssd_step_kernel<T, 8>);
    case 16: return go(ssd_step_kernel<T, 16>);
    default: return SSD_ERR_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace ssd

extern "C" int ssd_b200_step(const void* x, const float* a, const void* B, const void* C, const void* dt,
                             const float* D, const void* z, float* state, void* y, int32_t batch, int32_t nheads,
                             int32_t headdim, int32_t dstate, int32_t ngroups, int32_t dtype, void* stream) {
  if (!x || !a || !B || !C || !state || !y) return SSD_ERR_NULL_POINTER;
  if (batch <= 0 || nheads <= 0 || headdim <= 0 || dstate <= 0 || ngroups <= 0 || nheads % ngroups != 0)
    return SSD_ERR_BAD_SHAPE;
  if (headdim != ssd::kHeadDim || dstate % 16 != 0 || dstate / 16 > ssd::kMaxRowsPerThread) return SSD_ERR_UNSUPPORTED;
  if ((int64_t)batch * nheads > 0x7fffffffLL) return SSD_ERR_TOO_LARGE;
  if (reinterpret_cast<uintptr_t>(state) & 15) return SSD_ERR_MISALIGNED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SSD_DTYPE_F32:
      return ssd::launch_step<float>(x, a, B, C, dt, D, z, state, y, batch, nheads, dstate, ngroups, s);
    case SSD_DTYPE_F16:
      return ssd::launch_step<__half>(x, a, B, C, dt, D, z, state, y, batch, nheads, dstate, ngroups, s);
    case SSD_DTYPE_BF16:
      return ssd::launch_step<__nv_bfloat16>(x, a, B, C, dt, D, z, state, y, batch, nheads, dstate, ngroups, s);
    default:
      return SSD_ERR_UNSUPPORTED;
  }
}
