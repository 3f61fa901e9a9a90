// dt discretisation of SSDLayer.forward ahead of the core (model_ref.py:94, 102-103):
//   dt   = softplus(dt_raw + dt_bias[head])          in the layer's 16-bit (or fp32) dtype
//   A_dt = -exp(A_log[head]) * float(dt)             fp32, the per-token log-decay the core consumes
// dt_raw is read in place as a column slice of the projection output; both results are written contiguously.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "ssd_b200.h"
#include "ssd_common.cuh"

namespace ssd {
namespace {

template <typename T>
__global__ void __launch_bounds__(256)
dt_prologue_kernel(const T* __restrict__ dt_raw, int64_t sb, int64_t sl, const T* __restrict__ dt_bias,
                   const float* __restrict__ A_log, T* __restrict__ dt_out, float* __restrict__ A_dt, int batch,
                   int seqlen, int nheads) {
  const int64_t total = (int64_t)batch * seqlen * nheads;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int h = (int)(i % nheads);
    const int64_t r = i / nheads;
    const int t = (int)(r % seqlen);
    const int b = (int)(r / seqlen);
    // the reference adds in the layer's dtype, then softplus in that dtype (threshold 20, as torch)
    const float v = Cvt<T>::to_f(Cvt<T>::from_f(Cvt<T>::to_f(dt_raw[b * sb + (int64_t)t * sl + h]) +
                                                  (dt_bias ? Cvt<T>::to_f(dt_bias[h]) : 0.f)));
    const float sp = v > 20.f ? v : log1pf(expf(v));
    const T d = Cvt<T>::from_f(sp);
    dt_out[i] = d;
    A_dt[i] = -expf(A_log[h]) * Cvt<T>::to_f(d);
  }
}

template <typename T>
int launch_prologue(const void* dt_raw, int64_t sb, int64_t sl, const void* dt_bias, const float* A_log, void* dt_out,
                    float* A_dt, int batch, int seqlen, int nheads, cudaStream_t stream) {
  const int64_t total = (int64_t)batch * seqlen * nheads;
  const int grid = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  dt_prologue_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(dt_raw), sb, sl, static_cast<const T*>(dt_bias),
                                                  A_log, static_cast<T*>(dt_out), A_dt, batch, seqlen, nheads);
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

}  // namespace
}  // namespace ssd

extern "C" int ssd_b200_dt_prologue(const void* dt_raw, int64_t stride_b, int64_t stride_l, const void* dt_bias,
                                    const float* A_log, void* dt_out, float* A_dt_out, int32_t batch, int32_t seqlen,
                                    int32_t nheads, int32_t dtype, void* stream) {
  if (!dt_raw || !A_log || !dt_out || !A_dt_out) return SSD_ERR_NULL_POINTER;
  if (batch <= 0 || seqlen <= 0 || nheads <= 0) return SSD_ERR_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SSD_DTYPE_F32:
      return ssd::launch_prologue<float>(dt_raw, stride_b, stride_l, dt_bias, A_log, dt_out, A_dt_out, batch, seqlen,
                                         nheads, s);
    case SSD_DTYPE_F16:
      return ssd::launch_prologue<__half>(dt_raw, stride_b, stride_l, dt_bias, A_log, dt_out, A_dt_out, batch, seqlen,
                                          nheads, s);
    case SSD_DTYPE_BF16:
      return ssd::launch_prologue<__nv_bfloat16>(dt_raw, stride_b, stride_l, dt_bias, A_log, dt_out, A_dt_out, batch,
                                                 seqlen, nheads, s);
    default:
      return SSD_ERR_UNSUPPORTED;
  }
}
