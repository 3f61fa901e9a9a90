// Pieces shared by the tensor-core SSD kernels: tile constants, 16-bit pack/unpack,
// shared-memory vector access, and the host-side TMA descriptor builder.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "ssd_b200.h"

namespace ssd {
namespace tc {

constexpr int T = 128;          // tokens per tile
constexpr int P = 64;           // head dim
constexpr int kBlk = T * 128;   // bytes of one [128 rows x 64 cols] 16-bit swizzled block
constexpr float kLog2e = 1.4426950408889634f;

template <typename T16>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
template <typename T16>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Packed 16-bit fused multiply-add a * b + c.
template <typename T16>
__device__ __forceinline__ uint32_t fma2(uint32_t a, uint32_t b, uint32_t c);
template <>
__device__ __forceinline__ uint32_t fma2<__nv_bfloat16>(uint32_t a, uint32_t b, uint32_t c) {
  __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b),
                             *reinterpret_cast<const __nv_bfloat162*>(&c));
  return *reinterpret_cast<uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t fma2<__half>(uint32_t a, uint32_t b, uint32_t c) {
  __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b),
                      *reinterpret_cast<const __half2*>(&c));
  return *reinterpret_cast<uint32_t*>(&r);
}

// tanh of a packed pair of 16-bit values (one MUFU operation for the pair)
template <typename T16>
__device__ __forceinline__ uint32_t tanh2(uint32_t v);
template <>
__device__ __forceinline__ uint32_t tanh2<__nv_bfloat16>(uint32_t v) {
  uint32_t r;
  asm("tanh.approx.bf16x2 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
template <>
__device__ __forceinline__ uint32_t tanh2<__half>(uint32_t v) {
  uint32_t r;
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
// Packed 16-bit multiply of two values by one scalar (both given as packed pairs).  The reference forms
// X*dt and the decay-scaled operands in half precision too (model_ref.py:144,148).
template <typename T16>
__device__ __forceinline__ uint32_t mul2(uint32_t v, uint32_t s2);
template <>
__device__ __forceinline__ uint32_t mul2<__nv_bfloat16>(uint32_t v, uint32_t s2) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&v), *reinterpret_cast<const __nv_bfloat162*>(&s2));
  return *reinterpret_cast<uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t mul2<__half>(uint32_t v, uint32_t s2) {
  __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&v), *reinterpret_cast<const __half2*>(&s2));
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}


// ---------------------------------------------------------------------------- host side

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library has no
// link-time dependency on libcuda and loads on machines without a GPU.
inline EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

// [b, s, heads, inner] 16-bit tensor viewed innermost-first; box = 64 inner x 1 head x 128 tokens x 1 batch.
inline bool make_map(CUtensorMap* tm, const void* base, int dtype, int inner, int heads, int s, int b, const int64_t* st) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)heads, (cuuint64_t)s, (cuuint64_t)b};
  const cuuint64_t strides[3] = {(cuuint64_t)st[2] * 2, (cuuint64_t)st[1] * 2, (cuuint64_t)st[0] * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)T, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(tm, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool ok16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool stride_ok(const int64_t* st) {
  for (int i = 0; i < 3; ++i)
    if (st[i] <= 0 || st[i] % 8 != 0 || st[i] * 2 >= ((int64_t)1 << 40)) return false;
  return true;
}


}  // namespace tc
}  // namespace ssd
