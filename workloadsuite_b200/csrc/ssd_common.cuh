// Shared definitions of the SSD forward kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ssd_b200.h"

namespace ssd {

// Device status codes written to SsdArgs::status (0 = fine).
enum : int {
  STATUS_OK = 0,
  STATUS_WAIT_TIMEOUT_TMA = 1,   // a bounded wait for a TMA transfer ran out
  STATUS_WAIT_TIMEOUT_MMA = 2,   // a bounded wait for a tcgen05 commit ran out
  STATUS_WAIT_TIMEOUT_SYNC = 3,  // a bounded wait between warps of one CTA ran out
  STATUS_TMEM_ALLOC = 4,         // tensor memory could not be allocated
  STATUS_BAD_SMEM_ALIGNMENT = 5, // dynamic shared memory did not start on a 1024-byte boundary
  STATUS_WAIT_TIMEOUT_CHAIN = 6  // a bounded wait for the previous segment of a chained sequence ran out
};

// One launch of a scan over [seg_begin, seg_end) of every (batch, head) unit.
// Strides are in elements.  "unit" = batch * nheads + head.
struct ScanParams {
  const void* X;
  const float* A;
  const void* B;
  const void* C;
  const void* dt;      // may be null
  void* Y;             // may be null when compute_y == 0
  const float* init;   // state entering segment (unit, seg); null = zeros
  int64_t init_unit_stride, init_seg_stride;
  float* fin;          // state leaving segment (unit, seg); may be null
  int64_t fin_unit_stride, fin_seg_stride;
  float* fin_ld;       // sum of A over the segment; may be null
  int64_t finld_unit_stride, finld_seg_stride;
  int32_t* status;     // may be null
  int batch, seqlen, nheads, p, n, ngroups;
  int seg_len, nseg;
  int compute_y;
  int vec_ok;          // all row starts 16-byte aligned
  long long wait_clocks;   // bound of every device-side wait, in SM clock cycles
  int inject_lost_handover;   // SSD_FLAG_INJECT_LOST_HANDOVER: CTA 0 of a chained launch leaves without working
  // Chained mode (two-head tensor-core kernel only; 1): a piece of a sequence starts from the state that the
  // piece before it (on the neighbouring CTA) left in chain_state, once chain_flag says it is there.
  // Look-back mode (2): chain_state / chain_ld hold each CTA's state-from-zero and log-decay sum of the last
  // piece of its range; a piece folds those of the CTAs before it.
  int chain;
  float* chain_state;     // [slot][n*p], slot = 2 * CTA + head of the pair
  float* chain_ld;        // [slot] running sum of the log-decay up to the end of the piece
  int32_t* chain_flag;    // [slot], zeroed before the launch
  // Optional epilogue Y <- (Y + x * D[head]) * silu(z) (model_ref.py:116-118); either pointer may be null.
  const float* D;         // [h]
  const void* Z;          // [b,s,h,p], strides zs
  int64_t xs[3], as[3], bs[3], cs[3], dts[3], ys[3], zs[3];
};

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Launchers implemented in the kernel translation units.  Each returns an
// SSD_ERR_* code and enqueues on `stream`.
int launch_scan_f32(const ScanParams& prm, int dtype, cudaStream_t stream);
bool scan_f32_supports(int p, int n);
int scan_f32_tile_tokens();

// Y <- (Y + x * D[head]) * silu(z) in place over [b,s,h,p] (for the kernels that do not fuse it).
int launch_epilogue(const ScanParams& p, int dtype, cudaStream_t stream);

// `incoming` (nullable, may alias `states`) receives the state entering every segment, in the layout of `states`.
int launch_fold(const float* states, int64_t st_unit_stride, int64_t st_seg_stride, const float* ld,
                int64_t ld_unit_stride, int64_t ld_seg_stride, const float* init, float* out_single,
                float* out_final, float* out_ld, int upto, float* incoming, int64_t units, int64_t np,
                cudaStream_t stream);

// tcgen05 kernel family (ssd_tcgen05.cu)
bool tc_supports(const SsdArgs& a);
int tc_default_segments(const SsdArgs& a);
int launch_tc(const SsdArgs& a, const ScanParams& prm, cudaStream_t stream);

// two-heads-per-CTA tcgen05 kernel (ssd_tc2.cu): needs an even number of heads per B/C group
bool tc2_supports(const SsdArgs& a);
int tc2_default_segments(const SsdArgs& a);
int tc2_chain_mode(const SsdArgs& a, int nseg);   // 1: chained, 2: look-back (one launch each); 0: two passes + fold
int launch_tc2(const SsdArgs& a, const ScanParams& prm, cudaStream_t stream);


}  // namespace ssd
