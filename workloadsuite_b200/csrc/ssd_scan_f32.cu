// fp32 CUDA-core SSD scan: the token-by-token recurrence
//   H_t = exp(a_t) H_{t-1} + B_t (x) (x_t dt_t),   y_t = C_t . H_t
// which the chunked form of the reference (model_ref.py:135-162) is
// algebraically equal to.  It is the exact-arithmetic path (fp32 inputs, the
// 1e-4 tolerance) and the fallback for shapes the tensor-core kernel does not
// cover.  One CTA walks one (batch, head[, segment]) with the n x p state held
// in registers: thread (j, sl) owns column j of the state and the rows
// n_i = (k*SL + sl)*4 + q, so the B/C rows are read from shared memory as
// conflict-free float4 broadcasts and y_t is finished by a shuffle over the SL
// lanes that share a column.
#include <algorithm>
#include "ssd_common.cuh"

namespace ssd {

namespace {

constexpr int kThreads = 256;
constexpr int kTile = 32;  // tokens staged in shared memory per step

template <typename T>
__device__ __forceinline__ void load8(const T* src, float* dst);

template <>
__device__ __forceinline__ void load8<__half>(const __half* src, float* dst) {
  uint4 v = *reinterpret_cast<const uint4*>(src);
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    dst[2 * i] = f.x;
    dst[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* src, float* dst) {
  uint4 v = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    dst[2 * i] = f.x;
    dst[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* src, float* dst) {
  float4 a = *reinterpret_cast<const float4*>(src);
  float4 b = *reinterpret_cast<const float4*>(src + 4);
  dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
  dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
}

template <typename T>
__device__ __forceinline__ void store8(T* dst, const float* src);
template <>
__device__ __forceinline__ void store8<__half>(__half* dst, const float* src) {
  uint4 v;
  __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(src[2 * i], src[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float* src) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(src[2 * i], src[2 * i + 1]);
  *reinterpret_cast<uint4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float* src) {
  *reinterpret_cast<float4*>(dst) = make_float4(src[0], src[1], src[2], src[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(src[4], src[5], src[6], src[7]);
}

// Copies `rows` rows of `width` elements (row r at src + r*row_stride) into a
// dense fp32 [rows][width] shared-memory tile, optionally scaling row r by
// scale[r].
template <typename T>
__device__ __forceinline__ void stage_rows(const T* src, int64_t row_stride, int rows, int width, float* dst,
                                           bool vec_ok, int tid) {
  if (vec_ok) {
    const int per_row = width >> 3;
    for (int i = tid; i < rows * per_row; i += kThreads) {
      const int r = i / per_row, c = (i - r * per_row) << 3;
      load8<T>(src + r * row_stride + c, dst + r * width + c);
    }
  } else {
    for (int i = tid; i < rows * width; i += kThreads) {
      const int r = i / width, c = i - r * width;
      dst[r * width + c] = Cvt<T>::to_f(src[r * row_stride + c]);
    }
  }
}

template <typename T, int NS, int P>
__global__ void __launch_bounds__(kThreads) ssd_scan_f32_kernel(const ScanParams prm) {
  constexpr int SL = kThreads / P;  // lanes sharing one state column
  constexpr int NS4 = NS / 4;
  extern __shared__ __align__(16) float smem[];
  const int n = prm.n;
  float* Xs = smem;                  // [kTile][P]   x_t * dt_t
  float* Bs = Xs + kTile * P;        // [kTile][n]
  float* Cs = Bs + kTile * n;        // [kTile][n]
  float* Ys = Cs + kTile * n;        // [kTile][P]
  float* dec = Ys + kTile * P;       // [kTile]  exp(a_t)
  float* araw = dec + kTile;         // [kTile]  a_t

  const int unit = blockIdx.x;
  const int seg = blockIdx.y;
  const int bi = unit / prm.nheads, hi = unit - bi * prm.nheads;
  const int gi = hi / (prm.nheads / prm.ngroups);
  const int tid = threadIdx.x;
  const int j = tid / SL, sl = tid - j * SL;
  const bool vec_ok = prm.vec_ok != 0;

  const int t_begin = seg * prm.seg_len;
  const int t_end = min(prm.seqlen, t_begin + prm.seg_len);

  const T* Xg = static_cast<const T*>(prm.X) + bi * prm.xs[0] + hi * prm.xs[2];
  const T* Bg = static_cast<const T*>(prm.B) + bi * prm.bs[0] + gi * prm.bs[2];
  const T* Cg = static_cast<const T*>(prm.C) + bi * prm.cs[0] + gi * prm.cs[2];
  const float* Ag = prm.A + bi * prm.as[0] + hi * prm.as[2];
  const T* Dg = prm.dt ? static_cast<const T*>(prm.dt) + bi * prm.dts[0] + hi * prm.dts[2] : nullptr;
  T* Yg = prm.Y ? static_cast<T*>(prm.Y) + bi * prm.ys[0] + hi * prm.ys[2] : nullptr;

  float h[NS];
  if (prm.init) {
    const float* I = prm.init + unit * prm.init_unit_stride + seg * prm.init_seg_stride;
#pragma unroll
    for (int k = 0; k < NS4; ++k)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int ni = (k * SL + sl) * 4 + q;
        h[k * 4 + q] = (ni < n) ? I[(int64_t)ni * P + j] : 0.f;
      }
  } else {
#pragma unroll
    for (int k = 0; k < NS; ++k) h[k] = 0.f;
  }
  double asum = 0.0;

  for (int t0 = t_begin; t0 < t_end; t0 += kTile) {
    const int rows = min(kTile, t_end - t0);
    __syncthreads();  // previous tile fully consumed (Ys stored, Xs/Bs/Cs read)
    stage_rows<T>(Xg + (int64_t)t0 * prm.xs[1], prm.xs[1], rows, P, Xs, vec_ok, tid);
    stage_rows<T>(Bg + (int64_t)t0 * prm.bs[1], prm.bs[1], rows, n, Bs, vec_ok, tid);
    if (prm.compute_y) stage_rows<T>(Cg + (int64_t)t0 * prm.cs[1], prm.cs[1], rows, n, Cs, vec_ok, tid);
    if (tid < rows) {
      const float a = Ag[(int64_t)(t0 + tid) * prm.as[1]];
      araw[tid] = a;
      dec[tid] = expf(a);
    }
    __syncthreads();
    if (Dg) {  // x~ = x * dt (model_ref.py:144)
      for (int i = tid; i < rows * P; i += kThreads) {
        const int r = i / P;
        Xs[i] *= Cvt<T>::to_f(Dg[(int64_t)(t0 + r) * prm.dts[1]]);
      }
      __syncthreads();
    }
    if (prm.compute_y) {
      for (int t = 0; t < rows; ++t) {
        const float x = Xs[t * P + j];
        const float d = dec[t];
        const float4* B4 = reinterpret_cast<const float4*>(Bs + t * n);
        const float4* C4 = reinterpret_cast<const float4*>(Cs + t * n);
        float y = 0.f;
#pragma unroll
        for (int k = 0; k < NS4; ++k) {
          if ((k * SL) * 4 < n) {
            const float4 bv = B4[k * SL + sl];
            const float4 cv = C4[k * SL + sl];
            h[k * 4 + 0] = fmaf(h[k * 4 + 0], d, bv.x * x);
            h[k * 4 + 1] = fmaf(h[k * 4 + 1], d, bv.y * x);
            h[k * 4 + 2] = fmaf(h[k * 4 + 2], d, bv.z * x);
            h[k * 4 + 3] = fmaf(h[k * 4 + 3], d, bv.w * x);
            y = fmaf(cv.x, h[k * 4 + 0], y);
            y = fmaf(cv.y, h[k * 4 + 1], y);
            y = fmaf(cv.z, h[k * 4 + 2], y);
            y = fmaf(cv.w, h[k * 4 + 3], y);
          }
        }
#pragma unroll
        for (int m = 1; m < SL; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
        if (sl == 0) Ys[t * P + j] = y;
      }
    } else {
      for (int t = 0; t < rows; ++t) {
        const float x = Xs[t * P + j];
        const float d = dec[t];
        const float4* B4 = reinterpret_cast<const float4*>(Bs + t * n);
#pragma unroll
        for (int k = 0; k < NS4; ++k) {
          if ((k * SL) * 4 < n) {
            const float4 bv = B4[k * SL + sl];
            h[k * 4 + 0] = fmaf(h[k * 4 + 0], d, bv.x * x);
            h[k * 4 + 1] = fmaf(h[k * 4 + 1], d, bv.y * x);
            h[k * 4 + 2] = fmaf(h[k * 4 + 2], d, bv.z * x);
            h[k * 4 + 3] = fmaf(h[k * 4 + 3], d, bv.w * x);
          }
        }
      }
    }
    if (tid == 0 && prm.fin_ld) {
      for (int t = 0; t < rows; ++t) asum += (double)araw[t];
    }
    if (prm.compute_y) {
      __syncthreads();
      T* Yt = Yg + (int64_t)t0 * prm.ys[1];
      if (vec_ok) {
        constexpr int per_row = P >> 3;
        for (int i = tid; i < rows * per_row; i += kThreads) {
          const int r = i / per_row, c = (i - r * per_row) << 3;
          store8<T>(Yt + r * prm.ys[1] + c, Ys + r * P + c);
        }
      } else {
        for (int i = tid; i < rows * P; i += kThreads) {
          const int r = i / P, c = i - r * P;
          Yt[r * prm.ys[1] + c] = Cvt<T>::from_f(Ys[i]);
        }
      }
    }
  }

  if (prm.fin) {
    float* F = prm.fin + unit * prm.fin_unit_stride + seg * prm.fin_seg_stride;
#pragma unroll
    for (int k = 0; k < NS4; ++k)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int ni = (k * SL + sl) * 4 + q;
        if (ni < n) F[(int64_t)ni * P + j] = h[k * 4 + q];
      }
  }
  if (prm.fin_ld && tid == 0)
    prm.fin_ld[unit * prm.finld_unit_stride + seg * prm.finld_seg_stride] = (float)asum;
}

// H_in(seg) for every segment of every unit, from the zero-start final states:
//   run = init; for seg: emit run; run = run * exp(D_seg) + F_seg.
__global__ void ssd_fold_kernel(const float* states, int64_t st_unit_stride, int64_t st_seg_stride, const float* ld,
                                int64_t ld_unit_stride, int64_t ld_seg_stride, const float* init, float* out_single,
                                float* out_final, float* out_ld, int upto, float* incoming, int64_t np) {
  const int64_t unit = blockIdx.x;
  const int64_t e = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= np) return;
  float run = init ? init[unit * np + e] : 0.f;
  const float* F = states + unit * st_unit_stride + e;
  float* G = incoming ? incoming + unit * st_unit_stride + e : nullptr;   // same layout as `states`
  const float* D = ld + unit * ld_unit_stride;
  for (int s = 0; s < upto; ++s) {
    const float f = F[(int64_t)s * st_seg_stride];
    if (G) G[(int64_t)s * st_seg_stride] = run;
    run = fmaf(run, expf(D[(int64_t)s * ld_seg_stride]), f);
  }
  if (out_single) out_single[unit * np + e] = run;
  if (out_final) out_final[unit * np + e] = run;
  if (out_ld && e == 0) {
    double tot = 0.0;
    for (int s = 0; s < upto; ++s) tot += (double)D[(int64_t)s * ld_seg_stride];
    out_ld[unit] = (float)tot;
  }
}

template <typename T, int NS, int P>
int launch_one(const ScanParams& prm, cudaStream_t stream) {
  const size_t smem = sizeof(float) * (size_t)(2 * kTile * P + 2 * kTile * prm.n + 2 * kTile);
  auto kern = ssd_scan_f32_kernel<T, NS, P>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return SSD_ERR_CUDA;
  }
  dim3 grid((unsigned)(prm.batch * prm.nheads), (unsigned)prm.nseg);
  kern<<<grid, kThreads, smem, stream>>>(prm);
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

template <typename T, int P>
int launch_p(const ScanParams& prm, cudaStream_t stream) {
  constexpr int SL = kThreads / P;
  const int per_thread = prm.n / SL;
  if (per_thread <= 4) return launch_one<T, 4, P>(prm, stream);
  if (per_thread <= 16) return launch_one<T, 16, P>(prm, stream);
  return launch_one<T, 32, P>(prm, stream);
}

template <typename T>
int launch_t(const ScanParams& prm, cudaStream_t stream) {
  switch (prm.p) {
    case 32: return launch_p<T, 32>(prm, stream);
    case 64: return launch_p<T, 64>(prm, stream);
    case 128: return launch_p<T, 128>(prm, stream);
    default: return SSD_ERR_UNSUPPORTED;
  }
}

}  // namespace

bool scan_f32_supports(int p, int n) {
  if (p != 32 && p != 64 && p != 128) return false;
  const int sl = kThreads / p;
  return n > 0 && n % (4 * sl) == 0 && n / sl <= 32;
}

int scan_f32_tile_tokens() { return kTile; }

int launch_scan_f32(const ScanParams& prm, int dtype, cudaStream_t stream) {
  if (!scan_f32_supports(prm.p, prm.n)) return SSD_ERR_UNSUPPORTED;
  switch (dtype) {
    case SSD_DTYPE_F32: return launch_t<float>(prm, stream);
    case SSD_DTYPE_F16: return launch_t<__half>(prm, stream);
    case SSD_DTYPE_BF16: return launch_t<__nv_bfloat16>(prm, stream);
    default: return SSD_ERR_UNSUPPORTED;
  }
}

// ---------------------------------------------------------------------------------------------
// Skip and gate of SSDLayer.forward after the core (model_ref.py:116-118), for the kernels that do
// not fuse it:  Y <- (Y + x * D[head]) * silu(z), fp32 arithmetic, one rounding.  One thread per
// 8 consecutive head-dim elements (16 bytes of a 16-bit row; rows are 16-byte aligned when vec_ok),
// one block per token.
template <typename T>
__global__ void __launch_bounds__(256)
ssd_epilogue_kernel(const ScanParams p) {
  // one block per token row (b, t); its threads walk the row's (head, 8-element vector) pairs: 32-bit index math only
  const int vec = p.p / 8;
  const int b = blockIdx.x / p.seqlen, t = blockIdx.x - b * p.seqlen;
  for (int i = threadIdx.x; i < p.nheads * vec; i += blockDim.x) {
    const int hh = i / vec, v = i - hh * vec;
    T* y = static_cast<T*>(p.Y) + b * p.ys[0] + (int64_t)t * p.ys[1] + hh * p.ys[2] + 8 * v;
    const T* x = static_cast<const T*>(p.X) + b * p.xs[0] + (int64_t)t * p.xs[1] + hh * p.xs[2] + 8 * v;
    const T* z = p.Z ? static_cast<const T*>(p.Z) + b * p.zs[0] + (int64_t)t * p.zs[1] + hh * p.zs[2] + 8 * v : nullptr;
    const float d = p.D ? p.D[hh] : 0.f;
    // eight elements per thread, moved as whole 16-byte (32-byte for fp32) vectors when the rows allow it
    T yv[8], xv[8], zv[8];
    constexpr int kVecs = sizeof(T) * 8 / 16;
    if (p.vec_ok) {
#pragma unroll
      for (int k = 0; k < kVecs; ++k) {
        reinterpret_cast<uint4*>(yv)[k] = reinterpret_cast<const uint4*>(y)[k];
        if (p.D) reinterpret_cast<uint4*>(xv)[k] = reinterpret_cast<const uint4*>(x)[k];
        if (z) reinterpret_cast<uint4*>(zv)[k] = reinterpret_cast<const uint4*>(z)[k];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        yv[e] = y[e];
        if (p.D) xv[e] = x[e];
        if (z) zv[e] = z[e];
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float acc = Cvt<T>::to_f(yv[e]);
      if (p.D) acc = fmaf(Cvt<T>::to_f(xv[e]), d, acc);
      if (z) {
        const float zz = Cvt<T>::to_f(zv[e]);
        acc *= zz / (1.f + __expf(-zz));
      }
      yv[e] = Cvt<T>::from_f(acc);
    }
    if (p.vec_ok) {
#pragma unroll
      for (int k = 0; k < kVecs; ++k) reinterpret_cast<uint4*>(y)[k] = reinterpret_cast<const uint4*>(yv)[k];
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = yv[e];
    }
  }
}

int launch_epilogue(const ScanParams& p, int dtype, cudaStream_t stream) {
  if (!p.D && !p.Z) return SSD_OK;
  if (p.p % 8 != 0) return SSD_ERR_UNSUPPORTED;
  const int64_t rows = (int64_t)p.batch * p.seqlen;
  if (rows > 0x7fffffffLL) return SSD_ERR_TOO_LARGE;
  const int grid = (int)rows;
  const int work = p.nheads * (p.p / 8);
  const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
  if (dtype == SSD_DTYPE_F32) ssd_epilogue_kernel<float><<<grid, threads, 0, stream>>>(p);
  else if (dtype == SSD_DTYPE_F16) ssd_epilogue_kernel<__half><<<grid, threads, 0, stream>>>(p);
  else ssd_epilogue_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

int launch_fold(const float* states, int64_t st_unit_stride, int64_t st_seg_stride, const float* ld,
                int64_t ld_unit_stride, int64_t ld_seg_stride, const float* init, float* out_single,
                float* out_final, float* out_ld, int upto, float* incoming, int64_t units, int64_t np,
                cudaStream_t stream) {
  if (units <= 0 || np <= 0) return SSD_ERR_BAD_SHAPE;
  if (units > 0x7fffffff || (np + 255) / 256 > 65535) return SSD_ERR_TOO_LARGE;
  dim3 grid((unsigned)units, (unsigned)((np + 255) / 256));
  ssd_fold_kernel<<<grid, 256, 0, stream>>>(states, st_unit_stride, st_seg_stride, ld, ld_unit_stride,
                                            ld_seg_stride, init, out_single, out_final, out_ld, upto,
                                            incoming, np);
  return cudaGetLastError() == cudaSuccess ? SSD_OK : SSD_ERR_CUDA;
}

}  // namespace ssd
