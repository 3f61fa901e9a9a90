// C ABI of the SSD forward (declared in include/ssd_b200.h): argument
// validation, kernel choice, sequence segmentation and the host-buffer pipeline.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "ssd_common.cuh"

namespace {

constexpr int kAbiVersion = 3;
constexpr int kSmCount = 148;  // B200

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int elem_size(int dtype) { return dtype == SSD_DTYPE_F32 ? 4 : 2; }

int validate(const SsdArgs* a) {
  if (!a) return SSD_ERR_NULL_POINTER;
  if (a->batch <= 0 || a->seqlen <= 0 || a->nheads <= 0 || a->headdim <= 0 || a->dstate <= 0 || a->ngroups <= 0)
    return SSD_ERR_BAD_SHAPE;
  if (a->nheads % a->ngroups != 0) return SSD_ERR_BAD_SHAPE;
  if (a->chunk <= 0 || a->seqlen % a->chunk != 0) return SSD_ERR_BAD_CHUNK;
  if (a->dtype != SSD_DTYPE_F32 && a->dtype != SSD_DTYPE_F16 && a->dtype != SSD_DTYPE_BF16)
    return SSD_ERR_UNSUPPORTED;
  if (a->kernel != SSD_KERNEL_AUTO && a->kernel != SSD_KERNEL_SCAN_F32 && a->kernel != SSD_KERNEL_TCGEN05)
    return SSD_ERR_UNSUPPORTED;
  if (a->nsegments < 0 || a->wait_limit_ms < 0) return SSD_ERR_BAD_SHAPE;
  if ((int64_t)a->batch * a->nheads > 0x7fffffffLL) return SSD_ERR_TOO_LARGE;
  return SSD_OK;
}

int validate_pointers(const SsdArgs* a) {
  if (!a->X || !a->A || !a->B) return SSD_ERR_NULL_POINTER;
  const bool state_only = (a->flags & SSD_FLAG_STATE_ONLY) != 0;
  if (!state_only && (!a->Y || !a->C)) return SSD_ERR_NULL_POINTER;
  if (state_only && !a->final_state) return SSD_ERR_NULL_POINTER;
  return SSD_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int resolve_kernel(const SsdArgs* a) {
  if (a->kernel == SSD_KERNEL_SCAN_F32) return SSD_KERNEL_SCAN_F32;
  if (a->kernel == SSD_KERNEL_TCGEN05) return SSD_KERNEL_TCGEN05;
  // (states that are only 4-byte aligned go to the fp32 scan, which moves them element by element)
  const bool st16 = aligned16(a->initial_state) && aligned16(a->final_state);
  return ssd::tc_supports(*a) && st16 ? SSD_KERNEL_TCGEN05 : SSD_KERNEL_SCAN_F32;
}

// The two-head kernel whenever the heads of a B/C group come in pairs, else one head per CTA.
bool use_tc2(const SsdArgs* a) { return ssd::tc2_supports(*a); }

int tile_tokens(int kernel) { return kernel == SSD_KERNEL_TCGEN05 ? 128 : ssd::scan_f32_tile_tokens(); }

// Number of independently scanned segments per sequence and their length.
void resolve_segments(const SsdArgs* a, int kernel, int* nseg, int* seg_len) {
  const int tile = tile_tokens(kernel);
  int want = a->nsegments;
  if (want <= 0) {
    if (kernel == SSD_KERNEL_TCGEN05) {
      want = use_tc2(a) ? ssd::tc2_default_segments(*a) : ssd::tc_default_segments(*a);
    } else {
      const int64_t units = (int64_t)a->batch * a->nheads;
      // Two passes cost about 1.5x the work of one, so split only when the
      // unsplit grid would leave most of the SMs idle.
      want = units >= (3 * kSmCount) / 2 ? 1 : (int)((4 * kSmCount + units - 1) / units);
      const int max_by_len = std::max(1, a->seqlen / 256);
      want = std::min(want, max_by_len);
    }
  }
  want = std::max(1, std::min(want, 65535));
  int len = (a->seqlen + want - 1) / want;
  len = (len + tile - 1) / tile * tile;
  *seg_len = len;
  *nseg = (a->seqlen + len - 1) / len;
}

bool strides_mult(const int64_t* s, int m) { return s[0] % m == 0 && s[1] % m == 0 && s[2] % m == 0; }

void fill_params(const SsdArgs* a, ssd::ScanParams* p) {
  std::memset(p, 0, sizeof(*p));
  p->X = a->X; p->A = a->A; p->B = a->B; p->C = a->C; p->dt = a->dt; p->Y = a->Y;
  p->D = a->D; p->Z = a->Z;
  p->status = a->status;
  p->batch = a->batch; p->seqlen = a->seqlen; p->nheads = a->nheads; p->p = a->headdim; p->n = a->dstate;
  p->ngroups = a->ngroups;
  for (int i = 0; i < 3; ++i) {
    p->xs[i] = a->x_stride[i]; p->as[i] = a->a_stride[i]; p->bs[i] = a->b_stride[i];
    p->cs[i] = a->c_stride[i]; p->dts[i] = a->dt_stride[i]; p->ys[i] = a->y_stride[i];
    p->zs[i] = a->z_stride[i];
  }
  const int per16 = 16 / elem_size(a->dtype);
  bool v = aligned16(a->X) && aligned16(a->B) && strides_mult(a->x_stride, per16) &&
           strides_mult(a->b_stride, per16) && a->headdim % 8 == 0 && a->dstate % 8 == 0;
  if (a->C) v = v && aligned16(a->C) && strides_mult(a->c_stride, per16);
  if (a->Y) v = v && aligned16(a->Y) && strides_mult(a->y_stride, per16);
  if (a->Z) v = v && aligned16(a->Z) && strides_mult(a->z_stride, per16);
  p->vec_ok = v ? 1 : 0;
  // the bound of the device-side waits: about a second by default; SM clocks run at up to ~2 GHz
  p->wait_clocks = a->wait_limit_ms > 0 ? (long long)a->wait_limit_ms * 2000000LL : 2000000000LL;
  p->inject_lost_handover = (a->flags & SSD_FLAG_INJECT_LOST_HANDOVER) ? 1 : 0;
}

// The gate rows are read with 16-byte loads by the fused epilogue; the stand-alone kernel has a scalar path.
bool z_vector_friendly(const SsdArgs* a) {
  if (!a->Z) return true;
  const int per16 = 16 / elem_size(a->dtype);
  return aligned16(a->Z) && strides_mult(a->z_stride, per16);
}

// The tensor-core kernels move the fp32 states as 16-byte vectors.
bool states_aligned16(const SsdArgs* a) { return aligned16(a->initial_state) && aligned16(a->final_state); }

int launch_kernel(int kernel, const SsdArgs* a, const ssd::ScanParams& prm, cudaStream_t stream) {
  if (kernel == SSD_KERNEL_TCGEN05) return use_tc2(a) ? ssd::launch_tc2(*a, prm, stream) : ssd::launch_tc(*a, prm, stream);
  return ssd::launch_scan_f32(prm, a->dtype, stream);
}

}  // namespace

extern "C" {

int ssd_b200_abi_version(void) { return kAbiVersion; }

const char* ssd_b200_strerror(int code) {
  switch (code) {
    case SSD_OK: return "ok";
    case SSD_ERR_NULL_POINTER: return "a required pointer is NULL";
    case SSD_ERR_BAD_SHAPE: return "invalid shape (sizes must be positive; n_heads must be divisible by n_groups)";
    case SSD_ERR_BAD_CHUNK: return "seq_len must be a positive multiple of chunk";
    case SSD_ERR_UNSUPPORTED: return "shape, dtype or kernel not supported by this build";
    case SSD_ERR_WORKSPACE: return "workspace missing or too small";
    case SSD_ERR_CUDA: return "a CUDA runtime call failed";
    case SSD_ERR_MISALIGNED: return "pointer or stride not aligned for the selected kernel";
    case SSD_ERR_TOO_LARGE: return "size beyond a fixed limit";
    case SSD_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out; the results are incomplete";
    default: return "unknown error code";
  }
}

const char* ssd_b200_kernel_name(const SsdArgs* args) {
  if (validate(args) != SSD_OK) return "invalid";
  return resolve_kernel(args) == SSD_KERNEL_TCGEN05 ? "tcgen05" : "scan_f32";
}

int ssd_b200_plan(const SsdArgs* args, int32_t* kernel_out, int32_t* nsegments_out, int32_t* launches_out) {
  const int rc = validate(args);
  if (rc != SSD_OK) return rc;
  const int kernel = resolve_kernel(args);
  int nseg, seg_len;
  resolve_segments(args, kernel, &nseg, &seg_len);
  const bool state_only = (args->flags & SSD_FLAG_STATE_ONLY) != 0;
  int launches = 1;
  if (nseg > 1) {
    const bool chained = kernel == SSD_KERNEL_TCGEN05 && use_tc2(args) && ssd::tc2_chain_mode(*args, nseg) != 0;
    launches = chained ? 1 : (state_only ? 2 : 3);
    if (!chained && (args->flags & SSD_FLAG_REUSE_SEGMENTS)) launches -= 1;
  }
  if (kernel_out) *kernel_out = kernel;
  if (nsegments_out) *nsegments_out = nseg;
  if (launches_out) *launches_out = launches;
  return SSD_OK;
}

size_t ssd_b200_workspace_bytes(const SsdArgs* args) {
  if (validate(args) != SSD_OK) return 0;
  const int kernel = resolve_kernel(args);
  int nseg, seg_len;
  resolve_segments(args, kernel, &nseg, &seg_len);
  if (nseg <= 1) return 0;
  const size_t units = (size_t)args->batch * args->nheads;
  const size_t np = (size_t)args->dstate * args->headdim;
  if (kernel == SSD_KERNEL_TCGEN05 && use_tc2(args) && ssd::tc2_chain_mode(*args, nseg) != 0) {
    // chained / look-back mode: one slot per CTA and head of the pair -- state, log-decay sum, ready flag
    const size_t slots = 2 * (size_t)kSmCount;
    return align_up(slots * np * sizeof(float), 256) + 2 * align_up(slots * sizeof(float), 256);
  }
  // two passes: zero-start segment states, states entering the segments, segment log-decay sums
  return 2 * align_up(units * nseg * np * sizeof(float), 256) + align_up(units * nseg * sizeof(float), 256);
}

// The forward proper.  `fuse_epilogue`: the selected kernel applies D / Z itself; otherwise they are dropped here
// and ssd_b200_forward() runs the stand-alone epilogue kernel afterwards.
static int forward_impl(const SsdArgs* args, void* stream_v, bool fuse_epilogue) {
  int rc = validate(args);
  if (rc != SSD_OK) return rc;
  rc = validate_pointers(args);
  if (rc != SSD_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int kernel = resolve_kernel(args);
  if (kernel == SSD_KERNEL_TCGEN05 && !ssd::tc_supports(*args)) return SSD_ERR_UNSUPPORTED;
  if (kernel == SSD_KERNEL_TCGEN05 && !states_aligned16(args)) return SSD_ERR_MISALIGNED;
  if (kernel == SSD_KERNEL_SCAN_F32 && !ssd::scan_f32_supports(args->headdim, args->dstate))
    return SSD_ERR_UNSUPPORTED;

  int nseg, seg_len;
  resolve_segments(args, kernel, &nseg, &seg_len);
  const bool state_only = (args->flags & SSD_FLAG_STATE_ONLY) != 0;
  const int64_t units = (int64_t)args->batch * args->nheads;
  const int64_t np = (int64_t)args->dstate * args->headdim;

  ssd::ScanParams prm;
  fill_params(args, &prm);
  prm.seg_len = seg_len;
  prm.nseg = nseg;
  if (!fuse_epilogue || state_only) prm.D = nullptr, prm.Z = nullptr;

  if (nseg <= 1) {
    prm.compute_y = state_only ? 0 : 1;
    prm.init = args->initial_state;
    prm.init_unit_stride = np;
    prm.fin = args->final_state;
    prm.fin_unit_stride = np;
    prm.fin_ld = args->final_logdecay;
    prm.finld_unit_stride = 1;
    return launch_kernel(kernel, args, prm, stream);
  }

  const size_t need = ssd_b200_workspace_bytes(args);
  if (!args->workspace || args->workspace_bytes < need) return SSD_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(args->workspace) & 255) return SSD_ERR_MISALIGNED;
  const int chain_mode = (kernel == SSD_KERNEL_TCGEN05 && use_tc2(args)) ? ssd::tc2_chain_mode(*args, nseg) : 0;
  if (chain_mode != 0) {
    // one launch: the pieces of a sequence pass their state through the workspace, one slot per CTA and head
    const size_t slots = 2 * (size_t)kSmCount;
    char* ws = static_cast<char*>(args->workspace);
    float* slot_state = reinterpret_cast<float*>(ws);
    float* slot_ld = reinterpret_cast<float*>(ws + align_up(slots * np * sizeof(float), 256));
    int32_t* flags = reinterpret_cast<int32_t*>(reinterpret_cast<char*>(slot_ld) + align_up(slots * sizeof(float), 256));
    // the ready flags must start at zero (the workspace keeps the previous call's contents)
    if (cudaMemsetAsync(flags, 0, slots * sizeof(int32_t), stream) != cudaSuccess) return SSD_ERR_CUDA;
    ssd::ScanParams pc = prm;
    pc.compute_y = state_only ? 0 : 1;
    pc.chain = chain_mode;
    pc.chain_state = slot_state;
    pc.chain_ld = slot_ld;
    pc.chain_flag = flags;
    pc.init = args->initial_state;   // only read by the first segment
    pc.init_unit_stride = np;
    pc.init_seg_stride = 0;
    pc.fin = args->final_state;      // only written by the last segment
    pc.fin_unit_stride = np;
    pc.fin_seg_stride = 0;
    pc.fin_ld = args->final_logdecay;
    pc.finld_unit_stride = 1;
    pc.finld_seg_stride = 0;
    return launch_kernel(kernel, args, pc, stream);
  }

  float* seg_states = static_cast<float*>(args->workspace);
  const size_t st_bytes = align_up((size_t)units * nseg * np * sizeof(float), 256);
  float* seg_in = reinterpret_cast<float*>(static_cast<char*>(args->workspace) + st_bytes);
  float* seg_ld = reinterpret_cast<float*>(static_cast<char*>(args->workspace) + 2 * st_bytes);

  // pass 1: every segment from a zero state, state and log-decay sum only
  if (!(args->flags & SSD_FLAG_REUSE_SEGMENTS)) {
    ssd::ScanParams p1 = prm;
    p1.compute_y = 0;
    p1.Y = nullptr;
    p1.init = nullptr;
    p1.fin = seg_states;
    p1.fin_unit_stride = (int64_t)nseg * np;
    p1.fin_seg_stride = np;
    p1.fin_ld = seg_ld;
    p1.finld_unit_stride = nseg;
    p1.finld_seg_stride = 1;
    rc = launch_kernel(kernel, args, p1, stream);
    if (rc != SSD_OK) return rc;
  }

  // fold: state entering each segment (kept apart from the zero-start states, so that those can be
  // reused), final state, total log-decay
  rc = ssd::launch_fold(seg_states, (int64_t)nseg * np, np, seg_ld, nseg, 1, args->initial_state, nullptr,
                        args->final_state, args->final_logdecay, nseg, state_only ? nullptr : seg_in, units, np,
                        stream);
  if (rc != SSD_OK || state_only) return rc;

  // pass 2: every segment again, seeded with its incoming state, writing Y
  ssd::ScanParams p2 = prm;
  p2.compute_y = 1;
  p2.init = seg_in;
  p2.init_unit_stride = (int64_t)nseg * np;
  p2.init_seg_stride = np;
  p2.fin = nullptr;
  p2.fin_ld = nullptr;
  return launch_kernel(kernel, args, p2, stream);
}

int ssd_b200_forward(const SsdArgs* args, void* stream_v) {
  int rc = validate(args);
  if (rc != SSD_OK) return rc;
  const bool state_only = (args->flags & SSD_FLAG_STATE_ONLY) != 0;
  if (state_only || (!args->D && !args->Z)) return forward_impl(args, stream_v, false);
  // skip and gate of model_ref.py:116-118: fused into the two-head tensor-core kernel, a kernel of their own otherwise
  const int kernel = resolve_kernel(args);
  const bool fuse = kernel == SSD_KERNEL_TCGEN05 && ssd::tc_supports(*args) && use_tc2(args) &&
                    z_vector_friendly(args) && !(args->flags & SSD_FLAG_SEPARATE_EPILOGUE);
  rc = forward_impl(args, stream_v, fuse);
  if (rc != SSD_OK || fuse) return rc;
  ssd::ScanParams ep;
  fill_params(args, &ep);
  return ssd::launch_epilogue(ep, args->dtype, static_cast<cudaStream_t>(stream_v));
}

int ssd_b200_fold_states(const float* states, int64_t states_shard_stride, const float* logdecay,
                         int64_t logdecay_shard_stride, const float* initial, float* out, int32_t nshards,
                         int32_t rank, int64_t units, int64_t np, void* stream) {
  if (!states || !logdecay || !out) return SSD_ERR_NULL_POINTER;
  if (nshards <= 0 || rank < 0 || rank > nshards || units <= 0 || np <= 0) return SSD_ERR_BAD_SHAPE;
  return ssd::launch_fold(states, np, states_shard_stride, logdecay, 1, logdecay_shard_stride, initial, out, nullptr,
                          nullptr, rank, nullptr, units, np, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
