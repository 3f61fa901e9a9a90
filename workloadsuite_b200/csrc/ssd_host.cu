// Host-buffer entry point: the SSD forward for callers whose tensors live in
// host memory.  The (batch, head-block) slices of the problem are independent
// scans, so the call is a three-stage pipeline over slices: host->device copy
// of slice i+1, kernels of slice i and device->host copy of slice i-1 run on
// three streams and overlap (PCIe is full duplex).
#include <algorithm>
#include <cstring>
#include <vector>

#include "ssd_common.cuh"

namespace {

constexpr int kSlots = 3;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
int esize(int dtype) { return dtype == SSD_DTYPE_F32 ? 4 : 2; }

struct Plan {
  int head_block;     // heads per slice
  int groups_block;   // groups a slice touches (>= 1)
  size_t x_bytes, a_bytes, y_bytes, dt_bytes, st_bytes, bc_bytes, ws_bytes, ld_bytes;
  size_t slot_bytes, batch_bytes, total_bytes;
};

bool basic_ok(const SsdArgs* a) {
  return a && a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->headdim > 0 && a->dstate > 0 && a->ngroups > 0 &&
         a->nheads % a->ngroups == 0 && a->chunk > 0 && a->seqlen % a->chunk == 0 &&
         (a->dtype == SSD_DTYPE_F32 || a->dtype == SSD_DTYPE_F16 || a->dtype == SSD_DTYPE_BF16);
}

void slice_args(const SsdArgs* a, int hb, SsdArgs* s) {
  const int hpg = a->nheads / a->ngroups;
  *s = *a;
  s->batch = 1;
  s->nheads = hb;
  s->ngroups = hb >= hpg ? hb / hpg : 1;
  s->flags = a->flags;
}

Plan make_plan(const SsdArgs* a) {
  Plan pl{};
  const int hpg = a->nheads / a->ngroups;
  const int e = esize(a->dtype);
  // Largest head block (dividing the heads, compatible with the groups) whose
  // X slice stays at or below ~32 MiB, so that several slices are in flight.
  const size_t per_head = (size_t)a->seqlen * a->headdim * e;
  const size_t total = per_head * a->nheads * a->batch;
  const size_t cap = std::max<size_t>((size_t)1 << 20, std::min<size_t>((size_t)32 << 20, total / 6));
  int best = 0;
  for (int hb = a->nheads; hb >= 1; --hb) {
    if (a->nheads % hb) continue;
    if (!(hb % hpg == 0 || hpg % hb == 0)) continue;
    if (best == 0) best = hb;
    if (per_head * hb <= cap || hb == 1) { best = hb; break; }
    best = hb;
  }
  pl.head_block = best;
  pl.groups_block = best >= hpg ? best / hpg : 1;
  pl.x_bytes = align_up(per_head * best, 256);
  pl.y_bytes = pl.x_bytes;
  pl.a_bytes = align_up((size_t)a->seqlen * a->nheads * 4, 256);
  pl.dt_bytes = a->dt ? align_up((size_t)a->seqlen * a->nheads * e, 256) : 0;
  pl.st_bytes = align_up((size_t)best * a->dstate * a->headdim * 4, 256);
  pl.ld_bytes = align_up((size_t)best * 4, 256);
  pl.bc_bytes = align_up((size_t)a->seqlen * a->ngroups * a->dstate * e, 256);
  SsdArgs s;
  slice_args(a, best, &s);
  pl.ws_bytes = align_up(ssd_b200_workspace_bytes(&s), 256);
  pl.slot_bytes = pl.x_bytes + pl.y_bytes + 2 * pl.st_bytes + pl.ld_bytes + pl.ws_bytes;
  pl.batch_bytes = 2 * pl.bc_bytes + pl.a_bytes + pl.dt_bytes;  // B, C, A, dt of one batch entry
  pl.total_bytes = kSlots * pl.slot_bytes + 2 * pl.batch_bytes + 256;
  return pl;
}

}  // namespace

extern "C" {

size_t ssd_b200_host_scratch_bytes(const SsdArgs* host) {
  if (!basic_ok(host)) return 0;
  return make_plan(host).total_bytes;
}

int ssd_b200_forward_host(const SsdArgs* host, void* dev_scratch, size_t dev_scratch_bytes) {
  if (!host) return SSD_ERR_NULL_POINTER;
  if (!basic_ok(host)) {
    if (host->nheads > 0 && host->ngroups > 0 && host->chunk > 0 && host->seqlen > 0 &&
        host->nheads % host->ngroups == 0 && host->seqlen % host->chunk != 0)
      return SSD_ERR_BAD_CHUNK;
    return SSD_ERR_BAD_SHAPE;
  }
  const bool state_only = (host->flags & SSD_FLAG_STATE_ONLY) != 0;
  if (!host->X || !host->A || !host->B) return SSD_ERR_NULL_POINTER;
  if (!state_only && (!host->Y || !host->C)) return SSD_ERR_NULL_POINTER;
  if (state_only && !host->final_state) return SSD_ERR_NULL_POINTER;
  if (host->D || host->Z) return SSD_ERR_UNSUPPORTED;   // the skip/gate epilogue is a device-buffer feature
  const Plan pl = make_plan(host);
  if (!dev_scratch || dev_scratch_bytes < pl.total_bytes) return SSD_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(dev_scratch) & 255) return SSD_ERR_MISALIGNED;

  const int e = esize(host->dtype);
  const int b = host->batch, s = host->seqlen, h = host->nheads, p = host->headdim, n = host->dstate,
            g = host->ngroups, hb = pl.head_block, hpg = h / g;
  const int blocks_per_batch = h / hb;
  const int nslices = b * blocks_per_batch;

  cudaStream_t st_in = nullptr, st_run = nullptr, st_out = nullptr;
  std::vector<cudaEvent_t> ev_in(nslices, nullptr), ev_run(nslices, nullptr), ev_out(nslices, nullptr);
  int rc = SSD_OK;
  auto ck = [&](cudaError_t err) { if (err != cudaSuccess && rc == SSD_OK) rc = SSD_ERR_CUDA; };
  ck(cudaStreamCreateWithFlags(&st_in, cudaStreamNonBlocking));
  ck(cudaStreamCreateWithFlags(&st_run, cudaStreamNonBlocking));
  ck(cudaStreamCreateWithFlags(&st_out, cudaStreamNonBlocking));
  for (int i = 0; i < nslices && rc == SSD_OK; ++i) {
    ck(cudaEventCreateWithFlags(&ev_in[i], cudaEventDisableTiming));
    ck(cudaEventCreateWithFlags(&ev_run[i], cudaEventDisableTiming));
    ck(cudaEventCreateWithFlags(&ev_out[i], cudaEventDisableTiming));
  }

  char* base = static_cast<char*>(dev_scratch);
  char* bc_base = base + kSlots * pl.slot_bytes;
  const char* hX = static_cast<const char*>(host->X);
  const char* hB = static_cast<const char*>(host->B);
  const char* hC = static_cast<const char*>(host->C);
  const char* hD = static_cast<const char*>(host->dt);
  char* hY = static_cast<char*>(host->Y);

  for (int i = 0; i < nslices && rc == SSD_OK; ++i) {
    const int bi = i / blocks_per_batch, blk = i % blocks_per_batch, h0 = blk * hb;
    char* slot = base + (size_t)(i % kSlots) * pl.slot_bytes;
    char* dX = slot;
    char* dY = dX + pl.x_bytes;
    char* dI = dY + pl.y_bytes;
    char* dF = dI + pl.st_bytes;
    char* dL = dF + pl.st_bytes;
    char* dW = dL + pl.ld_bytes;
    char* dB = bc_base + (size_t)(bi & 1) * pl.batch_bytes;
    char* dC = dB + pl.bc_bytes;
    char* dA = dC + pl.bc_bytes;
    char* dD = dA + pl.a_bytes;

    // stage 1: copies in (the slot is free once the slice that used it has left)
    if (i >= kSlots) ck(cudaStreamWaitEvent(st_in, ev_out[i - kSlots], 0));
    if (blk == 0) {
      // B, C, A, dt of this batch entry go to the buffer last used by entry bi-2
      if (bi >= 2) ck(cudaStreamWaitEvent(st_in, ev_run[(bi - 1) * blocks_per_batch - 1], 0));
      const size_t bytes = (size_t)s * g * n * e;
      ck(cudaMemcpyAsync(dB, hB + (size_t)bi * bytes, bytes, cudaMemcpyHostToDevice, st_in));
      if (hC) ck(cudaMemcpyAsync(dC, hC + (size_t)bi * bytes, bytes, cudaMemcpyHostToDevice, st_in));
      ck(cudaMemcpyAsync(dA, host->A + (size_t)bi * s * h, (size_t)s * h * 4, cudaMemcpyHostToDevice, st_in));
      if (hD) ck(cudaMemcpyAsync(dD, hD + (size_t)bi * s * h * e, (size_t)s * h * e, cudaMemcpyHostToDevice, st_in));
    }
    ck(cudaMemcpy2DAsync(dX, (size_t)hb * p * e, hX + ((size_t)bi * s * h + h0) * p * e, (size_t)h * p * e,
                         (size_t)hb * p * e, s, cudaMemcpyHostToDevice, st_in));
    if (host->initial_state)
      ck(cudaMemcpyAsync(dI, host->initial_state + ((size_t)bi * h + h0) * n * p, (size_t)hb * n * p * 4,
                         cudaMemcpyHostToDevice, st_in));
    ck(cudaEventRecord(ev_in[i], st_in));

    // stage 2: kernels
    ck(cudaStreamWaitEvent(st_run, ev_in[i], 0));
    SsdArgs sa;
    slice_args(host, hb, &sa);
    const int g0 = h0 / hpg;
    sa.X = dX; sa.A = reinterpret_cast<const float*>(dA) + h0;
    sa.B = dB + (size_t)g0 * n * e;
    sa.C = hC ? dC + (size_t)g0 * n * e : nullptr;
    sa.dt = hD ? dD + (size_t)h0 * e : nullptr;
    sa.initial_state = host->initial_state ? reinterpret_cast<const float*>(dI) : nullptr;
    sa.Y = state_only ? nullptr : dY;
    sa.final_state = host->final_state ? reinterpret_cast<float*>(dF) : nullptr;
    sa.final_logdecay = host->final_logdecay ? reinterpret_cast<float*>(dL) : nullptr;
    sa.workspace = pl.ws_bytes ? dW : nullptr;
    sa.workspace_bytes = pl.ws_bytes;
    sa.status = nullptr;
    const int64_t xs[3] = {(int64_t)s * hb * p, (int64_t)hb * p, p};
    const int64_t as[3] = {(int64_t)s * h, h, 1};
    const int64_t bs[3] = {(int64_t)s * g * n, (int64_t)g * n, n};
    for (int k = 0; k < 3; ++k) {
      sa.x_stride[k] = xs[k]; sa.y_stride[k] = xs[k]; sa.a_stride[k] = as[k]; sa.dt_stride[k] = as[k];
      sa.b_stride[k] = bs[k]; sa.c_stride[k] = bs[k];
    }
    if (rc == SSD_OK) {
      const int frc = ssd_b200_forward(&sa, st_run);
      if (frc != SSD_OK) rc = frc;
    }
    ck(cudaEventRecord(ev_run[i], st_run));

    // stage 3: copies out
    ck(cudaStreamWaitEvent(st_out, ev_run[i], 0));
    if (!state_only)
      ck(cudaMemcpy2DAsync(hY + ((size_t)bi * s * h + h0) * p * e, (size_t)h * p * e, dY, (size_t)hb * p * e,
                           (size_t)hb * p * e, s, cudaMemcpyDeviceToHost, st_out));
    if (host->final_state)
      ck(cudaMemcpyAsync(host->final_state + ((size_t)bi * h + h0) * n * p, dF, (size_t)hb * n * p * 4,
                         cudaMemcpyDeviceToHost, st_out));
    if (host->final_logdecay)
      ck(cudaMemcpyAsync(host->final_logdecay + (size_t)bi * h + h0, dL, (size_t)hb * 4, cudaMemcpyDeviceToHost,
                         st_out));
    ck(cudaEventRecord(ev_out[i], st_out));
  }

  if (st_in) ck(cudaStreamSynchronize(st_in));
  if (st_run) ck(cudaStreamSynchronize(st_run));
  if (st_out) ck(cudaStreamSynchronize(st_out));
  for (auto* v : {&ev_in, &ev_run, &ev_out})
    for (cudaEvent_t ev : *v)
      if (ev) cudaEventDestroy(ev);
  if (st_in) cudaStreamDestroy(st_in);
  if (st_run) cudaStreamDestroy(st_run);
  if (st_out) cudaStreamDestroy(st_out);
  return rc;
}

}  // extern "C"
