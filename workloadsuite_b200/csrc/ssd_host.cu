// Host-buffer entry point: the SSD forward for callers whose tensors live in
// host memory.  Each batch entry is cut along the SEQUENCE into chunks of a few
// thousand tokens: a chunk of X, Y, B, C, A, dt is one contiguous block of host
// memory (plain 1-D copies at full PCIe rate), and the scan carries over from
// chunk to chunk through the fp32 state, which stays on the device.  The call
// is a three-stage pipeline over chunks: host->device copies of chunk i+1,
// kernels of chunk i and device->host copy of chunk i-1 run on three streams
// and overlap (PCIe is full duplex).
#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include "ssd_common.cuh"

namespace {

constexpr int kSlots = 4;
constexpr int kMaxDevices = 64;

// Streams and events of the host-buffer pipeline, created on first use per device and kept.
struct Pipe {
  cudaStream_t st_in = nullptr, st_run = nullptr, st_out = nullptr;
  std::vector<cudaEvent_t> events;
};
Pipe g_pipes[kMaxDevices];
std::mutex g_pipes_mu[kMaxDevices];

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
int esize(int dtype) { return dtype == SSD_DTYPE_F32 ? 4 : 2; }
int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

struct Plan {
  int tokens;      // tokens per chunk (the last chunk of a sequence may be shorter)
  int nchunks;     // chunks per batch entry
  int group;       // batch entries per chunk (> 1 only when a whole entry is much smaller than a chunk)
  size_t x_bytes, a_bytes, dt_bytes, bc_bytes, ws_bytes, ld_bytes, st_bytes;   // a, dt, bc: one whole batch entry
  size_t slot_bytes, entry_bytes, ldall_bytes, total_bytes;
  int nslices;
};

bool basic_ok(const SsdArgs* a) {
  return a && a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->headdim > 0 && a->dstate > 0 && a->ngroups > 0 &&
         a->nheads % a->ngroups == 0 && a->chunk > 0 && a->seqlen % a->chunk == 0 &&
         (a->dtype == SSD_DTYPE_F32 || a->dtype == SSD_DTYPE_F16 || a->dtype == SSD_DTYPE_BF16);
}

// Arguments of the forward over one chunk of one batch entry (pointers are filled in by the caller).
void chunk_args(const SsdArgs* a, int tokens, int entries, SsdArgs* s) {
  *s = *a;
  s->batch = entries;
  s->seqlen = tokens;
  s->nsegments = 0;
  s->status = nullptr;   // (the pipeline points it at the status word inside its device scratch)
  s->D = nullptr;
  s->Z = nullptr;
  // `a` holds HOST pointers: kernel choice and scratch size must follow the device buffers, which are
  // 256-byte aligned, so the tensor pointers are cleared here (a shape query) and set by the pipeline
  s->X = nullptr; s->A = nullptr; s->B = nullptr; s->C = nullptr; s->Y = nullptr;
  s->initial_state = nullptr; s->final_state = nullptr; s->final_logdecay = nullptr;
  s->workspace = nullptr; s->workspace_bytes = 0;
  // the chunk's tensors are contiguous in the device buffers (kernel choice and scratch size depend on the strides)
  const int64_t h = a->nheads, p = a->headdim, g = a->ngroups, n = a->dstate;
  const int64_t xs[3] = {tokens * h * p, h * p, p}, as[3] = {tokens * h, h, 1}, bs[3] = {tokens * g * n, g * n, n};
  for (int k = 0; k < 3; ++k) {
    s->x_stride[k] = xs[k]; s->y_stride[k] = xs[k]; s->a_stride[k] = as[k]; s->dt_stride[k] = as[k];
    s->b_stride[k] = bs[k]; s->c_stride[k] = bs[k];
  }
}

struct Slice { int bi, nb, ci, t0, tokens; bool first, last; };   // nb batch entries from bi on

// The chunks of all batch entries in order.  The first entry opens and the last one closes with a ramp of smaller
// chunks (1/8, 1/8, 1/4, 1/2 of the regular length), so that the device->host stream starts early and the
// host->device stream ends late: the two directions then overlap for all but a fraction of a chunk.
std::vector<Slice> make_slices(const SsdArgs* host, int tokens_per_chunk, int group) {
  std::vector<Slice> slices;
  const int b = host->batch, s = host->seqlen;
  int unit = host->chunk / gcd_int(host->chunk, 128) * 128;
  if (s % unit != 0) unit = host->chunk;
  for (int bi = 0; bi < b && group > 1; bi += group)
    slices.push_back({bi, std::min(group, b - bi), 0, 0, s, true, true});
  for (int bi = 0; bi < b && group == 1; ++bi) {
    std::vector<int> lens;
    int left = s;
    const int ramp[4] = {tokens_per_chunk / 8, tokens_per_chunk / 8, tokens_per_chunk / 4, tokens_per_chunk / 2};
    std::vector<int> head, tail;
    if (bi == 0)
      for (int k = 0; k < 4; ++k) {
        const int len = ramp[k] / unit * unit;
        if (len > 0 && left - len >= tokens_per_chunk) { head.push_back(len); left -= len; }
      }
    if (bi == b - 1)
      for (int k = 0; k < 4; ++k) {
        const int len = ramp[k] / unit * unit;
        if (len > 0 && left - len >= tokens_per_chunk) { tail.insert(tail.begin(), len); left -= len; }
      }
    lens = head;
    while (left > 0) { const int len = std::min(tokens_per_chunk, left); lens.push_back(len); left -= len; }
    // (ramp-down pieces are listed largest first, so that the last copies are the small ones)
    std::sort(tail.begin(), tail.end(), [](int a, int c) { return a > c; });
    lens.insert(lens.end(), tail.begin(), tail.end());
    int t0 = 0;
    for (size_t k = 0; k < lens.size(); ++k) {
      slices.push_back({bi, 1, (int)k, t0, lens[k], k == 0, k + 1 == lens.size()});
      t0 += lens[k];
    }
  }
  return slices;
}

Plan make_plan(const SsdArgs* a) {
  Plan pl{};
  const int e = esize(a->dtype);
  // chunk length: a multiple of the caller's chunk and of the tensor-core tile (128) when the sequence allows,
  // sized so that the X chunk is at most 48 MiB (measured on the 2.7B layer shape, 84 MB of X per batch entry: two chunks
  // of 42 MB per entry 8.5 ms, chunks of 24 / 28 / 56 / 84 MB 8.9 / 9.0 / 9.1 / 9.0 ms; with 8 MiB chunks the copies
  // in both directions together reach 78 GB/s, with 24 MiB and more 82-86 GB/s)
  int unit = a->chunk / gcd_int(a->chunk, 128) * 128;
  if (a->seqlen % unit != 0) unit = a->chunk;
  const size_t per_token = (size_t)a->nheads * a->headdim * e;
  const size_t total = per_token * a->seqlen * a->batch;
  const size_t cap = std::max<size_t>((size_t)1 << 20, std::min<size_t>((size_t)48 << 20, total / 8));
  // ... and a batch entry is cut into equal chunks (no short remainder chunk at the end of every entry)
  long long tokens = (long long)(cap / per_token) / unit * unit;
  tokens = std::max<long long>(unit, std::min<long long>(tokens, a->seqlen));
  {
    const long long pieces = (a->seqlen + tokens - 1) / tokens;
    const long long even = ((a->seqlen + pieces - 1) / pieces + unit - 1) / unit * unit;
    tokens = std::max<long long>(unit, std::min<long long>(even, tokens));
  }
  pl.tokens = (int)tokens;
  pl.nchunks = (a->seqlen + pl.tokens - 1) / pl.tokens;
  // short sequences: several whole batch entries (contiguous in host memory) travel and run as one chunk
  const size_t per_entry = per_token * a->seqlen;
  pl.group = 1;
  if (pl.nchunks == 1 && a->batch > 1 && per_entry * 2 <= cap)
    pl.group = (int)std::min<size_t>((size_t)a->batch, cap / per_entry);
  const size_t k = (size_t)pl.group;
  pl.x_bytes = align_up(per_token * pl.tokens * k, 256);
  pl.a_bytes = align_up(k * a->seqlen * a->nheads * 4, 256);
  pl.dt_bytes = a->dt ? align_up(k * a->seqlen * a->nheads * e, 256) : 0;
  pl.bc_bytes = align_up(k * a->seqlen * a->ngroups * a->dstate * e, 256);
  pl.ld_bytes = align_up(k * a->nheads * 4, 256);
  pl.st_bytes = align_up(k * a->nheads * a->dstate * a->headdim * 4, 256);
  // scratch of the forward: the largest need over every (entries, tokens) shape the pipeline will launch
  const std::vector<Slice> slices = make_slices(a, pl.tokens, pl.group);
  pl.nslices = (int)slices.size();
  pl.ws_bytes = 0;
  int seen_nb = -1, seen_tokens = -1;
  for (const Slice& sl : slices) {
    if (sl.nb == seen_nb && sl.tokens == seen_tokens) continue;
    seen_nb = sl.nb; seen_tokens = sl.tokens;
    SsdArgs s;
    chunk_args(a, sl.tokens, sl.nb, &s);
    pl.ws_bytes = std::max(pl.ws_bytes, align_up(ssd_b200_workspace_bytes(&s), 256));
  }
  // per-slice log-decay sums stay on the device until the end (one copy back)
  pl.ldall_bytes = a->final_logdecay ? align_up((size_t)pl.nslices * k * a->nheads * 4, 256) : 0;
  pl.slot_bytes = 2 * pl.x_bytes + pl.ws_bytes;
  // B, C, A, dt travel once per batch entry (small copies cost a fixed ~10 us each), double-buffered
  pl.entry_bytes = 2 * pl.bc_bytes + pl.a_bytes + pl.dt_bytes;
  // + the carried state (ping-pong), the entering state and the leaving state of a batch entry (two each)
  // + every slice's log-decay sums + the status word of the kernels
  pl.total_bytes = kSlots * pl.slot_bytes + 2 * pl.entry_bytes + 6 * pl.st_bytes + pl.ldall_bytes + 256;
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
  const int b = host->batch, s = host->seqlen, h = host->nheads, p = host->headdim, n = host->dstate, g = host->ngroups;
  const std::vector<Slice> slices = make_slices(host, pl.tokens, pl.group);
  const int nslices = (int)slices.size();
  // The per-entry buffers (B, C, A, dt, entering and leaving state) exist twice; `set` alternates per entry (group).
  int last_run_user[2] = {-1, -1};     // last slice whose kernels read buffer set 0 / 1
  int last_leave_user[2] = {-1, -1};   // last slice whose final-state copy read the leaving-state buffer 0 / 1
  int nsets_used = 0;
  const size_t np = (size_t)n * p;

  int rc = SSD_OK;
  auto ck = [&](cudaError_t err) { if (err != cudaSuccess && rc == SSD_OK) rc = SSD_ERR_CUDA; };
  // The three streams and the events of the pipeline are kept per device between calls (creating and destroying some
  // sixty events and three streams costs a few per cent of a 9 ms call); calls on one device take turns.
  int dev = 0;
  ck(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return SSD_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_pipes_mu[dev]);
  Pipe& pipe = g_pipes[dev];
  if (!pipe.st_in) ck(cudaStreamCreateWithFlags(&pipe.st_in, cudaStreamNonBlocking));
  if (!pipe.st_run) ck(cudaStreamCreateWithFlags(&pipe.st_run, cudaStreamNonBlocking));
  if (!pipe.st_out) ck(cudaStreamCreateWithFlags(&pipe.st_out, cudaStreamNonBlocking));
  while (rc == SSD_OK && (int)pipe.events.size() < 3 * nslices) {
    cudaEvent_t ev = nullptr;
    ck(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    if (ev) pipe.events.push_back(ev);
  }
  if (rc != SSD_OK) return rc;
  cudaStream_t st_in = pipe.st_in, st_run = pipe.st_run, st_out = pipe.st_out;
  cudaEvent_t* ev_in = pipe.events.data();
  cudaEvent_t* ev_run = ev_in + nslices;
  cudaEvent_t* ev_out = ev_run + nslices;

  char* base = static_cast<char*>(dev_scratch);
  char* entry_base = base + kSlots * pl.slot_bytes;
  char* st_base = entry_base + 2 * pl.entry_bytes;
  float* carry[2] = {reinterpret_cast<float*>(st_base), reinterpret_cast<float*>(st_base + pl.st_bytes)};
  float* enter[2] = {reinterpret_cast<float*>(st_base + 2 * pl.st_bytes), reinterpret_cast<float*>(st_base + 3 * pl.st_bytes)};
  float* leave[2] = {reinterpret_cast<float*>(st_base + 4 * pl.st_bytes), reinterpret_cast<float*>(st_base + 5 * pl.st_bytes)};
  float* ld_all = reinterpret_cast<float*>(st_base + 6 * pl.st_bytes);   // [slice][entry of the group][head]
  int32_t* dev_status = reinterpret_cast<int32_t*>(st_base + 6 * pl.st_bytes + pl.ldall_bytes);
  // every kernel of the pipeline reports a wait that ran out to this word (the kernels run on st_run, in order)
  ck(cudaMemsetAsync(dev_status, 0, sizeof(int32_t), st_run));
  const char* hX = static_cast<const char*>(host->X);
  const char* hB = static_cast<const char*>(host->B);
  const char* hC = static_cast<const char*>(host->C);
  const char* hD = static_cast<const char*>(host->dt);
  char* hY = static_cast<char*>(host->Y);
  const bool want_state = host->final_state != nullptr;

  for (int i = 0; i < nslices && rc == SSD_OK; ++i) {
    const int bi = slices[i].bi, nb = slices[i].nb, ci = slices[i].ci, t0 = slices[i].t0, tokens = slices[i].tokens;
    const bool first = slices[i].first, last = slices[i].last;
    if (first) ++nsets_used;
    const int set = (nsets_used - 1) & 1;
    char* slot = base + (size_t)(i % kSlots) * pl.slot_bytes;
    char* dX = slot;
    char* dY = dX + pl.x_bytes;
    char* dW = dY + pl.x_bytes;
    float* dL = ld_all + (size_t)i * pl.group * h;
    char* eB = entry_base + (size_t)set * pl.entry_bytes;   // whole batch entries: B, C, A, dt
    char* eC = eB + pl.bc_bytes;
    char* eA = eC + pl.bc_bytes;
    char* eD = eA + pl.a_bytes;
    char* dB = eB + (size_t)t0 * g * n * e;
    char* dC = eC + (size_t)t0 * g * n * e;
    char* dA = eA + (size_t)t0 * h * 4;
    char* dD = eD + (size_t)t0 * h * e;
    const size_t tok0 = (size_t)bi * s + t0;   // first token of the chunk in the [b*s] token axis

    // stage 1: copies in (the slot is free once the chunk that used it has left); every block is contiguous
    if (i >= kSlots) ck(cudaStreamWaitEvent(st_in, ev_out[i - kSlots], 0));
    if (first) {
      // B, C, A, dt (and the entering state) of the whole batch entry; their buffers were last read by the kernels
      // of batch entry bi-2
      if (last_run_user[set] >= 0) ck(cudaStreamWaitEvent(st_in, ev_run[last_run_user[set]], 0));
      const size_t row0 = (size_t)bi * s, rows = (size_t)nb * s;
      ck(cudaMemcpyAsync(eB, hB + row0 * g * n * e, rows * g * n * e, cudaMemcpyHostToDevice, st_in));
      if (hC) ck(cudaMemcpyAsync(eC, hC + row0 * g * n * e, rows * g * n * e, cudaMemcpyHostToDevice, st_in));
      ck(cudaMemcpyAsync(eA, host->A + row0 * h, rows * h * 4, cudaMemcpyHostToDevice, st_in));
      if (hD) ck(cudaMemcpyAsync(eD, hD + row0 * h * e, rows * h * e, cudaMemcpyHostToDevice, st_in));
      if (host->initial_state)
        ck(cudaMemcpyAsync(enter[set], host->initial_state + (size_t)bi * h * np, (size_t)nb * h * np * 4,
                           cudaMemcpyHostToDevice, st_in));
    }
    ck(cudaMemcpyAsync(dX, hX + tok0 * h * p * e, (size_t)nb * tokens * h * p * e, cudaMemcpyHostToDevice, st_in));
    last_run_user[set] = i;
    ck(cudaEventRecord(ev_in[i], st_in));

    // stage 2: kernels; the state enters from the previous chunk of the sequence and leaves for the next one
    ck(cudaStreamWaitEvent(st_run, ev_in[i], 0));
    if (last && want_state && last_leave_user[set] >= 0)
      ck(cudaStreamWaitEvent(st_run, ev_out[last_leave_user[set]], 0));
    SsdArgs sa;
    chunk_args(host, tokens, nb, &sa);
    sa.X = dX; sa.A = reinterpret_cast<const float*>(dA); sa.B = dB;
    sa.C = hC ? dC : nullptr;
    sa.dt = hD ? dD : nullptr;
    sa.Y = state_only ? nullptr : dY;
    sa.initial_state = first ? (host->initial_state ? enter[set] : nullptr) : carry[(ci - 1) & 1];
    sa.final_state = last ? (want_state ? leave[set] : nullptr) : carry[ci & 1];
    sa.final_logdecay = host->final_logdecay ? dL : nullptr;
    sa.workspace = pl.ws_bytes ? dW : nullptr;
    sa.workspace_bytes = pl.ws_bytes;
    sa.status = dev_status;
    if (state_only && !sa.final_state) sa.final_state = carry[ci & 1];
    if (rc == SSD_OK) {
      const int frc = ssd_b200_forward(&sa, st_run);
      if (frc != SSD_OK) rc = frc;
    }
    ck(cudaEventRecord(ev_run[i], st_run));

    // stage 3: copies out
    ck(cudaStreamWaitEvent(st_out, ev_run[i], 0));
    if (!state_only)
      ck(cudaMemcpyAsync(hY + tok0 * h * p * e, dY, (size_t)nb * tokens * h * p * e, cudaMemcpyDeviceToHost, st_out));
    if (last && want_state) {
      ck(cudaMemcpyAsync(host->final_state + (size_t)bi * h * np, leave[set], (size_t)nb * h * np * 4,
                         cudaMemcpyDeviceToHost, st_out));
      last_leave_user[set] = i;
    }
    ck(cudaEventRecord(ev_out[i], st_out));
  }

  if (st_in) ck(cudaStreamSynchronize(st_in));
  if (st_run) ck(cudaStreamSynchronize(st_run));
  if (st_out) ck(cudaStreamSynchronize(st_out));
  int32_t dev_word = 0;
  if (rc == SSD_OK) ck(cudaMemcpy(&dev_word, dev_status, sizeof(dev_word), cudaMemcpyDeviceToHost));
  if (host->status) *host->status = dev_word;
  if (rc == SSD_OK && dev_word != 0) rc = SSD_ERR_DEVICE_WAIT;
  if (host->final_logdecay && rc == SSD_OK) {
    // per-slice sums, added up on the host
    std::vector<float> ld_host((size_t)nslices * pl.group * h, 0.f);
    ck(cudaMemcpy(ld_host.data(), ld_all, ld_host.size() * sizeof(float), cudaMemcpyDeviceToHost));
    std::vector<double> acc((size_t)b * h, 0.0);
    for (int i = 0; i < nslices; ++i)
      for (int eb = 0; eb < slices[i].nb; ++eb)
        for (int hh = 0; hh < h; ++hh)
          acc[(size_t)(slices[i].bi + eb) * h + hh] += ld_host[((size_t)i * pl.group + eb) * h + hh];
    for (size_t k = 0; k < acc.size(); ++k) host->final_logdecay[k] = (float)acc[k];
  }
  return rc;
}

}  // extern "C"
