/*
 * ssd_b200 -- C ABI of the B200 (sm_100a) Mamba-2 SSD chunked-scan forward.
 *
 * The reference project (ShouyangDong/WorkloadSuite) is pure Python/PyTorch and
 * has no FFI; the interface each entry point stands in for is therefore a Python
 * call site of the `mamba` workload, cited per function as file:line within the
 * reference checkout.
 *
 * Conventions
 *   - every pointer in SsdArgs is a DEVICE pointer owned by the caller; the
 *     library allocates nothing and keeps no state between calls (the one
 *     exception is documented at its declaration);
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*); no entry
 *     point synchronises the host with the device unless it says so;
 *   - every function returns SSD_OK (0) or a negative SSD_ERR_* code; nothing is
 *     thrown across the boundary and the process is never terminated;
 *   - asynchronous device-side problems (a bounded wait that ran out) are written
 *     to the int32 `status` word, to be read by the caller after the stream has
 *     been synchronised (0 = fine).
 */
#ifndef SSD_B200_H_
#define SSD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SSD_OK = 0,
  SSD_ERR_NULL_POINTER = -1,
  SSD_ERR_BAD_SHAPE = -2,      /* non-positive size, heads not divisible by groups */
  SSD_ERR_BAD_CHUNK = -3,      /* seqlen not a multiple of chunk (reference: EinopsError at model_ref.py:106) */
  SSD_ERR_UNSUPPORTED = -4,    /* shape/dtype/stride outside what the kernels cover */
  SSD_ERR_WORKSPACE = -5,      /* workspace missing or smaller than ssd_b200_workspace_bytes() */
  SSD_ERR_CUDA = -6,           /* a CUDA runtime call failed (launch, attribute) */
  SSD_ERR_MISALIGNED = -7,     /* pointer or stride not aligned as the chosen kernel needs */
  SSD_ERR_TOO_LARGE = -8,      /* size beyond a stated fixed limit */
  SSD_ERR_DEVICE_WAIT = -9     /* (host-buffer entry, which synchronises) a bounded device-side wait ran out */
};

enum { SSD_DTYPE_F32 = 0, SSD_DTYPE_F16 = 1, SSD_DTYPE_BF16 = 2 };

/* kernel selection */
enum {
  SSD_KERNEL_AUTO = 0,    /* tensor-core kernel when the shape allows, else the fp32 scan */
  SSD_KERNEL_SCAN_F32 = 1,/* fp32 token recurrence on CUDA cores (any dtype in, fp32 math) */
  SSD_KERNEL_TCGEN05 = 2  /* tcgen05/TMEM chunked kernel (f16/bf16 only) */
};

/* flags */
enum {
  SSD_FLAG_STATE_ONLY = 1,/* do not compute/write Y; only final_state / final_logdecay */
  SSD_FLAG_REUSE_SEGMENTS = 2,/* two-pass segmented scan only: the workspace still holds the per-segment
                                 results of the previous call on this stream with SSD_FLAG_STATE_ONLY, the same
                                 tensors, sizes and nsegments; do not recompute them (a sequence-sharded
                                 forward runs state-only first, exchanges states, then runs with this flag) */
  SSD_FLAG_SEPARATE_EPILOGUE = 4,/* apply D / Z with the stand-alone epilogue kernel even where the main kernel
                                    could fuse them (for comparisons) */
  SSD_FLAG_INJECT_LOST_HANDOVER = 8 /* testing the give-up path: in a launch whose sequences are handed from CTA to
                                    CTA, the first CTA leaves without working, so the CTA that continues its
                                    sequence runs into the bound of its wait (wait_limit_ms), reports status 6 and
                                    returns; Y and the states of that launch are then incomplete */
};

/*
 * Arguments of one SSD forward.  Mirrors the tensor arguments of
 *   SSDLayer._ssd_core(X_b, B_b, C_b, dt_b, A_dt_b, batch)   model_ref.py:123-131
 * with the chunk axis folded back into the sequence axis, B/C left un-broadcast
 * ([b,s,g,n]; head j reads group j / (nheads/ngroups), the rule of
 * model_ref.py:97-99) and the zero initial carry of model_ref.py:153 made an
 * optional input.  Strides are in ELEMENTS; the innermost axis (p or n) must
 * have stride 1.
 */
typedef struct SsdArgs {
  const void*  X;               /* [b,s,h,p]  dtype          model_ref.py:125 */
  const float* A;               /* [b,s,h]    fp32 per-token log-decay (A_dt) :129 */
  const void*  B;               /* [b,s,g,n]  dtype          :126 */
  const void*  C;               /* [b,s,g,n]  dtype          :127 */
  const void*  dt;              /* [b,s,h]    dtype, or NULL for dt == 1   :128,144 */
  const float* initial_state;   /* [b,h,n,p]  fp32 contiguous, or NULL for zeros :153 (16-byte aligned for the
                                   tensor-core kernel: SSD_KERNEL_AUTO takes the fp32 scan otherwise, an explicit
                                   SSD_KERNEL_TCGEN05 returns SSD_ERR_MISALIGNED; the same for final_state) */
  void*        Y;               /* [b,s,h,p]  dtype          :162 (NULL allowed with SSD_FLAG_STATE_ONLY) */
  float*       final_state;     /* [b,h,n,p]  fp32 contiguous, or NULL (the carry after the last chunk, :156) */
  float*       final_logdecay;  /* [b,h]      fp32 sum of A over the sequence, or NULL */
  void*        workspace;       /* >= ssd_b200_workspace_bytes() bytes, 256-byte aligned; may be NULL if that is 0 */
  size_t       workspace_bytes;
  int32_t*     status;          /* device int32, or NULL */
  int32_t batch, seqlen, nheads, headdim, dstate, ngroups;
  int32_t chunk;                /* the reference's block_len; seqlen % chunk must be 0 */
  int32_t dtype;                /* SSD_DTYPE_* of X, B, C, dt, Y */
  int32_t kernel;               /* SSD_KERNEL_* */
  int32_t flags;                /* SSD_FLAG_* */
  int32_t nsegments;            /* 0 = choose; 1 = whole sequences; >1 = cut each sequence (needs workspace): into
                                   this many independently scanned segments joined by a state fold, or, for the
                                   two-head tensor-core kernel's plain forward, at the points an even deal of
                                   all tiles over the SMs gives */
  int32_t wait_limit_ms;        /* bound of every device-side wait (a kernel that runs into it writes its code to
                                   `status` and returns); 0 = the default, about one second */
  int64_t x_stride[3];          /* b, s, h */
  int64_t a_stride[3];          /* b, s, h */
  int64_t b_stride[3];          /* b, s, g */
  int64_t c_stride[3];          /* b, s, g */
  int64_t dt_stride[3];         /* b, s, h */
  int64_t y_stride[3];          /* b, s, h */
  /* Optional fused epilogue of SSDLayer.forward after the core (model_ref.py:116-118):
   *   Y <- (Y + x * D[head]) * silu(z)
   * with x the X input, evaluated in fp32 and rounded once.  D == NULL skips the skip term, Z == NULL the gate. */
  const float* D;               /* [h]        fp32, or NULL            model_ref.py:116 */
  const void*  Z;               /* [b,s,h,p]  dtype, or NULL           model_ref.py:118 */
  int64_t z_stride[3];          /* b, s, h */
} SsdArgs;

/* Library/ABI version (bumped when SsdArgs changes). */
int ssd_b200_abi_version(void);

/* Text for an SSD_ERR_* code (static storage). */
const char* ssd_b200_strerror(int code);

/* Scratch bytes ssd_b200_forward() needs for these arguments (0 when the
 * sequence is not split).  Returns 0 for invalid arguments; ssd_b200_forward
 * reports the error.  No reference counterpart (the reference lets PyTorch
 * allocate its temporaries at model_ref.py:135-161). */
size_t ssd_b200_workspace_bytes(const SsdArgs* args);

/* Name of the kernel family SSD_KERNEL_AUTO resolves to for these arguments
 * ("scan_f32", "tcgen05") or "invalid". */
const char* ssd_b200_kernel_name(const SsdArgs* args);

/* How ssd_b200_forward() will run these arguments: the resolved SSD_KERNEL_* family, the number of
 * segments each sequence is cut into (2 stands for "cut" where the cut points follow from the grid),
 * and the number of kernel launches it enqueues: 1 for whole sequences; 1 plus a memset where the
 * two-head tensor-core kernel deals the tiles of all sequences out evenly inside one launch (states
 * handed from CTA to CTA, or folded from the pairs each CTA publishes for the last piece of its range);
 * 3 for the two-pass segmented scan (2 with SSD_FLAG_STATE_ONLY or SSD_FLAG_REUSE_SEGMENTS).  Any out
 * pointer may be NULL.  Returns SSD_OK or the validation error.  No reference counterpart. */
int ssd_b200_plan(const SsdArgs* args, int32_t* kernel, int32_t* nsegments, int32_t* launches);

/* (A Z whose address or strides are not multiples of 16 bytes is applied by the stand-alone epilogue kernel.)
 *
 * The SSD forward: replaces SSDLayer._ssd_core, model_ref.py:123-162
 * (in-chunk prefix sum :135, decay mask :139-141, C.B^T :143, Y_diag :145,
 * chunk states :148-150, inter-chunk recurrence :152-157, Y_off :160-161,
 * sum :162), plus the GQA broadcast of :97-99, the X*dt product of :144 and,
 * when D / Z are given, the skip and gate of :116-118 applied to Y before it is
 * written. */
int ssd_b200_forward(const SsdArgs* args, void* stream);

/* Fold per-shard results of a sequence-sharded scan into the state entering one
 * shard.  Shard q's zero-start final state is the fp32 block
 * states + q*states_shard_stride, laid out [units][np]; its summed log-decay is
 * logdecay + q*logdecay_shard_stride, laid out [units] (strides in floats, so
 * both may live in one all-gather buffer); initial is [units][np] or NULL.
 * Writes H_in(rank) = fold_{q<rank}(H <- exp(D_q) H + F_q) to out [units][np].
 * rank may equal nshards (state after the last shard).  The reference has no
 * sharded path; this is the linear-recurrence identity behind
 * model_ref.py:152-157 applied across shards. */
int ssd_b200_fold_states(const float* states, int64_t states_shard_stride, const float* logdecay,
                         int64_t logdecay_shard_stride, const float* initial, float* out, int32_t nshards,
                         int32_t rank, int64_t units, int64_t np, void* stream);

/* All-gather of the sequence shards' (state, log-decay) blocks through NVLink peer memory, for one process per
 * GPU on one node: the exchange step of the sequence-sharded forward as a kernel of this library (plain peer
 * stores and release/acquire flags at system scope, nothing else touches peer memory).  The reference has
 * no sharded path; the blocks exchanged are the operands of ssd_b200_fold_states() above.
 *   create      allocates this rank's receive buffer [world][slot_bytes] (slot_bytes rounded up to 16) and returns
 *               an opaque context and an SSD_XCHG_HANDLE_BYTES-byte handle to pass to the other ranks (any
 *               transport: the Python wrapper uses torch.distributed.all_gather_object);
 *   connect     opens the other ranks' buffers; `handles` is world handles in rank order (own entry ignored);
 *   buffer      this rank's receive buffer (device pointer): slot r holds rank r's block after an all_gather;
 *   all_gather  one kernel launch on `stream`: waits until every rank has entered the same exchange (so the
 *               previous one has been consumed), writes `send` (bytes <= slot_bytes, multiple of 16, 16-byte
 *               aligned) into slot `rank` of every rank's buffer, and completes once every rank's block has
 *               arrived here.  Every rank must call it the same number of times; the exchange counter lives in
 *               device memory, so a captured launch can be replayed.  A wait longer than wait_limit_ms (0: two
 *               seconds) writes 7 to *status (device int32, may be NULL) and ends the kernel.
 *   destroy     closes the peers' buffers and frees this rank's.
 * Return SSD_OK or an SSD_ERR_* code. */
#define SSD_XCHG_HANDLE_BYTES 64
int ssd_b200_xchg_create(size_t slot_bytes, int32_t world, void** ctx_out, void* handle_out);
int ssd_b200_xchg_connect(void* ctx, const void* handles, int32_t rank);
void* ssd_b200_xchg_buffer(void* ctx);
int ssd_b200_xchg_all_gather(void* ctx, const void* send, size_t bytes, int32_t* status, int32_t wait_limit_ms,
                             void* stream);
int ssd_b200_xchg_destroy(void* ctx);

/* Causal depthwise conv1d + SiLU, the producer of the core's X: replaces
 *   x = silu(conv1d(x.transpose)[..., :seq_len]).transpose     model_ref.py:83-86
 * (nn.Conv1d(d, d, taps, padding=taps-1, groups=d, bias) of model_ref.py:50-58) without the two
 * transposes:  y[b,t,c] = silu(bias[c] + sum_k weight[c,k] * x[b, t-(taps-1)+k, c]), zeros before t = 0.
 * x and y are [batch, seqlen, channels] with the channel axis contiguous and the given element strides
 * for batch and sequence (x may be a column slice of the projection output); weight is [channels, taps]
 * (the [d,1,taps] parameter), bias [channels] or NULL; all in `dtype`; fp32 accumulation, one rounding.
 * channels % 8 == 0, taps in 2..4. */
int ssd_b200_conv1d_silu(const void* x, const void* weight, const void* bias, void* y, int32_t batch,
                         int32_t seqlen, int32_t channels, int32_t taps, int32_t dtype, int64_t x_stride_b,
                         int64_t x_stride_l, int64_t y_stride_b, int64_t y_stride_l, void* stream);

/* dt discretisation ahead of the core: replaces
 *   dt = softplus(dt + dt_bias); A_dt = -exp(A_log) * dt.float()      model_ref.py:94, 102-103
 * dt_raw is [batch, seqlen, nheads] in `dtype` with the head axis contiguous and the given element strides
 * (a column slice of the projection output), dt_bias [nheads] in `dtype` or NULL, A_log [nheads] fp32.
 * Writes dt_out [batch, seqlen, nheads] in `dtype` and A_dt_out [batch, seqlen, nheads] fp32, both contiguous:
 * the `dt` and `A` arguments of ssd_b200_forward. */
int ssd_b200_dt_prologue(const void* dt_raw, int64_t stride_b, int64_t stride_l, const void* dt_bias,
                         const float* A_log, void* dt_out, float* A_dt_out, int32_t batch, int32_t seqlen,
                         int32_t nheads, int32_t dtype, void* stream);

/* One token of the recurrence with the state carried in place (decode-style use; the reference has only the chunked
 * forward, whose carry model_ref.py:152-157 reduces to this for a single token):
 *   state[b,h] <- exp(a[b,h]) * state[b,h] + B[b,g] (x) (dt[b,h] * x[b,h]);   y[b,h] = C[b,g] . state[b,h]
 * then, when given, y <- (y + x * D[h]) * silu(z)   (model_ref.py:116-118).
 * x, y, z are [batch, nheads, headdim], B and C [batch, ngroups, dstate], dt [batch, nheads] (NULL: x is already
 * scaled) in `dtype`, all contiguous; a [batch, nheads] is the token's fp32 log-decay (the reference's A_dt); D [nheads]
 * fp32 or NULL; state [batch, nheads, dstate, headdim] fp32, 16-byte aligned, updated in place (the layout of
 * SsdArgs.initial_state / final_state).  headdim == 64, dstate a multiple of 16 up to 256.  HBM-bound on the state. */
int ssd_b200_step(const void* x, const float* a, const void* B, const void* C, const void* dt, const float* D,
                  const void* z, float* state, void* y, int32_t batch, int32_t nheads, int32_t headdim,
                  int32_t dstate, int32_t ngroups, int32_t dtype, void* stream);

/* Whole forward with HOST buffers: copies X/A/B/C (and dt, initial_state when
 * given) from host memory, runs the forward and copies Y (and final_state) back,
 * pipelined over batch slices on internal streams.  Every pointer in `host` is a
 * host pointer (pinned memory gives the best rate), tensors contiguous; strides
 * in `host` are ignored.  `dev_scratch` is a caller-owned DEVICE buffer of at
 * least ssd_b200_host_scratch_bytes() bytes.  Synchronises the host before
 * returning.  `host->status`, when given, is a HOST int32 that receives the device status word; a non-zero
 * word also makes the call return SSD_ERR_DEVICE_WAIT.  Unlike the other entry points this one runs on
 * three CUDA streams of its own (created with their events on the first call per device and kept; calls on one device take
 * turns).  Stands in for calling the reference module with
 * CPU tensors (bench.py:217-233 builds inputs on the default device and calls Model). */
size_t ssd_b200_host_scratch_bytes(const SsdArgs* host);
int ssd_b200_forward_host(const SsdArgs* host, void* dev_scratch, size_t dev_scratch_bytes);

/* Fixed size of the scratch array behind ssd_b200_forward_static_scratch(). */
#define SSD_STATIC_SCRATCH_BYTES ((size_t)16 << 20)

/* ssd_b200_forward() for callers that cannot allocate device memory and have no
 * workspace to pass: a plugin inside a host runtime that owns the device heap
 * and forbids cudaMalloc on its request path, or a bare FFI client without an
 * allocator.  No counterpart in the reference (PyTorch allocates its
 * temporaries there, model_ref.py:135-161).
 *
 * Same arguments and results as ssd_b200_forward(); args->workspace and
 * args->workspace_bytes are ignored.  The scratch of the segmented scan comes
 * from one SSD_STATIC_SCRATCH_BYTES (16 MiB) array that is part of the library
 * image: every GPU that loads the library holds it until the process exits.
 *   - Returns SSD_ERR_TOO_LARGE when ssd_b200_workspace_bytes(args) exceeds
 *     that size (reduce args->nsegments, or use ssd_b200_forward()).
 *   - Calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - The first call on each device looks the array's device address up (with
 *     that device current) and keeps it; make that first call outside any
 *     stream capture.
 *   - All calls on one device share the array, and it keeps the previous call's
 *     contents.  The two-pass scan writes every segment state before it reads it;
 *     the single-launch (chained) scan needs its ready flags at zero, and the
 *     forward clears them itself with a memset on `stream` ahead of the kernel.
 *     The caller clears nothing.  Two calls whose kernels may overlap on the GPU
 *     (different streams) race on the array: serialise them.
 * ssd_b200_static_scratch_capacity() returns SSD_STATIC_SCRATCH_BYTES. */
size_t ssd_b200_static_scratch_capacity(void);
int ssd_b200_forward_static_scratch(const SsdArgs* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SSD_B200_H_ */
