/*
 * jvpfa.h -- C ABI of the B200 (sm_100a) JVP flash-attention library (libjvpfa.so).
 *
 * The entry points below are what a binding of the reference's attention path would call in
 * place of its Triton launches. All tensors are caller-owned device memory. Outputs are (B,H,N,D)
 * contiguous row-major, as the reference makes them; inputs may be strided views (see jvpfa_strides),
 * where the reference copies every non-contiguous input first (jvp_flash_attention/jvp_attention.py:2950,
 * 3007, 3107-3127). Every call is asynchronous on the given CUDA stream and returns a status code;
 * nothing here allocates device memory unless a comment on the entry point says otherwise.
 */
#ifndef JVPFA_H_
#define JVPFA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
enum { JVPFA_F16 = 0, JVPFA_BF16 = 1, JVPFA_F32 = 2 };
/* mask kinds: the reference's MASK_TYPE values (jvp_attention.py:2623-2656) */
enum { JVPFA_MASK_NONE = 0, JVPFA_MASK_BOOL = 1, JVPFA_MASK_ADDITIVE = 2 };

/* status codes */
enum {
  JVPFA_OK = 0,
  JVPFA_ERR_BAD_ARG = 1,       /* null pointer, non-positive size, misaligned pointer            */
  JVPFA_ERR_UNSUPPORTED = 2,   /* shape / dtype combination this library has no kernel for       */
  JVPFA_ERR_CAUSAL_MASK = 3,   /* causal together with a mask (ValueError in the reference)      */
  JVPFA_ERR_WORKSPACE = 4,     /* workspace missing or too small                                 */
  JVPFA_ERR_LAUNCH = 5,        /* CUDA reported an error at launch or tensor-map encoding        */
  JVPFA_ERR_DEVICE_TIMEOUT = 6,/* a bounded device-side wait gave up (see jvpfa_read_status)     */
  JVPFA_ERR_NO_ALLOC_LIMIT = 7 /* problem exceeds the fixed scratch of an allocation-free entry  */
};

/* A mask of logical shape (B,H,N,N) given by element strides; a stride of 0 broadcasts.
 * kind BOOL: one byte per element, non-zero = take part in attention.
 * kind ADDITIVE: `dtype` elements added to the scaled scores; -inf excludes an element. */
typedef struct jvpfa_mask {
  const void* ptr;
  int32_t kind;
  int32_t dtype;
  int64_t stride[4];
} jvpfa_mask;

/* Element strides of a (B,H,N,D) input tensor along B, H and N; the D axis must be contiguous. All zero means the
 * contiguous layout (H*N*D, N*D, D). A strided input (for instance q = qkv.permute(2,0,3,1,4)[0] of a fused projection,
 * or an upstream gradient that is a transposed view) is read in place by the tensor-core kernels when every stride
 * is a multiple of 16 bytes and the pointer is 16-byte aligned; otherwise, and for the shapes that run on the
 * CUDA-core kernels (head dimension above 128 or not a multiple of 8; fp32 above 64), the call returns
 * JVPFA_ERR_UNSUPPORTED and the caller copies the tensor first. */
typedef struct jvpfa_strides {
  int64_t b, h, n;
} jvpfa_strides;

/* Dual forward. Replaces the launch of _attn_fwd_tma / _attn_fwd in JVPAttn.forward
 * (jvp_attention.py:2773, 2807). Outputs: o, to (same dtype as q), lse2 and mu ((B,H,N) fp32:
 * base-2 log-sum-exp of the scaled, masked scores -- the reference's M, jvp_attention.py:2594 --
 * and mu = rowsum(P o tS), which the dual backward needs). tq/tk/tv/to may all be NULL for the
 * primal-only call (JVPAttn.fwd, jvp_attention.py:2915-2970). */
typedef struct jvpfa_fwd_args {
  int32_t B, H, N, D;
  int32_t dtype;
  int32_t causal;
  float sm_scale;
  jvpfa_mask mask;
  const uint8_t* mask_summary; /* optional output of jvpfa_mask_summary, else NULL */
  const void *q, *k, *v, *tq, *tk, *tv;
  void *o, *to;
  float *lse2, *mu;
  void* workspace;
  size_t workspace_bytes;
  jvpfa_strides q_strides, k_strides, v_strides, tq_strides, tk_strides, tv_strides;
  float dropout_p;        /* 0 = no dropout; see jvpfa_bwd_args */
  uint64_t dropout_seed;
} jvpfa_fwd_args;

/* Dual backward: gradients of sum(o*go)+sum(to*gto) for all six inputs. Replaces
 * _attn_bwd_preprocess + _attn_bwd / _attn_bwd_causal in JVPAttn.backward
 * (jvp_attention.py:3171, 3189), and adds what the reference leaves out: the gradient through
 * the tangent output and the tangent-input gradients (jvp_attention.py:3081, 3226).
 * Pass a zero tensor as gto when only the primal output has a gradient. tq == NULL selects the primal-only
 * backward (the reference's own case, jvp_attention.py:3080-3226): tk, tv, to, gto, dtq, dtk, dtv are then ignored
 * and only dq, dk, dv are written. */
typedef struct jvpfa_bwd_args {
  int32_t B, H, N, D;
  int32_t dtype;
  int32_t causal;
  float sm_scale;
  jvpfa_mask mask;
  const uint8_t* mask_summary;
  const void *q, *k, *v, *tq, *tk, *tv;
  const void *o, *to;
  const float *lse2, *mu;
  const void *go, *gto;
  void *dq, *dk, *dv, *dtq, *dtk, *dtv;
  void* workspace;
  size_t workspace_bytes;
  jvpfa_strides q_strides, k_strides, v_strides, tq_strides, tk_strides, tv_strides, go_strides, gto_strides;
  /* Dropout on the attention probabilities (after the softmax, kept entries scaled by 1 / (1 - p)); the tangent
   * output is the derivative of the dropped-out output for the same keep pattern. The pattern is a function of
   * (dropout_seed, batch*head unit, query, key) -- Philox4x32-10, see csrc/dropout.cuh -- and is regenerated by the
   * backward: pass the forward's dropout_p and dropout_seed. Tensor-core kernels only (fp16 / bf16 with a head dimension
   * that is a multiple of 8 up to 128; fp32 up to 64 with the workspace of its tensor-core path); calls that would run on
   * the CUDA-core kernels answer JVPFA_ERR_UNSUPPORTED. The reference sketches dropout
   * (jvp_attention.py:105-133) but raises NotImplementedError for dropout_p != 0 (:2550). */
  float dropout_p;
  uint64_t dropout_seed;
} jvpfa_bwd_args;

/* Library version (major*10000 + minor*100 + patch). */
int jvpfa_version(void);   /* 200: the args structs carry input strides */
/* Text for a status code. */
const char* jvpfa_error_string(int status);

/* Bytes of caller-provided scratch the calls below want (always >= 256: the first 4 bytes hold the device status
 * word that bounded waits write to; it must be zero before the first call). For fp32 inputs with a head dimension
 * of at most 64 this is the need of the tensor-core path, which keeps bf16 hi/lo splits of its operands in the
 * workspace (256 bytes per row and tensor); a call that is given less, but at least 256 bytes (forward) or
 * 256 + 16 bytes per row (backward), runs the same mathematics on the CUDA cores instead. */
size_t jvpfa_fwd_workspace_bytes(const jvpfa_fwd_args* args);
size_t jvpfa_bwd_workspace_bytes(const jvpfa_bwd_args* args);

/* Bytes of the mask summary for a mask over sequences of length N with Bm x Hm distinct (batch, head)
 * planes, and the kernel that fills it (`summary` 16-byte aligned). Per 64x64 tile: bit 0 = some element
 * kept, bit 1 = some element that needs the mask (a boolean False; an additive entry other than zero), which
 * lets the kernels skip fully excluded tiles and skip the mask on tiles whose entries are all True / all zero.
 * For a boolean mask the buffer also receives the mask packed into 64-bit words, once by query row and once
 * by key row, so that a kernel thread fetches the 32 entries it needs of a tile with one load whatever the
 * mask's strides are (2 * N^2 / 8 bytes per plane, N rounded up to 64). For an additive mask with contiguous,
 * 16-byte aligned rows the words mark the +-0 entries, and a tile whose other entries all carry one value
 * (0 / -inf, 0 / a large negative constant) is flagged (bit 2) with that value stored per tile: such tiles
 * are applied from the words too, all others are read element by element. The summary belongs to the
 * mask's contents: compute it again when they change. No reference counterpart (the reference reads the mask
 * element-wise in every tile, jvp_attention.py:250-262). */
size_t jvpfa_mask_summary_bytes(int32_t Bm, int32_t Hm, int32_t N);
int jvpfa_mask_summary(const jvpfa_mask* mask, int32_t B, int32_t H, int32_t N, uint8_t* summary, void* stream);

/* The two launches. `stream` is a cudaStream_t. */
int jvpfa_fwd(const jvpfa_fwd_args* args, void* stream);
int jvpfa_bwd(const jvpfa_bwd_args* args, void* stream);

/* Synchronises the stream, reads the status word at the start of `workspace`, clears it, and
 * returns JVPFA_OK or JVPFA_ERR_DEVICE_TIMEOUT (`detail`, if not NULL, receives the raw word:
 * 100 + the id of the wait that gave up). */
int jvpfa_read_status(void* workspace, void* stream, int32_t* detail);

/* Diagnostic: the SM clock that running kernels actually get. Launches a one-thread kernel on `stream` that reads its
 * SM's cycle counter and the global timer, sleeps for `duration_us` microseconds (1 .. 1000000) and reads them again;
 * `mhz_out` (device, one float) receives cycles per microsecond. Launched on a stream of its own just before a timed
 * region it runs beside the attention kernels (it needs no shared memory) and reports the clock under their load, which
 * on a power-limited part is well below what the management library shows between kernels. No reference counterpart. */
int jvpfa_sm_clock_probe(float* mhz_out, int32_t duration_us, void* stream);

/* Self-test of the failure-detection path. Launches one tiny kernel on `stream` in which a single thread waits, with
 * the kernels' own bounded wait, on a barrier that nothing arrives on: after `budget_us` microseconds (1 .. 1000000)
 * the wait gives up, writes 177 (100 + wait id 77) into the status word at the start of `workspace` and the kernel
 * returns normally; a second wait in the same kernel takes the short path of an already failed CTA. `out4` (device,
 * four int32) receives the two wait results (0 = gave up) and their durations in microseconds. Afterwards
 * jvpfa_read_status reports JVPFA_ERR_DEVICE_TIMEOUT once. Nothing faults, traps or spins without bound. No reference
 * counterpart (its errors are host-side Python exceptions, jvp_attention.py:2550, 2574, 3111). */
int jvpfa_selftest_timeout(void* workspace, int32_t budget_us, int32_t* out4, void* stream);

/* Largest problem (B*H*N query rows) the allocation-free backward accepts; its scratch is 256 B + 16 B per row. */
#define JVPFA_NO_ALLOC_MAX_ROWS 262144

/* Dual backward that allocates nothing. It has no counterpart in the reference (whose backward allocates
 * its scratch with torch, jvp_attention.py:3130-3133, 3153).
 *
 * For callers that cannot or must not allocate device memory: a plug-in inside a process whose memory
 * pool already holds nearly all of the GPU's memory (cudaMalloc would fail), or a latency-critical
 * path that must avoid the device-wide synchronisation of cudaMalloc / cudaFree. Same inputs, outputs
 * and results as jvpfa_bwd, except that `workspace` / `workspace_bytes` in `args` are ignored: the
 * scratch (status word + per-row statistics) is a fixed array inside the library image, 4 MiB + 256 B,
 * held by every GPU that loads the library until the process exits. Problems with more than
 * JVPFA_NO_ALLOC_MAX_ROWS rows (B*H*N) are refused with JVPFA_ERR_NO_ALLOC_LIMIT before anything runs.
 *
 * The first call on each device looks up the device address of that array (with that device current);
 * make that first call before starting any stream capture. With CUDA's default lazy module loading that
 * look-up is also where the driver sets the array up on the device, so a process whose memory pool is about
 * to claim the rest of the GPU's memory makes the first call before the pool grows (or sets
 * CUDA_MODULE_LOADING=EAGER). fp32 inputs run on the CUDA-core kernels here. Every call clears the status word at the
 * start of the array on `stream` and then reuses the rest as it is. All calls on a device share the
 * one array: two calls whose kernels can overlap on the GPU (different streams without an ordering
 * between them) race on it and give undefined results -- order them yourself.
 * If `status_word_out` (a device pointer) is not NULL the status word is copied there after the
 * kernels, on `stream`: 0 means no device-side wait gave up. */
int jvpfa_bwd_noalloc(const jvpfa_bwd_args* args, int32_t* status_word_out, void* stream);

/* jvpfa_bwd with caller-owned CUDA events recorded between its launches, for benchmarks that want the
 * duration of each kernel: events[0] is recorded on `stream` before the preprocess kernel, events[1], [2], [3]
 * before the three main kernels (gradients of the query side, of the key side, of the value side) and events[4]
 * after the last one (16-bit inputs with a head dimension of at most 64: the key side and the value side are one kernel,
 * events[3] and events[4] are recorded together after it). `events` holds five cudaEvent_t created by the caller with
 * timing enabled; n_events must be 5.
 * The library keeps no state for this. No reference counterpart (the reference times whole calls with perf_counter,
 * tests/test_jvp_attention.py:116-143). */
int jvpfa_bwd_marked(const jvpfa_bwd_args* args, void* stream, void* const* events, int32_t n_events);

#ifdef __cplusplus
}
#endif
#endif /* JVPFA_H_ */
