/*
 * fkda.h -- C ABI of the B200 (sm_100a) Kimi Delta Attention prefill.
 *
 * This is the drop-in boundary for the reference's one operator, `flash_kda.fwd`.  It replaces
 * the reference's host op `fwd(...)` (csrc/flash_kda.cpp:28-217), its workspace sizing
 * `get_workspace_size` (csrc/flash_kda.cpp:5-26) and the templated launch layer `launch_fwd`
 * (csrc/fwd.h:6-27, csrc/smxx/fwd_launch.cu:7-217), with the template booleans (state in / state
 * out / fp32 state / varlen) turned into run-time fields.  Plain pointers and sizes only: no torch
 * types, nothing is allocated, nothing synchronises, nothing throws.  All work is enqueued on the
 * CUDA stream passed in; all pointers are device pointers on the current device.
 *
 * Every function returns 0 on success or a negative fkda_error; fkda_last_error() then holds a
 * message for the calling thread.  Argument errors are reported before anything is launched,
 * as the reference does with TORCH_CHECK (csrc/flash_kda.cpp:44-174).
 */
#ifndef FKDA_H_
#define FKDA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum fkda_error {
  FKDA_OK = 0,
  FKDA_ERR_INVALID_ARGUMENT = -1,
  FKDA_ERR_WORKSPACE_TOO_SMALL = -2,
  FKDA_ERR_CUDA = -3,
  FKDA_ERR_DEVICE_STATUS = -4
} fkda_error;

typedef enum fkda_state_dtype { FKDA_STATE_NONE = 0, FKDA_STATE_BF16 = 1, FKDA_STATE_FP32 = 2 } fkda_state_dtype;

/* flags */
#define FKDA_FLAG_SCAN_SIMT 0x1u /* evaluate the recurrence on CUDA cores (verification aid, slow) */
#define FKDA_FLAG_SCAN_PLAIN 0x2u /* tcgen05 recurrence without look-ahead (kept for cross-checking) */
#define FKDA_FLAG_SCAN_LOOKAHEAD 0x4u /* always use the look-ahead recurrence kernel on whole sequences */
#define FKDA_FLAG_NO_FUSED_SHORT 0x10u /* fixed-length T <= 32: use the two-kernel path instead of the fused short-sequence kernel */
/* Bit-exact mode: evaluate fkda_fwd the way the reference does (tiles of 16 tokens, bf16 state between tiles, a bf16
 * rounding wherever the reference's kernels round and the same hardware approximations in the same places,
 * csrc/smxx/fwd_kernel1.cuh:265-508, fwd_kernel2.cuh:533-731): `out` and the final state are the same bits as those of
 * the reference's CUDA kernels on the same GPU.  One slow kernel, any shape; honoured by fkda_fwd only. */
#define FKDA_FLAG_REFERENCE_ROUNDING 0x20u
#define FKDA_FLAG_SCAN_NO_SEGMENTS 0x8u /* never cut sequences into runs that are walked in parallel */
/* Send a fixed-length call of any T to the fused short-sequence kernel, which by default takes T <= 32 only (it is a
 * complete forward pass, just slower than the two-kernel path beyond that; the flag exists so that tests can walk
 * many blocks with it). */
#define FKDA_FLAG_FUSED_ANY_T 0x40u
/* The token-parallel stage runs on the pipelined TMA + tcgen05 kernel (csrc/fkda_prepare_tc.cu: tile loads by TMA, the
 * intra-chunk products on tcgen05 with accumulators in tensor memory; three CTAs per SM, each a loop over (chunk, head)
 * items with the serial part of an item on a ninth warp while the other eight are on the next item).  This flag selects
 * the one-CTA-per-item form of that kernel instead (four CTAs per SM; at most 65535 sequences of at most 65535 chunks
 * each for equal lengths, else the call fails).  Same operand records. */
#define FKDA_FLAG_PREPARE_TCGEN05 0x80u
/* The same stage on the earlier kernel (vectorised global loads, mma.sync products).  Same operand records. */
#define FKDA_FLAG_PREPARE_MMA_SYNC 0x20000u
/* Cut every sequence of the batch into n (2..255) runs walked in parallel, whatever the planner would
 * choose; the workspace must then be sized with fkda_get_workspace_size_flags.  Together with FKDA_FLAG_SCAN_PLAIN or
 * FKDA_FLAG_SCAN_LOOKAHEAD both passes over the runs use that recurrence kernel (otherwise each pass picks the faster
 * one for its number of CTAs). */
#define FKDA_FLAG_SEGMENTS(n) (((uint32_t)(n) & 0xffu) << 8)

typedef struct fkda_fwd_params {
  /* bf16 [B*T][H][128], contiguous (reference: q,k,v,g of csrc/flash_kda.cpp:28-33) */
  const void* q;
  const void* k;
  const void* v;
  const void* g;
  const void* beta;          /* bf16 [B*T][H] logits; no transposed copy is needed            */
  void* out;                 /* bf16 [B*T][H][128], every valid row is written                  */
  const float* A_log;        /* fp32 [H]                                                        */
  const float* dt_bias;      /* fp32 [H][128]                                                   */
  const void* initial_state; /* [N][H][128 v][128 k] of state_dtype, or NULL (start from zero) */
  void* final_state;         /* same shape and dtype, or NULL                                   */
  const int64_t* cu_seqlens; /* device int64 [N+1], or NULL for B equal-length sequences        */
  void* workspace;           /* >= fkda_get_workspace_size bytes, 256-byte aligned              */
  int64_t workspace_bytes;
  int64_t B;                 /* batch; must be 1 when cu_seqlens is given                       */
  int64_t T;                 /* tokens per batch row (total tokens when cu_seqlens is given)    */
  int64_t H;                 /* heads                                                           */
  int64_t N;                 /* sequences: B, or len(cu_seqlens)-1                              */
  float scale;               /* applied to q (reference passes K^-0.5)                          */
  float lower_bound;         /* gate lower bound, expected in [-5, 0]; rejected outside [-5.2, 0] */
  int32_t state_dtype;       /* fkda_state_dtype of initial_state / final_state                 */
  uint32_t flags;
} fkda_fwd_params;

/* Bytes of scratch the forward pass needs (replaces get_workspace_size, csrc/flash_kda.cpp:5-26).
 * T_total = B*T.  The figure differs from the reference's: one 35328-byte operand record per
 * (head, 32-token chunk) plus a small header. */
int fkda_get_workspace_size(int64_t T_total, int64_t H, int64_t N, int64_t* bytes);

/* The same for a call that will carry `flags` (needed only with FKDA_FLAG_SEGMENTS, which enlarges the scratch).
 * No counterpart in the reference. */
int fkda_get_workspace_size_flags(int64_t T_total, int64_t H, int64_t N, int64_t flags, int64_t* bytes);

/* Bytes a call of exactly this form uses (fixed-length: T_per_seq tokens per sequence; varlen: the bound
 * T_total/32 + N chunks), where fkda_get_workspace_size covers both forms.  No counterpart in the reference. */
int fkda_workspace_bytes_exact(int64_t T_total, int64_t H, int64_t N, int varlen, int64_t T_per_seq, int64_t flags,
                               int64_t* bytes);

/* The planner of the segment-parallel recurrence: into how many runs (1 = none) a batch with `chains`
 * = N*H chains of `chunks_per_sequence` 32-token chunks is cut, and the run length in chunks.  (For a varlen batch the call plans with the average sequence length and
 * sets the run length on the device from the longest sequence.)  The reference has no
 * counterpart: its recurrence kernel always walks a whole sequence per CTA (csrc/smxx/fwd_kernel2.cuh:434-742). */
int fkda_plan_segments(int64_t chains, int64_t chunks_per_sequence, int* segments, int* chunks_per_segment);

/* The whole operator (replaces fwd(), csrc/flash_kda.cpp:28-217), enqueued on `stream`: prepare + scan, or, for
 * fixed-length sequences of at most 32 tokens, one fused kernel that uses the workspace for its status word only. */
int fkda_fwd(const fkda_fwd_params* p, void* cuda_stream);

/* The two stages on their own, for tests and profiling.  fkda_prepare fills the workspace
 * (reference K1, csrc/smxx/fwd_kernel1.cuh:107); fkda_scan consumes it (reference K2,
 * csrc/smxx/fwd_kernel2.cuh:115).  fkda_fwd == fkda_prepare followed by fkda_scan. */
int fkda_prepare(const fkda_fwd_params* p, void* cuda_stream);
int fkda_scan(const fkda_fwd_params* p, void* cuda_stream);

/* Token-wise prologue alone (the gate / L2-norm / sigmoid part of reference K1,
 * csrc/smxx/fwd_kernel1.cuh:265-339): qn,kn bf16 [rows][128] normalised q,k; gate fp32
 * [rows][128] = lower_bound*log2(e)*sigmoid(exp(A_log)*(g+dt_bias)); beta_act fp32 [rows].
 * rows = B*T*H laid out [token][head]. */
int fkda_prologue(const void* q, const void* k, const void* g, const void* beta, const float* A_log,
                  const float* dt_bias, float lower_bound, int64_t T_total, int64_t H, void* qn, void* kn,
                  float* gate, float* beta_act, void* cuda_stream);

/* Byte offset and size of the operand record of (head, chunk) inside the workspace, and the
 * number of records per head, so that a test can inspect what fkda_prepare wrote. */
int fkda_workspace_layout(int64_t T_total, int64_t H, int64_t N, int varlen, int64_t T_per_seq,
                          int64_t* records_offset, int64_t* record_bytes, int64_t* chunks_per_head);

/* Reads the device status word of a workspace after synchronising `stream`: 0 = fine,
 * 1 = cu_seqlens was not monotone inside [0, T_total], 2 = a bounded wait inside a kernel gave up.
 * The only call here that blocks the host. */
int fkda_read_status(const void* workspace, void* cuda_stream, int* status);

/* The forward pass with built-in scratch, for callers that cannot allocate device memory (a
 * server whose memory pool was fixed at start-up, a plugin living inside another component's
 * budget).  No counterpart in the reference, whose Python wrapper allocates a workspace per call.
 * Same parameter block as fkda_fwd; `workspace` and `workspace_bytes` are ignored.  The scratch
 * is a 64 MiB array inside the library image (fkda_static_ws_capacity()), held by every GPU the
 * library is loaded on; problems that need more are rejected with FKDA_ERR_WORKSPACE_TOO_SMALL.
 * The first call on a device looks the array's address up, so issue it outside stream capture; the
 * address is cached per device and does not survive a cudaDeviceReset.
 * All calls on a device share the array: calls that overlap on the GPU race and must be
 * serialised by the caller.  Allocates nothing.  fkda_static_ws_read_status is
 * fkda_read_status for the built-in scratch of the current device. */
int fkda_fwd_static_ws(const fkda_fwd_params* p, void* cuda_stream);
int64_t fkda_static_ws_capacity(void);
int fkda_static_ws_read_status(void* cuda_stream, int* status);
const char* fkda_static_ws_last_error(void);

/* Message of the last error on this thread ("" if none). */
const char* fkda_last_error(void);

/* Library version string. */
const char* fkda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FKDA_H_ */
