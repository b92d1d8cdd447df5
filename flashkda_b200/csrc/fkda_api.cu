// C ABI of the library (include/fkda.h): argument validation, workspace carving and launches.
// Host-side counterpart of the reference's csrc/flash_kda.cpp (validation, dispatch) and
// csrc/smxx/fwd_launch.cu (workspace carving, launches), without torch types.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "../../include/fkda.h"
#include "../../include/fkda_testing.h"
#include "fkda_common.cuh"

namespace fkda {
cudaError_t launch_chunk_prefix(const int64_t* cu, int N, int64_t T_total, int H, int n_segs, int* prefix, int* status,
                                cudaStream_t stream);
cudaError_t launch_prepare(const PrepParams& p, cudaStream_t stream);
cudaError_t launch_prepare_tc4(const PrepParams& p, cudaStream_t stream);
cudaError_t launch_prepare_pipe(const PrepParams& p, cudaStream_t stream);
cudaError_t launch_scan(const ScanParams& p, cudaStream_t stream);
cudaError_t launch_scan_simt(const ScanParams& p, cudaStream_t stream);
cudaError_t launch_scan2(const ScanParams& p, cudaStream_t stream);
cudaError_t launch_scan_short(const ScanParams& p, int sm_count, cudaStream_t stream);
cudaError_t launch_short16(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, const __nv_bfloat16* g,
                           const __nv_bfloat16* beta, const float* A_log, const float* dt_bias, const void* initial_state,
                           void* final_state, __nv_bfloat16* out, int64_t N, int T, int H, int state_fp32, float scale,
                           float gate_scale, int* status, cudaStream_t stream);
cudaError_t launch_refmode(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, const __nv_bfloat16* g,
                           const __nv_bfloat16* beta, const float* A_log, const float* dt_bias, const void* initial_state,
                           void* final_state, __nv_bfloat16* out, const int64_t* cu_seqlens, int64_t N, int64_t T, int64_t T_total,
                           int H, int state_fp32, float scale, float gate_scale, cudaStream_t stream);
cudaError_t launch_scan_segmented(const ScanParams& base, int n_segs, int seg_chunks, float* seg_buf, int kernel_choice,
                                  cudaStream_t stream);
#ifdef FKDA_TUNING
void set_prepare_trace(long long* buf);
void set_scan_trace(unsigned long long* buf);
cudaError_t launch_tmem_bench(int nwarps, int reps, long long* out, cudaStream_t stream);
cudaError_t launch_umma_bench(int nissuers, int reps, int ksteps, int n, int ts, long long* out, int* status, cudaStream_t stream);
#endif
cudaError_t launch_tmem_layout_probe(uint32_t* out, cudaStream_t stream);
cudaError_t launch_prologue(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* g, const __nv_bfloat16* beta,
                            const float* A_log, const float* dt_bias, float gate_scale, int64_t rows, int H, __nv_bfloat16* qn,
                            __nv_bfloat16* kn, float* gact, float* beta_act, cudaStream_t stream);
cudaError_t launch_umma_selftest(const __nv_bfloat16* A, const __nv_bfloat16* B, float* D, int mode, int reps, int* status,
                                 cudaStream_t stream);
}  // namespace fkda

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(FKDA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

struct Layout {
  int64_t prefix_off;      // int32 [N+1]
  int64_t records_off;
  int64_t chunks_per_head; // records per head
  int64_t seg_off;         // fp32 slots of the segment-parallel scan (seg_bytes may be 0)
  int64_t seg_bytes;
  int n_segs;              // runs per sequence (1: whole sequences), of seg_chunks chunks each
  int seg_chunks;
  int64_t total_bytes;
};

// Runs per sequence under `flags`: forced by FKDA_FLAG_SEGMENTS(n), switched off by the
// kernel-selection flags, else planned from the sizes.
int segments_for(int64_t chains, int64_t chunks_per_seq, int64_t flags, int* seg_chunks) {
  *seg_chunks = 0;
  if (flags & (FKDA_FLAG_SCAN_SIMT | FKDA_FLAG_SCAN_NO_SEGMENTS)) return 1;
  const int64_t forced = (flags >> 8) & 0xff;
  if ((flags & FKDA_FLAG_SCAN_PLAIN) && forced < 2) return 1;
  if (forced >= 2) {
    if (chunks_per_seq < forced) return 1;
    *seg_chunks = static_cast<int>((chunks_per_seq + forced - 1) / forced);
    return static_cast<int>(forced);
  }
  if (flags & FKDA_FLAG_SCAN_LOOKAHEAD) return 1;
  return fkda::plan_segments(chains, chunks_per_seq, seg_chunks, fkda::device_sm_count());
}

// `varlen` < 0: size for whichever mode needs more (the upper bound T_total/32 + N covers both).
bool make_layout(int64_t T_total, int64_t H, int64_t N, int varlen, int64_t T_per_seq, int64_t flags, Layout* L) {
  if (T_total < 0 || H <= 0 || N <= 0) return false;
  int64_t chunks;
  if (varlen == 0) chunks = N * ((T_per_seq + fkda::kChunk - 1) / fkda::kChunk);
  else chunks = T_total / fkda::kChunk + N;
  if (varlen < 0) {
    int64_t fixed_ub = (T_total + fkda::kChunk - 1) / fkda::kChunk + N;
    chunks = fixed_ub > chunks ? fixed_ub : chunks;
    if (T_total % N == 0) T_per_seq = T_total / N; else varlen = 1;   // a fixed-length call has T_total = N T
  }
  L->prefix_off = fkda::kWsHeaderBytes;
  int64_t prefix_bytes = ((2 * N + 1) * 4 + 255) / 256 * 256;   // chunk prefix [N+1] followed by the chain order [N]
  L->records_off = L->prefix_off + prefix_bytes;
  L->chunks_per_head = chunks;
  L->seg_off = L->records_off + chunks * H * static_cast<int64_t>(fkda::kRecBytes);
  L->n_segs = 1;
  L->seg_chunks = 0;
  if (N * H <= 0x7fffffffLL) {
    // Fixed-length: planned from the sequence length.  Varlen: the lengths are on the device, so the number of runs is
    // planned for sequences of the average length and the run length follows the longest sequence, on the device.
    // (A size query, varlen < 0, gets the same plan either way: both use T_total / N.)
    const int64_t per_seq = varlen > 0 ? (T_total / N + fkda::kChunk - 1) / fkda::kChunk : (T_per_seq + fkda::kChunk - 1) / fkda::kChunk;
    L->n_segs = segments_for(N * H, per_seq, flags, &L->seg_chunks);
  }
  L->seg_bytes = L->n_segs > 1 ? N * H * L->n_segs * 3 * fkda::kSegSlotFloats * 4 : 0;
  L->total_bytes = L->seg_off + L->seg_bytes;
  return true;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate(const fkda_fwd_params* p, Layout* L) {
  if (!p) return fail(FKDA_ERR_INVALID_ARGUMENT, "params is NULL");
  if (!p->q || !p->k || !p->v || !p->g || !p->beta || !p->out) return fail(FKDA_ERR_INVALID_ARGUMENT, "q, k, v, g, beta and out must be non-NULL");
  if (!p->A_log || !p->dt_bias) return fail(FKDA_ERR_INVALID_ARGUMENT, "A_log and dt_bias must be non-NULL");
  if (p->B <= 0 || p->H <= 0 || p->T < 0) return fail(FKDA_ERR_INVALID_ARGUMENT, "B and H must be positive and T non-negative");
  if (p->cu_seqlens) {
    if (p->B != 1) return fail(FKDA_ERR_INVALID_ARGUMENT, "B must be 1 when cu_seqlens is provided");
    if (p->N <= 0) return fail(FKDA_ERR_INVALID_ARGUMENT, "cu_seqlens must have at least 2 elements");
  } else if (p->N != p->B) {
    return fail(FKDA_ERR_INVALID_ARGUMENT, "N must equal B when cu_seqlens is not provided");
  }
  if ((p->initial_state || p->final_state) && p->state_dtype != FKDA_STATE_BF16 && p->state_dtype != FKDA_STATE_FP32)
    return fail(FKDA_ERR_INVALID_ARGUMENT, "state_dtype must be bf16 or fp32 when a state tensor is given");
  if (!std::isfinite(p->scale) || !std::isfinite(p->lower_bound)) return fail(FKDA_ERR_INVALID_ARGUMENT, "scale and lower_bound must be finite");
  if (p->lower_bound > 0.f || p->lower_bound < -5.2f)
    return fail(FKDA_ERR_INVALID_ARGUMENT, "lower_bound must lie in [-5.2, 0]: a 16-token sub-block may decay by at most 2^120");
  const void* ptrs[] = {p->q, p->k, p->v, p->g, p->out, p->dt_bias, p->initial_state, p->final_state};
  for (const void* x : ptrs)
    if (x && !aligned16(x)) return fail(FKDA_ERR_INVALID_ARGUMENT, "tensor base addresses must be 16-byte aligned");
  const int64_t T_total = p->B * p->T;
  if (p->H > 65535) return fail(FKDA_ERR_INVALID_ARGUMENT, "H must be at most 65535");
  if (p->N * p->H > 0x7fffffffLL) return fail(FKDA_ERR_INVALID_ARGUMENT, "N*H exceeds 2^31-1 chains");
  if (!make_layout(T_total, p->H, p->N, p->cu_seqlens ? 1 : 0, p->T, p->flags, L)) return fail(FKDA_ERR_INVALID_ARGUMENT, "bad sizes");
  if (L->chunks_per_head * p->H > 0x7fffffffLL) return fail(FKDA_ERR_INVALID_ARGUMENT, "too many (chunk, head) pairs for one call");
  if (!p->workspace) return fail(FKDA_ERR_INVALID_ARGUMENT, "workspace is NULL");
  if (reinterpret_cast<uintptr_t>(p->workspace) & 255u) return fail(FKDA_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
  if (p->workspace_bytes < L->total_bytes)
    return fail(FKDA_ERR_WORKSPACE_TOO_SMALL, "workspace has %lld bytes, %lld needed", (long long)p->workspace_bytes, (long long)L->total_bytes);
  return FKDA_OK;
}

int do_prepare(const fkda_fwd_params* p, const Layout& L, cudaStream_t stream, int wait_limit_us = 0, int first_load_only = 0) {
  uint8_t* ws = static_cast<uint8_t*>(p->workspace);
  int* status = reinterpret_cast<int*>(ws);
  int* prefix = reinterpret_cast<int*>(ws + L.prefix_off);
  cudaError_t e = cudaMemsetAsync(ws, 0, fkda::kWsHeaderBytes, stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
  if (p->cu_seqlens) {
    e = fkda::launch_chunk_prefix(p->cu_seqlens, static_cast<int>(p->N), p->B * p->T, static_cast<int>(p->H), L.n_segs, prefix, status, stream);
    if (e != cudaSuccess) return cuda_fail(e, "chunk_prefix launch");
  }
  fkda::PrepParams q{};
  q.q = static_cast<const __nv_bfloat16*>(p->q);
  q.k = static_cast<const __nv_bfloat16*>(p->k);
  q.v = static_cast<const __nv_bfloat16*>(p->v);
  q.g = static_cast<const __nv_bfloat16*>(p->g);
  q.beta = static_cast<const __nv_bfloat16*>(p->beta);
  q.A_log = p->A_log;
  q.dt_bias = p->dt_bias;
  q.cu_seqlens = p->cu_seqlens;
  q.chunk_prefix = prefix;
  q.records = ws + L.records_off;
  q.status = status;
  q.T = p->T;
  q.T_total = p->B * p->T;
  q.H = static_cast<int>(p->H);
  q.N = static_cast<int>(p->N);
  q.total_chunks = static_cast<int>(L.chunks_per_head);
  q.scale = p->scale;
  q.gate_scale = static_cast<float>(static_cast<double>(p->lower_bound) * 1.4426950408889634);
  q.wait_limit_us = wait_limit_us;
  q.first_load_only = first_load_only;
#ifdef FKDA_TUNING
  {
    static const char* dbg_env = getenv("FKDA_PREPARE_SKIP");   // phase-skip timing of the prepare kernel (results are wrong when set)
    q.dbg = dbg_env ? atoi(dbg_env) : 0;
  }
#endif
  if (p->flags & FKDA_FLAG_PREPARE_MMA_SYNC) e = fkda::launch_prepare(q, stream);
  else if (p->flags & FKDA_FLAG_PREPARE_TCGEN05) e = fkda::launch_prepare_tc4(q, stream);
  else e = fkda::launch_prepare_pipe(q, stream);
  if (e != cudaSuccess) return cuda_fail(e, "prepare launch");
  return FKDA_OK;
}

fkda::ScanParams scan_params(const fkda_fwd_params* p, const Layout& L) {
  uint8_t* ws = static_cast<uint8_t*>(p->workspace);
  fkda::ScanParams s{};
  s.records = ws + L.records_off;
  s.cu_seqlens = p->cu_seqlens;
  s.chunk_prefix = reinterpret_cast<const int*>(ws + L.prefix_off);
  s.seq_order = p->cu_seqlens ? s.chunk_prefix + (p->N + 1) : nullptr;
  s.initial_state = p->initial_state;
  s.final_state = p->final_state;
  s.out = static_cast<__nv_bfloat16*>(p->out);
  s.status = reinterpret_cast<int*>(ws);
  s.T = p->T;
  s.T_total = p->B * p->T;
  s.H = static_cast<int>(p->H);
  s.N = static_cast<int>(p->N);
  s.total_chunks = static_cast<int>(L.chunks_per_head);
  s.state_fp32 = p->state_dtype == FKDA_STATE_FP32 ? 1 : 0;
  if (p->cu_seqlens && L.n_segs > 1) s.seg_chunks_dev = s.status + 2;     // set by the chunk-prefix kernel
  return s;
}

int do_scan(const fkda_fwd_params* p, const Layout& L, cudaStream_t stream) {
  uint8_t* ws = static_cast<uint8_t*>(p->workspace);
  fkda::ScanParams s = scan_params(p, L);
  const int sms = fkda::device_sm_count();
  cudaError_t e;
  if (p->flags & FKDA_FLAG_SCAN_SIMT) e = fkda::launch_scan_simt(s, stream);
  else if ((p->flags & (FKDA_FLAG_SCAN_PLAIN | FKDA_FLAG_SCAN_LOOKAHEAD)) && L.n_segs > 1) {
    // a forced run count together with a forced kernel: both passes on that kernel
    e = fkda::launch_scan_segmented(s, L.n_segs, L.seg_chunks, reinterpret_cast<float*>(ws + L.seg_off),
                                    (p->flags & FKDA_FLAG_SCAN_PLAIN) ? 1 : 2, stream);
  } else if (p->flags & FKDA_FLAG_SCAN_PLAIN) e = fkda::launch_scan(s, stream);
  else if (!(p->flags & FKDA_FLAG_SCAN_LOOKAHEAD) && p->cu_seqlens == nullptr && p->T > 0 &&
             (p->T <= 2 * fkda::kChunk || (p->T <= 5 * fkda::kChunk && p->N * p->H > sms))) {
    // short chains: the state-I/O-oriented persistent kernel (up to two chunks always; up to five when there are more
    // chains than SMs, where it still beats the compact kernel: 0.122 against 0.150 ms at 2048 chains of three chunks,
    // 0.190 against 0.194 at six)
    e = fkda::launch_scan_short(s, sms, stream);
  } else if (!(p->flags & FKDA_FLAG_SCAN_LOOKAHEAD) && p->N * p->H > sms) {
    // More chains than SMs: the compact kernel, two CTAs per SM.  Equal-length chains: always.  Varlen: the
    // chunk-prefix kernel has decided on the device (status word 1); both kernels are launched and the CTAs of the
    // one that was not chosen leave at once.
    if (p->cu_seqlens == nullptr || p->N * p->H > 1024) {
      // (beyond about a thousand chains the empty launch would cost more than a wrong choice, and one long sequence
      // among so many chains rarely sets the duration)
      e = fkda::launch_scan(s, stream);
    } else {
      s.select = s.status + 1;
      s.select_want = 1;
      e = fkda::launch_scan(s, stream);
      s.select_want = 0;
      if (e == cudaSuccess) e = fkda::launch_scan2(s, stream);
    }
  } else if (L.n_segs > 1) {
    // few long chains: cut them into runs that are walked in parallel
    e = fkda::launch_scan_segmented(s, L.n_segs, L.seg_chunks, reinterpret_cast<float*>(ws + L.seg_off), 0, stream);
  } else e = fkda::launch_scan2(s, stream);
  if (e != cudaSuccess) return cuda_fail(e, "scan launch");
  return FKDA_OK;
}

}  // namespace

extern "C" {

int fkda_get_workspace_size_flags(int64_t T_total, int64_t H, int64_t N, int64_t flags, int64_t* bytes) {
  Layout L;
  if (!bytes) return fail(FKDA_ERR_INVALID_ARGUMENT, "bytes is NULL");
  if (!make_layout(T_total, H, N, -1, 0, flags, &L)) return fail(FKDA_ERR_INVALID_ARGUMENT, "T_total >= 0, H > 0 and N > 0 required");
  *bytes = L.total_bytes;
  return FKDA_OK;
}

int fkda_get_workspace_size(int64_t T_total, int64_t H, int64_t N, int64_t* bytes) {
  return fkda_get_workspace_size_flags(T_total, H, N, 0, bytes);
}

int fkda_plan_segments(int64_t chains, int64_t chunks_per_sequence, int* segments, int* chunks_per_segment) {
  if (!segments || !chunks_per_segment) return fail(FKDA_ERR_INVALID_ARGUMENT, "NULL pointer");
  *segments = fkda::plan_segments(chains, chunks_per_sequence, chunks_per_segment, fkda::device_sm_count());
  return FKDA_OK;
}

int fkda_workspace_layout(int64_t T_total, int64_t H, int64_t N, int varlen, int64_t T_per_seq, int64_t* records_offset,
                          int64_t* record_bytes, int64_t* chunks_per_head) {
  Layout L;
  if (!make_layout(T_total, H, N, varlen ? 1 : 0, T_per_seq, 0, &L)) return fail(FKDA_ERR_INVALID_ARGUMENT, "bad sizes");
  if (records_offset) *records_offset = L.records_off;
  if (record_bytes) *record_bytes = fkda::kRecBytes;
  if (chunks_per_head) *chunks_per_head = L.chunks_per_head;
  return FKDA_OK;
}

int fkda_workspace_bytes_exact(int64_t T_total, int64_t H, int64_t N, int varlen, int64_t T_per_seq, int64_t flags, int64_t* bytes) {
  Layout L;
  if (!bytes) return fail(FKDA_ERR_INVALID_ARGUMENT, "bytes is NULL");
  if (!make_layout(T_total, H, N, varlen ? 1 : 0, T_per_seq, flags, &L)) return fail(FKDA_ERR_INVALID_ARGUMENT, "bad sizes");
  *bytes = L.total_bytes;
  return FKDA_OK;
}

int fkda_prepare(const fkda_fwd_params* p, void* cuda_stream) {
  Layout L;
  int rc = validate(p, &L);
  if (rc != FKDA_OK) return rc;
  return do_prepare(p, L, static_cast<cudaStream_t>(cuda_stream));
}

int fkda_scan(const fkda_fwd_params* p, void* cuda_stream) {
  Layout L;
  int rc = validate(p, &L);
  if (rc != FKDA_OK) return rc;
  return do_scan(p, L, static_cast<cudaStream_t>(cuda_stream));
}

int fkda_fwd(const fkda_fwd_params* p, void* cuda_stream) {
  Layout L;
  int rc = validate(p, &L);
  if (rc != FKDA_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (p->flags & FKDA_FLAG_REFERENCE_ROUNDING) {
    // debugging aid: the reference's tile size, state type and rounding points (one kernel, any shape)
    cudaError_t e = cudaMemsetAsync(p->workspace, 0, fkda::kWsHeaderBytes, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
    e = fkda::launch_refmode(static_cast<const __nv_bfloat16*>(p->q), static_cast<const __nv_bfloat16*>(p->k),
                             static_cast<const __nv_bfloat16*>(p->v), static_cast<const __nv_bfloat16*>(p->g),
                             static_cast<const __nv_bfloat16*>(p->beta), p->A_log, p->dt_bias, p->initial_state, p->final_state,
                             static_cast<__nv_bfloat16*>(p->out), p->cu_seqlens, p->N, p->T, p->B * p->T, static_cast<int>(p->H),
                             p->state_dtype == FKDA_STATE_FP32 ? 1 : 0, p->scale,
                             static_cast<float>(static_cast<double>(p->lower_bound) * 1.4426950408889634), stream);
    if (e != cudaSuccess) return cuda_fail(e, "reference-rounding kernel launch");
    return FKDA_OK;
  }
  const bool fused_any_t = (p->flags & 0xff57u) == FKDA_FLAG_FUSED_ANY_T;
  if (p->cu_seqlens == nullptr && p->T > 0 && (fused_any_t || (p->T <= fkda::kFusedMaxT && (p->flags & 0xff57u) == 0))) {
    // short fixed-length sequences (a continuation step): one fused kernel, no operand records
    cudaError_t e = cudaMemsetAsync(p->workspace, 0, fkda::kWsHeaderBytes, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
    e = fkda::launch_short16(static_cast<const __nv_bfloat16*>(p->q), static_cast<const __nv_bfloat16*>(p->k),
                             static_cast<const __nv_bfloat16*>(p->v), static_cast<const __nv_bfloat16*>(p->g),
                             static_cast<const __nv_bfloat16*>(p->beta), p->A_log, p->dt_bias, p->initial_state, p->final_state,
                             static_cast<__nv_bfloat16*>(p->out), p->N, static_cast<int>(p->T), static_cast<int>(p->H),
                             p->state_dtype == FKDA_STATE_FP32 ? 1 : 0, p->scale,
                             static_cast<float>(static_cast<double>(p->lower_bound) * 1.4426950408889634),
                             static_cast<int*>(p->workspace), stream);
    if (e != cudaSuccess) return cuda_fail(e, "short-sequence kernel launch");
    return FKDA_OK;
  }
  rc = do_prepare(p, L, stream);
  if (rc != FKDA_OK) return rc;
  return do_scan(p, L, stream);
}

int fkda_prologue(const void* q, const void* k, const void* g, const void* beta, const float* A_log, const float* dt_bias,
                  float lower_bound, int64_t T_total, int64_t H, void* qn, void* kn, float* gate, float* beta_act,
                  void* cuda_stream) {
  if (!q || !k || !g || !beta || !A_log || !dt_bias || !qn || !kn || !gate || !beta_act)
    return fail(FKDA_ERR_INVALID_ARGUMENT, "NULL pointer");
  if (T_total < 0 || H <= 0 || H > 0x7fffffffLL) return fail(FKDA_ERR_INVALID_ARGUMENT, "bad sizes");
  cudaError_t e = fkda::launch_prologue(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(g),
      static_cast<const __nv_bfloat16*>(beta), A_log, dt_bias, static_cast<float>(static_cast<double>(lower_bound) * 1.4426950408889634),
      T_total * H, static_cast<int>(H), static_cast<__nv_bfloat16*>(qn), static_cast<__nv_bfloat16*>(kn), gate, beta_act,
      static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_fail(e, "prologue launch");
  return FKDA_OK;
}

int fkda_read_status(const void* workspace, void* cuda_stream, int* status) {
  if (!workspace || !status) return fail(FKDA_ERR_INVALID_ARGUMENT, "NULL pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaMemcpyAsync(status, workspace, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(status)");
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  if (*status != 0) return fail(FKDA_ERR_DEVICE_STATUS, "device status %d (%s)", *status,
                                *status == 1 ? "cu_seqlens not monotone inside [0, T_total]" : "a bounded wait inside a kernel gave up");
  return FKDA_OK;
}

int fkda_selftest_umma(const void* A, const void* B, float* D, int mode, int reps, int* status, void* cuda_stream) {
  if (!A || !B || !D || !status || mode < 0 || mode > 4 || reps < 1) return fail(FKDA_ERR_INVALID_ARGUMENT, "bad arguments");
  cudaError_t e = fkda::launch_umma_selftest(static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), D, mode,
                                             reps, status, static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_fail(e, "selftest launch");
  return FKDA_OK;
}

int fkda_debug_scan_giveup(const fkda_fwd_params* p, int stop_copies_after, int wait_limit_us, void* cuda_stream) {
  Layout L;
  int rc = validate(p, &L);
  if (rc != FKDA_OK) return rc;
  if (stop_copies_after < 1 || wait_limit_us < 1 || wait_limit_us > 1000000)
    return fail(FKDA_ERR_INVALID_ARGUMENT, "stop_copies_after >= 1 and 1 <= wait_limit_us <= 1000000 required");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  rc = do_prepare(p, L, stream);
  if (rc != FKDA_OK) return rc;
  fkda::ScanParams s = scan_params(p, L);
  s.seg_chunks_dev = nullptr;          // whole sequences on the look-ahead kernel
  s.wait_limit_us = wait_limit_us;
  s.stop_copies_after = stop_copies_after;
  cudaError_t e = fkda::launch_scan2(s, stream);
  if (e != cudaSuccess) return cuda_fail(e, "scan launch");
  return FKDA_OK;
}

int fkda_debug_prepare_giveup(const fkda_fwd_params* p, int wait_limit_us, void* cuda_stream) {
  Layout L;
  int rc = validate(p, &L);
  if (rc != FKDA_OK) return rc;
  if (wait_limit_us < 1 || wait_limit_us > 1000000) return fail(FKDA_ERR_INVALID_ARGUMENT, "1 <= wait_limit_us <= 1000000 required");
  if (p->flags & (FKDA_FLAG_PREPARE_TCGEN05 | FKDA_FLAG_PREPARE_MMA_SYNC))
    return fail(FKDA_ERR_INVALID_ARGUMENT, "the give-up aid drives the pipelined kernel: no kernel-selection flag");
  return do_prepare(p, L, static_cast<cudaStream_t>(cuda_stream), wait_limit_us, 1);
}

#ifdef FKDA_TUNING
int fkda_debug_tmem_bench(int nwarps, int reps, void* out, void* cuda_stream) {
  if (nwarps < 1 || nwarps > 16 || reps < 1 || !out) return fail(FKDA_ERR_INVALID_ARGUMENT, "bad arguments");
  cudaError_t e = fkda::launch_tmem_bench(nwarps, reps, static_cast<long long*>(out), static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_fail(e, "tmem bench launch");
  return FKDA_OK;
}

int fkda_debug_umma_bench(int issuers, int reps, int ksteps, int n, int a_in_tmem, void* out, int* status, void* cuda_stream) {
  if (issuers < 1 || issuers > 4 || reps < 1 || reps > 4096 || ksteps < 1 || ksteps > 8 || (n != 32 && n != 64 && n != 128) || !out || !status)
    return fail(FKDA_ERR_INVALID_ARGUMENT, "bad arguments");
  cudaError_t e = fkda::launch_umma_bench(issuers, reps, ksteps, n, a_in_tmem ? 1 : 0, static_cast<long long*>(out), status,
                                          static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_fail(e, "umma bench launch");
  return FKDA_OK;
}

#endif  // FKDA_TUNING

int fkda_debug_tmem_layout_probe(void* out, void* cuda_stream) {
  if (!out) return fail(FKDA_ERR_INVALID_ARGUMENT, "out is NULL");
  cudaError_t e = fkda::launch_tmem_layout_probe(static_cast<uint32_t*>(out), static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_fail(e, "tmem layout probe launch");
  return FKDA_OK;
}

#ifdef FKDA_TUNING
int fkda_debug_set_prepare_trace(void* device_buffer) {
  fkda::set_prepare_trace(static_cast<long long*>(device_buffer));
  return FKDA_OK;
}

int fkda_debug_set_scan_trace(void* device_buffer) {
  fkda::set_scan_trace(static_cast<unsigned long long*>(device_buffer));
  return FKDA_OK;
}
#endif

const char* fkda_last_error(void) { return g_err; }

const char* fkda_version(void) { return "fkda 0.1 (sm_100a)"; }

}  // extern "C"
