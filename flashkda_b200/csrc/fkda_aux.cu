// Auxiliary kernels around the two main ones:
//   * prologue_kernel: the token-wise prologue on its own (q/k L2 norm, activated gate, beta
//     sigmoid), a pure streaming kernel with 16-byte loads/stores.  The prepare kernel fuses
//     the same math; this entry exists so the stage can be tested and profiled alone.
//   * scan_simt_kernel: a plain-CUDA-core evaluation of the inter-chunk recurrence from the
//     same operand records.  Bring-up and verification aid (flag FKDA_FLAG_SCAN_SIMT): it
//     shares no tensor-core code with the tcgen05 scan, so a disagreement between the two
//     isolates descriptor/layout mistakes.  Not a dispatch target for production calls.
//   * umma_selftest_kernel: one-CTA products through exactly the descriptor flavours the scan
//     uses, read back from TMEM, for comparison with a host matmul.
#include "fkda_common.cuh"

namespace fkda {

// ---- standalone prologue -------------------------------------------------------------------------
// One warp per (token, head) row: lane l owns channels 4l..4l+3 (8-byte loads, 256 B per row).
// Two rows per warp iteration would give 16-byte accesses; instead each lane handles 8 channels
// of one of two rows (lanes 0-15 row A, lanes 16-31 row B) so every access is 16 bytes.
__global__ void __launch_bounds__(256) prologue_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                       const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ beta,
                                                       const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                       float gate_scale, int64_t rows, int H, __nv_bfloat16* __restrict__ qn,
                                                       __nv_bfloat16* __restrict__ kn, float* __restrict__ gact,
                                                       float* __restrict__ beta_act) {
  const int lane = threadIdx.x & 31;
  const int half = lane >> 4, l16 = lane & 15;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t pair = warp_global; pair * 2 < rows; pair += nwarps) {
    const int64_t row = pair * 2 + half;
    const bool valid = row < rows;
    const int h = valid ? static_cast<int>(row % H) : 0;
    const size_t off = static_cast<size_t>(valid ? row : 0) * kD + 8 * l16;
    uint4 qw = __ldg(reinterpret_cast<const uint4*>(q + off));
    uint4 kw = __ldg(reinterpret_cast<const uint4*>(k + off));
    uint4 gw = __ldg(reinterpret_cast<const uint4*>(g + off));
    float qf[8] = {bf_lo(qw.x), bf_hi(qw.x), bf_lo(qw.y), bf_hi(qw.y), bf_lo(qw.z), bf_hi(qw.z), bf_lo(qw.w), bf_hi(qw.w)};
    float kf[8] = {bf_lo(kw.x), bf_hi(kw.x), bf_lo(kw.y), bf_hi(kw.y), bf_lo(kw.z), bf_hi(kw.z), bf_lo(kw.w), bf_hi(kw.w)};
    float gf[8] = {bf_lo(gw.x), bf_hi(gw.x), bf_lo(gw.y), bf_hi(gw.y), bf_lo(gw.z), bf_hi(gw.z), bf_lo(gw.w), bf_hi(gw.w)};
    float sq = 0.f, sk = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sq = fmaf(qf[i], qf[i], sq);
      sk = fmaf(kf[i], kf[i], sk);
    }
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, d);
      sk += __shfl_xor_sync(0xffffffffu, sk, d);
    }
    const float rq = rsqrtf(sq + 1e-6f), rk = rsqrtf(sk + 1e-6f);
    const float a = ex2f(__ldg(A_log + h) * kLog2e);
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(dt_bias + h * kD + 8 * l16));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(dt_bias + h * kD + 8 * l16 + 4));
    const float bias[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    float ga[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) ga[i] = gate_scale * sigmoid_fast(a * (gf[i] + bias[i]));
    if (valid) {
      *reinterpret_cast<uint4*>(qn + off) = make_uint4(pack_bf16(qf[0] * rq, qf[1] * rq), pack_bf16(qf[2] * rq, qf[3] * rq),
                                                       pack_bf16(qf[4] * rq, qf[5] * rq), pack_bf16(qf[6] * rq, qf[7] * rq));
      *reinterpret_cast<uint4*>(kn + off) = make_uint4(pack_bf16(kf[0] * rk, kf[1] * rk), pack_bf16(kf[2] * rk, kf[3] * rk),
                                                       pack_bf16(kf[4] * rk, kf[5] * rk), pack_bf16(kf[6] * rk, kf[7] * rk));
      *reinterpret_cast<float4*>(gact + off) = make_float4(ga[0], ga[1], ga[2], ga[3]);
      *reinterpret_cast<float4*>(gact + off + 4) = make_float4(ga[4], ga[5], ga[6], ga[7]);
      if (l16 == 0) beta_act[row] = sigmoid_fast(__bfloat162float(beta[row]));
    }
  }
}

cudaError_t launch_prologue(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* g, const __nv_bfloat16* beta,
                            const float* A_log, const float* dt_bias, float gate_scale, int64_t rows, int H, __nv_bfloat16* qn,
                            __nv_bfloat16* kn, float* gact, float* beta_act, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  int64_t blocks = (rows / 2 + 7) / 8 + 1;    // 8 warps per block, 2 rows per warp pass
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  prologue_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(q, k, g, beta, A_log, dt_bias, gate_scale, rows, H, qn, kn,
                                                                     gact, beta_act);
  return cudaGetLastError();
}

// ---- CUDA-core evaluation of the recurrence from operand records ------------------------------------
constexpr int kSimtSmemBytes = kD * kD * 4 + kRecBytes + kChunk * kD * 4;

__device__ __forceinline__ float rec_bf(const uint8_t* base, int off) {
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + off));
}

__global__ void __launch_bounds__(256) scan_simt_kernel(const ScanParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* S = reinterpret_cast<float*>(smem);                       // [k][v]
  uint8_t* rec = smem + kD * kD * 4;
  float* U = reinterpret_cast<float*>(smem + kD * kD * 4 + kRecBytes);   // [tok][v]
  const int tid = threadIdx.x;
  const int chain = blockIdx.x;
  const int n = chain / p.H, h = chain - n * p.H;
  int64_t bos, eos;
  int chunk_base;
  if (p.cu_seqlens != nullptr) {
    bos = p.cu_seqlens[n];
    eos = p.cu_seqlens[n + 1];
    bos = bos < 0 ? 0 : (bos > p.T_total ? p.T_total : bos);
    eos = eos < bos ? bos : (eos > p.T_total ? p.T_total : eos);
    chunk_base = p.chunk_prefix[n];
  } else {
    bos = static_cast<int64_t>(n) * p.T;
    eos = bos + p.T;
    chunk_base = n * static_cast<int>((p.T + kChunk - 1) / kChunk);
  }
  int nchunks = static_cast<int>((eos - bos + kChunk - 1) / kChunk);
  {  // never read past the records of this head, whatever cu_seqlens claims
    const int avail = p.total_chunks > chunk_base ? p.total_chunks - chunk_base : 0;
    if (nchunks > avail) nchunks = avail;
  }
  const size_t state_off = (static_cast<size_t>(n) * p.H + h) * kD * kD;
  for (int i = tid; i < kD * kD; i += 256) {
    const int vv = i / kD, kk = i % kD;   // stored [v][k]
    float s0 = 0.f;
    if (p.initial_state != nullptr)
      s0 = p.state_fp32 ? reinterpret_cast<const float*>(p.initial_state)[state_off + i]
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.initial_state)[state_off + i]);
    S[kk * kD + vv] = s0;
  }
  __syncthreads();
  const int v = tid & 127, part = tid >> 7;   // each thread: one v column, 16 of the 32 tokens / 64 of the 128 k rows
  for (int c = 0; c < nchunks; ++c) {
    const uint4* src = reinterpret_cast<const uint4*>(p.records + (static_cast<size_t>(h) * p.total_chunks + chunk_base + c) * kRecBytes);
    for (int i = tid; i < kRecBytes / 16; i += 256) reinterpret_cast<uint4*>(rec)[i] = src[i];
    __syncthreads();
    float o[16];
    for (int t = 0; t < 16; ++t) {
      const int tok = part * 16 + t;
      float w = 0.f, oo = 0.f;
      for (int kk = 0; kk < kD; ++kk) {
        const float s = S[kk * kD + v];
        w = fmaf(rec_bf(rec, kRecWP + core_off(tok, kk, kD)), s, w);
        oo = fmaf(rec_bf(rec, kRecQP + core_off(tok, kk, kD)), s, oo);
      }
      U[tok * kD + v] = rec_bf(rec, kRecUP + core_off(v, tok, kChunk)) - w;
      o[t] = oo;
    }
    __syncthreads();
    const int64_t tok0 = bos + static_cast<int64_t>(c) * kChunk;
    for (int t = 0; t < 16; ++t) {
      const int tok = part * 16 + t;
      float oo = o[t];
      for (int j = 0; j <= tok; ++j) oo = fmaf(rec_bf(rec, kRecMQK + core_off(tok, j, kChunk)), U[j * kD + v], oo);
      if (tok0 + tok < eos) p.out[(static_cast<size_t>(tok0 + tok) * p.H + h) * kD + v] = __float2bfloat16_rn(oo);
    }
    const float* e = reinterpret_cast<const float*>(rec + kRecE);
    for (int kk = part * 64; kk < part * 64 + 64; ++kk) {
      float acc = S[kk * kD + v] * e[kk];
      for (int j = 0; j < kChunk; ++j) acc = fmaf(rec_bf(rec, kRecKR + core_off(j, kk, kD)), U[j * kD + v], acc);
      S[kk * kD + v] = acc;
    }
    __syncthreads();
  }
  if (p.final_state != nullptr)
    for (int i = tid; i < kD * kD; i += 256) {
      const int vv = i / kD, kk = i % kD;
      const float s = S[kk * kD + vv];
      if (p.state_fp32) reinterpret_cast<float*>(p.final_state)[state_off + i] = s;
      else reinterpret_cast<__nv_bfloat16*>(p.final_state)[state_off + i] = __float2bfloat16_rn(s);
    }
}

cudaError_t launch_scan_simt(const ScanParams& p, cudaStream_t stream) {
  static SmemOptIn opt_in;
  cudaError_t e = opt_in.ensure(scan_simt_kernel, kSimtSmemBytes);
  if (e != cudaSuccess) return e;
  const int64_t chains = static_cast<int64_t>(p.N) * p.H;
  if (chains == 0) return cudaSuccess;
  scan_simt_kernel<<<static_cast<unsigned>(chains), 256, kSimtSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

// ---- tcgen05 descriptor self-test -------------------------------------------------------------------
// mode 0: D[128][32]  = A[128][128] B[32][128]^T      (both K-major in shared memory, 8-row groups 2048 B apart)
// mode 1: D[128][128] = A[128][32]  B[32][128]         (A K-major 512 B groups; B read MN-major)
// mode 2: D[128][32]  = A[128][32]  B[32][32]^T        (both K-major, 512 B groups)
// mode 3: as mode 0 with A read from tensor memory (bf16 pairs per column)
// mode 4: as mode 1 with A read from tensor memory
// Inputs are row-major bf16 in global memory; `reps` > 1 re-issues the product with accumulation
// (result = reps * product).  D is written row-major fp32.  status[0] = 1 on a wait timeout.
__global__ void __launch_bounds__(128) umma_selftest_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                                                            float* __restrict__ Dout, int mode, int reps, int* status) {
  __shared__ __align__(1024) uint8_t sA[32768];
  __shared__ __align__(1024) uint8_t sB[8192];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool a_in_tmem = mode >= 3;
  const int shape = a_in_tmem ? mode - 3 : mode;         // 0: K=128,N=32   1: K=32,N=128 (B MN-major)   2: K=32,N=32
  const int ka = (shape == 0) ? 128 : 32;                // K extent
  const int nn = (shape == 1) ? 128 : 32;                // N extent
  for (int i = tid; i < 128 * ka; i += 128) {
    const int r = i / ka, c = i % ka;
    *reinterpret_cast<__nv_bfloat16*>(sA + core_off(r, c, ka)) = A[i];
  }
  if (shape == 1) {      // B given as [32 k][128 n], kept in that orientation (core layout of a [32][128] tile)
    for (int i = tid; i < 32 * 128; i += 128) *reinterpret_cast<__nv_bfloat16*>(sB + core_off(i / 128, i % 128, 128)) = B[i];
  } else {               // B given as [32 n][ka k]
    for (int i = tid; i < 32 * ka; i += 128) *reinterpret_cast<__nv_bfloat16*>(sB + core_off(i / ka, i % ka, ka)) = B[i];
  }
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&mbar), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 256);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t a_tm = tmem + 128;                      // A operand columns when read from tensor memory
  if (a_in_tmem) {
    // row `tid` of A -> TMEM lane `tid`, 16 columns (32 bf16) at a time
    for (int cb = 0; cb < ka / 32; ++cb) {
      uint32_t y[16];
      for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(A + tid * ka + cb * 32 + 2 * i);
        y[i] = *reinterpret_cast<const uint32_t*>(&v2);
      }
      tmem_st16(a_tm + (static_cast<uint32_t>(warp * 32) << 16) + cb * 16, y);
    }
    tmem_wait_st();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (tid == 0) {
    const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
    for (int rep = 0; rep < reps; ++rep) {
      const int ksteps = ka / 16;
      for (int ks = 0; ks < ksteps; ++ks) {
        const uint32_t acc = (rep > 0 || ks > 0) ? 1u : 0u;
        uint64_t bdesc;
        uint32_t idesc;
        if (shape == 0) { bdesc = umma_desc(b_addr + ks * 256, 128, 2048); idesc = umma_idesc_bf16(128, 32, 0, 0); }
        else if (shape == 1) { bdesc = umma_desc(b_addr + ks * 4096, 2048, 128); idesc = umma_idesc_bf16(128, 128, 0, 1); }
        else { bdesc = umma_desc(b_addr + ks * 256, 128, 512); idesc = umma_idesc_bf16(128, 32, 0, 0); }
        if (a_in_tmem) umma_ts(tmem, a_tm + ks * 8, bdesc, idesc, acc);
        else umma_ss(tmem, umma_desc(a_addr + ks * 256, 128, shape == 0 ? 2048 : 512), bdesc, idesc, acc);
      }
    }
    umma_commit(smem_u32(&mbar));
  }
  const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&mbar), 0, &abort_flag));
  if (ok) {
    tc_fence_after();
    for (int cb = 0; cb < nn / 32; ++cb) {
      uint32_t x[32];
      tmem_ld32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + cb * 32, x);
      tmem_wait_ld();
      for (int i = 0; i < 32; ++i) Dout[(warp * 32 + lane) * nn + cb * 32 + i] = __uint_as_float(x[i]);
    }
  } else if (lane == 0) {
    atomicExch(status, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

#ifdef FKDA_TUNING
// Micro-benchmark of tensor-memory access (tuning aid): `nwarps` warps each move `reps` x 32 columns between
// registers and their TMEM lane quadrant; out[warp*4 + {0,1,2,3}] = cycles for {ld, st, st16-packed, ld+st} loops.
__global__ void __launch_bounds__(512) tmem_bench_kernel(int reps, long long* out) {
  __shared__ uint32_t tmem_slot;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tq = tmem_slot + (static_cast<uint32_t>((warp & 3) * 32) << 16) + (warp >> 2) * 128;
  uint32_t x[32];
  uint32_t y[16];
  for (int i = 0; i < 32; ++i) x[i] = lane + i;
  for (int i = 0; i < 16; ++i) y[i] = lane * 3 + i;
  for (int i = 0; i < 4; ++i) tmem_st32(tq + 32 * i, x);
  tmem_wait_st();
  __syncthreads();
  long long t0 = clock64();
  for (int r = 0; r < reps; ++r) tmem_ld32(tq + 32 * (r & 3), x);
  tmem_wait_ld();
  long long t1 = clock64();
  __syncthreads();
  long long t2 = clock64();
  for (int r = 0; r < reps; ++r) tmem_st32(tq + 32 * (r & 3), x);
  tmem_wait_st();
  long long t3 = clock64();
  __syncthreads();
  long long t4 = clock64();
  for (int r = 0; r < reps; ++r) tmem_st16(tq + 16 * (r & 7), y);
  tmem_wait_st();
  long long t5 = clock64();
  __syncthreads();
  long long t6 = clock64();
  for (int r = 0; r < reps; ++r) {
    tmem_ld32(tq + 32 * (r & 3), x);
    tmem_wait_ld();
    for (int i = 0; i < 32; ++i) x[i] += 1;
    tmem_st32(tq + 32 * (r & 3), x);
  }
  tmem_wait_st();
  long long t7 = clock64();
  if (lane == 0) {
    out[warp * 4 + 0] = t1 - t0;
    out[warp * 4 + 1] = t3 - t2;
    out[warp * 4 + 2] = t5 - t4;
    out[warp * 4 + 3] = t7 - t6 + (x[5] == 0xdeadbeef);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_slot, 512);
  }
}

#endif  // FKDA_TUNING

// Records the register <-> (lane, column) maps of the 16-lane tensor-memory fragment shapes that the scan kernel's
// state warps use.  One warp.  out[0][t][r], out[1][t][r]: what tcgen05.ld.16x256b.x8 returns for lanes 0-15 and
// 16-31 of a 32 x 64 tile holding (lane << 8 | column); out[2][lane][c]: the tile after a 16x256b.x8 store of
// (1 << 16 | t << 8 | r) to its lanes 0-15; out[3][lane][c] (c < 32): after a 16x128b.x8 store of (2 << 16 | t << 8 | r)
// to lanes 16-31 of a 32-column tile.  All read back with the 32x32b shape, whose map is lane = thread, column = register.
__global__ void __launch_bounds__(32) tmem_layout_probe_kernel(uint32_t* out) {
  __shared__ uint32_t tmem_slot;
  const int lane = threadIdx.x;
  tmem_alloc(smem_u32(&tmem_slot), 256);
  tmem_relinquish();
  tc_fence_before();
  __syncwarp();
  tc_fence_after();
  const uint32_t t0 = tmem_slot;
  uint32_t x[32], y[16];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = (static_cast<uint32_t>(lane) << 8) | static_cast<uint32_t>(half * 32 + i);
    tmem_st32(t0 + half * 32, x);
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) x[i] = 0xffffffffu;
  tmem_st32(t0 + 64, x);
  tmem_st32(t0 + 96, x);
  tmem_st32(t0 + 128, x);
  tmem_wait_st();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    tmem_ld_16x256b_x8(t0 + (static_cast<uint32_t>(16 * half) << 16), x);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) out[(half * 32 + lane) * 32 + i] = x[i];
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) x[i] = (1u << 16) | (static_cast<uint32_t>(lane) << 8) | static_cast<uint32_t>(i);
  tmem_st_16x256b_x8(t0 + 64, x);
#pragma unroll
  for (int i = 0; i < 16; ++i) y[i] = (2u << 16) | (static_cast<uint32_t>(lane) << 8) | static_cast<uint32_t>(i);
  tmem_st_16x128b_x8(t0 + 128 + (16u << 16), y);
  tmem_wait_st();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    tmem_ld32(t0 + 64 + half * 32, x);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) out[2 * 2048 + lane * 64 + half * 32 + i] = x[i];
  }
  tmem_ld32(t0 + 128, x);
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < 32; ++i) out[3 * 2048 + lane * 64 + i] = x[i];
  tc_fence_before();
  __syncwarp();
  tmem_dealloc(t0, 256);
}

cudaError_t launch_tmem_layout_probe(uint32_t* out, cudaStream_t stream) {
  tmem_layout_probe_kernel<<<1, 32, 0, stream>>>(out);
  return cudaGetLastError();
}

#ifdef FKDA_TUNING
// Micro-benchmark of tcgen05.mma issue and completion (tuning aid): `nissuers` (1..4) threads in different warps each
// issue `reps` products of `ksteps` M=128 instructions (K = 16 each) with N = `n` into their own 128 TMEM columns,
// A from shared memory (ts = 0) or tensor memory (ts = 1), then commit and wait.  out[issuer*2 + {0,1}] = cycles until
// the last instruction was issued / until the commit arrived.  Operand contents are irrelevant (zeros).
__global__ void __launch_bounds__(128) umma_bench_kernel(int nissuers, int reps, int ksteps, int n, int ts, long long* out, int* status) {
  __shared__ __align__(1024) uint8_t sA[16384];
  __shared__ __align__(1024) uint8_t sB[16384];
  __shared__ __align__(8) uint64_t mbar[4];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < 4096; i += 128) {
    reinterpret_cast<uint32_t*>(sA)[i] = 0u;
    reinterpret_cast<uint32_t*>(sB)[i] = 0u;
  }
  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&mbar[i]), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  {  // defined contents for the A operand columns read from tensor memory (columns 448..511 of every lane)
    uint32_t z[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) z[i] = 0u;
    tmem_st32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + 448, z);
    tmem_st32(tmem + (static_cast<uint32_t>(warp * 32) << 16) + 480, z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  bool ok = true;
  if (warp < nissuers && lane == 0) {
    const uint32_t idesc = n == 128 ? umma_idesc_bf16(128, 128, 0, 0) : (n == 64 ? umma_idesc_bf16(128, 64, 0, 0) : umma_idesc_bf16(128, 32, 0, 0));
    const uint32_t d = tmem + 96 * warp;           // up to 128 columns each (overlapping between issuers), clear of the A columns at 448
    const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
    const long long t0 = clock64();
    for (int rep = 0; rep < reps; ++rep)
      for (int ks = 0; ks < ksteps; ++ks) {
        // 8-row groups 1024 bytes apart and four k-step offsets: every operand byte read lies inside its 16 KB array
        // (16 groups x 1024 + 3 x 256 + 128 = 17280 - 1024 = 16256 at most)
        const uint64_t bdesc = umma_desc(b_addr + (ks & 3) * 256, 128, 1024);
        if (ts) umma_ts(d, tmem + 448 + (ks & 7) * 8, bdesc, idesc, (rep | ks) ? 1u : 0u);
        else umma_ss(d, umma_desc(a_addr + (ks & 3) * 256, 128, 1024), bdesc, idesc, (rep | ks) ? 1u : 0u);
      }
    const long long t1 = clock64();
    umma_commit(smem_u32(&mbar[warp]));
    ok = mbar_wait(smem_u32(&mbar[warp]), 0, &abort_flag);
    const long long t2 = clock64();
    out[warp * 2 + 0] = t1 - t0;
    out[warp * 2 + 1] = t2 - t0;
    if (!ok) atomicExch(status, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

cudaError_t launch_umma_bench(int nissuers, int reps, int ksteps, int n, int ts, long long* out, int* status, cudaStream_t stream) {
  umma_bench_kernel<<<1, 128, 0, stream>>>(nissuers, reps, ksteps, n, ts, out, status);
  return cudaGetLastError();
}

cudaError_t launch_tmem_bench(int nwarps, int reps, long long* out, cudaStream_t stream) {
  tmem_bench_kernel<<<1, nwarps * 32, 0, stream>>>(reps, out);
  return cudaGetLastError();
}

#endif  // FKDA_TUNING

cudaError_t launch_umma_selftest(const __nv_bfloat16* A, const __nv_bfloat16* B, float* D, int mode, int reps, int* status,
                                 cudaStream_t stream) {
  umma_selftest_kernel<<<1, 128, 0, stream>>>(A, B, D, mode, reps, status);
  return cudaGetLastError();
}

}  // namespace fkda
