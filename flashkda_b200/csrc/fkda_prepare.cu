// Token-parallel half of the KDA prefill: one CTA per (32-token chunk, head).
//
// Replaces the reference's K1 (csrc/smxx/fwd_kernel1.cuh:107-586) with a chunk-32 WY
// formulation.  Per chunk it fuses
//   * the prologue: q/k L2 norm, gate activation and its in-chunk cumulative sum, beta sigmoid
//     (16-byte coalesced loads straight from the [T,H,128] tensors; no beta transpose),
//   * the decay application in two 16-token sub-blocks, so that every 2^(+-cumsum) factor stays
//     inside the fp32/bf16 exponent range for lower_bound >= -5 (16 * 5 * log2(e) = 115.4 < 126),
//   * the intra-chunk products A = tril(k+ k-^T,-1) * beta and M = tril(q+ k-^T), with the
//     cross sub-block quadrant taken between "decayed from sub-block start" and "decayed to
//     sub-block end" operands (both factors <= 1),
//   * T = (I + A)^-1 by fp32 forward substitution (two 16x16 diagonal blocks + one merge),
//   * w' = T diag(beta) k+ and u' = T diag(beta) v,
// and writes one operand record (fkda_common.cuh) for the scan kernel.
#include "fkda_common.cuh"

namespace fkda {

// ---- tiny scheduling kernel (varlen): chunk_prefix[n] = sum_{m<n} ceil(len_m / 32) -------------------
// Replaces the reference's one-thread prefix kernel (fwd_kernel1.cuh:89-104) and also checks
// that cu_seqlens is monotone and inside [0, T_total]; violations are clamped and reported
// through the status word instead of faulting later.
// It also picks the recurrence kernel for batches with more chains than SMs (status[1] = 1: the compact
// kernel, two CTAs per SM): the compact kernel moves more chunks per SM and second but walks one chain more slowly,
// so it is chosen unless the longest sequence alone would then set the duration.
// For batches with few chains that are walked in runs (n_segs > 1) it sets the run length, status[2]: the longest
// sequence's chunks spread over the runs, at least 8 chunks.
constexpr int kOrderMax = 4096;      // batches of more sequences keep the given order
__global__ void chunk_prefix_kernel(const int64_t* __restrict__ cu, int N, int64_t T_total, int H, int n_segs, int sms,
                                    int* __restrict__ prefix, int* __restrict__ status) {
  __shared__ int warp_sums[32];
  __shared__ int carry;
  __shared__ int longest;
  if (threadIdx.x == 0) {
    carry = 0;
    longest = 0;
    prefix[0] = 0;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < N; base += blockDim.x) {
    int n = base + threadIdx.x;
    int cnt = 0;
    if (n < N) {
      int64_t a = cu[n], b = cu[n + 1];
      if (a < 0 || b < a || b > T_total || (n == 0 && a != 0)) {
        atomicCAS(status, kStatusOk, kStatusBadCuSeqlens);
        a = a < 0 ? 0 : (a > T_total ? T_total : a);
        b = b < a ? a : (b > T_total ? T_total : b);
      }
      cnt = static_cast<int>((b - a + kChunk - 1) / kChunk);
      atomicMax(&longest, cnt);
    }
    int x = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int s = (lane < (blockDim.x >> 5)) ? warp_sums[lane] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int y = __shfl_up_sync(0xffffffffu, s, d);
        if (lane >= d) s += y;
      }
      warp_sums[lane] = s;  // inclusive over warps
    }
    __syncthreads();
    int incl = x + (warp > 0 ? warp_sums[warp - 1] : 0) + carry;
    if (n < N) prefix[n + 1] = incl;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    // More chains than SMs.  Sequences of about the same length: the compact kernel holds twice as many chains at once,
    // where the look-ahead kernel would need a second wave.  Otherwise, from two chains per SM on: chunk steps per SM at
    // the compact kernel's rate (1.25 us) against the longest chain walked alone (1.95 us), with a margin of 15 % in
    // favour of the look-ahead kernel.
    const long long chains = static_cast<long long>(N) * H, total_steps = static_cast<long long>(prefix[N]) * H;
    const bool alike = static_cast<long long>(longest) * N * 100 <= 130ll * prefix[N];
    const bool throughput = chains >= 2 * sms && static_cast<long long>(longest) * 195 * sms * 100 <= total_steps * 125 * 85;
    status[1] = (chains > sms && (alike || throughput)) ? 1 : 0;
    const int run_len = n_segs > 1 ? (longest + n_segs - 1) / n_segs : 0;
    status[2] = run_len < 8 ? 8 : run_len;
  }
  // Chain order for the scan: longest sequences first (longest-processing-time-first packing of unequal chains
  // onto the SMs; the reference walks sequences in the given order).  order[] follows prefix[] in memory.
  int* order = prefix + (N + 1);
  if (N <= kOrderMax) {
    // bitonic sort of (chunks descending, index ascending) keys in shared memory
    __shared__ unsigned long long keys[kOrderMax];
    __syncthreads();                                   // prefix[] of the last block of sequences is complete
    int P = 1;
    while (P < N) P <<= 1;
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
      unsigned long long key = ~0ull;                  // padding sorts last
      if (i < N) {
        const unsigned len = static_cast<unsigned>(prefix[i + 1] - prefix[i]);
        key = (static_cast<unsigned long long>(0xffffffffu - len) << 32) | static_cast<unsigned>(i);
      }
      keys[i] = key;
    }
    __syncthreads();
    for (int k = 2; k <= P; k <<= 1)
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int t = threadIdx.x; t < (P >> 1); t += blockDim.x) {     // one compare-exchange per pair
          const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1)), partner = i | j;
          const unsigned long long x = keys[i], y = keys[partner];
          const bool ascending = (i & k) == 0;
          if ((x > y) == ascending) { keys[i] = y; keys[partner] = x; }
        }
        __syncthreads();
      }
    for (int i = threadIdx.x; i < N; i += blockDim.x) order[i] = static_cast<int>(keys[i] & 0xffffffffu);
  } else {
    for (int n = threadIdx.x; n < N; n += blockDim.x) order[n] = n;
  }
}

// ---- shared-memory plan of the prepare kernel (byte offsets) --------------------------------------
// The record under construction occupies [0, kRecBytes); everything is arranged so that four CTAs fit one SM.
// Raw q, k, g tiles are staged at the start of the record image ([3][32 tok][256 B], 16-byte chunks XOR-swizzled by
// the token index) before anything of the record is written.  The WP and UP regions are written last, so until the
// intra-chunk products are done they hold three temporaries.  KR, E and QP are final after P2 and leave early; once
// that copy has read them (checked before the barrier that ends P4) the KR region holds the fp32 inverse and the QP
// region receives the v tile, which is fetched only then.
constexpr int kSmStageQKG = 0;               // 24 KB, dead after P1
constexpr int kSmKM = kRecWP;                // [32][128] k-, relative to own sub-block start   (dead after P4)
constexpr int kSmKP1 = kRecUP;               // [16][128] k+ of sub-block 1 rel. to its own start (dead after P4)
constexpr int kSmQP1 = kRecUP + 4096;        // [16][128] q+ of sub-block 1 rel. to its own start (dead after P4)
constexpr int kLd = 36;                      // row stride (floats) of the small fp32 matrices: 16-byte aligned rows
constexpr int kSmT = kRecKR;                 // [32][36] fp32 T                                  (from P5 on)
constexpr int kSmX = kSmT + 32 * kLd * 4;    // [16][36] fp32                                    (P5)
static_assert(kSmX + 16 * kLd * 4 <= kRecKR + 8192, "T and X fit the KR region");
constexpr int kSmV = kRecQP;                 // [32 tok][256 B] v, chunks XOR-swizzled by the token index (from P5 on)
constexpr int kSmKPP = kRecBytes;            // [32][128] k+ from chunk start (rows 0-15 double as sub-block operand)
constexpr int kSmKR0 = kSmKPP + 8192;        // [16][128] k of sub-block 0 decayed to the sub-block end (dead after P4)
constexpr int kSmTB = kSmKR0;                // [32][32] bf16 T diag(beta)                       (from P5 on)
constexpr int kSmA = kSmKR0 + 4096;          // [32][36] fp32 A
constexpr int kSmTot = kSmA + 32 * kLd * 4;  // [2][128] fp32 sub-block log2 decays
constexpr int kSmSsq = kSmTot + 1024;        // [2][32][4] fp32 partial sums of squares
constexpr int kSmBeta = kSmSsq + 1024;       // [32] fp32 sigmoid(beta)
constexpr int kPrepSmemBytes = kSmBeta + 128;
static_assert(kPrepSmemBytes * 4 + 4 * 1024 <= 227 * 1024, "four CTAs per SM");


// 16x16x128 product of two core-layout operands (rows of A times rows of B), fp32 accumulators
// in the mma.sync C layout: acc[nt][0..1] -> (row lane/4, col 8nt + 2(lane%4) + {0,1}), acc[nt][2..3] -> row + 8.
__device__ __forceinline__ void block16_product(uint32_t a_base, uint32_t b_base, int lane, float (&acc)[2][4]) {
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
  const int mi = lane >> 3, r = lane & 7;
  const uint32_t a_lane = a_base + (mi & 1) * 2048 + (mi >> 1) * 128 + r * 16;
  const uint32_t b_lane = b_base + (mi >> 1) * 2048 + (mi & 1) * 128 + r * 16;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
    ldsm_x4(a_lane + ks * 256, a0, a1, a2, a3);
    ldsm_x4(b_lane + ks * 256, b0, b1, b2, b3);
    mma_bf16_16816(acc[0], a0, a1, a2, a3, b0, b1);
    mma_bf16_16816(acc[1], a0, a1, a2, a3, b2, b3);
  }
}

// kShortPath: compiled with the shortcuts for chunks of at most 16 valid tokens (launched when such chunks are a
// large share of the call: short fixed-length sequences); without it the kernel has no trace of them.
template <bool kShortPath>
__global__ void __launch_bounds__(256, 4) prepare_kernel(const PrepParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef FKDA_TUNING
  const int dbg = p.dbg;       // phase-skip timing (results are wrong when set): only in builds made for tuning
#else
  constexpr int dbg = 0;
#endif
  // consecutive CTAs take consecutive heads of the same chunk: together they read whole [H x 256 B] token rows,
  // which keeps concurrent DRAM accesses inside the same pages
  const int h = static_cast<int>(blockIdx.x % static_cast<unsigned>(p.H));
  const int gc = static_cast<int>(blockIdx.x / static_cast<unsigned>(p.H));

  // ---- chunk -> (sequence, first token, valid length) -------------------------------------------
  int64_t t0;
  int len;
  if (p.cu_seqlens != nullptr) {
    if (gc >= p.chunk_prefix[p.N]) return;
    int lo = 0, hi = p.N - 1;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (p.chunk_prefix[mid] <= gc) lo = mid; else hi = mid - 1;
    }
    int64_t bos = p.cu_seqlens[lo], eos = p.cu_seqlens[lo + 1];
    bos = bos < 0 ? 0 : (bos > p.T_total ? p.T_total : bos);
    eos = eos < bos ? bos : (eos > p.T_total ? p.T_total : eos);
    t0 = bos + static_cast<int64_t>(gc - p.chunk_prefix[lo]) * kChunk;
    int64_t rem = eos - t0;
    len = rem < kChunk ? static_cast<int>(rem) : kChunk;
  } else {
    const int cps = static_cast<int>((p.T + kChunk - 1) / kChunk);
    const int n = gc / cps, lc = gc - n * cps;
    t0 = static_cast<int64_t>(n) * p.T + static_cast<int64_t>(lc) * kChunk;
    int64_t rem = p.T - static_cast<int64_t>(lc) * kChunk;
    len = rem < kChunk ? static_cast<int>(rem) : kChunk;
  }

  // ---- thread -> two (row, 8-column) items of one sub-block ------------------------------------------
  const int r8 = tid & 7;
  const int cm = tid >> 3;
  const int j = cm & 15;        // 8-column group: channels 8j .. 8j+7
  const int sb = cm >> 4;       // sub-block (tokens 16sb .. 16sb+15); warps 0-3 -> 0, warps 4-7 -> 1
  const int row0 = sb * 16 + r8, row1 = row0 + 8;
  // A chunk with at most 16 valid tokens (the last chunk of a sequence, or a whole short sequence) has an all-zero
  // second sub-block: its warps skip the transcendental work and every product that involves it is known to be zero.
  const bool short_chunk = kShortPath && len <= 16;
  const bool sb_live = sb == 0 || !short_chunk;     // uniform per warp

  float* s_tot = reinterpret_cast<float*>(smem + kSmTot);
  float* s_ssq = reinterpret_cast<float*>(smem + kSmSsq);
  float* s_beta = reinterpret_cast<float*>(smem + kSmBeta);
  float* s_A = reinterpret_cast<float*>(smem + kSmA);
  float* s_T = reinterpret_cast<float*>(smem + kSmT);
  float* s_X = reinterpret_cast<float*>(smem + kSmX);
  const uint32_t sbase = smem_u32(smem);
  uint8_t* const rec_dst = p.records + (static_cast<size_t>(h) * p.total_chunks + gc) * kRecBytes;

  // ---- P1: loads, partial sums of squares, v tile, beta, gate and its in-sub-block running sum ------
  uint4 qw[2], kw[2];
  float G[2][8];      // log2 cumulative decay relative to the sub-block start
  {
    // coalesced asynchronous loads: 16 consecutive lanes fetch one 256-byte token row of one tensor
    {
      const int lrow = tid >> 4, lchunk = tid & 15;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = lrow + 16 * hf;
        const bool valid = (row < len) && !(dbg & 64);
        const size_t off = (static_cast<size_t>(t0 + (valid ? row : 0)) * p.H + h) * kD + 8 * lchunk;
        const uint32_t nbytes = valid ? 16u : 0u;
        const uint32_t dst = sbase + stage_off(row, lchunk);
        cp_async16(dst + kSmStageQKG, p.q + off, nbytes);
        cp_async16(dst + kSmStageQKG + 8192, p.k + off, nbytes);
        cp_async16(dst + kSmStageQKG + 16384, p.g + off, nbytes);
      }
    }
    if (tid < kChunk) {
      float b = 0.f;
      if (tid < len) b = sigmoid_fast(__bfloat162float(p.beta[static_cast<size_t>(t0 + tid) * p.H + h]));
      s_beta[tid] = b;
    }
    // gate: gamma = gate_scale * sigmoid(a (g + bias)) = hgs * tanh(ha g + ha bias) + hgs
    const float ha = 0.5f * ex2f(__ldg(p.A_log + h) * kLog2e);
    const float hgs = 0.5f * p.gate_scale;
    float hab[8];
    {
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * j));
      const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * j + 4));
      hab[0] = ha * b0.x; hab[1] = ha * b0.y; hab[2] = ha * b0.z; hab[3] = ha * b0.w;
      hab[4] = ha * b1.x; hab[5] = ha * b1.y; hab[6] = ha * b1.z; hab[7] = ha * b1.w;
    }
    cp_async_wait_all();
    __syncthreads();
    uint4 gw[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = hf ? row1 : row0;
      qw[hf] = *reinterpret_cast<const uint4*>(smem + kSmStageQKG + stage_off(row, j));
      kw[hf] = *reinterpret_cast<const uint4*>(smem + kSmStageQKG + 8192 + stage_off(row, j));
      gw[hf] = *reinterpret_cast<const uint4*>(smem + kSmStageQKG + 16384 + stage_off(row, j));
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = hf ? row1 : row0;
      float f[8], sq = 0.f, sk = 0.f;
      unpack8(qw[hf], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) sq = fmaf(f[i], f[i], sq);
      unpack8(kw[hf], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) sk = fmaf(f[i], f[i], sk);
      // lanes sharing r8 inside the warp hold 4 different column groups of the same row
      sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sk += __shfl_xor_sync(0xffffffffu, sk, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 16);
      sk += __shfl_xor_sync(0xffffffffu, sk, 16);
      if (lane < 8) {
        s_ssq[(0 * kChunk + row) * 4 + (warp & 3)] = sq;
        s_ssq[(1 * kChunk + row) * 4 + (warp & 3)] = sk;
      }
      unpack8(gw[hf], f);
      const bool valid = row < len;
      if (!sb_live) {
#pragma unroll
        for (int i = 0; i < 8; ++i) G[hf][i] = 0.f;
        continue;
      }
      if (dbg & 32) {
#pragma unroll
        for (int i = 0; i < 8; ++i) G[hf][i] = f[i];
        continue;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float x = valid ? fmaf(tanh_approx(fmaf(f[i], ha, hab[i])), hgs, hgs) : 0.f;
        // inclusive scan over the 8 rows held by the 8 lanes of this group
#pragma unroll
        for (int d = 1; d < 8; d <<= 1) {
          const float y = __shfl_up_sync(0xffffffffu, x, d, 8);
          if (r8 >= d) x += y;
        }
        G[hf][i] = x;
      }
    }
  }
  float tot[8];       // log2 decay of this thread's whole sub-block
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float first_half = __shfl_sync(0xffffffffu, G[0][i], 7, 8);
    G[1][i] += first_half;
    tot[i] = __shfl_sync(0xffffffffu, G[1][i], 7, 8);
  }
  if (r8 == 0) {
    *reinterpret_cast<float4*>(s_tot + sb * kD + 8 * j) = make_float4(tot[0], tot[1], tot[2], tot[3]);
    *reinterpret_cast<float4*>(s_tot + sb * kD + 8 * j + 4) = make_float4(tot[4], tot[5], tot[6], tot[7]);
  }
  __syncthreads();

  if (dbg & 16) goto store_record;
  // ---- P2: norms and every decayed operand ------------------------------------------------------------
  if (!sb_live) {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = hf ? row1 : row0, lrow = row - 16;
      *reinterpret_cast<uint4*>(smem + kSmKM + core_off(row, 8 * j, kD)) = z;
      *reinterpret_cast<uint4*>(smem + kSmKP1 + core_off(lrow, 8 * j, kD)) = z;
      *reinterpret_cast<uint4*>(smem + kSmQP1 + core_off(lrow, 8 * j, kD)) = z;
      *reinterpret_cast<uint4*>(smem + kRecKR + core_off(row, 8 * j, kD)) = z;
      *reinterpret_cast<uint4*>(smem + kSmKPP + core_off(row, 8 * j, kD)) = z;
      *reinterpret_cast<uint4*>(smem + kRecQP + core_off(row, 8 * j, kD)) = z;
    }
  } else {
    // per-channel factors: fa = 2^(own sub-block total), fb = 2^(other sub-block total)
    __nv_bfloat162 fa2[4], fb2[4], fab2[4];
    {
      float fa[8], fb[8], fab[8];
      const float4 t0v = *reinterpret_cast<const float4*>(s_tot + (1 - sb) * kD + 8 * j);
      const float4 t1v = *reinterpret_cast<const float4*>(s_tot + (1 - sb) * kD + 8 * j + 4);
      const float to[8] = {t0v.x, t0v.y, t0v.z, t0v.w, t1v.x, t1v.y, t1v.z, t1v.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        fa[i] = ex2f(tot[i]);
        fb[i] = ex2f(to[i]);
        fab[i] = fa[i] * fb[i];
      }
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        fa2[m] = __floats2bfloat162_rn(fa[2 * m], fa[2 * m + 1]);
        fb2[m] = __floats2bfloat162_rn(fb[2 * m], fb[2 * m + 1]);
        fab2[m] = __floats2bfloat162_rn(fab[2 * m], fab[2 * m + 1]);
      }
      if (sb == 0 && r8 == 0) {
        float* e = reinterpret_cast<float*>(smem + kRecE) + 8 * j;
        *reinterpret_cast<float4*>(e) = make_float4(ex2f(tot[0] + to[0]), ex2f(tot[1] + to[1]), ex2f(tot[2] + to[2]), ex2f(tot[3] + to[3]));
        *reinterpret_cast<float4*>(e + 4) = make_float4(ex2f(tot[4] + to[4]), ex2f(tot[5] + to[5]), ex2f(tot[6] + to[6]), ex2f(tot[7] + to[7]));
      }
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = hf ? row1 : row0;      // chunk row
      const int lrow = row - sb * 16;        // row inside the sub-block
      const float4 sq4 = *reinterpret_cast<const float4*>(s_ssq + (0 * kChunk + row) * 4);
      const float4 sk4 = *reinterpret_cast<const float4*>(s_ssq + (1 * kChunk + row) * 4);
      const float rq = rsqrtf(sq4.x + sq4.y + sq4.z + sq4.w + 1e-6f) * p.scale;
      const float rk = rsqrtf(sk4.x + sk4.y + sk4.z + sk4.w + 1e-6f);
      // The row norm is folded into the decay factor in fp32 (rk 2^G etc.), rounded to bf16 once, and applied to the raw
      // bf16 inputs with packed bf16x2 multiplies: no unpacking of q/k, half the multiply and conversion count.
      const uint32_t qraw[4] = {qw[hf].x, qw[hf].y, qw[hf].z, qw[hf].w};
      const uint32_t kraw[4] = {kw[hf].x, kw[hf].y, kw[hf].z, kw[hf].w};
      __nv_bfloat162 kp[4], qp[4], km[4], t[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float pw0 = ex2f(G[hf][2 * m]), pw1 = ex2f(G[hf][2 * m + 1]);
        const float ip0 = ex2f(-G[hf][2 * m]), ip1 = ex2f(-G[hf][2 * m + 1]);
        const __nv_bfloat162 k2 = *reinterpret_cast<const __nv_bfloat162*>(&kraw[m]);
        const __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162*>(&qraw[m]);
        kp[m] = __hmul2(k2, __floats2bfloat162_rn(rk * pw0, rk * pw1));   // decayed from the sub-block start (<= |khat|)
        qp[m] = __hmul2(q2, __floats2bfloat162_rn(rq * pw0, rq * pw1));
        km[m] = __hmul2(k2, __floats2bfloat162_rn(rk * ip0, rk * ip1));   // inverse decay, up to 2^115 for lower_bound = -5
      }
      auto as_u4 = [](const __nv_bfloat162 (&x)[4]) {
        return make_uint4(*reinterpret_cast<const uint32_t*>(&x[0]), *reinterpret_cast<const uint32_t*>(&x[1]),
                          *reinterpret_cast<const uint32_t*>(&x[2]), *reinterpret_cast<const uint32_t*>(&x[3]));
      };
      *reinterpret_cast<uint4*>(smem + kSmKM + core_off(row, 8 * j, kD)) = as_u4(km);
      if (sb == 0) {
        *reinterpret_cast<uint4*>(smem + kSmKPP + core_off(row, 8 * j, kD)) = as_u4(kp);
        *reinterpret_cast<uint4*>(smem + kRecQP + core_off(row, 8 * j, kD)) = as_u4(qp);
#pragma unroll
        for (int m = 0; m < 4; ++m) t[m] = __hmul2(km[m], fa2[m]);      // decayed to the sub-block end
        *reinterpret_cast<uint4*>(smem + kSmKR0 + core_off(lrow, 8 * j, kD)) = as_u4(t);
#pragma unroll
        for (int m = 0; m < 4; ++m) t[m] = __hmul2(km[m], fab2[m]);     // ... and on through sub-block 1
        *reinterpret_cast<uint4*>(smem + kRecKR + core_off(row, 8 * j, kD)) = as_u4(t);
      } else {
        *reinterpret_cast<uint4*>(smem + kSmKP1 + core_off(lrow, 8 * j, kD)) = as_u4(kp);
        *reinterpret_cast<uint4*>(smem + kSmQP1 + core_off(lrow, 8 * j, kD)) = as_u4(qp);
#pragma unroll
        for (int m = 0; m < 4; ++m) t[m] = __hmul2(km[m], fa2[m]);      // decayed to the chunk end
        *reinterpret_cast<uint4*>(smem + kRecKR + core_off(row, 8 * j, kD)) = as_u4(t);
#pragma unroll
        for (int m = 0; m < 4; ++m) t[m] = __hmul2(kp[m], fb2[m]);      // decayed from the chunk start
        *reinterpret_cast<uint4*>(smem + kSmKPP + core_off(row, 8 * j, kD)) = as_u4(t);
#pragma unroll
        for (int m = 0; m < 4; ++m) t[m] = __hmul2(qp[m], fb2[m]);
        *reinterpret_cast<uint4*>(smem + kRecQP + core_off(row, 8 * j, kD)) = as_u4(t);
      }
    }
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0 && !(dbg & 8)) {
    // the parts of the record that are final after P2 leave now and overlap with the remaining phases
    bulk_s2g(rec_dst + kRecKR, sbase + kRecKR, 8192);
    bulk_s2g(rec_dst + kRecE, sbase + kRecE, 512);
    bulk_s2g(rec_dst + kRecQP, sbase + kRecQP, 8192);
    bulk_commit();
  }

  if (dbg & 1) goto store_record;
  // ---- P4: the six 16x16x128 intra-chunk products (one warp each) --------------------------------------
  if (warp < 6) {
    const int which = warp % 3;            // 0: (0,0) block, 1: (1,1) block, 2: (1,0) block
    const bool is_m = warp >= 3;           // q-side (M) instead of k-side (A)
    uint32_t a_base, b_base;
    if (which == 0) {
      a_base = sbase + (is_m ? kRecQP : kSmKPP);
      b_base = sbase + kSmKM;
    } else {
      a_base = sbase + (is_m ? kSmQP1 : kSmKP1);
      b_base = sbase + (which == 1 ? kSmKM + 4096 : kSmKR0);
    }
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (which == 0 || !short_chunk) block16_product(a_base, b_base, lane, acc);
    const int rbase = (which == 0) ? 0 : 16, cbase = (which == 1) ? 16 : 0;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int lr = (lane >> 2) + half * 8, lc = nt * 8 + (lane & 3) * 2;
        const int r = rbase + lr, c = cbase + lc;
        float x0 = acc[nt][half * 2], x1 = acc[nt][half * 2 + 1];
        if (!is_m) {
          const float br = s_beta[r];
          if (which != 2) {               // strictly lower triangle of a diagonal block
            x0 = (lc < lr) ? x0 * br : 0.f;
            x1 = (lc + 1 < lr) ? x1 * br : 0.f;
          } else {
            x0 *= br;
            x1 *= br;
          }
          *reinterpret_cast<float2*>(s_A + r * kLd + c) = make_float2(x0, x1);
        } else {
          if (which != 2) {               // lower triangle including the diagonal
            x0 = (lc <= lr) ? x0 : 0.f;
            x1 = (lc + 1 <= lr) ? x1 : 0.f;
          }
          *reinterpret_cast<uint32_t*>(smem + kRecMQK + core_off(r, c, kChunk)) = pack_bf16(x0, x1);
        }
      }
  } else if (warp == 6) {
    // upper-right quadrant of M (rows 0-15, cols 16-31) is zero: two 8-row groups x two column blocks
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = lane + 32 * i;       // 128 uint32 = 512 B: blocks (rg 0..1, cb 2..3), 128 B each
      const int blk = idx >> 5, w = idx & 31;
      const int rg = blk >> 1, cb = 2 + (blk & 1);
      *reinterpret_cast<uint32_t*>(smem + kRecMQK + rg * 512 + cb * 128 + w * 4) = 0u;
    }
  }
  if (tid == 0) bulk_wait_read0();      // the early copy has read KR, E, QP: their regions may be reused
  __syncthreads();
  {
    // v tile -> the QP region (same coalesced, swizzled staging as q, k, g); needed by P6 only, arrives during P5
    const int lrow = tid >> 4, lchunk = tid & 15;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = lrow + 16 * hf;
      const bool valid = (row < len) && !(dbg & 64);
      const size_t off = (static_cast<size_t>(t0 + (valid ? row : 0)) * p.H + h) * kD + 8 * lchunk;
      cp_async16(sbase + kSmV + stage_off(row, lchunk), p.v + off, valid ? 16u : 0u);
    }
  }

  if (dbg & 2) goto after_p5;
  // ---- P5: T = (I + A)^-1 and TB = T diag(beta), all inside warp 0 (no block-wide barriers) -------------------
  if (warp == 0) {
    if (!(dbg & 512)) {
      // forward substitution, one column of one diagonal block per lane: x_i = [i==c] - sum_{j<i} A_ij x_j.
      // Rows of A are read four entries at a time; entries on and above the diagonal are zero.
      const int b = lane >> 4, c = lane & 15;
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) x[i] = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = (i == c) ? 1.f : 0.f;
#pragma unroll
        for (int q4 = 0; 4 * q4 < i; ++q4) {
          const float4 a4 = *reinterpret_cast<const float4*>(s_A + (b * 16 + i) * kLd + b * 16 + 4 * q4);
          acc = fmaf(-a4.x, x[4 * q4], acc);
          acc = fmaf(-a4.y, x[4 * q4 + 1], acc);
          acc = fmaf(-a4.z, x[4 * q4 + 2], acc);
          acc = fmaf(-a4.w, x[4 * q4 + 3], acc);
        }
        x[i] = acc;
        s_T[(b * 16 + i) * kLd + b * 16 + c] = acc;
      }
    }
    __syncwarp();
    const int g = lane >> 2, t4 = lane & 3;
    if (short_chunk) {                 // A_10 = 0: T_10 = 0
      const int i = lane >> 1, c8 = (lane & 1) * 8;
      *reinterpret_cast<float4*>(s_T + (16 + i) * kLd + c8) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(s_T + (16 + i) * kLd + c8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // T_10 = -T_11 (A_10 T_00): two 16x16x16 products on the tensor cores in tf32 (11-bit significands, finer than
    // the bf16 the result is rounded to), fp32 accumulation
    auto small_product = [&](const float* A, const float* B, float* D, float sign) {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const int k0 = 8 * ks;
        const uint32_t a0 = to_tf32(A[g * kLd + k0 + t4]), a1 = to_tf32(A[(g + 8) * kLd + k0 + t4]);
        const uint32_t a2 = to_tf32(A[g * kLd + k0 + t4 + 4]), a3 = to_tf32(A[(g + 8) * kLd + k0 + t4 + 4]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
          mma_tf32_1688(acc[nt], a0, a1, a2, a3, to_tf32(B[(k0 + t4) * kLd + 8 * nt + g]), to_tf32(B[(k0 + t4 + 4) * kLd + 8 * nt + g]));
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        *reinterpret_cast<float2*>(D + g * kLd + 8 * nt + 2 * t4) = make_float2(sign * acc[nt][0], sign * acc[nt][1]);
        *reinterpret_cast<float2*>(D + (g + 8) * kLd + 8 * nt + 2 * t4) = make_float2(sign * acc[nt][2], sign * acc[nt][3]);
      }
    };
    if (!(dbg & 256) && !short_chunk) {
      small_product(s_A + 16 * kLd, s_T, s_X, 1.f);                       // X = A_10 T_00
      __syncwarp();
      small_product(s_T + 16 * kLd + 16, s_X, s_T + 16 * kLd, -1.f);      // T_10 = -T_11 X
    }
    __syncwarp();
    {
      // TB = T diag(beta) as a bf16 core-layout operand; lane = row, four entries per shared-memory load
      const int r = lane;
      uint8_t* row = smem + kSmTB + (r >> 3) * 512 + (r & 7) * 16;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {          // 8 columns per 16-byte store
        const float4 ta = *reinterpret_cast<const float4*>(s_T + r * kLd + q4 * 8);
        const float4 tb = *reinterpret_cast<const float4*>(s_T + r * kLd + q4 * 8 + 4);
        const float4 ba = *reinterpret_cast<const float4*>(s_beta + q4 * 8);
        const float4 bb = *reinterpret_cast<const float4*>(s_beta + q4 * 8 + 4);
        const float tv[8] = {ta.x, ta.y, ta.z, ta.w, tb.x, tb.y, tb.z, tb.w};
        const float bv[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
        float t[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int c = q4 * 8 + e;
          const bool nz = (c <= r) && !(r < 16 && c >= 16);
          t[e] = nz ? tv[e] * bv[e] : 0.f;
        }
        *reinterpret_cast<uint4*>(row + q4 * 128) = pack8(t);
      }
    }
  }
after_p5:
  cp_async_wait_all();
  __syncthreads();

  if (dbg & 4) goto store_record;
  // ---- P6: w' = TB k+ (warps 0-3, 32 k-columns each) ; u'^T = v^T TB^T (warps 4-7, 32 v-rows each) -----
  {
    const int mi = lane >> 3, r = lane & 7;
    float acc[2][4][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
    if (warp < 4) {
      const int nb = warp * 4;             // first 8-column tile of this warp
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        if (ks == 1 && short_chunk) break;       // k+ rows 16-31 are zero
        uint32_t a[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
          ldsm_x4(sbase + kSmTB + (2 * mt + (mi & 1)) * 512 + (2 * ks + (mi >> 1)) * 128 + r * 16, a[mt][0], a[mt][1], a[mt][2],
                  a[mt][3]);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          // transposed loads: matrices (token group 2ks + (mi&1), column tile nb + 2np + (mi>>1))
          uint32_t b0, b1, b2, b3;
          ldsm_x4_trans(sbase + kSmKPP + (2 * ks + (mi & 1)) * 2048 + (nb + 2 * np + (mi >> 1)) * 128 + r * 16, b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma_bf16_16816(acc[mt][2 * np], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
            mma_bf16_16816(acc[mt][2 * np + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
          }
        }
      }
      // fragments -> core matrices of WP [32 tok][128 k]
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int np = 0; np < 2; ++np)
          stsm_x4(sbase + kRecWP + (2 * mt + (mi & 1)) * 2048 + (nb + 2 * np + (mi >> 1)) * 128 + r * 16,
                  pack_bf16(acc[mt][2 * np][0], acc[mt][2 * np][1]), pack_bf16(acc[mt][2 * np][2], acc[mt][2 * np][3]),
                  pack_bf16(acc[mt][2 * np + 1][0], acc[mt][2 * np + 1][1]), pack_bf16(acc[mt][2 * np + 1][2], acc[mt][2 * np + 1][3]));
    } else {
      const int vc0 = (warp & 3) * 4;      // first 8-wide v tile of this warp's 32 rows
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        if (ks == 1 && short_chunk) break;       // v rows 16-31 are zero
        uint32_t a[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)     // A = v^T: transposed loads of (token group 2ks + (mi>>1), v tile vc0 + 2mt + (mi&1))
          ldsm_x4_trans(sbase + kSmV + stage_off((2 * ks + (mi >> 1)) * 8 + r, vc0 + 2 * mt + (mi & 1)), a[mt][0], a[mt][1],
                        a[mt][2], a[mt][3]);
#pragma unroll
        for (int np = 0; np < 2; ++np) {   // B = TB^T: plain loads of (token group 2np + (mi>>1), k tile 2ks + (mi&1))
          uint32_t b0, b1, b2, b3;
          ldsm_x4(sbase + kSmTB + (2 * np + (mi >> 1)) * 512 + (2 * ks + (mi & 1)) * 128 + r * 16, b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma_bf16_16816(acc[mt][2 * np], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
            mma_bf16_16816(acc[mt][2 * np + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
          }
        }
      }
      // fragments -> core matrices of UP [128 v][32 tok]
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int np = 0; np < 2; ++np)
          stsm_x4(sbase + kRecUP + (vc0 + 2 * mt + (mi & 1)) * 512 + (2 * np + (mi >> 1)) * 128 + r * 16,
                  pack_bf16(acc[mt][2 * np][0], acc[mt][2 * np][1]), pack_bf16(acc[mt][2 * np][2], acc[mt][2 * np][3]),
                  pack_bf16(acc[mt][2 * np + 1][0], acc[mt][2 * np + 1][1]), pack_bf16(acc[mt][2 * np + 1][2], acc[mt][2 * np + 1][3]));
    }
  }
store_record:
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0 && !(dbg & 8)) {
    bulk_s2g(rec_dst + kRecMQK, sbase + kRecMQK, 2048);
    bulk_s2g(rec_dst + kRecWP, sbase + kRecWP, 8192);
    bulk_s2g(rec_dst + kRecUP, sbase + kRecUP, 8192);
    bulk_commit();
    bulk_wait_read0();
  }
}

cudaError_t launch_chunk_prefix(const int64_t* cu, int N, int64_t T_total, int H, int n_segs, int* prefix, int* status,
                                cudaStream_t stream) {
  chunk_prefix_kernel<<<1, N > 256 ? 1024 : 256, 0, stream>>>(cu, N, T_total, H, n_segs, device_sm_count(), prefix, status);
  return cudaGetLastError();
}

cudaError_t launch_prepare(const PrepParams& p, cudaStream_t stream) {
  if (p.total_chunks == 0 || p.H == 0) return cudaSuccess;
  // fixed-length sequences whose last chunk holds at most 16 tokens, and that chunk is at least a quarter of them
  const int64_t tail = p.T % kChunk;
  const bool short_path = p.cu_seqlens == nullptr && tail >= 1 && tail <= 16 && p.T < 4 * kChunk;
  auto kernel = short_path ? prepare_kernel<true> : prepare_kernel<false>;
  static SmemOptIn opt_in[2];
  cudaError_t e = opt_in[short_path ? 1 : 0].ensure(kernel, kPrepSmemBytes);
  if (e != cudaSuccess) return e;
  const unsigned grid = static_cast<unsigned>(p.total_chunks) * static_cast<unsigned>(p.H);
  kernel<<<grid, 256, kPrepSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fkda
