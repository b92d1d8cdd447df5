// Fused forward pass for batches of short fixed-length sequences: one CTA per (sequence, head) chain walks the
// sequence in blocks of 16 tokens,
// reads q, k, v, g, beta and the chain's state, and writes out and the new state - no operand record goes through
// global memory, and between blocks the state stays in shared memory in fp32.  This is the shape of a continuation / decode step after a prefill: per chain 16 KB of inputs
// against 128 KB of fp32 state in and out, so the kernel is a stream over the states.
//
// Replaces, for these shapes, both of the reference's kernels (csrc/smxx/fwd_kernel1.cuh:107-586 and
// fwd_kernel2.cuh:115-839), whose K2 spends most of its time loading and converting states here.  The algebra is
// the single sub-block case of the chunked form used by the other kernels:
//     k+ = khat 2^G, q+ = scale qhat 2^G, k- = khat 2^-G, kr = k- 2^Gtot, e = 2^Gtot        (G: running log2 decay)
//     A = tril(k+ k-^T, -1) diag_rows(beta),  M = tril(q+ k-^T),  T = (I + A)^-1,  w' = T diag(beta) k+,  u' = T diag(beta) v
//     U = u' - w' S,   O = q+ S + M U,   S' = diag(e) S + kr^T U                              (S: [k][v], stored [v][k])
// Every warp owns 16 rows v of the state as fp32 mma.sync accumulator fragments: the same registers, rounded to
// bf16, are the B fragments of w' S and q+ S, and after scaling by e they are the accumulator of the update.  The
// state rows travel as whole-row bulk copies (fully coalesced) through a padded staging buffer in shared memory:
// the copy in is issued before anything else and lands while the operands are being formed; the copy out is issued
// per warp as soon as its 16 rows are done.
#include "fkda_common.cuh"

namespace fkda {
namespace short16 {

constexpr int kRows = 16;
constexpr int kThreads = 256;
constexpr int kLdS = 20;                         // row stride (floats) of the 16x16 fp32 matrices
// shared memory (byte offsets)
constexpr int kStQ = 0;                          // staged q, k, g, v: [16 tok][256 B], 16-byte chunks XOR-swizzled by the row
constexpr int kStK = kStQ + 4096;
constexpr int kStG = kStK + 4096;
constexpr int kStV = kStG + 4096;
constexpr int kKP = kStV + 4096;                 // bf16 [16][128] tiles in the 8x8 core-matrix layout
constexpr int kQP = kKP + 4096;
constexpr int kKM = kQP + 4096;
constexpr int kKR = kKM + 4096;
constexpr int kWP = kKR + 4096;
constexpr int kTB = kWP + 4096;                  // bf16 [16][16] T diag(beta), core layout
constexpr int kMQK = kTB + 512;                  // bf16 [16][16]
constexpr int kA = kMQK + 512;                   // fp32 [16][20]
constexpr int kT = kA + kRows * kLdS * 4;        // fp32 [16][20]
constexpr int kE = kT + kRows * kLdS * 4;        // fp32 [128] decay of the whole block
constexpr int kTot = kE + 512;                   // fp32 [2][128] log2 decay of rows 0-7 and of rows 8-15
constexpr int kSsq = kTot + 1024;                // fp32 [2][16][4] partial sums of squares (q, k)
constexpr int kBeta = kSsq + 512;                // fp32 [16]
constexpr int kBar = kBeta + 64;                 // mbarrier of the state copy, abort flag
constexpr int kState = (kBar + 16 + 127) / 128 * 128;   // [128 v] state rows, padded: fragment reads hit 32 distinct banks
constexpr int kStride32 = 512 + 32;              // fp32 rows: stride = 8 words mod 32 (8-byte reads by half-warps)
constexpr int kStride16 = 256 + 16;              // bf16 rows: stride = 4 words mod 32 (4-byte reads)
constexpr int kSmemBytes = kState + kD * kStride32;
static_assert(2 * (kSmemBytes + 1024) <= 227 * 1024, "two CTAs per SM");

__device__ __forceinline__ uint4 as_u4(const __nv_bfloat162 (&x)[4]) {
  return make_uint4(*reinterpret_cast<const uint32_t*>(&x[0]), *reinterpret_cast<const uint32_t*>(&x[1]),
                    *reinterpret_cast<const uint32_t*>(&x[2]), *reinterpret_cast<const uint32_t*>(&x[3]));
}

struct Params {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* g;
  const __nv_bfloat16* beta;
  const float* A_log;
  const float* dt_bias;
  const void* initial_state;
  void* final_state;
  __nv_bfloat16* out;
  int T;                 // tokens per sequence
  int H;
  int state_fp32;
  float scale;
  float gate_scale;      // lower_bound * log2(e)
  int* status;           // device status word (a bounded wait that gives up is recorded there)
};

// kOneBlock: T <= 16, compiled without the block loop's bookkeeping
template <bool kOneBlock>
__global__ void __launch_bounds__(kThreads, 2) short16_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chain = blockIdx.x;
  const int n = chain / p.H, h = chain - n * p.H;       // consecutive CTAs: consecutive heads of the same tokens
  const int64_t t_seq0 = static_cast<int64_t>(n) * p.T;
  const int nblk = kOneBlock ? 1 : (p.T + kRows - 1) / kRows;

  float* s_A = reinterpret_cast<float*>(smem + kA);
  float* s_T = reinterpret_cast<float*>(smem + kT);
  float* s_e = reinterpret_cast<float*>(smem + kE);
  float* s_tot = reinterpret_cast<float*>(smem + kTot);
  float* s_ssq = reinterpret_cast<float*>(smem + kSsq);
  float* s_beta = reinterpret_cast<float*>(smem + kBeta);

  // ---- the state: one bulk copy per row into the padded staging buffer, issued before anything else --------------
  const uint32_t bar = sbase + kBar;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kBar + 8);
  const int row_bytes = p.state_fp32 ? 512 : 256;
  const int in_off = p.state_fp32 ? 0 : kStride16;     // bf16 rows arrive in the second half of their fp32 slot
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar, kD);
    fence_mbar_init();
  }
  __syncthreads();
  if (p.initial_state != nullptr && tid < kD) {
    mbar_arrive_expect_tx(bar, row_bytes);
    bulk_g2s(sbase + kState + tid * kStride32 + in_off,
             static_cast<const uint8_t*>(p.initial_state) + (static_cast<size_t>(chain) * kD + tid) * row_bytes, row_bytes, bar);
  }
  // ---- inputs: coalesced asynchronous loads, 16 lanes per 256-byte token row; q, k, g and v of the next block are
  // requested as soon as the staging of the current block has been consumed
  auto load_qkg = [&](int blk) {
    const int lrow = tid >> 4, chunk = tid & 15;
    const bool valid = kRows * blk + lrow < p.T;
    const size_t off = (static_cast<size_t>(t_seq0 + (valid ? kRows * blk + lrow : 0)) * p.H + h) * kD + 8 * chunk;
    const uint32_t nbytes = valid ? 16u : 0u;
    const uint32_t dst = sbase + stage_off(lrow, chunk);
    cp_async16(dst + kStQ, p.q + off, nbytes);
    cp_async16(dst + kStK, p.k + off, nbytes);
    cp_async16(dst + kStG, p.g + off, nbytes);
  };
  auto load_v = [&](int blk) {
    const int lrow = tid >> 4, chunk = tid & 15;
    const bool valid = kRows * blk + lrow < p.T;
    const size_t off = (static_cast<size_t>(t_seq0 + (valid ? kRows * blk + lrow : 0)) * p.H + h) * kD + 8 * chunk;
    cp_async16(sbase + kStV + stage_off(lrow, chunk), p.v + off, valid ? 16u : 0u);
  };
  load_qkg(0);
  load_v(0);
  // thread -> one (row, 8-column) item: rows 0-7 in warps 0-3, rows 8-15 in warps 4-7
  const int r8 = tid & 7;
  const int j = (tid >> 3) & 15;
  const int half = tid >> 7;
  const int row = r8 + 8 * half;
  const float ha = 0.5f * ex2f(__ldg(p.A_log + h) * kLog2e);
  const float hgs = 0.5f * p.gate_scale;
  float hab[8];
  {
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * j));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * j + 4));
    hab[0] = ha * b0.x; hab[1] = ha * b0.y; hab[2] = ha * b0.z; hab[3] = ha * b0.w;
    hab[4] = ha * b1.x; hab[5] = ha * b1.y; hab[6] = ha * b1.z; hab[7] = ha * b1.w;
  }
  const int g = lane >> 2, t4 = lane & 3;
  const int mi = lane >> 3, r = lane & 7;
  const int v0 = 16 * warp + g;
  uint8_t* const srow = smem + kState + v0 * kStride32;
  bool failed = false;

  for (int blk = 0; blk < nblk; ++blk) {
  const int64_t t0 = t_seq0 + kRows * blk;
  const int len = p.T - kRows * blk < kRows ? p.T - kRows * blk : kRows;
  if (tid < kRows) {
    float b = 0.f;
    if (tid < len) b = sigmoid_fast(__bfloat162float(p.beta[static_cast<size_t>(t0 + tid) * p.H + h]));
    s_beta[tid] = b;
  }
  cp_async_wait_all();
  __syncthreads();
  if (*abort_flag) { failed = true; break; }

  // ---- norms, gate, running decay ---------------------------------------------------------------------------------
  const uint4 qw = *reinterpret_cast<const uint4*>(smem + kStQ + stage_off(row, j));
  const uint4 kw = *reinterpret_cast<const uint4*>(smem + kStK + stage_off(row, j));
  float G[8];
  {
    float f[8], sq = 0.f, sk = 0.f;
    unpack8(qw, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) sq = fmaf(f[i], f[i], sq);
    unpack8(kw, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) sk = fmaf(f[i], f[i], sk);
    sq += __shfl_xor_sync(0xffffffffu, sq, 8);
    sk += __shfl_xor_sync(0xffffffffu, sk, 8);
    sq += __shfl_xor_sync(0xffffffffu, sq, 16);
    sk += __shfl_xor_sync(0xffffffffu, sk, 16);
    if (lane < 8) {
      s_ssq[(0 * kRows + row) * 4 + (warp & 3)] = sq;
      s_ssq[(1 * kRows + row) * 4 + (warp & 3)] = sk;
    }
    const uint4 gw = *reinterpret_cast<const uint4*>(smem + kStG + stage_off(row, j));
    unpack8(gw, f);
    const bool valid = row < len;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float x = valid ? fmaf(tanh_approx(fmaf(f[i], ha, hab[i])), hgs, hgs) : 0.f;
#pragma unroll
      for (int d = 1; d < 8; d <<= 1) {          // inclusive scan over the 8 rows held by the 8 lanes of this group
        const float y = __shfl_up_sync(0xffffffffu, x, d, 8);
        if (r8 >= d) x += y;
      }
      G[i] = x;
    }
    float th[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) th[i] = __shfl_sync(0xffffffffu, G[i], 7, 8);
    if (r8 == 0) {
      *reinterpret_cast<float4*>(s_tot + half * kD + 8 * j) = make_float4(th[0], th[1], th[2], th[3]);
      *reinterpret_cast<float4*>(s_tot + half * kD + 8 * j + 4) = make_float4(th[4], th[5], th[6], th[7]);
    }
  }
  __syncthreads();

  // ---- decayed operands ---------------------------------------------------------------------------------------------
  {
    const float4 a0 = *reinterpret_cast<const float4*>(s_tot + 8 * j);
    const float4 a1 = *reinterpret_cast<const float4*>(s_tot + 8 * j + 4);
    const float4 c0 = *reinterpret_cast<const float4*>(s_tot + kD + 8 * j);
    const float4 c1 = *reinterpret_cast<const float4*>(s_tot + kD + 8 * j + 4);
    const float lo[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float hi[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float fa[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (half) G[i] += lo[i];
      fa[i] = ex2f(lo[i] + hi[i]);
    }
    if (tid < 128 && r8 == 0) {
      *reinterpret_cast<float4*>(s_e + 8 * j) = make_float4(fa[0], fa[1], fa[2], fa[3]);
      *reinterpret_cast<float4*>(s_e + 8 * j + 4) = make_float4(fa[4], fa[5], fa[6], fa[7]);
    }
    const float4 sq4 = *reinterpret_cast<const float4*>(s_ssq + (0 * kRows + row) * 4);
    const float4 sk4 = *reinterpret_cast<const float4*>(s_ssq + (1 * kRows + row) * 4);
    const float rq = rsqrtf(sq4.x + sq4.y + sq4.z + sq4.w + 1e-6f) * p.scale;
    const float rk = rsqrtf(sk4.x + sk4.y + sk4.z + sk4.w + 1e-6f);
    const uint32_t qraw[4] = {qw.x, qw.y, qw.z, qw.w};
    const uint32_t kraw[4] = {kw.x, kw.y, kw.z, kw.w};
    __nv_bfloat162 kp[4], qp[4], km[4], kr[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const float pw0 = ex2f(G[2 * m]), pw1 = ex2f(G[2 * m + 1]);
      const float ip0 = ex2f(-G[2 * m]), ip1 = ex2f(-G[2 * m + 1]);
      const __nv_bfloat162 k2 = *reinterpret_cast<const __nv_bfloat162*>(&kraw[m]);
      const __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162*>(&qraw[m]);
      kp[m] = __hmul2(k2, __floats2bfloat162_rn(rk * pw0, rk * pw1));
      qp[m] = __hmul2(q2, __floats2bfloat162_rn(rq * pw0, rq * pw1));
      km[m] = __hmul2(k2, __floats2bfloat162_rn(rk * ip0, rk * ip1));
      kr[m] = __hmul2(km[m], __floats2bfloat162_rn(fa[2 * m], fa[2 * m + 1]));
    }
    *reinterpret_cast<uint4*>(smem + kKP + core_off(row, 8 * j, kD)) = as_u4(kp);
    *reinterpret_cast<uint4*>(smem + kQP + core_off(row, 8 * j, kD)) = as_u4(qp);
    *reinterpret_cast<uint4*>(smem + kKM + core_off(row, 8 * j, kD)) = as_u4(km);
    *reinterpret_cast<uint4*>(smem + kKR + core_off(row, 8 * j, kD)) = as_u4(kr);
  }
  __syncthreads();
  if (!kOneBlock && blk + 1 < nblk) load_qkg(blk + 1);

  // ---- A, M (one warp each), then T = (I + A)^-1 and T diag(beta) inside warp 0 --------------------------------
  if (warp < 2) {
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const uint32_t a_lane = sbase + (warp == 0 ? kKP : kQP) + (mi & 1) * 2048 + (mi >> 1) * 128 + r * 16;
    const uint32_t b_lane = sbase + kKM + (mi >> 1) * 2048 + (mi & 1) * 128 + r * 16;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
      ldsm_x4(a_lane + ks * 256, a0, a1, a2, a3);
      ldsm_x4(b_lane + ks * 256, b0, b1, b2, b3);
      mma_bf16_16816(acc[0], a0, a1, a2, a3, b0, b1);
      mma_bf16_16816(acc[1], a0, a1, a2, a3, b2, b3);
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int lr = g + 8 * hh, lc = nt * 8 + 2 * t4;
        float x0 = acc[nt][2 * hh], x1 = acc[nt][2 * hh + 1];
        if (warp == 0) {                 // strictly lower triangle, rows scaled by beta
          const float br = s_beta[lr];
          x0 = (lc < lr) ? x0 * br : 0.f;
          x1 = (lc + 1 < lr) ? x1 * br : 0.f;
          *reinterpret_cast<float2*>(s_A + lr * kLdS + lc) = make_float2(x0, x1);
        } else {                         // lower triangle with the diagonal
          x0 = (lc <= lr) ? x0 : 0.f;
          x1 = (lc + 1 <= lr) ? x1 : 0.f;
          *reinterpret_cast<uint32_t*>(smem + kMQK + core_off(lr, lc, kRows)) = pack_bf16(x0, x1);
        }
      }
    if (warp == 0) {
      __syncwarp();
      if (lane < kRows) {
        // forward substitution, one column per lane: x_i = [i == c] - sum_{j<i} A_ij x_j
        const int c = lane;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float a = (i == c) ? 1.f : 0.f;
#pragma unroll
          for (int q4 = 0; 4 * q4 < i; ++q4) {
            const float4 a4 = *reinterpret_cast<const float4*>(s_A + i * kLdS + 4 * q4);
            a = fmaf(-a4.x, x[4 * q4], a);
            a = fmaf(-a4.y, x[4 * q4 + 1], a);
            a = fmaf(-a4.z, x[4 * q4 + 2], a);
            a = fmaf(-a4.w, x[4 * q4 + 3], a);
          }
          x[i] = a;
          s_T[i * kLdS + c] = a;
        }
      }
      __syncwarp();
      if (lane < kRows) {
        // T diag(beta) as a bf16 core-layout operand; lane = row
        const int rr = lane;
        uint8_t* dst = smem + kTB + (rr >> 3) * 256 + (rr & 7) * 16;
#pragma unroll
        for (int q8 = 0; q8 < 2; ++q8) {
          const float4 ta = *reinterpret_cast<const float4*>(s_T + rr * kLdS + 8 * q8);
          const float4 tb = *reinterpret_cast<const float4*>(s_T + rr * kLdS + 8 * q8 + 4);
          const float4 ba = *reinterpret_cast<const float4*>(s_beta + 8 * q8);
          const float4 bb = *reinterpret_cast<const float4*>(s_beta + 8 * q8 + 4);
          const float tv[8] = {ta.x, ta.y, ta.z, ta.w, tb.x, tb.y, tb.z, tb.w};
          const float bv[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
          uint32_t w[4];
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) {
            const int c = 8 * q8 + 2 * e2;
            w[e2] = pack_bf16(c <= rr ? tv[2 * e2] * bv[2 * e2] : 0.f, c + 1 <= rr ? tv[2 * e2 + 1] * bv[2 * e2 + 1] : 0.f);
          }
          *reinterpret_cast<uint4*>(dst + q8 * 128) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }
  __syncthreads();

  // ---- w' = TB k+ (this warp's 16 k-columns, to shared memory) and u' = TB v (this warp's 16 v, kept) ------------
  float up[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  {
    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
    ldsm_x4(sbase + kTB + (mi & 1) * 256 + (mi >> 1) * 128 + r * 16, a0, a1, a2, a3);
    float wp[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    ldsm_x4_trans(sbase + kKP + (mi & 1) * 2048 + (2 * warp + (mi >> 1)) * 128 + r * 16, b0, b1, b2, b3);
    mma_bf16_16816(wp[0], a0, a1, a2, a3, b0, b1);
    mma_bf16_16816(wp[1], a0, a1, a2, a3, b2, b3);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int c = 16 * warp + 8 * nt + 2 * t4;
      *reinterpret_cast<uint32_t*>(smem + kWP + core_off(g, c, kD)) = pack_bf16(wp[nt][0], wp[nt][1]);
      *reinterpret_cast<uint32_t*>(smem + kWP + core_off(g + 8, c, kD)) = pack_bf16(wp[nt][2], wp[nt][3]);
    }
    ldsm_x4_trans(sbase + kStV + stage_off(8 * (mi & 1) + r, 2 * warp + (mi >> 1)), b0, b1, b2, b3);
    mma_bf16_16816(up[0], a0, a1, a2, a3, b0, b1);
    mma_bf16_16816(up[1], a0, a1, a2, a3, b2, b3);
  }
  __syncthreads();
  if (!kOneBlock && blk + 1 < nblk) load_v(blk + 1);

  // ---- this warp's 16 rows of the state -> accumulator fragments -----------------------------------------------------
  // tile jt covers state columns k = 8jt .. 8jt+7: S[jt][0,1] = row v0, columns 8jt + 2t, +1; S[jt][2,3] = row v0 + 8
  float S[16][4];
  if (blk == 0 && p.initial_state == nullptr) {
#pragma unroll
    for (int jt = 0; jt < 16; ++jt) S[jt][0] = S[jt][1] = S[jt][2] = S[jt][3] = 0.f;
  } else {
    if (blk == 0) mbar_wait(bar, 0, abort_flag);     // gives up after 2 s and raises the abort flag, seen at the next block top / the exit
    if (blk > 0 || p.state_fp32) {
#pragma unroll
      for (int jt = 0; jt < 16; ++jt) {
        const float2 lo = *reinterpret_cast<const float2*>(srow + (8 * jt + 2 * t4) * 4);
        const float2 hi = *reinterpret_cast<const float2*>(srow + 8 * kStride32 + (8 * jt + 2 * t4) * 4);
        S[jt][0] = lo.x; S[jt][1] = lo.y; S[jt][2] = hi.x; S[jt][3] = hi.y;
      }
    } else {
#pragma unroll
      for (int jt = 0; jt < 16; ++jt) {
        const uint32_t lo = *reinterpret_cast<const uint32_t*>(srow + kStride16 + (8 * jt + 2 * t4) * 2);
        const uint32_t hi = *reinterpret_cast<const uint32_t*>(srow + 8 * kStride32 + kStride16 + (8 * jt + 2 * t4) * 2);
        S[jt][0] = bf_lo(lo); S[jt][1] = bf_hi(lo); S[jt][2] = bf_lo(hi); S[jt][3] = bf_hi(hi);
      }
    }
  }

  // ---- W = w' S and O = q+ S on this warp's 16 v (B fragments = the state registers rounded to bf16) -------------
  float Wa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  float Oa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  {
    const uint32_t w_lane = sbase + kWP + (mi & 1) * 2048 + (mi >> 1) * 128 + r * 16;
    const uint32_t q_lane = sbase + kQP + (mi & 1) * 2048 + (mi >> 1) * 128 + r * 16;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t w0, w1, w2, w3, q0, q1, q2, q3;
      ldsm_x4(w_lane + ks * 256, w0, w1, w2, w3);
      ldsm_x4(q_lane + ks * 256, q0, q1, q2, q3);
#pragma unroll
      for (int m = 0; m < 2; ++m) {     // v tile m: rows v0 (m = 0) or v0 + 8 (m = 1) of the state
        const uint32_t b0 = pack_bf16(S[2 * ks][2 * m], S[2 * ks][2 * m + 1]);
        const uint32_t b1 = pack_bf16(S[2 * ks + 1][2 * m], S[2 * ks + 1][2 * m + 1]);
        mma_bf16_16816(Wa[m], w0, w1, w2, w3, b0, b1);
        mma_bf16_16816(Oa[m], q0, q1, q2, q3, b0, b1);
      }
    }
  }
  // U = u' - W as bf16, then its four 8x8 tiles transposed: Ut[m][hh] = tile (tokens 8hh.., v tile m)^T,
  // i.e. this thread holds U[token 8hh + 2t, +1][v = 8m + g]
  uint32_t Ut[2][2];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    Ut[m][0] = movmatrix_trans(pack_bf16(up[m][0] - Wa[m][0], up[m][1] - Wa[m][1]));
    Ut[m][1] = movmatrix_trans(pack_bf16(up[m][2] - Wa[m][2], up[m][3] - Wa[m][3]));
  }
  {  // O += M U
    uint32_t a0, a1, a2, a3;
    ldsm_x4(sbase + kMQK + (mi & 1) * 256 + (mi >> 1) * 128 + r * 16, a0, a1, a2, a3);
    mma_bf16_16816(Oa[0], a0, a1, a2, a3, Ut[0][0], Ut[0][1]);
    mma_bf16_16816(Oa[1], a0, a1, a2, a3, Ut[1][0], Ut[1][1]);
  }
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const int vcol = 16 * warp + 8 * m + 2 * t4;
    if (g < len)
      *reinterpret_cast<uint32_t*>(p.out + (static_cast<size_t>(t0 + g) * p.H + h) * kD + vcol) = pack_bf16(Oa[m][0], Oa[m][1]);
    if (g + 8 < len)
      *reinterpret_cast<uint32_t*>(p.out + (static_cast<size_t>(t0 + g + 8) * p.H + h) * kD + vcol) = pack_bf16(Oa[m][2], Oa[m][3]);
  }

  // ---- S' = diag(e) S + U^T kr: A = U^T (rows v, K = tokens), B = kr read transposed, accumulators = the state ----
  const bool last = kOneBlock || blk + 1 == nblk;
  if (!last || p.final_state != nullptr) {
#pragma unroll
    for (int jp = 0; jp < 8; ++jp) {   // two column tiles per transposed load
      uint32_t b0, b1, b2, b3;
      ldsm_x4_trans(sbase + kKR + (mi & 1) * 2048 + (2 * jp + (mi >> 1)) * 128 + r * 16, b0, b1, b2, b3);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int jt = 2 * jp + q;
        const float2 e2 = *reinterpret_cast<const float2*>(s_e + 8 * jt + 2 * t4);
        S[jt][0] *= e2.x; S[jt][1] *= e2.y; S[jt][2] *= e2.x; S[jt][3] *= e2.y;
        mma_bf16_16816(S[jt], Ut[0][0], Ut[1][0], Ut[0][1], Ut[1][1], q ? b2 : b0, q ? b3 : b1);
      }
    }
    // back into this warp's staging rows (nobody else touches them): fp32 between blocks, the caller's type at the end
    if (!last || p.state_fp32) {
#pragma unroll
      for (int jt = 0; jt < 16; ++jt) {
        *reinterpret_cast<float2*>(srow + (8 * jt + 2 * t4) * 4) = make_float2(S[jt][0], S[jt][1]);
        *reinterpret_cast<float2*>(srow + 8 * kStride32 + (8 * jt + 2 * t4) * 4) = make_float2(S[jt][2], S[jt][3]);
      }
    } else {
#pragma unroll
      for (int jt = 0; jt < 16; ++jt) {
        *reinterpret_cast<uint32_t*>(srow + (8 * jt + 2 * t4) * 2) = pack_bf16(S[jt][0], S[jt][1]);
        *reinterpret_cast<uint32_t*>(srow + 8 * kStride32 + (8 * jt + 2 * t4) * 2) = pack_bf16(S[jt][2], S[jt][3]);
      }
    }
  }
  }  // blocks

  if (failed || *abort_flag > 0) {
    // the state copy may still be landing: give it a moment before this CTA's shared memory goes away
    const uint64_t t_begin = globaltimer_ns();
    while (!mbar_try_wait(bar, 0) && globaltimer_ns() - t_begin < 20000000ull) {}
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);
    return;
  }
  if (p.final_state != nullptr) {      // one bulk copy per row, per warp as soon as its rows are done
    fence_proxy_async_smem();
    __syncwarp();
    if (lane < 16) {
      const int vr = 16 * warp + lane;
      bulk_s2g(static_cast<uint8_t*>(p.final_state) + (static_cast<size_t>(chain) * kD + vr) * row_bytes,
               sbase + kState + vr * kStride32, row_bytes);
      bulk_commit();
      bulk_wait_read0();               // shared memory must outlive the copy's reads
    }
  }
}

}  // namespace short16

cudaError_t launch_short16(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, const __nv_bfloat16* g,
                           const __nv_bfloat16* beta, const float* A_log, const float* dt_bias, const void* initial_state,
                           void* final_state, __nv_bfloat16* out, int64_t N, int T, int H, int state_fp32, float scale,
                           float gate_scale, int* status, cudaStream_t stream) {
  if (N * H == 0) return cudaSuccess;
  short16::Params p{q, k, v, g, beta, A_log, dt_bias, initial_state, final_state, out, T, H, state_fp32, scale, gate_scale, status};
  auto kernel = T <= short16::kRows ? short16::short16_kernel<true> : short16::short16_kernel<false>;
  static SmemOptIn opt_in[2];
  cudaError_t e = opt_in[T <= short16::kRows ? 1 : 0].ensure(kernel, short16::kSmemBytes);
  if (e != cudaSuccess) return e;
  kernel<<<static_cast<unsigned>(N * H), short16::kThreads, short16::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fkda
