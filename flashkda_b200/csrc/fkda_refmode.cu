// Reference-rounding mode (flag FKDA_FLAG_REFERENCE_ROUNDING): the forward pass evaluated the way the reference does
// - tiles of 16 tokens, the state kept in bf16 between tiles, a bf16 rounding at every point where the reference's
// kernels round, the same hardware approximations (tanh.approx, ex2.approx, rsqrt.approx) in the same places and the
// same mma.sync m16n8k16 products in the same k order (restated from the reference's own oracle,
// tests/torch_ref.py:62-247, and its kernels csrc/smxx/fwd_kernel1.cuh:265-508, fwd_kernel2.cuh:533-731) - instead of
// the chunk-32 / fp32-state form of the production kernels.  `out` and the final state are then the same bits as
// those of the reference's CUDA kernels run on the same GPU (tests/test_gpu_reference_bits.py).  It is several times
// slower than the production path and exists so that a disagreement with the reference can be told apart from rounding.
//
// One CTA of 256 threads per (sequence, head) chain walks the tiles; fixed-length batches and varlen alike.
// Per tile (rows i = 0..15, channel k, G = running sum of the log2 gate):
//     kd = bf(kn bf(2^G)), qd = bf(bf(qn bf(2^G)) bf(scale)), ki = bf(kn bf(2^-G)), kr = bf(ki bf(2^G15)),  kn = bf(k / |k|)
//     L = tril(kd ki^T, -1) sigmoid(beta_i) (fp32),  M = bf(tril(qd ki^T)),  INV = bf((I + L)^-1) by 8x8 blocks
//     W = bf(kd S),  V' = bf(bf(v - W) bf(sigmoid(beta))),  U = bf(INV V'),  out = bf(bf(qd S) + bf(M U))
//     S = bf(fma(S, 2^G15, kr^T U))
#include "fkda_common.cuh"

namespace fkda {
namespace refmode {

constexpr int kRows = 16;
constexpr int kThreads = 256;
constexpr int kLdS = 20;
// shared memory (byte offsets)
constexpr int kStQ = 0;                          // staged q, k, g, v: [16 tok][256 B], 16-byte chunks XOR-swizzled by the row
constexpr int kStK = kStQ + 4096;
constexpr int kStG = kStK + 4096;
constexpr int kStV = kStG + 4096;
constexpr int kKD = kStV + 4096;                 // bf16 [16][128] tiles in the 8x8 core-matrix layout
constexpr int kQD = kKD + 4096;
constexpr int kKI = kQD + 4096;
constexpr int kKR = kKI + 4096;
constexpr int kINV = kKR + 4096;                 // bf16 [16][16], core layout
constexpr int kMQK = kINV + 512;                 // bf16 [16][16]
constexpr int kL = kMQK + 512;                   // fp32 [16][20]
constexpr int kP = kL + kRows * kLdS * 4;        // fp32 [16][20]: bf16-valued inverses of the diagonal 8x8 blocks
constexpr int kX = kP + kRows * kLdS * 4;        // fp32 [8][12] scratch of the merge
constexpr int kE = kX + 8 * 12 * 4;              // fp32 [128] 2^G15
constexpr int kPart = kE + 512;                  // fp32 [2][16][16] partial sums of squares (q, k)
constexpr int kBeta = kPart + 2048;              // fp32 [16] sigmoid(beta), then [16] its bf16 rounding
constexpr int kState = (kBeta + 128 + 127) / 128 * 128;
constexpr int kStride = 512 + 32;                // fp32 state rows, padded (see fkda_short16.cu)
constexpr int kSmemBytes = kState + kD * kStride;

__device__ __forceinline__ float rbf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

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
  const int64_t* cu_seqlens;
  int64_t T;             // tokens per sequence (fixed-length) or in total (varlen)
  int64_t T_total;
  int H;
  int state_fp32;
  float scale;
  float gate_scale;
};

__global__ void __launch_bounds__(kThreads, 1) refmode_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chain = blockIdx.x;
  const int n = chain / p.H, h = chain - n * p.H;
  int64_t bos, eos;
  if (p.cu_seqlens != nullptr) {
    bos = p.cu_seqlens[n];
    eos = p.cu_seqlens[n + 1];
    bos = bos < 0 ? 0 : (bos > p.T_total ? p.T_total : bos);
    eos = eos < bos ? bos : (eos > p.T_total ? p.T_total : eos);
  } else {
    bos = static_cast<int64_t>(n) * p.T;
    eos = bos + p.T;
  }
  const int nblk = static_cast<int>((eos - bos + kRows - 1) / kRows);

  float* s_L = reinterpret_cast<float*>(smem + kL);
  float* s_P = reinterpret_cast<float*>(smem + kP);
  float* s_X = reinterpret_cast<float*>(smem + kX);
  float* s_e = reinterpret_cast<float*>(smem + kE);
  float* s_part = reinterpret_cast<float*>(smem + kPart);
  float* s_beta = reinterpret_cast<float*>(smem + kBeta);

  // ---- state -> fp32 staging rows holding bf16 values (an fp32 state is rounded on entry, as the reference does) ---
  for (int i = tid; i < kD * kD; i += kThreads) {
    const int vv = i >> 7, kk = i & 127;
    float s0 = 0.f;
    if (p.initial_state != nullptr) {
      const size_t idx = (static_cast<size_t>(chain) * kD + vv) * kD + kk;
      s0 = p.state_fp32 ? rbf(reinterpret_cast<const float*>(p.initial_state)[idx])
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.initial_state)[idx]);
    }
    *reinterpret_cast<float*>(smem + kState + vv * kStride + kk * 4) = s0;
  }

  // thread -> (row, 8-column group): the 16 rows of a group sit in 16 consecutive lanes
  const int row = tid & 15;
  const int j = tid >> 4;
  const float a_exp = ex2f(__ldg(p.A_log + h) * kLog2e);
  float bias[8];
  {
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * j));
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * j + 4));
    bias[0] = b0.x; bias[1] = b0.y; bias[2] = b0.z; bias[3] = b0.w;
    bias[4] = b1.x; bias[5] = b1.y; bias[6] = b1.z; bias[7] = b1.w;
  }
  const __nv_bfloat16 scale_bf = __float2bfloat16_rn(p.scale);
  const int g = lane >> 2, t4 = lane & 3;
  const int mi = lane >> 3, r = lane & 7;
  const int v0 = 16 * warp + g;
  uint8_t* const srow = smem + kState + v0 * kStride;

  for (int blk = 0; blk < nblk; ++blk) {
    const int64_t t0 = bos + static_cast<int64_t>(kRows) * blk;
    const int len = eos - t0 < kRows ? static_cast<int>(eos - t0) : kRows;
    __syncthreads();                       // the previous tile is done with everything below
    {
      const int lrow = tid >> 4, chunk = tid & 15;
      const bool valid = lrow < len;
      const size_t off = (static_cast<size_t>(t0 + (valid ? lrow : 0)) * p.H + h) * kD + 8 * chunk;
      const uint32_t nbytes = valid ? 16u : 0u;
      const uint32_t dst = sbase + stage_off(lrow, chunk);
      cp_async16(dst + kStQ, p.q + off, nbytes);
      cp_async16(dst + kStK, p.k + off, nbytes);
      cp_async16(dst + kStG, p.g + off, nbytes);
      cp_async16(dst + kStV, p.v + off, nbytes);
    }
    if (tid < kRows) {
      // rows past the end take a zero logit (sigmoid 1/2), as in the reference
      const float blog = tid < len ? __bfloat162float(p.beta[static_cast<size_t>(t0 + tid) * p.H + h]) : 0.f;
      const float b = sigmoid_fast(blog);
      s_beta[tid] = b;
      s_beta[16 + tid] = rbf(b);
    }
    cp_async_wait_all();
    __syncthreads();

    // ---- partial sums of squares (8 FMAs per group), gate, sequential running sum over the 16 rows ------------------
    const uint4 qw = *reinterpret_cast<const uint4*>(smem + kStQ + stage_off(row, j));
    const uint4 kw = *reinterpret_cast<const uint4*>(smem + kStK + stage_off(row, j));
    float qf[8], kf[8], G[8];
    {
      qf[0] = bf_lo(qw.x); qf[1] = bf_hi(qw.x); qf[2] = bf_lo(qw.y); qf[3] = bf_hi(qw.y);
      qf[4] = bf_lo(qw.z); qf[5] = bf_hi(qw.z); qf[6] = bf_lo(qw.w); qf[7] = bf_hi(qw.w);
      kf[0] = bf_lo(kw.x); kf[1] = bf_hi(kw.x); kf[2] = bf_lo(kw.y); kf[3] = bf_hi(kw.y);
      kf[4] = bf_lo(kw.z); kf[5] = bf_hi(kw.z); kf[6] = bf_lo(kw.w); kf[7] = bf_hi(kw.w);
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) sq = fmaf(qf[i], qf[i], sq);
#pragma unroll
      for (int i = 0; i < 8; ++i) sk = fmaf(kf[i], kf[i], sk);
      s_part[(0 * kRows + row) * 16 + j] = sq;
      s_part[(1 * kRows + row) * 16 + j] = sk;
      const uint4 gw = *reinterpret_cast<const uint4*>(smem + kStG + stage_off(row, j));
      const float gf[8] = {bf_lo(gw.x), bf_hi(gw.x), bf_lo(gw.y), bf_hi(gw.y), bf_lo(gw.z), bf_hi(gw.z), bf_lo(gw.w), bf_hi(gw.w)};
      const bool valid = row < len;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float x = valid ? p.gate_scale * sigmoid_fast(a_exp * (gf[i] + bias[i])) : 0.f;
#pragma unroll
        for (int d = 1; d < kRows; ++d) {      // row d = row d-1 + its own term, one row after the other
          const float prev = __shfl_up_sync(0xffffffffu, x, 1, 16);
          if (row == d) x = prev + x;
        }
        G[i] = x;
      }
    }
    float gte[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) gte[i] = ex2f(__shfl_sync(0xffffffffu, G[i], 15, 16));
    if (row == 0) {
      *reinterpret_cast<float4*>(s_e + 8 * j) = make_float4(gte[0], gte[1], gte[2], gte[3]);
      *reinterpret_cast<float4*>(s_e + 8 * j + 4) = make_float4(gte[4], gte[5], gte[6], gte[7]);
    }
    __syncthreads();

    // ---- row norms (sixteen partials, pairwise tree over distances 8, 4, 2, 1) and the decayed operands --------------
    {
      float inv[2];
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        float pp[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pp[i] = s_part[(w * kRows + row) * 16 + i];
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) {
          float nx[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) nx[i] = pp[i] + pp[i ^ off];
#pragma unroll
          for (int i = 0; i < 16; ++i) pp[i] = nx[i];
        }
        inv[w] = rsqrtf(pp[0] + 1e-6f);      // the approximate reciprocal square root, as the reference's kernel takes it
      }
      const bool valid = row < len;
      uint32_t kd[4], qd[4], ki[4], kr[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        __nv_bfloat162 qn, kn, e2, ne2, g2;
        qn.x = __float2bfloat16_rn(valid ? qf[2 * m] * inv[0] : 0.f);
        qn.y = __float2bfloat16_rn(valid ? qf[2 * m + 1] * inv[0] : 0.f);
        kn.x = __float2bfloat16_rn(valid ? kf[2 * m] * inv[1] : 0.f);
        kn.y = __float2bfloat16_rn(valid ? kf[2 * m + 1] * inv[1] : 0.f);
        e2 = __floats2bfloat162_rn(ex2f(G[2 * m]), ex2f(G[2 * m + 1]));
        ne2 = __floats2bfloat162_rn(ex2f(-G[2 * m]), ex2f(-G[2 * m + 1]));
        g2 = __floats2bfloat162_rn(gte[2 * m], gte[2 * m + 1]);
        const __nv_bfloat162 kd2 = __hmul2(kn, e2);
        const __nv_bfloat162 qd2 = __hmul2(__hmul2(qn, e2), __nv_bfloat162(scale_bf, scale_bf));
        const __nv_bfloat162 ki2 = __hmul2(kn, ne2);
        const __nv_bfloat162 kr2 = __hmul2(ki2, g2);
        kd[m] = *reinterpret_cast<const uint32_t*>(&kd2);
        qd[m] = *reinterpret_cast<const uint32_t*>(&qd2);
        ki[m] = *reinterpret_cast<const uint32_t*>(&ki2);
        kr[m] = *reinterpret_cast<const uint32_t*>(&kr2);
      }
      *reinterpret_cast<uint4*>(smem + kKD + core_off(row, 8 * j, kD)) = make_uint4(kd[0], kd[1], kd[2], kd[3]);
      *reinterpret_cast<uint4*>(smem + kQD + core_off(row, 8 * j, kD)) = make_uint4(qd[0], qd[1], qd[2], qd[3]);
      *reinterpret_cast<uint4*>(smem + kKI + core_off(row, 8 * j, kD)) = make_uint4(ki[0], ki[1], ki[2], ki[3]);
      *reinterpret_cast<uint4*>(smem + kKR + core_off(row, 8 * j, kD)) = make_uint4(kr[0], kr[1], kr[2], kr[3]);
    }
    __syncthreads();

    // ---- L, M (one warp each), then INV = bf((I + L)^-1) inside warp 0 ------------------------------------------------
    if (warp < 2) {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const uint32_t a_lane = sbase + (warp == 0 ? kKD : kQD) + (mi & 1) * 2048 + (mi >> 1) * 128 + r * 16;
      const uint32_t b_lane = sbase + kKI + (mi >> 1) * 2048 + (mi & 1) * 128 + r * 16;
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
          if (warp == 0) {
            const float br = s_beta[lr];
            *reinterpret_cast<float2*>(s_L + lr * kLdS + lc) = make_float2(lc < lr ? x0 * br : 0.f, lc + 1 < lr ? x1 * br : 0.f);
          } else {
            *reinterpret_cast<uint32_t*>(smem + kMQK + core_off(lr, lc, kRows)) = pack_bf16(lc <= lr ? x0 : 0.f, lc + 1 <= lr ? x1 : 0.f);
          }
        }
      if (warp == 0) {
        __syncwarp();
        if (lane < kRows) {
          // inverses of the two diagonal 8x8 blocks by forward substitution, one column per lane, rounded to bf16
          const int b = lane >> 3, c = lane & 7;
          float x[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float a = (i == c) ? 1.f : 0.f;
#pragma unroll
            for (int jj = 0; jj < i; ++jj) a = fmaf(-s_L[(8 * b + i) * kLdS + 8 * b + jj], x[jj], a);
            x[i] = a;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            s_P[(8 * b + i) * kLdS + 8 * b + c] = rbf(x[i]);
            s_P[(8 * b + i) * kLdS + 8 * (1 - b) + c] = 0.f;
          }
        }
        __syncwarp();
        // off-diagonal block: INV10 = bf( bf(-(P11 bf(L10))) P00 ), both products accumulated in fp32
        const int oi = lane >> 2, oj = (lane & 3) * 2;    // two entries (oi, oj), (oi, oj + 1) per lane
        {
          float x0 = 0.f, x1 = 0.f;
#pragma unroll
          for (int l = 0; l < 8; ++l) {
            const float pl = s_P[(8 + oi) * kLdS + 8 + l];
            x0 = fmaf(pl, rbf(s_L[(8 + l) * kLdS + oj]), x0);
            x1 = fmaf(pl, rbf(s_L[(8 + l) * kLdS + oj + 1]), x1);
          }
          s_X[oi * 12 + oj] = rbf(-x0);
          s_X[oi * 12 + oj + 1] = rbf(-x1);
        }
        __syncwarp();
        {
          float y0 = 0.f, y1 = 0.f;
#pragma unroll
          for (int l = 0; l < 8; ++l) {
            const float xl = s_X[oi * 12 + l];
            y0 = fmaf(xl, s_P[l * kLdS + oj], y0);
            y1 = fmaf(xl, s_P[l * kLdS + oj + 1], y1);
          }
          s_P[(8 + oi) * kLdS + oj] = rbf(y0);
          s_P[(8 + oi) * kLdS + oj + 1] = rbf(y1);
        }
        __syncwarp();
        if (lane < kRows) {
          const int rr = lane;
          uint8_t* dst = smem + kINV + (rr >> 3) * 256 + (rr & 7) * 16;
#pragma unroll
          for (int q8 = 0; q8 < 2; ++q8) {
            uint32_t w[4];
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) w[e2] = pack_bf16(s_P[rr * kLdS + 8 * q8 + 2 * e2], s_P[rr * kLdS + 8 * q8 + 2 * e2 + 1]);
            *reinterpret_cast<uint4*>(dst + q8 * 128) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    __syncthreads();

    // ---- this warp's 16 state rows: W = bf(kd S), O0 = bf(qd S) --------------------------------------------------------
    float S[16][4];
#pragma unroll
    for (int jt = 0; jt < 16; ++jt) {
      const float2 lo = *reinterpret_cast<const float2*>(srow + (8 * jt + 2 * t4) * 4);
      const float2 hi = *reinterpret_cast<const float2*>(srow + 8 * kStride + (8 * jt + 2 * t4) * 4);
      S[jt][0] = lo.x; S[jt][1] = lo.y; S[jt][2] = hi.x; S[jt][3] = hi.y;
    }
    float Wa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    float Oa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const uint32_t k_lane = sbase + kKD + (mi & 1) * 2048 + (mi >> 1) * 128 + r * 16;
      const uint32_t q_lane = sbase + kQD + (mi & 1) * 2048 + (mi >> 1) * 128 + r * 16;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t w0, w1, w2, w3, q0, q1, q2, q3;
        ldsm_x4(k_lane + ks * 256, w0, w1, w2, w3);
        ldsm_x4(q_lane + ks * 256, q0, q1, q2, q3);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const uint32_t b0 = pack_bf16(S[2 * ks][2 * m], S[2 * ks][2 * m + 1]);         // exact: the state holds bf16 values
          const uint32_t b1 = pack_bf16(S[2 * ks + 1][2 * m], S[2 * ks + 1][2 * m + 1]);
          mma_bf16_16816(Wa[m], w0, w1, w2, w3, b0, b1);
          mma_bf16_16816(Oa[m], q0, q1, q2, q3, b0, b1);
        }
      }
    }
    // V' = bf(bf(v - bf(W)) bf(beta)) in the accumulator layout: rows g / g + 8, columns 16 warp + 8 m + 2 t, +1
    uint32_t Vt[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int tok = g + 8 * hh, vcol = 16 * warp + 8 * m + 2 * t4;
        const uint32_t vw = *reinterpret_cast<const uint32_t*>(smem + kStV + stage_off(tok, vcol >> 3) + (vcol & 7) * 2);
        const float bb = s_beta[16 + tok];
        // bf16 arithmetic, one rounding per operation as the reference's bf16 operators have it (an fp32 difference
        // rounded afterwards rounds twice where the operands' exponents lie more than sixteen apart)
        const uint32_t w2 = pack_bf16(Wa[m][2 * hh], Wa[m][2 * hh + 1]);
        const __nv_bfloat162 d2 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&vw), *reinterpret_cast<const __nv_bfloat162*>(&w2));
        const __nv_bfloat162 a2 = __hmul2(d2, __floats2bfloat162_rn(bb, bb));
        Vt[m][hh] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&a2));
      }
    // U = bf(INV V')
    uint32_t Ut[2][2];
    {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(sbase + kINV + (mi & 1) * 256 + (mi >> 1) * 128 + r * 16, a0, a1, a2, a3);
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        float u[4] = {0.f, 0.f, 0.f, 0.f};
        mma_bf16_16816(u, a0, a1, a2, a3, Vt[m][0], Vt[m][1]);
        Ut[m][0] = movmatrix_trans(pack_bf16(u[0], u[1]));
        Ut[m][1] = movmatrix_trans(pack_bf16(u[2], u[3]));
      }
    }
    // out = bf(bf(qd S) + bf(M U))
    {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(sbase + kMQK + (mi & 1) * 256 + (mi >> 1) * 128 + r * 16, a0, a1, a2, a3);
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        float mu[4] = {0.f, 0.f, 0.f, 0.f};
        mma_bf16_16816(mu, a0, a1, a2, a3, Ut[m][0], Ut[m][1]);
        const int vcol = 16 * warp + 8 * m + 2 * t4;
        if (g < len)
          *reinterpret_cast<__nv_bfloat162*>(p.out + (static_cast<size_t>(t0 + g) * p.H + h) * kD + vcol) =
              __hadd2(__floats2bfloat162_rn(Oa[m][0], Oa[m][1]), __floats2bfloat162_rn(mu[0], mu[1]));
        if (g + 8 < len)
          *reinterpret_cast<__nv_bfloat162*>(p.out + (static_cast<size_t>(t0 + g + 8) * p.H + h) * kD + vcol) =
              __hadd2(__floats2bfloat162_rn(Oa[m][2], Oa[m][3]), __floats2bfloat162_rn(mu[2], mu[3]));
      }
    }
    // S = bf(fma(S, 2^G15, kr^T U)), tile by tile
#pragma unroll
    for (int jp = 0; jp < 8; ++jp) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_trans(sbase + kKR + (mi & 1) * 2048 + (2 * jp + (mi >> 1)) * 128 + r * 16, b0, b1, b2, b3);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int jt = 2 * jp + q;
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        mma_bf16_16816(d, Ut[0][0], Ut[1][0], Ut[0][1], Ut[1][1], q ? b2 : b0, q ? b3 : b1);
        const float2 e2 = *reinterpret_cast<const float2*>(s_e + 8 * jt + 2 * t4);
        S[jt][0] = rbf(fmaf(S[jt][0], e2.x, d[0]));
        S[jt][1] = rbf(fmaf(S[jt][1], e2.y, d[1]));
        S[jt][2] = rbf(fmaf(S[jt][2], e2.x, d[2]));
        S[jt][3] = rbf(fmaf(S[jt][3], e2.y, d[3]));
      }
    }
#pragma unroll
    for (int jt = 0; jt < 16; ++jt) {
      *reinterpret_cast<float2*>(srow + (8 * jt + 2 * t4) * 4) = make_float2(S[jt][0], S[jt][1]);
      *reinterpret_cast<float2*>(srow + 8 * kStride + (8 * jt + 2 * t4) * 4) = make_float2(S[jt][2], S[jt][3]);
    }
  }

  // ---- final state: the bf16 values, widened if the caller's tensors are fp32 -----------------------------------------
  __syncthreads();
  if (p.final_state != nullptr)
    for (int i = tid; i < kD * kD; i += kThreads) {
      const int vv = i >> 7, kk = i & 127;
      const float s = *reinterpret_cast<const float*>(smem + kState + vv * kStride + kk * 4);
      const size_t idx = (static_cast<size_t>(chain) * kD + vv) * kD + kk;
      if (p.state_fp32) reinterpret_cast<float*>(p.final_state)[idx] = s;
      else reinterpret_cast<__nv_bfloat16*>(p.final_state)[idx] = __float2bfloat16_rn(s);
    }
}

}  // namespace refmode

cudaError_t launch_refmode(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v, const __nv_bfloat16* g,
                           const __nv_bfloat16* beta, const float* A_log, const float* dt_bias, const void* initial_state,
                           void* final_state, __nv_bfloat16* out, const int64_t* cu_seqlens, int64_t N, int64_t T, int64_t T_total,
                           int H, int state_fp32, float scale, float gate_scale, cudaStream_t stream) {
  if (N * H == 0) return cudaSuccess;
  refmode::Params p{q, k, v, g, beta, A_log, dt_bias, initial_state, final_state, out, cu_seqlens, T, T_total, H, state_fp32, scale, gate_scale};
  static SmemOptIn opt_in;
  cudaError_t e = opt_in.ensure(refmode::refmode_kernel, refmode::kSmemBytes);
  if (e != cudaSuccess) return e;
  refmode::refmode_kernel<<<static_cast<unsigned>(N * H), refmode::kThreads, refmode::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fkda
