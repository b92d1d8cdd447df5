// Token-parallel half of the KDA prefill on the Blackwell data path: TMA-staged inputs, the intra-chunk products on
// tcgen05 with accumulators in tensor memory.
//
// Replaces the reference's K1 (csrc/smxx/fwd_kernel1.cuh:107-586: one 16-token tile per CTA, mma.sync products on
// two of eight warps, a one-warp inverse) and writes the same operand record as fkda_prepare.cu (fkda_common.cuh),
// so every recurrence kernel consumes its output unchanged.  An item is one (32-token chunk, head) pair.  Two kernels:
//
//   prepare_pipe_kernel (default)   three CTAs per SM, each a loop over items with two operand buffers: eight element
//                                   warps work on item i while a ninth warp does the serial part of item i - 1
//   prepare_tc4_kernel              one CTA of eight warps per item, four CTAs per SM, phases separated by CTA-wide
//                                   barriers; other resident CTAs fill the waits of the serial part
//
// Both: q, k, g, v arrive as [32 tok][64 ch] TMA boxes with the 128-byte swizzle; the element-wise work (L2 norms, gate,
// running sums of the log2 decay, decayed operands KPm, QPm, KMm in bf16 core-matrix layout) runs on CUDA cores with
// every thread owning two (row, 8 channel) pieces; first products [A; M] = [KPm; QPm] KMm^T (M = 128, N = 32, K = 128);
// A from tensor memory, T = (I + A)^-1 by fp32 forward substitution on the two 16 x 16 diagonal blocks (one column per
// lane) and two tf32 products for the block below them, TB^T as an MN-major operand; second products
// (w')^T = KPm^T TB^T and (u')^T = v^T TB^T (M = 128, N = 32, K = 32).
//
// Decay ranges: with G the running log2 decay inside the chunk and P its value after the first 16 tokens, the
// products use k+ = khat 2^(G - P) and k- = khat 2^(P - G): both stay inside 2^(+-115.4) for lower_bound >= -5
// (16 tokens x 5 x log2 e), every needed product k+_i k-_j (j <= i) is <= 1 in magnitude, and one 32 x 32 product
// covers both sub-blocks and their cross block.  w' is formed from k+ and multiplied by 2^P per channel on the way out.
#include <cuda.h>

#include "fkda_common.cuh"

namespace fkda {
namespace prep_tc {

#ifdef FKDA_TUNING
static long long* g_trace = nullptr;      // timeline buffer of a tuning build (see the trace macros of the kernels)
#endif

// ---- PTX wrappers used only here ------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
// the same box into the L2 only (no shared-memory destination, nothing to wait for)
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0),
               "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// 16 lanes x 32 columns in the accumulator-fragment shape: registers 4j, 4j+1 = (lane t/4, columns 8j + 2(t%4), +1),
// 4j+2, 4j+3 = (lane t/4 + 8, same columns), j = 0..3
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// stores the transposes of four 8x8 tiles of 16-bit elements held as mma fragments (thread t: row t/4, columns 2(t%4), +1);
// lane 8m + r supplies the address of row r of tile m
__device__ __forceinline__ void stsm_x4_trans(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ void st_global_16(void* p, const uint4& v) {
  asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- the stages that both kernels of this file run on their warps ---------------------------------------------------------

constexpr int kLdA = 36;      // floats per row of the fp32 A and T matrices of the inverse

// A thread's share of an item between the two element phases: two (row, 8 channel) pieces of q, k, v (raw bf16) and of
// the running log2 decay G (relative to the boundary between the two 16-token sub-blocks).
struct ElementPieces {
  uint4 qw[2], kw[2], vw[2];
  float G[2][8];
};
// thread -> pieces: rows sb * 16 + r8 and + 8 of sub-block sb, channels 8 j .. 8 j + 7
struct ElementMap {
  int r8, j, sb, row0, row1, hh, cj;
  __device__ __forceinline__ explicit ElementMap(int tid) {
    const int cm = tid >> 3;
    r8 = tid & 7;
    j = cm & 15;
    sb = cm >> 4;
    row0 = sb * 16 + r8;
    row1 = row0 + 8;
    hh = j >> 3;
    cj = j & 7;
  }
};

// First element phase: the swizzled tiles q | k | g | v (8192 bytes each, two [32 tok][128 B] halves) -> registers, partial
// sums of squares to s_ssq [2][32][4], the gate and its running sum, 2^(sub-block total) to s_ex [2][128].  A rendezvous
// of the eight warps must follow.  `ha` = exp(A_log[h]) / 2, b0 / b1 = dt_bias[h][8 j ..].
__device__ __forceinline__ void element_phase1(const uint8_t* tiles, float* s_ssq, float* s_ex, const ElementMap& m, int lane, int warp,
                                               int len, float ha, const float4& b0, const float4& b1, float gate_scale, ElementPieces& pc) {
  const int r8 = m.r8, j = m.j, sb = m.sb, row0 = m.row0, row1 = m.row1, hh = m.hh, cj = m.cj;
  {
    const uint8_t* stg = tiles + hh * 4096;
    const int sw = (cj ^ r8) << 4;
    const bool valid0 = row0 < len, valid1 = row1 < len;
    const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
    uint4 gw[2];
    pc.qw[0] = *reinterpret_cast<const uint4*>(stg + row0 * 128 + sw);
    pc.qw[1] = *reinterpret_cast<const uint4*>(stg + row1 * 128 + sw);
    pc.kw[0] = *reinterpret_cast<const uint4*>(stg + 8192 + row0 * 128 + sw);
    pc.kw[1] = *reinterpret_cast<const uint4*>(stg + 8192 + row1 * 128 + sw);
    gw[0] = *reinterpret_cast<const uint4*>(stg + 16384 + row0 * 128 + sw);
    gw[1] = *reinterpret_cast<const uint4*>(stg + 16384 + row1 * 128 + sw);
    pc.vw[0] = *reinterpret_cast<const uint4*>(stg + 24576 + row0 * 128 + sw);
    pc.vw[1] = *reinterpret_cast<const uint4*>(stg + 24576 + row1 * 128 + sw);
    if (!valid0) { pc.qw[0] = z4; pc.kw[0] = z4; gw[0] = z4; pc.vw[0] = z4; }      // rows past the sequence end belong to somebody else
    if (!valid1) { pc.qw[1] = z4; pc.kw[1] = z4; gw[1] = z4; pc.vw[1] = z4; }
    const float hgs = 0.5f * gate_scale;
    const float hab[8] = {ha * b0.x, ha * b0.y, ha * b0.z, ha * b0.w, ha * b1.x, ha * b1.y, ha * b1.z, ha * b1.w};
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = hf ? row1 : row0;
      float e8[8], sq = 0.f, sk = 0.f;
      unpack8(pc.qw[hf], e8);
#pragma unroll
      for (int i = 0; i < 8; ++i) sq = fmaf(e8[i], e8[i], sq);
      unpack8(pc.kw[hf], e8);
#pragma unroll
      for (int i = 0; i < 8; ++i) sk = fmaf(e8[i], e8[i], sk);
      sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sk += __shfl_xor_sync(0xffffffffu, sk, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 16);
      sk += __shfl_xor_sync(0xffffffffu, sk, 16);
      if (lane < 8) {
        s_ssq[(0 * kChunk + row) * 4 + (warp & 3)] = sq;
        s_ssq[(1 * kChunk + row) * 4 + (warp & 3)] = sk;
      }
      unpack8(gw[hf], e8);
      const bool valid = hf ? valid1 : valid0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float x = valid ? fmaf(tanh_approx(fmaf(e8[i], ha, hab[i])), hgs, hgs) : 0.f;
#pragma unroll
        for (int d = 1; d < 8; d <<= 1) {
          const float y = __shfl_up_sync(0xffffffffu, x, d, 8);
          if (r8 >= d) x += y;
        }
        pc.G[hf][i] = x;
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) pc.G[1][i] += __shfl_sync(0xffffffffu, pc.G[0][i], 7, 8);
    float tot[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) tot[i] = __shfl_sync(0xffffffffu, pc.G[1][i], 7, 8);
    if (sb == 0) {      // exponents of sub-block 0 become relative to its end
#pragma unroll
      for (int i = 0; i < 8; ++i) { pc.G[0][i] -= tot[i]; pc.G[1][i] -= tot[i]; }
    }
    if (r8 == 7) {      // 2^(sub-block total) per channel, once for the CTA
      *reinterpret_cast<float4*>(s_ex + sb * kD + 8 * j) = make_float4(ex2f(tot[0]), ex2f(tot[1]), ex2f(tot[2]), ex2f(tot[3]));
      *reinterpret_cast<float4*>(s_ex + sb * kD + 8 * j + 4) = make_float4(ex2f(tot[4]), ex2f(tot[5]), ex2f(tot[6]), ex2f(tot[7]));
    }
  }
}

// Second element phase: the decayed operands KPm | QPm | KMm | VC (bf16, core-matrix layout [32][128], 8192 bytes each) over
// the tiles at `ops`, and the record parts that are final at this point (QP, KR, E) straight to global memory.
__device__ __forceinline__ void element_phase2(uint8_t* ops, const float* s_ssq, const float* s_ex, uint8_t* rec_dst, const ElementMap& m,
                                               float scale, const ElementPieces& pc) {
  const int r8 = m.r8, j = m.j, sb = m.sb, row0 = m.row0, row1 = m.row1;
  {
    if (sb == 0 && r8 == 0) {
      const float4 p0 = *reinterpret_cast<const float4*>(s_ex + 8 * j), p1 = *reinterpret_cast<const float4*>(s_ex + 8 * j + 4);
      const float4 q0 = *reinterpret_cast<const float4*>(s_ex + kD + 8 * j), q1 = *reinterpret_cast<const float4*>(s_ex + kD + 8 * j + 4);
      float* e = reinterpret_cast<float*>(rec_dst + kRecE) + 8 * j;
      *reinterpret_cast<float4*>(e) = make_float4(p0.x * q0.x, p0.y * q0.y, p0.z * q0.z, p0.w * q0.w);
      *reinterpret_cast<float4*>(e + 4) = make_float4(p1.x * q1.x, p1.y * q1.y, p1.z * q1.z, p1.w * q1.w);
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = hf ? row1 : row0;
      const int off = core_off(row, 8 * j, kD);
      *reinterpret_cast<uint4*>(ops + 24576 + off) = pc.vw[hf];       // v goes on to the products as it is
      const float4 sq4 = *reinterpret_cast<const float4*>(s_ssq + (0 * kChunk + row) * 4);
      const float4 sk4 = *reinterpret_cast<const float4*>(s_ssq + (1 * kChunk + row) * 4);
      const float rq = rsqrtf(sq4.x + sq4.y + sq4.z + sq4.w + 1e-6f) * scale;
      const float rk = rsqrtf(sk4.x + sk4.y + sk4.z + sk4.w + 1e-6f);
      // each factor is formed in fp32, rounded to bf16 once and applied to the raw bf16 input with a packed multiply
      const uint32_t qraw[4] = {pc.qw[hf].x, pc.qw[hf].y, pc.qw[hf].z, pc.qw[hf].w};
      const uint32_t kraw[4] = {pc.kw[hf].x, pc.kw[hf].y, pc.kw[hf].z, pc.kw[hf].w};
      __nv_bfloat162 kpm[4], qpm[4], kmm[4], qp[4], kr[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float2 cq = *reinterpret_cast<const float2*>(s_ex + 8 * j + 2 * m);
        const float2 cr = *reinterpret_cast<const float2*>(s_ex + kD + 8 * j + 2 * m);
        const float pw0 = ex2f(pc.G[hf][2 * m]), pw1 = ex2f(pc.G[hf][2 * m + 1]);
        const float ip0 = ex2f(-pc.G[hf][2 * m]), ip1 = ex2f(-pc.G[hf][2 * m + 1]);
        const __nv_bfloat162 k2 = *reinterpret_cast<const __nv_bfloat162*>(&kraw[m]);
        const __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162*>(&qraw[m]);
        const float kp0 = rk * pw0, kp1 = rk * pw1, qp0 = rq * pw0, qp1 = rq * pw1, km0 = rk * ip0, km1 = rk * ip1;
        kpm[m] = __hmul2(k2, __floats2bfloat162_rn(kp0, kp1));
        qpm[m] = __hmul2(q2, __floats2bfloat162_rn(qp0, qp1));
        kmm[m] = __hmul2(k2, __floats2bfloat162_rn(km0, km1));
        qp[m] = __hmul2(q2, __floats2bfloat162_rn(qp0 * cq.x, qp1 * cq.y));
        kr[m] = __hmul2(k2, __floats2bfloat162_rn(km0 * cr.x, km1 * cr.y));
      }
      auto as_u4 = [](const __nv_bfloat162(&x)[4]) {
        return make_uint4(*reinterpret_cast<const uint32_t*>(&x[0]), *reinterpret_cast<const uint32_t*>(&x[1]),
                          *reinterpret_cast<const uint32_t*>(&x[2]), *reinterpret_cast<const uint32_t*>(&x[3]));
      };
      *reinterpret_cast<uint4*>(ops + off) = as_u4(kpm);
      *reinterpret_cast<uint4*>(ops + 8192 + off) = as_u4(qpm);
      *reinterpret_cast<uint4*>(ops + 16384 + off) = as_u4(kmm);
      st_global_16(rec_dst + kRecQP + off, as_u4(qp));
      st_global_16(rec_dst + kRecKR + off, as_u4(kr));
    }
  }
}

// The serial part on one warp: A (lanes 0-31 of tensor memory at taddr_a, 32 columns) -> fp32 A beta in sA -> T = (I + A)^-1
// in sT (both [32][kLdA]; the upper right block of sA is scratch) -> TB^T bf16 [32][32] in core layout at tbt.
__device__ __forceinline__ void inverse_to_tbt(uint32_t taddr_a, float* sA, float* sT, uint8_t* tbt, float bi, int lane) {
  float* sX = sA + 16;
  {
    uint32_t a0[32];
    tmem_ld32(taddr_a, a0);
    tmem_wait_ld();
#pragma unroll
    for (int q4 = 0; q4 < 8; ++q4) {
      float4 r;
      r.x = (4 * q4 + 0 < lane) ? __uint_as_float(a0[4 * q4 + 0]) * bi : 0.f;
      r.y = (4 * q4 + 1 < lane) ? __uint_as_float(a0[4 * q4 + 1]) * bi : 0.f;
      r.z = (4 * q4 + 2 < lane) ? __uint_as_float(a0[4 * q4 + 2]) * bi : 0.f;
      r.w = (4 * q4 + 3 < lane) ? __uint_as_float(a0[4 * q4 + 3]) * bi : 0.f;
      *reinterpret_cast<float4*>(sA + lane * kLdA + 4 * q4) = r;
    }
  }
  __syncwarp();
  {
    // the two 16 x 16 diagonal blocks by forward substitution, one column of one block per lane
    const int bb = lane >> 4, c = lane & 15;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        if (4 * q4 < i) {
          const float4 a4 = *reinterpret_cast<const float4*>(sA + (bb * 16 + i) * kLdA + bb * 16 + 4 * q4);
          part[q4] = fmaf(a4.x, x[4 * q4], part[q4]);
          part[q4] = fmaf(a4.y, x[4 * q4 + 1], part[q4]);
          part[q4] = fmaf(a4.z, x[4 * q4 + 2], part[q4]);
          part[q4] = fmaf(a4.w, x[4 * q4 + 3], part[q4]);
        }
      }
      x[i] = ((i == c) ? 1.f : 0.f) - ((part[0] + part[1]) + (part[2] + part[3]));
      sT[(bb * 16 + i) * kLdA + bb * 16 + c] = x[i];
    }
  }
  __syncwarp();
  {
    // T_10 = -T_11 (A_10 T_00): two 16x16x16 products in tf32 on mma.sync, fp32 accumulation
    const int g = lane >> 2, t4 = lane & 3;
    auto small_product = [&](const float* A, const float* B, float* D, float sign) {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const int k0 = 8 * ks;
        const uint32_t f0 = to_tf32(A[g * kLdA + k0 + t4]), f1 = to_tf32(A[(g + 8) * kLdA + k0 + t4]);
        const uint32_t f2 = to_tf32(A[g * kLdA + k0 + t4 + 4]), f3 = to_tf32(A[(g + 8) * kLdA + k0 + t4 + 4]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
          mma_tf32_1688(acc[nt], f0, f1, f2, f3, to_tf32(B[(k0 + t4) * kLdA + 8 * nt + g]), to_tf32(B[(k0 + t4 + 4) * kLdA + 8 * nt + g]));
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        *reinterpret_cast<float2*>(D + g * kLdA + 8 * nt + 2 * t4) = make_float2(sign * acc[nt][0], sign * acc[nt][1]);
        *reinterpret_cast<float2*>(D + (g + 8) * kLdA + 8 * nt + 2 * t4) = make_float2(sign * acc[nt][2], sign * acc[nt][3]);
      }
    };
    small_product(sA + 16 * kLdA, sT, sX, 1.f);                      // X = A_10 T_00
    __syncwarp();
    small_product(sT + 16 * kLdA + 16, sX, sT + 16 * kLdA, -1.f);    // T_10 = -T_11 X
  }
  __syncwarp();
  {
    // row `lane` of TB^T: TB^T[c][i] = T[i][c] beta_c (zero above the diagonal), bf16
    uint8_t* row = tbt + (lane >> 3) * 512 + (lane & 7) * 16;
#pragma unroll
    for (int cb = 0; cb < 4; ++cb) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i0 = 8 * cb + 2 * e;
        const float v0 = (i0 >= lane) ? sT[i0 * kLdA + lane] * bi : 0.f;
        const float v1 = (i0 + 1 >= lane) ? sT[(i0 + 1) * kLdA + lane] * bi : 0.f;
        w[e] = pack_bf16(v0, v1);
      }
      *reinterpret_cast<uint4*>(row + cb * 128) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// tril of the 32 fp32 columns a lane read from the M half of the first products -> row `lane` of MQK (bf16, core layout)
__device__ __forceinline__ void mqk_row(const uint32_t (&u)[32], uint8_t* mqk, int lane) {
  uint8_t* mrow = mqk + (lane >> 3) * 512 + (lane & 7) * 16;
#pragma unroll
  for (int cb = 0; cb < 4; ++cb) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = 8 * cb + 2 * e;
      w[e] = pack_bf16((c <= lane) ? __uint_as_float(u[c]) : 0.f, (c + 1 <= lane) ? __uint_as_float(u[c + 1]) : 0.f);
    }
    *reinterpret_cast<uint4*>(mrow + cb * 128) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// (w')^T of channels 32 q .. + 31 (two 16-lane fragments f0, f1: lanes = channels, columns = tokens) -> WP [32 tok][128 k]
// at shared address wp: scaled back from "relative to the sub-block boundary" by s_ex, rounded, transposed by the store
__device__ __forceinline__ void wp_quadrant(const uint32_t (&f0)[16], const uint32_t (&f1)[16], uint32_t wp, const float* s_ex, int q, int lane) {
  const int m = lane >> 3, r = lane & 7;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint32_t(&f)[16] = half ? f1 : f0;
    const int k0 = 32 * q + 16 * half;
    const float ca = s_ex[k0 + (lane >> 2)], cb = s_ex[k0 + 8 + (lane >> 2)];
#pragma unroll
    for (int jp = 0; jp < 2; ++jp) {
      uint32_t w[4];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int jt = 2 * jp + jj;
        w[2 * jj] = pack_bf16(__uint_as_float(f[4 * jt]) * ca, __uint_as_float(f[4 * jt + 1]) * ca);
        w[2 * jj + 1] = pack_bf16(__uint_as_float(f[4 * jt + 2]) * cb, __uint_as_float(f[4 * jt + 3]) * cb);
      }
      const int tok = 8 * (2 * jp + (m >> 1)) + r, kc = k0 + 8 * (m & 1);
      stsm_x4_trans(wp + (tok >> 3) * 2048 + (kc >> 3) * 128 + (tok & 7) * 16, w[0], w[1], w[2], w[3]);
    }
  }
}

// (u')^T of v channel 32 q + lane (32 fp32 columns = tokens) -> its row of UP [128 v][32 tok] (bf16, core layout) at up
__device__ __forceinline__ void up_row(const uint32_t (&u)[32], uint8_t* up, int q, int lane) {
  const int v = 32 * q + lane;
  uint8_t* row = up + (v >> 3) * 512 + (v & 7) * 16;
#pragma unroll
  for (int cb = 0; cb < 4; ++cb)
    *reinterpret_cast<uint4*>(row + cb * 128) =
        make_uint4(pack_bf16(__uint_as_float(u[8 * cb]), __uint_as_float(u[8 * cb + 1])), pack_bf16(__uint_as_float(u[8 * cb + 2]), __uint_as_float(u[8 * cb + 3])),
                   pack_bf16(__uint_as_float(u[8 * cb + 4]), __uint_as_float(u[8 * cb + 5])), pack_bf16(__uint_as_float(u[8 * cb + 6]), __uint_as_float(u[8 * cb + 7])));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up once through the runtime (no link-time dependency on the driver library).
EncodeTiledFn encode_tiled_fn() {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (fn != nullptr) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess ||
      ptr == nullptr) {
    (void)cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  cached.store(fn, std::memory_order_release);
  return fn;
}

// [T_total][H][128] bf16 tensor as a 3-d map (channel, head, token) read in [32 tok][1 head][64 ch] boxes with the
// 128-byte swizzle; tokens past T_total read as zero.
bool make_map(CUtensorMap* map, const void* base, int64_t T_total, int H) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(T_total)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kD) * 2, static_cast<cuuint64_t>(kD) * 2 * static_cast<cuuint64_t>(H)};
  const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(kChunk)};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace prep_tc

// =====================================================================================================================
// The pipelined kernel: a short software pipeline inside each CTA.  Eight element warps do every item's element-wise
// work in lock step, and a ninth warp owns the serial part (A from tensor memory, T = (I + A)^-1, TB^T, issue of the
// second products) of the item the element warps have just left.  Three CTAs per SM, each a loop over items
// blockIdx.x, blockIdx.x + gridDim.x, ...; two 32 KB operand buffers per CTA alternate between consecutive items.
//
//   element warps, iteration i:  wait tiles(i) | sums of squares, gate, running sums | barrier | decayed operands over the
//                                tiles, QP / KR / E to the record | barrier | one thread: first products(i) -> D1[i & 1]
//                                | then item i - 1: wait D2 | WP, UP over the dead QPm / KMm of its buffer, MQK | barrier |
//                                one thread: bulk stores(i - 1), then the tile loads of item i + 1 into that buffer
//   matrix warp, item i:         decode item i + 2 and ask the L2 for its tiles | sigmoid(beta) | wait D1[i & 1] |
//                                A -> T -> TB^T in the dead QPm / KMm of buffer i & 1 | second products(i) -> D2
// What sets the speed is how many element warps of an SM have work at the same time, not the length of any one of
// these chains: a ten-warp form with a warp of its own for every single-thread issue job, a form with three buffers
// and two CTAs per SM, and one with two matrix warps all ran at the same 3.7 to 4.2 thousand cycles per item and SM.
// Tensor memory: D1 twice (its M half is read one iteration later), D2 once (guarded by a "read" barrier).
namespace prep_pipe {

using namespace prep_tc;

constexpr int kElemThreads = 256;
constexpr int kMatrixWarp = 8;
constexpr int kThreads = 288;
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kColD1 = 0;            // 2 buffers x 32 columns: lanes 0-31 A, 32-63 M
constexpr uint32_t kColD2 = 64;           // (w')^T 32 | (u')^T 32
constexpr int kBufBytes = 32768;          // tiles q | k | g | v, then KPm | QPm | KMm | VC (8192 each)
constexpr int kSmBuf = 0;
constexpr int kOffA = 8192;               // inside a buffer after the first products: fp32 A [32][36] over QPm
constexpr int kOffT = 16384;              // fp32 T [32][36] over KMm
constexpr int kOffTbt = 16384 + 6144;     // TB^T bf16 [32][32], core layout
constexpr int kSmMqk = 2 * kBufBytes;     // MQK bf16 [32][32] on its way to the record
constexpr int kSmSsq = kSmMqk + 2048;     // [2][32][4] partial sums of squares
constexpr int kSmEx = kSmSsq + 1024;      // 2 items x [2][128] 2^(sub-block total)
constexpr int kSmInfo = kSmEx + 2048;     // 4 items x {t0, len, h, gc, 2^A_log / 2}
constexpr int kSmBias = kSmInfo + 128;    // 2 items x dt_bias[h][128] (arrives with the tiles)
constexpr int kSmBars = kSmBias + 1024;
constexpr int kSmMisc = kSmBars + 64;
constexpr int kSmemBytes = 71 * 1024;
static_assert(kSmMisc + 16 <= kSmemBytes, "shared memory plan");
static_assert(3 * (kSmemBytes + 1024) <= 227 * 1024, "three CTAs per SM");
static_assert(32 * kLdA * 4 <= 6144, "A and T fit before TB^T");
enum { B_LOAD = 0 /*[2]*/, B_D1 = 2 /*[2]*/, B_D2 = 4, B_D2_READ = 5, B_COUNT = 6 };

struct ItemInfo {
  long long t0;
  int len, h, gc, pad[3];
};
static_assert(sizeof(ItemInfo) == 32, "item info");

__device__ __forceinline__ ItemInfo decode_item(const PrepParams& p, unsigned item) {
  ItemInfo r;
  r.h = static_cast<int>(item % static_cast<unsigned>(p.H));
  r.gc = static_cast<int>(item / static_cast<unsigned>(p.H));
  // half of exp(A_log[h]): the per-head factor of the gate, once per item instead of once per thread
  r.pad[0] = __float_as_int(0.5f * ex2f(__ldg(p.A_log + r.h) * kLog2e));
  r.pad[1] = r.pad[2] = 0;
  if (p.cu_seqlens != nullptr) {
    int lo = 0, hi = p.N - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.chunk_prefix[mid] <= r.gc) lo = mid; else hi = mid - 1;
    }
    long long bos = p.cu_seqlens[lo], eos = p.cu_seqlens[lo + 1];
    bos = bos < 0 ? 0 : (bos > p.T_total ? p.T_total : bos);
    eos = eos < bos ? bos : (eos > p.T_total ? p.T_total : eos);
    r.t0 = bos + static_cast<long long>(r.gc - p.chunk_prefix[lo]) * kChunk;
    const long long rem = eos - r.t0;
    r.len = rem < kChunk ? static_cast<int>(rem) : kChunk;
  } else {
    const unsigned cps = static_cast<unsigned>((p.T + kChunk - 1) / kChunk);
    const unsigned n = static_cast<unsigned>(r.gc) / cps, lc = static_cast<unsigned>(r.gc) - n * cps;
    r.t0 = static_cast<long long>(n) * p.T + static_cast<long long>(lc) * kChunk;
    const long long rem = p.T - static_cast<long long>(lc) * kChunk;
    r.len = rem < kChunk ? static_cast<int>(rem) : kChunk;
  }
  return r;
}

// rendezvous of the element warps; returns whether any of them has given up
__device__ __forceinline__ bool elem_barrier_any(bool failed) {
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(any)
      : "r"(static_cast<uint32_t>(failed))
      : "memory");
  return any != 0;
}

__global__ void __launch_bounds__(kThreads, 3)
prepare_pipe_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_v, const PrepParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kSmMisc + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmMisc);
  auto bar = [&](int i) { return sbase + kSmBars + 8 * i; };
  auto info_of = [&](int it) { return reinterpret_cast<ItemInfo*>(smem + kSmInfo + (it & 3) * 32); };
  float* s_ssq = reinterpret_cast<float*>(smem + kSmSsq);

  const unsigned total_items = static_cast<unsigned>(p.cu_seqlens != nullptr ? p.chunk_prefix[p.N] : p.total_chunks) * static_cast<unsigned>(p.H);
  if (blockIdx.x >= total_items) return;
  const int n_it = static_cast<int>((total_items - blockIdx.x + gridDim.x - 1) / gridDim.x);
  if ((sbase & 1023u) != 0u) {       // the swizzled tiles need this alignment: report instead of computing garbage
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);
    return;
  }

  // the tile loads of one item into one buffer (one thread)
  auto issue_load = [&](int it) {
    const ItemInfo* f = info_of(it);
    const uint32_t full = bar(B_LOAD + (it & 1));
    const uint32_t dst = sbase + kSmBuf + (it & 1) * kBufBytes;
    const int tc = static_cast<int>(f->t0), h = f->h;
    mbar_arrive_expect_tx(full, kBufBytes + 512);
    bulk_g2s(sbase + kSmBias + (it & 1) * 512, p.dt_bias + static_cast<size_t>(h) * kD, 512, full);
    tma_load_3d(dst, &tm_q, 0, h, tc, full);
    tma_load_3d(dst + 4096, &tm_q, 64, h, tc, full);
    tma_load_3d(dst + 8192, &tm_k, 0, h, tc, full);
    tma_load_3d(dst + 12288, &tm_k, 64, h, tc, full);
    tma_load_3d(dst + 16384, &tm_g, 0, h, tc, full);
    tma_load_3d(dst + 20480, &tm_g, 64, h, tc, full);
    tma_load_3d(dst + 24576, &tm_v, 0, h, tc, full);
    tma_load_3d(dst + 28672, &tm_v, 64, h, tc, full);
  };
  // decode item `it` into its info slot and ask the L2 for its tiles (one thread, an iteration ahead of the load)
  auto decode_and_prefetch = [&](int it) {
    const ItemInfo f = decode_item(p, blockIdx.x + static_cast<unsigned>(it) * gridDim.x);
    *info_of(it) = f;
    const int tc = static_cast<int>(f.t0);
    tma_prefetch_3d(&tm_q, 0, f.h, tc);
    tma_prefetch_3d(&tm_q, 64, f.h, tc);
    tma_prefetch_3d(&tm_k, 0, f.h, tc);
    tma_prefetch_3d(&tm_k, 64, f.h, tc);
    tma_prefetch_3d(&tm_g, 0, f.h, tc);
    tma_prefetch_3d(&tm_g, 64, f.h, tc);
    tma_prefetch_3d(&tm_v, 0, f.h, tc);
    tma_prefetch_3d(&tm_v, 64, f.h, tc);
  };

  if (tid == 0) {
    *abort_flag = p.wait_limit_us > 0 ? -p.wait_limit_us : 0;
    mbar_init(bar(B_LOAD), 1);
    mbar_init(bar(B_LOAD + 1), 1);
    mbar_init(bar(B_D1), 1);
    mbar_init(bar(B_D1 + 1), 1);
    mbar_init(bar(B_D2), 1);
    mbar_init(bar(B_D2_READ), 8);
    fence_mbar_init();
    *info_of(0) = decode_item(p, blockIdx.x);
    issue_load(0);
    if (n_it > 1) {
      *info_of(1) = decode_item(p, blockIdx.x + gridDim.x);
      if (!p.first_load_only) issue_load(1);      // (test aid: else a wait that nothing completes)
    }
    if (n_it > 2) decode_and_prefetch(2);
  }
  if (warp == kMatrixWarp) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  if (warp == kMatrixWarp) {
    // ===== matrix warp ====================================================================================================
    int it = 0;
    for (; it < n_it; ++it) {
      const int b = it & 1;
      uint8_t* buf = smem + kSmBuf + b * kBufBytes;
      float* sA = reinterpret_cast<float*>(buf + kOffA);
      float* sT = reinterpret_cast<float*>(buf + kOffT);
      // the load barrier of this item has an arrival by the thread that wrote the item's info: acquire it
      if (!__all_sync(0xffffffffu, mbar_wait_parked(bar(B_LOAD + b), (it >> 1) & 1, abort_flag))) { failed = true; break; }
      // this warp has time to spare: it decodes the item after next and asks the L2 for its tiles (its info slot was
      // last read when item it - 2 went to the record, an iteration ago)
      if (lane == 0 && it >= 1 && it + 2 < n_it) decode_and_prefetch(it + 2);
      __syncwarp();
      const ItemInfo f = *info_of(it);
      const float bi = lane < f.len ? sigmoid_fast(__bfloat162float(p.beta[static_cast<size_t>(f.t0 + lane) * p.H + f.h])) : 0.f;
      if (!__all_sync(0xffffffffu, mbar_wait_parked(bar(B_D1 + b), (it >> 1) & 1, abort_flag))) { failed = true; break; }
      tc_fence_after();
      inverse_to_tbt(tmem + kColD1 + 32 * b, sA, sT, buf + kOffTbt, bi, lane);
      fence_proxy_async_smem();
      __syncwarp();
      // D2 still holds the previous item until the element warps have read it
      if (it >= 1 && !__all_sync(0xffffffffu, mbar_wait_parked(bar(B_D2_READ), (it - 1) & 1, abort_flag))) { failed = true; break; }
      if (lane == 0) {
        constexpr uint32_t idesc2 = umma_idesc_bf16(128, 32, 1, 1);
        tc_fence_after();
        const uint32_t bs = sbase + kSmBuf + b * kBufBytes;
        const uint64_t ak = umma_desc(bs, 2048, 128), av = umma_desc(bs + 24576, 2048, 128);
        const uint64_t bt = umma_desc(bs + kOffTbt, 512, 128);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          umma_ss(tmem + kColD2, ak + ks * 256, bt + ks * 64, idesc2, ks != 0);
          umma_ss(tmem + kColD2 + 32, av + ks * 256, bt + ks * 64, idesc2, ks != 0);
        }
        umma_commit(bar(B_D2));
      }
      __syncwarp();
    }
    if (lane == 0 && it > 0 && (failed || *abort_flag > 0)) {
      // (giving up; every way out of the loop lies before the issue, so items 0 .. it - 1 were issued) the second
      // products issued last: their arrival must land before the barrier's memory goes away
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(bar(B_D2), (it - 1) & 1))
        if (globaltimer_ns() - t0 > 20000000ull) break;
    }
  } else {
    // ===== element warps ==================================================================================================
    const ElementMap em(tid);
    const int q = warp & 3;
    int loads_issued = n_it > 1 ? 2 : 1;     // (thread 0)

    // item jt (the previous iteration's): WP, UP, MQK out of tensor memory, then to the record; the thread that stores
    // them goes on to load the item after next into the buffer this frees
    auto output = [&](int jt) {
      const int pb = jt & 1;
      uint8_t* buf = smem + kSmBuf + pb * kBufBytes;
      const float* s_ex = reinterpret_cast<const float*>(smem + kSmEx + pb * 1024);
      const bool ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(B_D2), jt & 1, abort_flag));
      if (!ok) {
        failed = true;
      } else {
        tc_fence_after();
        const uint32_t tq = tmem + (static_cast<uint32_t>(q * 32) << 16) + kColD2;
        if (warp < 4) {
          uint32_t f0[16], f1[16];
          tmem_ld_16x256b_x4(tq, f0);
          tmem_ld_16x256b_x4(tq + (16u << 16), f1);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_D2_READ));
          wp_quadrant(f0, f1, sbase + kSmBuf + pb * kBufBytes + 8192, s_ex, q, lane);
        } else {
          uint32_t u[32];
          tmem_ld32(tq + 32, u);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_D2_READ));
          up_row(u, buf + 16384, q, lane);
          if (warp == 5) {
            // tril(q+ k-^T) -> MQK (lanes 32-63 of D1; complete since before the second products were issued)
            if (__all_sync(0xffffffffu, mbar_wait_parked(bar(B_D1 + pb), (jt >> 1) & 1, abort_flag))) {
              tc_fence_after();
              tmem_ld32(tmem + (32u << 16) + kColD1 + 32 * pb, u);
              tmem_wait_ld();
              tc_fence_before();
              mqk_row(u, smem + kSmMqk, lane);
            } else {
              failed = true;
            }
          }
        }
      }
      fence_proxy_async_smem();
      const bool any = elem_barrier_any(failed);
      if (tid == 0 && !any) {
        const ItemInfo* f = info_of(jt);
        uint8_t* const rec = p.records + (static_cast<size_t>(f->h) * p.total_chunks + f->gc) * kRecBytes;
        const uint32_t bs = sbase + kSmBuf + pb * kBufBytes;
        bulk_s2g(rec + kRecMQK, sbase + kSmMqk, 2048);
        bulk_s2g(rec + kRecWP, bs + 8192, 8192);
        bulk_s2g(rec + kRecUP, bs + 16384, 8192);
        bulk_commit();
        bulk_wait_read0();
        if (jt + 2 < n_it && !p.first_load_only) {
          issue_load(jt + 2);
          ++loads_issued;
        }
      }
      return any;
    };

    bool any = false;
    int it = 0;
    for (; it <= n_it && !any; ++it) {
      if (it < n_it) {
      const int b = it & 1;
      uint8_t* buf = smem + kSmBuf + b * kBufBytes;
      float* s_ex = reinterpret_cast<float*>(smem + kSmEx + b * 1024);
      if (!mbar_wait_parked(bar(B_LOAD + b), (it >> 1) & 1, abort_flag)) failed = true;
      const ItemInfo f = *info_of(it);
      const int h = f.h, len = f.len;
      const float ha = __int_as_float(f.pad[0]);
      const float4 b0 = *reinterpret_cast<const float4*>(smem + kSmBias + b * 512 + 32 * em.j);
      const float4 b1 = *reinterpret_cast<const float4*>(smem + kSmBias + b * 512 + 32 * em.j + 16);
      uint8_t* const rec_dst = p.records + (static_cast<size_t>(h) * p.total_chunks + f.gc) * kRecBytes;

      // ---- sums of squares, gate and its running sum ----------------------------------------------------------------
      ElementPieces pc;
      element_phase1(buf, s_ssq, s_ex, em, lane, warp, len, ha, b0, b1, p.gate_scale, pc);
      asm volatile("bar.sync 1, 256;" ::: "memory");      // every thread holds its share of the tiles; sums and totals are complete

      // ---- decayed operands over the tiles, record parts that are final now straight to global memory ---------------
      element_phase2(buf, s_ssq, s_ex, rec_dst, em, p.scale, pc);
      fence_proxy_async_smem();
      any = elem_barrier_any(failed);
      if (any) break;
      // ---- first products [A; M] = [KPm; QPm] KMm^T (rows 64-127 of the A operand are KMm and VC: lanes nobody reads) --
      if (tid == 0) {
        constexpr uint32_t idesc1 = umma_idesc_bf16(128, 32, 0, 0);
        tc_fence_after();
        const uint32_t bs = sbase + kSmBuf + b * kBufBytes;
        const uint64_t a = umma_desc(bs, 128, 2048);
        const uint64_t bd = umma_desc(bs + 16384, 128, 2048);
#pragma unroll
        for (int i = 0; i < 8; ++i) umma_ss(tmem + kColD1 + 32 * b, a + i * 16, bd + i * 16, idesc1, i > 0);
        umma_commit(bar(B_D1 + b));
      }
      }
      if (it >= 1) any = output(it - 1);
    }
    if (any) failed = true;
    if (tid == 0 && (failed || *abort_flag > 0)) {
      // wait (bounded) for loads still in flight so that the CTA does not exit under them
      for (int n = loads_issued > 2 ? loads_issued - 2 : 0; n < loads_issued; ++n) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(bar(B_LOAD + (n & 1)), (n >> 1) & 1))
          if (globaltimer_ns() - t0 > 20000000ull) break;
      }
      // ... and for the first products issued last: their arrival must land before the barrier's memory goes away
      // (leaving at the rendezvous, before the issue, keeps `it`; leaving after an output step has advanced it)
      const int issued1 = it < n_it ? it : n_it;
      if (issued1 > 0) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(bar(B_D1 + ((issued1 - 1) & 1)), ((issued1 - 1) >> 1) & 1))
          if (globaltimer_ns() - t0 > 20000000ull) break;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (failed || *abort_flag > 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);
  if (warp == kMatrixWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace prep_pipe

// =====================================================================================================================
// The one-CTA-per-item kernel: eight warps per (chunk, head) item, four CTAs per SM, every warp doing element-wise
// work, phases separated by CTA-wide barriers, on the data path of the kernel above (TMA tile loads, the intra-chunk
// products and w' / u' on tcgen05 with TMEM accumulators, 128 columns per CTA).  Other resident CTAs fill the waits
// of the serial part (first products -> inverse on one warp -> second products).  About a tenth slower than the
// pipelined kernel; no loop, no buffer reuse: the form to compare against.
namespace prep_tc4 {

using namespace prep_tc;

constexpr int kThreads = 256;
constexpr uint32_t kTmemCols = 128;
constexpr unsigned kGridY = 32768;        // chunks of a packed batch per grid row of the y dimension
constexpr uint32_t kColD1 = 0;            // 32 columns: lanes 0-31 A, 32-63 M
constexpr uint32_t kColD2 = 64;           // (w')^T 32 | (u')^T 32
// shared memory (bytes).  [0, 32768): the staged q, k, g, v tiles (two [32 tok][128 B] swizzled halves each), then, once
// every thread holds its share in registers, KPm | QPm | KMm | VC (core layout [32][128], 8192 each); after the first
// products the QPm and KMm regions receive WP and UP.
constexpr int kSmX = 0;
constexpr int kSmA = 32768;                              // fp32 A [32][36]; its unused upper right block holds the merge scratch
constexpr int kSmT = kSmA + 32 * kLdA * 4;               // fp32 T [32][36]
constexpr int kSmTbt = kSmT + 32 * kLdA * 4;             // TB^T bf16 [32][32], core layout
constexpr int kSmMqk = kSmTbt + 2048;                    // MQK bf16 [32][32], core layout
constexpr int kSmSsq = kSmMqk + 2048;                    // [2][32][4] partial sums of squares
constexpr int kSmEx = kSmSsq + 1024;                     // [2][128] 2^(sub-block total)
constexpr int kSmBeta = kSmEx + 1024;                    // [32] sigmoid(beta)
constexpr int kSmBars = kSmBeta + 128;                   // 3 mbarriers
constexpr int kSmMisc = kSmBars + 32;                    // tmem base, abort flag
constexpr int kSmemBytes = 49152;                        // a multiple of 1024: the next CTA's tiles stay 1024-byte aligned
static_assert(kSmMisc + 16 <= kSmemBytes, "shared memory plan");
static_assert(4 * (kSmemBytes + 1024) <= 227 * 1024, "four CTAs per SM");
enum { B_LOAD = 0, B_D1 = 1, B_D2 = 2 };

// Phase timeline of 32 CTAs from the middle of the grid (tuning builds only): entry [cta * 16 + event] = clock64().
#ifdef FKDA_TUNING
#define P4TRACE(ev)                                                                                                    \
  do {                                                                                                                 \
    const unsigned lin_ = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);                              \
    if (trace != nullptr && lin_ >= 16384u && lin_ < 16416u) trace[(lin_ - 16384u) * 16 + (ev)] = clock64();           \
  } while (0)
#else
#define P4TRACE(ev) do { } while (0)
#endif

__global__ void __launch_bounds__(kThreads, 4)
prepare_tc4_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_v, const PrepParams p,
                   long long* trace) {
  (void)trace;
  if (threadIdx.x == 0) P4TRACE(0);
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kSmMisc + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmMisc);
  auto bar = [&](int i) { return sbase + kSmBars + 8 * i; };
  float* s_ssq = reinterpret_cast<float*>(smem + kSmSsq);
  float* s_ex = reinterpret_cast<float*>(smem + kSmEx);
  float* s_beta = reinterpret_cast<float*>(smem + kSmBeta);
  float* sA = reinterpret_cast<float*>(smem + kSmA);
  float* sT = reinterpret_cast<float*>(smem + kSmT);

  // grid: x = head (consecutive CTAs take consecutive heads of the same chunk: adjacent rows in memory); equal
  // lengths: y = chunk of the sequence, z = sequence; cu_seqlens: y + kGridY z = chunk of the packed batch.  No division
  // on the way to the first load: everything up to the set-up barrier is latency that every item pays.
  const int h = static_cast<int>(blockIdx.x);
  const float a_log = __ldg(p.A_log + h);
  const ElementMap em(tid);
  const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * em.j));
  const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.dt_bias + h * kD + 8 * em.j + 4));
  int gc;
  int64_t t0;
  int len;
  if (p.cu_seqlens != nullptr) {
    gc = static_cast<int>(blockIdx.y + blockIdx.z * kGridY);
    if (gc >= p.chunk_prefix[p.N]) return;
    int lo = 0, hi = p.N - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.chunk_prefix[mid] <= gc) lo = mid; else hi = mid - 1;
    }
    int64_t bos = p.cu_seqlens[lo], eos = p.cu_seqlens[lo + 1];
    bos = bos < 0 ? 0 : (bos > p.T_total ? p.T_total : bos);
    eos = eos < bos ? bos : (eos > p.T_total ? p.T_total : eos);
    t0 = bos + static_cast<int64_t>(gc - p.chunk_prefix[lo]) * kChunk;
    const int64_t rem = eos - t0;
    len = rem < kChunk ? static_cast<int>(rem) : kChunk;
  } else {
    const int lc = static_cast<int>(blockIdx.y), n = static_cast<int>(blockIdx.z);
    gc = n * static_cast<int>(gridDim.y) + lc;
    t0 = static_cast<int64_t>(n) * p.T + static_cast<int64_t>(lc) * kChunk;
    const int64_t rem = p.T - static_cast<int64_t>(lc) * kChunk;
    len = rem < kChunk ? static_cast<int>(rem) : kChunk;
  }
  // sigmoid(beta) of the 32 tokens: the load is issued before the serial set-up below, on a warp that has none of it
  float beta_raw = 0.f;
  if (warp == 2 && lane < len) beta_raw = __bfloat162float(p.beta[static_cast<size_t>(t0 + lane) * p.H + h]);
  if ((sbase & 1023u) != 0u) {       // the swizzled tiles need this alignment: report instead of computing garbage
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);
    return;
  }
  uint8_t* const rec_dst = p.records + (static_cast<size_t>(h) * p.total_chunks + gc) * kRecBytes;

  if (tid == 0) {
    mbar_init(bar(B_LOAD), 1);
    mbar_init(bar(B_D1), 1);
    mbar_init(bar(B_D2), 1);
    fence_mbar_init();
    const uint32_t full = bar(B_LOAD);
    mbar_arrive_expect_tx(full, 32768);
    const int tc = static_cast<int>(t0);
    tma_load_3d(sbase + kSmX, &tm_q, 0, h, tc, full);
    tma_load_3d(sbase + kSmX + 4096, &tm_q, 64, h, tc, full);
    tma_load_3d(sbase + kSmX + 8192, &tm_k, 0, h, tc, full);
    tma_load_3d(sbase + kSmX + 12288, &tm_k, 64, h, tc, full);
    tma_load_3d(sbase + kSmX + 16384, &tm_g, 0, h, tc, full);
    tma_load_3d(sbase + kSmX + 20480, &tm_g, 64, h, tc, full);
    tma_load_3d(sbase + kSmX + 24576, &tm_v, 0, h, tc, full);
    tma_load_3d(sbase + kSmX + 28672, &tm_v, 64, h, tc, full);
    P4TRACE(14);
  }
  if (warp == 1) {
    if (lane == 0) *abort_flag = 0;
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 2) s_beta[lane] = lane < len ? sigmoid_fast(beta_raw) : 0.f;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;
  if (tid == 0) P4TRACE(13);

  // ---- P1: staged tiles -> registers, partial sums of squares, gate and its running sum ----------------------------
  if (!mbar_wait_parked(bar(B_LOAD), 0, abort_flag)) failed = true;
  if (tid == 0) P4TRACE(1);
  ElementPieces pc;
  element_phase1(smem + kSmX, s_ssq, s_ex, em, lane, warp, len, 0.5f * ex2f(a_log * kLog2e), b0, b1, p.gate_scale, pc);
  __syncthreads();      // every thread holds its share of the tiles; sums of squares and sub-block totals are complete
  if (tid == 0) P4TRACE(2);

  // ---- P2: decayed operands over the staging area, record parts that are final now straight to global memory ------
  element_phase2(smem + kSmX, s_ssq, s_ex, rec_dst, em, p.scale, pc);
  fence_proxy_async_smem();
  __syncthreads();
  if (tid == 0) P4TRACE(3);

  // ---- first products [A; M] = [KPm; QPm] KMm^T (rows 64-127 of the A operand are KMm and VC: lanes nobody reads) --
  if (tid == 0 && !failed) {
    constexpr uint32_t idesc1 = umma_idesc_bf16(128, 32, 0, 0);
    tc_fence_after();
    const uint64_t a = umma_desc(sbase + kSmX, 128, 2048);
    const uint64_t b = umma_desc(sbase + kSmX + 16384, 128, 2048);
#pragma unroll
    for (int i = 0; i < 8; ++i) umma_ss(tmem + kColD1, a + i * 16, b + i * 16, idesc1, i > 0);
    umma_commit(bar(B_D1));
    P4TRACE(4);
  }
  if (warp == 0) {
    // ---- T = (I + A)^-1 and TB^T on one warp -------------------------------------------------------------------------
    const bool ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(B_D1), 0, abort_flag));
    if (ok) {
      tc_fence_after();
      if (lane == 0) P4TRACE(5);
      inverse_to_tbt(tmem + kColD1, sA, sT, smem + kSmTbt, s_beta[lane], lane);
      fence_proxy_async_smem();
      if (lane == 0) P4TRACE(8);
    } else {
      failed = true;
    }
  } else if (warp == 1) {
    // ---- tril(q+ k-^T) -> MQK ------------------------------------------------------------------------------------------
    const bool ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(B_D1), 0, abort_flag));
    if (ok) {
      tc_fence_after();
      uint32_t a0[32];
      tmem_ld32(tmem + (32u << 16) + kColD1, a0);
      tmem_wait_ld();
      mqk_row(a0, smem + kSmMqk, lane);
      fence_proxy_async_smem();
    } else {
      failed = true;
    }
  }
  tc_fence_before();
  __syncthreads();

  // ---- second products (w')^T = KPm^T TB^T, (u')^T = VC^T TB^T -----------------------------------------------------------
  if (tid == 0 && !failed && *abort_flag <= 0) {
    constexpr uint32_t idesc2 = umma_idesc_bf16(128, 32, 1, 1);
    tc_fence_after();
    const uint64_t ak = umma_desc(sbase + kSmX, 2048, 128), av = umma_desc(sbase + kSmX + 24576, 2048, 128);
    const uint64_t bt = umma_desc(sbase + kSmTbt, 512, 128);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      umma_ss(tmem + kColD2, ak + ks * 256, bt + ks * 64, idesc2, ks != 0);
      umma_ss(tmem + kColD2 + 32, av + ks * 256, bt + ks * 64, idesc2, ks != 0);
    }
    umma_commit(bar(B_D2));
    P4TRACE(9);
  }
  {
    // ---- output: warps 0-3 turn (w')^T into WP (over the QPm region), warps 4-7 (u')^T into UP (over the KMm region) ---
    const bool ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(B_D2), 0, abort_flag));
    const int q = warp & 3;
    const uint32_t tq = tmem + (static_cast<uint32_t>(q * 32) << 16) + kColD2;
    if (tid == 0) P4TRACE(10);
    if (!ok) {
      failed = true;
    } else if (warp < 4) {
      tc_fence_after();
      uint32_t f0[16], f1[16];
      tmem_ld_16x256b_x4(tq, f0);
      tmem_ld_16x256b_x4(tq + (16u << 16), f1);
      tmem_wait_ld();
      wp_quadrant(f0, f1, sbase + kSmX + 8192, s_ex, q, lane);
    } else {
      tc_fence_after();
      uint32_t u[32];
      tmem_ld32(tq + 32, u);
      tmem_wait_ld();
      up_row(u, smem + kSmX + 16384, q, lane);
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) P4TRACE(11);
  if (tid == 0 && !failed && *abort_flag <= 0) {
    bulk_s2g(rec_dst + kRecMQK, sbase + kSmMqk, 2048);
    bulk_s2g(rec_dst + kRecWP, sbase + kSmX + 8192, 8192);
    bulk_s2g(rec_dst + kRecUP, sbase + kSmX + 16384, 8192);
    bulk_commit();
    bulk_wait_read0();
    P4TRACE(12);
  }
  if (failed || *abort_flag > 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace prep_tc4

cudaError_t launch_prepare_pipe(const PrepParams& p, cudaStream_t stream) {
  if (p.total_chunks == 0 || p.H == 0 || p.T_total == 0) return cudaSuccess;
  CUtensorMap tq, tk, tg, tv;
  if (!prep_tc::make_map(&tq, p.q, p.T_total, p.H) || !prep_tc::make_map(&tk, p.k, p.T_total, p.H) ||
      !prep_tc::make_map(&tg, p.g, p.T_total, p.H) || !prep_tc::make_map(&tv, p.v, p.T_total, p.H))
    return cudaErrorInvalidValue;
  static SmemOptIn opt_in;
  cudaError_t e = opt_in.ensure(prep_pipe::prepare_pipe_kernel, prep_pipe::kSmemBytes);
  if (e != cudaSuccess) return e;
  const long long items = static_cast<long long>(p.total_chunks) * p.H;
  const long long slots = 3ll * device_sm_count();
  const unsigned grid = static_cast<unsigned>(items < slots ? items : slots);
  prep_pipe::prepare_pipe_kernel<<<grid, prep_pipe::kThreads, prep_pipe::kSmemBytes, stream>>>(tq, tk, tg, tv, p);
  return cudaGetLastError();
}

// whether the grid of the kernel above can hold the call (x = heads; equal lengths: y = chunks of a sequence,
// z = sequences; packed batch: y + kGridY z = chunk)
bool prepare_tc4_applicable(const PrepParams& p) {
  if (p.H > 65535) return false;
  if (p.cu_seqlens == nullptr) return (p.T + kChunk - 1) / kChunk <= 65535 && p.N <= 65535;
  return (static_cast<long long>(p.total_chunks) + prep_tc4::kGridY - 1) / prep_tc4::kGridY <= 65535;
}

cudaError_t launch_prepare_tc4(const PrepParams& p, cudaStream_t stream) {
  if (p.total_chunks == 0 || p.H == 0 || p.T_total == 0) return cudaSuccess;
  CUtensorMap tq, tk, tg, tv;
  if (!prep_tc::make_map(&tq, p.q, p.T_total, p.H) || !prep_tc::make_map(&tk, p.k, p.T_total, p.H) ||
      !prep_tc::make_map(&tg, p.g, p.T_total, p.H) || !prep_tc::make_map(&tv, p.v, p.T_total, p.H))
    return cudaErrorInvalidValue;
  static SmemOptIn opt_in;
  cudaError_t e = opt_in.ensure(prep_tc4::prepare_tc4_kernel, prep_tc4::kSmemBytes);
  if (e != cudaSuccess) return e;
  if (!prepare_tc4_applicable(p)) return cudaErrorInvalidConfiguration;
  dim3 grid;
  if (p.cu_seqlens == nullptr) {
    grid = dim3(static_cast<unsigned>(p.H), static_cast<unsigned>((p.T + kChunk - 1) / kChunk), static_cast<unsigned>(p.N));
  } else {
    const unsigned chunks = static_cast<unsigned>(p.total_chunks);
    grid = dim3(static_cast<unsigned>(p.H), chunks < prep_tc4::kGridY ? chunks : prep_tc4::kGridY, (chunks + prep_tc4::kGridY - 1) / prep_tc4::kGridY);
  }
#ifdef FKDA_TUNING
  long long* trace = prep_tc::g_trace;
#else
  long long* trace = nullptr;
#endif
  prep_tc4::prepare_tc4_kernel<<<grid, prep_tc4::kThreads, prep_tc4::kSmemBytes, stream>>>(tq, tk, tg, tv, p, trace);
  return cudaGetLastError();
}

#ifdef FKDA_TUNING
void set_prepare_trace(long long* buf) { prep_tc::g_trace = buf; }
#endif

}  // namespace fkda
