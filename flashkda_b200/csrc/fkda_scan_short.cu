// Inter-chunk recurrence for SHORT chains (fixed-length batches of at most two 32-token chunks per sequence,
// e.g. continuation of many sequences by a few tokens).  Such a call is dominated by moving the 128x128 state in
// and out (64 KB each way per chain in fp32), not by the recurrence, so this kernel is built for throughput over
// chains rather than latency along one: persistent CTAs walk chains round-robin, the next chain's state and operand
// record are fetched by bulk async copies while the current chain computes, and the final state leaves through
// bulk stores that overlap with the next chain.
//
// Replaces, for these shapes, the same part of the reference as the other scan kernels
// (csrc/smxx/fwd_kernel2.cuh:115-839; its state load/convert :239-318 and final-state store :786-835 are what
// dominate there).  Per chunk, with S^T in tensor memory (lanes = v, columns = k):
//     [W^T | O^T] = Sb [wp; qp]^T           Sb = bf16 copy of S^T (A operand from tensor memory), N = 64
//     U^T = up^T - W^T                      -> bf16 A operand in tensor memory
//     S^T = S^T diag(e) + U^T kr ;  O^T += U^T mqk^T
//
// Warp roles (512 threads): 0 = record producer, 1 = MMA issuer and TMEM owner, 2-3 idle, 4-11 = state warps (two
// groups of four; group g owns state columns [64g, 64g+64); group 0 also forms U), 12-15 = output warps.
// All barriers run on through the chains; every role counts chunks and chains the same way.  Every wait is bounded.
#include "fkda_common.cuh"

namespace fkda {
namespace scan_short {

constexpr int kThreads = 16 * 32;
constexpr int kRing = 2;                         // operand records in flight
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0;                    // 128 fp32
constexpr uint32_t kColWO = 128;                 // 64: W^T (32) | O^T (32)
constexpr uint32_t kColSb = 192;                 // 64: bf16 pairs of S^T
constexpr uint32_t kColUt = 256;                 // 16: bf16 pairs of U^T

constexpr int kRowStride = 528;                  // bytes per staged state row (512 + 16: conflict-free row reads)
constexpr int kStateStg = 128 * kRowStride;      // 67584
constexpr int kSmRec = 0;                        // kRing records
constexpr int kSmState = kSmRec + kRing * kRecBytes;       // 2 staging buffers
constexpr int kSmOutStg = kSmState + 2 * kStateStg;        // 4 warps x [32 tok][32 v] bf16
constexpr int kSmBars = kSmOutStg + 4 * 2048;
constexpr int kSmMisc = kSmBars + 128;
constexpr int kSmemBytes = kSmMisc + 64 + 1024;

enum { BAR_FULL = 0, BAR_EMPTY = 2, BAR_STFULL = 4, BAR_WFULL = 6, BAR_OFULL, BAR_SFULL, BAR_UREADY, BAR_SBREADY, BAR_OFREE, BAR_COUNT };

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t backoff_ns = 0) {
  const bool ok = mbar_wait(bar, parity, abort_flag, backoff_ns);
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ void pack32(const uint32_t (&x)[32], uint32_t (&y)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) y[i] = pack_bf16(__uint_as_float(x[2 * i]), __uint_as_float(x[2 * i + 1]));
}
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1) scan_short_kernel(const ScanParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kSmMisc + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmMisc);
  auto bar = [&](int i) { return sbase + kSmBars + 8 * i; };

  // fixed-length only: every chain has the same number of chunks
  const int nchunks = static_cast<int>((p.T + kChunk - 1) / kChunk);
  const int nchains = p.N * p.H;
  const int first = blockIdx.x, step = gridDim.x;
  const int my_chains = first < nchains ? (nchains - first + step - 1) / step : 0;
  const bool has_in = p.initial_state != nullptr;
  const uint32_t row_bytes = p.state_fp32 ? 512u : 256u;      // one state row in global memory

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kRing; ++s) {
      mbar_init(bar(BAR_FULL + s), 1);
      mbar_init(bar(BAR_EMPTY + s), 1 + 8);     // MMA commit + state warps
      mbar_init(bar(BAR_STFULL + s), 8);        // one arrive.expect_tx per state warp
    }
    mbar_init(bar(BAR_WFULL), 1);
    mbar_init(bar(BAR_OFULL), 1);
    mbar_init(bar(BAR_SFULL), 1);
    mbar_init(bar(BAR_UREADY), 4);
    mbar_init(bar(BAR_SBREADY), 8);
    mbar_init(bar(BAR_OFREE), 4);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  auto chain_of = [&](int i) { return first + i * step; };
  auto rec_ptr = [&](int chain, int c) {
    const int n = chain / p.H, h = chain - n * p.H;
    return p.records + (static_cast<size_t>(h) * p.total_chunks + static_cast<size_t>(n) * nchunks + c) * kRecBytes;
  };

  if (warp == 0) {
    // ===== record producer: global chunk counter g runs over all chunks of all of this CTA's chains ============
    if (lane == 0) {
      int g = 0;
      for (int i = 0; i < my_chains && !failed; ++i)
        for (int c = 0; c < nchunks; ++c, ++g) {
          const int s = g % kRing, k = g / kRing;
          if (k > 0 && !mbar_wait(bar(BAR_EMPTY + s), (k - 1) & 1, abort_flag, 32)) { failed = true; break; }
          mbar_arrive_expect_tx(bar(BAR_FULL + s), kRecBytes);
          bulk_g2s(sbase + kSmRec + s * kRecBytes, rec_ptr(chain_of(i), c), kRecBytes, bar(BAR_FULL + s));
        }
      if (failed || *abort_flag > 0) {
        // wait (bounded) for the copies still in flight, so that the CTA does not exit under them
        for (int j = g > kRing ? g - kRing : 0; j < g; ++j) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(bar(BAR_FULL + j % kRing), (j / kRing) & 1))
            if (globaltimer_ns() - t0 > 20000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer ==========================================================================================
    if (lane == 0) {
      constexpr uint32_t idesc_n32 = umma_idesc_bf16(128, 32, 0, 0);
      constexpr uint32_t idesc_n64 = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_n128_bmn = umma_idesc_bf16(128, 128, 0, 1);
      const int total = my_chains * nchunks;
      for (int g = 0; g < total; ++g) {
        const int s = g % kRing, k = g / kRing;
        const uint32_t rec = sbase + kSmRec + s * kRecBytes;
        if (!mbar_wait(bar(BAR_FULL + s), k & 1, abort_flag)) { failed = true; break; }
        if (!mbar_wait(bar(BAR_SBREADY), g & 1, abort_flag)) { failed = true; break; }
        if (g > 0 && !mbar_wait(bar(BAR_OFREE), (g - 1) & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const uint64_t bw = umma_desc(rec + kRecWP, 128, 2048);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ts(tmem + kColWO, tmem + kColSb + ks * 8, bw + ks * 16, idesc_n64, ks > 0);
        umma_commit(bar(BAR_WFULL));
        if (!mbar_wait(bar(BAR_UREADY), g & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        const uint64_t bk = umma_desc(rec + kRecKR, 2048, 128);
        umma_ts(tmem + kColS, tmem + kColUt, bk, idesc_n128_bmn, 1);
        umma_ts(tmem + kColS, tmem + kColUt + 8, bk + 256, idesc_n128_bmn, 1);
        umma_commit(bar(BAR_SFULL));
        const uint64_t bm = umma_desc(rec + kRecMQK, 128, 512);
        umma_ts(tmem + kColWO + 32, tmem + kColUt, bm, idesc_n32, 1);
        umma_ts(tmem + kColWO + 32, tmem + kColUt + 8, bm + 16, idesc_n32, 1);
        umma_commit(bar(BAR_OFULL));
        umma_commit(bar(BAR_EMPTY + s));
      }
      if (!failed && total > 0) {
        const int g = total - 1;
        if (!mbar_wait(bar(BAR_EMPTY + g % kRing), (g / kRing) & 1, abort_flag)) failed = true;
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ===== state warps ===========================================================================================
    const int grp = (warp - 4) >> 2;
    const int qd = warp & 3;
    const int v = qd * 32 + lane;
    const uint32_t tq = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    const uint32_t half_bytes = row_bytes >> 1;                  // this lane's half row: 64 state values
    auto stg_row = [&](int buf) { return smem + kSmState + buf * kStateStg + v * kRowStride + grp * half_bytes; };
    auto state_gptr = [&](const void* base, int chain) {
      return reinterpret_cast<const uint8_t*>(base) + (static_cast<size_t>(chain) * kD + v) * row_bytes + grp * half_bytes;
    };
    auto fetch_state = [&](int i) {       // bulk-load this lane's half row of chain i into staging buffer i & 1
      const int buf = i & 1;
      if (lane == 0) mbar_arrive_expect_tx(bar(BAR_STFULL + buf), has_in ? 32 * half_bytes : 0);
      __syncwarp();
      if (has_in) bulk_g2s(smem_u32(stg_row(buf)), state_gptr(p.initial_state, chain_of(i)), half_bytes, bar(BAR_STFULL + buf));
    };
    int g = 0;
    int fetched = 0, consumed = 0;      // incoming states asked for / arrived and waited for
    if (my_chains > 0) { fetch_state(0); fetched = 1; }
    for (int i = 0; i < my_chains && !failed; ++i) {
      const int buf = i & 1;
      if (i + 1 < my_chains) {
        bulk_wait_read_all();            // this lane's final-state store out of the other buffer (chain i-1) has been read
        fetch_state(i + 1);
        fetched = i + 2;
      }
      if (!warp_wait(bar(BAR_STFULL + buf), (i >> 1) & 1, abort_flag)) { failed = true; break; }
      consumed = i + 1;
      if (!warp_wait(bar(BAR_FULL + g % kRing), (g / kRing) & 1, abort_flag)) { failed = true; break; }
      // ---- initial state -> TMEM: bf16 copy (undecayed) and fp32 pre-decayed by the first chunk's e --------------
      {
        const float* e0 = reinterpret_cast<const float*>(smem + kSmRec + (g % kRing) * kRecBytes + kRecE) + 64 * grp;
        const float e_l = e0[lane], e_h = e0[32 + lane];
        const uint8_t* row = stg_row(buf);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t x[32], y[16];
          if (!has_in) {
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] = 0u;
          } else if (p.state_fp32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 w = *reinterpret_cast<const uint4*>(row + half * 128 + j * 16);
              x[4 * j] = w.x; x[4 * j + 1] = w.y; x[4 * j + 2] = w.z; x[4 * j + 3] = w.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 w = *reinterpret_cast<const uint4*>(row + half * 64 + j * 16);
              x[8 * j] = w.x << 16; x[8 * j + 1] = w.x & 0xffff0000u; x[8 * j + 2] = w.y << 16; x[8 * j + 3] = w.y & 0xffff0000u;
              x[8 * j + 4] = w.z << 16; x[8 * j + 5] = w.z & 0xffff0000u; x[8 * j + 6] = w.w << 16; x[8 * j + 7] = w.w & 0xffff0000u;
            }
          }
          pack32(x, y);
          tmem_st16(tq + kColSb + 32 * grp + 16 * half, y);
#pragma unroll
          for (int j = 0; j < 32; ++j) x[j] = __float_as_uint(__uint_as_float(x[j]) * __shfl_sync(0xffffffffu, half ? e_h : e_l, j));
          tmem_st32(tq + kColS + 64 * grp + 32 * half, x);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_SBREADY));
      }
      for (int c = 0; c < nchunks && !failed; ++c, ++g) {
        const int s = g % kRing;
        const uint8_t* rec = smem + kSmRec + s * kRecBytes;
        if (grp == 0) {
          // ---- U epilogue (group 0): U^T = up^T - W^T as a bf16 operand in tensor memory --------------------------
          if (!warp_wait(bar(BAR_WFULL), g & 1, abort_flag)) { failed = true; break; }
          tc_fence_after();
          uint32_t w[32], y[16];
          tmem_ld32(tq + kColWO, w);
          const uint8_t* up_row = rec + kRecUP + (v >> 3) * 512 + (v & 7) * 16;
          uint4 t[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) t[j] = *reinterpret_cast<const uint4*>(up_row + j * 128);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            y[4 * j + 0] = pack_bf16(bf_lo(t[j].x) - __uint_as_float(w[8 * j + 0]), bf_hi(t[j].x) - __uint_as_float(w[8 * j + 1]));
            y[4 * j + 1] = pack_bf16(bf_lo(t[j].y) - __uint_as_float(w[8 * j + 2]), bf_hi(t[j].y) - __uint_as_float(w[8 * j + 3]));
            y[4 * j + 2] = pack_bf16(bf_lo(t[j].z) - __uint_as_float(w[8 * j + 4]), bf_hi(t[j].z) - __uint_as_float(w[8 * j + 5]));
            y[4 * j + 3] = pack_bf16(bf_lo(t[j].w) - __uint_as_float(w[8 * j + 6]), bf_hi(t[j].w) - __uint_as_float(w[8 * j + 7]));
          }
          tmem_st16(tq + kColUt, y);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(BAR_UREADY));
        }
        const bool last = (c + 1 == nchunks);
        float e_l = 1.f, e_h = 1.f;
        if (!last) {   // decay factors of the next chunk of this chain (its record is the next one in the ring)
          if (!warp_wait(bar(BAR_FULL + (g + 1) % kRing), ((g + 1) / kRing) & 1, abort_flag)) { failed = true; break; }
          const float* e = reinterpret_cast<const float*>(smem + kSmRec + ((g + 1) % kRing) * kRecBytes + kRecE) + 64 * grp;
          e_l = e[lane];
          e_h = e[32 + lane];
        }
        if (!warp_wait(bar(BAR_SFULL), g & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        if (lane == 0) mbar_arrive(bar(BAR_EMPTY + s));     // e of this record was read at the previous step
        uint32_t x0[32], x1[32];
        tmem_ld32(tq + kColS + 64 * grp, x0);
        tmem_ld32(tq + kColS + 64 * grp + 32, x1);
        tmem_wait_ld();
        if (!last) {
          // ---- S epilogue: bf16 copy of the new state, then pre-decay for the next chunk ---------------------------
          uint32_t y[16];
          pack32(x0, y);
          tmem_st16(tq + kColSb + 32 * grp, y);
#pragma unroll
          for (int j = 0; j < 32; ++j) x0[j] = __float_as_uint(__uint_as_float(x0[j]) * __shfl_sync(0xffffffffu, e_l, j));
          tmem_st32(tq + kColS + 64 * grp, x0);
          pack32(x1, y);
          tmem_st16(tq + kColSb + 32 * grp + 16, y);
#pragma unroll
          for (int j = 0; j < 32; ++j) x1[j] = __float_as_uint(__uint_as_float(x1[j]) * __shfl_sync(0xffffffffu, e_h, j));
          tmem_st32(tq + kColS + 64 * grp + 32, x1);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(BAR_SBREADY));
        } else if (p.final_state != nullptr) {
          // ---- final state: registers -> this chain's staging rows -> one bulk store per lane ------------------------
          uint8_t* row = stg_row(buf);
          if (p.state_fp32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              *reinterpret_cast<uint4*>(row + j * 16) = make_uint4(x0[4 * j], x0[4 * j + 1], x0[4 * j + 2], x0[4 * j + 3]);
              *reinterpret_cast<uint4*>(row + 128 + j * 16) = make_uint4(x1[4 * j], x1[4 * j + 1], x1[4 * j + 2], x1[4 * j + 3]);
            }
          } else {
            uint32_t y[16];
            pack32(x0, y);
#pragma unroll
            for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(row + j * 16) = make_uint4(y[4 * j], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]);
            pack32(x1, y);
#pragma unroll
            for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(row + 64 + j * 16) = make_uint4(y[4 * j], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]);
          }
          fence_proxy_async_smem();
          bulk_s2g(const_cast<uint8_t*>(state_gptr(p.final_state, chain_of(i))), smem_u32(row), half_bytes);
          bulk_commit();
        }
      }
    }
    if (failed) {
      // state copies asked for and never waited for: let them land (bounded) before the CTA may exit
      for (int j = consumed; j < fetched; ++j) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(bar(BAR_STFULL + (j & 1)), (j >> 1) & 1))
          if (globaltimer_ns() - t0 > 20000000ull) break;
      }
    }
    bulk_wait_read_all();
  } else if (warp >= 12) {
    // ===== output warps =============================================================================================
    const int qd = warp & 3;
    const uint32_t tq = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + kSmOutStg + qd * 2048);
    int g = 0;
    for (int i = 0; i < my_chains && !failed; ++i) {
      const int chain = chain_of(i);
      const int n = chain / p.H, h = chain - n * p.H;
      for (int c = 0; c < nchunks; ++c, ++g) {
        if (!warp_wait(bar(BAR_OFULL), g & 1, abort_flag, 32)) { failed = true; break; }
        tc_fence_after();
        uint32_t o[32];
        tmem_ld32(tq + kColWO + 32, o);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_OFREE));
#pragma unroll
        for (int j = 0; j < 32; ++j) stg[j * 32 + lane] = __float2bfloat16_rn(__uint_as_float(o[j]));
        __syncwarp();
        const int64_t tok0 = static_cast<int64_t>(n) * p.T + static_cast<int64_t>(c) * kChunk;
        const int64_t rem = p.T - static_cast<int64_t>(c) * kChunk;
        const int valid = rem < kChunk ? static_cast<int>(rem) : kChunk;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = j * 8 + (lane >> 2), c8 = (lane & 3) * 8;
          if (r < valid) {
            const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 32 + c8);
            *reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(tok0 + r) * p.H + h) * kD + qd * 32 + c8) = val;
          }
        }
        __syncwarp();
      }
    }
  }

  if (failed || *abort_flag > 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace scan_short

cudaError_t launch_scan_short(const ScanParams& p, int sm_count, cudaStream_t stream) {
  static SmemOptIn opt_in;
  cudaError_t e = opt_in.ensure(scan_short::scan_short_kernel, scan_short::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int64_t chains = static_cast<int64_t>(p.N) * p.H;
  if (chains == 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>(chains < sm_count ? chains : sm_count);
  scan_short::scan_short_kernel<<<grid, scan_short::kThreads, scan_short::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fkda
