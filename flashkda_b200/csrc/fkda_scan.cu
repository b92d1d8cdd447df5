// Inter-chunk recurrence of the KDA prefill, compact form: one CTA walks the chunks of one (sequence, head)
// chain with the 128x128 fp32 state resident in tensor memory, and two such CTAs share an SM.
//
// Replaces the reference's K2 (csrc/smxx/fwd_kernel2.cuh:115-839) for batches with more chains than SMs: every chain is a serial loop that leaves the SM idle most of the time, so two independent chains per SM
// nearly double the throughput, where the look-ahead kernel (fkda_scan2.cu), which shortens the loop of one chain
// per SM, would run the chains in more waves.  It is also the cross-check of the other recurrence kernels (flag
// FKDA_FLAG_SCAN_PLAIN).  Per 32-token chunk, with S the state at the chunk start held as S^T [v lanes][k columns]:
//     [W^T | O^T] = Sb [wp; qp]^T      tcgen05.mma  M=128 (v), N=64 (tokens of w' and of q+), K=128, A = bf16 copy of S in TMEM
//     U^T  = up^T - W^T                warps: TMEM -> registers -> bf16 operand in shared memory
//     S^T  = S^T diag(e) + U^T kr      tcgen05.mma  M=128, N=128 (k), K=32, accumulating in TMEM
//     O^T += U^T mqk^T                 tcgen05.mma  M=128, N=32, K=32
// The decay diag(e) and the bf16 operand copy of S are produced by one TMEM round trip per chunk.  Operand records
// arrive by bulk async copies through a 2-stage mbarrier ring.  Half of an SM: 256 TMEM columns, 88 KB of shared
// memory, 320 threads of at most 102 registers.
//
// Warp roles (320 threads): warp 0 = copy producer, warp 1 = MMA issuer (+ TMEM owner),
// warps 2-5 = state warps (U and S epilogues), warps 6-9 = output warps.  Each group of four
// consecutive warps covers the four TMEM lane quadrants (quadrant = warp index mod 4).
// Every wait is bounded; a wait that gives up raises an abort flag, records a status code and
// lets all roles fall through to the common exit, where TMEM is released.
#include "fkda_common.cuh"

namespace fkda {

constexpr int kStages = 2;
constexpr int kScanThreads = 320;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColW = 128, kColO = 160, kColSbd = 192;   // [W | O] adjacent: one N = 64 product; Sbd: two k per column

// shared-memory plan (byte offsets from a 1024-byte aligned base)
constexpr int kSmStage = 0;                                  // kStages records
constexpr int kSmUt = kSmStage + kStages * kRecBytes;        // [128 v][32 tok] bf16 U^T (core layout)
constexpr int kSmOutStg = kSmUt + 8192;                      // 4 warps x [32 tok][32 v] bf16 staging for out
constexpr int kSmBars = kSmOutStg + 4 * 2048;                // mbarriers
constexpr int kSmMisc = kSmBars + 128;                       // tmem base, abort flag
constexpr int kScanSmemBytes = kSmMisc + 64 + 1024;          // + slack for manual 1024-byte alignment
static_assert(2 * (kScanSmemBytes + 1024) <= 227 * 1024, "two CTAs per SM");

// mbarrier slots
enum { BAR_FULL = 0, BAR_EMPTY = BAR_FULL + kStages, BAR_WFULL = BAR_EMPTY + kStages, BAR_OFULL, BAR_SFULL, BAR_UREADY, BAR_SBREADY,
       BAR_OFREE, BAR_COUNT };
static_assert(BAR_COUNT * 8 <= 128, "barrier area");

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

// kSeg: CTAs walk runs of a sequence (segment-parallel form, see fkda_segscan.cu) instead of whole sequences
template <bool kSeg>
__global__ void __launch_bounds__(kScanThreads, 2) scan_kernel(const ScanParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kSmMisc + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmMisc);
  auto bar = [&](int i) { return sbase + kSmBars + 8 * i; };

  if (p.select != nullptr && *p.select != p.select_want) return;     // the other recurrence kernel was chosen
  // ---- chain -> tokens and records ---------------------------------------------------------------------
  const ChainView cv = chain_view<kSeg>(p, blockIdx.x);
  const int h = cv.h;
  const int64_t bos = cv.bos, eos = cv.eos;
  const int nchunks = cv.nchunks;
  const uint8_t* rec0 = p.records + (static_cast<size_t>(h) * p.total_chunks + cv.chunk_base) * kRecBytes;

  // The incoming state is read row by row in four dependent round trips further down: ask for its lines now, so that
  // those reads find them in the L2 (state warps: lane = row, 512 B or 256 B per row).
  if (warp >= 2 && warp < 6 && (cv.init_mode == 1 || cv.init_mode == 2)) {
    const int v = (warp & 3) * 32 + lane;
    const uint8_t* row = static_cast<const uint8_t*>(cv.init_base) + static_cast<size_t>(v) * kD * (cv.init_mode == 1 ? 4 : 2);
    const int lines = cv.init_mode == 1 ? 4 : 2;
    for (int i = 0; i < lines; ++i) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + 128 * i));
  }

  // ---- setup -----------------------------------------------------------------------------------------------
  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(BAR_FULL + s), 1);
      mbar_init(bar(BAR_EMPTY + s), 1 + 4);   // MMA commit + one arrival per state warp
    }
    mbar_init(bar(BAR_WFULL), 1);
    mbar_init(bar(BAR_OFULL), 1);
    mbar_init(bar(BAR_SFULL), 1);
    mbar_init(bar(BAR_UREADY), 4);
    mbar_init(bar(BAR_SBREADY), 4);
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

  if (warp == 0) {
    // ===== copy producer: one bulk copy per chunk record ===================================================
    if (lane == 0) {
      int issued = 0;
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % kStages, k = c / kStages;
        if (k > 0 && !mbar_wait(bar(BAR_EMPTY + s), (k - 1) & 1, abort_flag)) { failed = true; break; }
        mbar_arrive_expect_tx(bar(BAR_FULL + s), kRecBytes);
        bulk_g2s(sbase + kSmStage + s * kRecBytes, rec0 + static_cast<size_t>(c) * kRecBytes, kRecBytes, bar(BAR_FULL + s));
        issued = c + 1;
      }
      if (failed || *abort_flag > 0) {
        // wait (bounded) for copies still in flight so that the CTA does not exit under them
        for (int c = issued > kStages ? issued - kStages : 0; c < issued; ++c) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(bar(BAR_FULL + c % kStages), (c / kStages) & 1))
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
      const uint32_t ut_addr = sbase + kSmUt;
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % kStages, k = c / kStages;
        const uint32_t rec = sbase + kSmStage + s * kRecBytes;
        if (!mbar_wait(bar(BAR_FULL + s), k & 1, abort_flag)) { failed = true; break; }
        if (!mbar_wait(bar(BAR_SBREADY), c & 1, abort_flag)) { failed = true; break; }
        if (c > 0 && !mbar_wait(bar(BAR_OFREE), (c - 1) & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        // [W^T | O^T] = Sb [wp; qp]^T : A = bf16 copy of S in tensor memory (two k per column), B = the [64][128] tile
        // that WP and QP form in the record, K-major; 8 k-steps of 16
        {
          const uint64_t b = umma_desc(rec + kRecWP, 128, 2048);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) umma_ts(tmem + kColW, tmem + kColSbd + ks * 8, b + ks * 16, idesc_n64, ks > 0);
        }
        umma_commit(bar(BAR_WFULL));
        if (!mbar_wait(bar(BAR_UREADY), c & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        // S^T += U^T kr : A = Ut [128][32] K-major (8-row groups 512 B apart), B = KR [32 tok][128 k] read
        // MN-major: core matrices adjacent along k 128 B apart, 8-token groups 2048 B apart
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          umma_ss(tmem + kColS, umma_desc(ut_addr + ks * 256, 128, 512), umma_desc(rec + kRecKR + ks * 4096, 2048, 128),
                  idesc_n128_bmn, 1);
        umma_commit(bar(BAR_SFULL));
        // O^T += U^T mqk^T : B = MQK [32][32] K-major (8-row groups 512 B apart)
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          umma_ss(tmem + kColO, umma_desc(ut_addr + ks * 256, 128, 512), umma_desc(rec + kRecMQK + ks * 256, 128, 512),
                  idesc_n32, 1);
        umma_commit(bar(BAR_OFULL));
        umma_commit(bar(BAR_EMPTY + s));
      }
      // the last commit's arrival must have landed in shared memory before the CTA may exit
      if (!failed && nchunks > 0) {
        const int c = nchunks - 1;
        if (!mbar_wait(bar(BAR_EMPTY + c % kStages), (c / kStages) & 1, abort_flag)) failed = true;
      }
    }
  } else if (warp < 6) {
    // ===== state warps: own TMEM lanes [32q, 32q+32) = state rows v ==========================================
    const int qd = warp & 3;
    const int v = qd * 32 + lane;
    const uint32_t tq = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    const size_t row_off = static_cast<size_t>(v) * kD;                          // row v of this walk's state block
    uint8_t* ut_row = smem + kSmUt + (v >> 3) * 512 + (v & 7) * 16;    // + 128 * (tok / 8)

    // ---- initial state -> TMEM (pre-decayed by the first chunk's e) and its bf16 operand copy --------------
    bool ok = true;
    if (nchunks > 0) ok = warp_wait(bar(BAR_FULL + 0), 0, abort_flag);
    if (ok) {
      const float* e0 = reinterpret_cast<const float*>(smem + kSmStage + kRecE);
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t x[32];
        if (cv.init_mode == 1 || cv.init_mode == 2) {
          if (cv.init_mode == 1) {
            const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(cv.init_base) + row_off + cb * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 f = __ldg(src + i);
              x[4 * i] = __float_as_uint(f.x); x[4 * i + 1] = __float_as_uint(f.y);
              x[4 * i + 2] = __float_as_uint(f.z); x[4 * i + 3] = __float_as_uint(f.w);
            }
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(cv.init_base) + row_off + cb * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 w = __ldg(src + i);
              x[8 * i] = w.x << 16; x[8 * i + 1] = w.x & 0xffff0000u;
              x[8 * i + 2] = w.y << 16; x[8 * i + 3] = w.y & 0xffff0000u;
              x[8 * i + 4] = w.z << 16; x[8 * i + 5] = w.z & 0xffff0000u;
              x[8 * i + 6] = w.w << 16; x[8 * i + 7] = w.w & 0xffff0000u;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = (cv.init_mode == 3 && cb * 32 + i == v) ? 0x3f800000u : 0u;
        }
        if (nchunks > 0) {
          uint32_t y[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) y[i] = pack_bf16(__uint_as_float(x[2 * i]), __uint_as_float(x[2 * i + 1]));
          tmem_st16(tq + kColSbd + cb * 16, y);
#pragma unroll
          for (int i = 0; i < 16; ++i) mul2(x[2 * i], x[2 * i + 1], reinterpret_cast<const float2*>(e0)[cb * 16 + i]);
        }
        tmem_st32(tq + kColS + cb * 32, x);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_SBREADY));
    } else {
      failed = true;
    }

    for (int c = 0; c < nchunks && !failed; ++c) {
      const int s = c % kStages;
      const uint8_t* rec = smem + kSmStage + s * kRecBytes;
      // ---- U epilogue -------------------------------------------------------------------------------------
      if (!warp_wait(bar(BAR_WFULL), c & 1, abort_flag)) { failed = true; break; }
      tc_fence_after();
      {
        uint32_t w[32];
        tmem_ld32(tq + kColW, w);
        tmem_wait_ld();
        const uint8_t* up_row = rec + kRecUP + (v >> 3) * 512 + (v & 7) * 16;   // row v of UP [128 v][32 tok]
        float u[32];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 t = cv.zero_up ? make_uint4(0u, 0u, 0u, 0u) : *reinterpret_cast<const uint4*>(up_row + i * 128);
          u[8 * i + 0] = bf_lo(t.x) - __uint_as_float(w[8 * i + 0]);
          u[8 * i + 1] = bf_hi(t.x) - __uint_as_float(w[8 * i + 1]);
          u[8 * i + 2] = bf_lo(t.y) - __uint_as_float(w[8 * i + 2]);
          u[8 * i + 3] = bf_hi(t.y) - __uint_as_float(w[8 * i + 3]);
          u[8 * i + 4] = bf_lo(t.z) - __uint_as_float(w[8 * i + 4]);
          u[8 * i + 5] = bf_hi(t.z) - __uint_as_float(w[8 * i + 5]);
          u[8 * i + 6] = bf_lo(t.w) - __uint_as_float(w[8 * i + 6]);
          u[8 * i + 7] = bf_hi(t.w) - __uint_as_float(w[8 * i + 7]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(ut_row + i * 128) =
              make_uint4(pack_bf16(u[8 * i], u[8 * i + 1]), pack_bf16(u[8 * i + 2], u[8 * i + 3]),
                         pack_bf16(u[8 * i + 4], u[8 * i + 5]), pack_bf16(u[8 * i + 6], u[8 * i + 7]));
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(BAR_UREADY));
        mbar_arrive(bar(BAR_EMPTY + s));   // this warp is done reading up[] of the stage
      }
      // ---- S epilogue: bf16 operand copy of the new state, then pre-decay for the next chunk ------------
      if (c + 1 == nchunks) break;          // the last state is only read back once, below
      if (!warp_wait(bar(BAR_SFULL), c & 1, abort_flag)) { failed = true; break; }
      if (!warp_wait(bar(BAR_FULL + (c + 1) % kStages), ((c + 1) / kStages) & 1, abort_flag)) { failed = true; break; }
      tc_fence_after();
      {
        const float* e = reinterpret_cast<const float*>(smem + kSmStage + ((c + 1) % kStages) * kRecBytes + kRecE);
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t x[32], y[16];
          tmem_ld32(tq + kColS + cb * 32, x);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) y[i] = pack_bf16(__uint_as_float(x[2 * i]), __uint_as_float(x[2 * i + 1]));
          tmem_st16(tq + kColSbd + cb * 16, y);
#pragma unroll
          for (int i = 0; i < 16; ++i) mul2(x[2 * i], x[2 * i + 1], reinterpret_cast<const float2*>(e)[cb * 16 + i]);
          tmem_st32(tq + kColS + cb * 32, x);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_SBREADY));
    }

    // ---- final state -> global -------------------------------------------------------------------------------
    if (!failed && cv.fin_base != nullptr) {
      bool ok2 = true;
      if (nchunks > 0) ok2 = warp_wait(bar(BAR_SFULL), (nchunks - 1) & 1, abort_flag);
      if (ok2) {
        tc_fence_after();
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t x[32];
          tmem_ld32(tq + kColS + cb * 32, x);
          tmem_wait_ld();
          if (cv.fin_fp32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(cv.fin_base) + static_cast<size_t>(v) * cv.fin_stride + cb * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(x[4 * i]), __uint_as_float(x[4 * i + 1]), __uint_as_float(x[4 * i + 2]),
                                   __uint_as_float(x[4 * i + 3]));
          } else {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(cv.fin_base) + row_off + cb * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[i] = make_uint4(pack_bf16(__uint_as_float(x[8 * i]), __uint_as_float(x[8 * i + 1])),
                                  pack_bf16(__uint_as_float(x[8 * i + 2]), __uint_as_float(x[8 * i + 3])),
                                  pack_bf16(__uint_as_float(x[8 * i + 4]), __uint_as_float(x[8 * i + 5])),
                                  pack_bf16(__uint_as_float(x[8 * i + 6]), __uint_as_float(x[8 * i + 7])));
          }
        }
      } else {
        failed = true;
      }
    }
  } else {
    // ===== output warps: O^T (TMEM lanes = v, columns = tokens) -> out[token][h][v] ===========================
    const int qd = warp & 3;
    const uint32_t tq = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + kSmOutStg + qd * 2048);   // [32 tok][32 v]
    for (int c = 0; c < nchunks; ++c) {
      if (!warp_wait(bar(BAR_OFULL), c & 1, abort_flag)) { failed = true; break; }
      tc_fence_after();
      uint32_t o[32];
      tmem_ld32(tq + kColO, o);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_OFREE));
#pragma unroll
      for (int i = 0; i < 32; ++i) stg[i * 32 + lane] = __float2bfloat16_rn(__uint_as_float(o[i]));
      __syncwarp();
      const int64_t tok0 = bos + static_cast<int64_t>(c) * kChunk;
      const int valid = (eos - tok0) < kChunk ? static_cast<int>(eos - tok0) : kChunk;
      // each token row of this warp's 32 v-columns is 64 contiguous bytes: 4 lanes x 16 B, 8 rows per pass
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + (lane >> 2), c8 = (lane & 3) * 8;
        if (cv.write_out && r < valid) {
          const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 32 + c8);
          *reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(tok0 + r) * p.H + h) * kD + qd * 32 + c8) = val;
        }
      }
      __syncwarp();
    }
  }

  if (failed || *abort_flag > 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);

  // ---- common exit: every thread arrives here, TMEM goes back ------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

cudaError_t launch_scan(const ScanParams& p, cudaStream_t stream) {
  int64_t chains = static_cast<int64_t>(p.N) * p.H;
  if (p.seg_chunks > 0) chains *= p.seg_pass == 1 ? 2 * p.n_segs - 3 : p.n_segs - 1;
  if (chains <= 0) return cudaSuccess;
  auto kernel = p.seg_chunks > 0 ? scan_kernel<true> : scan_kernel<false>;
  static SmemOptIn opt_in[2];
  cudaError_t e = opt_in[p.seg_chunks > 0 ? 1 : 0].ensure(kernel, kScanSmemBytes);
  if (e != cudaSuccess) return e;
  kernel<<<static_cast<unsigned>(chains), kScanThreads, kScanSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fkda
