// Inter-chunk recurrence of the KDA prefill, look-ahead form: one CTA walks the chunks of one
// (sequence, head) chain with the 128x128 fp32 state resident in tensor memory.
//
// Replaces the reference's K2 (csrc/smxx/fwd_kernel2.cuh:115-839).  With S_c the state after chunk c
// (held as S^T: TMEM lanes = v, columns = k) and Sd_c = diag(e_{c+1}) S_c its pre-decayed form,
//     S_c     = Sd_{c-1} + kr_c^T U_c
//     W_{c+1} = wp_{c+1} S_c = wp_{c+1} Sd_{c-1} + X_{c+1} U_c ,   X_{c+1} = wp_{c+1} kr_c^T   (32x32)
//     O_{c+1} = qp_{c+1} Sd_{c-1} + Y_{c+1} U_c + mqk_{c+1} U_{c+1} , Y_{c+1} = qp_{c+1} kr_c^T
//     U_c     = up_c - W_c
// so the serial chain per chunk is only  U_c -> (tiny K=32 MMA) -> W_{c+1} -> U_{c+1};  the state
// update, its decay and the refresh of its bf16 operand copy run beside that chain, and X, Y are
// products of operand records only and are computed ahead of time.  All products are tcgen05.mma
// with M = 128; U^T and the bf16 copy of Sd are MMA A-operands read from tensor memory.
//
// Warp roles (896 threads): 0 = bulk-copy producer; 1, 2, 3 = one MMA-issuing thread each (products on
// U / on the decayed state / X,Y), ordered among each other through tcgen05.commit + mbarriers;
// 4-7 = U warps (critical chain); 8-23 = state warps (four groups of four, 32 state columns each: the decay of a chunk takes
// them about 1300 cycles; kStateBlocks = 2 makes it eight warps of 64 columns, 1580 cycles, 96 instead of 72 registers,
// 1 % slower); 24-27 = output warps (two of them also turn X, Y into bf16 operands).  Every wait is bounded; a wait that gives up raises an abort flag, records a
// status code and lets all roles fall through to the common exit, where TMEM is released.
#include "fkda_common.cuh"

namespace fkda {
namespace scan2 {

// Optional timeline trace (bring-up / tuning aid): when a buffer has been registered with
// fkda_debug_set_scan_trace, CTA 0 records clock64() at a few points of each role for its first
// 32 chunks: entry [(role * 32 + chunk) * 8 + event].  No effect when no buffer is registered.
// Compiled in only with -DFKDA_TUNING.
#ifdef FKDA_TUNING
static unsigned long long* g_trace = nullptr;
#define FKDA_TRACE(role, c, ev)                                                                         \
  do {                                                                                                  \
    if (trace != nullptr && (c) < 32) trace[((role) * 32 + (c)) * 8 + (ev)] = static_cast<unsigned long long>(clock64()); \
  } while (0)
#else
#define FKDA_TRACE(role, c, ev) do { } while (0)
#endif

constexpr int kStages = 5;
constexpr int kStateBlocks = 1;                         // 32-column blocks of the state per state warp (1: sixteen warps; 2: eight)
constexpr int kStateWarps = 16 / kStateBlocks;
constexpr int kOutWarp0 = 8 + kStateWarps;              // first output warp
constexpr int kThreads = (kOutWarp0 + 4) * 32;
constexpr uint32_t kTmemCols = 512;
// tensor-memory columns
constexpr uint32_t kColS = 0;                   // 128: state accumulator S^T [v][k], fp32
constexpr uint32_t kColWO = 128;                // 2 x 64: [W^T | O^T], each [v][tok] of 32 columns
constexpr uint32_t kColW = kColWO;              //   W of buffer b at kColW + 64 b
constexpr uint32_t kColO = kColWO + 32;         //   O of buffer b at kColO + 64 b
constexpr uint32_t kColXA = 256;                // 2 x 32: [X;Y] accumulator, lanes 0-31 X rows, 32-63 Y rows
constexpr uint32_t kColSbd = 320;               // 2 x 64: bf16 copy of Sd [v][k], two k per column
constexpr uint32_t kColUt = 448;                // 2 x 16: bf16 U^T [v][tok], two tokens per column

// shared memory (byte offsets from a 1024-byte aligned base)
constexpr int kSmStage = 0;
constexpr int kSmXY = kSmStage + kStages * kRecBytes;   // 2 x [64][32] bf16 (core layout): rows 0-31 X, 32-63 Y
constexpr int kSmOutStg = kSmXY + 2 * 4096;             // 4 warps x [32 tok][32 v] bf16
constexpr int kSmBars = kSmOutStg + 4 * 2048;
constexpr int kSmMisc = kSmBars + 256;
constexpr int kSmZero = kSmMisc + 64;                    // 512 zero bytes: stands in for u' where it is taken as zero
constexpr int kSmemBytes = kSmZero + 512 + 1024;

enum {
  BAR_FULL = 0,                    // [kStages] record landed
  BAR_EMPTY = BAR_FULL + kStages,  // [kStages] record no longer needed
  BAR_WFULL = BAR_EMPTY + kStages, // [2] W buffer complete
  BAR_OFULL = BAR_WFULL + 2,       // [2] O buffer complete
  BAR_XFULL = BAR_OFULL + 2,       // [2] X/Y accumulator complete
  BAR_XREADY = BAR_XFULL + 2,      // [2] X/Y bf16 operands in shared memory
  BAR_OFREE = BAR_XREADY + 2,      // [2] O buffer drained
  BAR_AFULL = BAR_OFREE + 2,       // [2] products on the decayed state have landed in the W/O buffer
  BAR_WFREE = BAR_AFULL + 2,       // [2] W buffer read by the U warps
  BAR_XYFREE = BAR_WFREE + 2,      // [2] products that read the X/Y operands of a buffer are complete
  BAR_SFULL = BAR_XYFREE + 2,      // state update of a chunk complete
  BAR_UREADY,                      // U^T of a chunk in tensor memory
  BAR_SREADY,                      // decayed state (fp32 accumulator) ready for the next update; phase 0 = initial state,
                                   // phase k = after chunk k-1.  Watched by issuer 1 only, which cannot fall behind.
  BAR_SBDREADY,                    // [2] bf16 copy of the decayed state ready, same phases: barrier ph & 1, its phase ph >> 1.
                                   // Released before BAR_SREADY: the products that read the copy head the longest chain.
                                   // Watched by issuer 2, which the data flow lets lag two phases: hence two barriers.
  BAR_COUNT = BAR_SBDREADY + 2
};
static_assert(BAR_COUNT * 8 <= 256, "barrier area");

__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t backoff_ns = 0) {
  const bool ok = mbar_wait(bar, parity, abort_flag, backoff_ns);
  return __all_sync(0xffffffffu, ok);
}
// use count of the X/Y buffers: chunk c >= 1 uses buffer c & 1
__device__ __forceinline__ uint32_t xy_use(int c) { return (c & 1) ? (c >> 1) : (c >> 1) - 1; }

__device__ __forceinline__ void pack32(const uint32_t (&x)[32], uint32_t (&y)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) y[i] = pack_bf16(__uint_as_float(x[2 * i]), __uint_as_float(x[2 * i + 1]));
}

// The state warps' per-chunk loop: decay the updated state for the next chunk and refresh its bf16 copy.  A function
// of its own (not inlined) so that its registers are allotted independently of the other warp roles.
__device__ __noinline__ bool state_warp_loop(uint8_t* smem, uint32_t tq, int grp, int nchunks, int warp, int lane,
                                             unsigned long long* trace) {
  const uint32_t sbase = smem_u32(smem);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kSmMisc + 4);
  auto bar = [&](int i) { return sbase + kSmBars + 8 * i; };
  auto full_bar = [&](int c) { return bar(BAR_FULL + c % kStages); };
  auto full_par = [&](int c) { return static_cast<uint32_t>((c / kStages) & 1); };
  bool failed = false;
  for (int c = 0; c + 1 < nchunks && !failed; ++c) {
    if (!warp_wait(full_bar(c + 1), full_par(c + 1), abort_flag)) { failed = true; break; }
    // The decay factors of the next chunk are the same for every lane: every lane reads the same address (a broadcast,
    // one wavefront per load), two factors per load and per packed fp32x2 multiply.
    const float2* e2 = reinterpret_cast<const float2*>(smem + kSmStage + ((c + 1) % kStages) * kRecBytes + kRecE) + 16 * kStateBlocks * grp;
    if (!warp_wait(bar(BAR_SFULL), c & 1, abort_flag)) { failed = true; break; }
    const int trole = 2;
    const bool tr_on = (warp == 8) && lane == 0;
    if (tr_on) FKDA_TRACE(trole, c, 0);
    tc_fence_after();
    if (tr_on) FKDA_TRACE(trole, c, 1);
    uint32_t x[kStateBlocks][32], y[16];
#pragma unroll
    for (int blk = 0; blk < kStateBlocks; ++blk) tmem_ld32(tq + kColS + 32 * (kStateBlocks * grp + blk), x[blk]);
    tmem_wait_ld();
    if (tr_on) FKDA_TRACE(trole, c, 2);
    // the bf16 copy first: the products that read it head the longest chain of the step
#pragma unroll
    for (int blk = 0; blk < kStateBlocks; ++blk) {
#pragma unroll
      for (int i = 0; i < 16; ++i) mul2(x[blk][2 * i], x[blk][2 * i + 1], e2[16 * blk + i]);
      if (tr_on && blk == 0) FKDA_TRACE(trole, c, 6);
      pack32(x[blk], y);
      tmem_st16(tq + kColSbd + 64 * (c & 1) + 16 * (kStateBlocks * grp + blk), y);
      if (tr_on && blk == 0) FKDA_TRACE(trole, c, 7);
    }
    tmem_wait_st();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(BAR_SBDREADY + ((c + 1) & 1)));
#pragma unroll
    for (int blk = 0; blk < kStateBlocks; ++blk) tmem_st32(tq + kColS + 32 * (kStateBlocks * grp + blk), x[blk]);
    if (tr_on) FKDA_TRACE(trole, c, 4);
    tmem_wait_st();
    if (tr_on) FKDA_TRACE(trole, c, 5);
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      if (tr_on) FKDA_TRACE(trole, c, 3);
      if (warp < 16) FKDA_TRACE(5, c, warp - 8);          // arrival time of the first eight state warps
      mbar_arrive(bar(BAR_SREADY));
      mbar_arrive(bar(BAR_EMPTY + (c + 1) % kStages));    // done with e of record c+1
    }
  }
  return failed;
}

// kSeg: CTAs walk runs of a sequence (segment-parallel form) instead of whole sequences
template <bool kSeg>
__global__ void __launch_bounds__(kThreads, 1) scan2_kernel(const ScanParams p, unsigned long long* trace_buf) {
#ifdef FKDA_TUNING
  unsigned long long* trace = (blockIdx.x == 0) ? trace_buf : nullptr;
#else
  unsigned long long* trace = nullptr;
  (void)trace_buf;
#endif
  if (threadIdx.x == 0) FKDA_TRACE(4, 31, 1);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kSmMisc + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmMisc);
  auto bar = [&](int i) { return sbase + kSmBars + 8 * i; };
  auto full_bar = [&](int c) { return bar(BAR_FULL + c % kStages); };
  auto full_par = [&](int c) { return static_cast<uint32_t>((c / kStages) & 1); };

  if (p.select != nullptr && *p.select != p.select_want) return;     // the other recurrence kernel was chosen
  // ---- chain -> tokens and records ---------------------------------------------------------------------
  // variant: 0 = the recurrence proper; 1 = offset half of a run's affine map (zero state in, no output);
  // 2 = transition half (identity in, u' taken as zero, no output)
  int chain = blockIdx.x, seg = 0, variant = 0;
  if constexpr (kSeg) {
    const int per = p.seg_pass == 1 ? 2 * p.n_segs - 3 : p.n_segs - 1;
    chain = blockIdx.x / per;
    const int j = blockIdx.x - chain * per;
    if (p.seg_pass == 1) {
      if (j > 0) { seg = 1 + ((j - 1) >> 1); variant = 1 + ((j - 1) & 1); }
    } else {
      seg = 1 + j;
    }
  }
  const int slot = chain / p.H, h = chain - slot * p.H;
  const int n = p.seq_order != nullptr ? p.seq_order[slot] : slot;     // varlen: longest sequences first
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
  if constexpr (kSeg) {
    // where the state comes from and goes to: the caller's tensors, or the per-run slots of the segment buffer
    const size_t chain_state = (static_cast<size_t>(n) * p.H + h) * kD * kD;
    const void* init_base = nullptr;     // this chain's [128 v][128 k] block
    int init_mode = 0;                   // 0 = zero, 1 = fp32, 2 = bf16, 3 = identity
    void* fin_base = nullptr;
    int fin_fp32 = p.state_fp32;
    if (p.initial_state != nullptr) {
      init_mode = p.state_fp32 ? 1 : 2;
      init_base = static_cast<const uint8_t*>(p.initial_state) + chain_state * (p.state_fp32 ? 4 : 2);
    }
    if (p.final_state != nullptr) fin_base = static_cast<uint8_t*>(p.final_state) + chain_state * (p.state_fp32 ? 4 : 2);
    float* slots = p.seg_buf + (static_cast<size_t>(n) * p.H + h) * p.n_segs * 3 * kSegSlotFloats;
    const int run_len = p.seg_chunks_dev != nullptr ? *p.seg_chunks_dev : p.seg_chunks;
    const int c_begin = seg * run_len < nchunks ? seg * run_len : nchunks;
    const int c_end = (seg == p.n_segs - 1 || (seg + 1) * run_len > nchunks) ? nchunks : (seg + 1) * run_len;
    if (seg < p.n_segs - 1) {
      const int64_t run_end = bos + static_cast<int64_t>(c_end) * kChunk;
      eos = run_end < eos ? run_end : eos;
    }
    bos += static_cast<int64_t>(c_begin) * kChunk;
    chunk_base += c_begin;
    nchunks = c_end - c_begin;
    if (p.seg_pass == 1) {
      if (variant == 0) {
        fin_base = slots + (1 * 3 + 2) * kSegSlotFloats;                 // state at the start of run 1
      } else {
        init_mode = variant == 2 ? 3 : 0;
        init_base = nullptr;
        fin_base = slots + (seg * 3 + (variant == 2 ? 0 : 1)) * kSegSlotFloats;
      }
      fin_fp32 = 1;
    } else {
      init_mode = 1;
      init_base = slots + (seg * 3 + 2) * kSegSlotFloats;
      if (seg != p.n_segs - 1) fin_base = nullptr;
    }
    // parked in shared memory for the state warps, which have no registers to spare
    if (tid == 0) {
      *reinterpret_cast<const void**>(smem + kSmMisc + 8) = init_base;
      *reinterpret_cast<void**>(smem + kSmMisc + 16) = fin_base;
      *reinterpret_cast<int*>(smem + kSmMisc + 24) = init_mode;
      *reinterpret_cast<int*>(smem + kSmMisc + 28) = fin_fp32;
    }
  }
  const bool write_out = !kSeg || variant == 0;
  const bool zero_up = kSeg && variant == 2;
  const uint8_t* rec0 = p.records + (static_cast<size_t>(h) * p.total_chunks + chunk_base) * kRecBytes;

  // ---- setup -----------------------------------------------------------------------------------------------
  if (kSeg && tid < 128) reinterpret_cast<uint32_t*>(smem + kSmZero)[tid] = 0u;
  if (tid == 0) {
    *abort_flag = p.wait_limit_us > 0 ? -p.wait_limit_us : 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(BAR_FULL + s), 1);
      mbar_init(bar(BAR_EMPTY + s), 1 + 4 + kStateWarps);   // MMA commit + U warps + state warps
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(BAR_WFULL + b), 1);
      mbar_init(bar(BAR_OFULL + b), 1);
      mbar_init(bar(BAR_XFULL + b), 1);
      mbar_init(bar(BAR_XREADY + b), 2);
      mbar_init(bar(BAR_OFREE + b), 4);
      mbar_init(bar(BAR_AFULL + b), 1);
      mbar_init(bar(BAR_WFREE + b), 4);
      mbar_init(bar(BAR_XYFREE + b), 1);
    }
    mbar_init(bar(BAR_SFULL), 1);
    mbar_init(bar(BAR_UREADY), 4);
    mbar_init(bar(BAR_SREADY), kStateWarps);
    mbar_init(bar(BAR_SBDREADY + 0), kStateWarps);
    mbar_init(bar(BAR_SBDREADY + 1), kStateWarps);
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
  if (tid == 0) FKDA_TRACE(4, 31, 0);

  bool failed = false;

  if (warp == 0) {
    // ===== copy producer: one bulk copy per chunk record ===================================================
    if (lane == 0) {
      int issued = 0;
      for (int c = 0; c < nchunks; ++c) {
        if (p.stop_copies_after > 0 && c >= p.stop_copies_after) break;     // test aid: the consumers' next wait runs out
        const int s = c % kStages, k = c / kStages;
        if (k > 0 && !mbar_wait(bar(BAR_EMPTY + s), (k - 1) & 1, abort_flag, 64)) { failed = true; break; }
        FKDA_TRACE(4, c, 0);
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
    // ===== MMA issuer 1: products on U_c (finish W_{c+1} first: it is the serial chain) =====================
    if (lane == 0) {
      constexpr uint32_t idesc_n32 = umma_idesc_bf16(128, 32, 0, 0);
      constexpr uint32_t idesc_n64 = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_n128_bmn = umma_idesc_bf16(128, 128, 0, 1);
      for (int c = 0; c < nchunks; ++c) {
        const uint32_t rec = sbase + kSmStage + (c % kStages) * kRecBytes;
        const uint32_t ut = tmem + kColUt + 16 * (c & 1);
        const bool more = c + 1 < nchunks;
        FKDA_TRACE(0, c, 6);
        if (!mbar_wait(bar(BAR_SREADY), c & 1, abort_flag)) { failed = true; break; }
        FKDA_TRACE(0, c, 7);
        if (!mbar_wait(bar(BAR_UREADY), c & 1, abort_flag)) { failed = true; break; }
        tc_fence_after();
        FKDA_TRACE(0, c, 0);
        {  // S^T += U^T kr : kr [32 tok][128 k] read MN-major (k-adjacent core matrices 128 B apart, token groups 2048 B)
          const uint64_t bk = umma_desc(rec + kRecKR, 2048, 128);
          umma_ts(tmem + kColS, ut, bk, idesc_n128_bmn, 1);
          umma_ts(tmem + kColS, ut + 8, bk + 256, idesc_n128_bmn, 1);
          umma_commit(bar(BAR_SFULL));
        }
        {  // O_c += U_c^T mqk_c^T (O_c's other terms were issued in earlier iterations / by issuer 2): before the products
           // for W_{c+1}, whose inputs (the products on the decayed state) wait for this output buffer's predecessor to drain
          const uint64_t bm = umma_desc(rec + kRecMQK, 128, 512);
          umma_ts(tmem + kColO + 64 * (c & 1), ut, bm, idesc_n32, 1);
          umma_ts(tmem + kColO + 64 * (c & 1), ut + 8, bm + 16, idesc_n32, 1);
          umma_commit(bar(BAR_OFULL + (c & 1)));
        }
        if (more) {
          // [W_{c+1} | O_{c+1}] += U_c^T [X_{c+1}; Y_{c+1}]^T : one N = 64 product per k-step, on top of the
          // products on the decayed state that issuer 2 placed there
          if (!mbar_wait(bar(BAR_AFULL + ((c + 1) & 1)), ((c + 1) >> 1) & 1, abort_flag)) { failed = true; break; }
          if (!mbar_wait(bar(BAR_XREADY + ((c + 1) & 1)), xy_use(c + 1) & 1u, abort_flag)) { failed = true; break; }
          tc_fence_after();
          const uint64_t bx = umma_desc(sbase + kSmXY + 4096 * ((c + 1) & 1), 128, 512);
          umma_ts(tmem + kColWO + 64 * ((c + 1) & 1), ut, bx, idesc_n64, 1);
          umma_ts(tmem + kColWO + 64 * ((c + 1) & 1), ut + 8, bx + 16, idesc_n64, 1);
          umma_commit(bar(BAR_WFULL + ((c + 1) & 1)));
        } else if (!mbar_wait(bar(BAR_AFULL + (c & 1)), (c >> 1) & 1, abort_flag)) { failed = true; break; }
        if (more) umma_commit(bar(BAR_XYFREE + ((c + 1) & 1)));
        umma_commit(bar(BAR_EMPTY + c % kStages));
        FKDA_TRACE(0, c, 1);
      }
      // the last commit's arrival must have landed in shared memory before the CTA may exit
      if (!failed && nchunks > 0) {
        const int c = nchunks - 1;
        if (!mbar_wait(bar(BAR_EMPTY + c % kStages), (c / kStages) & 1, abort_flag)) failed = true;
      }
    }
  } else if (warp == 2) {
    // ===== MMA issuer 2: [W_c | O_c] = Sd_{c-2} [wp_c; qp_c]^T (A from tensor memory, N = 64) ==============
    if (lane == 0) {
      constexpr uint32_t idesc_n64 = umma_idesc_bf16(128, 64, 0, 0);
      for (int c = 0; c < nchunks; ++c) {
        if (!mbar_wait(full_bar(c), full_par(c), abort_flag)) { failed = true; break; }
        if (c >= 2) {   // the buffer's previous contents have been consumed
          if (!mbar_wait(bar(BAR_WFREE + (c & 1)), ((c - 2) >> 1) & 1, abort_flag)) { failed = true; break; }
          if (!mbar_wait(bar(BAR_OFREE + (c & 1)), ((c - 2) >> 1) & 1, abort_flag)) { failed = true; break; }
        }
        {
          const int ph = c < 2 ? 0 : c - 1;       // needs the copy of Sd_{c-2}
          if (!mbar_wait(bar(BAR_SBDREADY + (ph & 1)), (ph >> 1) & 1, abort_flag)) { failed = true; break; }
        }
        tc_fence_after();
        FKDA_TRACE(0, c, 2);
        const uint32_t sbd = tmem + kColSbd + 64 * (c & 1);
        const uint64_t b = umma_desc(sbase + kSmStage + (c % kStages) * kRecBytes + kRecWP, 128, 2048);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ts(tmem + kColWO + 64 * (c & 1), sbd + ks * 8, b + ks * 16, idesc_n64, ks > 0);
        umma_commit(bar(BAR_AFULL + (c & 1)));
        if (c == 0) umma_commit(bar(BAR_WFULL + 0));
        FKDA_TRACE(0, c, 3);
      }
    }
  } else if (warp == 3) {
    // ===== MMA issuer 3: [X_c; Y_c] = [wp_c; qp_c] kr_{c-1}^T (records only, runs ahead) ======================
    if (lane == 0) {
      constexpr uint32_t idesc_n32 = umma_idesc_bf16(128, 32, 0, 0);
      for (int c = 1; c < nchunks; ++c) {
        if (!mbar_wait(full_bar(c - 1), full_par(c - 1), abort_flag, 64)) { failed = true; break; }
        if (!mbar_wait(full_bar(c), full_par(c), abort_flag, 64)) { failed = true; break; }
        if (c >= 3) {   // accumulator read by the X/Y epilogue of chunk c-2, its operands consumed by the U products
          if (!mbar_wait(bar(BAR_XREADY + (c & 1)), xy_use(c - 2) & 1u, abort_flag, 64)) { failed = true; break; }
          if (!mbar_wait(bar(BAR_XYFREE + (c & 1)), xy_use(c - 2) & 1u, abort_flag, 64)) { failed = true; break; }
        }
        tc_fence_after();
        FKDA_TRACE(0, c, 4);
        const uint64_t a = umma_desc(sbase + kSmStage + (c % kStages) * kRecBytes + kRecWP, 128, 2048);
        const uint64_t b = umma_desc(sbase + kSmStage + ((c - 1) % kStages) * kRecBytes + kRecKR, 128, 2048);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) umma_ss(tmem + kColXA + 32 * (c & 1), a + ks * 16, b + ks * 16, idesc_n32, ks > 0);
        umma_commit(bar(BAR_XFULL + (c & 1)));
        FKDA_TRACE(0, c, 5);
      }
    }
  } else if (warp < 8) {
    // ===== U warps: U^T = up^T - W^T, as a bf16 A operand in tensor memory (the serial chain) =============
    const int qd = warp & 3;
    const int v = qd * 32 + lane;
    const uint32_t tq = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    for (int c = 0; c < nchunks; ++c) {
      const uint8_t* rec = smem + kSmStage + (c % kStages) * kRecBytes;
      if (!warp_wait(full_bar(c), full_par(c), abort_flag)) { failed = true; break; }
      if (!warp_wait(bar(BAR_WFULL + (c & 1)), (c >> 1) & 1, abort_flag)) { failed = true; break; }
      tc_fence_after();
      if (warp == 4 && lane == 0) FKDA_TRACE(1, c, 0);
      uint32_t w[32], y[16];
      tmem_ld32(tq + kColW + 64 * (c & 1), w);
      const uint8_t* up_row = zero_up ? smem + kSmZero : rec + kRecUP + (v >> 3) * 512 + (v & 7) * 16;   // row v of UP [128 v][32 tok]
      uint4 t[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) t[i] = *reinterpret_cast<const uint4*>(up_row + i * 128);
      tmem_wait_ld();
      if (warp == 4 && lane == 0) FKDA_TRACE(1, c, 1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        y[4 * i + 0] = pack_bf16(bf_lo(t[i].x) - __uint_as_float(w[8 * i + 0]), bf_hi(t[i].x) - __uint_as_float(w[8 * i + 1]));
        y[4 * i + 1] = pack_bf16(bf_lo(t[i].y) - __uint_as_float(w[8 * i + 2]), bf_hi(t[i].y) - __uint_as_float(w[8 * i + 3]));
        y[4 * i + 2] = pack_bf16(bf_lo(t[i].z) - __uint_as_float(w[8 * i + 4]), bf_hi(t[i].z) - __uint_as_float(w[8 * i + 5]));
        y[4 * i + 3] = pack_bf16(bf_lo(t[i].w) - __uint_as_float(w[8 * i + 6]), bf_hi(t[i].w) - __uint_as_float(w[8 * i + 7]));
      }
      tmem_st16(tq + kColUt + 16 * (c & 1), y);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (warp == 4) FKDA_TRACE(1, c, 2);
        mbar_arrive(bar(BAR_UREADY));
        mbar_arrive(bar(BAR_WFREE + (c & 1)));
        mbar_arrive(bar(BAR_EMPTY + c % kStages));   // this warp is done reading up[] of the record
      }
    }
  } else if (warp < kOutWarp0) {
    // ===== state warps: groups of four; group g owns state columns k in [32 kStateBlocks g, + 32 kStateBlocks) ============
    const int grp = (warp - 8) >> 2;
    const int qd = warp & 3;
    const int v = qd * 32 + lane;
    const uint32_t tq = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    const size_t row_off = static_cast<size_t>(v) * kD;                          // row v of this chain's state
    const void* init_base;
    int init_mode;                      // 0 = zero, 1 = fp32, 2 = bf16, 3 = identity
    if constexpr (kSeg) {
      init_base = *reinterpret_cast<const void* volatile*>(smem + kSmMisc + 8);
      init_mode = *reinterpret_cast<volatile int*>(smem + kSmMisc + 24);
    } else {
      const size_t chain_state = (static_cast<size_t>(n) * p.H + h) * kD * kD;
      init_base = static_cast<const uint8_t*>(p.initial_state) + chain_state * (p.state_fp32 ? 4 : 2);
      init_mode = p.initial_state == nullptr ? 0 : (p.state_fp32 ? 1 : 2);
    }

    // ---- initial state: S <- e_0 S_init; bf16 copies of S_init (buffer 0) and e_0 S_init (buffer 1) --------
    // All global loads of this thread's 64 state values are issued before anything is waited for.
    uint32_t xi[kStateBlocks][32];
#pragma unroll
    for (int half = 0; half < kStateBlocks; ++half) {
      const int cb = kStateBlocks * grp + half;     // 32-column block
      if (init_mode == 1 || init_mode == 2) {
        if (init_mode == 1) {
          const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(init_base) + row_off + cb * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 f = __ldg(src + i);
            xi[half][4 * i] = __float_as_uint(f.x); xi[half][4 * i + 1] = __float_as_uint(f.y);
            xi[half][4 * i + 2] = __float_as_uint(f.z); xi[half][4 * i + 3] = __float_as_uint(f.w);
          }
        } else {
          const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(init_base) + row_off + cb * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 w = __ldg(src + i);
            xi[half][8 * i] = w.x << 16; xi[half][8 * i + 1] = w.x & 0xffff0000u;
            xi[half][8 * i + 2] = w.y << 16; xi[half][8 * i + 3] = w.y & 0xffff0000u;
            xi[half][8 * i + 4] = w.z << 16; xi[half][8 * i + 5] = w.z & 0xffff0000u;
            xi[half][8 * i + 6] = w.w << 16; xi[half][8 * i + 7] = w.w & 0xffff0000u;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) xi[half][i] = (init_mode == 3 && cb * 32 + i == v) ? 0x3f800000u : 0u;
      }
    }
    if (warp == 8 && lane == 0) FKDA_TRACE(2, 30, 0);
    bool ok = true;
    if (nchunks > 0) ok = warp_wait(full_bar(0), 0, abort_flag);
    if (warp == 8 && lane == 0) FKDA_TRACE(2, 30, 1);
    if (ok) {
      const float2* e0 = reinterpret_cast<const float2*>(smem + kSmStage + kRecE);      // decay factors of chunk 0
#pragma unroll
      for (int half = 0; half < kStateBlocks; ++half) {
        const int cb = kStateBlocks * grp + half;
        uint32_t y[16];
        if (nchunks > 0) {
          pack32(xi[half], y);
          tmem_st16(tq + kColSbd + 0 + cb * 16, y);
#pragma unroll
          for (int i = 0; i < 16; ++i) mul2(xi[half][2 * i], xi[half][2 * i + 1], e0[16 * cb + i]);
          pack32(xi[half], y);
          tmem_st16(tq + kColSbd + 64 + cb * 16, y);
        }
        tmem_st32(tq + kColS + cb * 32, xi[half]);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (warp == 8) FKDA_TRACE(2, 30, 2);
        mbar_arrive(bar(BAR_SBDREADY + 0));
        mbar_arrive(bar(BAR_SREADY));
        if (nchunks > 0) mbar_arrive(bar(BAR_EMPTY + 0));   // done with e of record 0
      }
    } else {
      failed = true;
    }

    // ---- per chunk: decay the updated state for the next chunk and refresh its bf16 copy ------------------
    if (!failed) failed = state_warp_loop(smem, tq, grp, nchunks, warp, lane, trace);

    // ---- final state -> global -------------------------------------------------------------------------------
    void* fin_base;
    int fin_fp32;
    if constexpr (kSeg) {
      fin_base = *reinterpret_cast<void* volatile*>(smem + kSmMisc + 16);
      fin_fp32 = *reinterpret_cast<volatile int*>(smem + kSmMisc + 28);
    } else {
      const size_t chain_state = (static_cast<size_t>(n) * p.H + h) * kD * kD;
      fin_base = p.final_state == nullptr ? nullptr : static_cast<uint8_t*>(p.final_state) + chain_state * (p.state_fp32 ? 4 : 2);
      fin_fp32 = p.state_fp32;
    }
    if (!failed && fin_base != nullptr) {
      bool ok2 = true;
      if (nchunks > 0) ok2 = warp_wait(bar(BAR_SFULL), (nchunks - 1) & 1, abort_flag);
      if (ok2) {
        tc_fence_after();
        if (warp == 8 && lane == 0) FKDA_TRACE(2, 30, 3);
#pragma unroll 1
        for (int half = 0; half < kStateBlocks; ++half) {
          const int cb = kStateBlocks * grp + half;
          uint32_t x[32];
          tmem_ld32(tq + kColS + cb * 32, x);
          tmem_wait_ld();
          if (fin_fp32) {
            // (a transition map goes into its slot with padded rows: the map chaining reads it in one piece)
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(fin_base) + (zero_up ? static_cast<size_t>(v) * kSegMapStride : row_off) + cb * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              dst[i] = make_float4(__uint_as_float(x[4 * i]), __uint_as_float(x[4 * i + 1]), __uint_as_float(x[4 * i + 2]),
                                   __uint_as_float(x[4 * i + 3]));
          } else {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(fin_base) + row_off + cb * 32);
            uint32_t y[16];
            pack32(x, y);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
          }
        }
      } else {
        failed = true;
      }
    }
  } else {
    // ===== output warps: O^T (TMEM lanes = v, columns = tokens) -> out[token][h][v]; X/Y -> bf16 operands ======
    const int qd = warp & 3;
    const uint32_t tq = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + kSmOutStg + qd * 2048);   // [32 tok][32 v]
    auto xy_epilogue = [&](int c) -> bool {     // accumulator lanes 0-31 = X rows, 32-63 = Y rows (warps on quadrants 0, 1)
      if (qd >= 2) return true;
      if (!warp_wait(bar(BAR_XFULL + (c & 1)), xy_use(c) & 1u, abort_flag, 32)) return false;
      tc_fence_after();
      if (warp == kOutWarp0 && lane == 0) FKDA_TRACE(3, c, 0);
      uint32_t x[32], y[16];
      tmem_ld32(tq + kColXA + 32 * (c & 1), x);
      tmem_wait_ld();
      pack32(x, y);
      const int r = qd * 32 + lane;
      uint8_t* row = smem + kSmXY + 4096 * (c & 1) + (r >> 3) * 512 + (r & 7) * 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(row + i * 128) = make_uint4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (warp == kOutWarp0) FKDA_TRACE(3, c, 1);
        mbar_arrive(bar(BAR_XREADY + (c & 1)));
      }
      return true;
    };
    for (int c = 0; c < nchunks; ++c) {
      if (c == 0 && nchunks > 1 && !xy_epilogue(1)) { failed = true; break; }
      if (c + 2 < nchunks && !xy_epilogue(c + 2)) { failed = true; break; }
      if (!warp_wait(bar(BAR_OFULL + (c & 1)), (c >> 1) & 1, abort_flag, 32)) { failed = true; break; }
      tc_fence_after();
      if (warp == kOutWarp0 && lane == 0) FKDA_TRACE(3, c, 2);
      uint32_t o[32];
      tmem_ld32(tq + kColO + 64 * (c & 1), o);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_OFREE + (c & 1)));
#pragma unroll
      for (int i = 0; i < 32; ++i) stg[i * 32 + lane] = __float2bfloat16_rn(__uint_as_float(o[i]));
      __syncwarp();
      const int64_t tok0 = bos + static_cast<int64_t>(c) * kChunk;
      const int valid = (eos - tok0) < kChunk ? static_cast<int>(eos - tok0) : kChunk;
      // each token row of this warp's 32 v-columns is 64 contiguous bytes: 4 lanes x 16 B, 8 rows per pass
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + (lane >> 2), c8 = (lane & 3) * 8;
        if (write_out && r < valid) {
          const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 32 + c8);
          *reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(tok0 + r) * p.H + h) * kD + qd * 32 + c8) = val;
        }
      }
      __syncwarp();
      if (warp == kOutWarp0 && lane == 0) FKDA_TRACE(3, c, 3);
    }
  }

  if (warp == 8 && lane == 0) FKDA_TRACE(2, 30, 4);
  if (failed || *abort_flag > 0) atomicCAS(p.status, kStatusOk, kStatusWaitTimeout);

  // ---- common exit: every thread arrives here, TMEM goes back ------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace scan2

cudaError_t launch_scan2(const ScanParams& p, cudaStream_t stream) {
  int64_t chains = static_cast<int64_t>(p.N) * p.H;
  if (p.seg_chunks > 0) chains *= p.seg_pass == 1 ? 2 * p.n_segs - 3 : p.n_segs - 1;
  if (chains <= 0) return cudaSuccess;
  auto kernel = p.seg_chunks > 0 ? scan2::scan2_kernel<true> : scan2::scan2_kernel<false>;
  static SmemOptIn opt_in[2];
  cudaError_t e = opt_in[p.seg_chunks > 0 ? 1 : 0].ensure(kernel, scan2::kSmemBytes);
  if (e != cudaSuccess) return e;
#ifdef FKDA_TUNING
  unsigned long long* trace = scan2::g_trace;
#else
  unsigned long long* trace = nullptr;
#endif
  kernel<<<static_cast<unsigned>(chains), scan2::kThreads, scan2::kSmemBytes, stream>>>(p, trace);
  return cudaGetLastError();
}

#ifdef FKDA_TUNING
void set_scan_trace(unsigned long long* buf) { scan2::g_trace = buf; }
#endif

}  // namespace fkda
