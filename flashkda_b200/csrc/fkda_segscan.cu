// Segment-parallel form of the inter-chunk recurrence for batches with few, long chains.
//
// The reference walks every (sequence, head) chain with one CTA from the first chunk to the last
// (csrc/smxx/fwd_kernel2.cuh:434-742), so a call with fewer chains than SMs leaves most of the GPU idle.  A run
// of chunks acts on the state Z = S^T ([v][k]) as an affine map, Z_end = Z_start M + N, because every chunk does
//     Z' = Z (diag(e) - w'^T kr) + u'^T kr .
// Here each sequence is cut into runs; a recurrence kernel itself (the look-ahead or the compact one, whichever gets
// the pass's CTAs through faster) produces M (walk from the identity with u' = 0) and N (walk from zero) of the inner
// runs in parallel, this file chains them into the state at the start of every run, and a second launch of a
// recurrence kernel walks all runs in parallel from those states.
#include "fkda_common.cuh"

namespace fkda {

cudaError_t launch_scan2(const ScanParams& p, cudaStream_t stream);
cudaError_t launch_scan(const ScanParams& p, cudaStream_t stream);

namespace {

constexpr int kCmbRows = 16;                              // state rows per CTA: one m16 tile
constexpr int kMapStride = kSegMapStride;                 // floats per map row, in its slot and here (B fragments: bank 8 t + g)
constexpr int kMapStg = kD * kMapStride * 4;
constexpr int kZStride = 132;                             // floats per staged state row (A fragments: bank 4 g + t)
constexpr int kMapBufs = 3;                               // maps in flight
constexpr int kCmbM = 0;                                  // kMapBufs x [128][136] fp32: transition maps
constexpr int kCmbZ = kCmbM + kMapBufs * kMapStg;         // [16][132] fp32: this CTA's rows of the state
constexpr int kCmbBars = kCmbZ + kCmbRows * kZStride * 4;
constexpr int kCmbSmemBytes = kCmbBars + 64 + 128;
static_assert(kCmbSmemBytes <= 227 * 1024, "map buffers fit one SM");

// Z_start[run + 1] = Z_start[run] M[run] + N[run] for run = 1 .. n_segs-2; rows of Z are independent, so each CTA
// carries sixteen of them through all runs.  The maps arrive by bulk copies (one per map: its slot holds it with padded
// rows) three runs ahead, so the serial chain of runs sees shared-memory latency only.  The products run on the tensor cores in
// tf32 with both operands split into a leading and a trailing part (three mma per tile: the error of the split, about
// 2^-21 relative, is that of an fp32 product), fp32 accumulation on top of N.
__global__ void __launch_bounds__(256) seg_combine_kernel(float* seg_buf, int n_segs, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
  const uint32_t sbase = smem_u32(smem);
  float* z = reinterpret_cast<float*>(smem + kCmbZ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kCmbBars + 32);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* slots = seg_buf + static_cast<size_t>(blockIdx.x) * n_segs * 3 * kSegSlotFloats;
  const int r_base = blockIdx.y * kCmbRows;
  auto load_map = [&](int run) {      // one thread: the whole slot, rows padded as the recurrence kernel left them
    const int b = (run - 1) % kMapBufs;
    mbar_arrive_expect_tx(sbase + kCmbBars + 8 * b, kMapStg);
    bulk_g2s(sbase + kCmbM + b * kMapStg, slots + (run * 3 + 0) * kSegSlotFloats, kMapStg, sbase + kCmbBars + 8 * b);
  };
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kMapBufs; ++i) mbar_init(sbase + kCmbBars + 8 * i, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0)
    for (int run = 1; run <= kMapBufs && run + 1 < n_segs; ++run) load_map(run);
  {
    // the state at the start of run 1: thread -> (row, eight columns)
    const int r = tid >> 4, c = (tid & 15) * 8;
    const float* src = slots + (1 * 3 + 2) * kSegSlotFloats + static_cast<size_t>(r_base + r) * kD + c;
    const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src + 4));
    *reinterpret_cast<float4*>(z + r * kZStride + c) = a;
    *reinterpret_cast<float4*>(z + r * kZStride + c + 4) = b;
  }
  __syncthreads();
  const int g = lane >> 2, t = lane & 3;
  const int n0 = warp * 16;              // this warp's sixteen output columns
  // N of a run: mma C layout, rows g and g + 8, columns n0 + 8 nt + 2 t + {0, 1}; fetched one run ahead (its latency
  // would otherwise sit on the serial chain of runs)
  auto load_n = [&](int run, float (&d)[2][4]) {
    const float* N = slots + (run * 3 + 1) * kSegSlotFloats + static_cast<size_t>(r_base) * kD;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float2 lo = *reinterpret_cast<const float2*>(N + g * kD + n0 + 8 * nt + 2 * t);
      const float2 hi = *reinterpret_cast<const float2*>(N + (g + 8) * kD + n0 + 8 * nt + 2 * t);
      d[nt][0] = lo.x; d[nt][1] = lo.y; d[nt][2] = hi.x; d[nt][3] = hi.y;
    }
  };
  float next_n[2][4];
  if (n_segs > 2) load_n(1, next_n);
  for (int run = 1; run + 1 < n_segs; ++run) {
    const int b = (run - 1) % kMapBufs;
    float acc[2][4];                  // accumulators start from N
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = next_n[nt][i];
    if (run + 2 < n_segs) load_n(run + 1, next_n);
    if (tid < 64 && run + 5 < n_segs)     // and the lines of a later N into the L2: 16 rows of 512 bytes
      asm volatile("prefetch.global.L2 [%0];" ::"l"(slots + ((run + 4) * 3 + 1) * kSegSlotFloats +
                                                     static_cast<size_t>(r_base + (tid >> 2)) * kD + (tid & 3) * 32));
    const bool ok = mbar_wait(sbase + kCmbBars + 8 * b, ((run - 1) / kMapBufs) & 1, abort_flag, 32);
    if (!__syncthreads_and(ok)) {
      if (tid == 0) {
        atomicCAS(status, kStatusOk, kStatusWaitTimeout);
        // do not leave while a copy may still be landing in this CTA's shared memory
        for (int r2 = run; r2 < run + kMapBufs && r2 + 1 < n_segs; ++r2) {     // the maps that have been asked for
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(sbase + kCmbBars + 8 * ((r2 - 1) % kMapBufs), ((r2 - 1) / kMapBufs) & 1))
            if (globaltimer_ns() - t0 > 20000000ull) break;
        }
      }
      break;
    }
    const float* M = reinterpret_cast<const float*>(smem + kCmbM + b * kMapStg);
    // four accumulators per tile, used in turn: the 48 mma of a tile would otherwise form one dependent chain
    float part[2][3][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int q = 0; q < 3; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) part[nt][q][i] = 0.f;
#pragma unroll 2
    for (int ks = 0; ks < kD / 8; ks += 2) {
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int k0 = 8 * (ks + kk);
        const float af[4] = {z[g * kZStride + k0 + t], z[(g + 8) * kZStride + k0 + t], z[g * kZStride + k0 + t + 4],
                             z[(g + 8) * kZStride + k0 + t + 4]};
        uint32_t ah[4], al[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ah[i] = to_tf32(af[i]);
          al[i] = to_tf32(af[i] - __uint_as_float(ah[i]));
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float b0 = M[(k0 + t) * kMapStride + n0 + 8 * nt + g], b1 = M[(k0 + t + 4) * kMapStride + n0 + 8 * nt + g];
          const uint32_t bh0 = to_tf32(b0), bh1 = to_tf32(b1);
          const uint32_t bl0 = to_tf32(b0 - __uint_as_float(bh0)), bl1 = to_tf32(b1 - __uint_as_float(bh1));
          mma_tf32_1688(part[nt][0], al[0], al[1], al[2], al[3], bh0, bh1);
          mma_tf32_1688(part[nt][1], ah[0], ah[1], ah[2], ah[3], bl0, bl1);
          if (kk == 0) mma_tf32_1688(part[nt][2], ah[0], ah[1], ah[2], ah[3], bh0, bh1);
          else mma_tf32_1688(acc[nt], ah[0], ah[1], ah[2], ah[3], bh0, bh1);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] += (part[nt][0][i] + part[nt][1][i]) + part[nt][2][i];
    __syncthreads();                  // every thread is done with z and with map buffer b
    if (tid == 0 && run + kMapBufs + 1 < n_segs) load_map(run + kMapBufs);
    float* zs = slots + ((run + 1) * 3 + 2) * kSegSlotFloats + static_cast<size_t>(r_base) * kD;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int c = n0 + 8 * nt + 2 * t;
      *reinterpret_cast<float2*>(z + g * kZStride + c) = make_float2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<float2*>(z + (g + 8) * kZStride + c) = make_float2(acc[nt][2], acc[nt][3]);
      *reinterpret_cast<float2*>(zs + g * kD + c) = make_float2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<float2*>(zs + (g + 8) * kD + c) = make_float2(acc[nt][2], acc[nt][3]);
    }
    __syncthreads();
  }
}

}  // namespace

cudaError_t launch_scan_segmented(const ScanParams& base, int n_segs, int seg_chunks, float* seg_buf, int kernel_choice,
                                  cudaStream_t stream) {
  ScanParams p = base;
  p.seg_chunks = seg_chunks;
  p.n_segs = n_segs;
  p.seg_buf = seg_buf;
  // either recurrence kernel can walk the runs: whichever gets the pass's CTAs through in less time
  const int64_t chains = static_cast<int64_t>(p.N) * p.H;
  bool compact1, compact2;
  const int sms = device_sm_count();
  pass_cost_x100(chains * (2 * n_segs - 3), &compact1, sms);
  pass_cost_x100(chains * (n_segs - 1), &compact2, sms);
  if (kernel_choice) compact1 = compact2 = kernel_choice == 1;   // forced: 1 compact, 2 look-ahead
  p.seg_pass = 1;
  cudaError_t e = compact1 ? launch_scan(p, stream) : launch_scan2(p, stream);
  if (e != cudaSuccess) return e;
  if (n_segs > 2) {
    static SmemOptIn opt_in;
    e = opt_in.ensure(seg_combine_kernel, kCmbSmemBytes);
    if (e != cudaSuccess) return e;
    const dim3 grid(static_cast<unsigned>(chains), kD / kCmbRows);
    seg_combine_kernel<<<grid, 256, kCmbSmemBytes, stream>>>(seg_buf, n_segs, p.status);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  p.seg_pass = 2;
  return compact2 ? launch_scan(p, stream) : launch_scan2(p, stream);
}

}  // namespace fkda
