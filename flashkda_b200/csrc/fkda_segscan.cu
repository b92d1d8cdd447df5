// Segment-parallel form of the inter-chunk recurrence for batches with few, long chains.
//
// The reference walks every (sequence, head) chain with one CTA from the first chunk to the last
// (csrc/smxx/fwd_kernel2.cuh:434-742), so a call with fewer chains than SMs leaves most of the GPU idle.  A run
// of chunks acts on the state Z = S^T ([v][k]) as an affine map, Z_end = Z_start M + N, because every chunk does
//     Z' = Z (diag(e) - w'^T kr) + u'^T kr .
// Here each sequence is cut into runs; the look-ahead scan kernel itself produces M (walk from the identity with
// u' = 0) and N (walk from zero) of the inner runs in parallel, this file chains them into the state at the start
// of every run, and a second launch of the scan kernel walks all runs in parallel from those states.
#include "fkda_common.cuh"

namespace fkda {

cudaError_t launch_scan2(const ScanParams& p, cudaStream_t stream);
cudaError_t launch_scan(const ScanParams& p, cudaStream_t stream);

namespace {

constexpr int kMapBytes = kD * kD * 4;
constexpr int kCmbM = 0;                                  // 2 x [128][128] fp32: transition maps, double-buffered
constexpr int kCmbZ = kCmbM + 2 * kMapBytes;              // [rows per CTA <= 32][128] fp32: this CTA's rows of the state
constexpr int kCmbBars = kCmbZ + 32 * kD * 4;
constexpr int kCmbSmemBytes = kCmbBars + 64 + 128;

// Z_start[run + 1] = Z_start[run] M[run] + N[run] for run = 1 .. n_segs-2; rows of Z are independent, so each CTA
// carries kRows of them (8, 16 or 32, by the number of chains) through all runs.  The 64 KB maps arrive by bulk copies two runs ahead, so the serial
// chain of runs sees shared-memory latency only.  fp32 throughout.
template <int kRows>
__global__ void __launch_bounds__(256) seg_combine_kernel(float* seg_buf, int n_segs, int* status) {
  constexpr int kPer = kRows / 2;                        // rows per thread
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
  const uint32_t sbase = smem_u32(smem);
  float (*z)[kD] = reinterpret_cast<float (*)[kD]>(smem + kCmbZ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kCmbBars + 16);
  const int tid = threadIdx.x;
  float* slots = seg_buf + static_cast<size_t>(blockIdx.x) * n_segs * 3 * kSegSlotFloats;
  auto load_map = [&](int run) {      // one thread
    const int b = (run - 1) & 1;
    mbar_arrive_expect_tx(sbase + kCmbBars + 8 * b, kMapBytes);
    bulk_g2s(sbase + kCmbM + b * kMapBytes, slots + (run * 3 + 0) * kSegSlotFloats, kMapBytes, sbase + kCmbBars + 8 * b);
  };
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(sbase + kCmbBars, 1);
    mbar_init(sbase + kCmbBars + 8, 1);
    fence_mbar_init();
    for (int run = 1; run <= 2 && run + 1 < n_segs; ++run) load_map(run);
  }
  const int k = tid & (kD - 1);
  const int rl = (tid >> 7) * kPer;                      // this thread's rows within the CTA's block
  const int r0 = blockIdx.y * kRows + rl;
  float acc[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    acc[i] = slots[(1 * 3 + 2) * kSegSlotFloats + static_cast<size_t>(r0 + i) * kD + k];
    z[rl + i][k] = acc[i];
  }
  __syncthreads();
  for (int run = 1; run + 1 < n_segs; ++run) {
    const int b = (run - 1) & 1;
    const float* N = slots + (run * 3 + 1) * kSegSlotFloats;
#pragma unroll
    for (int i = 0; i < kPer; ++i) acc[i] = N[static_cast<size_t>(r0 + i) * kD + k];
    const bool ok = mbar_wait(sbase + kCmbBars + 8 * b, ((run - 1) >> 1) & 1, abort_flag, 32);
    if (!__syncthreads_and(ok)) {
      if (tid == 0) {
        atomicCAS(status, kStatusOk, kStatusWaitTimeout);
        // do not leave while a copy may still be landing in this CTA's shared memory
        for (int bb = 0; bb < 2; ++bb) {
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(sbase + kCmbBars + 8 * bb, ((run - 1 + (bb != b)) >> 1) & 1))
            if (globaltimer_ns() - t0 > 20000000ull) break;
        }
      }
      break;
    }
    const float* M = reinterpret_cast<const float*>(smem + kCmbM + b * kMapBytes);
#pragma unroll 2
    for (int j = 0; j < kD; j += 4) {
      const float m0 = M[(j + 0) * kD + k], m1 = M[(j + 1) * kD + k], m2 = M[(j + 2) * kD + k], m3 = M[(j + 3) * kD + k];
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        const float4 zr = *reinterpret_cast<const float4*>(&z[rl + i][j]);
        acc[i] = fmaf(zr.x, m0, acc[i]);
        acc[i] = fmaf(zr.y, m1, acc[i]);
        acc[i] = fmaf(zr.z, m2, acc[i]);
        acc[i] = fmaf(zr.w, m3, acc[i]);
      }
    }
    __syncthreads();                  // every thread is done with z and with map buffer b
    if (tid == 0 && run + 3 < n_segs) load_map(run + 2);
    float* zs = slots + ((run + 1) * 3 + 2) * kSegSlotFloats;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      z[rl + i][k] = acc[i];
      zs[static_cast<size_t>(r0 + i) * kD + k] = acc[i];
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
  pass_cost_x100(chains * (2 * n_segs - 3), &compact1);
  pass_cost_x100(chains * (n_segs - 1), &compact2);
  if (kernel_choice) compact1 = compact2 = kernel_choice == 1;   // forced: 1 compact, 2 look-ahead
  p.seg_pass = 1;
  cudaError_t e = compact1 ? launch_scan(p, stream) : launch_scan2(p, stream);
  if (e != cudaSuccess) return e;
  if (n_segs > 2) {
    // one CTA per SM (two 64 KB map buffers); a step costs about 1.4 us + 0.3 us per row, so: the fewest rows per CTA
    // (8, 16, 32) that still keep the CTAs within one wave
    const int rows = chains * (kD / 8) <= kPlanSms ? 8 : (chains * (kD / 16) <= kPlanSms ? 16 : 32);
    auto kernel = rows == 32 ? seg_combine_kernel<32> : (rows == 16 ? seg_combine_kernel<16> : seg_combine_kernel<8>);
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCmbSmemBytes);
    if (e != cudaSuccess) return e;
    const dim3 grid(static_cast<unsigned>(chains), kD / rows);
    kernel<<<grid, 256, kCmbSmemBytes, stream>>>(seg_buf, n_segs, p.status);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  p.seg_pass = 2;
  return compact2 ? launch_scan(p, stream) : launch_scan2(p, stream);
}

}  // namespace fkda
