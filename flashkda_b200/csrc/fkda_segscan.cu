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

namespace {

constexpr int kRowsPerCta = 8;

// Z_start[run + 1] = Z_start[run] M[run] + N[run] for run = 1 .. n_segs-2; rows of Z are independent, so each CTA
// carries kRowsPerCta of them through all runs.  fp32 throughout.
__global__ void __launch_bounds__(256) seg_combine_kernel(float* seg_buf, int n_segs) {
  __shared__ float z[kRowsPerCta][kD];
  float* slots = seg_buf + static_cast<size_t>(blockIdx.x) * n_segs * 3 * kSegSlotFloats;
  const int k = threadIdx.x & (kD - 1);
  const int rl = (threadIdx.x >> 7) * 4;                 // this thread's four rows within the CTA's block
  const int r0 = blockIdx.y * kRowsPerCta + rl;
  float acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[i] = slots[(1 * 3 + 2) * kSegSlotFloats + static_cast<size_t>(r0 + i) * kD + k];
    z[rl + i][k] = acc[i];
  }
  __syncthreads();
  for (int run = 1; run + 1 < n_segs; ++run) {
    const float* M = slots + (run * 3 + 0) * kSegSlotFloats;
    const float* N = slots + (run * 3 + 1) * kSegSlotFloats;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = N[static_cast<size_t>(r0 + i) * kD + k];
#pragma unroll 8
    for (int j = 0; j < kD; ++j) {
      const float m = M[j * kD + k];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(z[rl + i][j], m, acc[i]);
    }
    __syncthreads();
    float* zs = slots + ((run + 1) * 3 + 2) * kSegSlotFloats;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      z[rl + i][k] = acc[i];
      zs[static_cast<size_t>(r0 + i) * kD + k] = acc[i];
    }
    __syncthreads();
  }
}

}  // namespace

cudaError_t launch_scan_segmented(const ScanParams& base, int n_segs, int seg_chunks, float* seg_buf, cudaStream_t stream) {
  ScanParams p = base;
  p.seg_chunks = seg_chunks;
  p.n_segs = n_segs;
  p.seg_buf = seg_buf;
  p.seg_pass = 1;
  cudaError_t e = launch_scan2(p, stream);
  if (e != cudaSuccess) return e;
  if (n_segs > 2) {
    const dim3 grid(static_cast<unsigned>(p.N) * p.H, kD / kRowsPerCta);
    seg_combine_kernel<<<grid, 256, 0, stream>>>(seg_buf, n_segs);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  p.seg_pass = 2;
  return launch_scan2(p, stream);
}

}  // namespace fkda
