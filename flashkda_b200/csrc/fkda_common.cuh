// Shared definitions for the sm_100a KDA prefill kernels: the per-chunk operand record that
// the prepare kernel writes and the scan kernel consumes, the shared-memory "core matrix"
// layout both sides agree on, and thin wrappers over the PTX this code relies on
// (mbarrier, bulk async copies, tcgen05 MMA / TMEM access, ldmatrix, mma.sync).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace fkda {

constexpr int kD = 128;            // head dimension (K = V = 128, as in csrc/flash_kda.cpp:110 of the reference)
constexpr int kChunk = 32;         // tokens per chunk of the WY formulation
constexpr float kLog2e = 1.4426950408889634f;

// ---- per-(head, chunk) operand record -----------------------------------------------------
// All bf16 matrices use the core-matrix layout below, so that a record is at the same time
// (a) what ldmatrix wants in the prepare kernel and (b) a no-swizzle tcgen05 operand tile that
// the scan kernel can bring into shared memory with one bulk copy.
//   KR  [32 tok][128 k]  khat * decay to chunk end
//   MQK [32 tok][32 tok] tril(q+ k-^T)
//   E   [128] fp32       whole-chunk decay per channel
//   WP  [32 tok][128 k]  T diag(beta) k+      (k+ = khat * decay from chunk start)
//   QP  [32 tok][128 k]  qhat * decay from chunk start * scale   (directly after WP: the two
//                        form one [64][128] operand tile)
//   UP  [128 v][32 tok]  (T diag(beta) v)^T   (core layout; read row-wise by the scan's U epilogue)
constexpr int kRecKR = 0;
constexpr int kRecMQK = 8192;
constexpr int kRecE = 10240;
constexpr int kRecWP = 10752;
constexpr int kRecQP = 18944;
constexpr int kRecUP = 27136;
constexpr int kRecBytes = 35328;

// workspace header (bytes): [0,64) status words, [256, 256+4*(N+1)) chunk prefix, records after
constexpr int kWsHeaderBytes = 256;

// status codes written to workspace status word 0 (first error wins)
enum : int {
  kStatusOk = 0,
  kStatusBadCuSeqlens = 1,   // cu_seqlens not monotone / out of range
  kStatusWaitTimeout = 2,    // a bounded mbarrier wait gave up
};

// Core-matrix layout of a [rows][cols] bf16 tile: 8x8 blocks of 128 contiguous bytes (8 rows of
// 16 B); blocks adjacent along the columns are 128 B apart, 8-row groups are cols*16 B apart.
__host__ __device__ __forceinline__ constexpr int core_off(int r, int c, int cols) {
  return (r >> 3) * (cols * 16) + (c >> 3) * 128 + (r & 7) * 16 + (c & 7) * 2;
}

// ---- small numeric helpers ---------------------------------------------------------------------
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// sigmoid through the MUFU tanh, the form the reference kernels use (csrc/smxx/utils.cuh:50-53)
__device__ __forceinline__ float sigmoid_fast(float x) { return fmaf(tanh_approx(0.5f * x), 0.5f, 0.5f); }

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with a suspend-time hint: the hardware parks the warp until the phase completes or about `ns` nanoseconds
// have passed, so a waiter takes no issue slots from the warps that work.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait built on it, for kernels in which most warps wait most of the time.  Same contract as mbar_wait.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_hint(bar, parity, 4000u)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait_hint(bar, parity, 4000u)) {
    const int f = *abort_flag;
    if (f > 0) return false;
    const uint64_t limit = f < 0 ? static_cast<uint64_t>(-f) * 1000ull : 2000000000ull;
    if (globaltimer_ns() - t0 > limit) {
      *abort_flag = 1;
      return false;
    }
  }
  return true;
}
// Non-blocking probe of a barrier phase (for polling loops that watch several barriers).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Gives up after `kWaitLimitNs` or as soon as another thread of the CTA has given
// up (`*abort_flag > 0`); the caller then leaves its loop, so a lost arrival can never hang
// the GPU.  Returns true when the barrier phase completed.  A kernel may initialise the flag word to -L instead of 0:
// nobody has given up, and the limit is L microseconds instead (how a test makes a wait run out quickly).
constexpr uint64_t kWaitLimitNs = 2000000000ull;
// `backoff_ns` > 0 makes a waiter that is not on the critical path sleep between probes, so that it does not take
// issue slots from the warps that are.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t backoff_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (backoff_ns) __nanosleep(backoff_ns);
    if (((++spins) & 63u) == 0u) {
      const int f = *abort_flag;
      if (f > 0) return false;
      const uint64_t limit = f < 0 ? static_cast<uint64_t>(-f) * 1000ull : kWaitLimitNs;
      if (globaltimer_ns() - t0 > limit) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// generic-proxy writes to shared memory -> visible to the async proxy (bulk copies, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- bulk async copies (the TMA engine, untiled form; 16-byte aligned addresses and sizes) ------
__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}
// 16-byte asynchronous global->shared copy; `src_bytes` = 0 writes zeros instead (the address must still be valid).
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Fire-and-forget prefetch of a contiguous global range into L2 (16-byte aligned address, size multiple of 16).
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// ---- tcgen05: TMEM allocation, MMA, commit, fences -----------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, no swizzle.  For a K-major operand `lbo` is the byte distance
// between core matrices adjacent along K and `sbo` the distance between 8-row groups; for an
// MN-major operand `sbo` is the distance between core matrices adjacent along M/N and `lbo`
// the distance between 8-deep groups along K.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version of this architecture
  return d;         // layout type (bits 61..63) = 0: no swizzle
}
// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A is read from tensor memory (lane = row, each 32-bit column holds two
// consecutive K elements, low half first); issued by one thread.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns; lane i of the warp reads/writes TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
      "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}

// 16-lane fragment shapes.  16x256b.x8: 16 TMEM lanes x 64 columns; thread t of the warp holds, for j = 0..7, registers
// 4j, 4j+1 = (lane t/4, columns 8j + 2(t%4), +1) and 4j+2, 4j+3 = (lane t/4 + 8, same columns) - the accumulator
// fragment of mma.sync.  16x128b.x8: 16 lanes x 32 columns; registers 2j, 2j+1 = (lane t/4 | t/4 + 8, column 4j + t%4).
// A thread therefore touches a quarter of the columns only, and two fp32 columns that pack into one bf16x2 word
// sit in one thread.  The lane field of the address selects lanes 0-15 or 16-31 of the warp's quadrant.
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x8.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};" ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%16], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}

// ---- warp-level mma.sync helpers (prepare kernel's small products) --------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void stsm_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8,f32) += A(16x8,tf32,row) * B(8x8,tf32,col); operands are fp32 bit patterns rounded to tf32 by the caller.
// Fragments (g = lane / 4, t = lane % 4): a0 (g, t), a1 (g+8, t), a2 (g, t+4), a3 (g+8, t+4); b0 (k = t, n = g),
// b1 (k = t+4, n = g); c0, c1 (g, 2t | 2t+1), c2, c3 (g+8, same).
__device__ __forceinline__ void mma_tf32_1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

// ---- small helpers shared by the token-parallel kernels ---------------------------------------------
// byte offset of 16-byte chunk `chunk` of token row `row` in a staged [rows][256 B] tile whose chunks are XOR-swizzled by
// the row index (conflict-free for row-wise 16-byte reads and for ldmatrix over eight consecutive rows)
// a, b (fp32 bit patterns) *= e.x, e.y as one packed fp32x2 multiply (same rounding as two scalar multiplies)
__device__ __forceinline__ void mul2(uint32_t& a, uint32_t& b, const float2& e) {
  unsigned long long x, y, z;
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "r"(a), "r"(b));
  asm("mov.b64 %0, {%1, %2};" : "=l"(y) : "f"(e.x), "f"(e.y));
  asm("mul.f32x2 %0, %1, %2;" : "=l"(z) : "l"(x), "l"(y));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(z));
}

__device__ __forceinline__ int stage_off(int row, int chunk) { return row * 256 + ((chunk ^ (row & 7)) << 4); }

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
  f[0] = bf_lo(w.x); f[1] = bf_hi(w.x); f[2] = bf_lo(w.y); f[3] = bf_hi(w.y);
  f[4] = bf_lo(w.z); f[5] = bf_hi(w.z); f[6] = bf_lo(w.w); f[7] = bf_hi(w.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
// transpose of an 8x8 tile of 16-bit elements held one row pair per thread (mma fragment layout)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// ---- kernel parameter blocks ---------------------------------------------------------------
struct PrepParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* g;
  const __nv_bfloat16* beta;
  const float* A_log;
  const float* dt_bias;
  const int64_t* cu_seqlens;   // device, N+1 entries, or nullptr (fixed length)
  const int* chunk_prefix;     // device, N+1 entries (varlen only)
  uint8_t* records;            // record r of head h at ((h * total_chunks + r) * kRecBytes)
  int* status;
  int64_t T;                   // tokens per sequence (fixed length)
  int64_t T_total;
  int H;
  int N;
  int total_chunks;            // records per head (upper bound for varlen)
  float scale;
  float gate_scale;            // lower_bound * log2(e)
  int dbg;                     // tuning aid: bit mask of phases to skip (0 in production)
  int wait_limit_us;           // 0: the waits give up after kWaitLimitNs; else after this many microseconds (test aid)
  int first_load_only;         // 0: normal; 1: a CTA of the pipelined kernel loads the tiles of its first item only (test aid)
};

struct ScanParams {
  const uint8_t* records;
  const int64_t* cu_seqlens;
  const int* chunk_prefix;
  const int* seq_order;        // device, N entries: sequences by decreasing length (varlen only), or nullptr
  const void* initial_state;   // [N][H][128 v][128 k] or nullptr
  void* final_state;           // same, or nullptr
  __nv_bfloat16* out;          // [T_total][H][128]
  int* status;
  int64_t T;
  int64_t T_total;
  int H;
  int N;
  int total_chunks;
  int state_fp32;              // dtype of both state tensors: 1 = fp32, 0 = bf16
  // Segment-parallel form (batches with few chains): every sequence is cut into n_segs runs of
  // seg_chunks chunks (varlen: of *seg_chunks_dev chunks, runs beyond a sequence's end being empty) and each CTA walks one run.  Pass 1 walks run 0 from the caller's state (its outputs are
  // final) and, for the runs 1 .. n_segs-2, the two halves of the affine map  Z_end = Z_start M + N  that a run
  // applies to the state Z = S^T: N from a zero state, M from the identity with u' taken as zero.  A small kernel
  // chains the maps into the state at the start of every run; pass 2 walks runs 1 .. n_segs-1 from those.
  int seg_chunks;              // 0: one CTA per whole sequence
  int n_segs;
  int seg_pass;                // 1 or 2
  float* seg_buf;              // fp32 [(n*H + h)][n_segs][3][128][128]: 0 = M, 1 = N, 2 = state at the start of the run
  const int* select;           // device word, or nullptr: the kernel runs only if *select == select_want
  int select_want;
  const int* seg_chunks_dev;   // varlen batches: run length decided on the device from the longest sequence (else nullptr)
  // Test aids of the look-ahead kernel's give-up path (both 0 in production): a wait limit in microseconds instead of
  // the default, and a number of records after which the copy producer stops issuing copies, so that the consumers'
  // next wait runs out with nothing in flight.
  int wait_limit_us;
  int stop_copies_after;
};

constexpr int kSegMapStride = 136;             // floats per row of a transition map M in its slot: the map chaining reads
                                               // whole slots into shared memory, where this stride keeps its fragment loads conflict-free
constexpr int64_t kSegSlotFloats = 128 * kSegMapStride;   // every slot has room for the padded form
constexpr int kDefaultSms = 148;       // SMs of a B200: assumed where no device can be asked

// SM count of the current device, asked once per device and cached; the kernel-selection rules, the planner of the
// segment-parallel form and the workspace size all use this one figure, so that a size query and the launch agree.
inline int device_sm_count() {
  static std::atomic<int> cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return kDefaultSms;
  }
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    return kDefaultSms;
  }
  cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// Opt-in of a kernel to its dynamic shared-memory size, made once per device instead of before every launch.
struct SmemOptIn {
  std::atomic<unsigned long long> done{0};
  template <class Kernel>
  cudaError_t ensure(Kernel kernel, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return e;
  }
};

// Fixed-length sequences of at most this many tokens take the fused short-sequence kernel (fkda_short16.cu).
constexpr int64_t kFusedMaxT = 32;

// Duration of a pass of `ctas` CTAs in hundredths of one chunk step of the look-ahead kernel, per chunk of run length,
// and the kernel that achieves it: the look-ahead kernel runs one CTA per SM, the compact kernel two at 1.58 times the
// step (measured).
inline int64_t pass_cost_x100(int64_t ctas, bool* compact, int64_t sms, int64_t la_step_x100 = 100) {
  const int64_t la = (ctas + sms - 1) / sms * la_step_x100, co = (ctas + 2 * sms - 1) / (2 * sms) * 158;
  *compact = co < la;
  return co < la ? co : la;
}

// How many runs to cut each sequence of a batch into (1 = walk whole sequences), and their length in chunks (varlen
// batches: called with the average sequence length; the run length is then set on the device from the longest one).  Pass 1 holds chains * (2 n - 3) CTAs and pass 2 chains * (n - 1), both walking ceil(chunks / n) chunks, each
// on whichever recurrence kernel gets that many CTAs through faster; chaining the maps costs about three chunk steps
// per run.  The plan is a pure function of the sizes and the device's SM count, so that the workspace size and the
// launch agree.
inline int plan_segments(int64_t chains, int64_t chunks, int* seg_chunks, int64_t sms) {
  *seg_chunks = 0;
  if (chains <= 0 || chains * 3 > sms || chunks < 48) return 1;
  bool c;
  const int64_t whole = pass_cost_x100(chains, &c, sms) * chunks;
  int64_t best = whole, best_n = 1;
  for (int64_t n = 3; n <= 160; ++n) {
    const int64_t len = (chunks + n - 1) / n;
    if (len < 8) break;
    if ((n - 1) * len >= chunks) continue;       // the last run would be empty
    // (a run walks its chunks about a tenth more slowly than a whole sequence; each pass costs about ten chunk steps of
    // launch, set-up and state traffic; a step of the map chaining about two and a half, per wave of its chains x 8 CTAs)
    const int64_t cmb_waves = (chains * 8 + sms - 1) / sms;
    const int64_t cost = (pass_cost_x100(chains * (2 * n - 3), &c, sms, 110) + pass_cost_x100(chains * (n - 1), &c, sms, 110)) * len + 100 * 20 +
                         250 * (n - 2) * cmb_waves;
    if (cost < best) { best = cost; best_n = n; }
  }
  if (best_n == 1 || best * 4 > whole * 3) return 1;
  *seg_chunks = static_cast<int>((chunks + best_n - 1) / best_n);
  return static_cast<int>(best_n);
}

// What one CTA of a recurrence kernel walks: a whole (sequence, head) chain, or, in the segment-parallel form (kSeg), one
// run of it in one of three variants - 0: the recurrence proper; 1: offset half of the run's affine map (zero state in, no
// output); 2: transition half (identity in, u' taken as zero, no output).  Pass 1 holds, per chain, run 0 (variant 0)
// followed by (variant 1, variant 2) of the runs 1 .. n_segs-2; pass 2 holds the runs 1 .. n_segs-1 (variant 0).
struct ChainView {
  int n, h;
  int64_t bos, eos;            // tokens of this walk
  int chunk_base, nchunks;     // first record of this walk (index within the head's records), number of chunks
  const void* init_base;       // [128 v][128 k] block the walk starts from (init_mode 1: fp32, 2: bf16), or nothing
  int init_mode;               // 0 = zero, 1 = fp32, 2 = bf16, 3 = identity
  void* fin_base;              // where the state goes afterwards, or nullptr
  int fin_fp32;
  int fin_stride;              // elements per row there (128; a transition map's slot: kSegMapStride)
  bool write_out, zero_up;
};
template <bool kSeg>
__device__ __forceinline__ ChainView chain_view(const ScanParams& p, int block) {
  ChainView cv;
  int chain = block, seg = 0, variant = 0;
  if constexpr (kSeg) {
    const int per = p.seg_pass == 1 ? 2 * p.n_segs - 3 : p.n_segs - 1;
    chain = block / per;
    const int j = block - chain * per;
    if (p.seg_pass == 1) {
      if (j > 0) { seg = 1 + ((j - 1) >> 1); variant = 1 + ((j - 1) & 1); }
    } else {
      seg = 1 + j;
    }
  }
  const int slot = chain / p.H;
  cv.h = chain - slot * p.H;
  cv.n = p.seq_order != nullptr ? p.seq_order[slot] : slot;     // varlen: longest sequences first
  if (p.cu_seqlens != nullptr) {
    cv.bos = p.cu_seqlens[cv.n];
    cv.eos = p.cu_seqlens[cv.n + 1];
    cv.bos = cv.bos < 0 ? 0 : (cv.bos > p.T_total ? p.T_total : cv.bos);
    cv.eos = cv.eos < cv.bos ? cv.bos : (cv.eos > p.T_total ? p.T_total : cv.eos);
    cv.chunk_base = p.chunk_prefix[cv.n];
  } else {
    cv.bos = static_cast<int64_t>(cv.n) * p.T;
    cv.eos = cv.bos + p.T;
    cv.chunk_base = cv.n * static_cast<int>((p.T + kChunk - 1) / kChunk);
  }
  cv.nchunks = static_cast<int>((cv.eos - cv.bos + kChunk - 1) / kChunk);
  {  // never read past the records of this head, whatever cu_seqlens claims
    const int avail = p.total_chunks > cv.chunk_base ? p.total_chunks - cv.chunk_base : 0;
    if (cv.nchunks > avail) cv.nchunks = avail;
  }
  const size_t chain_state = (static_cast<size_t>(cv.n) * p.H + cv.h) * kD * kD;
  cv.init_base = nullptr;
  cv.init_mode = 0;
  cv.fin_base = nullptr;
  cv.fin_fp32 = p.state_fp32;
  cv.fin_stride = kD;
  if (p.initial_state != nullptr) {
    cv.init_mode = p.state_fp32 ? 1 : 2;
    cv.init_base = static_cast<const uint8_t*>(p.initial_state) + chain_state * (p.state_fp32 ? 4 : 2);
  }
  if (p.final_state != nullptr) cv.fin_base = static_cast<uint8_t*>(p.final_state) + chain_state * (p.state_fp32 ? 4 : 2);
  if constexpr (kSeg) {
    float* slots = p.seg_buf + (static_cast<size_t>(cv.n) * p.H + cv.h) * p.n_segs * 3 * kSegSlotFloats;
    const int run_len = p.seg_chunks_dev != nullptr ? *p.seg_chunks_dev : p.seg_chunks;
    const int c_begin = seg * run_len < cv.nchunks ? seg * run_len : cv.nchunks;
    const int c_end = (seg == p.n_segs - 1 || (seg + 1) * run_len > cv.nchunks) ? cv.nchunks : (seg + 1) * run_len;
    if (seg < p.n_segs - 1) {
      const int64_t run_end = cv.bos + static_cast<int64_t>(c_end) * kChunk;
      cv.eos = run_end < cv.eos ? run_end : cv.eos;
    }
    cv.bos += static_cast<int64_t>(c_begin) * kChunk;
    cv.chunk_base += c_begin;
    cv.nchunks = c_end - c_begin;
    if (p.seg_pass == 1) {
      if (variant == 0) {
        cv.fin_base = slots + (1 * 3 + 2) * kSegSlotFloats;                 // state at the start of run 1
      } else {
        cv.init_mode = variant == 2 ? 3 : 0;
        cv.init_base = nullptr;
        cv.fin_base = slots + (seg * 3 + (variant == 2 ? 0 : 1)) * kSegSlotFloats;
        if (variant == 2) cv.fin_stride = kSegMapStride;
      }
      cv.fin_fp32 = 1;
    } else {
      cv.init_mode = 1;
      cv.init_base = slots + (seg * 3 + 2) * kSegSlotFloats;
      if (seg != p.n_segs - 1) cv.fin_base = nullptr;
    }
  }
  cv.write_out = !kSeg || variant == 0;
  cv.zero_up = kSeg && variant == 2;
  return cv;
}

}  // namespace fkda
