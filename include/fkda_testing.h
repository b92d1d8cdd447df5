/*
 * fkda_testing.h -- test-support entry points of libfkda.so.  Not part of the operator's ABI
 * (include/fkda.h): these exist so that the GPU tests can exercise building blocks and failure
 * paths of the kernels in isolation.  None has a counterpart in the reference, which ships no
 * unit tests of its device helpers (its tests call flash_kda.fwd only, tests/test_fwd_full.py).
 */
#ifndef FKDA_TESTING_H_
#define FKDA_TESTING_H_

#include "fkda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* One-CTA tcgen05 products in the descriptor flavours the kernels use (see umma_selftest_kernel in
 * csrc/fkda_aux.cu for the modes).  A, B bf16 row-major, D fp32 row-major, all device pointers;
 * status int32, set to 1 if a bounded wait gave up. */
int fkda_selftest_umma(const void* A, const void* B, float* D, int mode, int reps, int* status,
                       void* cuda_stream);

/* Self-test of the 16-lane tensor-memory fragment shapes the recurrence kernels rely on (tcgen05.ld/st
 * 16x256b and 16x128b): out = uint32[4][2048], the register <-> (lane, column) maps as read back
 * through the 32x32b shape (see tmem_layout_probe_kernel).  One warp, a few microseconds. */
int fkda_debug_tmem_layout_probe(void* out, void* cuda_stream);

/* The give-up path of the bounded waits, provoked without a fault: fkda_prepare followed by the
 * look-ahead recurrence kernel on whole sequences, in which the copy producer of every chain stops
 * issuing copies after `stop_copies_after` records and every wait gives up after `wait_limit_us`
 * microseconds instead of two seconds.  A chain with more records than that then finds a barrier
 * that nothing will complete; its CTA must record status 2, release its tensor memory and return.
 * Nothing is in flight when the wait runs out.  Read the outcome with fkda_read_status. */
int fkda_debug_scan_giveup(const fkda_fwd_params* p, int stop_copies_after, int wait_limit_us, void* cuda_stream);

/* The same for the token-parallel stage: fkda_prepare on the pipelined kernel, in which every CTA loads the tiles of
 * its first item only and every wait gives up after `wait_limit_us` microseconds.  A CTA with a second item waits for
 * tiles that nothing will bring; it must record status 2, wait for what it still has in flight, release its tensor
 * memory and return.  (A CTA has a second item once the call has more than three (chunk, head) items per SM.) */
int fkda_debug_prepare_giveup(const fkda_fwd_params* p, int wait_limit_us, void* cuda_stream);

#ifdef FKDA_TUNING
/* The following exist only in builds made with -DFKDA_TUNING (FKDA_NVCC_EXTRA=-DFKDA_TUNING python -m
 * flashkda_b200.build --force). */

/* Registers (or, with NULL, removes) a device buffer of 32*16 int64 into which CTA 0 of the TMA + tcgen05 token-parallel
 * kernel records clock64() at the stage boundaries of its first 32 items (events: see PTRACE in csrc/fkda_prepare_tc.cu). */
int fkda_debug_set_prepare_trace(void* device_buffer);

/* Registers (or, with NULL, removes) a device buffer of 6*32*8 uint64 into which CTA 0 of the look-ahead
 * recurrence kernel records clock64() at a few points of each warp role for its first 32 chunks. */
int fkda_debug_set_scan_trace(void* device_buffer);

/* One CTA of `nwarps` (<= 16) warps times `reps` 32-column TMEM loads / stores per warp;
 * out = int64[nwarps][4] cycles for {loads, stores, 16-column stores, load+store round trips}. */
int fkda_debug_tmem_bench(int nwarps, int reps, void* out, void* cuda_stream);

/* `issuers` (1..4) threads of one CTA each issue `reps` products of `ksteps` (1..8) tcgen05.mma
 * instructions (M = 128, K = 16, N = n in {32, 64, 128}; A from shared or tensor memory) and wait for their commit;
 * out = int64[issuers][2] cycles {until the last instruction was issued, until the commit arrived}; status[0] = 1 if
 * a bounded wait gave up. */
int fkda_debug_umma_bench(int issuers, int reps, int ksteps, int n, int a_in_tmem, void* out, int* status, void* cuda_stream);
#endif

#ifdef __cplusplus
}
#endif
#endif /* FKDA_TESTING_H_ */
