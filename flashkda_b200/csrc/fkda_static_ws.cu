// fkda_fwd_static_ws: the forward pass for callers that are not allowed to allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the operator:
// an inference server that sized and pinned its whole memory pool at start-up and forbids
// allocations afterwards, a plugin that runs inside someone else's memory budget, or code
// running while the framework's allocator is locked.  The normal entry point, fkda_fwd, already
// allocates nothing itself, but it needs a caller-provided workspace, which such a caller may
// have no way to obtain.  This entry point takes the same parameter block, ignores its
// `workspace` fields and uses a scratch array that is part of the library image instead.
//
// The scratch is a file-scope __device__ array of kStaticWsBytes (64 MiB).  Every GPU on which a
// process loads this library holds that much memory until the process exits, which is why the
// limit is modest: it covers problems with (tokens/32 + sequences) * heads <= 1899 chunk
// records, e.g. 1888 tokens at 32 heads.  Larger problems are rejected with an error; use
// fkda_fwd with your own workspace for those.
//
// In host code the array's name is only a handle: the device address has to be asked for with
// cudaGetSymbolAddress while the device in question is current.  That is done on the first call
// on each device and cached (the cache does not survive a cudaDeviceReset), so make that first call outside any
// stream capture.  All calls on a
// device share the one array and it keeps whatever the previous call left in it: the status
// header is cleared at the start of every call and every record that is read is rewritten
// first, but two calls that overlap on the GPU (different streams, or different threads) race
// on it and must be serialised by the caller.
#include <cstdio>
#include <mutex>

#include "../../include/fkda.h"
#include "fkda_common.cuh"

namespace {

constexpr int64_t kStaticWsBytes = 64ll << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];

std::mutex g_mu;
void* g_ws_ptr[kMaxDevices] = {};
thread_local char g_msg[256] = "";

}  // namespace

extern "C" {

const char* fkda_static_ws_last_error(void) { return g_msg; }

int64_t fkda_static_ws_capacity(void) { return kStaticWsBytes; }

int fkda_fwd_static_ws(const fkda_fwd_params* p, void* cuda_stream) {
  g_msg[0] = '\0';
  if (!p) {
    snprintf(g_msg, sizeof(g_msg), "params is NULL");
    return FKDA_ERR_INVALID_ARGUMENT;
  }
  // size check first, with this entry point's own limit in the message
  int64_t records_off = 0, record_bytes = 0, chunks = 0;
  if (p->B <= 0 || p->H <= 0 || p->T < 0 || p->N <= 0 ||
      fkda_workspace_layout(p->B * p->T, p->H, p->N, p->cu_seqlens != nullptr, p->T, &records_off, &record_bytes, &chunks) != FKDA_OK) {
    snprintf(g_msg, sizeof(g_msg), "bad sizes (B, H, N must be positive, T non-negative)");
    return FKDA_ERR_INVALID_ARGUMENT;
  }
  const int64_t need = records_off + chunks * p->H * record_bytes;
  if (need > kStaticWsBytes) {
    snprintf(g_msg, sizeof(g_msg),
             "problem needs %lld bytes of scratch but the built-in scratch holds %lld: use fkda_fwd with a caller workspace",
             (long long)need, (long long)kStaticWsBytes);
    return FKDA_ERR_WORKSPACE_TOO_SMALL;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_msg, sizeof(g_msg), "cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    return FKDA_ERR_CUDA;
  }
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_ws_ptr[dev] == nullptr) {
      // one-time set-up for this device: translate the symbol into this device's address
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_static_ws);
      if (e != cudaSuccess || ptr == nullptr) {
        snprintf(g_msg, sizeof(g_msg), "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        return FKDA_ERR_CUDA;
      }
      g_ws_ptr[dev] = ptr;
    }
    ws = g_ws_ptr[dev];
  }
  fkda_fwd_params q = *p;
  q.workspace = ws;
  q.workspace_bytes = kStaticWsBytes;
  {
    // few long chains would be cut into runs, which needs room beyond the records: where that room is missing the
    // sequences are walked whole instead (slower, same result) rather than refused.  Decided on this call's exact
    // layout, not on the upper bound that a size query gives.
    int64_t exact = 0;
    if (fkda_workspace_bytes_exact(p->B * p->T, p->H, p->N, p->cu_seqlens != nullptr, p->T, p->flags, &exact) == FKDA_OK &&
        exact > kStaticWsBytes)
      q.flags |= FKDA_FLAG_SCAN_NO_SEGMENTS;
  }
  const int rc = fkda_fwd(&q, cuda_stream);
  if (rc != FKDA_OK) snprintf(g_msg, sizeof(g_msg), "%s", fkda_last_error());
  return rc;
}

int fkda_static_ws_read_status(void* cuda_stream, int* status) {
  int dev = -1;
  void* ws = nullptr;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices) {
    std::lock_guard<std::mutex> lock(g_mu);
    ws = g_ws_ptr[dev];
  }
  if (ws == nullptr) {
    snprintf(g_msg, sizeof(g_msg), "no call of fkda_fwd_static_ws has been made on this device yet");
    return FKDA_ERR_INVALID_ARGUMENT;
  }
  const int rc = fkda_read_status(ws, cuda_stream, status);
  if (rc != FKDA_OK) snprintf(g_msg, sizeof(g_msg), "%s", fkda_last_error());
  return rc;
}

}  // extern "C"
