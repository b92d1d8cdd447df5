"""ctypes binding of libfkda.so and the torch-facing wrappers.

`fwd` keeps the reference's Python signature (flash_kda/__init__.py:5) and error behaviour:
every argument problem raises RuntimeError before anything is launched (the reference's
TORCH_CHECKs, csrc/flash_kda.cpp:44-174, surface the same way), results are written in place
into `out` / `final_state`, the call returns None and does not synchronise.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfkda.so")
_lib = None

FLAG_SCAN_SIMT = 0x1
FLAG_SCAN_PLAIN = 0x2
FLAG_SCAN_LOOKAHEAD = 0x4
FLAG_SCAN_NO_SEGMENTS = 0x8
FLAG_NO_FUSED_SHORT = 0x10
FLAG_REFERENCE_ROUNDING = 0x20
FLAG_FUSED_ANY_T = 0x40
FLAG_PREPARE_TCGEN05 = 0x80
FLAG_PREPARE_MMA_SYNC = 0x20000


def FLAG_SEGMENTS(n: int) -> int:
    """Flag bits that cut every sequence of the batch into `n` runs walked in parallel."""
    return (int(n) & 0xff) << 8
_STATE_NONE, _STATE_BF16, _STATE_FP32 = 0, 1, 2


class FwdParams(ctypes.Structure):
    """Mirror of `fkda_fwd_params` (include/fkda.h)."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("g", ctypes.c_void_p),
        ("beta", ctypes.c_void_p), ("out", ctypes.c_void_p), ("A_log", ctypes.c_void_p),
        ("dt_bias", ctypes.c_void_p), ("initial_state", ctypes.c_void_p), ("final_state", ctypes.c_void_p),
        ("cu_seqlens", ctypes.c_void_p), ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
        ("B", ctypes.c_int64), ("T", ctypes.c_int64), ("H", ctypes.c_int64), ("N", ctypes.c_int64),
        ("scale", ctypes.c_float), ("lower_bound", ctypes.c_float), ("state_dtype", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
    ]


def lib_path() -> str:
    return _LIB_PATH


def lib():
    """Loads libfkda.so once.  Raises if it has not been built (python -m flashkda_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m flashkda_b200.build`. "
                "flash_kda has no CPU or PyTorch fallback.")
        L = ctypes.CDLL(_LIB_PATH)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.fkda_get_workspace_size.argtypes = [i64, i64, i64, ctypes.POINTER(i64)]
        L.fkda_get_workspace_size_flags.argtypes = [i64, i64, i64, i64, ctypes.POINTER(i64)]
        L.fkda_plan_segments.argtypes = [i64, i64, ctypes.POINTER(ci), ctypes.POINTER(ci)]
        L.fkda_fwd.argtypes = [ctypes.POINTER(FwdParams), vp]
        L.fkda_prepare.argtypes = [ctypes.POINTER(FwdParams), vp]
        L.fkda_scan.argtypes = [ctypes.POINTER(FwdParams), vp]
        L.fkda_prologue.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_float, i64, i64, vp, vp, vp, vp, vp]
        L.fkda_workspace_layout.argtypes = [i64, i64, i64, ci, i64, ctypes.POINTER(i64), ctypes.POINTER(i64),
                                            ctypes.POINTER(i64)]
        L.fkda_read_status.argtypes = [vp, vp, ctypes.POINTER(ci)]
        L.fkda_selftest_umma.argtypes = [vp, vp, vp, ci, ci, vp, vp]
        L.fkda_debug_tmem_layout_probe.argtypes = [vp, vp]
        L.fkda_debug_tmem_layout_probe.restype = ci
        L.fkda_debug_scan_giveup.argtypes = [ctypes.POINTER(FwdParams), ci, ci, vp]
        L.fkda_debug_scan_giveup.restype = ci
        L.fkda_debug_prepare_giveup.argtypes = [ctypes.POINTER(FwdParams), ci, vp]
        L.fkda_debug_prepare_giveup.restype = ci
        if hasattr(L, "fkda_debug_umma_bench"):        # builds made with -DFKDA_TUNING only
            L.fkda_debug_umma_bench.argtypes = [ci, ci, ci, ci, ci, vp, vp, vp]
            L.fkda_debug_umma_bench.restype = ci
        L.fkda_last_error.restype = ctypes.c_char_p
        L.fkda_version.restype = ctypes.c_char_p
        for name in ("fkda_get_workspace_size", "fkda_get_workspace_size_flags", "fkda_plan_segments", "fkda_fwd", "fkda_prepare", "fkda_scan", "fkda_prologue",
                     "fkda_workspace_layout", "fkda_read_status", "fkda_selftest_umma"):
            getattr(L, name).restype = ci
        _lib = L
    return _lib


def last_error() -> str:
    return lib().fkda_last_error().decode()


def _check(rc):
    if rc != 0:
        raise RuntimeError(f"flash_kda: {last_error()} (code {rc})")


def get_workspace_size(T_total: int, H: int, N: int = 1, flags: int = 0) -> int:
    """Bytes of scratch `fwd` allocates per call (counterpart of the reference's
    get_workspace_size, csrc/flash_kda.cpp:5-26; the figure itself differs).  `flags` matters only
    with FLAG_SEGMENTS(n), which needs room for the per-run states."""
    out = ctypes.c_int64(0)
    if flags:
        _check(lib().fkda_get_workspace_size_flags(T_total, H, N, int(flags), ctypes.byref(out)))
    else:
        _check(lib().fkda_get_workspace_size(T_total, H, N, ctypes.byref(out)))
    return out.value


def plan_segments(chains: int, chunks_per_sequence: int):
    """(runs per sequence, chunks per run) the recurrence uses for a batch of `chains` chains of that many chunks (varlen: the
    average sequence length; the run length then follows the longest sequence); (1, 0) = whole sequences."""
    a, b = ctypes.c_int(0), ctypes.c_int(0)
    _check(lib().fkda_plan_segments(chains, chunks_per_sequence, ctypes.byref(a), ctypes.byref(b)))
    return a.value, b.value


def workspace_layout(T_total, H, N, varlen, T_per_seq):
    a, b, c = ctypes.c_int64(0), ctypes.c_int64(0), ctypes.c_int64(0)
    _check(lib().fkda_workspace_layout(T_total, H, N, int(bool(varlen)), T_per_seq, ctypes.byref(a),
                                       ctypes.byref(b), ctypes.byref(c)))
    return a.value, b.value, c.value


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _validate(q, k, v, g, beta, out, A_log, dt_bias, initial_state, final_state, cu_seqlens, workspace=None):
    """The reference's checks, in the reference's order and wording (csrc/flash_kda.cpp:44-174),
    plus a same-device check the reference lacks."""
    main = (q, k, v, g, beta, out)
    _require(all(isinstance(t, torch.Tensor) for t in main + (A_log, dt_bias)), "all inputs must be tensors")
    if workspace is not None:
        # what the reference requires of its workspace argument (csrc/flash_kda.cpp:44-47), checked before its pointer
        # and size reach the kernels
        _require(isinstance(workspace, torch.Tensor) and workspace.is_cuda and workspace.is_contiguous(),
                 "workspace must be a contiguous CUDA tensor")
        _require(workspace.dtype == torch.uint8, "workspace must be uint8")
        _require(workspace.device == q.device, "workspace must be on the same CUDA device as q")
    _require(all(t.is_cuda for t in main), "all tensors must be on CUDA")
    _require(all(t.is_contiguous() for t in main), "all tensors must be contiguous")
    for name, t in zip(("q", "k", "v", "g", "beta", "out"), main):
        _require(t.dtype == torch.bfloat16, f"{name} must be bfloat16")
    state_dtype = _STATE_NONE
    for name, st in (("initial_state", initial_state), ("final_state", final_state)):
        if st is not None:
            _require(st.is_cuda and st.is_contiguous(), f"{name} must be contiguous CUDA tensor")
            _require(st.dtype in (torch.bfloat16, torch.float32), f"{name} must be bfloat16 or float32")
    if initial_state is not None and final_state is not None:
        _require(initial_state.dtype == final_state.dtype, "initial_state and final_state must have the same dtype")
    for st in (initial_state, final_state):
        if st is not None:
            state_dtype = _STATE_FP32 if st.dtype == torch.float32 else _STATE_BF16
    _require(A_log.is_cuda and A_log.is_contiguous(), "A_log must be contiguous CUDA tensor")
    _require(A_log.dtype == torch.float32, "A_log must be float32")
    _require(dt_bias.is_cuda and dt_bias.is_contiguous(), "dt_bias must be contiguous CUDA tensor")
    _require(dt_bias.dtype == torch.float32, "dt_bias must be float32")
    for name, t in zip(("q", "k", "v", "g", "out"), (q, k, v, g, out)):
        _require(t.dim() == 4, f"{name} must be [B, T, H, D]")
    _require(beta.dim() == 3, "beta must be [B, T, H]")
    B, T, H, D = q.shape
    _require(k.shape == q.shape, "k must match q shape")
    _require(v.shape == q.shape, "v must match q shape")
    _require(g.shape == q.shape, "g must match q shape")
    _require(out.shape == q.shape, "out must match q shape")
    _require(tuple(beta.shape) == (B, T, H), "beta must be [B, T, H] matching q")
    _require(A_log.dim() == 1 and A_log.shape[0] == H, "A_log must be [H]")
    _require(dt_bias.dim() == 2 and tuple(dt_bias.shape) == (H, D), "dt_bias must be [H, D]")
    _require(D == 128, "currently only supports D == 128")
    if cu_seqlens is not None:
        _require(B == 1, "B must be 1 when cu_seqlens is provided")
        _require(cu_seqlens.is_cuda, "cu_seqlens must be on CUDA")
        _require(cu_seqlens.dtype == torch.int64, "cu_seqlens must be int64")
        _require(cu_seqlens.dim() == 1, "cu_seqlens must be 1D")
        _require(cu_seqlens.is_contiguous(), "cu_seqlens must be contiguous")
        N = cu_seqlens.numel() - 1
        _require(N > 0, "cu_seqlens must have at least 2 elements")
    else:
        N = B
    for name, st in (("initial_state", initial_state), ("final_state", final_state)):
        if st is not None:
            _require(st.dim() == 4 and tuple(st.shape) == (N, H, D, D), f"{name} must be [N, H, D, D]")
    dev = q.device
    for t in (k, v, g, beta, out, A_log, dt_bias, initial_state, final_state, cu_seqlens):
        _require(t is None or t.device == dev, "all tensors must be on the same CUDA device")
    return B, T, H, N, state_dtype


def _ptr(t):
    return None if t is None else t.data_ptr()


def _params(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state, final_state,
            cu_seqlens, workspace, flags):
    B, T, H, N, state_dtype = _validate(q, k, v, g, beta, out, A_log, dt_bias, initial_state, final_state,
                                        cu_seqlens, workspace)
    if workspace is None:
        workspace = torch.empty(get_workspace_size(B * T, H, N, flags), dtype=torch.uint8, device=q.device)
    p = FwdParams(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(out), _ptr(A_log), _ptr(dt_bias),
                  _ptr(initial_state), _ptr(final_state), _ptr(cu_seqlens), _ptr(workspace),
                  workspace.numel(), B, T, H, N, float(scale), float(lower_bound), state_dtype, int(flags))
    return p, workspace


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def fwd(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
        cu_seqlens=None, *, workspace=None, flags=0):
    """FlashKDA forward (Kimi Delta Attention prefill); same contract as the reference's
    `flash_kda.fwd` (flash_kda/__init__.py:5-41).

    q, k, g: bf16 [B, T, H, 128]; v, out: bf16 [B, T, H, 128]; beta: bf16 [B, T, H] logits;
    A_log: fp32 [H]; dt_bias: fp32 [H, 128]; initial_state / final_state: bf16 or fp32
    [N, H, 128, 128] (same dtype when both are given) or None; cu_seqlens: int64 [N+1] on the
    device, requires B == 1.  `out` and `final_state` are written in place; returns None.

    `workspace` (keyword-only, optional) lets a caller that must not allocate pass a uint8 CUDA
    tensor of at least `get_workspace_size(B*T, H, N)` bytes; by default one is allocated per
    call from torch's caching allocator, as the reference does (flash_kda/__init__.py:38).
    """
    p, ws = _params(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state, final_state,
                    cu_seqlens, workspace, flags)
    with torch.cuda.device(q.device):
        _check(lib().fkda_fwd(ctypes.byref(p), _stream(q)))
    return None


def prepare(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
            cu_seqlens=None, *, workspace=None, flags=0):
    """Stage 1 only (prologue + intra-chunk): fills and returns the workspace."""
    p, ws = _params(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state, final_state,
                    cu_seqlens, workspace, flags)
    with torch.cuda.device(q.device):
        _check(lib().fkda_prepare(ctypes.byref(p), _stream(q)))
    return ws


def scan(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
         cu_seqlens=None, *, workspace, flags=0):
    """Stage 2 only (inter-chunk recurrence) from a workspace filled by `prepare`."""
    p, ws = _params(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state, final_state,
                    cu_seqlens, workspace, flags)
    with torch.cuda.device(q.device):
        _check(lib().fkda_scan(ctypes.byref(p), _stream(q)))
    return None


def prologue(q, k, g, beta, A_log, dt_bias, lower_bound):
    """Token-wise prologue alone.  Returns (q_normalised bf16, k_normalised bf16,
    gate fp32 in log2 units, sigmoid(beta) fp32)."""
    B, T, H, D = q.shape
    _require(D == 128 and q.is_cuda and q.is_contiguous(), "q must be contiguous CUDA [B, T, H, 128]")
    qn, kn = torch.empty_like(q), torch.empty_like(k)
    gate = torch.empty(B, T, H, D, dtype=torch.float32, device=q.device)
    bact = torch.empty(B, T, H, dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        _check(lib().fkda_prologue(_ptr(q), _ptr(k), _ptr(g), _ptr(beta), _ptr(A_log), _ptr(dt_bias),
                                   float(lower_bound), B * T, H, _ptr(qn), _ptr(kn), _ptr(gate), _ptr(bact),
                                   _stream(q)))
    return qn, kn, gate, bact


def read_status(workspace) -> int:
    """Synchronises the current stream and returns the device status word of `workspace`
    (0 = fine).  Raises RuntimeError for a non-zero status."""
    st = ctypes.c_int(0)
    with torch.cuda.device(workspace.device):
        _check(lib().fkda_read_status(_ptr(workspace), _stream(workspace), ctypes.byref(st)))
    return st.value


def selftest_umma(A, B, mode, reps=1):
    """Runs one tcgen05 product flavour of the scan kernel on one CTA; returns D (fp32)."""
    n = 128 if mode in (1, 4) else 32
    D = torch.zeros(128, n, dtype=torch.float32, device=A.device)
    status = torch.zeros(1, dtype=torch.int32, device=A.device)
    with torch.cuda.device(A.device):
        _check(lib().fkda_selftest_umma(_ptr(A), _ptr(B), _ptr(D), mode, reps, _ptr(status), _stream(A)))
    torch.cuda.synchronize(A.device)
    if int(status.item()) != 0:
        raise RuntimeError("tcgen05 self-test: a bounded wait gave up")
    return D


def tmem_layout_probe(device="cuda"):
    """Register <-> (lane, column) maps of the 16-lane tensor-memory fragment shapes (int32 [4, 2048];
    see tmem_layout_probe_kernel in csrc/fkda_aux.cu)."""
    out = torch.zeros(4, 2048, dtype=torch.int32, device=device)
    with torch.cuda.device(out.device):
        _check(lib().fkda_debug_tmem_layout_probe(_ptr(out), _stream(out)))
    torch.cuda.synchronize(out.device)
    return out.cpu()


def scan_giveup(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state=None, final_state=None,
                cu_seqlens=None, *, workspace, stop_copies_after=1, wait_limit_us=3000):
    """Test aid: prepare, then the look-ahead recurrence with a copy producer that stops after `stop_copies_after`
    records and waits that give up after `wait_limit_us` microseconds (include/fkda_testing.h)."""
    p, ws = _params(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, initial_state, final_state,
                    cu_seqlens, workspace, 0)
    with torch.cuda.device(q.device):
        _check(lib().fkda_debug_scan_giveup(ctypes.byref(p), int(stop_copies_after), int(wait_limit_us), _stream(q)))


def prepare_giveup(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, cu_seqlens=None, *, workspace, wait_limit_us=3000):
    """Test aid: the token-parallel stage on the pipelined kernel with CTAs that load the tiles of their first item
    only and waits that give up after `wait_limit_us` microseconds (include/fkda_testing.h)."""
    p, ws = _params(q, k, v, g, beta, scale, out, A_log, dt_bias, lower_bound, None, None, cu_seqlens, workspace, 0)
    with torch.cuda.device(q.device):
        _check(lib().fkda_debug_prepare_giveup(ctypes.byref(p), int(wait_limit_us), _stream(q)))


def umma_bench(issuers=1, reps=64, ksteps=8, n=64, a_in_tmem=True, device="cuda"):
    """(Builds made with -DFKDA_TUNING only.)  Cycles per tcgen05.mma (M = 128, K = 16, N = n) when `issuers` threads of one CTA each issue `reps` chains of
    `ksteps` accumulating instructions: returns (issue, complete) cycles per instruction for the slowest issuer."""
    out = torch.zeros(8, dtype=torch.int64, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    with torch.cuda.device(out.device):
        _check(lib().fkda_debug_umma_bench(issuers, reps, ksteps, n, int(bool(a_in_tmem)), _ptr(out), _ptr(status), _stream(out)))
    torch.cuda.synchronize(out.device)
    if int(status.item()) != 0:
        raise RuntimeError("tcgen05 benchmark: a bounded wait gave up")
    o = out.cpu().view(4, 2)[:issuers].double() / (reps * ksteps)
    return o[:, 0].max().item(), o[:, 1].max().item()
