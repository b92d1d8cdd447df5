"""GPU: the allocation-free entry point `fkda_fwd_static_ws` (built-in 64 MiB scratch), for
hosts that may not call cudaMalloc when they need the operator -- e.g. a serving process whose
device memory pool is fixed after start-up.  It is called through the C ABI exactly as such a
host would, and must reproduce `fkda_fwd` (caller workspace) on two calls in a row; the second
call has a different shape, so anything stale left in the shared scratch by the first would
show.  Collected last on purpose: a failure here cannot hide results of the other GPU tests.
"""
import ctypes

import pytest
import torch

import flashkda_b200 as F
from flashkda_b200._binding import FwdParams
from flashkda_b200.workloads import Workload, make_inputs
from helpers import OUT_MAX_ABS, STATE_REL, max_abs, rel_fro, to_cuda

pytestmark = pytest.mark.gpu


def _params(xc, x, out, fin, ws):
    B, T, H = x["q"].shape[:3]
    N = x["cu_seqlens"].numel() - 1 if x["cu_seqlens"] is not None else B
    p = lambda t: None if t is None else t.data_ptr()
    sd = 0
    for st in (xc["initial_state"], fin):
        if st is not None:
            sd = 2 if st.dtype == torch.float32 else 1
    return FwdParams(p(xc["q"]), p(xc["k"]), p(xc["v"]), p(xc["g"]), p(xc["beta"]), p(out), p(xc["A_log"]),
                     p(xc["dt_bias"]), p(xc["initial_state"]), p(fin), p(xc["cu_seqlens"]), p(ws),
                     0 if ws is None else ws.numel(), B, T, H, N, float(x["scale"]), float(x["lower_bound"]), sd, 0)


def _run_both(w):
    L = F.lib()
    L.fkda_fwd_static_ws.argtypes = [ctypes.POINTER(FwdParams), ctypes.c_void_p]
    L.fkda_fwd_static_ws.restype = ctypes.c_int
    L.fkda_static_ws_read_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
    L.fkda_static_ws_last_error.restype = ctypes.c_char_p
    x = make_inputs(w)
    xc = to_cuda(x)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, T, H = x["q"].shape[:3]
    fin_dt = None if x["final_state"] is None else x["final_state"].dtype
    mk_fin = lambda: None if fin_dt is None else torch.full((w.N, H, 128, 128), float("nan"), dtype=fin_dt, device="cuda")
    # existing entry point, caller-provided workspace
    out_a, fin_a = torch.full_like(xc["v"], float("nan")), mk_fin()
    ws = torch.empty(F.get_workspace_size(B * T, H, w.N), dtype=torch.uint8, device="cuda")
    pa = _params(xc, x, out_a, fin_a, ws)
    assert L.fkda_fwd(ctypes.byref(pa), stream) == 0, F.last_error()
    # new entry point: no workspace at all
    out_b, fin_b = torch.full_like(xc["v"], float("nan")), mk_fin()
    pb = _params(xc, x, out_b, fin_b, None)
    rc = L.fkda_fwd_static_ws(ctypes.byref(pb), stream)
    assert rc == 0, L.fkda_static_ws_last_error()
    st = ctypes.c_int(-1)
    assert L.fkda_static_ws_read_status(stream, ctypes.byref(st)) == 0 and st.value == 0
    torch.cuda.synchronize()
    assert not torch.isnan(out_b.float()).any()
    assert max_abs(out_b, out_a) <= OUT_MAX_ABS
    if fin_a is not None:
        assert rel_fro(fin_b, fin_a) <= STATE_REL
    return L


def test_static_scratch_entry_point_matches_fkda_fwd_twice_in_a_row():
    _run_both(Workload("first", H=4, B=2, T=200, state_in="fp32", state_out="fp32", seed=31))
    L = _run_both(Workload("second", H=3, seq_lens=[90, 7, 33], state_in="bf16", state_out="bf16", seed=32))
    # a problem beyond the built-in scratch is refused with a clear message, nothing is launched
    cap = L.fkda_static_ws_capacity
    cap.restype = ctypes.c_int64
    assert cap() == 64 << 20
    w = Workload("big", H=32, B=1, T=4096, seed=33)
    x = make_inputs(w)
    xc = to_cuda(x)
    out = torch.zeros_like(xc["v"])
    p = _params(xc, x, out, None, None)
    assert L.fkda_fwd_static_ws(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == -2
    assert b"built-in scratch" in L.fkda_static_ws_last_error()
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0


def test_static_scratch_walks_whole_sequences_when_the_runs_do_not_fit():
    """One long chain: the planner would cut it into runs, whose scratch does not fit the built-in array beside the
    records; the call is then served by the walk over whole sequences instead of being refused."""
    w = Workload("long", H=1, B=1, T=57600, state_in="fp32", state_out="fp32", seed=34)
    runs, _ = F.plan_segments(1, w.T // 32)
    assert runs > 1 and F.get_workspace_size(w.T, 1, 1) > (64 << 20) >= F.get_workspace_size(w.T, 1, 1, F.FLAG_SCAN_NO_SEGMENTS)
    _run_both(w)
