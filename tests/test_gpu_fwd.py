"""GPU parity of `flash_kda.fwd` (through the C ABI) against the CPU oracle.

Tolerances are the contract's: bf16 `out` max-abs error <= 2e-2 and final-state relative
(Frobenius) error <= 1e-2, both against the fp64 per-token recurrence.  The distance to the
reference's own chunk-16/bf16 algorithm (golden vectors, or its C port) is printed alongside.
The shape / state-variant matrix follows the reference's tests/test_fwd_full.py:48-205.
"""
import pytest
import torch

import flash_kda
import flashkda_b200 as F
import oracle
from flashkda_b200.workloads import Workload, baseline_workload, make_inputs
from helpers import OUT_MAX_ABS, STATE_REL, golden_names, load_golden, max_abs, rel_fro, to_cuda

pytestmark = pytest.mark.gpu


def run_gpu(x, fin_dtype, flags=0, check_status=True):
    xc = to_cuda(x)
    out = torch.full_like(xc["v"], float("nan"))
    fin = None
    if fin_dtype is not None:
        N = x["cu_seqlens"].numel() - 1 if x["cu_seqlens"] is not None else x["q"].shape[0]
        fin = torch.full((N, x["q"].shape[2], 128, 128), float("nan"), dtype=fin_dtype, device="cuda")
    init = xc["initial_state"]
    init_copy = None if init is None else init.clone()
    B, T, H = x["q"].shape[:3]
    N = x["cu_seqlens"].numel() - 1 if x["cu_seqlens"] is not None else B
    ws = torch.empty(F.get_workspace_size(B * T, H, N, flags), dtype=torch.uint8, device="cuda")
    flash_kda.fwd(xc["q"], xc["k"], xc["v"], xc["g"], xc["beta"], x["scale"], out, xc["A_log"], xc["dt_bias"],
                  x["lower_bound"], initial_state=init, final_state=fin, cu_seqlens=xc["cu_seqlens"],
                  workspace=ws, flags=flags)
    if check_status:
        assert F.read_status(ws) == 0
    torch.cuda.synchronize()
    if init is not None:
        assert torch.equal(init, init_copy), "initial_state was modified"
    return out.cpu(), None if fin is None else fin.cpu()


def check_against_f64(x, out, fin, tag, big_state=False):
    o64, s64 = oracle.recurrence_f64(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["A_log"],
                                     x["dt_bias"], x["lower_bound"], initial_state=x["initial_state"],
                                     cu_seqlens=x["cu_seqlens"])
    assert not torch.isnan(out.float()).any(), f"{tag}: some out rows were not written"
    e_out = max_abs(out, o64)
    e_st = rel_fro(fin, s64) if fin is not None else 0.0
    print(f"{tag}: out max-abs {e_out:.3e} (|out| max {o64.abs().max():.2f}), state rel {e_st:.3e}")
    if big_state:
        assert rel_fro(out, o64) <= 1e-2
    else:
        assert e_out <= OUT_MAX_ABS, f"{tag}: out max-abs error {e_out}"
    if fin is not None:
        assert not torch.isnan(fin.float()).any()
        assert e_st <= STATE_REL, f"{tag}: final-state relative error {e_st}"
    return o64, s64


@pytest.mark.parametrize("flags", [F.FLAG_SCAN_SIMT, F.FLAG_SCAN_PLAIN, 0], ids=["simt_checker", "tcgen05_plain", "tcgen05_lookahead"])
@pytest.mark.parametrize("name", golden_names())
def test_golden_cases(name, flags):
    x, ref_out, ref_fin = load_golden(name)
    fin_dtype = None if ref_fin is None else ref_fin.dtype
    out, fin = run_gpu(x, fin_dtype, flags)
    big = x["initial_state"] is not None and x["initial_state"].float().abs().max() > 100
    check_against_f64(x, out, fin, f"{name}[{flags}]", big_state=big)
    # distance to the reference's own (chunk-16, bf16-state) results
    d_out = rel_fro(out, ref_out) if big else max_abs(out, ref_out)
    d_st = rel_fro(fin, ref_fin) if fin is not None else 0.0
    print(f"{name}[{flags}]: vs reference vectors: out {d_out:.3e}, state rel {d_st:.3e}")
    assert d_out <= (1e-2 if big else OUT_MAX_ABS) and d_st <= STATE_REL


OTHER_PREPARE_KERNELS = {"mma_sync": F.FLAG_PREPARE_MMA_SYNC, "tcgen05_cta_per_item": F.FLAG_PREPARE_TCGEN05}


@pytest.mark.parametrize("kernel", list(OTHER_PREPARE_KERNELS))
@pytest.mark.parametrize("name", golden_names())
def test_golden_cases_on_the_other_token_parallel_kernels(name, kernel):
    """The token-parallel stage on the mma.sync kernel and on the one-CTA-per-item form of the TMA + tcgen05 kernel
    (the default is the pipelined TMA + tcgen05 kernel): same golden cases."""
    x, ref_out, ref_fin = load_golden(name)
    fin_dtype = None if ref_fin is None else ref_fin.dtype
    out, fin = run_gpu(x, fin_dtype, OTHER_PREPARE_KERNELS[kernel] | F.FLAG_NO_FUSED_SHORT)
    big = x["initial_state"] is not None and x["initial_state"].float().abs().max() > 100
    check_against_f64(x, out, fin, f"{name}[{kernel} prepare]", big_state=big)


def test_the_two_tcgen05_kernels_write_the_same_bits():
    """The pipelined kernel and the one-CTA-per-item kernel do the same arithmetic in the same order."""
    x = make_inputs(Workload("req", H=4, B=2, T=300, state_in="fp32", state_out="fp32", seed=65))
    o0, s0 = run_gpu(x, torch.float32)
    o1, s1 = run_gpu(x, torch.float32, F.FLAG_PREPARE_TCGEN05)
    assert torch.equal(o0.view(torch.int16), o1.view(torch.int16)) and torch.equal(s0, s1)


@pytest.mark.parametrize("kernel", ["tcgen05_pipelined", "tcgen05_cta_per_item"])
@pytest.mark.parametrize("case", ["fixed_tails", "varlen_ragged", "many_items", "long_repeat"])
def test_tma_tcgen05_token_parallel_kernel_shapes(case, kernel):
    """Shapes that stress the TMA + tcgen05 kernels: ragged last chunks, many short sequences (items of every
    length), more items than one pass of the CTAs holds, and repeated calls that must be bit-reproducible; each
    against the fp64 oracle and against the mma.sync kernel."""
    tc_flag = {"tcgen05_pipelined": 0, "tcgen05_cta_per_item": F.FLAG_PREPARE_TCGEN05}[kernel]
    if case == "fixed_tails":
        w = Workload("tc1", H=3, B=5, T=32 * 3 + 17, state_in="fp32", state_out="fp32", state_std=0.5, seed=61)
    elif case == "varlen_ragged":
        w = Workload("tc2", H=4, seq_lens=[1, 31, 32, 33, 0, 100, 7, 64, 250], state_in="bf16", state_out="bf16", state_std=0.5, seed=62)
    elif case == "many_items":
        w = Workload("tc3", H=8, B=6, T=2048 + 5, state_in="fp32", state_out="fp32", seed=63)
    else:
        w = Workload("tc4", H=16, B=2, T=1024, state_in="fp32", state_out="fp32", seed=64)
    x = make_inputs(w)
    dt = torch.bfloat16 if w.state_in == "bf16" else torch.float32
    out, fin = run_gpu(x, dt, tc_flag)
    check_against_f64(x, out, fin, f"{kernel} prepare, {case}")
    o0, s0 = run_gpu(x, dt, F.FLAG_PREPARE_MMA_SYNC)
    assert max_abs(out, o0) <= 1e-2 and rel_fro(fin, s0) <= (2e-2 if dt == torch.bfloat16 else 5e-3)
    if case == "long_repeat":
        for _ in range(4):
            o2, s2 = run_gpu(x, dt, tc_flag)
            assert torch.equal(o2.view(torch.int16), out.view(torch.int16)) and torch.equal(s2, fin)


STATE_IO = [(True, True), (True, False), (False, True), (False, False)]


@pytest.mark.parametrize("T", [16, 64, 256, 1024, 17, 37, 97, 1, 31, 32, 33])
@pytest.mark.parametrize("state", ["bf16", "fp32"])
@pytest.mark.parametrize("has_in,has_out", STATE_IO, ids=["in+out", "in_only", "out_only", "no_state"])
def test_fixed_length_matrix(T, state, has_in, has_out):
    H = 4 if T <= 256 else 2
    w = Workload("m", H=H, B=1, T=T, state_in=state if has_in else None, state_out=state if has_out else None,
                 state_std=0.5, seed=T)
    x = make_inputs(w)
    fin_dtype = None if not has_out else (torch.bfloat16 if state == "bf16" else torch.float32)
    out, fin = run_gpu(x, fin_dtype)
    check_against_f64(x, out, fin, f"T{T}-{state}-{has_in}-{has_out}")


VARLEN = [[16], [16, 16], [4, 8, 12], [64, 128, 256], [1300, 547, 2048, 963, 271, 3063], [1024] * 8,
          [20, 50, 100], [17, 33, 65], [1, 1, 1, 40]]


@pytest.mark.parametrize("seq_lens", VARLEN, ids=lambda s: "seqs" + "_".join(map(str, s)))
@pytest.mark.parametrize("state", ["bf16", "fp32"])
def test_varlen_matrix(seq_lens, state):
    H = 2 if sum(seq_lens) > 2000 else 4
    w = Workload("v", H=H, seq_lens=seq_lens, state_in=state, state_out=state, state_std=0.5, seed=len(seq_lens))
    x = make_inputs(w)
    out, fin = run_gpu(x, torch.bfloat16 if state == "bf16" else torch.float32)
    check_against_f64(x, out, fin, f"varlen{seq_lens}-{state}")


@pytest.mark.parametrize("kernel", ["default", "short", "lookahead", "plain"])
@pytest.mark.parametrize("B,T,state", [(300, 16, "fp32"), (37, 33, "bf16"), (5, 64, "fp32"), (200, 1, None), (3, 32, "bf16"),
                                       (70, 9, "bf16"), (33, 16, None)])
def test_short_chains_all_scan_kernels(B, T, state, kernel):
    """By default sequences of at most 16 tokens go to the fused short-sequence kernel and those of at most two
    chunks to the persistent short-chain kernel; the other recurrence kernels must give the same answers on the
    same shapes ("short": the two-kernel path with the persistent short-chain kernel also for T <= 16)."""
    flags = {"default": 0, "short": F.FLAG_NO_FUSED_SHORT, "lookahead": F.FLAG_SCAN_LOOKAHEAD, "plain": F.FLAG_SCAN_PLAIN}[kernel]
    w = Workload("s", H=3, B=B, T=T, state_in=state, state_out=state or "fp32", state_std=0.5, seed=B + T)
    x = make_inputs(w)
    fin_dtype = torch.bfloat16 if state == "bf16" else torch.float32
    out, fin = run_gpu(x, fin_dtype, flags)
    check_against_f64(x, out, fin, f"short-B{B}xT{T}-{state}-{kernel}")


@pytest.mark.parametrize("T,state", [(65, "fp32"), (96, "bf16"), (129, "fp32"), (160, None)])
def test_many_chains_of_up_to_five_chunks(T, state):
    """More chains than SMs and at most five chunks each: the persistent short-chain kernel takes these too; same
    answers as the look-ahead kernel and the fp64 recurrence."""
    w = Workload("s5", H=4, B=40, T=T, state_in=state, state_out=state or "fp32", state_std=0.5, seed=T, lower_bound=-1.0)
    x = make_inputs(w)
    dt = torch.bfloat16 if state == "bf16" else torch.float32
    o1, s1 = run_gpu(x, dt)
    check_against_f64(x, o1, s1, f"160 chains of T={T}, {state} state")
    o0, s0 = run_gpu(x, dt, F.FLAG_SCAN_LOOKAHEAD)
    assert max_abs(o1, o0) <= 1e-2 and rel_fro(s1, s0) <= (2e-2 if state == "bf16" else 5e-3)


@pytest.mark.parametrize("B,T", [(2, 64), (2, 1024), (4, 256), (8, 128), (64, 16)])
def test_batched(B, T):
    w = Workload("b", H=4, B=B, T=T, state_in="fp32", state_out="fp32", seed=B)
    x = make_inputs(w)
    out, fin = run_gpu(x, torch.float32)
    check_against_f64(x, out, fin, f"B{B}xT{T}")


@pytest.mark.parametrize("regime", ["g=-8", "g=8", "g=U(-8,8)", "bias=+-8", "lb=-2", "H32"])
def test_gate_regimes(regime):
    """Gate sweeps in the spirit of the reference's accuracy tests (tests/test_fwd.py:45-68)."""
    H = 32 if regime == "H32" else 2
    w = Workload("g", H=H, B=1, T=512, state_in="fp32", state_out="fp32", state_std=1.0, seed=7,
                 lower_bound=-2.0 if regime == "lb=-2" else -5.0)
    x = make_inputs(w)
    gen = torch.Generator().manual_seed(3)
    if regime == "g=-8":
        x["g"] = torch.full_like(x["g"], -8.0)
    elif regime == "g=8":
        x["g"] = torch.full_like(x["g"], 8.0)
    elif regime == "g=U(-8,8)":
        x["g"] = (torch.rand(x["g"].shape, generator=gen) * 16 - 8).bfloat16()
    elif regime == "bias=+-8":
        x["g"] = torch.zeros_like(x["g"])
        x["dt_bias"] = torch.where(torch.rand(x["dt_bias"].shape, generator=gen) < 0.5, -8.0, 8.0)
    if regime in ("g=-8", "g=8", "g=U(-8,8)", "bias=+-8"):
        x["A_log"] = torch.zeros_like(x["A_log"])
    out, fin = run_gpu(x, torch.float32)
    check_against_f64(x, out, fin, regime)


def test_state_handoff_split_equals_unsplit():
    """Prefill 160 tokens at once, or 96 then 64 with final_state fed back as initial_state."""
    w = Workload("s", H=2, B=1, T=160, state_in="fp32", state_out="fp32", seed=21)
    x = make_inputs(w)
    o_all, s_all = run_gpu(x, torch.float32)
    cut = lambda a, b: {k: (v[:, a:b].contiguous() if k in ("q", "k", "v", "g", "beta") else v) for k, v in x.items()}
    xa = cut(0, 96)
    o1, s1 = run_gpu(xa, torch.float32)
    xb = cut(96, 160)
    xb["initial_state"] = s1
    o2, s2 = run_gpu(xb, torch.float32)
    assert max_abs(torch.cat([o1, o2], 1), o_all) <= 2e-2
    assert rel_fro(s2, s_all) <= 2e-3


@pytest.mark.parametrize("flags", [F.FLAG_SCAN_NO_SEGMENTS, 0], ids=["whole_sequences", "planned_runs"])
def test_long_chains_repeated_calls_stay_in_step(flags):
    """Long chains exercise every barrier of the look-ahead kernel thousands of times; repeated calls must never
    trip a bounded wait (status 0) and must be bit-reproducible (no race on tensor- or shared memory).  With 32
    chains the planner would cut the sequences into runs: both forms are walked."""
    w = Workload("long", H=16, B=2, T=4096, state_in="fp32", state_out="fp32", seed=99)
    x = make_inputs(w)
    ref = None
    for _ in range(6):
        out, fin = run_gpu(x, torch.float32, flags)   # asserts status == 0
        if ref is None:
            ref = (out, fin)
        else:
            assert torch.equal(out.view(torch.int16), ref[0].view(torch.int16)) and torch.equal(fin, ref[1])
    sub = {k: (v[:, :, :2].contiguous() if k in ("q", "k", "v", "g", "beta") else v) for k, v in x.items()}
    sub["A_log"], sub["dt_bias"], sub["initial_state"] = x["A_log"][:2], x["dt_bias"][:2], x["initial_state"][:, :2].contiguous()
    o64, s64 = oracle.recurrence_f64(sub["q"], sub["k"], sub["v"], sub["g"], sub["beta"], x["scale"], sub["A_log"],
                                     sub["dt_bias"], x["lower_bound"], initial_state=sub["initial_state"])
    assert max_abs(ref[0][:, :, :2], o64) <= OUT_MAX_ABS and rel_fro(ref[1][:, :2], s64) <= STATE_REL


def test_bounded_wait_gives_up_and_the_context_stays_usable():
    """A wait that nothing will complete: the copy producer of a two-chunk chain stops after the first record and the
    waits are given three milliseconds.  The call must return (no hang), the status word must say 2, and the CTA must
    have released its tensor memory - seen by a normal call right afterwards, which needs all of it.  Nothing faults
    and no copy is in flight when the wait runs out."""
    w = Workload("giveup", H=1, B=1, T=64, state_in="fp32", state_out="fp32", seed=3)
    x = make_inputs(w)
    xc = to_cuda(x)
    ws = torch.empty(F.get_workspace_size(64, 1, 1), dtype=torch.uint8, device="cuda")
    fin = torch.zeros(1, 1, 128, 128, device="cuda")
    F.scan_giveup(xc["q"], xc["k"], xc["v"], xc["g"], xc["beta"], x["scale"], xc["out"], xc["A_log"], xc["dt_bias"],
                  x["lower_bound"], initial_state=xc["initial_state"], final_state=fin, workspace=ws,
                  stop_copies_after=1, wait_limit_us=3000)
    with pytest.raises(RuntimeError, match="bounded wait"):
        F.read_status(ws)
    torch.cuda.synchronize()
    # a single-chunk chain never meets the missing record: same entry point, status 0
    w1 = Workload("giveup1", H=1, B=1, T=32, state_in="fp32", state_out="fp32", seed=3)
    x1 = make_inputs(w1)
    x1c = to_cuda(x1)
    fin1 = torch.zeros(1, 1, 128, 128, device="cuda")
    F.scan_giveup(x1c["q"], x1c["k"], x1c["v"], x1c["g"], x1c["beta"], x1["scale"], x1c["out"], x1c["A_log"], x1c["dt_bias"],
                  x1["lower_bound"], initial_state=x1c["initial_state"], final_state=fin1, workspace=ws,
                  stop_copies_after=1, wait_limit_us=3000)
    assert F.read_status(ws) == 0
    # and the normal path works right after the give-up (tensor memory was released, the context is intact)
    out, fin2 = run_gpu(x, torch.float32, F.FLAG_SCAN_LOOKAHEAD)
    check_against_f64(x, out, fin2, "after a give-up")


def test_bounded_wait_of_the_token_parallel_kernel_gives_up_and_the_context_stays_usable():
    """The same for the pipelined token-parallel kernel: every CTA loads the tiles of its first item only and the waits
    are given three milliseconds.  With 600 (chunk, head) items some CTAs have a second item whose tiles never come:
    the call must return, status 2, tensor memory released (a normal call right afterwards passes); with fewer items
    than CTAs nobody meets the missing load and the status stays 0.  Nothing faults, and what a CTA still has in
    flight when it gives up (its first item's products) has landed before it leaves."""
    w = Workload("pgiveup", H=1, B=1, T=32 * 600, state_in="fp32", state_out="fp32", seed=6)
    x = make_inputs(w)
    xc = to_cuda(x)
    ws = torch.empty(F.get_workspace_size(32 * 600, 1, 1), dtype=torch.uint8, device="cuda")
    F.prepare_giveup(xc["q"], xc["k"], xc["v"], xc["g"], xc["beta"], x["scale"], xc["out"], xc["A_log"], xc["dt_bias"],
                     x["lower_bound"], workspace=ws, wait_limit_us=3000)
    with pytest.raises(RuntimeError, match="bounded wait"):
        F.read_status(ws)
    torch.cuda.synchronize()
    w1 = Workload("pgiveup1", H=1, B=1, T=32 * 100, state_in="fp32", state_out="fp32", seed=6)
    x1 = make_inputs(w1)
    x1c = to_cuda(x1)
    F.prepare_giveup(x1c["q"], x1c["k"], x1c["v"], x1c["g"], x1c["beta"], x1["scale"], x1c["out"], x1c["A_log"], x1c["dt_bias"],
                     x1["lower_bound"], workspace=ws, wait_limit_us=3000)
    assert F.read_status(ws) == 0
    out, fin = run_gpu(x, torch.float32)
    check_against_f64(x, out, fin, "after a give-up of the token-parallel kernel")


def test_deterministic_and_tail_rows_untouched():
    w = Workload("d", H=2, seq_lens=[45, 3], state_in="bf16", state_out="bf16", seed=4)
    x = make_inputs(w)
    o1, s1 = run_gpu(x, torch.bfloat16)
    o2, s2 = run_gpu(x, torch.bfloat16)
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16)) and torch.equal(s1.view(torch.int16), s2.view(torch.int16))


def test_bad_cu_seqlens_reports_status_instead_of_faulting():
    w = Workload("c", H=2, seq_lens=[40, 24], seed=9)
    x = make_inputs(w)
    x["cu_seqlens"] = torch.tensor([0, 50, 40], dtype=torch.int64)     # not monotone
    xc = to_cuda(x)
    ws = torch.empty(F.get_workspace_size(64, 2, 2), dtype=torch.uint8, device="cuda")
    flash_kda.fwd(xc["q"], xc["k"], xc["v"], xc["g"], xc["beta"], x["scale"], xc["out"], xc["A_log"],
                  xc["dt_bias"], x["lower_bound"], cu_seqlens=xc["cu_seqlens"], workspace=ws)
    with pytest.raises(RuntimeError, match="cu_seqlens"):
        F.read_status(ws)


def test_argument_errors_raise_before_launch():
    w = Workload("e", H=2, B=1, T=32, seed=1)
    xc = to_cuda(make_inputs(w))
    call = lambda **kw: flash_kda.fwd(*[kw.get(n, xc[n]) for n in ("q", "k", "v", "g", "beta", "scale", "out", "A_log",
                                                                    "dt_bias", "lower_bound")],
                                      **{n: kw[n] for n in ("initial_state", "final_state", "cu_seqlens") if n in kw})
    with pytest.raises(RuntimeError, match="q must be bfloat16"):
        call(q=xc["q"].float())
    with pytest.raises(RuntimeError, match="contiguous"):
        call(k=xc["k"].transpose(1, 2))
    with pytest.raises(RuntimeError, match="A_log must be"):
        call(A_log=xc["A_log"][:1])
    with pytest.raises(RuntimeError, match="same dtype"):
        call(initial_state=torch.zeros(1, 2, 128, 128, device="cuda"),
             final_state=torch.zeros(1, 2, 128, 128, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match=r"\[N, H, D, D\]"):
        call(final_state=torch.zeros(2, 2, 128, 128, device="cuda"))
    with pytest.raises(RuntimeError, match="int64"):
        call(cu_seqlens=torch.tensor([0, 32], dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError, match="workspace must be a contiguous CUDA tensor"):      # a host tensor
        flash_kda.fwd(*[xc[n] for n in ("q", "k", "v", "g", "beta", "scale", "out", "A_log", "dt_bias", "lower_bound")],
                      workspace=torch.empty(F.get_workspace_size(32, 2, 1), dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="workspace must be a contiguous CUDA tensor"):      # a strided view
        flash_kda.fwd(*[xc[n] for n in ("q", "k", "v", "g", "beta", "scale", "out", "A_log", "dt_bias", "lower_bound")],
                      workspace=torch.empty(2 * F.get_workspace_size(32, 2, 1), dtype=torch.uint8, device="cuda")[::2])
    with pytest.raises(RuntimeError, match="workspace must be uint8"):
        flash_kda.fwd(*[xc[n] for n in ("q", "k", "v", "g", "beta", "scale", "out", "A_log", "dt_bias", "lower_bound")],
                      workspace=torch.empty(F.get_workspace_size(32, 2, 1), dtype=torch.float32, device="cuda"))
    with pytest.raises(RuntimeError, match="D == 128"):
        z = torch.zeros(1, 32, 2, 64, dtype=torch.bfloat16, device="cuda")
        flash_kda.fwd(z, z, z, z, xc["beta"], 0.1, z.clone(), xc["A_log"], torch.zeros(2, 64, device="cuda"), -5.0)


def test_baseline_config0_through_default_allocation():
    """Headline configuration 0 (B=1, T=1024, H=4, fp32 final state) with the per-call workspace
    allocation of the plain `flash_kda.fwd` signature."""
    x = make_inputs(baseline_workload(0))
    xc = to_cuda(x)
    out = torch.empty_like(xc["v"])
    fin = torch.empty(1, 4, 128, 128, device="cuda")
    flash_kda.fwd(xc["q"], xc["k"], xc["v"], xc["g"], xc["beta"], x["scale"], out, A_log=xc["A_log"],
                  dt_bias=xc["dt_bias"], lower_bound=x["lower_bound"], final_state=fin)
    torch.cuda.synchronize()
    check_against_f64(x, out.cpu(), fin.cpu(), "C0")


@pytest.mark.parametrize("state", ["fp32", "bf16", "none"])
@pytest.mark.parametrize("runs", [2, 3, 5])
def test_segment_parallel_scan_forced_runs(runs, state):
    """Sequences cut into runs walked in parallel (affine maps of the inner runs chained in fp32) give the same
    result as the walk over whole sequences; ragged last chunk, last run shorter than the others."""
    w = Workload("seg", H=2, B=2, T=32 * 13 + 7, state_in=None if state == "none" else state,
                 state_out="fp32" if state == "none" else state, state_std=0.5, seed=31 + runs)
    x = make_inputs(w)
    fin_dtype = torch.bfloat16 if state == "bf16" else torch.float32
    o_seg, s_seg = run_gpu(x, fin_dtype, F.FLAG_SCAN_LOOKAHEAD | F.FLAG_SEGMENTS(runs))
    o_ref, s_ref = run_gpu(x, fin_dtype, F.FLAG_SCAN_LOOKAHEAD)
    check_against_f64(x, o_seg, s_seg, f"runs={runs} state={state}")
    assert max_abs(o_seg, o_ref) <= 1e-2
    assert rel_fro(s_seg, s_ref) <= 5e-3


@pytest.mark.parametrize("kernel", ["compact", "lookahead"])
def test_segment_parallel_scan_on_either_recurrence_kernel(kernel):
    """Both recurrence kernels can walk the runs; with a forced kernel both passes use it.  Twelve chains, so the
    chaining of the maps runs in its many-chain shape (32 state rows per CTA); an incoming state that matters."""
    flag = F.FLAG_SCAN_PLAIN if kernel == "compact" else F.FLAG_SCAN_LOOKAHEAD
    w = Workload("segk", H=6, B=2, T=32 * 21 + 11, state_in="fp32", state_out="fp32", state_std=0.5, seed=5, lower_bound=-1.0)
    x = make_inputs(w)
    o_seg, s_seg = run_gpu(x, torch.float32, flag | F.FLAG_SEGMENTS(4))
    o_ref, s_ref = run_gpu(x, torch.float32, F.FLAG_SCAN_LOOKAHEAD)
    check_against_f64(x, o_seg, s_seg, f"segments on the {kernel} kernel")
    assert max_abs(o_seg, o_ref) <= 1e-2 and rel_fro(s_seg, s_ref) <= 5e-3


def test_segment_parallel_scan_planned_many_chains():
    """Twenty-four chains of 256 chunks: the planner cuts them, the first pass has more CTAs than SMs and runs on the
    compact kernel, the second on the look-ahead kernel."""
    w = Workload("segmany", H=12, B=2, T=8192 - 13, state_in="bf16", state_out="bf16", state_std=0.5, seed=9)
    runs, run_chunks = F.plan_segments(w.H * w.B, (w.T + 31) // 32)
    assert runs >= 3 and w.H * w.B * (2 * runs - 3) > 148 >= w.H * w.B * (runs - 1), (runs, run_chunks)
    x = make_inputs(w)
    o1, s1 = run_gpu(x, torch.bfloat16)
    check_against_f64(x, o1, s1, f"planned runs={runs}x{run_chunks}, 24 chains")
    o0, s0 = run_gpu(x, torch.bfloat16, F.FLAG_SCAN_NO_SEGMENTS)
    assert max_abs(o1, o0) <= 1e-2 and rel_fro(s1, s0) <= 2e-2


@pytest.mark.parametrize("kernel", ["compact", "lookahead"])
@pytest.mark.parametrize("state", ["fp32", "bf16"])
def test_segment_parallel_scan_of_variable_length_sequences(kernel, state):
    """Varlen batches are cut into runs too: the run length is set on the device from the longest sequence, shorter
    sequences end in empty runs (which pass the state through), an empty sequence has only empty runs."""
    flag = F.FLAG_SCAN_PLAIN if kernel == "compact" else F.FLAG_SCAN_LOOKAHEAD
    w = Workload("segvar", H=2, seq_lens=[32 * 13 + 7, 0, 40, 32 * 30, 1], state_in=state, state_out=state, state_std=0.5,
                 seed=17, lower_bound=-1.0)
    x = make_inputs(w)
    dt = torch.bfloat16 if state == "bf16" else torch.float32
    o_seg, s_seg = run_gpu(x, dt, flag | F.FLAG_SEGMENTS(4))
    o_ref, s_ref = run_gpu(x, dt, F.FLAG_SCAN_LOOKAHEAD)
    check_against_f64(x, o_seg, s_seg, f"varlen segments on the {kernel} kernel, {state} state")
    assert max_abs(o_seg, o_ref) <= 1e-2 and rel_fro(s_seg, s_ref) <= (2e-2 if state == "bf16" else 5e-3)


def test_segment_parallel_scan_planned_for_variable_length_sequences():
    """Two long sequences of unequal length, three heads: the planner cuts them (number of runs from the average
    length, run length from the longest on the device)."""
    w = Workload("segvarplan", H=3, seq_lens=[2900, 5100], state_in="fp32", state_out="fp32", state_std=0.5, seed=18)
    runs, _ = F.plan_segments(6, (8000 // 2 + 31) // 32)
    assert runs >= 3
    x = make_inputs(w)
    assert F.get_workspace_size(8000, 3, 2) - F.get_workspace_size(8000, 3, 2, F.FLAG_SCAN_NO_SEGMENTS) == 6 * runs * 3 * 128 * 136 * 4
    o1, s1 = run_gpu(x, torch.float32)
    check_against_f64(x, o1, s1, f"varlen planned runs={runs}")
    o0, s0 = run_gpu(x, torch.float32, F.FLAG_SCAN_NO_SEGMENTS)
    assert max_abs(o1, o0) <= 1e-2 and rel_fro(s1, s0) <= 5e-3
    assert not torch.equal(o1.view(torch.int16), o0.view(torch.int16)), "the two paths round differently: equal outputs mean the runs were not used"


def test_segment_parallel_scan_planned():
    """A batch with few long chains takes the segment-parallel path by itself (the planner's choice), within the
    same tolerances; a second call on the same workspace reproduces the first bit for bit."""
    w = Workload("segplan", H=4, B=1, T=4096 + 19, state_in="fp32", state_out="fp32", state_std=0.5, seed=77)
    runs, run_chunks = F.plan_segments(w.H * w.B, (w.T + 31) // 32)
    assert runs >= 3 and (runs - 1) * run_chunks < (w.T + 31) // 32
    x = make_inputs(w)
    o1, s1 = run_gpu(x, torch.float32)
    check_against_f64(x, o1, s1, f"planned runs={runs}x{run_chunks}")
    o0, s0 = run_gpu(x, torch.float32, F.FLAG_SCAN_NO_SEGMENTS)
    assert max_abs(o1, o0) <= 1e-2 and rel_fro(s1, s0) <= 5e-3
    o2, s2 = run_gpu(x, torch.float32)
    assert torch.equal(o1.view(torch.int16), o2.view(torch.int16)) and torch.equal(s1, s2)


@pytest.mark.parametrize("T", [1, 5, 8, 16, 17, 24, 32])
@pytest.mark.parametrize("state", ["fp32", "bf16"])
def test_fused_short_sequences_match_two_kernel_path(T, state):
    """The fused kernel (T <= 32: one or two blocks of 16 tokens) against the two-kernel path on the same inputs
    (gate regime with little decay, so that the incoming state matters), and its state hand-off: two 8-token steps
    equal one 16-token step."""
    w = Workload("f16", H=4, B=19, T=T, state_in=state, state_out=state, state_std=0.5, seed=T, lower_bound=-1.0)
    x = make_inputs(w)
    dt = torch.bfloat16 if state == "bf16" else torch.float32
    o1, s1 = run_gpu(x, dt)
    o0, s0 = run_gpu(x, dt, F.FLAG_NO_FUSED_SHORT)
    check_against_f64(x, o1, s1, f"fused T={T} {state}")
    assert max_abs(o1, o0) <= 1e-2 and rel_fro(s1, s0) <= (2e-2 if state == "bf16" else 5e-3)
    if T == 16 and state == "fp32":
        cut = lambda a, b: {k: (v[:, a:b].contiguous() if k in ("q", "k", "v", "g", "beta") else v) for k, v in x.items()}
        xa, xb = cut(0, 8), cut(8, 16)
        oa, sa = run_gpu(xa, dt)
        xb["initial_state"] = sa
        ob, sb = run_gpu(xb, dt)
        assert max_abs(torch.cat([oa, ob], 1), o1) <= 1e-2 and rel_fro(sb, s1) <= 5e-3


@pytest.mark.parametrize("T,state", [(75, "fp32"), (1001, "bf16")])
def test_fused_kernel_walks_many_blocks(T, state):
    """The fused kernel is a complete forward pass; the dispatch only sends T <= 32 to it because the two-kernel path
    is faster beyond.  With the flag that lifts the limit it must reproduce a 5-block and a 63-block walk (ragged last
    block, bf16 and fp32 state)."""
    w = Workload("fb", H=2, B=3, T=T, state_in=state, state_out=state, state_std=0.5, seed=T, lower_bound=-1.0)
    x = make_inputs(w)
    dt = torch.bfloat16 if state == "bf16" else torch.float32
    out, fin = run_gpu(x, dt, F.FLAG_FUSED_ANY_T)
    check_against_f64(x, out, fin, f"fused-many-blocks T={T}")
    o0, s0 = run_gpu(x, dt)
    assert not torch.equal(out.view(torch.int16), o0.view(torch.int16)), "the flag did not change the path"


def test_runs_on_the_current_stream():
    """Like the reference (csrc/flash_kda.cpp:136) the call enqueues on torch's current stream and does not synchronise:
    on a side stream it gives the result of the default stream, and the caller's stream ordering is what protects it."""
    w = Workload("stream", H=4, B=2, T=300, state_in="fp32", state_out="fp32", seed=8)
    x = to_cuda(make_inputs(w))
    def call(out, fin):
        flash_kda.fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], out, x["A_log"], x["dt_bias"], x["lower_bound"],
                      initial_state=x["initial_state"], final_state=fin)
    o0, f0 = torch.empty_like(x["v"]), torch.empty(2, 4, 128, 128, device="cuda")
    call(o0, f0)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    o1, f1 = torch.empty_like(x["v"]), torch.empty(2, 4, 128, 128, device="cuda")
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call(o1, f1)
    side.synchronize()
    assert torch.equal(o0.view(torch.int16), o1.view(torch.int16)) and torch.equal(f0, f1)


@pytest.mark.parametrize("name", golden_names())
def test_reference_rounding_mode_reproduces_golden_vectors(name):
    """With FLAG_REFERENCE_ROUNDING the forward pass uses the reference's tile size, bf16 state and rounding points
    (one slow kernel): its results are then the reference's own, bit for bit, for most elements - the golden vectors
    were made by the reference's tests/torch_ref.py - where the production path agrees with only a quarter of them.
    What differs comes from the hardware tanh / exp2 and the summation order of the tensor cores."""
    x, ref_out, ref_fin = load_golden(name)
    fin_dtype = None if ref_fin is None else ref_fin.dtype
    out, fin = run_gpu(x, fin_dtype, F.FLAG_REFERENCE_ROUNDING)
    same = (out.view(torch.int16) == ref_out.view(torch.int16)).float().mean().item()
    diff = (out.float() - ref_out.float()).abs()
    rel = (diff / ref_out.float().abs().clamp_min(1e-3)).max().item()
    print(f"{name}: out identical {same:.4f}, max rel diff {rel:.3e}")
    assert same >= 0.88 and rel <= 0.1                      # at most a few bf16 ulps apart anywhere
    if fin is not None:
        if fin.dtype == torch.bfloat16:
            same_s = (fin.view(torch.int16) == ref_fin.view(torch.int16)).float().mean().item()
            assert same_s >= 0.97, same_s
        else:
            assert rel_fro(fin, ref_fin) <= 1.5e-3 and (fin == ref_fin).float().mean().item() >= 0.97
    check_against_f64(x, out, fin, f"{name}[reference rounding]",
                      big_state=x["initial_state"] is not None and x["initial_state"].float().abs().max() > 100)


def test_reference_rounding_mode_matches_the_c_port_on_a_varlen_batch():
    """Same mode against the oracle's C port of the reference algorithm (ragged varlen batch, bf16 state in and out)."""
    w = Workload("refmode", H=3, seq_lens=[37, 1, 16, 100, 15], state_in="bf16", state_out="bf16", state_std=0.5, seed=5,
                 lower_bound=-2.0)
    x = make_inputs(w)
    out, fin = run_gpu(x, torch.bfloat16, F.FLAG_REFERENCE_ROUNDING)
    o_ref, s_ref = oracle.chunk16(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["A_log"], x["dt_bias"],
                                  x["lower_bound"], initial_state=x["initial_state"], cu_seqlens=x["cu_seqlens"],
                                  final_state_dtype=torch.bfloat16)
    same_o = (out.view(torch.int16) == o_ref.view(torch.int16)).float().mean().item()
    same_s = (fin.view(torch.int16) == s_ref.view(torch.int16)).float().mean().item()
    print(f"identical: out {same_o:.4f}, state {same_s:.4f}")
    assert same_o >= 0.88 and same_s >= 0.95
    check_against_f64(x, out, fin, "reference rounding, varlen")
