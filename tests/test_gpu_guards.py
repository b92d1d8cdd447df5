"""GPU: nothing outside the rows and buffers a call owns is written.

compute-sanitizer is not available where these tests run, so out-of-bounds writes are looked for
with canaries: `out`, `final_state` and the workspace are views into larger buffers whose
surroundings hold a bit pattern, and varlen calls get tensors with more rows than
`cu_seqlens[-1]` covers.  After the call the guard bands and the surplus rows must be
bit-unchanged, for every kernel form.  The reference has a slow path just for this: a tail tile
must not overwrite the next sequence's rows (csrc/smxx/fwd_kernel2.cuh:757-766).
"""
import pytest
import torch

import flash_kda
import flashkda_b200 as F
import oracle
from flashkda_b200.workloads import Workload, make_inputs
from helpers import OUT_MAX_ABS, STATE_REL, max_abs, rel_fro

pytestmark = pytest.mark.gpu

GUARD = 4096          # bytes on either side
PATTERN = 0x5A


def guarded(nbytes, align=256):
    """A zero-copy uint8 view of `nbytes` with GUARD patterned bytes before and after it."""
    pad = (-nbytes) % align
    buf = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device="cuda")
    return buf, buf[GUARD:GUARD + nbytes]


def guards_intact(buf, nbytes):
    return bool((buf[:GUARD] == PATTERN).all()) and bool((buf[GUARD + nbytes:] == PATTERN).all())


def run_guarded(w, surplus_rows, flags):
    x = make_inputs(w)
    B, T, H = x["q"].shape[:3]
    Tt = T + surplus_rows                       # rows the tensors really have
    cu = x["cu_seqlens"]
    gen = torch.Generator().manual_seed(5)

    def widen(t):                               # append rows of plausible data that no sequence owns
        if surplus_rows == 0:
            return t.cuda()
        extra = torch.randn(B, surplus_rows, *t.shape[2:], generator=gen).to(t.dtype)
        return torch.cat([t, extra], 1).contiguous().cuda()

    q, k, v, g, beta = (widen(x[n]) for n in ("q", "k", "v", "g", "beta"))
    out_buf, out_u8 = guarded(B * Tt * H * 128 * 2)
    out = out_u8.view(torch.bfloat16).view(B, Tt, H, 128)
    out_u8.fill_(PATTERN)
    fin_dt = None if x["final_state"] is None else x["final_state"].dtype
    fin_buf = fin = None
    if fin_dt is not None:
        esz = 2 if fin_dt == torch.bfloat16 else 4
        fin_buf, fin_u8 = guarded(w.N * H * 128 * 128 * esz)
        fin = fin_u8.view(fin_dt).view(w.N, H, 128, 128)
    ws_bytes = F.get_workspace_size(B * Tt, H, w.N, flags)
    ws_buf, ws = guarded(ws_bytes)
    init = None if x["initial_state"] is None else x["initial_state"].cuda()
    flash_kda.fwd(q, k, v, g, beta, x["scale"], out, x["A_log"].cuda(), x["dt_bias"].cuda(), x["lower_bound"],
                  initial_state=init, final_state=fin, cu_seqlens=None if cu is None else cu.cuda(), workspace=ws, flags=flags)
    assert F.read_status(ws) == 0
    torch.cuda.synchronize()
    assert guards_intact(out_buf, out_u8.numel()), "bytes around `out` were written"
    assert guards_intact(ws_buf, ws_bytes), "bytes around the workspace were written"
    if fin is not None:
        assert guards_intact(fin_buf, fin.numel() * fin.element_size()), "bytes around `final_state` were written"
    if surplus_rows:
        tail = out[:, T:].contiguous().view(torch.uint8)
        assert bool((tail == PATTERN).all()), "out rows past cu_seqlens[-1] were written"
    # and the rows that are owned are right
    o64, s64 = oracle.recurrence_f64(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["A_log"], x["dt_bias"],
                                     x["lower_bound"], initial_state=x["initial_state"], cu_seqlens=cu)
    assert max_abs(out[:, :T].cpu(), o64) <= OUT_MAX_ABS
    if fin is not None:
        assert rel_fro(fin.cpu(), s64) <= STATE_REL


FORMS = {
    "default": 0,
    "lookahead": F.FLAG_SCAN_LOOKAHEAD,
    "compact": F.FLAG_SCAN_PLAIN,
    "segmented": F.FLAG_SCAN_LOOKAHEAD | F.FLAG_SEGMENTS(3),
    "segmented_compact": F.FLAG_SCAN_PLAIN | F.FLAG_SEGMENTS(3),
    "simt": F.FLAG_SCAN_SIMT,
    "mma_sync_prepare": F.FLAG_PREPARE_MMA_SYNC,
    "tcgen05_cta_per_item_prepare": F.FLAG_PREPARE_TCGEN05,
    "reference_rounding": F.FLAG_REFERENCE_ROUNDING,
}


@pytest.mark.parametrize("form", list(FORMS))
@pytest.mark.parametrize("seq_lens", [[45, 3], [17, 33, 65, 5], [32 * 9 + 1, 70]], ids=lambda s: "seqs" + "_".join(map(str, s)))
def test_varlen_tail_rows_and_guard_bands(seq_lens, form):
    state = "bf16" if len(seq_lens) == 2 else "fp32"
    w = Workload("guard", H=3, seq_lens=seq_lens, state_in=state, state_out=state, state_std=0.5, seed=sum(seq_lens))
    run_guarded(w, surplus_rows=41, flags=FORMS[form])


@pytest.mark.parametrize("B,T,flags", [(5, 16, 0), (7, 23, 0), (4, 9, F.FLAG_NO_FUSED_SHORT), (9, 50, 0), (3, 33, 0), (40, 129, 0),
                                       (200, 150, 0), (2, 300, 0)],
                         ids=["fused16", "fused23", "short9", "short50", "short33", "fixed129", "manyshort150", "fixed300"])
def test_fixed_length_guard_bands(B, T, flags):
    """Fixed-length forms (fused short-sequence kernel, persistent short-chain kernel, short-chunk prepare, plain path)
    with partial last chunks: guard bands around out, final state and workspace stay untouched."""
    w = Workload("guardf", H=3, B=B, T=T, state_in="fp32", state_out="fp32", state_std=0.5, seed=B * 1000 + T)
    run_guarded(w, surplus_rows=0, flags=flags)
