"""Bit-exact mode against the reference's own CUDA kernels (reference contract: tests/test_fwd_full.py:90-94,
tests/test_fwd.py:260-261, `torch.equal` of the kernel's result with its torch restatement on the GPU).

With FKDA_FLAG_REFERENCE_ROUNDING the forward pass uses the reference's 16-token tile, bf16 state between tiles, its
rounding points and the same hardware approximations (tanh.approx, ex2.approx, rsqrt.approx, mma.sync m16n8k16 in the same
k order).  The reference's unmodified extension, built for sm_100a into baseline/_ref, runs on the same tensors: `out`
and the final state must be the same bits.  Skipped where that build is absent."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

import flashkda_b200 as F  # noqa: E402
from flashkda_b200.workloads import Workload, make_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


def _reference():
    try:
        import flash_kda_C as R
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"reference extension not built in baseline/_ref: {type(e).__name__}: {e}")
    return R


def _both(w):
    R = _reference()
    dev = torch.device("cuda", 0)
    x = make_inputs(w, device=dev)
    B, T, H = x["q"].shape[:3]
    ws_ref = torch.empty(R.get_workspace_size(B * T, H, w.N), dtype=torch.uint8, device=dev)
    out_ref, out = torch.zeros_like(x["v"]), torch.zeros_like(x["v"])
    fin_ref = None if x["final_state"] is None else torch.zeros_like(x["final_state"])
    fin = None if x["final_state"] is None else torch.zeros_like(x["final_state"])
    kw = dict(initial_state=x["initial_state"], cu_seqlens=x["cu_seqlens"])
    R.fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], float(x["scale"]), out_ref, ws_ref, x["A_log"], x["dt_bias"],
          x["lower_bound"], final_state=fin_ref, **kw)
    F.fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], out, x["A_log"], x["dt_bias"], x["lower_bound"],
          final_state=fin, flags=F.FLAG_REFERENCE_ROUNDING, **kw)
    torch.cuda.synchronize()
    return out, out_ref, fin, fin_ref


def _assert_same_bits(out, out_ref, fin, fin_ref):
    assert torch.equal(out.view(torch.int16), out_ref.view(torch.int16))
    if fin is not None:
        it = torch.int32 if fin.dtype == torch.float32 else torch.int16
        assert torch.equal(fin.view(it), fin_ref.view(it))


STATES = [(None, None), (None, "fp32"), ("fp32", "fp32"), ("bf16", "bf16"), ("bf16", None)]


@pytest.mark.parametrize("state", STATES, ids=lambda s: f"{s[0]}-{s[1]}")
@pytest.mark.parametrize("T", [1, 16, 17, 31, 33, 37, 97, 256, 1024])
def test_fixed_length_matches_the_reference_kernels_bit_for_bit(T, state):
    w = Workload("bits", H=4, B=2, T=T, state_in=state[0], state_out=state[1], seed=100 + T)
    _assert_same_bits(*_both(w))


@pytest.mark.parametrize("state", [(None, "fp32"), ("bf16", "bf16"), ("fp32", "fp32")], ids=lambda s: f"{s[0]}-{s[1]}")
@pytest.mark.parametrize("lens", [[100, 33, 257, 16, 700], [1, 15, 16, 17, 31, 32, 33], [1300, 547, 2048, 963, 271, 3063]],
                         ids=["mixed", "edges", "reference_bench"])
def test_varlen_matches_the_reference_kernels_bit_for_bit(lens, state):
    w = Workload("bitsv", H=3, seq_lens=lens, state_in=state[0], state_out=state[1], seed=7)
    _assert_same_bits(*_both(w))


def test_headline_shape_matches_the_reference_kernels_bit_for_bit():
    w = Workload("bitsC1", H=8, B=2, T=8192, state_in="fp32", state_out="fp32", seed=9)
    _assert_same_bits(*_both(w))
