"""GPU: the drop-in claim end to end.  flash-linear-attention's `chunk_kda` dispatcher looks for a
module named `flash_kda` (find_spec) and, under inference mode with the in-kernel gate / L2-norm /
beta-sigmoid flags, routes the call to `flash_kda.fwd` (reference README "FLA integration";
fla/ops/kda/backends/flashkda.py).  Here that module is this repository's: the unmodified FLA
caller must reach our `fwd`, with its own argument massaging (scale=None, 1-D dt_bias, int32
cu_seqlens, fp32 final state it allocates itself), and the results must match the oracle."""
import os

import pytest
import torch

import flash_kda
import oracle
from flashkda_b200.workloads import Workload, make_inputs
from helpers import OUT_MAX_ABS, STATE_REL, max_abs, rel_fro, to_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("varlen", [False, True], ids=["batched", "varlen"])
def test_fla_chunk_kda_dispatches_to_this_flash_kda(varlen, monkeypatch):
    os.environ.pop("FLA_FLASH_KDA", None)
    try:
        from fla.ops.kda import chunk_kda
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"flash-linear-attention not importable here: {e}")
    calls = []
    real_fwd = flash_kda.fwd

    def spy(*a, **kw):
        calls.append(1)
        return real_fwd(*a, **kw)

    monkeypatch.setattr(flash_kda, "fwd", spy)
    w = Workload("fla", H=4, seq_lens=[70, 33, 25], state_in="fp32", seed=77) if varlen else \
        Workload("fla", H=4, B=2, T=96, state_in="fp32", seed=78)
    x = make_inputs(w)
    xc = to_cuda(x)
    cu32 = None if xc["cu_seqlens"] is None else xc["cu_seqlens"].to(torch.int32)
    with torch.inference_mode():
        out, fin = chunk_kda(xc["q"], xc["k"], xc["v"], xc["g"], xc["beta"], scale=None,
                             initial_state=xc["initial_state"], output_final_state=True,
                             use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                             cu_seqlens=cu32, safe_gate=True, lower_bound=x["lower_bound"],
                             transpose_state_layout=True, A_log=xc["A_log"], dt_bias=xc["dt_bias"].reshape(-1))
    torch.cuda.synchronize()
    if not calls:
        pytest.skip("this FLA build did not route chunk_kda to the flash_kda backend")
    o64, s64 = oracle.recurrence_f64(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["A_log"], x["dt_bias"],
                                     x["lower_bound"], initial_state=x["initial_state"], cu_seqlens=x["cu_seqlens"])
    assert fin.dtype == torch.float32
    assert max_abs(out.cpu(), o64) <= OUT_MAX_ABS
    assert rel_fro(fin.cpu(), s64) <= STATE_REL
