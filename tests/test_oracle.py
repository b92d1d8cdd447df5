"""CPU-only: pins the oracle (oracle/kda_oracle.c) against vectors produced by the reference's
own tests/torch_ref.py, and the fp64 recurrence against both."""
import pytest
import torch

import oracle
from helpers import OUT_MAX_ABS, STATE_REL, golden_names, load_golden, max_abs, rel_fro


@pytest.mark.parametrize("name", golden_names())
def test_chunk16_port_matches_reference_vectors(name):
    x, ref_out, ref_fin = load_golden(name)
    fin_dtype = None if ref_fin is None else ref_fin.dtype
    out, fin = oracle.chunk16(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["A_log"],
                              x["dt_bias"], x["lower_bound"], initial_state=x["initial_state"],
                              final_state_dtype=fin_dtype, cu_seqlens=x["cu_seqlens"])
    # Same rounding points as the reference; only fp32 summation order and tanhf-vs-torch.tanh
    # differ, so all but a sliver of the bf16 outputs must be bit-identical and the rest one
    # or two bf16 ulps away.
    mism = (out.view(torch.int16) != ref_out.view(torch.int16)).float().mean().item()
    assert mism < 2e-2, f"{name}: {mism:.4f} of outputs differ from the reference vectors"
    scale_ref = ref_out.float().abs().max().item()
    assert max_abs(out, ref_out) <= 2 ** -6 * max(scale_ref, 1.0)
    if ref_fin is not None:
        assert rel_fro(fin, ref_fin) < 2e-3


@pytest.mark.parametrize("name", golden_names())
def test_fp64_recurrence_agrees_with_reference_vectors(name):
    x, ref_out, ref_fin = load_golden(name)
    out, fin = oracle.recurrence_f64(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"],
                                     x["A_log"], x["dt_bias"], x["lower_bound"],
                                     initial_state=x["initial_state"], cu_seqlens=x["cu_seqlens"])
    big_state = x["initial_state"] is not None and x["initial_state"].float().abs().max() > 100
    if not big_state:
        assert max_abs(ref_out, out) <= OUT_MAX_ABS
    else:  # arange-valued stress state: outputs are O(1e4); compare relatively
        assert rel_fro(ref_out, out) < 1e-2
    if ref_fin is not None:
        assert rel_fro(ref_fin, fin) <= STATE_REL


def test_recurrence_split_equals_unsplit():
    """initial_state/final_state are the resumable state: running 96 tokens in one call equals
    64 tokens then 32 tokens with the state handed over."""
    x, _, _ = load_golden("fixed_T97_H2_bf16state")
    cut = lambda t, a, b: t[:, a:b].contiguous()
    args = lambda a, b: (cut(x["q"], a, b), cut(x["k"], a, b), cut(x["v"], a, b), cut(x["g"], a, b),
                         cut(x["beta"], a, b), x["scale"], x["A_log"], x["dt_bias"], x["lower_bound"])
    o_all, s_all = oracle.recurrence_f64(*args(0, 96), initial_state=x["initial_state"])
    o1, s1 = oracle.recurrence_f64(*args(0, 64), initial_state=x["initial_state"])
    o2, s2 = oracle.recurrence_f64(*args(64, 96), initial_state=s1.float())
    assert max_abs(torch.cat([o1, o2], 1), o_all) < 1e-5
    assert rel_fro(s2, s_all) < 1e-6


def test_chunk_operands_reproduce_recurrence():
    """The chunk-32 WY operands (what the prepare kernel is checked against) reproduce the
    per-token recurrence when pushed through U = up - wp S, out = qpp S + mqk U,
    S' = diag(ec) S + kr^T U."""
    x, _, _ = load_golden("fixed_T97_H2_bf16state")
    T, H, C = 97, 2, 32
    o_ref, s_ref = oracle.recurrence_f64(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"],
                                         x["A_log"], x["dt_bias"], x["lower_bound"],
                                         initial_state=x["initial_state"])
    for h in range(H):
        S = x["initial_state"][0, h].double().t().clone()          # [K][V]
        for t0 in range(0, T, C):
            n = min(C, T - t0)
            r = oracle.chunk_operands(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"],
                                      x["A_log"], x["dt_bias"], x["lower_bound"], h, t0, n, C)
            U = r["up"] - r["wp"] @ S
            O = r["qpp"] @ S + r["mqk"] @ U
            S = r["ec"][:, None] * S + r["kr"].t() @ U
            assert max_abs(O[:n], o_ref[0, t0:t0 + n, h]) < 1e-9
        assert rel_fro(S.t(), s_ref[0, h]) < 1e-12
