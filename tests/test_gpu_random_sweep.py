"""Seeded random sweep of shapes, state variants, gate regimes and call forms against the fp64 recurrence.

Complements the fixed matrices of test_gpu_fwd.py (which follow the reference's tests/test_fwd_full.py:48-205): every
case draws batch / length / heads / varlen mix / state dtypes / lower bound / gate scale at random, so that kernel
selection (fused short-sequence kernel, persistent short-chain scan, look-ahead scan, segment-parallel scan, short-chunk
prepare) and ragged edges meet in combinations nobody wrote down."""
import random

import pytest
import torch

import flashkda_b200 as F
from flashkda_b200.workloads import Workload, make_inputs
from test_gpu_fwd import check_against_f64, run_gpu

pytestmark = pytest.mark.gpu


def draw_case(seed):
    rng = random.Random(seed)
    H = rng.choice([1, 2, 3, 4, 6])
    state_in = rng.choice([None, "bf16", "fp32"])
    state_out = state_in if state_in is not None else rng.choice([None, "bf16", "fp32"])
    lower_bound = rng.choice([-5.0, -5.0, -2.0, -0.5])
    kind = rng.choice(["fixed_short", "fixed", "fixed_long", "varlen", "varlen_many"])
    if kind == "fixed_short":
        B, T, seq = rng.randint(1, 40), rng.randint(1, 70), None
    elif kind == "fixed":
        B, T, seq = rng.randint(1, 6), rng.randint(71, 700), None
    elif kind == "fixed_long":
        B, T, seq = 1, rng.randint(1536, 2600), None            # few long chains: the planner cuts them into runs
        H = rng.choice([1, 2, 4])
    elif kind == "varlen":
        seq = [rng.randint(1, 400) for _ in range(rng.randint(1, 6))]
        B, T = 1, sum(seq)
    else:
        seq = [rng.randint(1, 40) for _ in range(rng.randint(8, 60))]
        B, T = 1, sum(seq)
    w = Workload(f"sweep{seed}_{kind}", H=H, B=B, T=T, seq_lens=seq, state_in=state_in, state_out=state_out,
                 state_std=rng.choice([0.02, 0.5]), seed=1000 + seed, lower_bound=lower_bound)
    return w, rng


@pytest.mark.parametrize("seed", range(48))
def test_random_case(seed):
    w, rng = draw_case(seed)
    x = make_inputs(w)
    if rng.random() < 0.3:       # gates near the ends of their range
        x["g"] = torch.full_like(x["g"], rng.choice([-6.0, 6.0]))
    fin_dtype = {None: None, "bf16": torch.bfloat16, "fp32": torch.float32}[w.state_out]
    out, fin = run_gpu(x, fin_dtype)
    big = x["initial_state"] is not None and w.state_std > 0.1
    check_against_f64(x, out, fin, w.name, big_state=big and x["initial_state"].float().abs().max() > 100)
