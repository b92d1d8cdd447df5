"""Shared helpers for the parity tests: golden-vector loading and error measures."""
import glob
import os

import numpy as np
import torch

from flashkda_b200.workloads import baseline_workload, make_inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances of the parity contract, against an fp32/fp64 evaluation of the operator:
OUT_MAX_ABS = 2e-2      # bf16 `out`, max absolute error
STATE_REL = 1e-2        # final state, relative Frobenius error


def _bf(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def golden_names():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "*.npz")))


def load_golden(name):
    """Returns (inputs dict as for flash_kda.fwd, ref_out bf16, ref_final or None)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    if "q" in z:
        x = dict(q=_bf(z["q"]), k=_bf(z["k"]), v=_bf(z["v"]), g=_bf(z["g"]), beta=_bf(z["beta"]),
                 A_log=torch.from_numpy(z["A_log"].copy()), dt_bias=torch.from_numpy(z["dt_bias"].copy()))
        x["initial_state"] = None
        if "initial_state" in z:
            x["initial_state"] = _bf(z["initial_state"]) if bool(z["initial_is_bf16"]) \
                else torch.from_numpy(z["initial_state"].copy())
    else:
        x = make_inputs(baseline_workload(0))
        chk = sum(float(x[key].double().sum()) for key in ("q", "k", "v", "g", "beta", "A_log", "dt_bias"))
        assert abs(chk - float(z["input_checksum"])) < 1e-6 * max(1.0, abs(chk)), \
            "seeded CPU generator no longer reproduces the inputs the golden vectors were made from"
        x = {key: x[key] for key in ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "initial_state")}
    x["scale"] = float(z["scale"])
    x["lower_bound"] = float(z["lower_bound"])
    x["cu_seqlens"] = torch.from_numpy(z["cu_seqlens"].copy()) if "cu_seqlens" in z else None
    out = _bf(z["out"])
    fin = None
    if "final_state" in z:
        fin = _bf(z["final_state"]) if bool(z["final_is_bf16"]) else torch.from_numpy(z["final_state"].copy())
    return x, out, fin


def max_abs(a, b):
    return (a.double() - b.double()).abs().max().item()


def rel_fro(a, b):
    """||a-b|| / ||b|| with b the trusted side."""
    b = b.double()
    return ((a.double() - b).norm() / (b.norm() + 1e-30)).item()


# ---- operand-record decoding (layout defined in flashkda_b200/csrc/fkda_common.cuh) ----
REC = dict(KR=0, MQK=8192, E=10240, WP=10752, QP=18944, UP=27136, BYTES=35328)


def _core_index(rows, cols):
    r = torch.arange(rows).view(-1, 1)
    c = torch.arange(cols).view(1, -1)
    return ((r // 8) * (cols * 16) + (c // 8) * 128 + (r % 8) * 16 + (c % 8) * 2) // 2


def decode_record(rec_u8):
    """rec_u8: CPU uint8 tensor of one 35328-byte record -> dict of float64 matrices."""
    def bf(off, nbytes):
        return rec_u8[off:off + nbytes].view(torch.bfloat16)
    idx = _core_index(32, 128)
    out = {}
    for name in ("WP", "QP", "KR"):
        out[name.lower()] = bf(REC[name], 8192)[idx].double()
    out["up"] = bf(REC["UP"], 8192)[_core_index(128, 32)].t().double()     # stored transposed: [128 v][32 tok]
    out["mqk"] = bf(REC["MQK"], 2048)[_core_index(32, 32)].double()
    out["ec"] = rec_u8[REC["E"]:REC["E"] + 512].view(torch.float32).double()
    return out


def to_cuda(x):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in x.items()}
