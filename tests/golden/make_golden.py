"""Generate golden vectors by running the reference's own oracle, tests/torch_ref.py.

Run in a container that has the reference checkout mounted:

    python tests/golden/make_golden.py /path/to/reference

tests/torch_ref.py needs a GPU for two calls only; both are substituted here, in memory,
without touching the reference's files:
  * its inline CUDA extension `sigmoid_tanh_fp32` (tanh.approx based) -> tanh(x/2)/2+1/2 in fp32,
  * `torch.mm(a, b, out_dtype=float32)` (no CPU kernel) -> fp32 matmul of the up-cast operands
    (bf16 products are exact in fp32; only the summation order differs).
Everything else -- the chunk loop and every bf16 rounding point -- is the reference's code.
Each .npz holds the inputs (bf16 as uint16 bit patterns) and the reference's `out` and
`final_state`, so the tests need neither the reference nor a particular RNG.
"""
import math
import os
import sys
import types

import numpy as np
import torch
import torch.utils.cpp_extension as cpp_ext

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from flashkda_b200.workloads import Workload, baseline_workload, make_inputs  # noqa: E402


def import_reference_oracle(ref_root):
    cpp_ext.load_inline = lambda *a, **k: types.SimpleNamespace(
        sigmoid_tanh_fp32=lambda x: torch.tanh(x * 0.5) * 0.5 + 0.5)
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    import torch_ref as R
    _mm = torch.mm

    def mm(a, b, out_dtype=None):
        if out_dtype is None:
            return _mm(a, b)
        return _mm(a.float(), b.float()).to(out_dtype)

    torch.mm = mm
    return R


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 \
        else t.contiguous().numpy()


def reference_style_inputs(T, H, seed=42):
    """Input distributions of the reference's exact-match matrix (tests/test_fwd_full.py:26-44):
    pre-normalised q/k, U(0,1) A_log and dt_bias, and an arange-valued (huge) initial state."""
    import torch.nn.functional as F
    torch.manual_seed(seed)
    q = F.normalize(torch.randn(1, T, H, 128), p=2, dim=-1).to(torch.bfloat16)
    k = F.normalize(torch.randn(1, T, H, 128), p=2, dim=-1).to(torch.bfloat16)
    v = torch.randn(1, T, H, 128).to(torch.bfloat16)
    g = torch.randn(1, T, H, 128).to(torch.bfloat16)
    beta = torch.randn(1, T, H).to(torch.bfloat16)
    A_log = torch.rand(H)
    dt_bias = torch.rand(H, 128)
    return dict(q=q, k=k, v=v, g=g, beta=beta, A_log=A_log, dt_bias=dt_bias,
                scale=1.0 / math.sqrt(128), lower_bound=-5.0)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    ref_root = sys.argv[1]
    R = import_reference_oracle(ref_root)
    cases = []

    w = baseline_workload(0)
    cases.append(("c0_B1_T1024_H4_fp32out", make_inputs(w), False))

    w = Workload("tail97", H=2, B=1, T=97, state_in="bf16", state_out="bf16", seed=1)
    cases.append(("fixed_T97_H2_bf16state", make_inputs(w), True))

    w = Workload("varlen", H=2, seq_lens=[17, 33, 65, 5], state_in="fp32", state_out="fp32",
                 state_std=1.0, seed=2)
    cases.append(("varlen_17_33_65_5_H2_fp32state", make_inputs(w), True))

    w = Workload("batched", H=2, B=3, T=48, state_in=None, state_out="bf16", lower_bound=-2.0, seed=3)
    cases.append(("batched_B3_T48_H2_lb2", make_inputs(w), True))

    x = reference_style_inputs(64, 1)
    st = torch.arange(128 * 128, dtype=torch.float32).reshape(1, 1, 128, 128).to(torch.bfloat16).float()
    x.update(initial_state=st, final_state=torch.zeros_like(st), out=torch.zeros_like(x["v"]),
             cu_seqlens=None)
    cases.append(("refstyle_T64_H1_arange_state", x, True))

    for name, x, keep_inputs in cases:
        out = torch.zeros_like(x["v"])
        fin = None if x["final_state"] is None else torch.zeros_like(x["final_state"])
        init = None if x["initial_state"] is None else x["initial_state"].clone()
        R.torch_ref(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], out, x["A_log"],
                    x["dt_bias"], x["lower_bound"], initial_state=init, final_state=fin,
                    cu_seqlens=x["cu_seqlens"])
        rec = dict(out=bits(out), scale=np.float64(x["scale"]), lower_bound=np.float64(x["lower_bound"]))
        if fin is not None:
            rec["final_state"] = bits(fin)
            rec["final_is_bf16"] = np.bool_(fin.dtype == torch.bfloat16)
        if x["cu_seqlens"] is not None:
            rec["cu_seqlens"] = x["cu_seqlens"].numpy()
        if keep_inputs:
            for key in ("q", "k", "v", "g", "beta", "A_log", "dt_bias"):
                rec[key] = bits(x[key])
            if init is not None:
                rec["initial_state"] = bits(init)
                rec["initial_is_bf16"] = np.bool_(init.dtype == torch.bfloat16)
        else:
            # inputs come from flashkda_b200.workloads (seeded CPU generator); keep a fingerprint
            rec["input_checksum"] = np.float64(sum(float(x[key].double().sum()) for key in
                                                   ("q", "k", "v", "g", "beta", "A_log", "dt_bias")))
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **rec)
        print(name, "->", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
