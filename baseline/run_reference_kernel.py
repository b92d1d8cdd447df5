"""Time the UNMODIFIED reference CUDA extension (flash_kda_C, built for sm_100a into
baseline/_ref by `pip install --target baseline/_ref` from a copy of the reference with the
CUTLASS headers of the flashinfer wheel linked in as its `cutlass/` submodule) on the same
synthetic workloads as bench.py, with the same CUDA-event method, and report its distance to
this repository's kernels.  Informational: the "same GPU, reference kernels" comparison.
Usage: python baseline/run_reference_kernel.py [config ...]
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

from flashkda_b200.workloads import Workload, baseline_workload, make_inputs  # noqa: E402


def main():
    try:
        import flash_kda_C as R
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference_kernel", "unavailable": f"{type(e).__name__}: {e}"}))
        return
    import flashkda_b200 as F
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfgs = [int(a) for a in sys.argv[1:]] or [1]
    extra = {91: Workload("ref_bench_T8192_H96", H=96, B=1, T=8192, state_in="bf16", state_out="bf16"),
             92: Workload("ref_bench_T8192_H64", H=64, B=1, T=8192, state_in="bf16", state_out="bf16"),
             93: Workload("ref_bench_varlen6_H96", H=96, seq_lens=[1300, 547, 2048, 963, 271, 3063], state_in="bf16", state_out="bf16"),
             94: Workload("ref_bench_1024x8_H96", H=96, seq_lens=[1024] * 8, state_in="bf16", state_out="bf16")}
    for c in cfgs:
        w = extra[c] if c in extra else baseline_workload(c)
        x = make_inputs(w, device=dev)
        B, T, H = x["q"].shape[:3]
        ws_ref = torch.empty(R.get_workspace_size(B * T, H, w.N), dtype=torch.uint8, device=dev)
        ws = torch.empty(F.get_workspace_size(B * T, H, w.N), dtype=torch.uint8, device=dev)
        out_ref, out = torch.zeros_like(x["v"]), torch.zeros_like(x["v"])
        fin_ref = None if x["final_state"] is None else torch.zeros_like(x["final_state"])
        kw = dict(initial_state=x["initial_state"], cu_seqlens=x["cu_seqlens"])

        def ref():
            R.fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], float(x["scale"]), out_ref, ws_ref, x["A_log"], x["dt_bias"],
                  x["lower_bound"], final_state=fin_ref, **kw)

        def ours():
            F.fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], out, x["A_log"], x["dt_bias"], x["lower_bound"],
                  final_state=x["final_state"], workspace=ws, **kw)

        res = {"impl": "reference_kernel", "workload": w.name}
        for name, fn in (("reference_ms", ref), ("this_repo_ms", ours)):
            for _ in range(5):
                fn()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for _ in range(20):
                fn()
            b.record()
            torch.cuda.synchronize()
            res[name] = a.elapsed_time(b) / 20
        res["tokens"] = w.total_tokens
        res["reference_tokens_per_s"] = w.total_tokens / (res["reference_ms"] * 1e-3)
        res["this_repo_tokens_per_s"] = w.total_tokens / (res["this_repo_ms"] * 1e-3)
        res["out_max_abs_diff"] = (out.float() - out_ref.float()).abs().max().item()
        if fin_ref is not None:
            res["state_rel_diff"] = ((x["final_state"].float() - fin_ref.float()).norm() / fin_ref.float().norm()).item()
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
