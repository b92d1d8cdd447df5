#!/usr/bin/env python
"""Benchmark of `flash_kda.fwd` (Kimi Delta Attention prefill) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 1|2|3|4] [--shard seq|head]
    python bench.py --impl reference            # the CPU restatement of the reference on host cores

One "step" is one `flash_kda.fwd` call over the whole synthetic batch.  At N=1 the workload is
the configuration the headline metric is quoted on: fixed-length prefill B=4, T=8192, H=32,
K=V=128, fp32 initial and final state.  With N ranks (one process per GPU, launched by
torch.distributed.run) every rank runs that workload on its own 4 sequences of a global batch
of 4N sequences: the operator has no cross-sequence or cross-head term, so ranks exchange
nothing on the data path (NCCL carries only the timing reduction) and the run is weak scaling.
`--shard head` instead splits the heads of the fixed N=1 workload over the ranks (strong scaling).

The JSON line carries:
  value        tokens/s over all ranks, inputs resident in HBM, CUDA-event timed, max over ranks, through the plain
               drop-in call (the workspace is allocated inside every call, as the reference's wrapper does);
               `preallocated_workspace` holds the same with a caller-provided workspace, `sustained` the same calls
               kept up for 0.6 s with the SM clock seen meanwhile
  e2e          tokens/s through the same public call with HOST (pinned) buffers: host->device
               copies of q,k,v,g,beta,state and device->host copies of out and final_state
               inside the timed region (fixed-length batches: one call per sequence, so that the
               copies of neighbouring sequences overlap with the forward pass; `mode` says which)
  roofline     dominant kernel: the algorithmic bytes that kernel itself moves / its mean duration,
               against the measured HBM copy bandwidth; `roofline_call` (the headline) is the
               call's algorithmic bytes over the whole call (all kernels)
  parity       a sample of (sequence, head) chains of the timed call's result against the fp64
               recurrence (N = 1, together with the CPU baseline leg)
  reference_kernel  the reference's own CUDA kernels, built unmodified for sm_100a, timed on the same
               inputs in the same process when that build is present (N = 1)
  strong       (N > 1) the fixed configurations 1 and 3 with their heads split over the N ranks: ms,
               tokens/s, efficiency against one GPU running the whole configuration, roofline fraction
  cpu_baseline the oracle's C port of the reference algorithm on this box's host cores, on a
               bounded sample of the same workload
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from flashkda_b200.workloads import (Workload, algorithmic_bytes, baseline_workload,  # noqa: E402
                                     make_inputs)

METRIC = "flash_kda.fwd tokens/s at H=32,K=V=128"
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.samples, self.proc, self.thread, self.gpu = [], None, None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [p.strip() for p in line.split(",")]))

    def stop(self, t_begin, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.samples if t_begin - 0.05 <= t <= t_end + 0.15 and len(r) >= 6]
        if not rows:
            rows = [r for _, r in self.samples if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": int(rows[0][1]) if rows[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(rows)}


def cpu_baseline_sample(w: Workload, target_s=12.0, nthreads=0):
    """Times the oracle's C port of the reference's chunk-16 algorithm (oracle/kda_oracle.c,
    restating tests/torch_ref.py of the reference) on the first tokens of sequence 0, all heads,
    of the same workload.  Returns (tokens_per_s, cores, description)."""
    import oracle
    # all host threads this process may use (torchrun pins OMP_NUM_THREADS=1, so ask the OS instead)
    cores = (len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()) if nthreads <= 0 else nthreads

    def run(B, T):
        ww = Workload("cpu_sample", H=w.H, B=B, T=T, lower_bound=w.lower_bound, state_in=w.state_in,
                      state_out=w.state_out, state_std=w.state_std, seed=w.seed)
        x = make_inputs(ww)
        fin_dtype = None if x["final_state"] is None else x["final_state"].dtype
        t0 = time.perf_counter()
        oracle.chunk16(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["A_log"], x["dt_bias"],
                       x["lower_bound"], initial_state=x["initial_state"], final_state_dtype=fin_dtype,
                       nthreads=cores)
        return time.perf_counter() - t0

    run(1, 64)                              # load the library, warm the threads
    pilot_T = 512
    pilot = run(1, pilot_T)
    want = pilot_T * target_s / max(pilot, 1e-6)        # tokens that would take target_s
    T_seq = w.T if w.seq_lens is None else 8192
    B_max = w.B if w.seq_lens is None else 4
    if want <= T_seq:
        B, T = 1, int(max(256, want) // 256 * 256)
    else:
        B, T = int(min(B_max, want // T_seq)), T_seq     # at most the whole workload
    dt = run(B, T)
    return B * T / dt, cores, f"{B} x {T} tokens (first sequences of the workload), all {w.H} heads, {w.state_in or 'no'} state in"


def workload_config(w, B, T, H_local, N):
    """The `config` object, the same in both arms: what is computed, nothing about how."""
    return {"workload": w.name, "B_per_gpu": B, "T": T, "H_per_gpu": H_local, "K": 128, "V": 128, "N_per_gpu": N,
            "state": f"{w.state_in} in / {w.state_out} out", "lower_bound": w.lower_bound}


def reference_arm(args, w, rank):
    """`--impl reference`: the reference's algorithm on the host cores (it has no CPU
    implementation of its own -- tests/torch_ref.py is GPU-only Python -- so this is the C port in
    oracle/, kind "port"), all host threads, on a bounded sample per step."""
    if rank != 0:
        return
    per_step = max(2.0, 40.0 / max(1, args.steps + args.warmup))
    vals = []
    desc, cores = "", 1
    for i in range(args.warmup + args.steps):
        v, cores, desc = cpu_baseline_sample(w, target_s=per_step)
        if i >= args.warmup:
            vals.append(v)
    value = sum(vals) / len(vals)
    sample_T = int(desc.split()[0]) * int(desc.split()[2])
    B, T = (1, w.total_tokens) if w.seq_lens is not None else (w.B, w.T)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sample_T / value,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(w, B, T, w.H, w.N),
            "run": {"where": "host cores of rank 0", "chunk": 16},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def time_cuda(fn, steps, stream):
    """Mean milliseconds per call of `fn` over `steps` back-to-back calls, CUDA events on `stream`."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record(stream)
    for _ in range(steps):
        fn()
    b.record(stream)
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def bind_near_gpu(local_rank, local_world):
    """Binds this process to host cores of the NUMA node its GPU hangs on (before any pinned memory is allocated), the
    node's cores being shared out among the ranks of the node.  Returns a description for the JSON line."""
    try:
        pr = torch.cuda.get_device_properties(local_rank)
        bus = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            node = 0
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
        cpus = []
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            cpus += list(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return {"numa_node": node, "bound": False, "why": "no allowed core on that node"}
        per = max(1, len(allowed) // max(1, local_world))
        mine = allowed[local_rank * per:(local_rank + 1) * per] or allowed
        os.sched_setaffinity(0, mine)
        return {"numa_node": node, "bound": True, "cores": len(mine), "pci": bus}
    except Exception as e:  # noqa: BLE001  (sysfs layout, permissions: binding is best effort)
        return {"bound": False, "why": f"{type(e).__name__}: {e}"}


def make_caller(flash_kda, x, ws, flags):
    """One forward call over the batch `x`: with `ws` the caller's workspace is used, with None the call allocates its
    own (the plain drop-in signature; the extra keywords of this repository's wrapper are then not passed at all)."""
    pos = (x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["out"], x["A_log"], x["dt_bias"], x["lower_bound"])
    kw = dict(initial_state=x["initial_state"], final_state=x["final_state"], cu_seqlens=x["cu_seqlens"])
    if ws is not None or flags:
        kw.update(workspace=ws, flags=flags)
    return lambda: flash_kda.fwd(*pos, **kw)


def strong_scaling(F, flash_kda, cfg_idx, world, rank, dev, stream, steps, flags, dist):
    """Configuration `cfg_idx` as a fixed problem: one GPU runs all of it (rank 0 alone, the others wait), then its heads
    are split over the ranks.  Returns ms on one GPU, ms on N (max over ranks), tokens/s, efficiency, roofline fraction."""
    from flashkda_b200.sharding import plan, reduce_max_ms
    w = baseline_workload(cfg_idx)
    res = {"workload": w.name, "tokens": w.total_tokens, "heads_per_gpu": w.H // world}
    t_one = 0.0
    if rank == 0:
        x = make_inputs(w, device=dev)
        B, T, H = x["q"].shape[:3]
        ws = torch.empty(F.get_workspace_size(B * T, H, w.N, flags), dtype=torch.uint8, device=dev)
        call = make_caller(flash_kda, x, ws, flags)
        for _ in range(3):
            call()
        t_one = time_cuda(call, steps, stream)
        del x, ws, call
        torch.cuda.empty_cache()
    torch.cuda.synchronize()
    dist.barrier()
    shard = plan(w, world, rank, "head")
    x = make_inputs(shard.workload, device=dev, heads=shard.heads)
    B, T, H = x["q"].shape[:3]
    ws = torch.empty(F.get_workspace_size(B * T, H, w.N, flags), dtype=torch.uint8, device=dev)
    call = make_caller(flash_kda, x, ws, flags)
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    dist.barrier()
    t_n = time_cuda(call, steps, stream)
    t_one, t_n = reduce_max_ms([t_one, t_n], world, dev)
    peak, _ = measured_peaks()
    alg = algorithmic_bytes(w.total_tokens, w.H, w.N, w.state_in, w.state_out)
    res.update({"ms_one_gpu": t_one, "ms": t_n, "tokens_per_s": w.total_tokens / (t_n * 1e-3),
                "efficiency": t_one / (world * t_n), "roofline_frac": alg / (t_n * 1e-3) / 1e9 / (world * peak),
                "roofline_frac_one_gpu": alg / (t_one * 1e-3) / 1e9 / peak})
    del x, ws, call
    torch.cuda.empty_cache()
    return res


def reference_kernel_leg(x, w, ms_ours, stream, steps):
    """The reference's own CUDA extension (built unmodified for sm_100a into baseline/_ref) on the same inputs."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(ref_dir):
        return {"unavailable": "baseline/_ref is not installed on this machine"}
    try:
        if ref_dir not in sys.path:
            sys.path.append(ref_dir)          # after ROOT: `flash_kda` stays this repository's module
        import flash_kda_C as R
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}
    B, T, H = x["q"].shape[:3]
    out_ref = torch.empty_like(x["v"])
    fin_ref = None if x["final_state"] is None else torch.empty_like(x["final_state"])

    def ref():        # as the reference's Python wrapper does: the workspace is allocated inside the call
        ws_ref = torch.empty(R.get_workspace_size(B * T, H, w.N), dtype=torch.uint8, device=x["q"].device)
        R.fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], float(x["scale"]), out_ref, ws_ref, x["A_log"], x["dt_bias"],
              x["lower_bound"], initial_state=x["initial_state"], final_state=fin_ref, cu_seqlens=x["cu_seqlens"])
    try:
        for _ in range(3):
            ref()
        ms = time_cuda(ref, steps, stream)
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}
    res = {"ms": ms, "tokens_per_s": w.total_tokens / (ms * 1e-3), "ratio": ms / ms_ours,
           "out_max_abs_diff": (x["out"].float() - out_ref.float()).abs().max().item()}
    if fin_ref is not None:
        res["state_rel_diff"] = ((x["final_state"].float() - fin_ref.float()).norm() / fin_ref.float().norm()).item()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="fkda", choices=["fkda", "reference"])
    ap.add_argument("--config", type=int, default=1, help="index of the headline configuration (1..4)")
    ap.add_argument("--shard", default="seq", choices=["seq", "head"])
    ap.add_argument("--shape", default=None, help="B,T,H override of the fixed-length workload (profiling on a small case)")
    ap.add_argument("--flags", type=lambda v: int(v, 0), default=0,
                    help="FKDA_FLAG_* bits passed to every call (kernel selection; tuning aid)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline and the parity check done with it")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the strong-scaling block")
    ap.add_argument("--no-reference-kernel", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "fkda" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    w = baseline_workload(args.config)
    if args.shape:
        b_, t_, h_ = (int(v) for v in args.shape.split(","))
        w = Workload(f"custom_B{b_}_T{t_}_H{h_}", H=h_, B=b_, T=t_, lower_bound=w.lower_bound, state_in=w.state_in,
                     state_out=w.state_out, state_std=w.state_std)

    if args.impl == "reference":
        reference_arm(args, w, rank)
        return

    import flash_kda
    import flashkda_b200 as F

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: flash_kda has no CPU path")
    F.lib()   # fail loudly if the CUDA library is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    binding = bind_near_gpu(local_rank, local_world)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # stdout carries the one JSON line: whatever NCCL prints while the communicator is set up (its version banner
        # goes to stdout by plain printf) is sent to stderr
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    # ---- this rank's shard ------------------------------------------------------------------------
    from flashkda_b200.sharding import plan, reduce_max_ms
    shard = plan(w, world, rank, args.shard)
    w_local, heads, tokens_global, scaling = shard.workload, shard.heads, shard.tokens_global, shard.scaling
    x = make_inputs(w_local, device=dev, heads=heads)
    H_local = x["q"].shape[2]
    B, T = x["q"].shape[:2]
    N = w.N
    ws = torch.empty(F.get_workspace_size(B * T, H_local, N, args.flags), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)
    call_ws = make_caller(flash_kda, x, ws, args.flags)               # caller-provided workspace
    call = make_caller(flash_kda, x, None, 0) if not args.flags else call_ws     # the plain drop-in call

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        call_ws()
        call()
    assert F.read_status(ws) == 0

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    t_begin = time.time()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        call()
    ev1.record(stream)
    barrier()
    t_end = time.time()
    ms = ev0.elapsed_time(ev1) / args.steps
    # The timed region lasts a few tens of milliseconds, nvidia-smi reports every 100 ms: the same calls are kept going
    # for 0.6 s more, which gives the clock record enough samples under this very load and, timed as a whole, the
    # figure for sustained operation.
    sustained = None
    if rank == 0:
        n_hold = 0
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_hold = time.time()
        h0.record(stream)
        while time.time() - t_hold < 0.6:
            for _ in range(20):
                call()
            n_hold += 20
            torch.cuda.synchronize()
        h1.record(stream)
        torch.cuda.synchronize()
        t_end = time.time()
        sustained = {"ms_per_step": h0.elapsed_time(h1) / n_hold, "calls": n_hold, "seconds": t_end - t_hold}
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "timed region and 0.6 s more of the same calls"
        sustained["sm_mhz_median"] = clocks.get("sm_mhz")
    ms_ws = time_cuda(call_ws, max(3, min(args.steps, 10)), stream)
    assert F.read_status(ws) == 0

    # ---- per-kernel durations (same stream, CUDA events), for the roofline of the dominant kernel ----
    kw = dict(initial_state=x["initial_state"], final_state=x["final_state"], cu_seqlens=x["cu_seqlens"], workspace=ws,
              flags=args.flags)
    pos = (x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["out"], x["A_log"], x["dt_bias"], x["lower_bound"])
    ksteps = max(3, min(args.steps, 10))
    # short fixed-length sequences take one fused kernel: the call is the kernel
    fused = x["cu_seqlens"] is None and 0 < T <= 32 and (args.flags & 0xFF57) == 0
    ms_prepare = 0.0 if fused else time_cuda(lambda: F.prepare(*pos, **kw), ksteps, stream)
    ms_scan = 0.0 if fused else time_cuda(lambda: F.scan(*pos, **kw), ksteps, stream)
    call_ws()                      # leave the results of a complete call in out / final_state for the checks below
    torch.cuda.synchronize()

    # ---- end to end from host buffers ----------------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        names_in = ["q", "k", "v", "g", "beta"] + (["initial_state"] if x["initial_state"] is not None else [])
        names_out = ["out"] + (["final_state"] if x["final_state"] is not None else [])
        host = {n: x[n].cpu().pin_memory() for n in names_in + names_out}
        h2d = sum(host[n].numel() * host[n].element_size() for n in names_in)
        d2h = sum(host[n].numel() * host[n].element_size() for n in names_out)

        # Fixed-length batches are fed one sequence at a time: the host->device copy of sequence b+1, the forward pass
        # of sequence b and the device->host copy of sequence b-1 run on three streams (sequences are independent, so
        # the per-sequence calls compute exactly what the batched call computes); consecutive steps are pipelined the
        # same way (a step's uploads start while the previous step's results still travel to the host), and the clock
        # stops when the last step's results are on the host.  Varlen and B = 1: one copy, one call.
        sliced = x["cu_seqlens"] is None and B > 1 and world >= 1
        e2e_mode = "per-sequence calls, copies overlapped on 2 extra streams, also across steps" if sliced else "one copy in, one call, one copy out"
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        if sliced:
            ws1 = torch.empty(F.get_workspace_size(T, H_local, 1, args.flags), dtype=torch.uint8, device=dev)
            done = [None] * B      # forward pass of sequence b issued (previous step): its inputs may be overwritten
            copied = [None] * B    # results of sequence b on their way to the host (previous step): wait before rewriting them

            def e2e_step(compute=True):
                s_in.wait_stream(stream)
                for b_ in range(B):
                    with torch.cuda.stream(s_in):
                        if done[b_] is not None:
                            s_in.wait_event(done[b_])
                        for n in names_in:
                            x[n][b_:b_ + 1].copy_(host[n][b_:b_ + 1], non_blocking=True)
                        ev_in = torch.cuda.Event()
                        ev_in.record(s_in)
                    stream.wait_event(ev_in)
                    if copied[b_] is not None:
                        stream.wait_event(copied[b_])
                    if compute:
                        flash_kda.fwd(x["q"][b_:b_ + 1], x["k"][b_:b_ + 1], x["v"][b_:b_ + 1], x["g"][b_:b_ + 1], x["beta"][b_:b_ + 1],
                                      x["scale"], x["out"][b_:b_ + 1], x["A_log"], x["dt_bias"], x["lower_bound"],
                                      initial_state=None if x["initial_state"] is None else x["initial_state"][b_:b_ + 1],
                                      final_state=None if x["final_state"] is None else x["final_state"][b_:b_ + 1],
                                      workspace=ws1, flags=args.flags)
                    done[b_] = torch.cuda.Event()
                    done[b_].record(stream)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(done[b_])
                        for n in names_out:
                            host[n][b_:b_ + 1].copy_(x[n][b_:b_ + 1], non_blocking=True)
                        copied[b_] = torch.cuda.Event()
                        copied[b_].record(s_out)

            def e2e_drain():
                stream.wait_stream(s_out)
        else:
            def e2e_step(compute=True):
                for n in names_in:
                    x[n].copy_(host[n], non_blocking=True)
                if compute:
                    call_ws()
                for n in names_out:
                    host[n].copy_(x[n], non_blocking=True)

            def e2e_drain():
                pass

        def time_e2e(compute):
            e_steps = max(2, min(args.steps, 10))
            for _ in range(2):
                e2e_step(compute)
            e2e_drain()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(e_steps):
                e2e_step(compute)
            e2e_drain()                  # the last step's results have reached the host before the clock stops
            b.record(stream)
            barrier()
            return a.elapsed_time(b) / e_steps

        ms_e2e_local = time_e2e(True)
        ms_copy_local = time_e2e(False)      # control: the same copies on the same buffers, no kernel
        e2e = (ms_e2e_local, h2d, d2h, e2e_mode, ms_copy_local)

    # ---- reduce over ranks: max time -------------------------------------------------------------------
    ms, ms_ws, ms_prepare, ms_scan, ms_e2e, ms_copy = reduce_max_ms(
        [ms, ms_ws, ms_prepare, ms_scan, e2e[0] if e2e else 0.0, e2e[4] if e2e else 0.0], world, dev)

    strong = None
    if world > 1 and not args.no_strong and args.config == 1 and not args.shape:
        strong = []
        for cfg in (1, 3):
            if baseline_workload(cfg).H % world == 0:
                strong.append(strong_scaling(F, flash_kda, cfg, world, rank, dev, stream, max(3, min(args.steps, 10)), args.flags, dist))

    # kernels per call: prepare, the recurrence (one launch, or pass 1 + map chaining + pass 2 when sequences are cut
    # into runs), plus the chunk prefix for varlen
    runs = 1
    varlen = x["cu_seqlens"] is not None
    chains = N * H_local
    per_seq_chunks = ((B * T) // N + 31) // 32 if varlen else (T + 31) // 32     # varlen: planned for the average length
    forced = (args.flags >> 8) & 0xFF
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    if not (args.flags & 0x9) and not ((args.flags & 0x2) and forced < 2):
        runs = forced if forced >= 2 else (1 if args.flags & 0x4 else F.plan_segments(chains, per_seq_chunks)[0])
    if not varlen and 0 < T <= 64 and not (args.flags & 0x4):
        runs = 1
    if chains > sms and not (args.flags & 0x7):
        runs = 1                      # more chains than SMs: the compact kernel on whole sequences
    recurrence = 1 if runs == 1 else 2 + (1 if runs > 2 else 0)
    if varlen and sms < chains <= 1024 and not (args.flags & 0x7):
        recurrence = 2                # both recurrence kernels are launched; the one not chosen on the device leaves at once
    launches_per_call = 1 + (1 if varlen else 0) + recurrence
    if fused:
        launches_per_call = 1

    if rank == 0:
        peak, peak_kind = measured_peaks()
        alg = algorithmic_bytes(B * T, H_local, N, w.state_in, w.state_out)      # per rank, per call
        # what each kernel moves of those bytes: the token-parallel kernel reads q, k, v, g, beta; the recurrence writes
        # out and moves the states (its other input, the operand records, is not algorithmic)
        alg_prepare = 1026 * B * T * H_local
        alg_scan = alg - alg_prepare
        dom_name, dom_ms, dom_alg = ("scan", ms_scan, alg_scan) if ms_scan >= ms_prepare else ("prepare", ms_prepare, alg_prepare)
        if fused:
            dom_name, dom_ms, dom_alg = "short16", ms_ws, alg
        ach = dom_alg / (dom_ms * 1e-3) / 1e9
        ach_call = alg / (ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": tokens_global / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(w, B, T, H_local, N),
            "run": {"sharding": f"{args.shard} x{world}, no data-path collective", "chunk": 32, "host_binding": binding,
                    "l2": "inputs + outputs per call (%.2f GB) larger than the 126 MB L2; no explicit flush" % (alg / 1e9),
                    "timed_call": "flash_kda.fwd with its default per-call workspace allocation" if not args.flags else "caller workspace (flags given)"},
            "gpu_launches": launches_per_call * args.steps,
            "preallocated_workspace": {"ms_per_step": ms_ws, "value": tokens_global / (ms_ws * 1e-3)},
            "sustained": sustained,
            "kernels_ms": {"short16": ms_ws} if fused else {"prepare": ms_prepare, "scan": ms_scan},
            "roofline": {"bound": "hbm", "kernel": dom_name, "achieved": ach, "peak": peak, "unit": "GB/s",
                         "frac": ach / peak, "peak_source": peak_kind, "algorithmic_bytes": dom_alg,
                         "call_algorithmic_bytes": alg,
                         "traffic": (SHORT16_TRAFFIC_BYTES_PER_CHAIN * N * H_local
                                     if fused and T == 16 and w.state_in == "fp32" and w.state_out == "fp32" else
                                     TRAFFIC_BYTES_PER_TOKEN_HEAD.get(dom_name) and
                                     TRAFFIC_BYTES_PER_TOKEN_HEAD[dom_name] * B * T * H_local)},
            "roofline_call": {"achieved": ach_call, "peak": peak, "unit": "GB/s", "frac": ach_call / peak,
                              "frac_sustained": alg / (sustained["ms_per_step"] * 1e-3) / 1e9 / peak if sustained else None},
            "clocks": clocks,
        }
        if e2e:
            line["e2e"] = {"value": tokens_global / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                           "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2], "mode": e2e[3],
                           "h2d_gbs_per_rank": e2e[1] / (ms_e2e * 1e-3) / 1e9, "d2h_gbs_per_rank": e2e[2] / (ms_e2e * 1e-3) / 1e9,
                           "copy_only_control": {"ms_per_step": ms_copy, "value": tokens_global / (ms_copy * 1e-3),
                                                 "h2d_gbs_all_ranks": world * e2e[1] / (ms_copy * 1e-3) / 1e9,
                                                 "what": "the same host<->device copies on the same buffers, no kernel"}}
        if strong:
            line["strong"] = strong
        if world == 1 and not args.no_cpu_baseline:
            import oracle
            longest = 0 if not varlen else max(range(N), key=lambda i: w.seq_lens[i])
            pairs = sorted({(longest, 0), (N // 2, H_local // 2), (N - 1, H_local - 1)})
            r = oracle.sampled_parity(x, x["out"], x["final_state"], pairs)
            line["parity"] = {"out_max_abs": r["out_max_abs"], "state_rel": r["state_rel"], "out_rmse_ratio": r["out_rmse_ratio"],
                              "chains_checked": [list(p_) for p_ in pairs], "against": "fp64 per-token recurrence (oracle)",
                              "tolerance": {"out_max_abs": 2e-2, "state_rel": 1e-2}}
            v, cores, desc = cpu_baseline_sample(w)
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc}
        if world == 1 and not args.no_reference_kernel:
            line["reference_kernel"] = reference_kernel_leg(x, w, ms, stream, max(3, min(args.steps, 10)))
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes per token-head of each kernel, from ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum per launch / token-heads of the captured case).
SHORT16_TRAFFIC_BYTES_PER_CHAIN = 140_400   # profiles/short16_kernel_B128xT16xH32.md (T = 16, fp32 state in and out), scaled by chains
# ncu dram bytes per token-head: profiles/prepare_pipe_kernel_prepare_tc4_kernel_B8xT1024xH16.md (prepare) and
# profiles/prepare_kernel_scan2_kernel_B8xT1024xH16.md (scan), scaled by token-heads
TRAFFIC_BYTES_PER_TOKEN_HEAD = {"prepare": 1774, "scan": 1313}

if __name__ == "__main__":
    main()
