"""Seeded synthetic workloads for `flash_kda.fwd`.

The reference measures and tests on synthetic random tensors only
(benchmarks/bench_fwd.py:56-66, tests/test_fwd_full.py:26-44), so these generators are the
whole data story.  Every tensor comes from one `torch.Generator` seeded per workload, drawn
in the fixed order q, k, v, g, beta, A_log, dt_bias, initial_state.  With device="cpu" the bits
are reproducible across machines (used by the parity tests); a CUDA device draws from the
CUDA generator instead (same distributions, used by the benchmark for speed).
"""
import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

D = 128


@dataclass
class Workload:
    name: str
    H: int
    B: int = 1
    T: int = 0                       # tokens per sequence (fixed-length) or total (varlen)
    seq_lens: Optional[List[int]] = None
    lower_bound: float = -5.0
    state_in: Optional[str] = None   # None | "bf16" | "fp32"
    state_out: Optional[str] = None
    state_std: float = 0.02
    seed: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def N(self) -> int:
        return len(self.seq_lens) if self.seq_lens is not None else self.B

    @property
    def total_tokens(self) -> int:
        return sum(self.seq_lens) if self.seq_lens is not None else self.B * self.T


def _dt(name):
    return {None: None, "bf16": torch.bfloat16, "fp32": torch.float32}[name]


def draw_c2_seq_lens(seed: int = 0, n: int = 16, lo: int = 256, hi: int = 16384) -> List[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=gen).tolist()


def baseline_workload(idx: int) -> Workload:
    """The five configurations the headline metric is defined on."""
    if idx == 0:
        return Workload("C0_cpu_ref_B1_T1024_H4", H=4, B=1, T=1024, state_out="fp32")
    if idx == 1:
        return Workload("C1_fixed_B4_T8192_H32", H=32, B=4, T=8192, state_in="fp32", state_out="fp32")
    if idx == 2:
        lens = draw_c2_seq_lens()
        return Workload("C2_varlen_N16_H32", H=32, B=1, T=sum(lens), seq_lens=lens,
                        state_in="bf16", state_out="bf16")
    if idx == 3:
        return Workload("C3_long_B1_T131072_H64", H=64, B=1, T=131072, lower_bound=-2.0,
                        state_in="fp32", state_out="fp32")
    if idx == 4:
        return Workload("C4_short_B512_T16_H32", H=32, B=512, T=16, state_in="fp32", state_out="fp32")
    raise ValueError(idx)


def make_inputs(w: Workload, device="cpu", heads: Optional[range] = None):
    """Returns a dict with q,k,v,g,beta,A_log,dt_bias,scale,lower_bound,initial_state,
    final_state (pre-allocated or None), out (pre-allocated), cu_seqlens (or None).

    `heads` draws only that slice of the head axis (for head-sharded multi-GPU runs); the
    per-head statistics do not depend on the slice.
    """
    dev = torch.device(device)
    gen = torch.Generator(device=dev if dev.type == "cuda" else "cpu").manual_seed(w.seed)
    H = len(heads) if heads is not None else w.H
    B, T = (1, w.total_tokens) if w.seq_lens is not None else (w.B, w.T)

    def randn(*shape, dtype=torch.float32, std=1.0):
        x = torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32)
        if std != 1.0:
            x = x * std
        return x.to(dtype)

    q = randn(B, T, H, D, dtype=torch.bfloat16)
    k = randn(B, T, H, D, dtype=torch.bfloat16)
    v = randn(B, T, H, D, dtype=torch.bfloat16)
    g = randn(B, T, H, D, dtype=torch.bfloat16)
    beta = randn(B, T, H, dtype=torch.bfloat16)
    A_log = torch.log(torch.empty(H, device=dev).uniform_(1.0, 16.0, generator=gen))
    dt_bias = randn(H, D, std=0.1)
    N = w.N
    init = None
    if w.state_in is not None:
        init = randn(N, H, D, D, dtype=_dt(w.state_in), std=w.state_std)
    fin = None
    if w.state_out is not None:
        fin = torch.empty(N, H, D, D, dtype=_dt(w.state_out), device=dev)
    cu = None
    if w.seq_lens is not None:
        cu = torch.tensor([0] + list(torch.tensor(w.seq_lens).cumsum(0).tolist()),
                          dtype=torch.int64, device=dev)
    return dict(q=q, k=k, v=v, g=g, beta=beta, A_log=A_log, dt_bias=dt_bias,
                scale=1.0 / math.sqrt(D), lower_bound=w.lower_bound, initial_state=init,
                final_state=fin, out=torch.empty_like(v), cu_seqlens=cu)


def algorithmic_bytes(total_tokens: int, H: int, N: int, state_in: Optional[str],
                      state_out: Optional[str]) -> int:
    """Bytes the operator must move: q,k,v,g read + out written (5 x 256 B) and beta read (2 B)
    per token-head, plus the recurrent state in and out per (sequence, head)."""
    sz = {None: 0, "bf16": 2, "fp32": 4}
    return 1282 * total_tokens * H + N * H * D * D * (sz[state_in] + sz[state_out])
