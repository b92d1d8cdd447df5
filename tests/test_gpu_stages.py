"""GPU: the building blocks one at a time -- tcgen05 descriptor flavours, the prologue kernel,
and the prepare kernel's operand records against the fp64 chunk operands of the oracle."""
import math

import pytest
import torch

import flashkda_b200 as F
import oracle
from flashkda_b200.workloads import Workload, make_inputs
from helpers import decode_record, to_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("reps", [1, 2])
def test_umma_descriptor_flavours(mode, reps):
    """Modes 0-2: both operands in shared memory; 3, 4: A operand read from tensor memory."""
    g = torch.Generator().manual_seed(mode)
    shape = mode - 3 if mode >= 3 else mode
    ka = 128 if shape == 0 else 32
    A = torch.randn(128, ka, generator=g).bfloat16()
    B = (torch.randn(32, 128, generator=g) if shape == 1 else torch.randn(32, ka, generator=g)).bfloat16()
    ref = A.double() @ (B.double() if shape == 1 else B.double().t())
    D = F.selftest_umma(A.cuda(), B.cuda(), mode, reps).cpu().double()
    err = (D - reps * ref).abs().max().item()
    assert err < 1e-3 * max(1.0, ref.abs().max().item()), \
        f"mode {mode} reps {reps}: max err {err}; D[0,:4]={D[0,:4].tolist()} ref[0,:4]={(reps*ref)[0,:4].tolist()}"


def test_prologue_kernel():
    w = Workload("p", H=3, B=2, T=37, seed=5)
    x = make_inputs(w)
    xc = to_cuda(x)
    qn, kn, gate, bact = F.prologue(xc["q"], xc["k"], xc["g"], xc["beta"], xc["A_log"], xc["dt_bias"], -5.0)
    torch.cuda.synchronize()
    q64, k64 = x["q"].double(), x["k"].double()
    qr = q64 * torch.rsqrt((q64 * q64).sum(-1, keepdim=True) + 1e-6)
    kr = k64 * torch.rsqrt((k64 * k64).sum(-1, keepdim=True) + 1e-6)
    gr = -5.0 * math.log2(math.e) * torch.sigmoid(
        torch.exp(x["A_log"].double()).view(1, 1, -1, 1) * (x["g"].double() + x["dt_bias"].double()))
    br = torch.sigmoid(x["beta"].double())
    assert (qn.cpu().double() - qr).abs().max() < 4e-3       # bf16 rounding of values <= 1
    assert (kn.cpu().double() - kr).abs().max() < 4e-3
    assert (gate.cpu().double() - gr).abs().max() < 8e-3     # tanh.approx: ~2^-11 relative on |g| <= 7.2
    assert (bact.cpu().double() - br).abs().max() < 1e-3


@pytest.mark.parametrize("kernel", ["mma_sync", "tcgen05_cta_per_item", "tcgen05_pipelined"])
@pytest.mark.parametrize("case", ["fixed", "varlen", "strong_decay"])
def test_prepare_records_match_fp64_operands(case, kernel):
    """Operand records of the three token-parallel kernels (the default pipelined TMA + tcgen05 one, its
    one-CTA-per-item form and the mma.sync one) against the fp64 chunk operands of the oracle."""
    flags = {"mma_sync": F.FLAG_PREPARE_MMA_SYNC, "tcgen05_cta_per_item": F.FLAG_PREPARE_TCGEN05, "tcgen05_pipelined": 0}[kernel]
    if case == "fixed":
        w = Workload("f", H=2, B=2, T=80, seed=11)
    elif case == "varlen":
        w = Workload("v", H=2, seq_lens=[17, 33, 64, 5], seed=12)
    else:
        w = Workload("s", H=2, B=1, T=64, seed=13)
    x = make_inputs(w)
    if case == "strong_decay":      # push the gate to its floor: g large, A_log large
        x["g"] = torch.full_like(x["g"], 8.0)
        x["A_log"] = torch.full_like(x["A_log"], 2.0)
    xc = to_cuda(x)
    ws = F.prepare(xc["q"], xc["k"], xc["v"], xc["g"], xc["beta"], xc["scale"], xc["out"], xc["A_log"],
                   xc["dt_bias"], xc["lower_bound"], cu_seqlens=xc["cu_seqlens"], flags=flags)
    assert F.read_status(ws) == 0
    ws = ws.cpu()
    B, T = x["q"].shape[:2]
    T_total, H, N = B * T, w.H, w.N
    rec_off, rec_bytes, per_head = F.workspace_layout(T_total, H, N, x["cu_seqlens"] is not None, T)
    lens = w.seq_lens if w.seq_lens is not None else [w.T] * w.B
    flat = {k: x[k].reshape(1, T_total, *x[k].shape[2:]).contiguous() for k in ("q", "k", "v", "g", "beta")}
    worst = {}
    gc, t_seq = 0, 0
    for L in lens:
        for t0 in range(0, L, 32):
            n = min(32, L - t0)
            for h in range(H):
                o = rec_off + (h * per_head + gc) * rec_bytes
                got = decode_record(ws[o:o + rec_bytes])
                exp = oracle.chunk_operands(flat["q"], flat["k"], flat["v"], flat["g"], flat["beta"], x["scale"],
                                            x["A_log"], x["dt_bias"], x["lower_bound"], h, t_seq + t0, n, 32)
                for key, e in (("wp", exp["wp"]), ("qp", exp["qpp"]), ("kr", exp["kr"]), ("up", exp["up"]),
                               ("mqk", exp["mqk"]), ("ec", exp["ec"])):
                    err = (got[key] - e).abs().max().item() / max(e.abs().max().item(), 1e-3)
                    worst[key] = max(worst.get(key, 0.0), err)
            gc += 1
        t_seq += L
    print("prepare", case, kernel, {k: f"{v:.2e}" for k, v in worst.items()})
    # bf16 operands: relative to the tile's largest entry; products of bf16-rounded factors ~1e-2.  qp and kr are built
    # with packed bf16 multiplies (two and three roundings of 2^-9 each).
    assert worst["qp"] < 8e-3 and worst["kr"] < 1.2e-2 and worst["ec"] < 2e-3, worst
    assert worst["mqk"] < 2e-2 and worst["wp"] < 3e-2 and worst["up"] < 3e-2, worst


@pytest.mark.parametrize("case", ["fixed_many_iterations", "varlen_many_sequences", "tails"])
def test_pipelined_kernel_writes_the_records_of_the_cta_per_item_kernel_bit_for_bit(case):
    """The pipelined token-parallel kernel reuses two operand buffers, two accumulators and its barriers over many
    items per CTA; the one-CTA-per-item kernel does the same arithmetic with nothing reused.  Their operand records
    must be the same bytes: a stale tile, a buffer overwritten too early or a lost phase would show here, on shapes
    with up to 74 items per CTA, ragged sequences and repeated calls."""
    if case == "fixed_many_iterations":
        w = Workload("p1", H=32, B=4, T=8192, seed=21)
    elif case == "varlen_many_sequences":
        import random
        rnd = random.Random(5)
        w = Workload("p2", H=8, seq_lens=[rnd.choice([0, 1, 7, 31, 32, 33, 63, 64, 65, 100, 257, 1000]) for _ in range(300)], seed=22)
    else:
        w = Workload("p3", H=5, B=7, T=32 * 40 + 3, seed=23)
    x = make_inputs(w, device="cuda")
    args = (x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["out"], x["A_log"], x["dt_bias"], x["lower_bound"])
    B, T = x["q"].shape[:2]
    size = F.get_workspace_size(B * T, w.H, w.N)

    def records(flags):      # (zero-filled first: what a kernel does not write compares equal)
        ws = torch.zeros(size, dtype=torch.uint8, device="cuda")
        F.prepare(*args, cu_seqlens=x["cu_seqlens"], workspace=ws, flags=flags)
        assert F.read_status(ws) == 0
        return ws[256:]

    ref = records(F.FLAG_PREPARE_TCGEN05)
    assert int(ref.count_nonzero()) > size // 2
    for _ in range(3):
        assert torch.equal(records(0), ref)


def test_tmem_16_lane_fragment_shapes():
    """tcgen05.ld/st with the 16-lane shapes (16x256b.x8, 16x128b.x8) follow the mma accumulator fragment map that
    the helpers in csrc/fkda_common.cuh document: thread t, register 4j+q <-> lane t/4 + 8(q/2), column 8j + 2(t%4) + q%2."""
    import numpy as np
    o = F.tmem_layout_probe().numpy().astype(np.int64) & 0xFFFFFFFF
    ld = o[0].reshape(2, 32, 32)
    t = np.arange(32)[:, None]
    r = np.arange(32)[None, :]
    lane = t // 4 + 8 * ((r % 4) // 2)
    col = 8 * (r // 4) + 2 * (t % 4) + (r % 2)
    for half in range(2):
        assert np.array_equal(ld[half], ((lane + 16 * half) << 8) | col)
    st = o[2].reshape(32, 64)
    exp = np.full((32, 64), 0xFFFFFFFF, dtype=np.int64)
    exp[lane, col] = (1 << 16) | (t << 8) | r
    assert np.array_equal(st, exp)
    s3 = o[3].reshape(32, 64)[:, :32]
    r16 = np.arange(16)[None, :]
    exp3 = np.full((32, 32), 0xFFFFFFFF, dtype=np.int64)
    exp3[16 + t // 4 + 8 * (r16 % 2), 4 * (r16 // 2) + t % 4] = (2 << 16) | (t << 8) | r16
    assert np.array_equal(s3, exp3)


def test_umma_bench_runs_inside_its_operand_arrays():
    """The tcgen05.mma micro-benchmark (tuning aid, builds made with -DFKDA_TUNING only) completes for every shape it
    accepts; accumulating instructions of one thread are serialised by the accumulator (over 100 cycles each), those
    of several threads overlap."""
    if not hasattr(F.lib(), "fkda_debug_umma_bench"):
        pytest.skip("library built without -DFKDA_TUNING")
    one = F.umma_bench(issuers=1, reps=16, ksteps=8, n=128, a_in_tmem=False)
    four = F.umma_bench(issuers=4, reps=16, ksteps=8, n=32, a_in_tmem=True)
    assert one[1] > 60 and four[1] > 60
    assert F.umma_bench(issuers=2, reps=8, ksteps=2, n=64, a_in_tmem=True)[1] > 0


@pytest.mark.parametrize("N", [1, 5, 300, 4096])
def test_chunk_prefix_and_chain_order(N):
    """The scheduling kernel of varlen calls: chunk prefix sums and the order in which the recurrence takes the
    sequences (longest first, ties in the given order), read back from the workspace header."""
    import flashkda_b200 as F
    from flashkda_b200.workloads import Workload, make_inputs
    g = torch.Generator().manual_seed(N)
    lens = [int(v) for v in torch.randint(0, 200 if N < 1000 else 40, (N,), generator=g)]
    if N >= 5:
        lens[3] = 0
    w = Workload("order", H=1, seq_lens=lens, seed=N)
    x = make_inputs(w, device="cuda")
    ws = F.prepare(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["out"], x["A_log"], x["dt_bias"], x["lower_bound"],
                   cu_seqlens=x["cu_seqlens"])
    assert F.read_status(ws) == 0
    head = ws[256:256 + 4 * (2 * N + 1)].view(torch.int32).cpu()
    chunks = torch.tensor([(v + 31) // 32 for v in lens], dtype=torch.int64)
    assert torch.equal(head[:N + 1].long(), torch.cat([torch.zeros(1, dtype=torch.int64), chunks.cumsum(0)]))
    want = sorted(range(N), key=lambda i: (-int(chunks[i]), i))
    assert head[N + 1:].tolist() == want
