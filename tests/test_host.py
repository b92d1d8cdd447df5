"""CPU-only checks of the host side: the C-ABI library loads and exports what include/fkda.h
declares, sizes are sane, and argument errors surface as RuntimeError before any launch."""
import ctypes
import math
import os
import re

import pytest
import torch

import flash_kda
import flashkda_b200 as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    """Every function the two headers declare (the part of the test-support header that only tuning builds have
    left out)."""
    names = set()
    for header in ("fkda.h", "fkda_testing.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"#ifdef FKDA_TUNING.*?#endif", "", text, flags=re.S)
        names |= set(re.findall(r"\b(fkda_[a-z_0-9]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert "fkda_fwd" in names and "fkda_get_workspace_size" in names and len(names) >= 8
    L = ctypes.CDLL(F.lib_path())
    for n in names:
        assert hasattr(L, n), f"libfkda.so does not export {n}"


def test_params_struct_matches_header_field_order():
    text = open(os.path.join(ROOT, "include", "fkda.h")).read()
    body = text[text.index("typedef struct fkda_fwd_params {"):text.index("} fkda_fwd_params;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b([A-Za-z_]+);", body)
    from flashkda_b200._binding import FwdParams
    assert fields == [f[0] for f in FwdParams._fields_]


def test_workspace_size():
    a = F.get_workspace_size(32768, 32, 4)
    assert a == 256 + 256 + (32768 // 32 + 4) * 32 * 35328
    assert F.get_workspace_size(0, 1, 1) > 0
    assert F.get_workspace_size(64, 2, 1) < F.get_workspace_size(128, 2, 1)
    with pytest.raises(RuntimeError):
        F.get_workspace_size(16, 0, 1)
    off, rec, per_head = F.workspace_layout(8192 * 4, 32, 4, 0, 8192)
    assert rec == 35328 and per_head == 4 * 256 and off % 256 == 0
    off, rec, per_head = F.workspace_layout(100, 2, 3, 1, 0)
    assert per_head == 100 // 32 + 3


def test_drop_in_module_surface():
    import inspect
    sig = inspect.signature(flash_kda.fwd)
    names = list(sig.parameters)
    assert names[:13] == ["q", "k", "v", "g", "beta", "scale", "out", "A_log", "dt_bias", "lower_bound",
                          "initial_state", "final_state", "cu_seqlens"]
    for n in ("initial_state", "final_state", "cu_seqlens"):
        assert sig.parameters[n].default is None
    assert callable(flash_kda.get_workspace_size)


def _cpu_args(B=1, T=16, H=2):
    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt)
    return dict(q=z(B, T, H, 128), k=z(B, T, H, 128), v=z(B, T, H, 128), g=z(B, T, H, 128), beta=z(B, T, H),
                scale=1 / math.sqrt(128), out=z(B, T, H, 128), A_log=z(H, dt=torch.float32),
                dt_bias=z(H, 128, dt=torch.float32), lower_bound=-5.0)


def test_cpu_tensors_are_rejected_not_computed():
    # no CPU path: the product must refuse, not fall back
    with pytest.raises(RuntimeError, match="CUDA"):
        flash_kda.fwd(**_cpu_args())


def test_c_abi_rejects_bad_params_without_a_gpu():
    from flashkda_b200._binding import FwdParams
    L = F.lib()
    p = FwdParams()
    assert L.fkda_fwd(ctypes.byref(p), None) == -1 and "non-NULL" in F.last_error()
    assert L.fkda_fwd(None, None) == -1
    # plausible pointers but inconsistent sizes: still rejected before any CUDA call
    p = FwdParams(*([0x1000] * 8), None, None, 0x2000, 0x3000, 1 << 40, 2, 16, 2, 2, 0.1, -5.0, 0, 0)
    assert L.fkda_fwd(ctypes.byref(p), None) == -1 and "B must be 1" in F.last_error()
    p = FwdParams(*([0x1000] * 8), None, None, None, 0x3000, 1 << 40, 2, 16, 2, 3, 0.1, -5.0, 0, 0)
    assert L.fkda_fwd(ctypes.byref(p), None) == -1 and "N must equal B" in F.last_error()
    p = FwdParams(*([0x1000] * 8), None, None, None, 0x3000, 1 << 40, 2, 16, 2, 2, 0.1, -7.0, 0, 0)
    assert L.fkda_fwd(ctypes.byref(p), None) == -1 and "lower_bound" in F.last_error()
    p = FwdParams(*([0x1000] * 8), 0x5000, None, None, 0x3000, 1 << 40, 2, 16, 2, 2, 0.1, -5.0, 0, 0)
    assert L.fkda_fwd(ctypes.byref(p), None) == -1 and "state_dtype" in F.last_error()
    p = FwdParams(*([0x1000] * 8), None, None, None, 0x3000, 1024, 2, 16, 2, 2, 0.1, -5.0, 0, 0)
    assert L.fkda_fwd(ctypes.byref(p), None) == -2 and "workspace" in F.last_error()
    p = FwdParams(0x1001, *([0x1000] * 7), None, None, None, 0x3000, 1 << 40, 2, 16, 2, 2, 0.1, -5.0, 0, 0)
    assert L.fkda_fwd(ctypes.byref(p), None) == -1 and "aligned" in F.last_error()


def test_segment_planner_is_consistent_with_the_workspace_size():
    """Few long chains are cut into runs; many chains or short sequences are not.  The last run is never empty and
    the workspace grows by three fp32 slots of 128 x 136 floats per (chain, run)."""
    import flashkda_b200 as F
    assert F.plan_segments(128, 256) == (1, 0)          # one chain per SM already
    assert F.plan_segments(8, 16) == (1, 0)             # too short to be worth it
    for chains, chunks in [(8, 4096), (16, 256), (1, 4096), (4, 129), (36, 1000)]:
        runs, per = F.plan_segments(chains, chunks)
        assert runs >= 3 and per * runs >= chunks and (runs - 1) * per < chunks, (chains, chunks, runs, per)
        H, N, T = chains, 1, chunks * 32
        grown = F.get_workspace_size(T, H, N) - F.get_workspace_size(T, H, N, F.FLAG_SCAN_NO_SEGMENTS)
        assert grown == chains * runs * 3 * 128 * 136 * 4
    # a forced run count sizes the workspace the same way
    assert (F.get_workspace_size(32 * 20, 2, 1, F.FLAG_SEGMENTS(4)) - F.get_workspace_size(32 * 20, 2, 1, F.FLAG_SCAN_NO_SEGMENTS)
            == 2 * 4 * 3 * 128 * 136 * 4)


def test_flag_constants_match_the_header():
    text = open(os.path.join(ROOT, "include", "fkda.h")).read()
    values = {m.group(1): int(m.group(2), 16) for m in re.finditer(r"#define\s+(FKDA_FLAG_\w+)\s+(0x[0-9a-fA-F]+)u", text)}
    assert values["FKDA_FLAG_SCAN_SIMT"] == F.FLAG_SCAN_SIMT
    assert values["FKDA_FLAG_SCAN_PLAIN"] == F.FLAG_SCAN_PLAIN
    assert values["FKDA_FLAG_SCAN_LOOKAHEAD"] == F.FLAG_SCAN_LOOKAHEAD
    assert values["FKDA_FLAG_SCAN_NO_SEGMENTS"] == F.FLAG_SCAN_NO_SEGMENTS
    assert values["FKDA_FLAG_NO_FUSED_SHORT"] == F.FLAG_NO_FUSED_SHORT
    assert values["FKDA_FLAG_REFERENCE_ROUNDING"] == F.FLAG_REFERENCE_ROUNDING
    assert values["FKDA_FLAG_FUSED_ANY_T"] == F.FLAG_FUSED_ANY_T
    assert values["FKDA_FLAG_PREPARE_TCGEN05"] == F.FLAG_PREPARE_TCGEN05
    assert values["FKDA_FLAG_PREPARE_MMA_SYNC"] == F.FLAG_PREPARE_MMA_SYNC
    assert F.FLAG_SEGMENTS(5) == 5 << 8 and "FKDA_FLAG_SEGMENTS(n)" in text


def test_new_entry_points_reject_bad_arguments_without_a_gpu():
    L = ctypes.CDLL(F.lib_path())
    i64, ci = ctypes.c_int64, ctypes.c_int
    L.fkda_get_workspace_size_flags.argtypes = [i64, i64, i64, i64, ctypes.POINTER(i64)]
    L.fkda_plan_segments.argtypes = [i64, i64, ctypes.POINTER(ci), ctypes.POINTER(ci)]
    L.fkda_last_error.restype = ctypes.c_char_p
    out = i64(0)
    assert L.fkda_get_workspace_size_flags(1024, 4, 1, 0, None) < 0
    assert L.fkda_get_workspace_size_flags(-1, 4, 1, 0, ctypes.byref(out)) < 0 and L.fkda_last_error()
    assert L.fkda_get_workspace_size_flags(1024, 0, 1, 0, ctypes.byref(out)) < 0
    assert L.fkda_plan_segments(8, 4096, None, None) < 0
    a, b = ci(0), ci(0)
    assert L.fkda_plan_segments(0, 4096, ctypes.byref(a), ctypes.byref(b)) == 0 and a.value == 1 and b.value == 0
    # kernel-selection flags that exclude the segment-parallel walk must not reserve room for it
    base = F.get_workspace_size(32 * 4096, 8, 1, F.FLAG_SCAN_NO_SEGMENTS)
    assert F.get_workspace_size(32 * 4096, 8, 1, F.FLAG_SCAN_PLAIN) == base
    assert F.get_workspace_size(32 * 4096, 8, 1, F.FLAG_SCAN_LOOKAHEAD) == base
    assert F.get_workspace_size(32 * 4096, 8, 1) > base


def test_segment_planner_invariants_over_a_grid_of_sizes():
    """Whatever the planner decides, the runs tile the sequence: none is empty, none shorter than eight chunks, at most
    160 of them (the flag field holds 255); batches of fifty chains or more and sequences below 48 chunks are left whole."""
    for chains in list(range(1, 50)) + [50, 64, 148, 149, 1000]:
        for chunks in (1, 47, 48, 49, 100, 129, 256, 1000, 4096, 4097, 32768, 40000):
            runs, per = F.plan_segments(chains, chunks)
            if chains >= 50 or chunks < 48:
                assert (runs, per) == (1, 0), (chains, chunks, runs, per)
                continue
            assert runs == 1 and per == 0 or (3 <= runs <= 160 and per >= 8 and runs * per >= chunks and (runs - 1) * per < chunks), \
                (chains, chunks, runs, per)
