"""B200-native Kimi Delta Attention prefill, behind the reference's `flash_kda.fwd` signature.

Python host side of the drop-in boundary: mirrors flash_kda/__init__.py:5-41 and the argument
checks of csrc/flash_kda.cpp:44-174 of the reference, then calls the C-ABI library
(include/fkda.h) through ctypes with raw device pointers and torch's current CUDA stream.
There is no CPU or PyTorch fallback: without the compiled library, or without a CUDA device,
`fwd` raises.
"""
from ._binding import (FLAG_FUSED_ANY_T, FLAG_PREPARE_MMA_SYNC, FLAG_PREPARE_TCGEN05, FLAG_NO_FUSED_SHORT, FLAG_REFERENCE_ROUNDING, FLAG_SCAN_LOOKAHEAD, FLAG_SCAN_NO_SEGMENTS, FLAG_SCAN_PLAIN, FLAG_SCAN_SIMT, FLAG_SEGMENTS, fwd, get_workspace_size, last_error, lib, lib_path,
                       plan_segments, prepare, prologue, read_status, scan, scan_giveup, prepare_giveup, selftest_umma, tmem_layout_probe, umma_bench, workspace_layout)

__all__ = ["fwd", "get_workspace_size", "prepare", "scan", "prologue", "read_status",
           "workspace_layout", "selftest_umma", "lib", "lib_path", "last_error", "FLAG_SCAN_SIMT", "FLAG_SCAN_PLAIN", "FLAG_SCAN_LOOKAHEAD",
           "FLAG_SCAN_NO_SEGMENTS", "FLAG_NO_FUSED_SHORT", "FLAG_REFERENCE_ROUNDING", "FLAG_SEGMENTS", "plan_segments", "tmem_layout_probe", "umma_bench", "scan_giveup", "prepare_giveup", "FLAG_FUSED_ANY_T", "FLAG_PREPARE_TCGEN05", "FLAG_PREPARE_MMA_SYNC"]
