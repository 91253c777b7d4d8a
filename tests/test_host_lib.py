"""CPU-side checks of the C-ABI library and the host logic: it builds, loads, exports
every symbol the header declares, mirrors the struct layouts, and rejects bad
arguments before touching a device."""

import ctypes as C
import re
from pathlib import Path

import pytest

from sgl_amd_mono_b200 import _lib as L
from sgl_amd_mono_b200 import ops
from sgl_amd_mono_b200.build import build_library

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build_library()
    return L.load()


def test_exports_every_declared_symbol(lib):
    header = (ROOT / "include" / "mono_b200.h").read_text()
    declared = set(re.findall(r"\b(mono_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(L.SYMBOLS), f"binding and header differ: {declared ^ set(L.SYMBOLS)}"


def test_abi_version_and_struct_mirrors(lib):
    assert lib.mono_abi_version() == 1
    for i, st in enumerate(L._STRUCTS):
        assert lib.mono_struct_size(i) == C.sizeof(st), st.__name__
    assert L.GemvArgs.job.offset % 64 == 0


def test_bad_arguments_are_refused_with_a_message(lib):
    a = L.GemvArgs()
    a.njobs, a.rows = 0, 4
    assert lib.mono_gemv_launch(C.byref(a), None) == -1
    assert b"njobs" in lib.mono_last_error()
    s = L.SparseMlaArgs()
    s.rows = 99
    assert lib.mono_sparse_mla_launch(C.byref(s), None) == -1
    r = L.ReduceArgs()
    r.rows, r.n = 2, 7
    assert lib.mono_reduce_launch(C.byref(r), None) == -1
    t = L.Tmap()
    assert lib.mono_tmap_encode(C.byref(t), 8, 100, 4, 1, 100, 400) == -1  # unaligned base / stride
    assert b"multiples of 16" in lib.mono_last_error()


def test_scratch_and_peer_sizes(lib):
    assert lib.mono_sparse_mla_scratch_bytes(8, 16, 2048) >= 8 * 32 * 16 * (1024 + 8)
    assert lib.mono_reduce_peer_bytes(8, 7168, 8) == 2 * 8 * 16 * 3584 * 8


@pytest.mark.parametrize("k_tiles,rbs,wk", [(56, 17, L.W_FP8), (12, 192, L.W_FP8), (4, 16, L.W_FP8),
                                            (128, 56, L.W_FP8), (8, 768, L.W_MXFP4), (3, 16, L.W_MXFP4),
                                            (64, 1010, L.W_BF16), (2, 56, L.W_FP8)])
def test_plan_split_covers_k_in_whole_groups(k_tiles, rbs, wk):
    split, n = ops.plan_split(k_tiles, rbs, wk)
    assert split * n >= k_tiles > split * (n - 1)
    # FP8 segments may span 32 tiles on the tcgen05 consumer (the default), 16 on the warp-MMA one
    assert split <= (32 if wk == L.W_FP8 else ops._MAX_SEG_TILES[wk])
    if n > 1:
        assert split % 4 == 0


def test_runner_refuses_cpu_tensors():
    import torch

    with pytest.raises(ValueError, match="CUDA"):
        ops.require(torch.zeros(2, 4), "x")
