"""The allocation-free sparse MLA entry point (``mono_sparse_mla_launch_noalloc``).

Some callers of this library cannot allocate device memory: a serving process gives
whatever the model leaves free to its KV-cache pool, so code that attaches or runs
afterwards has no safe way to obtain a scratch buffer.  For them the library carries a
small fixed scratch array of its own.  This test calls that entry point through the
C ABI, twice in a row on different inputs (the array keeps the previous call's
partials, so the second call proves nothing stale leaks through), and compares each
result with the regular entry point, which uses a caller-provided scratch buffer.
Both run the same kernels, so the outputs must be identical; the comparison still uses
the hidden-state tolerance of the other parity tests as its stated bound.

The file name sorts last so that a run stopping at the first failure has already
executed every other test.
"""

import ctypes as C

import pytest
import torch

from sgl_amd_mono_b200 import _lib as L
import synth
from util import assert_close_hidden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCALE = 192**-0.5


def _args(q, pages, sel, out, scratch, topk):
    a = L.SparseMlaArgs()
    a.rows, a.heads, a.topk, a.topk_ld, a.sm_scale = q.shape[0], q.shape[1], topk, sel.shape[1], SCALE
    a.q, a.kv_pages, a.n_pages = q.data_ptr(), pages.data_ptr(), pages.shape[0]
    a.topk_slots, a.out = sel.data_ptr(), out.data_ptr()
    a.scratch = None if scratch is None else scratch.data_ptr()
    return a


def _both(lib, rows, heads, ctx, topk, seed):
    q, pages, sel, _ = synth.sparse_mla_inputs(rows, heads, ctx, topk, device=DEV, seed=seed)
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.full((rows, heads, 512), float("nan"), dtype=torch.bfloat16, device=DEV)
    scratch = torch.zeros(lib.mono_sparse_mla_scratch_bytes(rows, heads, topk), dtype=torch.uint8, device=DEV)
    L.check(lib.mono_sparse_mla_launch(C.byref(_args(q, pages, sel, want, scratch, topk)), stream), "regular entry point")
    got = torch.full_like(want, float("nan"))
    L.check(lib.mono_sparse_mla_launch_noalloc(C.byref(_args(q, pages, sel, got, None, topk)), stream), "no-alloc entry point")
    torch.cuda.synchronize()
    return got, want


def test_two_calls_in_a_row_match_the_regular_entry_point():
    lib = L.load()
    # first call: the largest shape the built-in scratch serves
    got, want = _both(lib, 8, 16, 4096, 2048, seed=21)
    assert_close_hidden(got, want, "no-alloc call 1")
    assert torch.equal(got, want)
    # second call, smaller and on other data: partials of call 1 are still in the array
    got2, want2 = _both(lib, 3, 8, 700, 320, seed=22)
    assert_close_hidden(got2, want2, "no-alloc call 2")
    assert torch.equal(got2, want2)


def test_shapes_beyond_the_built_in_scratch_are_refused():
    lib = L.load()
    q, pages, sel, _ = synth.sparse_mla_inputs(2, 32, 512, 256, device=DEV, seed=23)
    out = torch.zeros(2, 32, 512, dtype=torch.bfloat16, device=DEV)
    rc = lib.mono_sparse_mla_launch_noalloc(C.byref(_args(q, pages, sel, out, None, 256)), None)
    assert rc == -1
    assert b"exceeds the built-in scratch" in lib.mono_last_error()
