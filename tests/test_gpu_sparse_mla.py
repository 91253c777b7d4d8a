"""Sparse MLA decode attention (BASELINE config 2) through the C ABI against the oracle."""

import pytest
import torch

from oracle import stages as S
import synth
from util import assert_close_hidden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCALE = 192**-0.5


def _run(rows, heads, ctx, topk, seed=0, edit=None):
    from sgl_amd_mono_b200.attention import SparseMlaOp

    q, pages, sel, _ = synth.sparse_mla_inputs(rows, heads, ctx, topk, seed=seed)
    if edit:
        edit(q, pages, sel)
    op = SparseMlaOp(heads, topk, DEV, sm_scale=SCALE)
    out = op(q.to(DEV), pages.to(DEV), sel.to(DEV)).clone()
    torch.cuda.synchronize()
    return q, pages, sel, out, op


@pytest.mark.parametrize("rows,heads,ctx,topk", [(1, 16, 4096, 2048), (4, 16, 4096, 2048), (8, 16, 2100, 2048),
                                                 (2, 8, 300, 256), (3, 40, 1000, 512), (2, 128, 700, 320)])
def test_matches_oracle(rows, heads, ctx, topk):
    q, pages, sel, out, _ = _run(rows, heads, ctx, topk)
    ref = S.sparse_mla(q, pages, sel, SCALE)
    assert_close_hidden(out, ref, f"rows={rows} heads={heads} ctx={ctx} topk={topk}")


def test_short_ragged_and_invalid_entries():
    def edit(q, pages, sel):
        sel[0, 5] = -1  # an invalid entry mid-list is masked
        sel[1, 100:] = -1  # a short row
        sel[2, :] = -1  # an empty row (pad): reads nothing, returns zeros

    q, pages, sel, out, _ = _run(3, 16, 500, 256, seed=3, edit=edit)
    ref = S.sparse_mla(q, pages, sel, SCALE)
    assert_close_hidden(out, ref, "ragged")
    assert float(out[2].float().abs().max()) == 0.0


def test_replay_and_negative_control():
    q, pages, sel, out, op = _run(4, 16, 2048, 1024, seed=4)
    qd, pd, sd = q.to(DEV), pages.to(DEV), sel.to(DEV)
    for _ in range(3):
        assert torch.equal(op(qd, pd, sd), out)
    sd2 = sd.clone()
    sd2[0, 0] = sd[0, 1]
    assert not torch.equal(op(qd, pd, sd2)[0], out[0])


def test_full_size_config2_property():
    """Context 32768, 8 rows: softmax weights sum to one, so with every cached latent of a
    row's selection replaced by one constant row the output must equal that row's latent."""
    q, pages, sel, _ = synth.sparse_mla_inputs(8, 16, 32768, 2048, seed=5)
    from sgl_amd_mono_b200.attention import SparseMlaOp

    pages = pages.to(DEV)
    const = pages[1, 7 * 576 : 8 * 576].clone()
    pages[:, : 64 * 576] = const.repeat(64)
    pages[:, 64 * 576 :].view(torch.float32)[:] = 0.25
    op = SparseMlaOp(16, 2048, DEV, sm_scale=SCALE)
    out = op(q.to(DEV), pages, sel.to(DEV))
    want = (const[:512].view(torch.float8_e4m3fn).float() * 0.25).bfloat16().float()
    assert torch.allclose(out.float(), want.expand_as(out), atol=2e-2, rtol=2**-7)


@pytest.mark.parametrize("fmt_name", ["A8", "MX8N"])
def test_merge_stages_the_heads_for_the_next_gemv(fmt_name):
    """The merge can also write every head's output as that head's quantised activation set: same bf16
    output, and the planes and scales of a staging launch run on that output, bit for bit."""
    from sgl_amd_mono_b200 import _lib as L
    from sgl_amd_mono_b200 import ops

    rows, heads = 5, 16
    q, pages, sel, out, op = _run(rows, heads, 3000, 512, seed=6)
    fmt = getattr(L, "ACT_" + fmt_name)
    staged = ops.ActBuf(fmt, 512, DEV, segs=heads)
    ref = ops.ActBuf(fmt, 512, DEV, segs=heads)
    out2 = op(q.to(DEV), pages.to(DEV), sel.to(DEV), staged=staged).clone()
    ops.act_prep_heads(rows, heads, 512, ref, src_bf16=out2)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    assert torch.equal(staged.planes, ref.planes) and bool(ref.planes.any())
    for name in ("scale_f32", "scale_e8"):
        a, b = getattr(staged, name), getattr(ref, name)
        assert (a is None) == (b is None)
        if a is not None:
            assert torch.equal(a, b) and bool(b.any())


@pytest.mark.parametrize("rows,heads,ctx,topk", [(2, 128, 700, 320), (8, 128, 16384, 2048), (3, 64, 5000, 2048),
                                                 (1, 96, 300, 256), (6, 64, 8192, 8192)])
def test_tcgen05_split_matches_oracle_and_the_warp_mma_split(rows, heads, ctx, topk, monkeypatch):
    """From 64 local heads the split runs on tcgen05 with every head of a row in one task (cache rows kept as
    E4M3, queries and probabilities as exact hi / lo E4M3 planes).  Same tolerance against the oracle as the
    warp-MMA split, and the two splits agree to a few bf16 ulps of the largest output."""
    def edit(q, pages, sel):
        sel[0, 7] = -1  # an invalid entry mid-list
        if rows > 1:
            sel[1, topk // 3:] = -1  # a short row: whole chunks without a key

    monkeypatch.setenv("MONO_MLA_TC", "1")
    q, pages, sel, out_tc, _ = _run(rows, heads, ctx, topk, seed=7, edit=edit)
    monkeypatch.setenv("MONO_MLA_TC", "0")
    _, _, _, out_mma, _ = _run(rows, heads, ctx, topk, seed=7, edit=edit)
    ref = S.sparse_mla(q, pages, sel, SCALE)
    print("tcgen05:", assert_close_hidden(out_tc, ref, "tcgen05 split"), "warp MMA:", assert_close_hidden(out_mma, ref, "warp-MMA split"))
    d = float((out_tc.float() - out_mma.float()).abs().max())
    assert d <= 2.0**-6 * float(ref.float().abs().max()) + 1e-3, f"the two splits differ by {d}"
