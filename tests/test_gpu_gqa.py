"""GQA block-sparse attention on the GPU through the C ABI against the CPU oracle
(BASELINE config 4's attention path at small sizes)."""

import pytest
import torch

from oracle import gqa as OG
from oracle import quant as Q
from sgl_amd_mono_b200 import _lib as L
import synth
from sgl_amd_mono_b200 import ops
from sgl_amd_mono_b200.gqa import BLOCK, CFG_GQA_TINY, TOPK_BLOCKS, GqaAttentionOp
from util import assert_close_hidden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(rows, ctx, seed=0, pad=()):
    cfg = CFG_GQA_TINY
    w = synth.gqa_weights(cfg, 0, DEV)
    t = synth.gqa_step(cfg, rows, ctx, DEV)
    for r in pad:
        t.slots[r] = -1
    before = (t.k_cache.clone(), t.v_cache.clone(), t.index_cache.clone())
    x = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(seed)).bfloat16().to(DEV)
    op = GqaAttentionOp(cfg, w, DEV, max_ctx=ctx)
    out = op.launch(x, t).clone()
    torch.cuda.synchronize()
    rc, words = ops.guard_read(op.guard)
    assert rc == 0, f"guard words {words}"
    return cfg, w, t, x, op, out, before


def _head_rows(cfg, op, rows):
    """The projection's summed f32 rows as the kernel saw them: [rows, heads, 128]."""
    qkv = op.qkv[:, :rows].sum(0) if op.ns_qkv == 1 else None
    if qkv is None:  # the kernel adds the K splits in order
        qkv = torch.zeros_like(op.qkv[0, :rows])
        for s in range(op.ns_qkv):
            qkv = qkv + op.qkv[s, :rows]
    return qkv.cpu().reshape(rows, -1, 128)


@pytest.mark.parametrize("rows,ctx", [(1, 700), (4, 2100), (3, 64 * 16 + 5), (2, 300)])
def test_front_scores_selection_and_attention(rows, ctx):
    cfg, w, t, x, op, out, before = _run(rows, ctx)
    core = op.core
    heads = _head_rows(cfg, op, rows)
    nq, nk = cfg.q_local, cfg.kv_local
    cos, sin = t.cos.cpu(), t.sin.cpu()
    kc, vc, ic = t.k_cache.cpu(), t.v_cache.cpu(), t.index_cache.cpu()
    for r in range(rows):
        pos, slot = int(t.positions[r]), int(t.slots[r])
        c, s = cos[pos], sin[pos]
        # ---- front: q / index q values and the inserted cache bytes are bit-exact given the sums
        for h in range(nq):
            want = OG.head_norm_rope(heads[r, h], w["g_q"].cpu(), c, s, cfg.eps)
            assert torch.equal(core.q[r, h].cpu().float(), want), f"q head {h} of row {r}"
        want_iq = OG.head_norm_rope(heads[r, nq + 2 * nk], w["g_iq"].cpu(), c, s, cfg.eps)
        assert torch.equal(core.iq[r].cpu().float(), want_iq)
        page, off = slot // BLOCK, slot % BLOCK
        for h in range(nk):
            kn = OG.head_norm_rope(heads[r, nq + h], w["g_k"].cpu(), c, s, cfg.eps)
            assert torch.equal(kc[page, off, h], OG.fp8_scaled_bytes(kn, w["k_scale"])), "K cache bytes"
            assert torch.equal(vc[page, off, h], OG.fp8_scaled_bytes(Q.bf(heads[r, nq + nk + h]), w["v_scale"])), "V cache bytes"
        ikn = OG.head_norm_rope(heads[r, nq + 2 * nk + 1], w["g_ik"].cpu(), c, s, cfg.eps)
        assert torch.equal(ic[page, off], Q.e4m3_bytes(ikn)), "index cache bytes"
        # ---- scores against the oracle's, selection bit-exact given the kernel's own scores
        seq = pos + 1
        n_blk = -(-seq // BLOCK)
        pt = t.page_table[r].cpu().long()
        keys = Q.e4m3_from_bytes(ic[pt[:n_blk]].reshape(-1, 128))
        sc_ref = OG.block_scores(want_iq, keys, seq, cfg.sm_scale)
        sc = core.scores[r, :n_blk].cpu()
        assert torch.allclose(sc, sc_ref, rtol=1e-4, atol=1e-3)
        blocks, n_ctx = OG.select_blocks(sc, seq, cfg.init_blocks, cfg.local_blocks)
        got = core.sel_blocks[r].cpu().tolist()
        assert got[: len(blocks)] == blocks and all(b == -1 for b in got[len(blocks):])
        assert int(core.n_ctx[r]) == n_ctx
        assert core.sel_pages[r, : len(blocks)].cpu().tolist() == pt[blocks].tolist()
        # ---- attention over the selected keys
        for h in range(nk):
            G = nq // nk
            kk = Q.e4m3_from_bytes(kc[pt[blocks], :, h].reshape(-1, 128))
            vv = Q.e4m3_from_bytes(vc[pt[blocks], :, h].reshape(-1, 128))
            qh = core.q[r, h * G : (h + 1) * G].cpu().float()
            want = OG.sparse_attention_row(qh, kk, vv, w["k_scale"], w["v_scale"], n_ctx, cfg.sm_scale)
            got_o = core.out[r].cpu().float().reshape(nq, 128)[h * G : (h + 1) * G]
            assert_close_hidden(got_o, want, f"attention row {r} kv head {h}", scale=float(want.abs().max()))
    # caches are untouched except at the inserted slots
    for cache, old in zip((t.k_cache, t.v_cache, t.index_cache), before):
        mask = torch.ones(cache.shape[0] * BLOCK, dtype=torch.bool, device=DEV)
        mask[t.slots[:rows]] = False
        assert torch.equal(cache.reshape(mask.numel(), -1)[mask], old.reshape(mask.numel(), -1)[mask])


def test_attention_half_output_and_replay():
    """o_proj + residual on top of the attention, against the oracle fed the kernel's own attention
    output; replays are bit-equal and a pad row comes back as its residual."""
    cfg, w, t, x, op, out, _ = _run(4, 1500, pad=(2,))
    attn = op.core.out[:4].cpu().float()
    wo = Q.fp8_block_dequant(w["o"].cpu(), w["o_s"].cpu())
    ref = Q.bf(x.cpu().float() + Q.bf(attn @ wo.T))
    keep = [0, 1, 3]
    assert_close_hidden(out[keep], ref[keep], "attention half", scale=float((ref - x.cpu().float()).abs().max()))
    assert torch.equal(out[2].cpu(), x[2].cpu()), "a pad row must come back as its residual"
    assert int(op.core.n_ctx[2]) == 0
    for _ in range(3):
        assert torch.equal(op.launch(x, t), out)


def test_layer_is_attention_half_then_moe_half():
    """The whole layer (BASELINE config 4's shape family at a small size): the MoE half on top of the
    attention half's output, against the FFN oracle fed that output."""
    from dataclasses import replace

    from oracle import layers as OL
    from sgl_amd_mono_b200.config import CFG_TINY_FFN
    from sgl_amd_mono_b200.gqa import GqaLayerOp

    cfg = CFG_GQA_TINY
    moe = replace(CFG_TINY_FFN, name="tiny_gqa_moe", hidden=cfg.hidden, inter=384, shared_fmt="none")
    w = {**synth.layer_weights(moe, 0, DEV), **synth.gqa_weights(cfg, 0, DEV)}
    t = synth.gqa_step(cfg, 5, 1800, DEV)
    x = torch.randn(5, cfg.hidden, generator=torch.Generator().manual_seed(3)).bfloat16().to(DEV)
    op = GqaLayerOp(cfg, moe, w, DEV, max_ctx=1800)
    out = op.launch(x, t).clone()
    torch.cuda.synchronize()
    rc, words = ops.guard_read(op.guard)
    assert rc == 0, f"guard words {words}"
    mid = op.attn.out[:5].cpu()
    wc = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
    ref, det = OL.ffn_block(moe, [wc], mid)
    assert torch.equal(op.ffn.ids[:5].cpu(), det["ids"]), "a near-tie flipped between the f32 logit sums: pick another seed"
    assert_close_hidden(out, ref, "layer output", scale=float((ref.float() - mid.float()).abs().max()))
    assert torch.equal(op.launch(x, t), out)


def test_short_context_keeps_every_block_in_order():
    cfg, w, t, x, op, out, _ = _run(2, 64 * 9 + 3)
    for r in range(2):
        seq = int(t.positions[r]) + 1
        n_blk = -(-seq // BLOCK)
        assert n_blk <= TOPK_BLOCKS
        assert op.core.sel_blocks[r, :n_blk].cpu().tolist() == list(range(n_blk))
        assert int(op.core.n_ctx[r]) == seq


def test_argument_checks():
    cfg = CFG_GQA_TINY
    w = synth.gqa_weights(cfg, 0, DEV)
    t = synth.gqa_step(cfg, 2, 300, DEV)
    op = GqaAttentionOp(cfg, w, DEV, max_ctx=300)
    with pytest.raises(ValueError, match="residual"):
        op.launch(torch.zeros(2, cfg.hidden + 1, dtype=torch.bfloat16, device=DEV), t)
    bad = synth.gqa_step(cfg, 2, 300, DEV)
    bad.k_cache = bad.k_cache[:, :, :1].contiguous()
    with pytest.raises(ValueError, match="k_cache"):
        op.launch(torch.zeros(2, cfg.hidden, dtype=torch.bfloat16, device=DEV), bad)
    a = L.GqaArgs()
    assert L.load().mono_gqa_front_launch(a, None) == -1  # MONO_E_ARG: nothing is launched
