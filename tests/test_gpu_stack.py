"""The tail launch (final norm + LM head), verify steps whose rows share a request, and a
small stack replayed from one CUDA graph, against the CPU oracle."""

from dataclasses import replace

import pytest
import torch

from oracle import layers as OL
from oracle import stages as S
from sgl_amd_mono_b200 import ops, synth
from sgl_amd_mono_b200.config import CFG_TINY

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CFG_TINY_FLASH = replace(CFG_TINY, name="tiny_flash", index_heads=0, vocab=5000)


def _cpu(w):
    return {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in w.items()}


@pytest.mark.parametrize("rows", [1, 8, 13])
def test_lm_head_matches_the_f32_tail(rows):
    from sgl_amd_mono_b200.tail import LmHeadOp

    g = torch.Generator().manual_seed(3)
    hidden, vocab = 1024, 5000
    w = (torch.randn(vocab, hidden, generator=g) * 0.02).bfloat16()
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
    h = torch.randn(rows, hidden, generator=g).bfloat16()
    op = LmHeadOp(hidden, w.to(DEV), gamma.to(DEV), 1e-6, DEV)
    got = op(h.to(DEV)).cpu()
    ref = S.tail_logits(h, gamma, 1e-6, w)
    assert got.shape == (rows, vocab) and got.dtype == torch.float32
    # the launch rounds the normalised rows to bf16 (MMA operand); the golden tail keeps f32
    assert float((got - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    assert torch.equal(got.argmax(-1), ref.argmax(-1))


def _tables(step):
    from sgl_amd_mono_b200.layer import StepTables

    t = lambda x: None if x is None else x.to(DEV)  # noqa: E731
    return StepTables(t(step.positions), t(step.slots), t(step.page_table), t(step.kv_pages), t(step.idx_pages),
                      t(step.cos), t(step.sin))


def test_verify_rows_of_one_request_see_their_earlier_drafts():
    """5 verify rows of one request + the same for a second request: row j attends the keys
    written by rows < j of this very step (written before any row attends)."""
    from sgl_amd_mono_b200.layer import MlaLayerOp

    cfg = CFG_TINY_FLASH
    w = synth.layer_weights(cfg, 0, DEV)
    step = synth.verify_step(cfg, n_req=2, tokens=5, ctx=200)
    rows = 10
    h = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
    op = MlaLayerOp(cfg, w, DEV, max_ctx=256)
    tables = _tables(step)
    out = op.launch(h.to(DEV), tables).clone()
    torch.cuda.synchronize()
    assert ops.guard_read(op.guard)[0] == 0
    # every row selected exactly its causal keys, in order, ending with its own slot
    tk = op.topk_slots[:rows].cpu()
    for i in range(rows):
        n = int(step.positions[i]) + 1
        want = S.slots_of_positions(step.page_table[i], torch.arange(n))
        assert tk[i, :n].tolist() == want.tolist() and int((tk[i, n:] >= 0).sum()) == 0
        assert tk[i, n - 1] == step.slots[i]
    ref, det = OL.layer_all_ranks(cfg, [_cpu(w)], h, step.positions, step.slots, step.page_table, step.cos, step.sin,
                                  step.kv_pages.clone(), None)
    cos = torch.nn.functional.cosine_similarity(op.h1[:rows].cpu().float().flatten(), det["h1"].float().flatten(), dim=0)
    assert float(cos) >= 0.999
    # dropping the earlier drafts of the step from the cache must change a later row (negative control)
    step2 = synth.verify_step(cfg, n_req=2, tokens=5, ctx=200)
    t2 = _tables(step2)
    t2.slots[:4] = -1  # rows 0..3 of request 0 write nothing
    out2 = op.launch(h.to(DEV), t2)
    assert not torch.equal(out2[4], out[4])


def test_stack_replays_from_one_graph():
    from sgl_amd_mono_b200.stack import DecoderStack

    cfg = CFG_TINY_FLASH
    n_layers, rows, ctx = 3, 7, 130
    ws = [synth.layer_weights(cfg, 0, DEV, layer=i) for i in range(n_layers)]

    # 5 verify rows of one request + 2 decode rows of two more requests would need ragged tables;
    # here: one request of 5 verify rows and a second of 2
    steps = [synth.verify_step(cfg, 7, 1, ctx, layer=i) for i in range(n_layers)]
    tables = [_tables(s) for s in steps]
    st = DecoderStack(cfg, ws, DEV, max_ctx=192, draft_weights=synth.layer_weights(cfg, 0, DEV, layer=99))
    h = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(6)).bfloat16().to(DEV)
    draft_tables = _tables(synth.verify_step(cfg, 7, 1, ctx, layer=99))
    x0, logits0 = st.step(h, tables, draft_tables)
    x0, logits0 = x0.clone(), logits0.clone()
    torch.cuda.synchronize()
    assert ops.guard_read(st.guard)[0] == 0
    st.capture(h, tables, draft_tables)
    for _ in range(3):
        x, logits = st.replay()
        torch.cuda.synchronize()
        # the caches already hold this step's rows, so a replay rewrites identical bytes
        assert torch.equal(x, x0) and torch.equal(logits, logits0)
    assert logits0.shape == (rows, cfg.vocab) and torch.isfinite(logits0).all()
    # oracle chain over the layers: cosine (selections are whole contexts here, no indexer)
    hh = h.cpu()
    for i in range(n_layers):
        s = steps[i]
        hh, _ = OL.layer_all_ranks(cfg, [_cpu(ws[i])], hh, s.positions, s.slots, s.page_table, s.cos, s.sin,
                                   s.kv_pages.clone(), None)
    cos = torch.nn.functional.cosine_similarity(x0.cpu().float().flatten(), hh.float().flatten(), dim=0)
    assert float(cos) >= 0.995, f"cosine after {n_layers} layers {float(cos):.6f}"
    ref_logits = S.tail_logits(hh, _cpu(ws[-1])["final_norm"], cfg.eps, _cpu(ws[-1])["lm_head"])
    cos = torch.nn.functional.cosine_similarity(logits0.cpu().flatten(), ref_logits.flatten(), dim=0)
    assert float(cos) >= 0.995
