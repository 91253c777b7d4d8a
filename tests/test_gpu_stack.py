"""The tail launch (final norm + LM head), verify steps whose rows share a request, and a
small stack replayed from one CUDA graph, against the CPU oracle."""

from dataclasses import replace

import pytest
import torch

from oracle import layers as OL
from oracle import stages as S
import synth
from sgl_amd_mono_b200 import ops
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
    dw = synth.layer_weights(cfg, 0, DEV, layer=99)
    st = DecoderStack(cfg, ws, DEV, max_ctx=192, draft_weights=dw)
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
    # oracle, layer by layer, each fed the kernels' own input rows of that layer (stage isolation: what layer i reads is
    # layer i - 1's `out` buffer), held to cosine 0.999 per layer and per row
    F = torch.nn.functional
    x_in = h.cpu()
    for i in range(n_layers):
        s = steps[i]
        ref_i, _ = OL.layer_all_ranks(cfg, [_cpu(ws[i])], x_in, s.positions, s.slots, s.page_table, s.cos, s.sin,
                                      s.kv_pages.clone(), None)
        got_i = st.layers[i].ffn.out[:rows].cpu()
        cos = F.cosine_similarity(got_i.float(), ref_i.float(), dim=-1)
        assert float(cos.min()) >= 0.999, f"layer {i}: min per-row cosine {float(cos.min()):.6f}"
        x_in = got_i
    assert torch.equal(x_in, x0.cpu())
    ref_logits = S.tail_logits(x0.cpu(), _cpu(ws[-1])["final_norm"], cfg.eps, _cpu(ws[-1])["lm_head"])
    cos = F.cosine_similarity(logits0.cpu(), ref_logits, dim=-1)
    assert float(cos.min()) >= 0.999
    assert torch.equal(logits0.argmax(-1).cpu(), ref_logits.argmax(-1))
    # the draft stage's output against the oracle on the draft's own tables and weights
    ds = synth.verify_step(cfg, 7, 1, ctx, layer=99)
    dref, _ = OL.layer_all_ranks(cfg, [_cpu(dw)], h.cpu(), ds.positions, ds.slots,
                                 ds.page_table, ds.cos, ds.sin, ds.kv_pages.clone(), None)
    dcos = F.cosine_similarity(st.draft_out.cpu().float(), dref.float(), dim=-1)
    assert float(dcos.min()) >= 0.999, f"draft stage: min per-row cosine {float(dcos.min()):.6f}"


def test_draft_layer_attends_its_window_and_routes_top3():
    """The draft model's stage (reference ``deepseek_v41/draft.py``): the target's layer with 128 experts top-3 (here 8,
    top-3) and window-only attention.  A block of 5 verify rows of one request + 3 of another: each row selects exactly
    its last `window` keys (its earlier drafts among them), and the layer matches the oracle stage by stage."""
    from layer_checks import check_mla_layer
    from sgl_amd_mono_b200.layer import MlaLayerOp

    cfg = replace(CFG_TINY_FLASH, name="tiny_draft", n_experts=8, top_k=3, window=128 + 16, vocab=0)
    w = synth.layer_weights(cfg, 0, DEV)
    step = synth.verify_step(cfg, n_req=2, tokens=4, ctx=700)
    rows = 8
    h = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(8)).bfloat16()
    op = MlaLayerOp(cfg, w, DEV, max_ctx=704)
    assert op.topk == 192 and op.window == 144
    tables = _tables(step)
    out = op.launch(h.to(DEV), tables).clone()
    torch.cuda.synchronize()
    assert ops.guard_read(op.guard)[0] == 0
    res = check_mla_layer(cfg, op, w, step, tables, h, out)
    assert op.ffn.ids[:rows].shape[1] == 3
    print("draft layer:", res["h1"], res["out"])
    # a short context (fewer keys than the window): every key, in order
    step2 = synth.verify_step(cfg, n_req=1, tokens=3, ctx=100)
    h2 = h[:3]
    t2 = _tables(step2)
    out2 = op.launch(h2.to(DEV), t2).clone()
    check_mla_layer(cfg, op, w, step2, t2, h2, out2, chain=False)


def test_ffn_runner_takes_the_attention_output_through_the_seam():
    """``FfnRunner(attn, residual, weights, slots) -> (out, res_out)`` (``minimax_m31/runner.py:145-167``): o_proj of the
    rank's attention output, the attention reduction and residual, then the MoE block; a pad row joins no expert."""
    from sgl_amd_mono_b200.config import CFG_TINY
    from sgl_amd_mono_b200.minimax_m31.runner import FfnRunner
    from oracle import quant as Q
    from util import assert_close_hidden

    cfg = replace(CFG_TINY, index_heads=0)
    w = synth.layer_weights(cfg, 0, DEV)
    rows = 5
    g = torch.Generator().manual_seed(12)
    attn = torch.randn(rows, cfg.heads_local * cfg.v_head, generator=g).bfloat16()
    residual = torch.randn(rows, cfg.hidden, generator=g).bfloat16()
    slots = torch.tensor([3, 4, -1, 9, 11], dtype=torch.int64)
    run = FfnRunner(cfg, w, DEV)
    out, res_out = run(attn.to(DEV), residual.to(DEV), w, slots.to(DEV))
    torch.cuda.synchronize()
    assert ops.guard_read(run.guard)[0] == 0
    wc = _cpu(w)
    live = slots >= 0
    part = attn.float() @ Q.fp8_block_dequant(wc["o_proj"], wc["o_proj_s"]).T
    h1 = S.allreduce_rank_order([part * live[:, None]], residual)
    assert_close_hidden(res_out, h1, "residual after the seam", scale=float((h1.float() - residual.float()).abs().max()))
    assert torch.equal(res_out[2].cpu(), residual[2])
    mp, ids, _, _ = OL.moe_partial(cfg, wc, res_out.cpu(), live)
    ref = S.allreduce_rank_order([mp], res_out.cpu())
    assert torch.equal(run.ffn.ids[:rows].cpu()[live], ids[live])
    assert_close_hidden(out, ref, "FFN output", scale=float((ref.float() - res_out.cpu().float()).abs().max()), max_abs=4e-2)
    assert torch.equal(out[2].cpu(), res_out[2].cpu()), "a pad row's MoE output is zero"
    with pytest.raises(ValueError, match="bound to the tensors"):
        run(attn.to(DEV), residual.to(DEV), dict(w), slots.to(DEV))
    out_b, res_b = run(None, residual.to(DEV), None, slots.to(DEV))
    assert res_b.data_ptr() == residual.to(DEV).data_ptr() or torch.equal(res_b.cpu(), residual)


def test_m31_spec_builds_nvfp4_experts_from_the_checkpoint_config():
    """MiniMax-M3.1-Flash's checkpoint config (``moe_quant_algo: NVFP4``, reference ``minimax_m31/spec.py:116-121`` and
    ``test/unit/test_minimax_m31_spec.py:16``) builds FFN launches over NVFP4 experts; the one-time repack of their
    scale bytes lands among the build context's copies; the block matches the CPU restatement."""
    from types import SimpleNamespace

    from sgl_amd_mono_b200.minimax_m31 import spec as m31
    from util import assert_close_hidden

    hf = SimpleNamespace(hidden_size=512, n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=256,
                         routed_scaling_factor=1.0, scoring_func="sigmoid", rms_norm_eps=1e-6, shared_expert_format="none",
                         quantization_config=dict(quant_method="mxfp8", moe_quant_algo="NVFP4"))
    assert m31.SPEC.config_disable_reasons(SimpleNamespace(tp_size=1, page_size=64, speculative_algorithm=None), hf) == []
    cfg = m31.layer_config(hf, 1)
    assert cfg.expert_fmt == "nvfp4"
    w = synth.layer_weights(cfg, 0, DEV)
    model = SimpleNamespace(layers=[SimpleNamespace(weights=w)])
    ctx = SimpleNamespace(tp_size=1, device=DEV, deadline_s=5.0, copies={}, widths=(16,), max_context=4096)
    built = m31.SPEC.build(model, hf, ctx)
    kinds = {k[0] for k in ctx.copies}
    assert kinds == {"NVFP4 scale bytes in tensor-core order"} and len(ctx.copies) == 2, ctx.copies.keys()
    rows = 6
    x = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(21)).bfloat16()
    slots = torch.arange(1, rows + 1, dtype=torch.int64)
    run = built.ops[0]
    out, res = run(None, x.to(DEV), None, slots.to(DEV))
    torch.cuda.synchronize()
    assert ops.guard_read(run.guard)[0] == 0
    ref, det = OL.ffn_block(cfg, [_cpu(w)], x)
    assert torch.equal(run.ffn.ids[:rows].cpu(), det["ids"])
    assert_close_hidden(out, ref, "M3.1 FFN launch over NVFP4 experts", scale=float((ref.float() - x.float()).abs().max()))
