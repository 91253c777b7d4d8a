"""Stage-by-stage comparison of one MLA (+ lightning-indexer) + MoE layer launch with the CPU
oracle, shared by the small-shape tests and the tests at the shapes the benchmark times.

Exact where the domain is integer or bytes (KV and index-key cache bytes given the kernel's own
pre-quantisation values, top-k positions and slots given the kernel's own scores, router ids
given the kernel's own scores), within the hidden-state tolerance elsewhere.  Each half of the
layer is fed the kernel's own upstream result (stage isolation, as the reference's
``test/kernels/deepseek_v41/check_k2.py:303-307`` does), so that a key or an expert that sits on
a near-tie does not charge the stage after it.
"""

import torch

from oracle import layers as OL
from oracle import stages as S
from sgl_amd_mono_b200.config import KV_DIM, PAGE
from util import assert_close_hidden, assert_literal_bar


class LazyExperts:
    """Expert tensors stay on the GPU; the oracle copies to the host only those it routes to."""

    def __init__(self, v):
        self.v, self.c = v, {}

    def __getitem__(self, e):
        e = int(e)
        if e not in self.c:
            self.c[e] = self.v[e].cpu()
        return self.c[e]


def cpu_weights(w, lazy=True):
    out = {}
    for k, v in w.items():
        if lazy and k in ("w13", "w13_s", "w2", "w2_s") and isinstance(v, torch.Tensor) and v.is_cuda:
            out[k] = LazyExperts(v)
        else:
            out[k] = v.cpu() if isinstance(v, torch.Tensor) else v
    return out


def check_mla_layer(cfg, op, w, step, dstep, h, out, pad=(), out_max_abs=4e-2, chain=True, literal=False):
    """``op`` has just run ``op.launch(h, dstep)`` -> ``out``; ``step`` holds the caches BEFORE the launch
    (CPU), ``dstep`` the device tables after it.  Returns the measured errors."""
    rows = h.shape[0]
    wc = cpu_weights(w)
    live = [r for r in range(rows) if r not in pad]
    kvp = step.kv_pages.clone()
    ixp = step.idx_pages.clone() if step.idx_pages is not None else None
    r = OL.attn_front(cfg, wc, h, step.positions, step.slots, step.cos, step.sin, kvp, ixp)
    res = {}
    # ---- cache rows: values close, bytes exact given the kernel's own bf16 values
    kv_k = op.kv_out[:rows].cpu().float()
    res["kv"] = assert_close_hidden(kv_k[live], torch.cat([r["latent"], r["k_pe"]], -1)[live], "latent | k_pe")
    row_b, row_s = S.kv_row_encode(kv_k[:, :512], kv_k[:, 512:])
    got_pages = dstep.kv_pages.cpu()
    for i in live:
        p, o = divmod(int(step.slots[i]), PAGE)
        assert torch.equal(got_pages[p, o * KV_DIM : (o + 1) * KV_DIM], row_b[i]), f"KV bytes of row {i}"
        assert got_pages[p, PAGE * KV_DIM :].view(torch.float32)[o] == row_s[i]
    changed = (got_pages != step.kv_pages).any(1).nonzero().flatten().tolist()
    assert set(changed) <= {int(step.slots[i]) // PAGE for i in live}, "only the live rows' pages may change"
    topk_k = op.topk_slots[:rows].cpu()
    if cfg.index_heads:
        # ---- index keys: bytes exact given the kernel's own f32 values
        ik_k = op.ik_out[:rows].cpu()
        assert torch.allclose(ik_k[live], r["idx_key"][live], atol=2e-2, rtol=2e-2)
        packed, codes = S.index_key_encode(ik_k)
        got_idx = dstep.idx_pages.cpu()
        for i in live:
            p, o = divmod(int(step.slots[i]), PAGE)
            assert torch.equal(got_idx[p, o * 64 : (o + 1) * 64], packed[i]), f"index key bytes of row {i}"
            assert torch.equal(got_idx[p, PAGE * 64 + o * 4 : PAGE * 64 + (o + 1) * 4], codes[i])
        assert_close_hidden(op.idx_q[:rows].cpu()[live], r["idx_q"][live], "index q", scale=float(r["idx_q"].abs().max()))
        assert torch.allclose(op.idx_w[:rows].cpu()[live], r["idx_w"][live], atol=1e-3, rtol=1e-3)
        # ---- scores close to the oracle's; top-k exact on the kernel's own scores
        sc_k = op.scores[:rows].cpu()
        pos_k = op.topk_pos[:rows].cpu()
        _, scores_o = OL.index_select(cfg, r, step.positions, step.slots, step.page_table, got_idx)
        for i in range(rows):
            if i in pad:
                assert int((topk_k[i] >= 0).sum()) == 0
                continue
            n = int(step.positions[i]) + 1
            ref_sc = scores_o[i]
            assert torch.allclose(sc_k[i, :n], ref_sc, atol=2e-2 * float(ref_sc.abs().max()), rtol=0), f"scores of row {i}"
            want = S.exact_topk_positions(sc_k[i], n, cfg.index_topk)
            assert pos_k[i, : want.numel()].tolist() == want.tolist(), f"top-k positions of row {i}"
            assert topk_k[i, : want.numel()].tolist() == S.slots_of_positions(step.page_table[i], want).tolist()
            assert int((topk_k[i, want.numel():] >= 0).sum()) == 0
    else:
        for i in live:  # no indexer: every causal key in order, or the last `window` of them
            n = int(step.positions[i]) + 1
            pos = torch.arange(n)[-cfg.window:] if getattr(cfg, "window", 0) else torch.arange(n)
            want = S.slots_of_positions(step.page_table[i], pos)
            got = topk_k[i][topk_k[i] >= 0]
            assert got.tolist() == want.tolist(), f"selection of row {i}"
    res["q"] = assert_close_hidden(op.q_full[:rows].cpu()[live], r["q_full"][live], "q_lat | q_pe",
                                   scale=float(r["q_full"].abs().max()))
    # ---- attention half on the kernel's own selection
    livemask = step.slots >= 0
    part = OL.attn_back(cfg, wc, r, topk_k, kvp)
    h1_ref = S.allreduce_rank_order([part * livemask[:, None]], h)
    attn_scale = float((h1_ref.float() - h.float()).abs().max())
    h1_k = op.h1[:rows].cpu()
    if literal:
        res["h1"] = assert_literal_bar(h1_k[live], h1_ref[live], "h1 after attention")
    else:
        res["h1"] = assert_close_hidden(h1_k[live], h1_ref[live], "h1 after attention", scale=attn_scale)
    res["attn_scale"] = attn_scale
    if op.ffn is None:
        return res
    # ---- MoE half on the kernel's own h1
    mp, ids_o, wts_o, _ = OL.moe_partial(cfg, wc, h1_k, livemask)
    ref = S.allreduce_rank_order([mp], h1_k)
    ids_k, wts_k = S.route_from_scores(op.ffn.scores[:rows].cpu(), wc.get("router_bias"), cfg.top_k, cfg.route_scale)
    for i in live:
        assert op.ffn.ids[i].cpu().tolist() == ids_k[i].tolist(), f"router ids of row {i}"
        assert ids_k[i].tolist() == ids_o[i].tolist(), "a near-tie flipped between the f32 logit sums: pick another seed"
        assert torch.allclose(op.ffn.weights[i].cpu(), wts_k[i], atol=1e-5, rtol=1e-5), f"route weights of row {i}"
    scale = float((ref.float() - h1_k.float()).abs().max())
    res["moe_scale"] = scale
    if literal:
        res["out"] = assert_literal_bar(out.cpu()[live], ref[live], "layer output")
    else:
        res["out"] = assert_close_hidden(out.cpu()[live], ref[live], "layer output", scale=scale, max_abs=out_max_abs)
    if chain:
        # end to end against the oracle's own chain: cosine only (selections may differ at the margin)
        full, _ = OL.layer_all_ranks(cfg, [wc], h, step.positions, step.slots, step.page_table, step.cos, step.sin,
                                     step.kv_pages.clone(), step.idx_pages.clone() if step.idx_pages is not None else None)
        cos = torch.nn.functional.cosine_similarity(out.cpu()[live].float().flatten(), full[live].float().flatten(), dim=0)
        assert float(cos) >= 0.999, f"end-to-end cosine {float(cos):.6f}"
        res["chain_cos"] = float(cos)
    for i in pad:
        assert torch.equal(out[i].cpu(), h[i]), "a pad row passes through unchanged"
    return res
