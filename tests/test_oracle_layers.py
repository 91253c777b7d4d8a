"""The layer-level oracle on the CPU: runs, is self-consistent, and agrees with the
product's host-side quantisers (the two are written independently)."""

import torch

from oracle import layers as OL
from oracle import quant as Q
from oracle import stages as S
from sgl_amd_mono_b200 import quant as PQ
import synth
from sgl_amd_mono_b200.config import CFG_FFN_MXFP4, CFG_TINY, CFG_TINY_FFN


def test_product_quantisers_match_oracle():
    g = torch.Generator().manual_seed(3)
    w = torch.randn(16, 256, generator=g) * 0.02
    a, b = PQ.mxfp4_quant(w), Q.mxfp4_quant(w)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    v = torch.randn(1000, generator=g) * 3
    assert torch.equal(PQ.e2m1_encode(v), Q.e2m1_encode(v))
    assert torch.equal(PQ.code_ceil(v.abs() + 1e-3), Q.code_ceil(v.abs() + 1e-3))


def test_kv_rows_of_synth_follow_oracle_rule():
    g = torch.Generator().manual_seed(4)
    vals, sc = synth.kv_rows_random(32, g, "cpu")
    v = torch.randn(32, 576, generator=torch.Generator().manual_seed(4)).bfloat16().float()
    row, sc2 = S.kv_row_encode(v[:, :512], v[:, 512:])
    assert torch.equal(sc, sc2) and torch.equal(row, vals)


def test_sparse_mla_matches_dense_softmax():
    q, pages, sel, _ = synth.sparse_mla_inputs(2, 4, 300, 128, seed=5)
    out = S.sparse_mla(q, pages, sel, 192**-0.5).float()
    for r in range(2):
        kv = S.kv_rows_gather(pages, sel[r][sel[r] >= 0])
        p = torch.softmax((q[r].float() @ kv.T) * 192**-0.5, -1)
        ref = p @ kv[:, :512]
        assert torch.allclose(out[r], ref, atol=2e-2, rtol=2e-2)


def test_ffn_block_tiny_runs_and_routes():
    cfg = CFG_TINY_FFN
    w = synth.layer_weights(cfg)
    x = torch.randn(4, cfg.hidden, generator=torch.Generator().manual_seed(0)).bfloat16()
    out, det = OL.ffn_block(cfg, [w], x)
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    assert det["ids"].shape == (4, cfg.top_k)
    assert torch.allclose(det["route_w"].sum(-1), torch.ones(4), atol=1e-5)
    assert float((out.float() - x.float()).abs().max()) > 0


def test_config1_shapes():
    cfg = CFG_FFN_MXFP4
    assert (cfg.hidden, cfg.n_experts, cfg.top_k, cfg.inter) == (2048, 64, 4, 768)
    w = synth.layer_weights(cfg)
    assert w["w13"].shape == (64, 1536, 1024) and w["w13_s"].shape == (64, 1536, 64)
    assert w["w2"].shape == (64, 2048, 384) and w["router"].dtype == torch.float32
    assert w["sh13"].dtype == torch.bfloat16


def test_layer_tiny_two_ranks_agree_on_topk():
    cfg = CFG_TINY.with_tp(2)
    ws = [synth.layer_weights(cfg, r) for r in range(2)]
    step = synth.decode_step(cfg, rows=2, ctx=300, pad_rows=())
    h = torch.randn(2, cfg.hidden, generator=torch.Generator().manual_seed(1)).bfloat16()
    out, det = OL.layer_all_ranks(cfg, ws, h, step.positions, step.slots, step.page_table, step.cos, step.sin,
                                  step.kv_pages, step.idx_pages)
    assert out.shape == h.shape
    topk = det["topk"]
    assert topk.shape == (2, cfg.index_topk)
    assert int((topk >= 0).sum()) == 2 * cfg.index_topk
    # this step's own slot is among each row's keys only if it scored into the top-k; all picks are distinct
    for r in range(2):
        assert topk[r].unique().numel() == cfg.index_topk
