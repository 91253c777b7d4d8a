"""Whole-layer CPU restatement (test infrastructure only): one rank's share of an
MLA + lightning-indexer + MoE decoder layer, and of a stand-alone MoE FFN block.

``cfg`` is duck-typed (any object with the attributes used below; the product's
``LayerConfig`` fits).  ``w`` is a dict of this rank's tensors in the layouts SGLang
loads them in (FP8 weights as uint8 E4M3 bytes + f32 128x128 block scales, MXFP4 as
packed nibbles + E8M0 codes).  Stage order follows glm53/gfx950/kernel.py (the stage
list at :171 and the stages cited in ``stages``).
"""

from __future__ import annotations

import torch

from . import quant as Q
from . import stages as S


def _w8(w, name):
    return w[name], w[name + "_s"]


def uk_uv(cfg, w, head: int, full=None):
    """Dequantised W_UK [nope, 512] and W_UV [v, 512] of local head ``head``."""
    per = cfg.nope + cfg.v_head
    if full is None:
        full = Q.fp8_block_dequant(*_w8(w, "kv_b"))
    blk = full[head * per : (head + 1) * per]
    return blk[: cfg.nope], blk[cfg.nope :]


def attn_front(cfg, w, h, positions, slots, cos, sin, kv_pages, idx_pages):
    """Input norm .. q / cache writes.  Returns a dict of the stage outputs."""
    r = {}
    x = S.rmsnorm(h, w["input_norm"], cfg.eps)
    qkv = S.gemv_fp8_block(x, *_w8(w, "qkv_a"))
    ql = cfg.q_lora
    r["qkv_a"] = qkv
    qa = S.rmsnorm(qkv[:, :ql], w["q_a_norm"], cfg.eps)
    lat = S.rmsnorm(qkv[:, ql : ql + 512], w["kv_a_norm"], cfg.eps)
    c, s = cos[positions.long()], sin[positions.long()]
    kpe = Q.bf(S.rope_interleaved(qkv[:, ql + 512 :], c, s))
    r["latent"], r["k_pe"], r["q_a"] = lat, kpe, qa
    row, scale = S.kv_row_encode(lat, kpe)
    S.kv_pages_write(kv_pages, slots, row, scale)
    hl = cfg.n_heads // cfg.tp
    q = S.gemv_fp8_block(qa, *_w8(w, "q_b")).reshape(-1, hl, cfg.nope + cfg.rope)
    q_nope = Q.bf(q[..., : cfg.nope])
    q_pe = Q.bf(S.rope_interleaved(q[..., cfg.nope :], c, s))
    q_lat = torch.empty(q.shape[0], hl, 512)
    kvb = Q.fp8_block_dequant(*_w8(w, "kv_b"))
    for hd in range(hl):
        wuk, _ = uk_uv(cfg, w, hd, kvb)
        q_lat[:, hd] = Q.bf(q_nope[:, hd] @ wuk)
    r["q_full"] = torch.cat([q_lat, q_pe], -1)
    if cfg.index_heads:
        ik = S.gemv_fp8_block(x, *_w8(w, "idx_wk"))
        ik = S.layernorm(ik, w["idx_k_norm_w"], w["idx_k_norm_b"])
        ik = torch.cat([S.rope_interleaved(ik[:, :64], c, s), ik[:, 64:]], -1)
        ik = S.fwht128(ik)
        r["idx_key"] = ik
        packed, codes = S.index_key_encode(ik)
        S.index_pages_write(idx_pages, slots, packed, codes)
        iq = S.gemv_fp8_block(qa, *_w8(w, "idx_wq_b")).reshape(-1, cfg.index_heads, 128)
        iq = torch.cat([S.rope_interleaved(iq[..., :64], c, s), iq[..., 64:]], -1)
        r["idx_q"] = Q.bf(S.fwht128(iq))
        # head weights stay f32 (glm53/gfx950/kernel.py:1781-1970 hands weights_proj on in f32)
        wts = x.float() @ w["idx_wproj"].float().T
        r["idx_w"] = wts * ((cfg.index_heads**-0.5) * (128**-0.5))
    return r


def index_select(cfg, r, positions, slots, page_table, idx_pages):
    """Scores of every causal key and the exact top-k, as global KV slots [S, topk] (-1 pad)."""
    rows = positions.shape[0]
    # without an indexer every causal key is attended
    width = cfg.index_topk if cfg.index_heads else int(positions.max()) + 1
    topk = torch.full((rows, width), -1, dtype=torch.int32)
    scores = []
    for s in range(rows):
        if slots[s] < 0:
            scores.append(torch.zeros(0))
            continue
        n = int(positions[s]) + 1
        pos = torch.arange(n)
        ksl = S.slots_of_positions(page_table[s], pos)
        if cfg.index_heads:
            sc = S.index_scores(r["idx_q"][s], r["idx_w"][s], S.index_keys_gather(idx_pages, ksl))
            sel = S.exact_topk_positions(sc, n, cfg.index_topk)
            scores.append(sc)
        else:
            # no indexer: every causal key, or the last `window` of them (the draft model's attention)
            sel = pos[-cfg.window:] if getattr(cfg, "window", 0) else pos
        topk[s, : sel.numel()] = ksl[sel].to(torch.int32)
    return topk, scores


def attn_back(cfg, w, r, topk, kv_pages):
    """Sparse MLA over the selected slots, W_UV, o_proj: this rank's f32 partial [S, H]."""
    hl = cfg.n_heads // cfg.tp
    lat = S.sparse_mla(r["q_full"].to(torch.bfloat16), kv_pages, topk,
                       S.sm_scale_mla(cfg.nope, cfg.rope)).float()
    o = torch.empty(lat.shape[0], hl, cfg.v_head)
    kvb = Q.fp8_block_dequant(*_w8(w, "kv_b"))
    for hd in range(hl):
        _, wuv = uk_uv(cfg, w, hd, kvb)
        o[:, hd] = Q.bf(lat[:, hd] @ wuv.T)
    r["attn_lat"], r["attn_o"] = lat, o
    return S.gemv_fp8_block(o.reshape(lat.shape[0], -1), *_w8(w, "o_proj"))


def _expert(cfg, w, x, e: int):
    if cfg.expert_fmt == "fp8_block":
        return S.expert_fp8(x, w["w13"][e], w["w13_s"][e], w["w2"][e], w["w2_s"][e])
    if cfg.expert_fmt == "nvfp4":
        return S.expert_nvfp4(x, w["w13"][e], w["w13_s"][e], w["w13_g"][e], w["w2"][e], w["w2_s"][e], w["w2_g"][e])
    return S.expert_mxfp4(x, w["w13"][e], w["w13_s"][e], w["w2"][e], w["w2_s"][e])


def _shared(cfg, w, x):
    if cfg.shared_fmt == "none":
        return torch.zeros(x.shape[0], cfg.hidden)
    if cfg.shared_fmt == "bf16":
        return S.expert_bf16(x, w["sh13"], w["sh2"])
    if cfg.shared_fmt == "fp8_block":
        return S.expert_fp8(x, w["sh13"], w["sh13_s"], w["sh2"], w["sh2_s"])
    if cfg.shared_fmt == "nvfp4":
        return S.expert_nvfp4(x, w["sh13"], w["sh13_s"], w["sh13_g"], w["sh2"], w["sh2_s"], w["sh2_g"])
    return S.expert_mxfp4(x, w["sh13"], w["sh13_s"], w["sh2"], w["sh2_s"])


def moe_partial(cfg, w, h1, live=None):
    """Post-attention norm, router, shared + routed experts: (f32 partial [S, H], ids, weights, logits).

    Pad rows (``live`` False) route nowhere and produce zeros (minimax_m31/runner.py:153-157).
    """
    x = S.rmsnorm(h1, w["post_norm"], cfg.eps)
    logits = x.float() @ w["router"].float().T
    ids, wts = S.route(logits, w.get("router_bias"), cfg.top_k, cfg.route_scale)
    out = torch.zeros(x.shape[0], cfg.hidden)
    for e in ids.unique().tolist():
        rows, ks = (ids == e).nonzero(as_tuple=True)
        out[rows] += wts[rows, ks, None] * _expert(cfg, w, x[rows], e)
    out = out + _shared(cfg, w, x)
    if live is not None:
        out = out * live[:, None].float()
    return out, ids, wts, logits


def layer_all_ranks(cfg, ws, h, positions, slots, page_table, cos, sin, kv_pages, idx_pages):
    """The whole layer over every rank's weights ``ws`` (list): returns (x_out bf16, details).

    The caches are replicated in the reference (every rank writes the same bytes);
    here they are written once.  Both all-reduces sum in rank order.
    """
    det = {}
    parts = []
    topk = None
    for rank, w in enumerate(ws):
        kvp = kv_pages if rank == 0 else kv_pages.clone()
        ixp = idx_pages if rank == 0 else (idx_pages.clone() if idx_pages is not None else None)
        r = attn_front(cfg, w, h, positions, slots, cos, sin, kvp, ixp)
        if topk is None:  # the indexer is replicated: every rank picks the same keys
            topk, scores = index_select(cfg, r, positions, slots, page_table, ixp)
            det["topk"], det["scores"], det["front0"] = topk, scores, r
        parts.append(attn_back(cfg, w, r, topk, kvp))
    live = slots >= 0
    h1 = S.allreduce_rank_order([p * live[:, None] for p in parts], h)
    det["h1"] = h1
    mparts = []
    for w in ws:
        p, ids, wts, logits = moe_partial(cfg, w, h1, live)
        mparts.append(p)
    det["ids"], det["route_w"], det["logits"] = ids, wts, logits
    return S.allreduce_rank_order(mparts, h1), det


def ffn_block(cfg, ws, x):
    """Stand-alone MoE FFN block (BASELINE config 1): out = x + sum_ranks moe(rmsnorm(x))."""
    parts, ids, wts, logits = [], None, None, None
    for w in ws:
        p, ids, wts, logits = moe_partial(cfg, w, x)
        parts.append(p)
    return S.allreduce_rank_order(parts, x), dict(ids=ids, route_w=wts, logits=logits, partials=parts)
