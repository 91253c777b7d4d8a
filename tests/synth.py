"""Seeded synthetic checkpoints, caches and decode steps in SGLang's loaded layouts.

There are no checkpoints or datasets in the build environment, so parity tests and
the benchmark run on random-init weights and caches with the reference's shapes and
value recipes: block-FP8 values ``randn -> E4M3`` with scales ``(0.5 + U) * K^-0.5``
(``test/kernels/glm53/check_layer.py:56-64,84-103``), MXFP4 and NVFP4 experts drawn
``N(0, 0.02)``, a shuffled page table (``test/kernels/glm53_flash/check_layer.py:276-279``)
and per-layer seeds ``1000 * layer + 7`` (weights) / ``+ 11`` (caches)
(``test/kernels/glm53/check_layer.py:84,171``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from sgl_amd_mono_b200 import quant
from sgl_amd_mono_b200.config import IDX_PAGE_BYTES, KV_DIM, KV_PAGE_BYTES, PAGE, LayerConfig


def _gen(seed: int, device) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def _norm(n, g, device, dtype=torch.bfloat16):
    return (1.0 + 0.1 * torch.randn(n, generator=g, device=device)).to(dtype)


def _experts(cfg: LayerConfig, n: int, g, device, fmt: str, chunk: int = 8):
    """(w13, w13_s, w2, w2_s) for ``n`` experts of this rank in format ``fmt``."""
    il, h = cfg.inter_local, cfg.hidden
    if fmt == "bf16":
        w13 = (torch.randn(n, 2 * il, h, generator=g, device=device) * 0.02).bfloat16()
        w2 = (torch.randn(n, h, il, generator=g, device=device) * 0.02).bfloat16()
        return w13, None, w2, None
    if fmt == "fp8_block":
        w13 = torch.empty(n, 2 * il, h, dtype=torch.uint8, device=device)
        w2 = torch.empty(n, h, il, dtype=torch.uint8, device=device)
        s13 = torch.empty(n, -(-2 * il // 128), -(-h // 128), device=device)
        s2 = torch.empty(n, -(-h // 128), -(-il // 128), device=device)
        for e0 in range(0, n, chunk):
            m = min(chunk, n - e0)
            w13[e0 : e0 + m], s13[e0 : e0 + m] = quant.random_fp8_block(2 * il, h, g, device, (m,))
            w2[e0 : e0 + m], s2[e0 : e0 + m] = quant.random_fp8_block(h, il, g, device, (m,))
        return w13, s13, w2, s2
    if fmt == "nvfp4":
        w13 = torch.empty(n, 2 * il, h // 2, dtype=torch.uint8, device=device)
        w2 = torch.empty(n, h, il // 2, dtype=torch.uint8, device=device)
        s13 = torch.empty(n, 2 * il, h // 16, dtype=torch.uint8, device=device)
        s2 = torch.empty(n, h, il // 16, dtype=torch.uint8, device=device)
        g13, g2 = torch.empty(n, device=device), torch.empty(n, device=device)
        for e0 in range(0, n, chunk):
            m = min(chunk, n - e0)
            w13[e0 : e0 + m], s13[e0 : e0 + m], g13[e0 : e0 + m] = quant.nvfp4_quant(
                torch.randn(m, 2 * il, h, generator=g, device=device) * 0.02)
            w2[e0 : e0 + m], s2[e0 : e0 + m], g2[e0 : e0 + m] = quant.nvfp4_quant(
                torch.randn(m, h, il, generator=g, device=device) * 0.02)
        return w13, (s13, g13), w2, (s2, g2)
    assert fmt == "mxfp4"
    w13 = torch.empty(n, 2 * il, h // 2, dtype=torch.uint8, device=device)
    w2 = torch.empty(n, h, il // 2, dtype=torch.uint8, device=device)
    s13 = torch.empty(n, 2 * il, h // 32, dtype=torch.uint8, device=device)
    s2 = torch.empty(n, h, il // 32, dtype=torch.uint8, device=device)
    for e0 in range(0, n, chunk):
        m = min(chunk, n - e0)
        w13[e0 : e0 + m], s13[e0 : e0 + m] = quant.mxfp4_quant(
            torch.randn(m, 2 * il, h, generator=g, device=device) * 0.02)
        w2[e0 : e0 + m], s2[e0 : e0 + m] = quant.mxfp4_quant(
            torch.randn(m, h, il, generator=g, device=device) * 0.02)
    return w13, s13, w2, s2


def layer_weights(cfg: LayerConfig, rank: int = 0, device="cpu", layer: int = 0, out_scale: float = 1.0) -> dict:
    """One rank's tensors of one layer.  Replicated tensors depend on the layer seed
    only, so they are identical on every rank; sharded ones also depend on the rank.
    ``out_scale`` multiplies the block scales of the projections that write into the
    residual stream (o_proj, the experts' down projections): with the reference's recipe a
    block adds values of magnitude 3..10 to the stream; 0.1 makes that O(1) ("unit scale")."""
    g = _gen(1000 * layer + 7, device)
    gs = _gen(1000 * layer + 7 + 101 * (rank + 1), device)
    w: dict = {}
    h = cfg.hidden
    if cfg.n_heads:
        hl = cfg.heads_local
        w["input_norm"] = _norm(h, g, device)
        w["qkv_a"], w["qkv_a_s"] = quant.random_fp8_block(cfg.q_lora + KV_DIM, h, g, device)
        w["q_a_norm"] = _norm(cfg.q_lora, g, device)
        w["kv_a_norm"] = _norm(cfg.kv_lora, g, device)
        if cfg.index_heads:
            w["idx_wq_b"], w["idx_wq_b_s"] = quant.random_fp8_block(cfg.index_heads * 128, cfg.q_lora, g, device)
            w["idx_wk"], w["idx_wk_s"] = quant.random_fp8_block(128, h, g, device)
            w["idx_k_norm_w"] = _norm(128, g, device, torch.float32)
            w["idx_k_norm_b"] = 0.1 * torch.randn(128, generator=g, device=device)
            w["idx_wproj"] = (torch.randn(cfg.index_heads, h, generator=g, device=device) * 0.02).bfloat16()
        w["q_b"], w["q_b_s"] = quant.random_fp8_block(hl * (cfg.nope + cfg.rope), cfg.q_lora, gs, device)
        w["kv_b"], w["kv_b_s"] = quant.random_fp8_block(hl * (cfg.nope + cfg.v_head), cfg.kv_lora, gs, device)
        w["o_proj"], w["o_proj_s"] = quant.random_fp8_block(h, hl * cfg.v_head, gs, device)
    if cfg.n_experts:
        w["post_norm"] = _norm(h, g, device)
        r = torch.randn(cfg.n_experts, h, generator=g, device=device) * 0.02
        w["router"] = r if cfg.router_dtype == "f32" else r.bfloat16()
        w["router_bias"] = 0.01 * torch.randn(cfg.n_experts, generator=g, device=device)
        w["w13"], w["w13_s"], w["w2"], w["w2_s"] = _experts(cfg, cfg.n_experts, gs, device, cfg.expert_fmt)
        if cfg.expert_fmt == "nvfp4":  # scale bytes per 16 values and one f32 scale per expert
            (w["w13_s"], w["w13_g"]), (w["w2_s"], w["w2_g"]) = w["w13_s"], w["w2_s"]
        if cfg.shared_fmt != "none":
            a, b, c, d = _experts(cfg, 1, gs, device, cfg.shared_fmt)
            w["sh13"], w["sh2"] = a[0], c[0]
            if cfg.shared_fmt == "nvfp4":
                w["sh13_s"], w["sh13_g"], w["sh2_s"], w["sh2_g"] = b[0][0], b[1], d[0][0], d[1]
            elif b is not None:
                w["sh13_s"], w["sh2_s"] = b[0], d[0]
    if out_scale != 1.0:
        for k in ("o_proj_s", "w2_s", "sh2_s"):
            if k in w and w[k] is not None and w[k].dtype == torch.float32:
                w[k] = w[k] * out_scale
    if cfg.vocab:
        w["final_norm"] = _norm(h, g, device)
        w["lm_head"] = (torch.randn(cfg.vocab // cfg.tp, h, generator=gs, device=device) * 0.02).bfloat16()
    return w


def kv_rows_random(n: int, g, device):
    """Random cached tokens: latents ~ N(0,1) -> (E4M3 bytes [n, 576], f32 scales [n])
    with the per-token power-of-two scale 2^ceil(log2(max(amax, 1e-4) / 448))."""
    v = torch.randn(n, KV_DIM, generator=g, device=device).bfloat16().float()
    amax = v.abs().amax(-1).clamp_min(1e-4) / 448.0
    sc = torch.exp2(quant.code_ceil(amax).float() - 127.0)
    return (v / sc[:, None]).to(quant.F8).view(torch.uint8), sc


@dataclass
class Step:
    """One decode step's fixed-address tables (``glm53/spec.py:467-496``)."""

    positions: torch.Tensor  # i64 [rows]
    slots: torch.Tensor  # i64 [rows], -1 = pad row
    page_table: torch.Tensor  # i32 [rows, pages per request]
    kv_pages: torch.Tensor  # u8 [pages, KV_PAGE_BYTES]
    idx_pages: torch.Tensor | None  # u8 [pages, IDX_PAGE_BYTES]
    cos: torch.Tensor  # bf16 [max_pos, 32]
    sin: torch.Tensor


def rope_tables(max_pos: int, device, dim: int = 64, theta: float = 10000.0):
    j = torch.arange(dim // 2, dtype=torch.float64)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * theta ** (-2.0 * j / dim)
    return ang.cos().to(torch.bfloat16).to(device), ang.sin().to(torch.bfloat16).to(device)


def decode_step(cfg: LayerConfig, rows: int, ctx: int, device="cpu", layer: int = 0,
                pad_rows=(), with_index: bool | None = None) -> Step:
    """``rows`` requests, each with ``ctx`` tokens of context; the new token of a
    request sits at position ctx - 1.  Every request owns ceil(ctx / 64) pages taken
    from a random permutation (3 spare pages, page 0 never used: slot 0 is SGLang's pad)."""
    g = _gen(1000 * layer + 11, device)
    per = -(-ctx // PAGE)
    n_pages = rows * per + 4
    perm = (torch.randperm(n_pages - 1, generator=g, device=device) + 1)[: rows * per]
    page_table = perm.reshape(rows, per).to(torch.int32)
    kv_pages = torch.zeros(n_pages, KV_PAGE_BYTES, dtype=torch.uint8, device=device)
    vals, sc = kv_rows_random(n_pages * PAGE, g, device)
    kv_pages[:, : PAGE * KV_DIM] = vals.reshape(n_pages, PAGE * KV_DIM)
    kv_pages[:, PAGE * KV_DIM :] = sc.reshape(n_pages, PAGE).contiguous().view(torch.uint8).reshape(n_pages, PAGE * 4)
    idx_pages = None
    if cfg.index_heads if with_index is None else with_index:
        idx_pages = torch.empty(n_pages, IDX_PAGE_BYTES, dtype=torch.uint8, device=device)
        idx_pages[:, : PAGE * 64] = torch.randint(0, 256, (n_pages, PAGE * 64), generator=g,
                                                   device=device, dtype=torch.uint8)
        idx_pages[:, PAGE * 64 :] = torch.randint(123, 130, (n_pages, PAGE * 4), generator=g,
                                                   device=device, dtype=torch.uint8)
    positions = torch.full((rows,), ctx - 1, dtype=torch.int64, device=device)
    slots = page_table[:, (ctx - 1) // PAGE].long() * PAGE + (ctx - 1) % PAGE
    for r in pad_rows:
        slots[r] = -1
        positions[r] = 0
    cos, sin = rope_tables(max(ctx, 64), device)
    return Step(positions, slots, page_table, kv_pages, idx_pages, cos, sin)


def sparse_mla_inputs(rows: int, heads: int, ctx: int, topk: int, device="cpu", seed: int = 0):
    """BASELINE config 2: bf16 q [rows, heads, 576] ~ N(0,1), FP8 latent pages, and
    ``topk`` slots per row sampled uniformly without replacement from its context
    (the pattern of ``test/kernels/glm53/check_layer.py:206-211``)."""
    g = _gen(seed, device)
    per = -(-ctx // PAGE)
    n_pages = rows * per + 4
    perm = (torch.randperm(n_pages - 1, generator=g, device=device) + 1)[: rows * per]
    page_table = perm.reshape(rows, per).to(torch.int32)
    kv_pages = torch.zeros(n_pages, KV_PAGE_BYTES, dtype=torch.uint8, device=device)
    vals, sc = kv_rows_random(n_pages * PAGE, g, device)
    kv_pages[:, : PAGE * KV_DIM] = vals.reshape(n_pages, PAGE * KV_DIM)
    kv_pages[:, PAGE * KV_DIM :] = sc.reshape(n_pages, PAGE).contiguous().view(torch.uint8).reshape(n_pages, PAGE * 4)
    q = torch.randn(rows, heads, KV_DIM, generator=g, device=device).bfloat16()
    sel = torch.full((rows, topk), -1, dtype=torch.int32, device=device)
    for r in range(rows):
        pos = torch.randperm(ctx, generator=g, device=device)[: min(topk, ctx)]
        sel[r, : pos.numel()] = (page_table[r].long()[pos // PAGE] * PAGE + pos % PAGE).to(torch.int32)
    return q, kv_pages, sel, page_table


def verify_step(cfg: LayerConfig, n_req: int, tokens: int, ctx: int, device="cpu", layer: int = 0) -> Step:
    """A speculative-verify step: ``n_req`` requests x ``tokens`` rows.  Row j of a request sits
    at position ctx - tokens + j and sees the keys up to itself; the rows of one request
    repeat its page-table row (``minimax_m3/metadata.py:7-42``; ``glm53/spec.py:489-491``)."""
    base = decode_step(cfg, n_req, ctx, device=device, layer=layer)
    rows = n_req * tokens
    req = torch.arange(rows, device=device) // tokens
    j = torch.arange(rows, device=device) % tokens
    positions = (ctx - tokens + j).to(torch.int64)
    page_table = base.page_table[req].contiguous()
    slots = page_table.gather(1, (positions // PAGE).unsqueeze(1)).squeeze(1).long() * PAGE + positions % PAGE
    return Step(positions, slots, page_table, base.kv_pages, base.idx_pages, base.cos, base.sin)


# ---------------------------------------------------------------- GQA block-sparse attention
def gqa_weights(cfg, rank: int = 0, device="cpu", layer: int = 0) -> dict:
    """One rank's tensors of the GQA attention half (``gqa.GqaConfig``): block-FP8 fused
    projection q | k | v | index q | index k and o_proj, Gemma head-norm weights near zero,
    the layer's fixed K / V cache scales."""
    g = _gen(1000 * layer + 7, device)
    gs = _gen(1000 * layer + 7 + 101 * (rank + 1), device)
    h = cfg.hidden
    w: dict = {"in_norm": _norm(h, g, device)}
    for k in ("g_q", "g_k", "g_iq", "g_ik"):
        w[k] = (0.1 * torch.randn(128, generator=g, device=device)).bfloat16()
    w["qkv"], w["qkv_s"] = quant.random_fp8_block(cfg.qkv_rows, h, gs, device)
    w["o"], w["o_s"] = quant.random_fp8_block(h, cfg.q_local * 128, gs, device)
    w["k_scale"], w["v_scale"] = 0.05, 0.04
    return w


def gqa_step(cfg, rows: int, ctx: int, device="cpu", layer: int = 0, ragged: bool = True):
    """Caches of ``rows`` requests with up to ``ctx`` cached tokens each (random E4M3 bytes, no
    NaN codes), a shuffled page table, and one decode row per request at its last position."""
    from sgl_amd_mono_b200.gqa import BLOCK, GqaTables

    g = _gen(1000 * layer + 11, device)
    blocks = -(-ctx // BLOCK)
    n_pages = rows * blocks + 1
    perm = torch.randperm(n_pages - 1, generator=g, device=device).to(torch.int32) + 1  # page 0 stays unused
    page_table = perm[: rows * blocks].reshape(rows, blocks).contiguous()

    def rnd(*shape):
        # E4M3 of N(0, 1) / scale-ish values: finite codes only
        return (torch.randn(*shape, generator=g, device=device) * 8.0).clamp(-440, 440).to(quant.F8).view(torch.uint8)

    k_cache = rnd(n_pages, BLOCK, cfg.kv_local, 128)
    v_cache = rnd(n_pages, BLOCK, cfg.kv_local, 128)
    index_cache = (torch.randn(n_pages, BLOCK, 128, generator=g, device=device)).to(quant.F8).view(torch.uint8)
    lens = [ctx - (17 * r if ragged else 0) for r in range(rows)]
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int64, device=device)
    slots = torch.stack([page_table[r, (lens[r] - 1) // BLOCK].long() * BLOCK + (lens[r] - 1) % BLOCK for r in range(rows)])
    cos, sin = rope_tables(ctx + 1, device, dim=64, theta=cfg.rope_theta)
    return GqaTables(positions, slots.contiguous(), page_table, k_cache, v_cache, index_cache, cos, sin)
