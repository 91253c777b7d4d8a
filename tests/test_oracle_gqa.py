"""The GQA block-sparse oracle on CPU: selection rules, sort keys, rotation, causal scores.

The reference holds no golden vectors for this path (its kernels are gfx950 programs and its
tests need a GPU), so these cases restate the rules its docstrings give
(``minimax_m3/gfx950/post_attn.py:466-592``, ``select.py:1-12``, ``index_score.py:1-12``)."""

import struct

import torch

from oracle import gqa as OG


def _bits(x: float) -> int:
    return struct.unpack("I", struct.pack("f", x))[0]


def test_sort_key_orders_like_the_float_and_pins_blocks():
    n = 40
    vals = [-3.5, -0.0, 0.0, 1e-30, 2.0, 7.5]
    keys = [OG.index_key(_bits(v), 10, n, 1, 2) for v in vals]
    assert keys == sorted(keys) and keys[1] == keys[2], "-0 and +0 share a key"
    assert OG.index_key(_bits(float("nan")), 10, n, 1, 2) == -(2**31), "NaN sorts below everything"
    first = OG.index_key(_bits(-5.0), 0, n, 1, 2)
    local = OG.index_key(_bits(-5.0), n - 1, n, 1, 2)
    assert first > local > OG.index_key(_bits(1e20), 10, n, 1, 2), "init blocks, then local blocks, then scores"


def test_selection_pins_ranks_and_places_the_tail_last():
    torch.manual_seed(0)
    seq = 64 * 30 + 7  # 31 blocks, the tail holds 7 keys
    scores = torch.randn(31)
    blocks, n_ctx = OG.select_blocks(scores, seq, init_blocks=1, local_blocks=2)
    assert len(blocks) == 16 and len(set(blocks)) == 16
    assert blocks[0] == 0, "the init block has the largest key"
    assert blocks[-1] == 30, "the tail block goes last"
    assert 29 in blocks, "both local blocks are pinned"
    rest = [b for b in blocks if b not in (0, 29, 30)]
    want = sorted(range(1, 29), key=lambda b: (float(scores[b]), b), reverse=True)[:13]
    assert rest == want, "the other 13 by (score, id) descending"
    assert n_ctx == 15 * 64 + 7


def test_ties_go_to_the_larger_block_id_and_short_contexts_keep_everything():
    scores = torch.zeros(40)
    blocks, _ = OG.select_blocks(scores, 64 * 40, init_blocks=0, local_blocks=0)
    assert blocks == list(range(38, 23, -1)) + [39], "equal keys: larger ids first, the tail block last"
    blocks, n_ctx = OG.select_blocks(torch.randn(9), 64 * 8 + 1, 1, 2)
    assert blocks == list(range(9)) and n_ctx == 64 * 8 + 1


def test_tail_not_selected_when_local_blocks_is_zero():
    scores = torch.arange(20, dtype=torch.float32).flip(0)  # block 0 best, the tail worst
    blocks, n_ctx = OG.select_blocks(scores, 64 * 19 + 5, init_blocks=0, local_blocks=0)
    assert blocks == list(range(16)) and n_ctx == 16 * 64


def test_head_norm_rope_keeps_pair_norms():
    torch.manual_seed(1)
    x = torch.randn(128)
    cos, sin = OG.neox_table(100)
    y0 = OG.head_norm_rope(x, torch.zeros(128), cos[0], sin[0], 1e-6)
    y = OG.head_norm_rope(x, torch.zeros(128), cos[37], sin[37], 1e-6)
    assert torch.equal(y[64:], y0[64:]), "dims past the rotary part are not rotated"
    n0 = y0[:32] ** 2 + y0[32:64] ** 2
    n1 = y[:32] ** 2 + y[32:64] ** 2
    assert torch.allclose(n0, n1, rtol=3e-2), "a rotation keeps each (i, i + 32) pair's norm (bf16 rounding aside)"
    assert abs(float((y0 * y0).mean()) - 1.0) < 2e-2


def test_block_scores_are_causal_maxima():
    torch.manual_seed(2)
    keys = torch.randn(300, 128)
    iq = torch.randn(128).bfloat16().float()
    sc = OG.block_scores(iq, keys, 200, 0.1)
    assert sc.shape == (4,)
    dots = keys[:200] @ iq
    scale = OG.index_scale_log2e(0.1)
    assert abs(float(sc[3]) - float(dots[192:200].max()) * scale) < 1e-5, "the tail block sees only its causal keys"
    keys2 = keys.clone()
    keys2[200:] = 1e3
    assert torch.equal(OG.block_scores(iq, keys2, 200, 0.1), sc)


def test_attention_half_inserts_the_new_token_and_leaves_pad_rows_alone():
    import synth
    from sgl_amd_mono_b200.gqa import CFG_GQA_TINY as cfg

    w = synth.gqa_weights(cfg, 0, "cpu")
    t = synth.gqa_step(cfg, 3, 1300, "cpu")
    t.slots[1] = -1
    x = torch.randn(3, cfg.hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
    caches = [t.k_cache.clone(), t.v_cache.clone(), t.index_cache.clone()]
    out = OG.attention_half(cfg, w, x, t.positions, t.slots, t.page_table, caches, t.cos, t.sin)
    assert out.shape == x.shape and out.dtype == torch.bfloat16
    assert torch.equal(out[1], x[1]), "a pad row comes back as its residual"
    assert not torch.equal(out[0], x[0])
    for r in (0, 2):
        page, off = int(t.slots[r]) // 64, int(t.slots[r]) % 64
        assert not torch.equal(caches[0][page, off], t.k_cache[page, off]), "the new token's K is inserted"
    changed = (caches[0] != t.k_cache).any(-1).any(-1).sum()
    assert int(changed) == 2, "nothing but the two live rows' slots is written"
    # the new token attends to itself: dropping its key changes the output
    caches2 = [t.k_cache.clone(), t.v_cache.clone(), t.index_cache.clone()]
    w2 = dict(w, v_scale=w["v_scale"] * 2)
    out2 = OG.attention_half(cfg, w2, x, t.positions, t.slots, t.page_table, caches2, t.cos, t.sin)
    assert not torch.equal(out2[0], out[0])


def test_attention_row_matches_plain_softmax():
    torch.manual_seed(3)
    q = torch.randn(4, 128).bfloat16().float()
    k = torch.randn(64 * 5, 128)
    v = torch.randn(64 * 5, 128)
    n_ctx = 64 * 4 + 9
    got = OG.sparse_attention_row(q, k, v, 0.05, 0.04, n_ctx, OG.sm_scale_gqa())
    s = (q @ k[:n_ctx].T) * (0.05 * OG.sm_scale_gqa())
    want = torch.softmax(s, -1) @ v[:n_ctx] * 0.04
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-3)
