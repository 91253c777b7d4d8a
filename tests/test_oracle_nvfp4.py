"""Known answers of the NVFP4 restatement (E2M1 values, an unsigned E4M3 scale byte per 16, an f32 scale per matrix).

The reference holds no NVFP4 arithmetic of its own: MiniMax-M3.1-Flash's NVFP4 experts run in SGLang's MoE runner
(``minimax_m31/spec.py:117-121``), so there are no golden vectors of the reference to pin these functions on.  They
are pinned on the format's published value tables instead: the eight E2M1 magnitudes, round-to-nearest-even at their
midpoints, E4M3 bytes of the block scales.
"""

import torch

import synth
from oracle import layers as OL
from oracle import quant as Q
from oracle import stages as S
from sgl_amd_mono_b200 import quant as PQ
from sgl_amd_mono_b200.config import CFG_TINY_FFN_NVFP4


def _codes(packed):
    return torch.stack([packed & 15, packed >> 4], -1).flatten(-2)


def test_every_e2m1_value_survives_with_scale_one():
    vals = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.5, -1, -1.5, -2, -3, -4, -6, 0.0])
    q, sb = Q.nvfp4_act_quant(vals[None])
    assert sb.tolist() == [[0x38]]  # amax 6 -> scale 1.0
    assert _codes(q)[0].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 9, 10, 11, 12, 13, 14, 15, 0]
    assert torch.equal(Q.nvfp4_dequant(q, sb, 1.0)[0], vals)


def test_midpoints_round_to_the_even_mantissa():
    vals = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 7.0])
    q, sb = Q.nvfp4_act_quant(vals[None])
    # amax 7 -> 7/6 = 1.1667 -> E4M3 1.125 (0x39); the values are divided by 1.125 before rounding
    assert sb.tolist() == [[0x39]]
    # with scale exactly 1 (amax 6) the ties are visible
    vals[-1] = 6.0
    q, sb = Q.nvfp4_act_quant(vals[None])
    assert sb.tolist() == [[0x38]]
    assert _codes(q)[0].tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 8, 10, 10, 12, 12, 14, 14, 7]


def test_block_scale_bytes():
    def scale_of(amax):
        v = torch.zeros(1, 16)
        v[0, 3] = amax
        return int(Q.nvfp4_act_quant(v)[1][0, 0])

    assert scale_of(6.0) == 0x38            # 1.0
    assert scale_of(6.0 * 1.0625) == 0x38   # midpoint of 1.0 and 1.125 -> even mantissa
    assert scale_of(6.0 * 1.1875) == 0x3A   # midpoint of 1.125 and 1.25 -> 1.25
    assert scale_of(12.0) == 0x40           # 2.0
    assert scale_of(6.0 * 448.0) == 0x7E    # the largest E4M3 value
    assert scale_of(1e9) == 0x7E            # saturates; the values then clamp at 6
    assert scale_of(0.0) == 0x01            # never zero: the smallest subnormal, 2^-9
    q, sb = Q.nvfp4_act_quant(torch.full((1, 16), 1e9))
    assert _codes(q)[0].tolist() == [7] * 16


def test_dequant_of_known_bytes():
    packed = torch.tensor([[0x7F, 0x19]], dtype=torch.uint8)  # -6, 6, -0.5, 0.5
    packed = torch.cat([packed, torch.zeros(1, 6, dtype=torch.uint8)], -1)
    sb = torch.tensor([[0x40]], dtype=torch.uint8)            # 2.0
    v = Q.nvfp4_dequant(packed, sb, 0.5)
    assert v[0, :4].tolist() == [-6.0, 6.0, -0.5, 0.5]


def test_weight_quantiser_is_a_fixed_point_and_matches_the_library_side():
    g = torch.Generator().manual_seed(3)
    w = torch.randn(3, 64, 128, generator=g) * 0.02
    w[1] *= 30
    p, s, gl = Q.nvfp4_quant(w)
    assert p.shape == (3, 64, 64) and s.shape == (3, 64, 8) and gl.shape == (3,)
    d = Q.nvfp4_dequant(p, s, gl)
    # error of a value: at most half of the widest E2M1 step (4 -> 6: 1/6 of the block's largest magnitude), a little
    # more where the block scale was rounded down to its E4M3 byte and the largest value clamps
    blk_amax = w.reshape(3, 64, 8, 16).abs().amax(-1, keepdim=True)
    err = (d - w).reshape(3, 64, 8, 16).abs()
    assert float((err / blk_amax).max()) < 0.18
    p2, s2, _ = Q.nvfp4_quant(d, gl)
    assert torch.equal(p, p2) and torch.equal(s, s2)
    for a, b in zip(PQ.nvfp4_quant(w), (p, s, gl)):
        assert torch.equal(a, b)
    # the largest block scale of each matrix is the largest E4M3 value
    assert s.reshape(3, -1).amax(-1).tolist() == [0x7E] * 3


def test_expert_is_the_matmul_of_the_dequantised_operands():
    cfg = CFG_TINY_FFN_NVFP4
    w = synth.layer_weights(cfg, 0, "cpu")
    x = torch.randn(4, cfg.hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
    e = 3
    got = S.expert_nvfp4(x, w["w13"][e], w["w13_s"][e], w["w13_g"][e], w["w2"][e], w["w2_s"][e], w["w2_g"][e])
    xq, xs = Q.nvfp4_act_quant(x)
    h = Q.nvfp4_dequant(xq, xs, 1.0) @ Q.nvfp4_dequant(w["w13"][e], w["w13_s"][e], w["w13_g"][e]).T
    il = cfg.inter_local
    mid = Q.bf(S.swiglu(h[:, :il], h[:, il:]))
    mq, ms = Q.nvfp4_act_quant(mid)
    want = Q.nvfp4_dequant(mq, ms, 1.0) @ Q.nvfp4_dequant(w["w2"][e], w["w2_s"][e], w["w2_g"][e]).T
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-6)
    ref, _ = OL.ffn_block(cfg, [w], x)  # the whole block runs on this format, shared expert included
    assert torch.isfinite(ref.float()).all()


def test_quantisation_error_of_the_block_against_float_weights():
    """The NVFP4 block stays close to the same block computed with the dequantised weights in float and unquantised
    activations: the format's own error, a few percent."""
    cfg = CFG_TINY_FFN_NVFP4
    w = synth.layer_weights(cfg, 0, "cpu")
    x = torch.randn(6, cfg.hidden, generator=torch.Generator().manual_seed(9)).bfloat16()
    xn = S.rmsnorm(x, w["post_norm"], cfg.eps).float()
    il = cfg.inter_local
    e = 0
    w13 = Q.nvfp4_dequant(w["w13"][e], w["w13_s"][e], w["w13_g"][e])
    w2 = Q.nvfp4_dequant(w["w2"][e], w["w2_s"][e], w["w2_g"][e])
    h = xn @ w13.T
    want = S.swiglu(h[:, :il], h[:, il:]) @ w2.T
    got = S.expert_nvfp4(Q.bf(xn), w["w13"][e], w["w13_s"][e], w["w13_g"][e], w["w2"][e], w["w2_s"][e], w["w2_g"][e])
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    assert float(cos) > 0.98


def test_scale_bytes_in_tensor_core_order():
    """The one-time repack of the weights' scale bytes: byte (r % 32) * 16 + (r // 32) * 4 + b of the 512-byte piece of
    (row block, 256-value tile, MMA) is the scale of row r, 16-value block b; padding rows and tiles hold 1.0."""
    from sgl_amd_mono_b200 import ops

    g = torch.Generator().manual_seed(11)
    mats, rows, kb = 2, 200, 40  # K = 640: two and a half tiles; one and a half row blocks
    ws = torch.randint(0, 127, (mats, rows, kb), generator=g, dtype=torch.uint8)
    t = ops.tile_nvfp4_scales(ws)
    assert t.shape == (mats, 2, 3 * 2048)
    for mat, r, k16 in [(0, 0, 0), (1, 37, 5), (0, 129, 17), (1, 199, 39), (0, 64, 16), (1, 127, 31)]:
        rb, rr = divmod(r, 128)
        tile, rem = divmod(k16, 16)
        mma, b = divmod(rem, 4)
        off = tile * 2048 + mma * 512 + (rr % 32) * 16 + (rr // 32) * 4 + b
        assert int(t[mat, rb, off]) == int(ws[mat, r, k16]), (mat, r, k16)
    # padding: rows 200..255 of block 1, tiles past K
    assert int(t[0, 1, (199 - 128 + 1) % 32 * 16 + ((199 - 128 + 1) // 32) * 4]) == 0x38
    assert set(t[0, 0, 2 * 2048 + 2 * 512 :].tolist()) == {0x38}
    # every source byte appears exactly once
    assert int((t != 0x38).sum()) <= mats * rows * kb
    assert sorted(t[t != 0x38].tolist()) == sorted(ws[ws != 0x38].tolist())


def test_mxfp4_scale_codes_in_tensor_core_order():
    """The same repack for MXFP4 codes: one 512-byte block per (128-row block, 128-value tile), byte
    (r % 32) * 16 + (r // 32) * 4 + g = row r, 32-value group g; padding holds the code of 2^0."""
    from sgl_amd_mono_b200 import ops

    g = torch.Generator().manual_seed(12)
    mats, rows, kb = 3, 130, 14  # K = 448: three and a half tiles
    ws = torch.randint(100, 126, (mats, rows, kb), generator=g, dtype=torch.uint8)
    t = ops.tile_mxfp4_scales(ws)
    assert t.shape == (mats, 2, 4 * 512)
    for mat, r, k32 in [(0, 0, 0), (2, 37, 5), (1, 129, 13), (0, 127, 12), (2, 64, 3)]:
        rb, rr = divmod(r, 128)
        tile, grp = divmod(k32, 4)
        assert int(t[mat, rb, tile * 512 + (rr % 32) * 16 + (rr // 32) * 4 + grp]) == int(ws[mat, r, k32]), (mat, r, k32)
    assert int(t[0, 1, 2 * 16]) == 127 and int(t[0, 0, 3 * 512 + 2]) == 127  # a row past the matrix; a group past K
    assert sorted(t[t != 127].tolist()) == sorted(ws.flatten().tolist())
