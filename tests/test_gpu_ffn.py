"""MoE FFN block on the GPU through the C ABI against the CPU oracle (BASELINE config 1
and the FP8 block-scaled expert path of config 3 at a small size)."""

from dataclasses import replace

import pytest
import torch

from oracle import layers as OL
from oracle import quant as Q
from oracle import stages as S
from sgl_amd_mono_b200 import _lib as L
import synth
from sgl_amd_mono_b200 import ops
from sgl_amd_mono_b200.config import CFG_FFN_MXFP4, CFG_TINY, CFG_TINY_FFN, CFG_TINY_FFN_NVFP4
from util import assert_close_hidden, assert_rel

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CFG_TINY_MOE8 = replace(CFG_TINY, name="tiny_moe_fp8", n_heads=0, index_heads=0)
# an intermediate size that ends inside a 256-value MXFP4 tile (config 4 at TP 4: 1536 / 4 = 384), no shared expert
CFG_TINY_FFN_384 = replace(CFG_TINY_FFN, name="tiny_ffn_mxfp4_k384", inter=384, shared_fmt="none")
# narrow experts: up/gate, activation and down run chained inside one launch by default
CFG_TINY_MOE8_256 = replace(CFG_TINY_MOE8, name="tiny_moe_fp8_chained", inter=256)


# NVFP4 experts: K that ends inside a 256-value tile and no shared expert; the 2048-wide block with 64 experts
CFG_TINY_NVFP4_384 = replace(CFG_TINY_FFN_NVFP4, name="tiny_ffn_nvfp4_k384", inter=384, shared_fmt="none")
CFG_FFN_NVFP4 = replace(CFG_FFN_MXFP4, name="ffn_nvfp4_2048", expert_fmt="nvfp4")


def _cpu(w):
    return {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in w.items()}


def _run(cfg, rows, seed=0, pad=()):
    from sgl_amd_mono_b200.moe import MoeFfn

    w = synth.layer_weights(cfg, 0, DEV)
    x = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(seed)).bfloat16()
    slots = torch.arange(1, rows + 1, dtype=torch.int64)
    for r in pad:
        slots[r] = -1
    ffn = MoeFfn(cfg, w, DEV)
    out = ffn(x.to(DEV), slots.to(DEV)).clone()
    torch.cuda.synchronize()
    rc, words = ops.guard_read(ffn.guard)
    assert rc == 0, f"guard words {words}"
    return ffn, w, x, slots, out


@pytest.mark.parametrize("cfg,rows", [(CFG_TINY_FFN, 1), (CFG_TINY_FFN, 4), (CFG_TINY_FFN, 11),
                                      (CFG_TINY_MOE8, 1), (CFG_TINY_MOE8, 8), (CFG_TINY_MOE8, 16),
                                      (CFG_FFN_MXFP4, 4), (CFG_TINY_FFN_384, 5), (CFG_TINY_FFN_384, 16),
                                      (CFG_TINY_MOE8_256, 8), (CFG_TINY_MOE8_256, 16),
                                      (CFG_TINY_FFN_NVFP4, 1), (CFG_TINY_FFN_NVFP4, 7), (CFG_TINY_FFN_NVFP4, 16),
                                      (CFG_TINY_NVFP4_384, 5), (CFG_FFN_NVFP4, 4)])
def test_ffn_block_matches_oracle(cfg, rows):
    ffn, w, x, slots, out = _run(cfg, rows)
    wc = _cpu(w)
    ref, det = OL.ffn_block(cfg, [wc], x)
    # routing is exact given the kernel's own scores: ties to the lower id, weights renormalised
    scores = ffn.scores[:rows].cpu()
    ids, wts = S.route_from_scores(scores, wc.get("router_bias"), cfg.top_k, cfg.route_scale)
    assert torch.equal(ffn.ids[:rows].cpu(), ids)
    assert torch.allclose(ffn.weights[:rows].cpu(), wts, rtol=1e-5, atol=1e-7)
    assert torch.allclose(scores, torch.sigmoid(det["logits"]), atol=1e-4)
    assert torch.equal(ids, det["ids"]), "a near-tie flipped between the f32 logit sums: pick another seed"
    n = int(ffn.n_expert.item())
    assert ffn.expert_list[:n].cpu().tolist() == sorted(set(ids.flatten().tolist()))
    scale = float((ref.float() - x.float()).abs().max())
    assert_close_hidden(out, ref, f"{cfg.name} rows={rows}", scale=scale)


def test_pad_rows_contribute_nothing():
    cfg = CFG_TINY_MOE8
    ffn, w, x, slots, out = _run(cfg, 4, pad=(1,))
    assert torch.equal(out[1].cpu(), x[1]), "a pad row must come back as its residual"
    assert ffn.ids[1].cpu().tolist() == [-1] * cfg.top_k
    ref, _ = OL.ffn_block(cfg, [_cpu(w)], x)
    keep = [0, 2, 3]
    scale = float((ref.float() - x.float()).abs().max())
    assert_close_hidden(out[keep], ref[keep], "live rows beside a pad row", scale=scale)


@pytest.mark.parametrize("rows", [1, 8, 16])
def test_tcgen05_and_warp_mma_paths_agree(rows):
    """The FP8 GEMV has two consumers (tcgen05 + TMEM, warp-level MMA); both compute every 128-k chunk
    exactly in f32 from the same E4M3 bytes, so they differ only in the order of f32 additions."""
    cfg = CFG_TINY_MOE8
    lib = L.load()
    old = lib.mono_set_gemv_tcgen05(1)
    try:
        ffn, w, x, slots, out_tc = _run(cfg, rows)
        lib.mono_set_gemv_tcgen05(0)
        ffn2, _, _, _, out_mma = _run(cfg, rows)
    finally:
        lib.mono_set_gemv_tcgen05(old)
    assert torch.equal(ffn.ids.cpu(), ffn2.ids.cpu())
    d = (out_tc.float() - out_mma.float()).abs()
    tol = 2.0 ** -7 * out_mma.float().abs().clamp_min(1.0)  # at most one bf16 ulp
    assert bool((d <= tol).all()), f"max diff {float(d.max())}"
    assert float((d > 0).float().mean()) < 0.05, "only rare last-bit differences are expected"


@pytest.mark.parametrize("mode", ["2", "1"])
@pytest.mark.parametrize("cfg,rows", [(CFG_FFN_MXFP4, 4), (CFG_TINY_FFN_384, 5), (CFG_TINY_FFN_384, 16)])
def test_block_scaled_mxfp4_agrees_with_the_group_kernel(cfg, rows, mode, monkeypatch):
    """MXFP4 experts on tcgen05 in three ways: kind::mxf8f6f4.block_scale (the MMA reads both operands' E8M0 codes from
    tensor memory and adds a task's whole K run in one accumulator) with the nibbles padded by TMA and the weights'
    codes fetched in tensor-core order (mode 2, the default) or spread and gathered by warps of the kernel (mode 1),
    and kind::f8f6f4 per 32-value group with the codes applied in the epilogue in f32 (mode 0).  Same bytes, same
    exact products; the block-scaled sum is formed inside the tensor core instead of group by group in f32, so the
    partial sums agree to f32 rounding of a K-long sum: |difference| <= 2^-18 x (largest partial sum of the launch),
    and the block's bf16 output to one ulp."""
    monkeypatch.setenv("MONO_TC4_BLOCK_SCALE", mode)
    ffn, w, x, slots, out_bs = _run(cfg, rows)
    n = int(ffn.n_expert.item())
    up_bs, dn_bs = ffn.up_r[: n * ffn.ns_up].float().cpu().clone(), ffn.down_p.float().cpu().clone()
    monkeypatch.setenv("MONO_TC4_BLOCK_SCALE", "0")
    ffn2, _, _, _, out_g = _run(cfg, rows)
    assert torch.equal(ffn.ids.cpu(), ffn2.ids.cpu())
    up_g, dn_g = ffn2.up_r[: n * ffn2.ns_up].float().cpu(), ffn2.down_p.float().cpu()
    for name, a, b in (("up/gate partial sums", up_bs, up_g), ("down partial sums", dn_bs, dn_g)):
        assert torch.isfinite(a).all(), name
        tol = 2.0 ** -18 * float(b.abs().max())
        assert float((a - b).abs().max()) <= tol, f"{name}: {float((a - b).abs().max())} > {tol}"
    d = (out_bs.float() - out_g.float()).abs()
    assert bool((d <= 2.0 ** -7 * out_g.float().abs().clamp_min(1.0)).all()), f"max diff {float(d.max())}"


@pytest.mark.parametrize("rows", [1, 8, 16])
def test_chained_launch_equals_separate_launches(rows, monkeypatch):
    """up/gate -> SwiGLU -> down inside one launch does the arithmetic of the separate launches in the
    same order: activations, scales and the block's output are bit-equal."""
    cfg = CFG_TINY_MOE8
    monkeypatch.setenv("MONO_MOE_CHAINED", "1")  # the default chains only narrow per-rank experts
    ffn, w, x, slots, out = _run(cfg, rows)
    assert ffn.chained is not None, "an FP8 block on the tcgen05 path can take the chained launch"
    monkeypatch.setenv("MONO_MOE_CHAINED", "0")
    ffn2, _, _, _, out2 = _run(cfg, rows)
    assert ffn2.chained is None
    n = int(ffn.n_expert.item())
    assert torch.equal(ffn.mid_r.planes[:n], ffn2.mid_r.planes[:n])
    assert torch.equal(ffn.mid_r.scale_f32[:n, :rows], ffn2.mid_r.scale_f32[:n, :rows])
    assert torch.equal(ffn.mid_s.planes, ffn2.mid_s.planes)
    assert torch.equal(ffn.down_p, ffn2.down_p)
    assert torch.equal(out, out2)
    # replays of the chained launch: the counters and stamps reset themselves
    xd, sd = x.to(DEV), slots.to(DEV)
    for _ in range(4):
        assert torch.equal(ffn(xd, sd), out)
    torch.cuda.synchronize()
    rc, words = ops.guard_read(ffn.guard)
    assert rc == 0, f"guard words {words}"


@pytest.mark.parametrize("cfg_name,rows", [("moe8", 1), ("moe8", 16), ("ffn", 11)])
def test_fused_router_equals_two_launches(cfg_name, rows, monkeypatch):
    """Logits and routing in one launch (the last CTA to finish its columns routes the step) give the
    bits of the logits launch followed by the routing launch, on every replay."""
    cfg = CFG_TINY_MOE8 if cfg_name == "moe8" else CFG_TINY_FFN
    monkeypatch.setenv("MONO_ROUTER_FUSED", "1")
    ffn, w, x, slots, out = _run(cfg, rows)
    assert ffn.router_fused
    monkeypatch.setenv("MONO_ROUTER_FUSED", "0")
    ffn2, _, _, _, out2 = _run(cfg, rows)
    assert not ffn2.router_fused
    xd, sd = x.to(DEV), slots.to(DEV)
    for _ in range(3):
        for name in ("logits", "scores", "ids", "weights", "n_expert"):
            assert torch.equal(getattr(ffn, name)[:rows], getattr(ffn2, name)[:rows]), name
        n = int(ffn.n_expert.item())
        assert torch.equal(ffn.expert_list[:n], ffn2.expert_list[:n])
        assert torch.equal(ffn.coef[:n], ffn2.coef[:n])
        assert torch.equal(out, out2)
        assert int(ffn.route_counter.item()) == 0, "the launch leaves its counter at zero"
        out = ffn(xd, sd).clone()
        torch.cuda.synchronize()


def test_paired_activation_launch_equals_two_launches(monkeypatch):
    """The shared expert's and the routed experts' activation stages in one launch write the bytes of
    the two single launches."""
    cfg, rows = CFG_TINY_MOE8, 7
    monkeypatch.setenv("MONO_MOE_CHAINED", "0")
    ffn, w, x, slots, out = _run(cfg, rows)
    assert ffn.chained is None and ffn.has_shared
    il = cfg.inter_local
    ref_r = ops.ActBuf(ffn.mid_r.fmt, il, DEV, segs=ffn.max_expert)
    ref_s = ops.ActBuf(ffn.mid_s.fmt, il, DEV)
    ops.mid(rows, il, ffn.up_r, ffn.ns_up, ref_r, n_slot=ffn.n_expert, max_slot=ffn.max_expert)
    ops.mid(rows, il, ffn.up_s, ffn.ns_up_s, ref_s, max_slot=1)
    torch.cuda.synchronize()
    n = int(ffn.n_expert.item())
    assert torch.equal(ffn.mid_r.planes[:n], ref_r.planes[:n])
    assert torch.equal(ffn.mid_r.scale_f32[:n, :rows], ref_r.scale_f32[:n, :rows])
    assert torch.equal(ffn.mid_s.planes, ref_s.planes)
    assert torch.equal(ffn.mid_s.scale_f32[..., :rows, :], ref_s.scale_f32[..., :rows, :])
    assert ffn.mid_s.planes.any() and ffn.mid_r.planes[:n].any()


def test_replays_are_bit_equal():
    cfg = CFG_TINY_MOE8
    ffn, w, x, slots, out = _run(cfg, 8)
    xd, sd = x.to(DEV), slots.to(DEV)
    for _ in range(5):
        again = ffn(xd, sd)
        torch.cuda.synchronize()
        assert torch.equal(again, out)
    # a perturbed input must change the output (negative control)
    x2 = xd.clone()
    x2[0, 0] += 1.0
    assert not torch.equal(ffn(x2, sd), out)


def test_nvfp4_activation_bytes_are_bit_exact():
    """Packed E2M1 values and E4M3 scale bytes of the NVFP4 activation format against the CPU restatement."""
    rows, k = 5, 512
    x = (torch.randn(rows, k, generator=torch.Generator().manual_seed(7)) * 2).bfloat16()
    x[2, 128:256] = 0   # all-zero blocks: the smallest scale, zero values
    x[3, 16:32] *= 4096  # a block whose scale saturates at 448: its values clamp at 6
    buf = ops.ActBuf(L.ACT_NVF4, k, DEV)
    ops.act_prep(rows, k, buf, src_bf16=x.to(DEV), round_bf16=False)
    torch.cuda.synchronize()
    q, sb = Q.nvfp4_act_quant(x)
    assert torch.equal(buf.planes[0, 0, :rows, : k // 2].cpu(), q)
    assert torch.equal(buf.scale_e8[0, :rows, : k // 16].cpu(), sb)
    assert int(buf.planes[0, :, rows:].abs().sum()) == 0
    assert int(sb[3, 1]) == 0x7E and int(sb[2, 8]) == 1


@pytest.mark.parametrize("n,k,rows", [(128, 256, 16), (200, 640, 5), (384, 2048, 1)])
def test_nvfp4_gemv_matches_dequantised_matmul(n, k, rows):
    """One dense NVFP4 job (kind::mxf4nvf4.block_scale) against the f32 matmul of both operands' dequantised values:
    every product and every scale is exact in f32, so only the summation inside the tensor core differs (5e-5 of the
    largest sum; a misplaced scale byte or nibble would show as percents)."""
    g = torch.Generator().manual_seed(n + k)
    wf = torch.randn(1, n, k, generator=g) * 0.05
    wf[0, :, 32:48] *= 40  # blocks with very different scales inside one MMA's 64 values
    wq, ws, wg = Q.nvfp4_quant(wf)
    x = (torch.randn(rows, k, generator=g) * torch.logspace(-2, 1, k // 16).repeat_interleave(16)).bfloat16()
    buf = ops.ActBuf(L.ACT_NVF4, k, DEV)
    ops.act_prep(rows, k, buf, src_bf16=x.to(DEV), round_bf16=False)
    gemv = ops.Gemv(L.W_NVFP4)
    st, ns = ops.plan_split(-(-k // 256), -(-n // 128), L.W_NVFP4)
    out = torch.full((ns, 16, n), float("nan"), device=DEV)
    assert gemv.add("w", wq.to(DEV), buf, out, wscale=ws.to(DEV), wglobal=wg.to(DEV), split_tiles=st, nsplit=ns) == ns
    gemv.launch(rows)
    torch.cuda.synchronize()
    xq, xs = Q.nvfp4_act_quant(x)
    ref = Q.nvfp4_dequant(xq, xs, 1.0) @ Q.nvfp4_dequant(wq[0], ws[0], 1.0).T * float(wg[0])
    got = out[:, :rows].cpu()
    assert torch.isfinite(got).all()
    assert_rel(got.sum(0), ref, f"NVFP4 GEMV {n}x{k}, {rows} rows", 5e-5)
    assert bool(torch.isnan(out[:, rows:]).all()), "rows past the step are not written"


@pytest.mark.parametrize("fmt", [L.ACT_A8, L.ACT_HILO, L.ACT_MX8, L.ACT_MX8N, L.ACT_BF16])
def test_activation_formats_are_bit_exact(fmt):
    rows, k = 5, 512
    x = (torch.randn(rows, k, generator=torch.Generator().manual_seed(7)) * 2).bfloat16()
    x[2, 128:256] = 0  # an all-zero chunk
    buf = ops.ActBuf(fmt, k, DEV)
    ops.act_prep(rows, k, buf, src_bf16=x.to(DEV), round_bf16=False)
    torch.cuda.synchronize()
    planes = buf.planes[0, :, :rows, : (2 * k if fmt == L.ACT_BF16 else k)].cpu()
    if fmt == L.ACT_A8:
        q, sc = Q.act_quant_128(x)
        assert torch.equal(planes[0], Q.e4m3_bytes(q))
        assert torch.equal(buf.scale_f32[0, :rows, : k // 128].cpu(), sc)
    elif fmt == L.ACT_HILO:
        hi, lo, sc = Q.split_hi_lo(x)
        assert torch.equal(planes[0], Q.e4m3_bytes(hi)) and torch.equal(planes[1], Q.e4m3_bytes(lo))
        assert torch.equal(buf.scale_f32[0, :rows, : k // 128].cpu(), sc)
    elif fmt in (L.ACT_MX8, L.ACT_MX8N):
        q, code = Q.mxfp8_quant(x)
        perm = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7] if fmt == L.ACT_MX8 else list(range(8)))
        want = Q.e4m3_bytes(q).reshape(rows, k // 8, 8)[:, :, perm].reshape(rows, k)
        assert torch.equal(planes[0], want)
        assert torch.equal(buf.scale_e8[0, :rows, : k // 32].cpu(), code)
    else:
        assert torch.equal(planes[0].contiguous().view(torch.bfloat16), x)
    # rows past the step stay zero
    assert int(buf.planes[0, :, rows:].abs().sum()) == 0


def _act_values(buf, seg, rows, k, fmt):
    """Dequantised values of an activation buffer segment, f32 [rows, k]."""
    pl = buf.planes[seg, 0, :rows].cpu()
    if fmt == L.ACT_A8:
        sc = buf.scale_f32[seg, :rows, : k // 128].cpu()
        return (Q.e4m3_from_bytes(pl[:, :k]).reshape(rows, -1, 128) * sc[..., None]).reshape(rows, k)
    if fmt in (L.ACT_MX8, L.ACT_MX8N):
        # MX8 is stored k0 k2 k4 k6 k1 k3 k5 k7, MX8N in natural order
        inv = torch.tensor([0, 4, 1, 5, 2, 6, 3, 7] if fmt == L.ACT_MX8 else list(range(8)))
        v = Q.e4m3_from_bytes(pl[:, :k]).reshape(rows, k // 8, 8)[:, :, inv].reshape(rows, k)
        return Q.mxfp8_dequant(v, buf.scale_e8[seg, :rows, : k // 32].cpu())
    if fmt == L.ACT_NVF4:
        return Q.nvfp4_dequant(pl[:, : k // 2], buf.scale_e8[seg, :rows, : k // 16].cpu(), 1.0)
    return pl[:, : 2 * k].contiguous().view(torch.bfloat16).float()


@pytest.mark.parametrize("cfg,rows", [(CFG_TINY_MOE8, 16), (CFG_TINY_MOE8, 3), (CFG_TINY_FFN, 11), (CFG_TINY_FFN_NVFP4, 9)])
def test_gemv_stages_in_isolation(cfg, rows):
    """Each GEMV against the oracle's dequantised matmul fed the kernel's own quantised
    operands: the only difference left is the f32 summation order."""
    ffn, w, x, slots, out = _run(cfg, rows)
    wc = _cpu(w)
    fp8, nv4 = cfg.expert_fmt == "fp8_block", cfg.expert_fmt == "nvfp4"

    def deq(name, e):
        if nv4:
            return Q.nvfp4_dequant(wc[name][e], wc[name + "_s"][e], wc[name + "_g"][e])
        return (Q.fp8_block_dequant if fp8 else Q.mxfp4_dequant)(wc[name][e], wc[name + "_s"][e])

    afmt = ffn.xq.fmt  # A8 for FP8 experts; MX8N (tcgen05 consumer) or MX8 (warp-MMA consumer) for MXFP4; NVF4
    assert ffn.mid_r.fmt == afmt
    h, il = cfg.hidden, cfg.inter_local
    n = int(ffn.n_expert.item())
    experts = ffn.expert_list[:n].cpu().tolist()
    xq = _act_values(ffn.xq, 0, rows, h, afmt)
    up = ffn.up_r.cpu().reshape(ffn.max_expert, ffn.ns_up, 16, 2 * il).sum(1)
    coef = ffn.coef[:n, :rows].cpu()
    down_ref = torch.zeros(rows, h)
    for u, e in enumerate(experts):
        assert_rel(up[u, :rows], xq @ deq("w13", e).T, f"up/gate of expert {e}")
        mid_k = _act_values(ffn.mid_r, u, rows, il, afmt)
        mid_o = S.swiglu(up[u, :rows, :il], up[u, :rows, il:])
        if fp8:
            q, sc = Q.act_quant_128(mid_o)
            mid_ref = (q.reshape(rows, -1, 128) * sc[..., None]).reshape(rows, il)
        elif nv4:
            mq, ms = Q.nvfp4_act_quant(Q.bf(mid_o))
            mid_ref = Q.nvfp4_dequant(mq, ms, 1.0)
            step = 2.0 * Q.e4m3_from_bytes(ms).repeat_interleave(16, -1)  # the widest E2M1 step (4 -> 6) of each block
        else:
            q, c = Q.mxfp8_quant(Q.bf(mid_o))
            mid_ref = Q.mxfp8_dequant(q, c)
        # the same values up to a rounding step of the few elements that sit on a boundary
        # (a chunk whose amax moved by an ulp rescales all its values by an ulp: not a flip)
        close = (mid_k - mid_ref).abs() <= ((1.2 * step) if nv4 else (0.13 * mid_ref.abs() + 1e-6))
        flipped = (mid_k - mid_ref).abs() > 1e-4 * mid_ref.abs() + 1e-7
        assert bool(close.all()) and float(flipped.float().mean()) < 0.02
        down_ref += coef[u, :, None] * (mid_k @ deq("w2", e).T)
    routed = ffn.down_p[: ffn.groups, :rows].cpu().sum(0)
    assert_rel(routed, down_ref, "routed down projection")


@pytest.mark.parametrize("dtype,n,k,rows", [(torch.float32, 257, 1024, 16), (torch.bfloat16, 256, 7168, 5)])
def test_rowdot_columns_per_cta_do_not_change_the_bits(dtype, n, k, rows, monkeypatch):
    """Two output columns per CTA share the activation loads; every column's sum keeps its order."""
    g = torch.Generator().manual_seed(n)
    w = torch.randn(n, k, generator=g).to(dtype).to(DEV)
    x = torch.randn(16, k, generator=g).bfloat16().to(DEV)
    outs = []
    for cols in ("1", "2"):
        monkeypatch.setenv("MONO_ROWDOT_COLS", cols)
        out = torch.zeros(16, n, device=DEV)
        ops.rowdot(rows, w, x, out, out_scale=0.5)
        torch.cuda.synchronize()
        outs.append(out.cpu())
    assert torch.equal(outs[0], outs[1])
    ref = 0.5 * (x[:rows].float().cpu() @ w.float().cpu().T)
    assert_rel(outs[1][:rows], ref, "rowdot", 1e-3)
    assert not bool(outs[1][rows:].any()), "rows past the step are not written"
