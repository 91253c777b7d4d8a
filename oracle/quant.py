"""Number formats of the decode path, restated on CPU (test infrastructure only).

Each helper cites the reference lines whose rule it follows (paths are relative to
the reference project).  All functions take and return torch CPU tensors.

The NVFP4 helpers (``nvfp4_*``) have no reference lines to follow: the reference leaves
that format's arithmetic to SGLang's MoE runner (minimax_m31/spec.py:117-121).  They
restate the published format and are checked against its value tables only: parity
unpinned against any reference output.
"""

from __future__ import annotations

import torch

F8 = torch.float8_e4m3fn
E4M3_MAX = 448.0
# E2M1 code -> value; codes 8..15 are the negatives (sign bit 3).
# test/kernels/deepseek_v41/check_ffn.py:22-39
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def bf(x: torch.Tensor) -> torch.Tensor:
    """Round to bf16 and widen back to f32 (test/kernels/deepseek_v41/check_ffn.py:124)."""
    return x.to(torch.bfloat16).float()


def e4m3(x: torch.Tensor) -> torch.Tensor:
    """Saturating round-to-nearest-even E4M3 round trip, returned as f32."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(F8).float()


def e4m3_bytes(x: torch.Tensor) -> torch.Tensor:
    """Saturating RNE E4M3 encoding as uint8."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(F8).view(torch.uint8)


def e4m3_from_bytes(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(F8).float()


def code_ceil(v: torch.Tensor) -> torch.Tensor:
    """Biased exponent of the smallest power of two >= v, v > 0 finite.

    test/kernels/deepseek_v41/check_ffn.py:86-89; device form
    glm53/gfx950/kernel.py:1452-1466 (exponent + (mantissa != 0)).
    """
    bits = v.float().contiguous().view(torch.int32)
    return ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).int()


def exp2_code(code: torch.Tensor) -> torch.Tensor:
    """2 ** (code - 127) as f32 for an E8M0 code."""
    return torch.exp2(code.float() - 127.0)


# ---------------------------------------------------------------- activations
def act_quant_128(x: torch.Tensor):
    """Per-128 FP8 activation quantisation of a block-FP8 GEMM input.

    glm53/gfx950/kernel.py:1440-1450: amax over the block, scale = amax / 448 (1.0 for
    an all-zero block), q = clamp(x * (448 / amax)) -> E4M3.  Returns (q as f32 values,
    scale f32 [..., K/128]).
    """
    g = x.float().reshape(*x.shape[:-1], -1, 128)
    amax = g.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    inv = torch.where(amax > 0, E4M3_MAX / amax, torch.ones_like(amax))
    q = e4m3(g * inv)
    return q.reshape(x.shape), scale.squeeze(-1)


def mxfp8_quant(x: torch.Tensor):
    """Per-32 MXFP8 activation quantisation, the "round-up" rule.

    glm53/gfx950/kernel.py:1452-1466, common/mx.py:27-39,
    test/kernels/deepseek_v41/check_ffn.py:92-104 ("aiter"): code =
    code_ceil(max(amax, 1e-10) / 448) clamped to 1..254, q = clamp(x * 2^-(code-127)).
    Returns (q as f32 values, E8M0 codes uint8 [..., K/32]).
    """
    g = x.float().reshape(*x.shape[:-1], -1, 32)
    amax = g.abs().amax(-1, keepdim=True)
    code = code_ceil(amax.clamp_min(1e-10) * (1.0 / E4M3_MAX)).clamp(1, 254)
    inv = torch.exp2(127.0 - code.float())
    q = e4m3(g * inv)
    return q.reshape(x.shape), code.squeeze(-1).to(torch.uint8)


def mxfp8_dequant(q: torch.Tensor, code: torch.Tensor) -> torch.Tensor:
    return q * exp2_code(code).repeat_interleave(32, -1)


def token_pow2_scale(amax: torch.Tensor) -> torch.Tensor:
    """Power-of-two per-token scale 2^ceil(log2(max(amax, 1e-4) / 448)).

    glm53/gfx950/kernel.py:2137-2162 (the ue8m0 index-key rule; here it covers the
    576 values of a latent KV row, as BASELINE config 2 asks for one f32 scale per
    token).  Computed on the bits of RN(max(amax, 1e-4) / 448).
    """
    v = amax.float().clamp_min(1e-4) / E4M3_MAX
    return exp2_code(code_ceil(v))


# ---------------------------------------------------------------- E2M1 / MXFP4
def e2m1_encode(v: torch.Tensor) -> torch.Tensor:
    """Saturating round-to-nearest-even E2M1 code (uint8, 0..15) of f32 values.

    deepseek_v4/gfx950/kernels/common.py:83-99 uses the hardware convert (RNE); the
    midpoints 0.25, 1.25, 2.5, 5 go to the even mantissa (0, 1, 2, 4) and 0.75, 1.75,
    3.5 go up (1, 2, 4).
    """
    a = v.float().abs()
    code = torch.zeros_like(a, dtype=torch.uint8)
    # boundaries between consecutive magnitudes, with the tie direction of RNE
    code = torch.where(a > 0.25, torch.tensor(1, dtype=torch.uint8), code)
    code = torch.where(a >= 0.75, torch.tensor(2, dtype=torch.uint8), code)
    code = torch.where(a > 1.25, torch.tensor(3, dtype=torch.uint8), code)
    code = torch.where(a >= 1.75, torch.tensor(4, dtype=torch.uint8), code)
    code = torch.where(a > 2.5, torch.tensor(5, dtype=torch.uint8), code)
    code = torch.where(a >= 3.5, torch.tensor(6, dtype=torch.uint8), code)
    code = torch.where(a > 5.0, torch.tensor(7, dtype=torch.uint8), code)
    sign = (torch.signbit(v.float())).to(torch.uint8) << 3
    return code | sign


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_VALUES + tuple(-x for x in E2M1_VALUES))
    return lut[code.long()]


def mxfp4_quant(w: torch.Tensor):
    """[N, K] f32 -> (packed uint8 [N, K/2], E8M0 codes uint8 [N, K/32]).

    Scale per 32 along K: sc = pow2_ceil(max(amax, 6 * 2^-126) / 6), q = clamp(v / sc,
    +-6) -> E2M1 (deepseek_v4/gfx950/kernels/stages/indexer.py:143-151).  Packing: even
    index in the low nibble (test/kernels/deepseek_v41/check_ffn.py:107-115).
    """
    n, k = w.shape[-2:]
    g = w.float().reshape(*w.shape[:-1], k // 32, 32)
    amax = g.abs().amax(-1, keepdim=True)
    code = code_ceil(amax.clamp_min(6.0 * 2.0**-126) / 6.0).clamp(0, 254)
    sc = exp2_code(code)
    q = e2m1_encode((g / sc).clamp(-6.0, 6.0)).reshape(*w.shape[:-1], k)
    packed = q[..., 0::2] | (q[..., 1::2] << 4)
    return packed.contiguous(), code.squeeze(-1).to(torch.uint8).contiguous()


def mxfp4_dequant(packed: torch.Tensor, code: torch.Tensor) -> torch.Tensor:
    """test/kernels/deepseek_v41/check_ffn.py:107-115."""
    p = packed.view(torch.uint8)
    v = torch.stack([e2m1_decode(p & 15), e2m1_decode(p >> 4)], -1).flatten(-2)
    return v * exp2_code(code.view(torch.uint8)).repeat_interleave(32, -1)


# ---------------------------------------------------------------- NVFP4 (E2M1 values, one E4M3 scale per 16, one f32 scale per tensor)
NVFP4_GROUP = 16


def nvfp4_quant(w: torch.Tensor, global_scale: torch.Tensor | None = None):
    """[.., K] f32 -> (packed uint8 [.., K/2], E4M3 scale bytes uint8 [.., K/16], f32 global scale [..leading dims of
    a matrix] or scalar).

    The published NVFP4 recipe (NVIDIA's block format for Blackwell: E2M1 elements, an unsigned E4M3 scale per 16
    elements, a per-tensor f32 scale that brings the block scales into E4M3's range): global = amax(tensor) /
    (6 * 448); block scale = E4M3(amax(block) / 6 / global), round to nearest even; element = E2M1(v / (scale *
    global)), round to nearest even, saturating at +-6.  Packing as MXFP4: even index in the low nibble.  A matrix
    is the last two dimensions; leading dimensions (experts) get a global scale each.
    """
    k = w.shape[-1]
    wf = w.float()
    if global_scale is None:
        red = tuple(range(max(wf.dim() - 2, 0), wf.dim()))
        global_scale = (wf.abs().amax(red) / (6.0 * 448.0)).clamp_min(2.0**-100)
    g = global_scale.reshape(*global_scale.shape, *([1] * (wf.dim() - global_scale.dim())))
    blk = wf.reshape(*wf.shape[:-1], k // NVFP4_GROUP, NVFP4_GROUP)
    sb = e4m3_bytes(blk.abs().amax(-1) / 6.0 / g)                      # [.., K/16] bytes, all >= 0
    sc = e4m3_from_bytes(sb) * g                                       # the scale a reader reconstructs
    q = e2m1_encode((blk / sc.clamp_min(2.0**-120).unsqueeze(-1)).clamp(-6.0, 6.0)).reshape(*wf.shape[:-1], k)
    q = torch.where((sc == 0).repeat_interleave(NVFP4_GROUP, -1), torch.zeros_like(q), q)
    packed = q[..., 0::2] | (q[..., 1::2] << 4)
    return packed.contiguous(), sb.contiguous(), global_scale.float().contiguous()


def nvfp4_dequant(packed: torch.Tensor, scale_bytes: torch.Tensor, global_scale) -> torch.Tensor:
    """element * E4M3 block scale * f32 global scale, all exact in f32."""
    p = packed.view(torch.uint8)
    v = torch.stack([e2m1_decode(p & 15), e2m1_decode(p >> 4)], -1).flatten(-2)
    g = torch.as_tensor(global_scale, dtype=torch.float32)
    g = g.reshape(*g.shape, *([1] * (v.dim() - g.dim())))
    return v * e4m3_from_bytes(scale_bytes.view(torch.uint8)).repeat_interleave(NVFP4_GROUP, -1) * g


def nvfp4_act_quant(x: torch.Tensor):
    """Activation rows [.., K] -> (packed uint8 [.., K/2], E4M3 scale bytes [.., K/16]) with global scale 1:
    block scale = E4M3(max(amax, 6 * 2^-9) / 6) rounded to nearest even (2^-9 is E4M3's smallest subnormal, so the
    scale is never zero), element = E2M1(v / scale), round to nearest even, saturating."""
    k = x.shape[-1]
    blk = x.float().reshape(*x.shape[:-1], k // NVFP4_GROUP, NVFP4_GROUP)
    sb = e4m3_bytes(blk.abs().amax(-1).clamp_min(6.0 * 2.0**-9) / 6.0)
    sc = e4m3_from_bytes(sb)
    q = e2m1_encode((blk / sc.unsqueeze(-1)).clamp(-6.0, 6.0)).reshape(*x.shape[:-1], k)
    return (q[..., 0::2] | (q[..., 1::2] << 4)).contiguous(), sb.contiguous()


# ---------------------------------------------------------------- block FP8 weights
def fp8_block_dequant(w: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """[N, K] E4M3 (uint8 or float8) with f32 [ceil(N/128), ceil(K/128)] scales -> f32.

    glm53/gfx950/kernel.py:35-42: the E4M3 value is widened exactly, the f32 partial
    sum of each 128-k chunk is multiplied by the block's scale.
    """
    if w.dtype == torch.uint8:
        w = w.view(F8)
    n, k = w.shape[-2:]
    s = scale.repeat_interleave(128, -2).repeat_interleave(128, -1)[..., :n, :k]
    return w.float() * s


def split_hi_lo(x: torch.Tensor):
    """The two-plane E4M3 image of bf16 activations used by the FP8 tensor-core path.

    Per 128-k chunk: e = code_ceil(max(amax, 2^-100) / 448); v = x * 2^-(e-127);
    hi = e4m3(v); lo = e4m3(v - hi).  hi + lo reproduces v to 8 significant bits for
    all but the chunk's smallest elements.  Returns (hi, lo, scale f32 [..., K/128]).
    No reference counterpart: the reference widens FP8 weights to bf16 instead
    (glm53/gfx950/kernel.py:823-845); this format keeps the same product in FP8 MMAs.
    """
    g = x.float().reshape(*x.shape[:-1], -1, 128)
    amax = g.abs().amax(-1, keepdim=True)
    code = code_ceil(amax.clamp_min(2.0**-100) / E4M3_MAX)
    sc = exp2_code(code)
    v = g / sc
    hi = e4m3(v)
    lo = e4m3(v - hi)
    return hi.reshape(x.shape), lo.reshape(x.shape), sc.squeeze(-1)
