"""Host-side number-format helpers of the library (torch ops; CPU or CUDA tensors).

Used to build synthetic checkpoints in SGLang's loaded layouts and by the weight
binding code.  The device kernels carry their own implementations of the activation
formats; these are for tensors that exist before a launch.

Rules follow the reference's device code:
  * E8M0 "round-up" code of a positive f32: exponent + (mantissa != 0)
    (``common/mx.py:27-39``).
  * MXFP4 weights: one E8M0 code per 32 values along K, sc = pow2_ceil(max(amax,
    6 * 2^-126) / 6), E2M1 by round-to-nearest-even
    (``deepseek_v4/gfx950/kernels/stages/indexer.py:143-151``); even index in the low
    nibble (``test/kernels/deepseek_v41/check_ffn.py:107-115``).
  * block-FP8 weights: E4M3 bytes with f32 128 x 128 scales
    (``glm53/gfx950/kernel.py:35-42``).
  * NVFP4 weights (the expert format of ``minimax_m31/spec.py:117-121``): E2M1 values, an E4M3 scale per 16
    along K, an f32 scale per matrix.
"""

from __future__ import annotations

import torch

F8 = torch.float8_e4m3fn


def code_ceil(v: torch.Tensor) -> torch.Tensor:
    bits = v.float().contiguous().view(torch.int32)
    return ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)


def e2m1_encode(v: torch.Tensor) -> torch.Tensor:
    a = v.float().abs()
    code = (
        (a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
        + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8)
        + (a > 5.0).to(torch.uint8)
    )
    return code | (torch.signbit(v.float()).to(torch.uint8) << 3)


def mxfp4_quant(w: torch.Tensor):
    """[..., N, K] float -> (packed uint8 [..., N, K/2], E8M0 uint8 [..., N, K/32])."""
    k = w.shape[-1]
    g = w.float().reshape(*w.shape[:-1], k // 32, 32)
    amax = g.abs().amax(-1, keepdim=True)
    code = code_ceil(amax.clamp_min(6.0 * 2.0**-126) / 6.0).clamp(0, 254)
    sc = torch.exp2(code.float() - 127.0)
    q = e2m1_encode((g / sc).clamp(-6.0, 6.0)).reshape(*w.shape[:-1], k)
    packed = q[..., 0::2] | (q[..., 1::2] << 4)
    return packed.contiguous(), code.squeeze(-1).to(torch.uint8).contiguous()


def nvfp4_quant(w: torch.Tensor):
    """[E, N, K] float -> (packed uint8 [E, N, K/2], E4M3 scale bytes uint8 [E, N, K/16], f32 tensor scales [E]).

    NVIDIA's published NVFP4 recipe: tensor scale = amax / (6 * 448) per matrix, block scale =
    E4M3(amax(block of 16) / 6 / tensor scale), value = E2M1(v / (block scale * tensor scale)), round to nearest
    even; even index in the low nibble.
    """
    k = w.shape[-1]
    wf = w.float()
    g = (wf.abs().amax((-2, -1)) / (6.0 * 448.0)).clamp_min(2.0**-100)
    blk = wf.reshape(*wf.shape[:-1], k // 16, 16)
    sb = (blk.abs().amax(-1) / 6.0 / g[:, None, None]).clamp(0.0, 448.0).to(F8)
    sc = sb.float() * g[:, None, None]
    q = e2m1_encode((blk / sc.clamp_min(2.0**-120).unsqueeze(-1)).clamp(-6.0, 6.0)).reshape(*wf.shape[:-1], k)
    q = torch.where((sc == 0).repeat_interleave(16, -1), torch.zeros_like(q), q)
    packed = q[..., 0::2] | (q[..., 1::2] << 4)
    return packed.contiguous(), sb.view(torch.uint8).contiguous(), g.float().contiguous()


def random_fp8_block(n: int, k: int, gen: torch.Generator, device, lead: tuple = ()):
    """Random block-FP8 weight: randn -> E4M3 bytes, scales (0.5 + U) * K^-0.5.

    The value recipe of ``test/kernels/glm53/check_layer.py:56-64``.
    """
    w = torch.randn(*lead, n, k, generator=gen, device=device).to(F8).view(torch.uint8)
    s = (0.5 + torch.rand(*lead, -(-n // 128), -(-k // 128), generator=gen, device=device)) * k**-0.5
    return w, s.float().contiguous()


def fp8_block_quant(w: torch.Tensor):
    """Quantise a float [N, K] weight to block-FP8 (amax / 448 per 128 x 128 block)."""
    n, k = w.shape
    pn, pk = -(-n // 128) * 128, -(-k // 128) * 128
    wp = torch.zeros(pn, pk, device=w.device)
    wp[:n, :k] = w.float()
    blk = wp.reshape(pn // 128, 128, pk // 128, 128)
    amax = blk.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    s = amax / 448.0
    q = (blk / s[:, None, :, None]).clamp(-448, 448).to(F8).view(torch.uint8)
    return q.reshape(pn, pk)[:n, :k].contiguous(), s.contiguous()
