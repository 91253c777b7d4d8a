"""Host-side integer rules of the reference, restated (test infrastructure only).

These are the pieces of the reference that are plain Python and could be run here;
``tests/golden/reference_host.pt`` holds their outputs and ``tests/test_oracle_golden.py``
checks this restatement against them.
"""

from __future__ import annotations

import torch

from . import quant as Q

SEL_CHUNK = 4096  # keys of one select chunk (glm53/gfx950/layout.py:44)
SEL_SLICES = 16  # most CTAs one row's top-k runs on (glm53/gfx950/layout.py:40)


def e8m0_code(scale: torch.Tensor) -> torch.Tensor:
    """E8M0 code of a power-of-two f32 scale: its exponent bits.

    deepseek_v41/gfx950/weights.py:7-15 (raises unless every scale is a power of two).
    """
    bits = scale.float().contiguous().view(torch.int32)
    if not bool(((bits & 0x807FFFFF) == 0).all()):
        raise RuntimeError("needs power-of-two block scales")
    return (bits >> 23).to(torch.uint8)


def mxfp8_exact_32x32(w: torch.Tensor):
    """bf16 [N, K] -> (E4M3 bytes, E8M0 codes [N/32, K/32]) when the weight is exactly
    representable with power-of-two 32 x 32 block scales (deepseek_v41/gfx950/weights.py:18-35)."""
    n, k = w.shape
    blocks = w.float().view(n // 32, 32, k // 32, 32)
    amax = blocks.abs().amax(dim=(1, 3))
    e = torch.ceil(torch.log2(amax.clamp_min(2.0**-126) / 448.0)).clamp(-127, 127)
    scale = torch.exp2(e)[:, None, :, None]
    q = (blocks / scale).to(Q.F8)
    if not torch.equal((q.float() * scale).to(w.dtype), w.view(n // 32, 32, k // 32, 32)):
        raise RuntimeError("the bf16 weight is not MXFP8 at 32 x 32 blocks")
    return q.view(n, k).contiguous().view(torch.uint8), (e + 127).to(torch.uint8).contiguous()


def rope_table_f32(freqs_cis: torch.Tensor) -> torch.Tensor:
    """[positions, 64] f32: 32 cos then 32 sin (deepseek_v41/gfx950/weights.py:38-48)."""
    return torch.cat([freqs_cis.real, freqs_cis.imag], -1).float().contiguous()


def causal_rows(req_to_token, pool, seq_lens, cols, slot_mapping, query_len: int, is_verify: bool,
                max_context_len: int):
    """Per-row block table and key count of a decode / verify step.

    minimax_m3/metadata.py:7-42: row j of a request sees prefix + j + 1 keys (clamped
    to the context limit); rows whose slot is <= 0 are pads: zero keys, zero table.
    """
    n = slot_mapping.numel()
    token = torch.arange(n, dtype=torch.int64)
    request = token // query_len
    rows = pool[request].long()
    table = req_to_token[rows[:, None], cols[None, :]] // 128
    lengths = seq_lens[request]
    if is_verify:
        lengths = (lengths + (token % query_len + 1).to(lengths.dtype)).clamp(max=max_context_len)
    pad = slot_mapping[:n] <= 0
    lengths = lengths.masked_fill(pad, 0)
    table = table.masked_fill(pad[:, None], 0)
    return table.to(torch.int32), lengths.to(torch.int32)


def select_slices(bound: int):
    """(slices, chunks per slice) of a row of ``bound`` keys whose top-k runs on several
    CTAs: runs of whole 4096-key chunks in position order (glm53/gfx950/layout.py:47-53)."""
    chunks = -(-bound // SEL_CHUNK)
    per = -(-chunks // SEL_SLICES)
    return -(-chunks // per), per
