"""``FfnRunner``: the reference's operator for the FFN-only launch
(``minimax_m31/runner.py:145-167``: ``__call__(attn, residual, weights, slots) -> (out, res_out)``)."""

from __future__ import annotations

import torch

from ..config import LayerConfig
from ..moe import MoeFfn


class FfnRunner:
    def __init__(self, cfg: LayerConfig, weights: dict, device, peer=None, guard=None, deadline_s: float = 5.0):
        self.ffn = MoeFfn(cfg, weights, device, peer=peer, guard=guard, deadline_s=deadline_s)

    def __call__(self, residual: torch.Tensor, slots: torch.Tensor | None = None):
        """Returns (out, res_out): the block's output stream and the residual it was added
        to.  Pad rows (slot < 0) route nowhere and come back unchanged."""
        out = self.ffn(residual, slots)
        return out, residual
