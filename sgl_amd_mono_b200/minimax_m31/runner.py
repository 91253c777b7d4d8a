"""``FfnRunner``: the reference's operator for the launch that starts after attention
(``minimax_m31/runner.py:145-167``: ``__call__(attn, residual, weights, slots) -> (out, res_out)``): o_proj of this
rank's attention output, the attention all-reduce and residual add, then the MoE block with its own all-reduce."""

from __future__ import annotations

import torch

from .. import _lib as L
from .. import ops
from ..config import LayerConfig
from ..moe import MoeFfn


class FfnRunner:
    def __init__(self, cfg: LayerConfig, weights: dict, device, peer=None, guard=None, deadline_s: float = 5.0, copies=None,
                 layer: int = 0):
        L.load()
        self.cfg, self.w, self.peer, self.layer, self.deadline_s = cfg, weights, peer, layer, deadline_s
        self.guard = guard if guard is not None else torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=device)
        self.ffn = MoeFfn(cfg, weights, device, peer=peer, guard=self.guard, site=2 * layer + 1, deadline_s=deadline_s,
                          copies=copies, layer=layer)
        self.attn_k = 0
        if "o_proj" in weights:  # the seam: o_proj (block-FP8) of this rank's attention output
            wo = weights["o_proj"]
            self.attn_k = wo.shape[1]
            h = cfg.hidden
            self.oq = ops.ActBuf(L.ACT_HILO, self.attn_k, device)
            st, ns = ops.plan_split(-(-self.attn_k // 128), -(-h // 128), L.W_FP8)
            self.ns_o = ns
            self.o_p = torch.zeros(ns, L.MAX_ROWS, h, dtype=torch.float32, device=device)
            self.o_g = ops.Gemv(L.W_FP8, self.guard, deadline_s)
            self.o_g.add("o_proj", wo, self.oq, self.o_p, wscale=weights["o_proj_s"], split_tiles=st, nsplit=ns)
            self.res_out = torch.zeros(L.MAX_ROWS, h, dtype=torch.bfloat16, device=device)

    def __call__(self, attn: torch.Tensor | None, residual: torch.Tensor, weights=None, slots: torch.Tensor | None = None):
        """``attn``: this rank's attention output bf16 ``[S, attn_k]`` (o_proj's input) or None for the block alone;
        ``weights``: the layer's tensors, which must be the ones the runner was built over (they are bound at build,
        ``minimax_m31/runner.py:88-123``); ``slots``: the step's slot mapping, a negative slot = a pad row (joins no
        expert, zero MoE output).  Returns (out, res_out): the reduced output stream and the residual after attention."""
        if weights is not None and weights is not self.w:
            raise ValueError("weights: the runner is bound to the tensors it was built over")
        rows = residual.shape[0]
        ops.require(residual, "residual", torch.bfloat16, (rows, self.cfg.hidden))
        if attn is None:
            return self.ffn(residual, slots), residual
        if not self.attn_k:
            raise ValueError("attn: the runner was built without an o_proj weight")
        ops.require(attn, "attn", torch.bfloat16, (rows, self.attn_k))
        ops.act_prep(rows, self.attn_k, self.oq, src_bf16=attn, round_bf16=False)
        self.o_g.launch(rows)
        seam = ops.PendingReduce(rows, self.cfg.hidden, self.o_p, self.ns_o, self.res_out, residual, slots, self.peer,
                                 2 * self.layer, self.guard, self.deadline_s)
        out = self.ffn(None, slots, pending=seam)  # the attention all-reduce runs inside the MoE half's norm launch
        return out, self.res_out[:rows]
