"""The tail launch: final RMSNorm and this rank's rows of the bf16 LM head.

Reference counterpart: ``glm53_flash/gfx950/kernel.py:3626-3770`` (``run_head``) behind
``FlashHeadOp`` (``glm53_flash/gfx950/runner.py:504-550``); golden model
``glm53_flash/check.py:284-302``.  The weight (1.06 GB at vocab 129280 x hidden 4096) is
streamed once by the bf16 GEMV job.  Without peers the logits come back as f32
``[rows, vocab]`` (up to 8 rows straight from the GEMV; wider steps split K, and a gather
launch adds the splits in order).  With peers every rank pushes its bf16-rounded share into
every rank's logits region and gathers f32 ``[rows, vocab]`` of the whole vocabulary, the
same bits on every rank (``kernel.py:3700-3770``).
"""

from __future__ import annotations

import torch

from . import _lib as L
from . import ops


class LmHeadOp:
    def __init__(self, hidden: int, w_head: torch.Tensor, final_norm: torch.Tensor, eps: float, device, guard=None,
                 peer=None, site: int = 254, deadline_s: float = 5.0):
        L.load()
        ops.require(w_head, "lm_head", torch.bfloat16)
        if w_head.dim() != 2 or w_head.shape[1] != hidden:
            raise ValueError(f"lm_head: shape {tuple(w_head.shape)}, needs [vocab / tp, {hidden}]")
        self.hidden, self.w, self.g, self.eps = hidden, w_head, final_norm, eps
        self.vocab_local = w_head.shape[0]
        self.guard = guard if guard is not None else torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=device)
        self.x = ops.ActBuf(L.ACT_BF16, hidden, device)
        k_tiles = -(-hidden * 2 // 128)
        self.gemv = {}
        self.logits = torch.zeros(1, L.MAX_ROWS, self.vocab_local, dtype=torch.float32, device=device)
        # up to 8 rows the whole K fits one activation slot: one pass, no partial sums
        for wide in (False, True):
            cap = 32 if wide else 64
            st, ns = ops.plan_split(k_tiles, -(-self.vocab_local // 128), L.W_BF16, cap=cap)
            buf = self.logits if ns == 1 else torch.zeros(ns, L.MAX_ROWS, self.vocab_local, dtype=torch.float32, device=device)
            g = ops.Gemv(L.W_BF16, self.guard, deadline_s)
            g.add("lm_head", w_head, self.x, buf, split_tiles=st, nsplit=ns)
            self.gemv[wide] = (g, buf, ns)
        self.peer, self.site, self.deadline_s = peer, site, deadline_s
        self.world = peer.world if peer is not None else 1
        self.gathered = torch.zeros(L.MAX_ROWS, self.world * self.vocab_local, dtype=torch.float32, device=device)

    def __call__(self, h: torch.Tensor | None, pending=None) -> torch.Tensor:
        """``pending``: the last layer's final reduction, left for this launch's norm staging to run."""
        if pending is not None:
            h = pending.out[: pending.rows]
        rows = h.shape[0]
        ops.require(h, "h", torch.bfloat16, (rows, self.hidden))
        if pending is not None:
            ops.reduce_norm(pending, self.x, gamma=self.g, eps=self.eps)
        else:
            ops.act_prep(rows, self.hidden, self.x, src_bf16=h, gamma=self.g, eps=self.eps)
        g, buf, ns = self.gemv[rows > 8]
        g.launch(rows)
        if ns == 1 and self.world == 1:
            return buf[0, :rows]
        ops.logits_gather(rows, self.vocab_local, buf, ns, self.gathered, peer=self.peer, site=self.site,
                          guard=self.guard, deadline_s=self.deadline_s)
        return self.gathered[:rows]
