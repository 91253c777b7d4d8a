"""Sparse MLA decode attention operator (BASELINE config 2; the attention stage of the layer).

Reference counterpart: the split / merge stages of ``glm53/gfx950/kernel.py:3638-4075``
behind ``Glm53LayerOp.launch`` (``glm53/gfx950/runner.py:240-321``).  Inputs are what
SGLang owns: the paged FP8 latent cache and the selected global KV slots of each row.
"""

from __future__ import annotations

import torch

from . import _lib as L
from . import ops
from .config import KV_DIM, KV_PAGE_BYTES


class SparseMlaOp:
    def __init__(self, heads: int, topk: int, device, max_rows: int = L.MAX_ROWS, sm_scale: float | None = None):
        lib = L.load()
        self.heads, self.topk, self.dev = heads, topk, device
        self.sm_scale = sm_scale if sm_scale is not None else (128 + 64) ** -0.5
        nbytes = lib.mono_sparse_mla_scratch_bytes(max_rows, heads, topk)
        self.scratch = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.out = torch.zeros(max_rows, heads, 512, dtype=torch.bfloat16, device=device)
        self.max_rows = max_rows

    def __call__(self, q: torch.Tensor, kv_pages: torch.Tensor, topk_slots: torch.Tensor, staged=None) -> torch.Tensor:
        """``staged``: an ``ops.ActBuf`` with one 512-value segment per head; the merge then also writes
        every head's output there as the W_UV GEMV's activation set (no separate staging launch)."""
        rows = q.shape[0]
        if not 1 <= rows <= self.max_rows:
            raise ValueError(f"q: {rows} rows, the op was built for 1..{self.max_rows}")
        ops.require(q, "q", torch.bfloat16, (rows, self.heads, KV_DIM))
        ops.require(kv_pages, "kv_pages", torch.uint8)
        if kv_pages.dim() != 2 or kv_pages.shape[1] != KV_PAGE_BYTES:
            raise ValueError(f"kv_pages: shape {tuple(kv_pages.shape)}, needs [pages, {KV_PAGE_BYTES}]")
        ops.require(topk_slots, "topk_slots", torch.int32)
        if topk_slots.dim() != 2 or topk_slots.shape[0] < rows or topk_slots.shape[1] < self.topk:
            raise ValueError(f"topk_slots: shape {tuple(topk_slots.shape)}, needs [>= {rows}, >= {self.topk}]")
        ops.sparse_mla(q, kv_pages, topk_slots, self.out, self.scratch, self.sm_scale, self.topk, staged=staged)
        return self.out[:rows]
