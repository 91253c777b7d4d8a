"""A whole decode step under one CUDA graph: every layer's launches, the draft stage and the tail.

Reference counterparts: the routed forward of a covered model (``deepseek_v41/spec.py:938-964``,
``_launch`` ``:709-772``), whose Python is captured once into SGLang's decode graph so that a
replay re-executes device work only (``glm53/spec.py:467-496``); the draft model's stage
(``deepseek_v41/draft.py:175-209``); the tail launch (``glm53_flash/gfx950/runner.py:504-550``).
Per-step values (slots, positions, page table, the input rows) live in fixed-address tensors
that the caller overwrites before a replay; the epoch word advances on the device.
"""

from __future__ import annotations

import torch

from . import _lib as L
from . import ops
from .config import LayerConfig
from .layer import MlaLayerOp, StepTables
from .tail import LmHeadOp


class DecoderStack:
    def __init__(self, cfg: LayerConfig, layer_weights: list[dict], device, max_ctx: int, peer=None,
                 draft_weights: dict | None = None, deadline_s: float = 5.0):
        self.cfg, self.dev, self.peer = cfg, device, peer
        self.guard = peer.guard if peer is not None else torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=device)
        self.layers = [MlaLayerOp(cfg, w, device, max_ctx, peer=peer, guard=self.guard, layer=i, deadline_s=deadline_s)
                       for i, w in enumerate(layer_weights)]
        self.draft = None
        if draft_weights is not None:
            self.draft = MlaLayerOp(cfg, draft_weights, device, max_ctx, peer=peer, guard=self.guard,
                                    layer=len(layer_weights), deadline_s=deadline_s)
        last = layer_weights[-1]
        # with a logits region in the peer buffer the tail gathers the whole vocabulary on every rank
        head_peer = peer if peer is not None and getattr(peer, "logits_table", None) is not None else None
        self.head = LmHeadOp(cfg.hidden, last["lm_head"], last["final_norm"], cfg.eps, device, guard=self.guard,
                             peer=head_peer, site=254, deadline_s=deadline_s) if "lm_head" in last else None
        self.graph = None

    def count_launches(self, h: torch.Tensor, tables, draft_tables=None, draft_rows: int = 0) -> int:
        """Kernels one eager step launches (the library counts its own launches; a graph replay launches none)."""
        lib = L.load()
        before = lib.mono_launch_count()
        self.step(h, tables, draft_tables, draft_rows)
        return int(lib.mono_launch_count() - before)

    def step(self, h: torch.Tensor, tables: list[StepTables], draft_tables: StepTables | None = None,
             draft_rows: int = 0):
        """One decode / verify step: returns (hidden rows, f32 logits or None)."""
        if self.draft is not None and draft_tables is not None:
            self.draft_out = self.draft.launch(h[:draft_rows] if draft_rows else h, draft_tables)
        x = self.run_layers(h, tables)
        logits = None
        if self.head is not None:
            if isinstance(x, ops.PendingReduce):
                logits = self.head(None, pending=x)
                x = x.out[: x.rows]
            else:
                logits = self.head(x)
        ops.epoch_advance(self.guard)
        return x, logits

    def run_layers(self, h: torch.Tensor, tables: list[StepTables]):
        """The layers in order.  A layer's last reduction (MoE all-reduce + residual) runs inside the next layer's
        input norm launch, the last layer's inside the tail's; without a tail it is launched on its own."""
        x, pend = h, None
        fuse = all(op.fuse_reduce and op.ffn is not None for op in self.layers)
        for i, (op, t) in enumerate(zip(self.layers, tables)):
            last = i == len(self.layers) - 1
            x = op.launch(None if pend is not None else x, t, pending=pend, defer=fuse and (not last or self.head is not None))
            pend = x if isinstance(x, ops.PendingReduce) else None
        return x

    def capture(self, h: torch.Tensor, tables, draft_tables=None, draft_rows: int = 0):
        """Runs the step once eagerly, then captures it; ``replay()`` re-runs the device work."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.step(h, tables, draft_tables, draft_rows)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self.out = self.step(h, tables, draft_tables, draft_rows)
        torch.cuda.current_stream().wait_stream(s)
        self.graph = g
        return self.out

    def replay(self):
        self.graph.replay()
        return self.out
