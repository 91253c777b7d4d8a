"""Host runner of one MLA + lightning-indexer + MoE decoder layer.

Reference counterpart: ``Glm53LayerOp.launch(h, caches, cos, sin, step) -> x_out``
(``glm53/gfx950/runner.py:240-321``) and ``Glm53Runtime`` (scratch, peer buffer and
guard words owned by the runner, allocated at build, ``runner.py:184-210``).  The
stage order is the reference kernel's (``glm53/gfx950/kernel.py:171``): input norm,
q_a|kv_a (+ index key, head weights), norms + RoPE + cache writes, q_b (+ index q),
absorb, index scores, exact top-k, sparse MLA, W_UV, o_proj, all-reduce + residual,
then the MoE half (``moe.MoeFfn``).
"""

from __future__ import annotations

import os

from dataclasses import dataclass

import torch

from . import _lib as L
from . import ops
from .attention import SparseMlaOp
from .config import IDX_PAGE_BYTES, KV_DIM, KV_PAGE_BYTES, LayerConfig
from .moe import MoeFfn


@dataclass
class StepTables:
    """Fixed-address tensors a decode step reads (``glm53/spec.py:467-496``)."""

    positions: torch.Tensor  # i64 [rows]
    slots: torch.Tensor  # i64 [rows]; < 0 = pad row
    page_table: torch.Tensor  # i32 [rows, pages]
    kv_pages: torch.Tensor  # u8 [pages, KV_PAGE_BYTES]
    idx_pages: torch.Tensor | None  # u8 [pages, IDX_PAGE_BYTES]
    cos: torch.Tensor  # bf16 [max_pos, 32]
    sin: torch.Tensor


class MlaLayerOp:
    def __init__(self, cfg: LayerConfig, w: dict, device, max_ctx: int, peer=None, guard=None, layer: int = 0,
                 deadline_s: float = 5.0, max_rows: int = L.MAX_ROWS, copies: dict | None = None):
        L.load()
        if cfg.nope != 128 or cfg.v_head != 128 or cfg.rope != 64 or cfg.kv_lora != 512:
            raise ValueError("the MLA kernels are built for nope 128, v 128, rope 64, kv_lora 512")
        self.cfg, self.w, self.dev, self.peer, self.layer = cfg, w, device, peer, layer
        self.deadline_s = deadline_s
        self.guard = guard if guard is not None else torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=device)
        # the index path (index queries + head weights, scores, top-k) runs on a second stream, forked after the q_b
        # projection and joined before the attention (a fork / join that a CUDA graph capture records too), beside
        # the W_UK absorb of the heads on the main one.  A high-priority stream: the index path is the longer of the
        # two branches, and its small launches should not queue behind the head blocks of the main branch
        self._side = torch.cuda.Stream(device=device, priority=-1) if os.environ.get("MONO_SIDE_STREAM", "1") == "1" else None
        # Weights towards L2 ahead of the stage that streams them (MONO_L2_PREFETCH=1; off by default): at the layer's
        # start q_b + index q (and W_UK / W_UV) while q_a | kv_a runs; when the attention starts o_proj (as much as
        # fits beside the attention's own working set) and the router.  Measured slower (config 3: 655 against 637 us
        # at TP 1, 244 against 238 us for a TP 8 shard): the stages in between live on memory round trips, and their
        # loads queue behind the prefetch traffic (q_a | kv_a 22 against 16 us, the attention merge 33 against 25 us).
        self._pf_stream = self._pf_front = self._pf_back = None
        if os.environ.get("MONO_L2_PREFETCH", "0") == "1":
            lim = int(os.environ.get("MONO_L2_PREFETCH_MB", "72")) << 20
            self._pf_front = ops.l2_prefetch_args([w["q_b"], w.get("idx_wq_b") if cfg.index_heads else None, w["kv_b"]], lim)
            self._pf_back = ops.l2_prefetch_args([w["o_proj"], w.get("router")], lim)
            self._pf_stream = torch.cuda.Stream(device=device)
            self._ev_pf = torch.cuda.Event()
            self._ev_pf_done = torch.cuda.Event()
        self._ev_fork, self._ev_join, self._ev_idxq = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
        self.head_after_idxq = os.environ.get("MONO_HEAD_AFTER_IDXQ", "1") != "0"
        # The index head weights depend on the normed input only and used to run beside mla_mid on the index branch.
        # Stamps showed what that costs: mla_mid's loads of the partial sums took 7 us with that launch running beside
        # it and 1.8 us alone (every CTA's loads completing at the same instant: launches that end on one branch stall
        # the loads in flight on the other).  They now run on the index branch after the index queries
        # (MONO_IDXW_LATE=0: the old place): 8 us off the front, 5 us onto the index branch.
        self.idxw_late = os.environ.get("MONO_IDXW_LATE", "1") != "0"
        h, hl, ql, ih = cfg.hidden, cfg.heads_local, cfg.q_lora, cfg.index_heads
        R = L.MAX_ROWS
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)  # noqa: E731
        self.x = ops.ActBuf(L.ACT_HILO, h, device)
        self.xbf = z(R, h, dt=torch.bfloat16)
        # ---- launch A: q_a|kv_a and the index-key projection
        self.gA = ops.Gemv(L.W_FP8, self.guard, deadline_s)
        kt = -(-h // 128)
        stA, nsA = ops.plan_split(kt, -(-(ql + KV_DIM) // 128) + (1 if ih else 0), L.W_FP8)
        self.nsA = nsA
        self.qkv_p = z(nsA, R, ql + KV_DIM)
        self.gA.add("qkv_a", w["qkv_a"], self.x, self.qkv_p, wscale=w["qkv_a_s"], split_tiles=stA, nsplit=nsA)
        self.ik_p = self.idx_w = self.iq_p = self.idx_q = self.scores = None
        if ih:
            self.ik_p = z(nsA, R, 128)
            self.gA.add("idx_wk", w["idx_wk"], self.x, self.ik_p, wscale=w["idx_wk_s"], split_tiles=stA, nsplit=nsA)
            self.idx_w = z(R, ih)
            self.ik_out = z(R, 128)
            self.idx_q = z(R, ih, 128, dt=torch.bfloat16)
            self.max_ctx = -(-max_ctx // 128) * 128
            self.scores = z(R, self.max_ctx)
        self.qa = ops.ActBuf(L.ACT_HILO, ql, device)
        self.kv_out = z(R, KV_DIM, dt=torch.bfloat16)
        # ---- launch B: q_b and the index-query projection
        self.gB = ops.Gemv(L.W_FP8, self.guard, deadline_s)
        ktb = -(-ql // 128)
        stB, nsB = ops.plan_split(ktb, -(-hl * 192 // 128) + (ih if ih else 0), L.W_FP8)
        self.nsB = nsB
        self.qb_p = z(nsB, R, hl * 192)
        self.gB.add("q_b", w["q_b"], self.qa, self.qb_p, wscale=w["q_b_s"], split_tiles=stB, nsplit=nsB)
        if ih:
            self.iq_p = z(nsB, R, ih * 128)
            self.gB.add("idx_wq_b", w["idx_wq_b"], self.qa, self.iq_p, wscale=w["idx_wq_b_s"], split_tiles=stB, nsplit=nsB)
        self.q_full = z(R, hl, KV_DIM, dt=torch.bfloat16)
        # without an indexer every cached key is attended: the "selection" is the whole context, or with a window
        # (the draft model: deepseek_v41/draft.py:34-35) the last `window` keys of each row
        self.window = 0 if ih else min(cfg.window, max_ctx)
        self.topk = cfg.index_topk if ih else (-(-self.window // 64) * 64 if self.window else -(-max_ctx // 64) * 64)
        if self.window:
            self._wcols = torch.arange(self.topk, dtype=torch.int64, device=device)
        if not ih:
            self.max_ctx = -(-max_ctx // 64) * 64 if self.window else self.topk
            self.scores = z(R, 128)
        self.topk_slots = torch.full((R, self.topk), -1, dtype=torch.int32, device=device)
        self.topk_pos = torch.full((R, self.topk), -1, dtype=torch.int32, device=device)
        self.mla_staged = os.environ.get("MONO_MLA_STAGED", "1") != "0"
        self.idxq_fused = (os.environ.get("MONO_IDXQ_FUSED", "0") != "0" and os.environ.get("MONO_INDEX_SCORE_TC", "1") != "0")
        self.attn = SparseMlaOp(hl, self.topk, device, max_rows=R, sm_scale=(cfg.nope + cfg.rope) ** -0.5)
        # ---- W_UV (per head) and o_proj
        self.lat = ops.ActBuf(L.ACT_HILO, 512, device, segs=hl)
        self.uv_p = z(1, R, hl * 128)
        self.gUV = ops.Gemv(L.W_FP8, self.guard, deadline_s)
        self.o = ops.ActBuf(L.ACT_HILO, hl * 128, device)
        # on the tcgen05 consumer the W_UV job can write its output straight into o_proj's activation planes
        # (MONO_UV_STAGED=1 / 0).  Measured on config 3: 6 us faster per layer with 128 local heads (128 CTAs
        # share the staging), 3.5 / 5 / 6 us slower with 64 / 32 / 16 (the staging lengthens the one task each
        # of those CTAs runs, and a staging launch of 2.4 us in between costs less than that): the default
        # follows the head count
        lib = L.load()
        tc_on = lib.mono_set_gemv_tcgen05(1)
        lib.mono_set_gemv_tcgen05(tc_on)
        self.uv_staged = bool(tc_on) and os.environ.get("MONO_UV_STAGED", "1" if hl >= 128 else "0") != "0"
        self.gUV.add("kv_b(W_UV)", w["kv_b"].view(hl, 256, 512), self.lat, self.uv_p, wscale=w["kv_b_s"].view(hl, 2, 4),
                     n_rows=128, row_off=128, rb_per_mat=1, n_mats=hl, act_per_mat=True, split_tiles=4, nsplit=1,
                     stage=self.o if self.uv_staged else None)
        kto = -(-hl * 128 // 128)
        stO, nsO = ops.plan_split(kto, -(-h // 128), L.W_FP8)
        self.nsO = nsO
        self.o_p = z(nsO, R, h)
        self.gO = ops.Gemv(L.W_FP8, self.guard, deadline_s)
        self.gO.add("o_proj", w["o_proj"], self.o, self.o_p, wscale=w["o_proj_s"], split_tiles=stO, nsplit=nsO)
        self.h1 = z(R, h, dt=torch.bfloat16)
        self.ffn = MoeFfn(cfg, w, device, max_rows=max_rows, peer=peer, guard=self.guard, site=2 * layer + 1,
                          deadline_s=deadline_s, copies=copies, layer=layer) if cfg.n_experts else None
        self._iargs = None
        # MONO_FUSE_REDUCE=0: every reduction (+ all-reduce + residual) is a launch of its own instead of running inside
        # the norm staging launch that consumes it (same bits either way)
        self.fuse_reduce = os.environ.get("MONO_FUSE_REDUCE", "1") != "0"

    def _prefetch(self, args) -> None:
        """Issues an L2 prefetch launch on its own branch, forked from here; the branch is joined at the layer's end."""
        if args is None or self._pf_stream is None:
            return
        main = torch.cuda.current_stream()
        self._ev_pf.record(main)
        self._pf_stream.wait_event(self._ev_pf)
        with torch.cuda.stream(self._pf_stream):
            ops.l2_prefetch(args)
            self._ev_pf_done.record(self._pf_stream)
        self._pf_pending = True

    def _join_prefetch(self) -> None:
        if getattr(self, "_pf_pending", False):
            torch.cuda.current_stream().wait_event(self._ev_pf_done)
            self._pf_pending = False

    def _window_slots(self, rows: int, step: StepTables) -> None:
        """The step's selection for window-only attention: row r takes positions pos_r - window + 1 .. pos_r (those
        that exist), in order, as global KV slots; pad rows take none.  A handful of fixed-shape torch ops, captured
        with the step like the reference's step tables (``glm53/spec.py:467-496``)."""
        pos = step.positions[:rows, None] - (self.window - 1) + self._wcols[None, :]
        ok = (pos >= 0) & (self._wcols[None, :] < self.window) & (step.slots[:rows, None] >= 0)
        p = pos.clamp(min=0)
        slot = step.page_table[:rows].gather(1, (p // 64).clamp(max=step.page_table.shape[1] - 1)).long() * 64 + p % 64
        self.topk_slots[:rows] = torch.where(ok, slot, torch.full_like(slot, -1)).to(torch.int32)

    def launch(self, h: torch.Tensor | None, step: StepTables, pending=None, defer: bool = False):
        """``pending`` (``ops.PendingReduce``): the layer before this one left its last reduction to this layer's input
        norm launch; ``h`` is then not read.  ``defer``: this layer's last reduction is returned unlaunched for the
        next stage.  Without either, and with ``MONO_FUSE_REDUCE=0``, every reduction is a launch of its own."""
        cfg, w = self.cfg, self.w
        if pending is not None:
            h = pending.out[: pending.rows]
        rows = h.shape[0]
        if not 1 <= rows <= L.MAX_ROWS:
            raise ValueError(f"h: {rows} rows, the launch serves 1..{L.MAX_ROWS}")
        ops.require(h, "h", torch.bfloat16, (rows, cfg.hidden))
        ops.require(step.positions, "step.positions", torch.int64, (rows,))
        ops.require(step.slots, "step.slots", torch.int64, (rows,))
        ops.require(step.page_table, "step.page_table", torch.int32)
        ops.require(step.kv_pages, "step.kv_pages", torch.uint8)
        if step.kv_pages.shape[-1] != KV_PAGE_BYTES:
            raise ValueError(f"step.kv_pages: page of {step.kv_pages.shape[-1]} bytes, needs {KV_PAGE_BYTES}")
        ih, hl = cfg.index_heads, cfg.heads_local
        if ih:
            ops.require(step.idx_pages, "step.idx_pages", torch.uint8)
            if step.idx_pages.shape[-1] != IDX_PAGE_BYTES:
                raise ValueError(f"step.idx_pages: page of {step.idx_pages.shape[-1]} bytes, needs {IDX_PAGE_BYTES}")
        if step.page_table.shape[1] * 64 > self.max_ctx:
            raise ValueError(f"step.page_table: {step.page_table.shape[1]} pages exceed the built context {self.max_ctx}")
        self._prefetch(self._pf_front)
        if pending is not None:
            ops.reduce_norm(pending, self.x, gamma=w["input_norm"], eps=cfg.eps, out_bf16=self.xbf)
        else:
            ops.act_prep(rows, cfg.hidden, self.x, src_bf16=h, gamma=w["input_norm"], eps=cfg.eps, out_bf16=self.xbf)
        self.gA.launch(rows)
        idxw_late = ih and self._side is not None and self.idxw_late
        if idxw_late:
            pass  # the index head weights run on the index branch, after the index queries (below)
        elif ih and self._side is not None:
            main = torch.cuda.current_stream()
            self._ev_fork.record(main)
            self._side.wait_event(self._ev_fork)
            with torch.cuda.stream(self._side):
                ops.rowdot(rows, w["idx_wproj"], self.xbf, self.idx_w, out_scale=(ih**-0.5) * (128**-0.5))
        elif ih:
            ops.rowdot(rows, w["idx_wproj"], self.xbf, self.idx_w, out_scale=(ih**-0.5) * (128**-0.5))
        ops.mla_mid(rows, cfg.q_lora, self.qkv_p, self.nsA, w, cfg.eps, step.cos, step.sin, step.positions, step.slots,
                    self.qa, step.kv_pages, step.idx_pages, self.kv_out, ik=self.ik_p, ik_nsum=self.nsA,
                    ik_out=self.ik_out if ih else None)
        self.gB.launch(rows)
        # MONO_IDXQ_FUSED=1: the score launch makes the index queries itself from the q_b partial sums instead of
        # a query launch before it.  Same bits, but measured 4 us (TP 8 shard) to 9 us (TP 1) slower per layer:
        # every score CTA repeats the 64 heads' sums, rotations and Hadamard butterflies.  Off by default.
        fused_q = bool(ih) and self.idxq_fused and self._side is not None
        ia = ops.index_args(rows, max(ih, 1), self.topk, self.idx_q, self.idx_w, step.idx_pages, step.page_table,
                            step.positions, step.slots, self.scores, self.topk_slots, self.topk_pos,
                            **(dict(iq=self.iq_p, iq_nsum=self.nsB, cos=step.cos, sin=step.sin) if fused_q else {}))
        if ih and self._side is not None:
            # index queries -> scores -> top-k on the side stream (behind the head weights already queued
            # there), the W_UK absorb of the heads on the main one; joined before the attention
            main = torch.cuda.current_stream()
            self._ev_fork.record(main)
            self._side.wait_event(self._ev_fork)
            with torch.cuda.stream(self._side):
                if not fused_q and idxw_late:
                    # the index queries and the index head weights in one launch
                    ops.index_prep(rows, ih, self.iq_p, self.nsB, step.cos, step.sin, step.positions, self.idx_q, w["idx_wproj"],
                                   self.xbf, self.idx_w, (ih**-0.5) * (128**-0.5))
                    self._ev_idxq.record(self._side)
                elif not fused_q:
                    ops.q_post(rows, 0, self.qb_p, self.nsB, w["kv_b"], w["kv_b_s"], step.cos, step.sin, step.positions,
                               self.q_full, ih, self.iq_p, self.nsB, self.idx_q)
                    self._ev_idxq.record(self._side)
                elif idxw_late:
                    ops.rowdot(rows, w["idx_wproj"], self.xbf, self.idx_w, out_scale=(ih**-0.5) * (128**-0.5))
                ops.index_score(ia)
                ops.index_topk(ia)
                self._ev_join.record(self._side)
            if not fused_q and self.head_after_idxq:
                # the heads' blocks (8 per head, all resident at once) would fill every SM while they wait for
                # q_b, and the index queries, which the longer branch starts with, would queue behind them
                main.wait_event(self._ev_idxq)
            ops.q_post(rows, hl, self.qb_p, self.nsB, w["kv_b"], w["kv_b_s"], step.cos, step.sin, step.positions,
                       self.q_full, 0, None, 0, None)
            main.wait_event(self._ev_join)
        else:
            ops.q_post(rows, hl, self.qb_p, self.nsB, w["kv_b"], w["kv_b_s"], step.cos, step.sin, step.positions,
                       self.q_full, ih, self.iq_p, self.nsB, self.idx_q)
            if ih:
                ops.index_score(ia)
            if self.window:
                self._window_slots(rows, step)
            else:
                ops.index_topk(ia)  # rows with at most topk keys keep every key in order
        self._prefetch(self._pf_back)
        # the merge of the attention splits also stages every head's output for the W_UV GEMV
        # (MONO_MLA_STAGED=0: a staging launch of its own)
        if self.mla_staged:
            self.attn(self.q_full[:rows], step.kv_pages, self.topk_slots, staged=self.lat)
        else:
            lat = self.attn(self.q_full[:rows], step.kv_pages, self.topk_slots)
            ops.act_prep_heads(rows, hl, 512, self.lat, src_bf16=lat)
        self.gUV.launch(rows)
        if not self.uv_staged:
            ops.act_prep(rows, hl * 128, self.o, src_f32=self.uv_p, nsum=1)
        self.gO.launch(rows)
        self._join_prefetch()
        # consecutive all-reduces of a step must alternate between the peer buffer's two regions (site % 2): a
        # rank may start pushing launch n + 1 while a peer still reads launch n's words.  A layer without an
        # FFN all-reduce therefore numbers its attention site by the layer alone
        attn = ops.PendingReduce(rows, cfg.hidden, self.o_p, self.nsO, self.h1, h, step.slots, self.peer,
                                 2 * self.layer if self.ffn is not None else self.layer, self.guard, self.deadline_s)
        if self.ffn is None:
            return attn if defer else attn.launch()
        if self.fuse_reduce:  # the attention all-reduce runs inside the MoE half's norm staging launch
            return self.ffn(None, step.slots, pending=attn, defer=defer)
        return self.ffn(attn.launch(), step.slots, defer=defer)
