"""Host runner of the GQA block-sparse attention half of a layer.

Reference counterparts: ``minimax_m3/gfx950/runner.py`` (``M3MonoRunner``: pointer-only
launches over SGLang's caches and step tables) and the stages of
``minimax_m3/gfx950/pre_attn.py`` / ``index_score.py`` / ``post_attn.py:466-1003``:
input RMSNorm -> fused q | k | v | index_q | index_k projection -> per-head norms, RoPE,
cache insert -> block scores -> top-16 block selection -> attention over the selected
blocks -> o_proj -> all-reduce + residual.  Everything is allocated in ``__init__``;
``launch`` only enqueues kernels on torch's current stream.
"""

from __future__ import annotations

import os

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L
from . import ops

HEAD_DIM = 128
BLOCK = 64
TOPK_BLOCKS = 16


@dataclass(frozen=True)
class GqaConfig:
    name: str
    hidden: int
    q_heads: int   # global
    kv_heads: int  # global
    tp: int = 1
    eps: float = 1e-6
    init_blocks: int = 1
    local_blocks: int = 2
    rope_theta: float = 1.0e6

    @property
    def q_local(self) -> int:
        return self.q_heads // self.tp

    @property
    def kv_local(self) -> int:
        return self.kv_heads // self.tp

    @property
    def qkv_rows(self) -> int:
        """Rows of a rank's fused projection: q | k | v | index q | index k heads."""
        return (self.q_local + 2 * self.kv_local + 2) * HEAD_DIM

    @property
    def sm_scale(self) -> float:
        return HEAD_DIM ** -0.5

    def with_tp(self, tp: int) -> "GqaConfig":
        from dataclasses import replace
        return replace(self, tp=tp)


CFG_GQA = GqaConfig(name="cfg4_gqa_block_sparse", hidden=6144, q_heads=48, kv_heads=8, tp=4)
CFG_GQA_TINY = GqaConfig(name="tiny_gqa_block_sparse", hidden=512, q_heads=8, kv_heads=2, tp=1)


@dataclass
class GqaTables:
    """One step's tables: what SGLang hands over (``minimax_m3/metadata.py:7-42``)."""

    positions: torch.Tensor   # int64 [rows]
    slots: torch.Tensor       # int64 [rows], page * 64 + offset, negative = pad
    page_table: torch.Tensor  # int32 [rows, blocks]
    k_cache: torch.Tensor     # uint8 [pages, 64, kv_local, 128]
    v_cache: torch.Tensor
    index_cache: torch.Tensor  # uint8 [pages, 64, 128]
    cos: torch.Tensor         # bf16 [positions, 32]
    sin: torch.Tensor


class GqaCore:
    """front -> score -> select -> attention, from the projection's partial sums."""

    def __init__(self, cfg: GqaConfig, w: dict, device, max_ctx: int):
        L.load()
        self.cfg, self.w, self.dev = cfg, w, device
        self.max_blocks = -(-max_ctx // BLOCK)
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)  # noqa: E731
        self.q = z(L.MAX_ROWS, cfg.q_local, HEAD_DIM, dt=torch.bfloat16)
        self.iq = z(L.MAX_ROWS, HEAD_DIM, dt=torch.bfloat16)
        self.scores = z(L.MAX_ROWS, self.max_blocks)
        self.sel_pages = z(L.MAX_ROWS, TOPK_BLOCKS, dt=torch.int32)
        self.sel_blocks = z(L.MAX_ROWS, TOPK_BLOCKS, dt=torch.int32)
        self.n_ctx = z(L.MAX_ROWS, dt=torch.int32)
        nbytes = L.load().mono_gqa_scratch_bytes(L.MAX_ROWS, cfg.q_local)
        self.scratch = z(nbytes // 4)
        self.out = z(L.MAX_ROWS, cfg.q_local * HEAD_DIM, dt=torch.bfloat16)
        for k in ("g_q", "g_k", "g_iq", "g_ik"):
            ops.require(w[k], k, torch.bfloat16, (HEAD_DIM,))

    def args(self, rows: int, qkv: torch.Tensor, nsum: int, t: GqaTables) -> L.GqaArgs:
        cfg, w = self.cfg, self.w
        ops.require(t.positions, "positions", torch.int64, (rows,))
        ops.require(t.slots, "slots", torch.int64, (rows,))
        ops.require(t.page_table, "page_table", torch.int32)
        ops.require(t.k_cache, "k_cache", torch.uint8)
        ops.require(t.v_cache, "v_cache", torch.uint8)
        ops.require(t.index_cache, "index_cache", torch.uint8)
        if tuple(t.k_cache.shape[1:]) != (BLOCK, cfg.kv_local, HEAD_DIM) or t.v_cache.shape != t.k_cache.shape:
            raise ValueError(f"k_cache / v_cache: shape {tuple(t.k_cache.shape)}, needs [pages, 64, {cfg.kv_local}, 128]")
        if tuple(t.index_cache.shape) != (t.k_cache.shape[0], BLOCK, HEAD_DIM):
            raise ValueError(f"index_cache: shape {tuple(t.index_cache.shape)}, needs [pages, 64, 128]")
        if t.page_table.shape[0] < rows or t.page_table.shape[1] > self.max_blocks:
            raise ValueError(f"page_table: shape {tuple(t.page_table.shape)}, needs [>= {rows}, <= {self.max_blocks}]")
        a = L.GqaArgs()
        a.rows, a.q_heads, a.kv_heads = rows, cfg.q_local, cfg.kv_local
        a.qkv, a.nsum, a.ld, a.sum_stride = qkv.data_ptr(), nsum, qkv.shape[-1], L.MAX_ROWS * qkv.shape[-1]
        a.g_q, a.g_k, a.g_iq, a.g_ik = (w[k].data_ptr() for k in ("g_q", "g_k", "g_iq", "g_ik"))
        a.eps = cfg.eps
        a.cos, a.sin = t.cos.data_ptr(), t.sin.data_ptr()
        a.positions, a.slots = t.positions.data_ptr(), t.slots.data_ptr()
        a.k_scale, a.v_scale = float(w["k_scale"]), float(w["v_scale"])
        a.k_cache, a.v_cache, a.index_cache = t.k_cache.data_ptr(), t.v_cache.data_ptr(), t.index_cache.data_ptr()
        a.n_pages = t.k_cache.shape[0]
        a.q_out, a.iq_out = self.q.data_ptr(), self.iq.data_ptr()
        a.page_table, a.pt_ld = t.page_table.data_ptr(), t.page_table.shape[1]
        a.scores, a.score_ld = self.scores.data_ptr(), t.page_table.shape[1]
        a.init_blocks, a.local_blocks = cfg.init_blocks, cfg.local_blocks
        a.sel_pages, a.sel_blocks, a.n_ctx = self.sel_pages.data_ptr(), self.sel_blocks.data_ptr(), self.n_ctx.data_ptr()
        a.sm_scale = cfg.sm_scale
        a.scratch, a.out = self.scratch.data_ptr(), self.out.data_ptr()
        return a

    def launch(self, rows: int, qkv: torch.Tensor, nsum: int, t: GqaTables) -> torch.Tensor:
        a = self.args(rows, qkv, nsum, t)
        lib, st = L.load(), ops._stream()
        L.check(lib.mono_gqa_front_launch(C.byref(a), st), "mono_gqa_front_launch")
        L.check(lib.mono_gqa_score_launch(C.byref(a), st), "mono_gqa_score_launch")
        L.check(lib.mono_gqa_select_launch(C.byref(a), st), "mono_gqa_select_launch")
        L.check(lib.mono_gqa_attn_launch(C.byref(a), st), "mono_gqa_attn_launch")
        return self.out[:rows]


class GqaAttentionOp:
    """The attention half: ``out = residual + allreduce(W_o attn(norm(residual)))``."""

    def __init__(self, cfg: GqaConfig, w: dict, device, max_ctx: int, peer=None, guard: torch.Tensor | None = None,
                 site: int = 0, deadline_s: float = 5.0):
        self.cfg, self.w, self.dev, self.peer, self.site, self.deadline_s = cfg, w, device, peer, site, deadline_s
        self.guard = guard if guard is not None else torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=device)
        h = cfg.hidden
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)  # noqa: E731
        self.core = GqaCore(cfg, w, device, max_ctx)
        # the bf16 normed input goes through the FP8 tensor cores exactly, as two E4M3 planes
        self.xq = ops.ActBuf(L.ACT_HILO, h, device)
        self.qkv_g = ops.Gemv(L.W_FP8, self.guard, deadline_s)
        st, ns = ops.plan_split(-(-h // 128), cfg.qkv_rows // 128, L.W_FP8)
        self.ns_qkv = ns
        self.qkv = z(ns, L.MAX_ROWS, cfg.qkv_rows)
        self.qkv_g.add("qkv", w["qkv"], self.xq, self.qkv, wscale=w["qkv_s"], split_tiles=st, nsplit=ns)
        ok = cfg.q_local * HEAD_DIM
        self.oq = ops.ActBuf(L.ACT_HILO, ok, device)
        self.o_g = ops.Gemv(L.W_FP8, self.guard, deadline_s)
        st, ns = ops.plan_split(-(-ok // 128), -(-h // 128), L.W_FP8)
        self.ns_o = ns
        self.o_p = z(ns, L.MAX_ROWS, h)
        self.o_g.add("o", w["o"], self.oq, self.o_p, wscale=w["o_s"], split_tiles=st, nsplit=ns)
        self.out = z(L.MAX_ROWS, h, dt=torch.bfloat16)

    def launch(self, residual: torch.Tensor, t: GqaTables, defer: bool = False):
        """``defer``: the o_proj reduction (+ all-reduce + residual) is returned unlaunched (``ops.PendingReduce``) for
        the stage that consumes it to run inside its own norm staging launch."""
        cfg, w = self.cfg, self.w
        rows = residual.shape[0]
        if not 1 <= rows <= L.MAX_ROWS:
            raise ValueError(f"residual: {rows} rows, the launch serves 1..{L.MAX_ROWS}")
        ops.require(residual, "residual", torch.bfloat16, (rows, cfg.hidden))
        ops.act_prep(rows, cfg.hidden, self.xq, src_bf16=residual, gamma=w["in_norm"], eps=cfg.eps)
        self.qkv_g.launch(rows)
        attn = self.core.launch(rows, self.qkv, self.ns_qkv, t)
        ops.act_prep(rows, cfg.q_local * HEAD_DIM, self.oq, src_bf16=attn, round_bf16=False)
        self.o_g.launch(rows)
        red = ops.PendingReduce(rows, cfg.hidden, self.o_p, self.ns_o, self.out, residual, t.slots, self.peer, self.site,
                                self.guard, self.deadline_s)
        return red if defer else red.launch()


class GqaLayerOp:
    """One decoder layer: the GQA block-sparse attention half, then the MoE half
    (reference: ``minimax_m3/gfx950/runner.py`` ``M3MonoRunner``: K1 + K4 per layer)."""

    def __init__(self, cfg: GqaConfig, moe_cfg, w: dict, device, max_ctx: int, peer=None, deadline_s: float = 5.0):
        from .moe import MoeFfn

        self.cfg, self.moe_cfg = cfg, moe_cfg
        self.guard = torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=device)
        self.attn = GqaAttentionOp(cfg, w, device, max_ctx, peer=peer, guard=self.guard, site=0, deadline_s=deadline_s)
        self.ffn = MoeFfn(moe_cfg, w, device, peer=peer, guard=self.guard, site=1, deadline_s=deadline_s)

    def launch(self, h: torch.Tensor, t: GqaTables) -> torch.Tensor:
        if self.attn.peer is not None and self.attn.peer.world > 1:
            ops.epoch_advance(self.guard)
        if os.environ.get("MONO_FUSE_REDUCE", "1") != "0":  # the attention all-reduce inside the MoE half's norm launch
            return self.ffn(None, t.slots, pending=self.attn.launch(h, t, defer=True))
        return self.ffn(self.attn.launch(h, t), t.slots)
