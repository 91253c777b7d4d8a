#!/usr/bin/env python
"""Benchmark of the decode hot path: µs per decoder layer and achieved HBM GB/s.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

One "step" is one pass of the workload's hot path over one batch of synthetic rows.
The JSON line carries: ``value`` (device-timed, inputs resident in HBM), ``e2e``
(the same call through the public op with pinned HOST inputs, copies inside the timed
region), ``roofline`` of the dominant kernel (timed alone with CUDA events) and
``cpu_baseline`` (the CPU oracle on a bounded sample, host cores).  Between timed
iterations a buffer larger than L2 is written so that no step starts warm.
``--impl reference`` times the CPU restatement of the reference's arithmetic on the
host cores (the reference's own kernels exist only for AMD gfx950 and cannot run here).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(1, str(ROOT / "tests"))  # the synthetic-input generator (tests/synth.py) lives beside the tests

L2_FLUSH_BYTES = 256 << 20
L2_NOTE = "256 MiB buffer written, then another 256 MiB read, between timed iterations"


class L2Flush:
    """Empties the 126 MB L2 between timed iterations: writes a 256 MiB buffer, then reads a second one.

    The write alone leaves the L2 full of dirty lines, and their write-back (126 MB of DRAM writes) is charged to
    whatever runs next: a 255 MB weight-streaming launch timed alone took 64.5 us after the write, 51.2 us after
    write + read, 49.2 us after a read alone, and 49.1 us of device time in a profiler capture of the same launch.  (A
    whole layer changes by 2 us of 620: its first, latency-bound stages absorb the write-back.)  After the read the
    L2 holds clean lines of an unrelated buffer, which is also what a layer finds in a running model: the
    previous layer's weights."""

    def __init__(self, dev):
        self.buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        self.rd = torch.ones(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
        self.acc = torch.zeros((), dtype=torch.float32, device=dev)

    def zero_(self):
        self.buf.zero_()
        torch.sum(self.rd, dim=0, out=self.acc)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


def measured_traffic(key, nbytes):
    """DRAM bytes per launch of the probed kernel: the ncu-measured traffic / algorithmic ratio of the
    same kernel on a capturable case (profiles/dram_traffic.json) times this launch's algorithmic
    bytes; None when no capture of that kernel is committed."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if key is None or not p.exists():
        return None
    d = json.loads(p.read_text()).get(key)
    return None if not d else int(nbytes * d["traffic_bytes"] / d["algorithmic_bytes"])


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < 5.0:  # nvidia-smi takes a moment to start
                time.sleep(0.02)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def time_steps(fn, steps: int, warmup: int, flush: "L2Flush | None", sampler=None):
    """Sum of per-step device times in ms (CUDA events on the current stream)."""
    for _ in range(warmup):
        if flush is not None:
            flush.zero_()
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        for a, b in evs:
            if flush is not None:
                flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs)


def count_kernel_launches(fn) -> int:
    """Kernels of this library that one call of ``fn`` launches: the library counts every launch it makes
    (``mono_launch_count``), so entry points that launch several kernels count as many."""
    from sgl_amd_mono_b200 import _lib as L

    lib = L.load()
    before = lib.mono_launch_count()
    fn()
    torch.cuda.synchronize()
    return int(lib.mono_launch_count() - before)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class Lazy:
    """Expert tensors stay where they were generated; the oracle copies to the host only those it routes to."""

    def __init__(self, v):
        self.v, self.c = v, {}

    def __getitem__(self, e):
        e = int(e)
        if e not in self.c:
            self.c[e] = self.v[e].cpu()
        return self.c[e]


def host_weights(w):
    return {k: (Lazy(v) if k in ("w13", "w13_s", "w2", "w2_s") else (v.cpu() if isinstance(v, torch.Tensor) else v))
            for k, v in w.items()}


def time_oracle(fn, runs: int):
    """One warm-up (it also pulls the routed experts to the host), then the median of ``runs`` runs, in us."""
    fn()
    ts = []
    for _ in range(runs):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts) * 1e6


# ------------------------------------------------------------------ workloads
class SparseMlaWorkload:
    """BASELINE config 2: sparse MLA decode attention alone, 8 rows x 16 local heads,
    FP8 latent cache with one f32 scale per token, 32768-token contexts, 2048 selected
    keys per row (uniform without replacement), softmax scale 1/sqrt(192)."""

    name = "cfg2_sparse_mla_8rows_16heads_ctx32768_top2048"
    layers_per_step = 1
    kernel = "sparse_mla_split_kernel + sparse_mla_merge_kernel"

    def __init__(self, rows=8, heads=16, ctx=32768, topk=2048):
        self.rows, self.heads, self.ctx, self.topk = rows, heads, ctx, topk
        if heads != 16:
            self.name = f"sparse_mla_{rows}rows_{heads}heads_ctx{ctx}_top{topk}"
        if heads >= 64:
            self.kernel = "mla_qsplit_kernel + sparse_mla_split_tc_kernel (tcgen05) + sparse_mla_merge_kernel"

    def make_inputs(self, dev, rank, tp):
        """Synthetic inputs only (torch): nothing of the kernel library is touched."""
        import synth

        self.dev = dev
        self.q, self.pages, self.sel, _ = synth.sparse_mla_inputs(self.rows, self.heads, self.ctx, self.topk, device=dev, seed=rank)

    def setup(self, dev, rank, world):
        from sgl_amd_mono_b200.attention import SparseMlaOp

        self.make_inputs(dev, rank, world)
        q, pages, sel = self.q, self.pages, self.sel
        self.op = SparseMlaOp(self.heads, self.topk, dev, sm_scale=192**-0.5)
        self.q_host, self.sel_host = q.cpu().pin_memory(), sel.cpu().pin_memory()
        self.q_in, self.sel_in = torch.empty_like(q), torch.empty_like(sel)
        self.out_host = torch.empty(self.rows, self.heads, 512, dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = 2

    def step(self):
        self.op(self.q, self.pages, self.sel)

    def e2e_step(self):
        self.q_in.copy_(self.q_host, non_blocking=True)
        self.sel_in.copy_(self.sel_host, non_blocking=True)
        out = self.op(self.q_in, self.pages, self.sel_in)
        self.out_host.copy_(out, non_blocking=True)
        torch.cuda.synchronize()

    def e2e_bytes(self):
        return self.q_host.numel() * 2 + self.sel_host.numel() * 4, self.out_host.numel() * 2

    def roofline_probe(self):
        b = self.rows * (self.topk * 580 + self.heads * 576 * 2 + self.heads * 512 * 2)
        return b, self.step

    def config(self):
        return {"workload": self.name, "rows": self.rows, "local_heads": self.heads, "context": self.ctx,
                "topk": self.topk, "kv_cache": "fp8_e4m3 + f32 scale per token, page 64",
                "l2": L2_NOTE}

    def oracle_step(self):
        from oracle import stages as S

        q, pages, sel = self.q.cpu(), self.pages.cpu(), self.sel.cpu()
        return (lambda: S.sparse_mla(q, pages, sel, 192**-0.5)), f"all {self.rows} rows"

    def cpu_sample(self):
        fn, what = self.oracle_step()
        return time_oracle(fn, 3), what + "; median of 3 after one warm-up"


class MoeWorkload:
    """The MoE FFN half of BASELINE config 3 (hidden 7168, 256 routed experts top-8 + 1
    shared, intermediate 2048, FP8 E4M3 with 128x128 block scales) at TP = number of
    GPUs, 8 decode rows: post-norm, router, shared + routed experts, all-reduce, residual."""

    layers_per_step = 1
    kernel = "gemv_tc_kernel (tcgen05 FP8 expert up/gate, timed as its own launch)"
    traffic_key = "fp8_expert_up_gate"

    def __init__(self, rows=8):
        self.rows = rows

    def make_inputs(self, dev, rank, tp, world=1):
        import synth
        from sgl_amd_mono_b200.config import CFG_V3
        from dataclasses import replace

        self.cfg = replace(CFG_V3, n_heads=0, index_heads=0).with_tp(tp)
        self.name = f"cfg3_moe_half_tp{tp}_{self.rows}rows" + ("_one_shard" if tp != world else "")
        self.w = synth.layer_weights(self.cfg, rank, dev)
        g = torch.Generator().manual_seed(0)
        self.x_host = torch.randn(self.rows, self.cfg.hidden, generator=g).bfloat16()
        self.distinct = None

    def setup(self, dev, rank, world, peer=None):
        from sgl_amd_mono_b200.moe import MoeFfn

        tp = getattr(self, "shard_of", 0) or world  # --shard-of N: one rank's share of TP = N, no peers
        self.make_inputs(dev, rank, tp, world)
        self.ffn = MoeFfn(self.cfg, self.w, dev, peer=peer)
        self.x_host = self.x_host.pin_memory()
        self.x = self.x_host.to(dev)
        self.x_in = torch.empty_like(self.x)
        self.out_host = torch.empty_like(self.x_host).pin_memory()
        self.ffn(self.x)
        torch.cuda.synchronize()
        self.distinct = int(self.ffn.n_expert.item())
        self.launches_per_step = 8

    def step(self):
        self.ffn(self.x)

    def e2e_step(self):
        self.x_in.copy_(self.x_host, non_blocking=True)
        out = self.ffn(self.x_in)
        self.out_host.copy_(out, non_blocking=True)
        torch.cuda.synchronize()

    def e2e_bytes(self):
        return self.x_host.numel() * 2, self.out_host.numel() * 2

    def roofline_probe(self):
        u = int(self.ffn.n_expert.item())
        c = self.cfg
        b = (u + 1) * 2 * c.inter_local * c.hidden
        return b, lambda: self.ffn.up.launch(self.rows)

    def config(self):
        c = self.cfg
        return {"workload": self.name, "rows": self.rows, "hidden": c.hidden, "experts": c.n_experts, "top_k": c.top_k,
                "inter": c.inter, "tp": c.tp, "distinct_experts": self.distinct,
                "weights": "fp8_e4m3 128x128 block scales", "l2": L2_NOTE}

    def oracle_step(self):
        from oracle import layers as OL

        w, x = host_weights(self.w), self.x_host.clone()

        def fn():
            _, ids, _, _ = OL.moe_partial(self.cfg, w, x)
            if self.distinct is None:
                self.distinct = int(ids.unique().numel())

        return fn, f"all {self.rows} rows"

    def cpu_sample(self):
        fn, what = self.oracle_step()
        return time_oracle(fn, 3), what + "; median of 3 after one warm-up"


class LayerWorkload:
    """BASELINE config 3: the full DeepSeek-V3-shaped MLA + lightning-indexer + MoE decoder
    layer (hidden 7168, 128 heads, q_lora 1536, kv_lora 512, 64 index heads with FP4 keys
    and top-2048, 256 experts top-8 + shared, FP8 128x128 block scales), context 16384,
    at TP = number of GPUs with both all-reduces inside the reduce kernel.  BASELINE lists
    TP 2/4/8; TP 1 is the same layer unsharded, which fits one GPU."""

    layers_per_step = 1
    kernel = "gemv_tc_kernel (tcgen05 FP8 expert up/gate, timed as its own launch)"
    traffic_key = "fp8_expert_up_gate"

    def __init__(self, rows=8, ctx=16384):
        self.rows, self.ctx = rows, ctx

    def make_inputs(self, dev, rank, tp, world=1):
        """Synthetic weights, caches, tables and rows (torch only: nothing of the kernel library is touched)."""
        import synth
        from sgl_amd_mono_b200.config import CFG_V3

        self.cfg = cfg = CFG_V3.with_tp(tp)
        self.name = f"cfg3_v3_mla_dsa_moe_layer_tp{tp}_{self.rows}rows_ctx{self.ctx}" + ("_one_shard" if tp != world else "")
        self.w = synth.layer_weights(cfg, rank, dev)
        self.step_in = synth.decode_step(cfg, self.rows, self.ctx, device=dev)
        g = torch.Generator().manual_seed(0)
        self.h_host = torch.randn(self.rows, cfg.hidden, generator=g).bfloat16()
        self.distinct = None

    def setup(self, dev, rank, world):
        from sgl_amd_mono_b200 import ops
        from sgl_amd_mono_b200.layer import MlaLayerOp, StepTables

        tp = getattr(self, "shard_of", 0) or world  # --shard-of N: one rank's share of TP = N, no peers
        self.make_inputs(dev, rank, tp, world)
        cfg = self.cfg
        self.peer = None
        if world > 1:
            import torch.distributed as dist
            from sgl_amd_mono_b200.common.peer import PeerBuffer

            self.cpu_group = dist.new_group(backend="gloo")
            self.peer = PeerBuffer(cfg.hidden, rank, world, self.cpu_group, dev)
        step = self.step_in
        # the oracle reads the caches as they were before the first step wrote this step's rows
        self.kv0, self.ix0 = step.kv_pages.cpu(), step.idx_pages.cpu()
        self.tables = StepTables(step.positions, step.slots, step.page_table, step.kv_pages, step.idx_pages, step.cos, step.sin)
        self.op = MlaLayerOp(cfg, self.w, dev, max_ctx=self.ctx, peer=self.peer,
                             guard=self.peer.guard if self.peer else None)
        self.ops = ops
        self.h_host = self.h_host.pin_memory()
        self.h = self.h_host.to(dev)
        self.h_in = torch.empty_like(self.h)
        self.out_host = torch.empty_like(self.h_host).pin_memory()
        self._eager()
        torch.cuda.synchronize()
        rc, words = ops.guard_read(self.op.guard)
        if rc != 0:
            raise RuntimeError(f"guard words after the first step: {words}")
        self.distinct = int(self.op.ffn.n_expert.item())
        self.launches_per_step = 23 + (1 if world > 1 else 0)
        # one CUDA graph of the step, as the reference times its layers (time_layers.py:38-77)
        self.graph = None
        if os.environ.get("MONO_BENCH_GRAPH", "1") == "1":
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._eager()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    self._eager()
            torch.cuda.current_stream().wait_stream(s)
            self.graph = g

    def _eager(self):
        self.out = self.op.launch(self.h, self.tables)
        if self.peer is not None:
            self.ops.epoch_advance(self.op.guard)

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._eager()

    def e2e_step(self):
        self.h.copy_(self.h_host, non_blocking=True)
        self.step()
        self.out_host.copy_(self.out, non_blocking=True)
        torch.cuda.synchronize()

    def e2e_bytes(self):
        return self.h_host.numel() * 2, self.out_host.numel() * 2

    def check(self):
        rc, words = self.ops.guard_read(self.op.guard)
        if rc != 0:
            raise RuntimeError(f"guard words after the timed steps: {words}")

    def layer_bytes(self):
        c, u = self.cfg, self.distinct
        hl, il, h = c.heads_local, c.inter_local, c.hidden
        rep = (c.q_lora + 576) * h + c.index_heads * 128 * c.q_lora + 128 * h + c.index_heads * h * 2 + c.n_experts * h * 2
        shard = hl * 192 * c.q_lora + hl * 256 * 512 + h * hl * 128
        experts = (1 + u) * 3 * il * h
        kv = self.rows * min(c.index_topk, self.ctx) * 580
        idx = self.rows * self.ctx * 68
        return rep + shard + experts + kv + idx, u

    def roofline_probe(self):
        u = self.distinct
        c = self.cfg
        return (u + 1) * 2 * c.inter_local * c.hidden, lambda: self.op.ffn.up.launch(self.rows)

    def config(self):
        c = self.cfg
        nbytes, u = self.layer_bytes()
        return {"workload": self.name, "rows": self.rows, "context": self.ctx, "hidden": c.hidden, "heads": c.n_heads,
                "experts": c.n_experts, "top_k": c.top_k, "inter": c.inter, "tp": c.tp, "distinct_experts": u,
                "layer_algorithmic_bytes_per_rank": nbytes, "cuda_graph": getattr(self, "graph", None) is not None,
                "weights": "fp8_e4m3 128x128 block scales", "l2": L2_NOTE}

    def oracle_step(self):
        """The CPU restatement of the whole layer over every row of the step (this rank's share)."""
        from oracle import layers as OL

        w, t = host_weights(self.w), self.step_in
        kv = getattr(self, "kv0", None)
        kv = kv if kv is not None else t.kv_pages.cpu()
        ix = getattr(self, "ix0", None)
        ix = ix if ix is not None else t.idx_pages.cpu()
        args = (self.cfg, [w], self.h_host.clone(), t.positions.cpu(), t.slots.cpu(), t.page_table.cpu(), t.cos.cpu(), t.sin.cpu())

        def fn():
            _, det = OL.layer_all_ranks(*args, kv.clone(), ix.clone())
            if self.distinct is None:
                self.distinct = int(det["ids"].unique().numel())

        return fn, f"all {self.rows} rows of this rank's layer share"

    def cpu_sample(self):
        fn, what = self.oracle_step()
        return time_oracle(fn, 1), what + "; one run after one warm-up"


class GqaLayerWorkload(LayerWorkload):
    """BASELINE config 4: a GQA block-sparse + MXFP4 MoE layer (hidden 6144, 48 q / 8 kv heads of 128,
    16 blocks x 64 tokens attended per row over a 65536-token context, FP8 attention projections, 256
    experts top-8 of intermediate 1536 in MXFP4, sigmoid router), 16 verify rows, one rank's share of
    TP 4 (or TP = number of GPUs)."""

    kernel = "gemv_mxf4_kernel (tcgen05 kind::mxf8f6f4.block_scale MXFP4 expert up/gate, nibbles padded by TMA, timed as its own launch)"
    traffic_key = "mxfp4_expert_up_gate"

    def __init__(self, rows=16, ctx=65536, expert_fmt="mxfp4"):
        """``expert_fmt`` "nvfp4": the same layer with NVFP4 experts (E4M3 scale per 16, 4-bit activations)."""
        super().__init__(rows, ctx)
        self.expert_fmt = expert_fmt
        if expert_fmt == "nvfp4":
            self.kernel = "gemv_nvf4_kernel (tcgen05 kind::mxf4nvf4.block_scale NVFP4 expert up/gate, timed as its own launch)"
            self.traffic_key = "nvfp4_expert_up_gate"

    def make_inputs(self, dev, rank, tp, world=1):
        import synth
        from sgl_amd_mono_b200.config import LayerConfig
        from sgl_amd_mono_b200.gqa import CFG_GQA

        self.gcfg = g = CFG_GQA.with_tp(tp)
        fmt = self.expert_fmt
        self.cfg = cfg = LayerConfig(name=f"cfg4_moe_{fmt}", hidden=g.hidden, n_experts=256, top_k=8, inter=1536, route_scale=1.0,
                                     expert_fmt=fmt, shared_fmt="none", router_dtype="bf16", eps=g.eps, tp=tp)
        self.name = f"cfg4_gqa_block_sparse_{fmt}_moe_layer_tp{tp}_{self.rows}rows_ctx{self.ctx}" + ("_one_shard" if tp != world else "")
        self.w = {**synth.layer_weights(cfg, rank, dev), **synth.gqa_weights(g, rank, dev)}
        self.tables = synth.gqa_step(g, self.rows, self.ctx, dev, ragged=False)
        gen = torch.Generator().manual_seed(0)
        self.h_host = torch.randn(self.rows, g.hidden, generator=gen).bfloat16()
        self.distinct = None
        # the rows' own pages, renumbered, as they are before the step inserts this step's rows
        t = self.tables
        self.row_caches = []
        for r in range(self.rows):
            pages = t.page_table[r].long()
            self.row_caches.append([c[pages.to(c.device)].cpu() for c in (t.k_cache, t.v_cache, t.index_cache)])

    def setup(self, dev, rank, world):
        from sgl_amd_mono_b200 import ops
        from sgl_amd_mono_b200.gqa import GqaLayerOp

        tp = getattr(self, "shard_of", 0) or (world if world > 1 else 4)
        self.make_inputs(dev, rank, tp, world)
        g, cfg = self.gcfg, self.cfg
        self.peer = None
        if world > 1:
            import torch.distributed as dist
            from sgl_amd_mono_b200.common.peer import PeerBuffer

            self.cpu_group = dist.new_group(backend="gloo")
            self.peer = PeerBuffer(g.hidden, rank, world, self.cpu_group, dev)
        self.op = GqaLayerOp(g, cfg, self.w, dev, max_ctx=self.ctx, peer=self.peer)
        self.ops = ops
        self.h_host = self.h_host.pin_memory()
        self.h = self.h_host.to(dev)
        self.out_host = torch.empty_like(self.h_host).pin_memory()
        self._eager()
        torch.cuda.synchronize()
        rc, words = ops.guard_read(self.op.guard)
        if rc != 0:
            raise RuntimeError(f"guard words after the first step: {words}")
        self.distinct = int(self.op.ffn.n_expert.item())
        self.launches_per_step = 19 + (1 if world > 1 else 0)
        self.graph = None
        if os.environ.get("MONO_BENCH_GRAPH", "1") == "1":
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._eager()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=s):
                    self._eager()
            torch.cuda.current_stream().wait_stream(s)
            self.graph = gr

    def _eager(self):
        self.out = self.op.launch(self.h, self.tables)

    def layer_bytes(self):
        g, c, u = self.gcfg, self.cfg, self.distinct
        h, il = g.hidden, c.inter_local
        attn_w = g.qkv_rows * h + h * g.q_local * 128 + c.n_experts * h * 2
        experts = u * (3 * il * h // 2 + 3 * il * h // self.scale_group)
        kv = self.rows * 16 * 64 * g.kv_local * 128 * 2
        idx = self.rows * self.ctx * 128
        return attn_w + experts + kv + idx, u

    def roofline_probe(self):
        u = self.distinct
        c = self.cfg
        return u * (2 * c.inter_local * c.hidden // 2 + 2 * c.inter_local * c.hidden // self.scale_group), lambda: self.op.ffn.up.launch(self.rows)

    @property
    def scale_group(self) -> int:
        """Weight values per scale byte."""
        return 16 if self.expert_fmt == "nvfp4" else 32

    def config(self):
        g, c = self.gcfg, self.cfg
        nbytes, u = self.layer_bytes()
        return {"workload": self.name, "rows": self.rows, "context": self.ctx, "hidden": g.hidden, "q_heads": g.q_heads,
                "kv_heads": g.kv_heads, "blocks_attended": 16, "block_tokens": 64, "experts": c.n_experts, "top_k": c.top_k,
                "inter": c.inter, "tp": c.tp, "distinct_experts": u, "layer_algorithmic_bytes_per_rank": nbytes,
                "cuda_graph": getattr(self, "graph", None) is not None, "weights": f"fp8_e4m3 attention projections, {self.expert_fmt} experts",
                "l2": L2_NOTE}

    def oracle_step(self):
        from oracle import gqa as OG
        from oracle import layers as OL

        w, t = host_weights(self.w), self.tables
        pos, cos, sin = t.positions.cpu(), t.cos.cpu(), t.sin.cpu()
        local = []
        for r in range(self.rows):
            pages = t.page_table[r].cpu().long()
            slot = int(t.slots[r])
            local.append((torch.arange(pages.numel(), dtype=torch.int32)[None],
                          torch.tensor([int((pages == slot // 64).nonzero()[0]) * 64 + slot % 64])))

        def fn():
            mids = []
            for r in range(self.rows):  # every row is its own request: its pages, renumbered from 0
                lpt, lslot = local[r]
                mids.append(OG.attention_half(self.gcfg, w, self.h_host[r : r + 1].clone(), pos[r : r + 1], lslot, lpt,
                                              [c.clone() for c in self.row_caches[r]], cos, sin))
            _, det = OL.ffn_block(self.cfg, [w], torch.cat(mids))
            if self.distinct is None:
                self.distinct = int(det["ids"].unique().numel())

        return fn, f"all {self.rows} rows of this rank's layer share"


class AllReduceWorkload:
    """The in-kernel tensor-parallel all-reduce alone (rows x 7168 bf16 per rank, pushes over
    IPC-mapped peer memory + rank-ordered sum + residual) next to an NCCL all-reduce of the
    same message, both replayed from CUDA graphs.  Needs --gpus >= 2."""

    layers_per_step = 1
    holds_nccl_graphs = True
    kernel = "reduce_kernel (push + rank-ordered sum)"

    def __init__(self, rows=8, n=7168):
        self.rows, self.n = rows, n

    def setup(self, dev, rank, world):
        import torch.distributed as dist
        from sgl_amd_mono_b200 import ops
        from sgl_amd_mono_b200.common.peer import PeerBuffer

        if world < 2:
            raise SystemExit("the allreduce workload needs --gpus >= 2")
        self.world, self.name = world, f"allreduce_{self.rows}x{self.n}_bf16_tp{world}"
        self.peer = PeerBuffer(self.n, rank, world, dist.new_group(backend="gloo"), dev)
        self.ops, self.dist = ops, dist
        g = torch.Generator().manual_seed(rank)
        self.part = torch.zeros(1, 16, self.n, device=dev)
        self.part[0, : self.rows] = torch.randn(self.rows, self.n, generator=g).to(dev)
        self.res = torch.zeros(self.rows, self.n, dtype=torch.bfloat16, device=dev)
        self.out = torch.zeros(16, self.n, dtype=torch.bfloat16, device=dev)
        self.msg = self.part[0, : self.rows].bfloat16().contiguous()
        self.launches_per_step = 2

        def ours():
            ops.reduce_rows(self.rows, self.n, self.part, 1, self.out, residual=self.res, peer=self.peer, site=0,
                            guard=self.peer.guard, deadline_s=10.0)
            ops.epoch_advance(self.peer.guard)

        def nccl():
            dist.all_reduce(self.msg)

        self.g_ours, self.g_nccl = self._graph(ours), self._graph(nccl)
        # the reduce-scatter + all-gather form of the same kernel (half the bytes per link, one more hop)
        self.rsag_us, self.g_rsag = None, None
        if (self.n // 2) % (2 * world) == 0:
            self.out_rsag = torch.zeros_like(self.out)
            old_env = os.environ.get("MONO_AR_RSAG")
            os.environ["MONO_AR_RSAG"] = "always"
            try:
                def ours_rsag():
                    ops.reduce_rows(self.rows, self.n, self.part, 1, self.out_rsag, residual=self.res, peer=self.peer, site=0,
                                    guard=self.peer.guard, deadline_s=10.0)
                    ops.epoch_advance(self.peer.guard)

                self.g_rsag = self._graph(ours_rsag)
            finally:
                if old_env is None:
                    del os.environ["MONO_AR_RSAG"]
                else:
                    os.environ["MONO_AR_RSAG"] = old_env
        # the NVLS variant: the same kernel, each word pushed by one multimem.st through the switch
        self.mc_us, self.mc_note = None, None
        try:
            from sgl_amd_mono_b200.common.peer import MulticastPeerBuffer

            self.peer_mc = MulticastPeerBuffer(self.n, rank, world, dist.group.WORLD, dev)
            self.out_mc = torch.zeros_like(self.out)

            def ours_mc():
                ops.reduce_rows(self.rows, self.n, self.part, 1, self.out_mc, residual=self.res, peer=self.peer_mc, site=0,
                                guard=self.peer_mc.guard, deadline_s=10.0)
                ops.epoch_advance(self.peer_mc.guard)

            self.g_mc = self._graph(ours_mc)
        except Exception as e:  # raised on every rank together (no multicast address): reported, not hidden
            self.g_mc, self.mc_note = None, f"{type(e).__name__}: {e}"[:200]
        # correctness against NCCL's sum of the same bf16 partials (NCCL's order is unspecified: tolerance)
        self.msg.copy_(self.part[0, : self.rows].bfloat16())
        self.g_nccl.replay()
        self.g_ours.replay()
        torch.cuda.synchronize()
        err = (self.out[: self.rows].float() - self.msg.float()).abs().max().item()
        if not err <= 0.05 * max(1.0, self.msg.float().abs().max().item()):
            raise RuntimeError(f"in-kernel all-reduce differs from NCCL by {err}")
        rc, words = ops.guard_read(self.peer.guard)
        if rc:
            raise RuntimeError(f"guard words {words}")
        self.nccl_us = self._time(self.g_nccl)
        if self.g_rsag is not None:
            self.g_rsag.replay()
            torch.cuda.synchronize()
            rc, words = ops.guard_read(self.peer.guard)
            if rc or not torch.equal(self.out_rsag, self.out):
                raise RuntimeError(f"the reduce-scatter form changed the all-reduce's bits (guard words {words})")
            self.rsag_us = self._time(self.g_rsag)
        if self.g_mc is not None:
            self.g_mc.replay()
            torch.cuda.synchronize()
            rc, words = ops.guard_read(self.peer_mc.guard)
            if rc or not torch.equal(self.out_mc, self.out):
                raise RuntimeError(f"multicast pushes changed the all-reduce's bits (guard words {words})")
            self.mc_us = self._time(self.g_mc)

    def check(self):
        rc, words = self.ops.guard_read(self.peer.guard)
        if rc != 0:
            raise RuntimeError(f"guard words after the timed steps: {words}")

    def _graph(self, fn):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                fn()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                fn()
        torch.cuda.current_stream().wait_stream(s)
        return g

    def _time(self, g, n=200):
        self.dist.barrier()
        for _ in range(20):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1000.0 / n

    def step(self):
        self.g_ours.replay()

    def e2e_step(self):
        self.step()
        torch.cuda.synchronize()

    def e2e_bytes(self):
        return 0, 0

    def roofline_probe(self):
        return self.rows * self.n * 2 * (self.world - 1), self.step

    def config(self):
        return {"workload": self.name, "rows": self.rows, "n": self.n, "tp": self.world,
                "nccl_allreduce_us": self.nccl_us, "in_kernel_allreduce_us_back_to_back": self._time(self.g_ours),
                "in_kernel_allreduce_multicast_us": self.mc_us, "multicast_unavailable": self.mc_note,
                "in_kernel_allreduce_rs_ag_us": self.rsag_us,
                "nvlink_peak_gbs_per_direction": 900, "l2": L2_NOTE}

    def cpu_sample(self):
        return float("nan"), "not applicable"


class StackWorkload:
    """BASELINE config 5: a 40-layer flash-sized MLA + MoE stack (hidden 4096, 64 heads, kv_lora
    512 + rope 64, 256 experts top-6 + shared, intermediate 1024, FP8 128x128), context 8192,
    bf16 LM head over vocab 129280, one decode step under one CUDA graph.  The step carries
    ``rows`` decode rows plus a 5-token verify of one more request (rows + 5 rows through the
    40 layers) and a single-layer draft stage on the 5 verify rows.  q_lora 1536, nope 128 and
    v 128 are this build's choice (BASELINE leaves them open); there is no indexer, so every
    cached key is attended."""

    kernel = "gemv_tc_kernel (tcgen05 FP8 expert up/gate of layer 0, timed as its own launch)"
    traffic_key = "fp8_expert_up_gate"

    def __init__(self, rows=1, ctx=8192, layers=40, verify=5):
        self.rows, self.ctx, self.n_layers, self.verify = rows, ctx, layers, verify
        self.layers_per_step = layers

    def make_inputs(self, dev, rank, tp, world=1, layers=None):
        """Synthetic weights, caches and tables of ``layers`` (default: all of them).  StepTables is a plain
        dataclass of tensors: nothing of the kernel library is touched."""
        import synth
        from sgl_amd_mono_b200.config import CFG_FLASH
        from sgl_amd_mono_b200.layer import StepTables
        from dataclasses import replace as dc_replace

        self.n_layers = int(os.environ.get("MONO_BENCH_LAYERS", self.n_layers))
        self.layers_per_step = self.n_layers
        self.cfg = cfg = CFG_FLASH.with_tp(tp)
        self.total = self.rows + self.verify
        self.name = (f"cfg5_flash_stack_{self.n_layers}layers_tp{tp}_{self.rows}rows_plus_{self.verify}verify_ctx{self.ctx}"
                     + ("_one_shard" if tp != world else ""))
        ids = list(range(self.n_layers)) if layers is None else list(layers)
        self.ws = []
        for i in ids:
            c = cfg if i == self.n_layers - 1 else dc_replace(cfg, vocab=0)
            self.ws.append(synth.layer_weights(c, rank, dev, layer=i))
        self.w0 = self.ws[0]

        # rows decode requests + one request verified with `verify` tokens: every row has its own
        # page-table row (the verify rows repeat theirs); one cache per layer
        def tables(layer):
            d = synth.decode_step(cfg, self.rows + 1, self.ctx, device=dev, layer=layer)
            req = torch.tensor(list(range(self.rows)) + [self.rows] * self.verify, device=dev)
            pos = torch.cat([d.positions[: self.rows], self.ctx - self.verify + torch.arange(self.verify, device=dev)])
            pt = d.page_table[req].contiguous()
            slots = pt.gather(1, (pos // 64).unsqueeze(1)).squeeze(1).long() * 64 + pos % 64
            return StepTables(pos, slots, pt, d.kv_pages, None, d.cos, d.sin)

        self._tables_of = tables
        self.tables = [tables(i) for i in ids]
        self.kv0 = self.tables[0].kv_pages.cpu()  # layer 0's cache before the first step writes this step's rows
        g = torch.Generator().manual_seed(0)
        self.h_host = torch.randn(self.total, cfg.hidden, generator=g).bfloat16()

    def setup(self, dev, rank, world):
        import synth
        from sgl_amd_mono_b200 import ops
        from sgl_amd_mono_b200.layer import StepTables
        from sgl_amd_mono_b200.stack import DecoderStack
        from dataclasses import replace as dc_replace

        tp = getattr(self, "shard_of", 0) or world
        self.make_inputs(dev, rank, tp, world)
        cfg, ws = self.cfg, self.ws
        self.peer = None
        if world > 1 and tp == world:
            import torch.distributed as dist
            from sgl_amd_mono_b200.common.peer import PeerBuffer

            self.peer = PeerBuffer(cfg.hidden, rank, world, dist.new_group(backend="gloo"), dev, logits_local=cfg.vocab // tp)
        draft_w = synth.layer_weights(dc_replace(cfg, vocab=0), rank, dev, layer=999)
        dt = self._tables_of(999)
        self.draft_tables = StepTables(dt.positions[self.rows:].contiguous(), dt.slots[self.rows:].contiguous(),
                                       dt.page_table[self.rows:].contiguous(), dt.kv_pages, None, dt.cos, dt.sin)
        self.stack = DecoderStack(cfg, ws, dev, max_ctx=self.ctx, peer=self.peer, draft_weights=draft_w)
        self.ops = ops
        self.h_host = self.h_host.pin_memory()
        self.h = self.h_host.to(dev)
        self.hd = self.h[self.rows:].contiguous()
        self._eager()
        torch.cuda.synchronize()
        self.check()
        self.launches_per_step = 0  # counted from an eager step by the caller (count_kernel_launches)
        self.logits_host = torch.empty(self.total, self.logits.shape[-1], dtype=torch.float32).pin_memory()
        self.graph = None
        if os.environ.get("MONO_BENCH_GRAPH", "1") == "1":
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._eager()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    self._eager()
            torch.cuda.current_stream().wait_stream(s)
            self.graph = g

    def _eager(self):
        st = self.stack
        st.draft.launch(self.hd, self.draft_tables)
        x = st.run_layers(self.h, self.tables)
        pending = isinstance(x, self.ops.PendingReduce)
        self.logits = st.head(None, pending=x) if pending else st.head(x)
        self.ops.epoch_advance(st.guard)

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._eager()

    def e2e_step(self):
        self.h.copy_(self.h_host, non_blocking=True)
        self.step()
        self.logits_host.copy_(self.logits, non_blocking=True)
        torch.cuda.synchronize()

    def e2e_bytes(self):
        return self.h_host.numel() * 2, self.logits_host.numel() * 4

    def check(self):
        rc, words = self.ops.guard_read(self.stack.guard)
        if rc != 0:
            raise RuntimeError(f"guard words: {words}")

    def layer_bytes(self):
        c = self.cfg
        hl, il, h = c.heads_local, c.inter_local, c.hidden
        fixed = (c.q_lora + 576) * h + c.n_experts * h * 2 + hl * 192 * c.q_lora + hl * 256 * 512 + h * hl * 128
        total, us = 0, []
        for op in self.stack.layers:
            u = int(op.ffn.n_expert.item())
            us.append(u)
            total += fixed + (1 + u) * 3 * il * h + self.total * self.ctx * 580
        total += (c.vocab // c.tp) * h * 2
        return total, round(sum(us) / len(us), 1)

    def roofline_probe(self):
        op = self.stack.layers[0]
        u = int(op.ffn.n_expert.item())
        return (u + 1) * 2 * self.cfg.inter_local * self.cfg.hidden, lambda: op.ffn.up.launch(self.total)

    def config(self):
        c = self.cfg
        nbytes, u = self.layer_bytes()
        return {"workload": self.name, "decode_rows": self.rows, "verify_rows": self.verify, "draft_layers": 1,
                "layers": self.n_layers, "context": self.ctx, "hidden": c.hidden, "heads": c.n_heads, "experts": c.n_experts,
                "top_k": c.top_k, "inter": c.inter, "vocab": c.vocab, "tp": c.tp, "mean_distinct_experts": u,
                "step_algorithmic_bytes_per_rank": nbytes, "cuda_graph": getattr(self, "graph", None) is not None,
                "l2": L2_NOTE}

    def oracle_step(self):
        from oracle import layers as OL

        w = host_weights(self.w0)
        t = self.tables[0]
        args = (self.cfg, [w], self.h_host.clone(), t.positions.cpu(), t.slots.cpu(), t.page_table.cpu(), t.cos.cpu(), t.sin.cpu())
        kv = self.kv0

        def fn():
            OL.layer_all_ranks(*args, kv.clone(), None)

        return fn, f"layer 0 of {self.n_layers}, all {self.total} rows (per layer)"

    def cpu_sample(self):
        fn, what = self.oracle_step()
        return time_oracle(fn, 1), what + "; one run after one warm-up"


WORKLOADS = {"stack": StackWorkload, "sparse_mla": SparseMlaWorkload, "moe": MoeWorkload, "layer": LayerWorkload,
             "gqa_layer": GqaLayerWorkload, "allreduce": AllReduceWorkload}
DEFAULT_WORKLOAD = "layer"


def measure_stack(args, dev, rank, flush) -> dict:
    """BASELINE config 5 on one GPU: 40 layers + LM head, 1 decode row + a 5-token verify, one CUDA graph per step.
    Device time per step (CUDA events, L2 flushed between steps) and the same step with its input rows copied from
    pinned host memory and the logits copied back."""
    wl = StackWorkload()
    wl.shard_of = 0
    wl.setup(dev, rank, 1)
    steps = max(3, min(args.steps, 10))
    ms = time_steps(wl.step, steps, 3, flush) / steps
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        wl.e2e_step()
    e2e = []
    for _ in range(steps):
        flush.zero_()
        a.record()
        wl.e2e_step()
        b.record()
        torch.cuda.synchronize()
        e2e.append(a.elapsed_time(b))
    wl.check()
    wl.launches_per_step = count_kernel_launches(wl._eager)
    h2d, d2h = wl.e2e_bytes()
    peak, _ = measured_peaks()
    return {"workload": wl.name, "steps": steps, "step_us": ms * 1000.0, "us_per_layer": ms * 1000.0 / wl.n_layers,
            "tokens_per_s": wl.rows / (ms * 1e-3), "e2e_step_us": statistics.median(e2e) * 1000.0,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "gpu_launches_per_step": wl.launches_per_step,
            "stack_frac_of_measured_hbm_peak": wl.layer_bytes()[0] / (ms * 1e-3) / 1e9 / peak}


# ------------------------------------------------------------------ main
def run_reference(args, wl_cls, rank: int) -> None:
    """The CPU restatement of the reference's arithmetic on the host cores, every row of the step, one warm-up
    and the median of max(5, steps capped at 7) runs (the reference's own kernels exist only for AMD gfx950).
    Only synthetic inputs are generated (torch, on the GPU when there is one, because drawing 11 GB of expert
    weights on the host takes minutes): no operator of the kernel library is built and the library is not loaded."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    kw = dict(rows=args.rows) if args.rows else {}
    if args.heads and args.workload == "sparse_mla":
        kw["heads"] = args.heads
    if args.workload == "gqa_layer" and args.expert_fmt != "mxfp4":
        kw["expert_fmt"] = args.expert_fmt
    wl = wl_cls(**kw)
    if not hasattr(wl, "oracle_step"):
        print(json.dumps({"impl": "reference", "unavailable": f"the {args.workload} workload has no CPU counterpart"}))
        return
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    # rank 0's share of TP = N, built without peers (the other ranks of a torchrun launch do no work)
    tp = args.shard_of or (args.gpus if args.gpus > 1 else (4 if args.workload == "gqa_layer" else 1))
    if args.workload == "stack":
        wl.make_inputs(dev, 0, tp, 1, layers=[0])
    else:
        wl.make_inputs(dev, 0, tp, 1) if args.workload != "sparse_mla" else wl.make_inputs(dev, 0, tp)
    fn, what = wl.oracle_step()
    runs = max(5, min(args.steps, 7))
    v = time_oracle(fn, runs)
    sample = f"{what}; median of {runs} runs after one warm-up"
    try:
        cfg = wl.config()
    except AttributeError:  # a workload whose byte count needs the built operators
        cfg = {"workload": wl.name}
    line = {
        "impl": "reference", "metric": "us_per_decoder_layer", "value": v, "unit": "us", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": v / 1000.0, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 over dequantised fp8/fp4", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": v, "unit": "us", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=os.environ.get("MONO_BENCH_WORKLOAD", DEFAULT_WORKLOAD), choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="rows of the step (default: 8; 16 for gqa_layer)")
    ap.add_argument("--heads", type=int, default=0, help="sparse_mla: local heads (default 16, config 2; 128 = config 3 at TP 1)")
    ap.add_argument("--expert-fmt", default="mxfp4", choices=["mxfp4", "nvfp4"], help="gqa_layer: format of the routed experts")
    ap.add_argument("--load-seconds", type=float, default=0.6, help="time under load before the timed steps")
    ap.add_argument("--shard-of", type=int, default=0, help="run one rank's share of TP = N on each GPU without peers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-stack", action="store_true", help="default workload at 1 GPU: leave out the config-5 stack measurement")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl_cls = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl_cls, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the monokernel path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device(dev))
    kw = dict(rows=args.rows) if args.rows else {}
    if args.heads and args.workload == "sparse_mla":
        kw["heads"] = args.heads
    if args.workload == "gqa_layer" and args.expert_fmt != "mxfp4":
        kw["expert_fmt"] = args.expert_fmt
    wl = wl_cls(**kw)
    wl.shard_of = args.shard_of
    def trace(what):  # MONO_BENCH_TRACE=1: progress on stderr, to see where a multi-rank run stops
        if os.environ.get("MONO_BENCH_TRACE") == "1":
            print(f"[bench rank {rank}] {what}", file=sys.stderr, flush=True)

    trace("setup")
    wl.setup(dev, rank, world)
    trace("setup done")
    flush = L2Flush(dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if hasattr(wl, "_eager"):
        wl.launches_per_step = count_kernel_launches(wl._eager)  # every rank runs the same extra step
    barrier()
    sampler = ClockSampler(local)
    sampler.__enter__()
    # keep the GPU under load for about 0.6 s so that the clock samples mean something; the
    # number of steps is fixed by rank 0 (ranks that exchange data must run the same count)
    t_probe = time.time()
    for _ in range(20):
        wl.step()
    torch.cuda.synchronize()
    n_load = torch.tensor([int(min(20000, max(0, args.load_seconds / max((time.time() - t_probe) / 20, 1e-6))))], device=dev)
    if dist is not None:
        dist.broadcast(n_load, src=0)
    for _ in range(int(n_load.item())):
        wl.step()
    torch.cuda.synchronize()
    trace(f"load phase done ({int(n_load.item())} steps); timed steps")
    total_ms = time_steps(wl.step, args.steps, args.warmup, flush)
    trace("timed steps done")
    barrier()
    t = torch.tensor([total_ms], device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    us_per_layer = ms_per_step * 1000.0 / wl.layers_per_step
    # end to end: pinned host inputs, copies and the result read inside the timed region
    for _ in range(3):
        wl.e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.e2e_step()
    e2e_ms = (time.perf_counter() - t0) * 1000.0 / args.steps
    t = torch.tensor([e2e_ms], device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_us = float(t.item()) * 1000.0 / wl.layers_per_step
    h2d, d2h = wl.e2e_bytes()
    # roofline of the dominant kernel, timed alone
    trace("e2e done; roofline probe")
    nbytes, probe = wl.roofline_probe()
    probe_ms = time_steps(probe, args.steps, 3, flush) / args.steps
    sampler.__exit__(None, None, None)
    if hasattr(wl, "check"):
        wl.check()  # the guard's error words must be clean after the timed steps
    peak, peak_src = measured_peaks()
    achieved = nbytes / (probe_ms * 1e-3) / 1e9
    trace("probe done; building the line")
    line = {
        "metric": "us_per_decoder_layer", "value": us_per_layer, "unit": "us", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3 weights / bf16 activations, f32 accumulate", "data": "synthetic",
        "config": wl.config(), "clocks": sampler.summary(), "gpu_launches": wl.launches_per_step * args.steps,
        "e2e": {"value": e2e_us, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        # layer_bytes() covers what one timed step reads (one layer, or the whole stack and its tail)
        "roofline": {"bound": "hbm", "kernel": wl.kernel, **({"layer_achieved_gbs": wl.layer_bytes()[0] / (ms_per_step * 1e-3) / 1e9,
                     "layer_frac": wl.layer_bytes()[0] / (ms_per_step * 1e-3) / 1e9 / peak} if hasattr(wl, "layer_bytes") else {}), "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": measured_traffic(getattr(wl, "traffic_key", None), nbytes),
                     "algorithmic_bytes": nbytes,
                     "kernel_us": probe_ms * 1000.0, "peak_source": peak_src},
    }
    cpu_wl = wl
    if rank == 0 and not args.no_cpu_baseline and args.workload == DEFAULT_WORKLOAD and world == 1 and not args.shard_of and not args.no_stack:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        v, sample = wl.cpu_sample()
        line["cpu_baseline"] = {"value": v, "unit": "us", "cores": cores, "kind": "port", "sample": sample}
    if hasattr(wl, "n_layers"):
        line["step_us"] = ms_per_step * 1000.0
        line["tokens_per_s"] = wl.rows * world / (ms_per_step * 1e-3) if getattr(wl, "shard_of", 0) else wl.rows / (ms_per_step * 1e-3)
    elif args.workload == DEFAULT_WORKLOAD and world == 1 and not args.shard_of and not args.no_stack:
        # BASELINE config 5 (the one config quoted at TP 1) next to the headline layer: the whole 40-layer stack + LM
        # head under one CUDA graph, timed in this same run after the layer workload's memory is given back
        cpu_wl = None
        del wl, probe
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        try:
            line["config5_stack"] = measure_stack(args, dev, rank, flush)
        except Exception as e:  # reported, never hidden: the headline line above stands on its own
            line["config5_stack"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        wl = None
    if rank == 0:
        if not args.no_cpu_baseline and "cpu_baseline" not in line:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            v, sample = cpu_wl.cpu_sample()
            line["cpu_baseline"] = {"value": v, "unit": "us", "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
        if getattr(cpu_wl, "holds_nccl_graphs", False):
            # tearing the communicator down under live CUDA graphs of its kernels does not return: the
            # line is out and every rank is past the barrier, so leave without the teardown
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
