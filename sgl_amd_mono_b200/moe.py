"""Host runner of the MoE FFN half of a layer (post-norm, router, shared + routed
experts, all-reduce, residual) and of the stand-alone FFN block.

Reference counterparts: ``minimax_m31/runner.py:145-167`` (``FfnRunner.__call__``:
tensors in, pointer-only launches, ``(out, res_out)`` back) and the FFN stages of
``glm53/gfx950/kernel.py:4199-5187``.  Everything is allocated in ``__init__``; a
call only launches kernels on torch's current stream, so it can be captured in a
CUDA graph and replayed.
"""

from __future__ import annotations

import os

import torch

from . import _lib as L
from . import ops
from .config import LayerConfig

_WK = {"fp8_block": L.W_FP8, "mxfp4": L.W_MXFP4, "bf16": L.W_BF16, "nvfp4": L.W_NVFP4}
_ACT = {"fp8_block": L.ACT_A8, "mxfp4": L.ACT_MX8, "bf16": L.ACT_BF16, "nvfp4": L.ACT_NVF4}


def _ktiles(t: torch.Tensor) -> int:
    """K of a weight in 128-byte tiles."""
    return -(-(t.shape[-1] * t.element_size()) // 128)


class MoeFfn:
    """``out = residual + allreduce(shared(x̂) + sum_k w_k expert_k(x̂))``, x̂ = RMSNorm(residual)."""

    def __init__(self, cfg: LayerConfig, w: dict, device, max_rows: int = L.MAX_ROWS, peer=None,
                 guard: torch.Tensor | None = None, site: int = 1, deadline_s: float = 5.0, copies: dict | None = None,
                 layer: int = 0):
        """``copies``: the build context's dict of one-time copies (key tuple -> tensor, ``glm53/spec.py:499-581``);
        the one repack this block may make (MXFP4 scale rows padded to whole tiles) is recorded there."""
        lib = L.load()  # fail loudly when the CUDA library is missing
        tc_on = lib.mono_set_gemv_tcgen05(1)  # read the switch ...
        lib.mono_set_gemv_tcgen05(tc_on)      # ... and put it back
        self.cfg, self.w, self.dev, self.peer, self.site = cfg, w, device, peer, site
        self.deadline_s = deadline_s
        self.guard = guard if guard is not None else torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=device)
        h, il, E, k = cfg.hidden, cfg.inter_local, cfg.n_experts, cfg.top_k
        self.max_expert = min(E, max_rows * k)
        efmt, sfmt = cfg.expert_fmt, cfg.shared_fmt
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)  # noqa: E731
        def act_of(fmt, weight):
            # MXFP4 weights on the tcgen05 consumer take natural-order MXFP8 activations
            if fmt == "mxfp4" and tc_on and ops.fp4_tma_ok(weight):
                return L.ACT_MX8N
            return _ACT[fmt]

        self.xq = ops.ActBuf(act_of(efmt, w["w13"]), h, device)
        self.xbf = z(L.MAX_ROWS, h, dt=torch.bfloat16)
        self.logits = z(L.MAX_ROWS, E)
        self.ids = z(L.MAX_ROWS, k, dt=torch.int32)
        self.weights = z(L.MAX_ROWS, k)
        self.scores = z(L.MAX_ROWS, E)
        self.expert_list = z(self.max_expert, dt=torch.int32)
        self.n_expert = z(1, dt=torch.int32)
        self.coef = z(self.max_expert, L.MAX_ROWS)
        self.mid_r = ops.ActBuf(act_of(efmt, w["w2"]), il, device, segs=self.max_expert)
        self.has_shared = sfmt != "none"
        same = self.has_shared and sfmt == efmt
        # ---- up / gate launch
        # the shared expert's dense job goes first: its weight tiles do not depend on the router,
        # so the launch can request them before the routing of this step is known
        self.up = ops.Gemv(_WK[efmt], self.guard, deadline_s, copies=copies, copy_tag=layer)
        self.up_sh = self.mid_s = self.up_s = None
        if self.has_shared:
            self.xs = self.xq if same else ops.ActBuf(act_of(sfmt, w["sh13"]), h, device)
            self.mid_s = ops.ActBuf(act_of(sfmt, w["sh2"]), il, device)
            st, ns = ops.plan_split(_ktiles(w["sh13"]), -(-2 * il // 128), _WK[sfmt])
            self.ns_up_s = ns
            self.up_s = z(ns, L.MAX_ROWS, 2 * il)
            g = self.up if same else ops.Gemv(_WK[sfmt], self.guard, deadline_s)
            g.add("sh13", w["sh13"], self.xs, self.up_s, wscale=w.get("sh13_s"), split_tiles=st, nsplit=ns,
                  wglobal=w.get("sh13_g"))
            self.up_sh = None if same else g
        # the tcgen05 consumer takes K segments of up to 32 tiles (no activation slot to fit): fewer K splits
        probe = ops.plan_split(_ktiles(w["w13"]), -(-2 * il // 128) * self.max_expert, _WK[efmt],
                               cap=32 if (efmt == "fp8_block" and tc_on) else None)
        # (finer up/gate tasks, 16 or 8 tiles instead of 28 at TP 8, measured 268 and 310 us per layer against 252)
        self.ns_up = probe[1]
        self.up_r = z(self.max_expert * self.ns_up, L.MAX_ROWS, 2 * il)
        got = self.up.add("w13", w["w13"], self.xq, self.up_r, mode=L.JOB_EXPERT_UP, wscale=w["w13_s"],
                          expert_list=self.expert_list, n_expert=self.n_expert, max_expert=self.max_expert,
                          split_tiles=probe[0], nsplit=probe[1], wglobal=w.get("w13_g"))
        assert got == self.ns_up
        # ---- down launch: routed expert groups, then the shared expert's K splits
        nrb = -(-h // 128)
        # expert groups: row blocks x groups tasks should fill whole rounds of the grid (one CTA per SM)
        sms = ops.sm_count()
        best = (0.0, 1)
        for g in range(1, min(self.max_expert, 16) + 1):
            tasks = nrb * g
            eff = (tasks / sms) / -(-tasks // sms)
            if tasks >= sms and eff > best[0] + 1e-9:
                best = (eff, g)
        self.groups = best[1] if best[0] > 0 else max(1, min(self.max_expert, -(-sms // nrb)))
        ns_dn_s = 0
        if self.has_shared:
            self.st_dn_s, ns_dn_s = ops.plan_split(_ktiles(w["sh2"]), nrb, _WK[sfmt])
        self.n_slices = self.groups + ns_dn_s
        self.down_p = z(self.n_slices, L.MAX_ROWS, h)
        self.down = ops.Gemv(_WK[efmt], self.guard, deadline_s, copies=copies, copy_tag=layer)
        self.down_sh = None
        if self.has_shared:
            g = self.down if same else ops.Gemv(_WK[sfmt], self.guard, deadline_s)
            g.add("sh2", w["sh2"], self.mid_s, self.down_p, wscale=w.get("sh2_s"), out_slice=self.groups,
                  split_tiles=self.st_dn_s, nsplit=ns_dn_s, wglobal=w.get("sh2_g"))
            self.down_sh = None if same else g
        self.down.add("w2", w["w2"], self.mid_r, self.down_p, mode=L.JOB_EXPERT_DOWN, wscale=w["w2_s"],
                      expert_list=self.expert_list, n_expert=self.n_expert, max_expert=self.max_expert,
                      coef=self.coef, nsplit=self.groups, wglobal=w.get("w2_g"))
        self.out = z(L.MAX_ROWS, h, dt=torch.bfloat16)
        # Router logits and routing in one launch (the CTA that finishes its logit columns last routes the step;
        # MONO_ROUTER_FUSED=0: two launches).  Measured on config 3 once the logit weights' loads no longer cost a
        # round trip each: 622.6 against 626.7 us at TP 1, equal for a TP 8 shard, one launch fewer
        self.route_counter = z(1, dt=torch.int32)
        self.router_fused = os.environ.get("MONO_ROUTER_FUSED", "1") != "0"
        # ---- one launch for up/gate -> SwiGLU -> down (FP8 on the tcgen05 path): the same jobs, chained
        self.chained = None
        # (the CTA that finishes an expert's last up/gate task computes the whole activation of that expert:
        # measured on config 3: faster at TP 8 (256 intermediate values per rank), slower from TP 4 down, where
        # an expert's activation is 4+ chunks per row and the separate activation launch spreads it better)
        chain_default = "1" if il <= 256 else "0"
        if efmt == "fp8_block" and (not self.has_shared or same) and tc_on and os.environ.get("MONO_MOE_CHAINED", chain_default) != "0":
            g = ops.Gemv(L.W_FP8, self.guard, deadline_s)
            first = 0
            if self.has_shared:
                g.add("sh13", w["sh13"], self.xs, self.up_s, wscale=w.get("sh13_s"), split_tiles=st, nsplit=self.ns_up_s)
                first = 1
            g.add("w13", w["w13"], self.xq, self.up_r, mode=L.JOB_EXPERT_UP, wscale=w["w13_s"],
                  expert_list=self.expert_list, n_expert=self.n_expert, max_expert=self.max_expert,
                  split_tiles=probe[0], nsplit=probe[1])
            if self.has_shared:
                g.add("sh2", w["sh2"], self.mid_s, self.down_p, wscale=w.get("sh2_s"), out_slice=self.groups,
                      split_tiles=self.st_dn_s, nsplit=ns_dn_s)
            g.add("w2", w["w2"], self.mid_r, self.down_p, mode=L.JOB_EXPERT_DOWN, wscale=w["w2_s"],
                  expert_list=self.expert_list, n_expert=self.n_expert, max_expert=self.max_expert,
                  coef=self.coef, nsplit=self.groups)
            if self.has_shared:
                g.chain(0, 2, 1)
            g.chain(first, first + (2 if self.has_shared else 1), self.max_expert)
            self.chained = g

    def __call__(self, residual: torch.Tensor | None, slots: torch.Tensor | None = None, pending=None, defer: bool = False):
        """``pending``: the reduction that produces this block's input rows has not been launched (``ops.PendingReduce``);
        it runs inside this block's norm staging launch and ``residual`` is not read.  ``defer``: the block's own final
        reduction is returned as an ``ops.PendingReduce`` instead of being launched, for the next stage to fuse."""
        cfg, w = self.cfg, self.w
        if pending is not None:
            residual = pending.out[: pending.rows]
        rows = residual.shape[0]
        if not 1 <= rows <= L.MAX_ROWS:
            raise ValueError(f"residual: {rows} rows, the launch serves 1..{L.MAX_ROWS}")
        ops.require(residual, "residual", torch.bfloat16, (rows, cfg.hidden))
        if slots is not None:
            ops.require(slots, "slots", torch.int64, (rows,))
        h, il = cfg.hidden, cfg.inter_local
        if pending is not None:
            ops.reduce_norm(pending, self.xq, gamma=w["post_norm"], eps=cfg.eps, out_bf16=self.xbf)
        else:
            ops.act_prep(rows, h, self.xq, src_bf16=residual, gamma=w["post_norm"], eps=cfg.eps, out_bf16=self.xbf)
        if self.has_shared and self.xs is not self.xq:
            ops.act_prep(rows, h, self.xs, src_bf16=self.xbf, round_bf16=False)
        rt = (rows, cfg.top_k, cfg.route_scale, self.logits, w.get("router_bias"), slots, self.ids,
              self.weights, self.scores, self.expert_list, self.n_expert, self.coef)
        if self.router_fused:
            ops.router(ops.rowdot_args(rows, w["router"], self.xbf, self.logits), ops.route_args(*rt), self.route_counter)
        else:
            ops.rowdot(rows, w["router"], self.xbf, self.logits)
            ops.route(*rt)
        final = ops.PendingReduce(rows, h, self.down_p, self.n_slices, self.out, residual, slots, self.peer, self.site,
                                  self.guard, self.deadline_s)
        if self.chained is not None:
            self.chained.launch(rows)
            return final if defer else final.launch()
        self.up.launch(rows)
        if self.up_sh is not None:
            self.up_sh.launch(rows)
        routed = ops.mid_args(rows, il, self.up_r, self.ns_up, self.mid_r, n_slot=self.n_expert, max_slot=self.max_expert,
                              round_bf16=cfg.expert_fmt != "fp8_block")
        if self.has_shared:  # both activation stages in one launch
            shared = ops.mid_args(rows, il, self.up_s, self.ns_up_s, self.mid_s, max_slot=1,
                                  round_bf16=cfg.shared_fmt != "fp8_block")
            ops.mid_pair(routed, shared)
        else:
            ops.mid(rows, il, self.up_r, self.ns_up, self.mid_r, n_slot=self.n_expert, max_slot=self.max_expert,
                    round_bf16=cfg.expert_fmt != "fp8_block")
        self.down.launch(rows)
        if self.down_sh is not None:
            self.down_sh.launch(rows)
        return final if defer else final.launch()
