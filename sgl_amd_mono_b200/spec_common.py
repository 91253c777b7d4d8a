"""What the per-model specs share: refusal reasons, the step tables, and the routed forward.

Reference counterparts: ``glm53/spec.py:173-208`` (``_config_disable_reasons``),
``:215-251`` (``_model_disable_reasons``), ``:296-417`` (``_Built.forward`` /
``_backbone`` / ``_layer``), ``:467-496`` (``_step``: the step's tables, built once a
step and, under a CUDA graph, inside the capture), ``:499-581`` (``_build``).
"""

from __future__ import annotations

import logging
from types import SimpleNamespace

import torch

from . import _lib as L
from . import check
from .config import KV_PAGE_BYTES, LayerConfig
from .registry import BuildContext, Plan

log = logging.getLogger("sgl_amd_mono_b200")
ISA = "sm_100a"
SM_COUNT = 148  # resident_blocks a spec declares before any device is visible: one CTA per SM of a B200
ROWS = tuple(range(1, L.MAX_ROWS + 1))
TP_SIZES = (1, 2, 4, 8)


def config_reasons(name: str, want: dict, cfg, hf_config, page_size: int = 64) -> list[str]:
    """Every reason this configuration cannot be served; the server refuses to start and
    lists them all (the reference's README: "lists every reason")."""
    reasons = [
        f"needs {name}'s {key} = {val!r}, got {getattr(hf_config, key, None)!r}"
        for key, val in want.items() if getattr(hf_config, key, None) != val
    ]
    if getattr(cfg, "page_size", None) not in (None, page_size):
        reasons.append(f"--page-size {cfg.page_size}: the caches need {page_size}")
    tp = getattr(cfg, "tp_size", 1)
    if tp not in TP_SIZES:
        reasons.append(f"--tp-size {tp}: the kernels are built for {TP_SIZES}")
    if not L.LIB_PATH.exists():
        reasons.append(f"{L.LIB_PATH.name} is not built (python -m sgl_amd_mono_b200.build); there is no fallback path")
    return reasons


def weight_reasons(layer: int, w: dict, expect: dict) -> list[str]:
    """Layout checks of one layer's SGLang tensors: {name: (dtype, shape)}."""
    out = []
    for name, (dtype, shape) in expect.items():
        t = w.get(name)
        if t is None:
            out.append(f"layer {layer}: {name} is missing")
        elif t.dtype != dtype or tuple(t.shape) != tuple(shape) or not t.is_contiguous():
            out.append(f"layer {layer}: {name} is {t.dtype} {tuple(t.shape)}, needs contiguous {dtype} {tuple(shape)}")
    return out


def step_tables(plan: Plan, positions, forward_batch, rows: int, max_position: int):
    """The step's rows for every launch, built once a step (``glm53/spec.py:467-496``):
    slots (SGLang's pad slot 0 becomes -1), clamped positions, the page-table rows."""
    if "step" not in plan.state:
        from .layer import StepTables

        loc = forward_batch.out_cache_loc[:rows].to(torch.int64)
        slots = torch.where(loc != 0, loc, torch.full_like(loc, -1))
        pos = positions[:rows].to(torch.int64).clamp(max=max_position)
        pos = torch.where(slots >= 0, pos, torch.zeros_like(pos))
        plan.state["step"] = SimpleNamespace(slots=slots, positions=pos, page_table=forward_batch.page_table[:rows])
        plan.state["tables"] = StepTables
    return plan.state["step"]


class Built:
    """The routed forward of a model whose covered layers run on the monokernels."""

    def __init__(self, model, cfg: LayerConfig, ops_by_layer: dict, max_rows: int, max_position: int, numerics=None):
        self.model, self.cfg, self.ops, self.max_rows, self.max_position = model, cfg, ops_by_layer, max_rows, max_position
        self.numerics = numerics  # the spec's bounds, read by check mode (MONO_CHECK=1)

    def forward(self, plan: Plan, input_ids, positions, forward_batch, input_embeds=None, *args, **kw):
        rows = plan.key.rows
        if rows > self.max_rows:  # a graph key the spec does not serve runs the model's own path
            return type(self.model).forward(self.model, input_ids, positions, forward_batch, input_embeds, *args, **kw)
        from .layer import StepTables

        st = step_tables(plan, positions, forward_batch, rows, self.max_position)
        h = input_embeds if input_embeds is not None else self.model.embed(input_ids)
        h = h[:rows]
        for i, layer in enumerate(model_layers(self.model)):
            op = self.ops.get(i)
            if op is None:  # an uncovered (dense) layer runs the model's own code
                h = layer.forward(h, positions, forward_batch)
                continue
            caches = forward_batch.caches[i]
            if caches.kv.shape[-1] != KV_PAGE_BYTES or caches.kv.dtype != torch.uint8:
                raise RuntimeError(f"layer {i}: MLA cache {caches.kv.dtype} {tuple(caches.kv.shape)}; "
                                   f"needs contiguous uint8 [pages, {KV_PAGE_BYTES}]")
            tables = StepTables(st.positions, st.slots, st.page_table, caches.kv, getattr(caches, "idx", None),
                                forward_batch.cos, forward_batch.sin)
            if self.numerics is not None and check.enabled():
                # check mode (glm53/spec.py:402-417): the same rows through the model's own layer, compared as they run
                ref = lambda x, t, layer=layer: {"out": layer.forward(x, positions, forward_batch)}  # noqa: E731
                h, _ = check.check_layer_launch(i, self.numerics, op, h, tables, ref)
            else:
                h = op.launch(h, tables)
        return self.model.finish(h, forward_batch) if hasattr(self.model, "finish") else h


def model_layers(model):
    """The decoder layers: SGLang's ``lm.model.layers``, or ``model.layers`` of a stand-alone model."""
    return getattr(model, "model", model).layers


def build_layers(model, cfg: LayerConfig, ctx: BuildContext, covered: list[int], make_op, bind=None, numerics=None) -> Built:
    """Builds one op per covered layer in layer order (a collective when tp_size > 1:
    every rank builds the same runtimes in the same order, ``glm53/spec.py:499-581``).  ``bind(i)`` returns
    layer i's tensors bound to SGLang's storage and records every one-time copy in ``ctx.copies``; without
    it the layer carries its tensors as a ``weights`` dict (the stand-alone synthetic model)."""
    ops_by_layer = {}
    before = len(ctx.copies)
    for i in covered:
        ops_by_layer[i] = make_op(i, bind(i) if bind is not None else model_layers(model)[i].weights)
    nbytes = sum(t.numel() * t.element_size() for t in ctx.copies.values() if isinstance(t, torch.Tensor))
    log.info("%s: %d layers on the monokernels, widths %s, TP %d; %d one-time copies (%.1f MB in all), every other "
             "tensor is read in place", cfg.name, len(covered), ctx.widths, ctx.tp_size, len(ctx.copies) - before, nbytes / 1e6)
    for key in list(ctx.copies)[before:]:
        t = ctx.copies[key]
        log.info("  copy %s: %s %s", key, getattr(t, "dtype", type(t).__name__), tuple(getattr(t, "shape", ())))
    return Built(model, cfg, ops_by_layer, max(ctx.widths), ctx.max_context - 1, numerics=numerics)
