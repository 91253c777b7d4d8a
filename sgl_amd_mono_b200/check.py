"""Check mode: every covered layer's launch is compared with the model's own layer as it runs.

Reference counterpart: ``glm53/check.py`` (``SGLANG_AMD_MONO_CHECK=1``; ``reference`` ``:183-236``, ``compare``
``:239-278``, ``_exact_topk_outputs`` ``:100-117``, ``_metrics`` ``:60-82``) and its use in the routed forward
(``glm53/spec.py:402-417``): outside CUDA-graph capture the layer's input rows are also run through SGLang's own
layer, and the launch's output stream, the cache rows it wrote and its selection are held to the bounds the spec
declares in ``NUMERICS``.  Here the switch is ``MONO_CHECK=1``; the comparison is plain torch on whatever
device the tensors live on, and it raises ``CheckError`` listing every bound that was exceeded.

What is compared, by the names the specs' ``NUMERICS`` tables use:

  layer.streams.cosine / max_abs   the output rows against the reference layer's (cosine is a lower bound)
  layer.kv.bytes.max_abs           the KV-cache rows the step wrote, byte for byte, against the reference's rows
  layer.index.bytes.max_abs        the index-key rows the step wrote
  layer.topk_exact.max_abs         keys of the exact top-k of the launch's OWN scores that its selection misses
  layer.router_ids.max_abs         rows whose expert ids differ from the exact top-k of the launch's own scores

The index-key rows a step is about to write are poisoned first (their scale codes set to the E8M0 NaN code):
a stage that read a row of this step before the step wrote it would turn its scores into NaN, which the
selection check then reports (``glm53/check.py:77-82``).
"""

from __future__ import annotations

import os

import torch

from .config import IDX_PAGE_BYTES, KV_DIM, PAGE

ENV = "MONO_CHECK"
POISON_CODE = 0xFF  # E8M0 NaN


class CheckError(AssertionError):
    pass


def enabled() -> bool:
    """Check mode is on (never inside a CUDA-graph capture: a captured step replays device work only)."""
    return os.environ.get(ENV) == "1" and not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing())


def _radix_keys(bits: torch.Tensor) -> torch.Tensor:
    b = bits.to(torch.int64)
    return torch.where(b >= 0, b + (1 << 31), ~b & 0xFFFFFFFF)


def stream_metrics(got: torch.Tensor, ref: torch.Tensor) -> dict:
    g, r = got.float().flatten(), ref.float().flatten()
    if not torch.isfinite(g).all():
        return {"cosine": float("-inf"), "max_abs": float("inf")}
    return {"cosine": float(torch.nn.functional.cosine_similarity(g, r, dim=0)), "max_abs": float((g - r).abs().max())}


def topk_missed(scores: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                picked: torch.Tensor, k: int) -> float:
    """Over the live rows with more than ``k`` keys: the most keys of the exact top-k of the launch's own ``scores``
    (radix-key order, ties to the lowest position) that the row's selection ``picked`` (global KV slots, -1 = none)
    misses.  NaN scores (a poisoned row that was read) count as a whole row missed."""
    missed = 0
    for s in range(positions.shape[0]):
        n = int(positions[s]) + 1
        if int(slots[s]) < 0 or n <= k:
            continue
        row = scores[s, :n].float()
        if torch.isnan(row).any():
            return float(k)
        keys = _radix_keys(row.contiguous().view(torch.int32))
        pos = torch.sort(keys, descending=True, stable=True).indices[:k]
        want = set((page_table[s, pos // PAGE].long() * PAGE + pos % PAGE).tolist())
        missed = max(missed, len(want - set(picked[s].tolist())))
    return float(missed)


def router_rows_off(scores: torch.Tensor, bias, ids: torch.Tensor, top_k: int, live: torch.Tensor) -> float:
    """Rows whose expert ids are not the exact top-k of the launch's own sigmoid scores + bias (ties to the lower id)."""
    key = scores.float() if bias is None else scores.float() + bias.float()
    want = torch.sort(key, dim=-1, descending=True, stable=True).indices[..., :top_k]
    bad = (want.to(ids.dtype) != ids).any(-1) & live
    return float(bad.sum())


def poison_index_rows(idx_pages: torch.Tensor, slots: torch.Tensor) -> None:
    """Sets the scale codes of the index-key rows at ``slots`` (>= 0) to the NaN code, before the launch that writes them."""
    for slot in slots.tolist():
        if slot >= 0:
            p, o = divmod(int(slot), PAGE)
            idx_pages[p, PAGE * 64 + o * 4 : PAGE * 64 + (o + 1) * 4] = POISON_CODE


def written_rows(kv_pages: torch.Tensor, idx_pages, slots: torch.Tensor):
    """(KV rows [n, 576] bytes, their f32 scales, index rows [n, 68] bytes) at the live slots, in row order."""
    kv, sc, ix = [], [], []
    for slot in slots.tolist():
        if slot < 0:
            continue
        p, o = divmod(int(slot), PAGE)
        kv.append(kv_pages[p, o * KV_DIM : (o + 1) * KV_DIM])
        sc.append(kv_pages[p, PAGE * KV_DIM :].view(torch.float32)[o])
        if idx_pages is not None:
            assert idx_pages.shape[-1] == IDX_PAGE_BYTES
            ix.append(torch.cat([idx_pages[p, o * 64 : (o + 1) * 64], idx_pages[p, PAGE * 64 + o * 4 : PAGE * 64 + (o + 1) * 4]]))
    return (torch.stack(kv) if kv else None, torch.stack(sc) if sc else None, torch.stack(ix) if ix else None)


def compare(layer: int, numerics, got: dict, ref: dict) -> dict:
    """``got`` / ``ref``: dicts with any of ``out``, ``kv_rows``, ``index_rows`` (tensors) and, in ``got`` only,
    ``topk_missed`` / ``router_rows_off`` (numbers from the functions above).  Returns the metrics; raises ``CheckError``
    naming every bound of ``numerics`` (a ``Numerics`` with ``.bounds``) that a metric breaks."""
    m: dict = {}
    if "out" in got and "out" in ref:
        sm = stream_metrics(got["out"], ref["out"])
        m["layer.streams.cosine"], m["layer.streams.max_abs"] = sm["cosine"], sm["max_abs"]
    for name, key in (("layer.kv.bytes.max_abs", "kv_rows"), ("layer.index.bytes.max_abs", "index_rows")):
        if got.get(key) is not None and ref.get(key) is not None:
            m[name] = float((got[key].to(torch.int16) - ref[key].to(torch.int16)).abs().max())
    if "topk_missed" in got:
        m["layer.topk_exact.max_abs"] = float(got["topk_missed"])
    if "router_rows_off" in got:
        m["layer.router_ids.max_abs"] = float(got["router_rows_off"])
    broken = []
    for name, value in m.items():
        if name not in numerics.bounds:
            continue
        bound = numerics.bound(name)
        ok = value >= bound if name.endswith("cosine") else value <= bound
        if not ok:
            broken.append(f"{name} = {value:.6g} (bound {bound})")
    if broken:
        raise CheckError(f"layer {layer}: " + "; ".join(broken))
    return m


def check_layer_launch(layer: int, numerics, op, h, tables, ref_layer):
    """Runs ``op.launch(h, tables)`` under check mode: poisons the step's index rows, launches, and compares with
    ``ref_layer(h, tables) -> {"out": ..., "kv_rows": ..., "index_rows": ...}`` (the model's own layer on the same rows,
    on caches of its own).  Returns (output, metrics)."""
    rows = h.shape[0]
    if tables.idx_pages is not None:
        poison_index_rows(tables.idx_pages, tables.slots[:rows])
    ref = ref_layer(h, tables)
    out = op.launch(h, tables)
    if isinstance(out, torch.Tensor) is False:  # a deferred reduction: check mode settles it here
        out = out.launch()
    torch.cuda.synchronize()
    kv_rows, _, ix_rows = written_rows(tables.kv_pages, tables.idx_pages, tables.slots[:rows])
    got = {"out": out, "kv_rows": kv_rows, "index_rows": ix_rows}
    cfg = op.cfg
    if cfg.index_heads:
        got["topk_missed"] = topk_missed(op.scores[:rows], tables.positions[:rows], tables.slots[:rows],
                                         tables.page_table[:rows], op.topk_slots[:rows], cfg.index_topk)
    if op.ffn is not None:
        got["router_rows_off"] = router_rows_off(op.ffn.scores[:rows], op.w.get("router_bias"), op.ffn.ids[:rows], cfg.top_k,
                                                 tables.slots[:rows] >= 0)
    return out, compare(layer, numerics, got, ref)
