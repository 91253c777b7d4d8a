"""Check mode's comparisons on CPU (reference: ``glm53/check.py:60-117,239-278``): metrics by the NUMERICS names, every
broken bound listed, the exact top-k of a launch's own scores, and the poison of not-yet-written index rows."""

import pytest
import torch

from sgl_amd_mono_b200 import check
from sgl_amd_mono_b200.config import IDX_PAGE_BYTES, PAGE
from sgl_amd_mono_b200.glm53.spec import NUMERICS


def test_metrics_and_bounds():
    g = torch.Generator().manual_seed(0)
    ref = torch.randn(4, 256, generator=g)
    got = ref + 1e-3 * torch.randn(4, 256, generator=g)
    kv = torch.randint(0, 255, (3, 576), dtype=torch.uint8, generator=g)
    m = check.compare(7, NUMERICS, {"out": got, "kv_rows": kv, "topk_missed": 0.0, "router_rows_off": 0.0},
                      {"out": ref, "kv_rows": kv.clone()})
    assert m["layer.streams.cosine"] > 0.9999 and m["layer.kv.bytes.max_abs"] == 0.0
    kv2 = kv.clone()
    kv2[1, 5] += 1
    with pytest.raises(check.CheckError) as e:
        check.compare(7, NUMERICS, {"out": ref * -1, "kv_rows": kv2, "topk_missed": 3.0}, {"out": ref, "kv_rows": kv})
    text = str(e.value)
    assert text.startswith("layer 7:") and "layer.streams.cosine" in text and "layer.kv.bytes.max_abs = 1" in text
    assert "layer.topk_exact.max_abs = 3" in text and "layer.streams.max_abs" in text


def test_topk_missed_counts_against_the_exact_selection_of_the_launchs_own_scores():
    g = torch.Generator().manual_seed(1)
    n, k = 700, 256
    scores = torch.randn(2, 704, generator=g)
    scores[1, ::3] = 0.5  # ties at and around the threshold
    positions = torch.tensor([n - 1, n - 1])
    slots = torch.tensor([5, -1])
    pt = (torch.randperm(22, generator=g) + 1).to(torch.int32).reshape(2, 11)
    from oracle import stages as S

    picked = torch.full((2, k), -1, dtype=torch.int32)
    picked[0] = S.slots_of_positions(pt[0], S.exact_topk_positions(scores[0], n, k)).to(torch.int32)
    assert check.topk_missed(scores, positions, slots, pt, picked, k) == 0.0
    slots[1] = 9
    picked[1] = S.slots_of_positions(pt[1], S.exact_topk_positions(scores[1], n, k)).to(torch.int32)
    assert check.topk_missed(scores, positions, slots, pt, picked, k) == 0.0
    picked[1, 10] = -1
    assert check.topk_missed(scores, positions, slots, pt, picked, k) == 1.0
    scores[0, 3] = float("nan")  # a poisoned row that was read
    assert check.topk_missed(scores, positions, slots, pt, picked, k) == float(k)


def test_router_rows_and_poison():
    sc = torch.tensor([[0.9, 0.1, 0.5, 0.5], [0.2, 0.8, 0.7, 0.1]])
    ids = torch.tensor([[0, 2], [1, 2]], dtype=torch.int32)
    live = torch.tensor([True, True])
    assert check.router_rows_off(sc, None, ids, 2, live) == 0.0  # the tie 0.5 / 0.5 goes to the lower id
    assert check.router_rows_off(sc, None, torch.tensor([[0, 3], [1, 2]], dtype=torch.int32), 2, live) == 1.0
    assert check.router_rows_off(sc, torch.tensor([0.0, 0.0, 0.0, 1.0]), torch.tensor([[3, 0], [3, 1]], dtype=torch.int32), 2, live) == 0.0
    pages = torch.zeros(3, IDX_PAGE_BYTES, dtype=torch.uint8)
    check.poison_index_rows(pages, torch.tensor([PAGE + 2, -1]))
    assert pages[1, PAGE * 64 + 8 : PAGE * 64 + 12].tolist() == [255] * 4 and int(pages.sum()) == 4 * 255


def test_enabled_reads_the_switch(monkeypatch):
    monkeypatch.delenv("MONO_CHECK", raising=False)
    assert not check.enabled()
    monkeypatch.setenv("MONO_CHECK", "1")
    assert check.enabled()
