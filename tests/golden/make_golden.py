"""Generates ``reference_host.pt``: outputs of the reference's own importable host
functions on small seeded inputs.  Run where the reference tree is mounted:

    PYTHONPATH=<reference root> python tests/golden/make_golden.py

Only pure-host modules of the reference import without FlyDSL / AITER / SGLang; its
device kernels cannot run here, so these vectors pin the oracle's integer rules
(radix key order, E8M0 codes, exact MXFP8 re-quantisation, rope table layout,
causal verify rows, select slices) and the f32 tail, nothing more.
"""

from __future__ import annotations

from pathlib import Path
from types import SimpleNamespace

import torch

from sgl_amd_mono.deepseek_v41.gfx950 import weights as v41w
from sgl_amd_mono.glm53 import check as glm_check
from sgl_amd_mono.glm53.gfx950.layout import select_slices
from sgl_amd_mono.glm53_flash import check as flash_check
from sgl_amd_mono.minimax_m3.metadata import prepare_token_rows

OUT = Path(__file__).resolve().parent / "reference_host.pt"


def main() -> None:
    g = torch.Generator().manual_seed(0)
    fx: dict = {}
    # radix keys of f32 score bits (glm53/check.py:94-97)
    scores = torch.cat([torch.randn(500, generator=g), torch.tensor([0.0, -0.0, 1e-30, -1e-30, 3.5, 3.5, -7.25])])
    bits = scores.view(torch.int32)
    fx["radix_bits"], fx["radix_keys"] = bits, glm_check._radix_keys(bits)
    # E8M0 codes of power-of-two block scales (deepseek_v41/gfx950/weights.py:7-15)
    e = torch.randint(-20, 10, (6, 5), generator=g).float()
    fx["e8m0_scale"], fx["e8m0_code"] = torch.exp2(e), v41w.e8m0(torch.exp2(e), "fixture")
    # exact MXFP8 re-quantisation of a bf16 weight (deepseek_v41/gfx950/weights.py:18-35)
    q0 = (torch.randn(64, 96, generator=g) * 40).clamp(-448, 448).to(torch.float8_e4m3fn)
    q0.view(torch.uint8)[::32, ::32] = 0x7E  # pin each 32 x 32 block's amax to 448 so the scale is unique
    sc = torch.exp2(torch.randint(-12, -2, (2, 3), generator=g).float())
    wbf = (q0.float() * sc.repeat_interleave(32, 0).repeat_interleave(32, 1)).to(torch.bfloat16)
    q, codes = v41w.mxfp8_exact(wbf, "fixture")
    fx["mx8_w"], fx["mx8_q"], fx["mx8_code"] = wbf, q.view(torch.uint8), codes
    # rope table layout (deepseek_v41/gfx950/weights.py:38-48)
    ang = torch.arange(16, dtype=torch.float64)[:, None] * 10000.0 ** (-torch.arange(32, dtype=torch.float64) / 32)
    fc = torch.polar(torch.ones_like(ang), ang).to(torch.complex64)
    fx["rope_freqs_cis"], fx["rope_table"] = fc, v41w.rope_table(fc, [])
    # f32 tail (glm53_flash/check.py:284-302) with one stream: post = 1, comb = 0
    x = torch.randn(3, 256, generator=g).bfloat16()
    owed = SimpleNamespace(x=x, residual=torch.zeros(3, 1, 256), post=torch.ones(3, 1), comb=torch.zeros(3, 1, 1))
    gn = (1 + 0.1 * torch.randn(256, generator=g)).bfloat16()
    wh = (torch.randn(40, 256, generator=g) * 0.02).bfloat16()
    fx["tail_x"], fx["tail_gamma"], fx["tail_w"] = x, gn, wh
    fx["tail_logits"] = flash_check.tail_fp32(owed, gn, 1e-6, wh)
    # causal verify rows (minimax_m3/metadata.py:7-42)
    req_to_token = torch.arange(4 * 1024, dtype=torch.int32).reshape(4, 1024)
    pool = torch.tensor([2, 0], dtype=torch.int64)
    seq_lens = torch.tensor([300, 17], dtype=torch.int32)
    cols = torch.arange(0, 1024, 128)
    slot_mapping = torch.tensor([5, 6, 7, 0, 9, 10, -1, 12], dtype=torch.int64)
    bt = torch.zeros(8, 8, dtype=torch.int32)
    sl = torch.zeros(8, dtype=torch.int32)
    prepare_token_rows(req_to_token, pool, seq_lens, cols, bt, sl, slot_mapping, 4, True, 302)
    fx["rows_in"] = dict(req_to_token=req_to_token, pool=pool, seq_lens=seq_lens, cols=cols,
                         slot_mapping=slot_mapping, query_len=4, max_context_len=302)
    fx["rows_block_table"], fx["rows_seq_lens"] = bt, sl
    # select slices (glm53/gfx950/layout.py:47-53)
    bounds = [1, 4096, 4097, 32769, 65536, 65537, 131072, 262192, (1 << 20) - 1, 1 << 20]
    fx["slice_bounds"] = bounds
    fx["slices"] = [select_slices(b) for b in bounds]
    # exact top-k of a row's own scores (glm53/check.py:100-117 `_exact_topk_outputs`): the reference's checker counts
    # how many keys of ITS exact top-k (radix keys, stable descending sort = ties to the lowest position) a selection
    # misses.  Stored: the inputs, the reference's own top-2048 slot sets, and the checker's answer on the selection
    # the oracle (oracle/stages.py exact_topk_positions) makes from the same scores.
    import sys

    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
    from oracle import stages as S  # the restatement under test

    from sgl_amd_mono.glm53.gfx950.runner import TOPK

    rows, n_max, per = 4, 6000, -(-6000 // 64)
    sc = torch.randn(rows, n_max, generator=g)
    sc[1] = sc[1].round()             # long runs of exact ties around the threshold
    sc[2, ::2] = -0.5                 # ties among negative scores
    sc[3, :2100] = torch.linspace(4, -4, 2100)
    positions = torch.tensor([5999, 4000, 2500, 2099])  # row 3 sees 2100 keys: 52 more than TOPK
    page_table = (torch.randperm(rows * per, generator=g) + 1).to(torch.int32).reshape(rows, per)
    picked, indptr, ref_sets = [], [0], []
    for r in range(rows):
        n = int(positions[r]) + 1
        pos = S.exact_topk_positions(sc[r], n, TOPK)
        picked += S.slots_of_positions(page_table[r], pos).tolist()
        indptr.append(len(picked))
        keys = glm_check._radix_keys(sc[r, :n].contiguous().view(torch.int32))
        ref_pos = torch.sort(keys, descending=True, stable=True).indices[:TOPK]
        ref_sets.append(sorted((page_table[r, ref_pos // 64].long() * 64 + ref_pos % 64).tolist()))
    step = SimpleNamespace(indptr=torch.tensor(indptr), topk=torch.tensor(picked), positions=positions,
                           page_table=page_table, req_ids=torch.arange(rows))
    answer = glm_check._exact_topk_outputs(step, sc.view(torch.int32), rows)
    assert answer == {"topk_exact": {"max_abs": 0.0}}, answer
    fx["topk_scores"], fx["topk_positions"], fx["topk_page_table"] = sc, positions, page_table
    fx["topk_k"], fx["topk_ref_sets"], fx["topk_checker_verdict"] = TOPK, ref_sets, answer
    torch.save(fx, OUT)
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
