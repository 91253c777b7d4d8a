"""The device-side producer of per-row step tables (``minimax_m3/metadata.py``) against the reference's own
outputs (golden fixture) and the CPU restatement; on a GPU: captured into a CUDA graph, fresh on every replay."""

from pathlib import Path

import pytest
import torch

from oracle import host as H
from sgl_amd_mono_b200.minimax_m3.metadata import TokenRows, prepare_token_rows


@pytest.fixture(scope="module")
def golden():
    return torch.load(Path(__file__).resolve().parent / "golden" / "reference_host.pt", weights_only=False)


def test_rows_match_the_references_output(golden):
    a = golden["rows_in"]
    bt = torch.full_like(golden["rows_block_table"], 7)
    sl = torch.full_like(golden["rows_seq_lens"], 7)
    prepare_token_rows(a["req_to_token"], a["pool"], a["seq_lens"], a["cols"], bt, sl, a["slot_mapping"], a["query_len"], True,
                       a["max_context_len"])
    assert torch.equal(bt, golden["rows_block_table"]) and torch.equal(sl, golden["rows_seq_lens"])


@pytest.mark.parametrize("query_len,is_verify", [(1, False), (5, True), (3, True)])
def test_rows_match_the_cpu_restatement_on_random_steps(query_len, is_verify):
    g = torch.Generator().manual_seed(query_len)
    n_req, ctx = 4, 2048
    req_to_token = torch.stack([torch.randperm(ctx * 2, generator=g)[:ctx] for _ in range(9)]).to(torch.int32)
    pool = torch.randperm(9, generator=g)[:n_req]
    seq_lens = torch.randint(1, ctx - 8, (n_req,), generator=g, dtype=torch.int32)
    seq_lens[0] = ctx - 2  # a verify request that runs into the context limit
    rows = n_req * query_len
    slots = torch.randint(1, 5000, (rows,), generator=g)
    slots[1 % rows] = 0
    slots[rows - 1] = -1
    cols = torch.arange(0, ctx, 128)
    bt, sl = torch.zeros(rows, cols.numel(), dtype=torch.int32), torch.zeros(rows, dtype=torch.int32)
    prepare_token_rows(req_to_token, pool, seq_lens, cols, bt, sl, slots, query_len, is_verify, ctx)
    want_bt, want_sl = H.causal_rows(req_to_token, pool, seq_lens, cols, slots, query_len, is_verify, ctx)
    assert torch.equal(bt, want_bt) and torch.equal(sl, want_sl)
    assert int(sl.max()) <= ctx and sl[1 % rows] == 0 and sl[rows - 1] == 0 and not bt[rows - 1].any()


def test_block_size_of_this_librarys_caches_and_refusals():
    req_to_token = torch.arange(2 * 512, dtype=torch.int32).reshape(2, 512)
    tr = TokenRows(4, 512, "cpu", block_tokens=64)
    bt, sl = tr(req_to_token, torch.tensor([1, 0]), torch.tensor([100, 9], dtype=torch.int32), torch.tensor([3, 4, 5, 6]), 2, True)
    assert bt.shape == (4, 8) and bt[0].tolist() == [8 + i for i in range(8)] and bt[2].tolist() == list(range(8))
    assert sl.tolist() == [101, 102, 10, 11]
    with pytest.raises(ValueError, match="whole requests"):
        prepare_token_rows(req_to_token, torch.tensor([1]), torch.tensor([5], dtype=torch.int32), tr.block_columns,
                           torch.zeros(3, 8, dtype=torch.int32), torch.zeros(3, dtype=torch.int32), torch.ones(3), 2, True, 512, 64)


@pytest.mark.gpu
def test_rows_are_fresh_on_every_replay_of_a_captured_graph():
    dev = "cuda:0"
    ctx, q = 1024, 4
    req_to_token = torch.arange(6 * ctx, dtype=torch.int32, device=dev).reshape(6, ctx)
    pool = torch.tensor([4, 1], device=dev)
    seq_lens = torch.tensor([300, 17], dtype=torch.int32, device=dev)
    slots = torch.tensor([5, 6, 7, 0, 9, 10, -1, 12], device=dev)
    tr = TokenRows(8, ctx, dev, block_tokens=64)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        tr(req_to_token, pool, seq_lens, slots, q, True)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            tr(req_to_token, pool, seq_lens, slots, q, True)
    torch.cuda.current_stream().wait_stream(s)
    for lens, pl in (([300, 17], [4, 1]), ([511, 40], [0, 5])):
        seq_lens.copy_(torch.tensor(lens, dtype=torch.int32))
        pool.copy_(torch.tensor(pl))
        g.replay()
        torch.cuda.synchronize()
        want_bt, want_sl = H.causal_rows(req_to_token.cpu(), pool.cpu(), seq_lens.cpu(), tr.block_columns.cpu(), slots.cpu(), q, True, ctx)
        want_bt = (req_to_token.cpu()[pool.cpu().repeat_interleave(q)][:, tr.block_columns.cpu()] // 64).to(torch.int32)
        want_bt[(slots.cpu() <= 0)] = 0
        assert torch.equal(tr.seq_lens.cpu(), want_sl)
        assert torch.equal(tr.block_table.cpu(), want_bt)
