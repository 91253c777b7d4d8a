"""The in-kernel all-reduce and the guard's failure path on ONE device.

The push / poll / rank-ordered sum of ``reduce_kernel`` (reference ``peer_reduce``,
``glm53/gfx950/kernel.py:1631-1688``) normally needs one GPU per rank.  Here rank r's own
region and W - 1 stand-in peer regions live on the same device, and the host writes the
peers' ``(bf16 pair, tag)`` words for the current epoch into rank r's region before the
launch, so that tags, parity, slot addressing and the summation order are all exercised
by a single launch.

The failure path follows ``test/kernels/test_guard_hip.py`` and ``common/guard.py:100-241``:
a wait whose partner never publishes gives up at its deadline, stores ``site + 1`` in the
deadline word, raises this rank's flag word at every peer, and every later wait returns
at once.  Every wait here is bounded and returns an error status: nothing traps, faults
or waits for ever, and the context stays usable (the tests after a failure launch again).
"""

import ctypes as C
import os
import time

import pytest
import torch

from oracle import quant as Q
from oracle import stages as S
from sgl_amd_mono_b200 import _lib as L
from sgl_amd_mono_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROWS_MAX = L.MAX_ROWS


class OneDeviceRanks:
    """Rank ``rank`` of ``world`` with every region on this device."""

    def __init__(self, world: int, rank: int, n: int):
        self.world, self.rank, self.n = world, rank, n
        words = 2 * world * ROWS_MAX * (n // 2)
        self.regions = [torch.zeros(words, dtype=torch.int64, device=DEV) for _ in range(world)]
        self.guards = [torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=DEV) for _ in range(world)]
        self.ptrs = torch.tensor([t.data_ptr() for t in self.regions], dtype=torch.int64, device=DEV)
        self.gptrs = torch.tensor([t.data_ptr() for t in self.guards], dtype=torch.int64, device=DEV)
        self.guard = self.guards[rank]

    def slot(self, region: torch.Tensor, parity: int, src: int) -> torch.Tensor:
        """[16, n/2] int64 view of ``[parity][src]`` of a region."""
        per = ROWS_MAX * (self.n // 2)
        off = (parity * self.world + src) * per
        return region[off : off + per].view(ROWS_MAX, self.n // 2)

    def publish(self, parity: int, src: int, partial_bf16: torch.Tensor, tag: int) -> None:
        """What rank ``src`` would have pushed into this rank's region: (bf16 pair, tag) words."""
        rows = partial_bf16.shape[0]
        pair = partial_bf16.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        self.slot(self.regions[self.rank], parity, src)[:rows] = (pair | (tag << 32)).to(DEV)

    def launch(self, rows, partial_f32, out, residual, site, deadline_s=5.0, slots=None, rsag=0):
        a = L.ReduceArgs()
        a.rsag = rsag
        a.rows, a.n, a.partial, a.nsum, a.ld = rows, self.n, partial_f32.data_ptr(), partial_f32.shape[0], self.n
        a.sum_stride = ROWS_MAX * self.n
        a.residual, a.out, a.slots = residual.data_ptr(), out.data_ptr(), None if slots is None else slots.data_ptr()
        a.world, a.rank = self.world, self.rank
        a.peer_ptrs, a.peer_guards = self.ptrs.data_ptr(), self.gptrs.data_ptr()
        a.tag, a.parity, a.deadline_ns, a.site, a.guard = 0, 0, int(deadline_s * 1e9), site, self.guard.data_ptr()
        L.check(L.load().mono_reduce_launch(C.byref(a), torch.cuda.current_stream().cuda_stream), "mono_reduce_launch")


def _tag(epoch: int, site: int) -> int:
    return epoch * 256 + site + 1


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 0), (8, 7)])
def test_all_reduce_sum_order_tags_and_parity_on_one_device(world, rank):
    n, rows, nsum = 1024, 5, 3
    g = torch.Generator().manual_seed(100 * world + rank)
    R = OneDeviceRanks(world, rank, n)
    out = torch.zeros(ROWS_MAX, n, dtype=torch.bfloat16, device=DEV)
    for epoch in range(4):
        site = 2 * epoch + (epoch & 1)  # several sites, both regions' worth of tags
        tag, parity = _tag(epoch, site), epoch & 1
        # values whose f32 sum depends on the order they are added in
        parts = [(torch.randn(rows, n, generator=g) * (10.0 ** (r % 3))).float() for r in range(world)]
        mine = torch.zeros(nsum, ROWS_MAX, n)
        split = torch.randn(nsum - 1, rows, n, generator=g)
        mine[: nsum - 1, :rows] = split
        mine[nsum - 1, :rows] = parts[rank] - split.sum(0)
        # the kernel adds its own slices in order before rounding to bf16: restate that here
        acc = torch.zeros(rows, n)
        for s in range(nsum):
            acc = acc + mine[s, :rows]
        parts[rank] = acc
        residual = torch.randn(rows, n, generator=g).bfloat16()
        for src in range(world):
            if src != rank:
                R.publish(parity, src, parts[src].bfloat16(), tag)
        R.launch(rows, mine.to(DEV), out, residual.to(DEV), site)
        torch.cuda.synchronize()
        rc, words = ops.guard_read(R.guard)
        assert rc == 0, f"epoch {epoch}: guard words {words}"
        want = S.allreduce_rank_order(parts, residual)
        assert torch.equal(out[:rows].cpu(), want), f"epoch {epoch}: not the rank-ordered f32 sum"
        # what this rank pushed arrived at every peer, in its own slot, with this launch's tag
        pair = parts[rank].bfloat16().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        for dst in range(world):
            got = R.slot(R.regions[dst], parity, rank)[:rows].cpu()
            assert torch.equal(got, pair | (tag << 32)), f"epoch {epoch}: push to rank {dst}"
            other = R.slot(R.regions[dst], parity ^ 1, rank)[:rows].cpu()
            assert not bool(((other >> 32) == tag).any()), "the other parity's slot is untouched by this launch"
        ops.epoch_advance(R.guard)
    torch.cuda.synchronize()
    assert int(R.guard[0]) == 4


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 2), (8, 5)])
def test_reduce_scatter_all_gather_form_on_one_device(world, rank):
    """The rs + ag form (``minimax_m3/gfx950/layout.py:33-34,97-114``): this rank sums only its own column slice (from
    the partials the others sent it), pushes the FINISHED words of that slice to everybody, and takes the other
    slices' finished words from their owners.  The host plays the other ranks; the result must be the all-to-all
    form's bits, and what this rank sends must be exactly: its partial of slice d to rank d, its finished slice to all."""
    n, rows = 1024, 13
    pairs, ps = n // 2, n // 2 // world
    g = torch.Generator().manual_seed(7 * world + rank)
    R = OneDeviceRanks(world, rank, n)
    out = torch.zeros(ROWS_MAX, n, dtype=torch.bfloat16, device=DEV)
    epoch, site = 0, 3
    tag, parity = _tag(epoch, site), 0
    parts = [(torch.randn(rows, n, generator=g) * (10.0 ** (r % 3))).float().bfloat16().float() for r in range(world)]
    residual = torch.randn(rows, n, generator=g).bfloat16()
    want = S.allreduce_rank_order(parts, residual)  # [rows, n] bf16: what every rank must end with
    mine = torch.zeros(1, ROWS_MAX, n)
    mine[0, :rows] = parts[rank]
    for src in range(world):
        if src == rank:
            continue
        # src's partial of MY slice, and src's finished words of ITS slice, both in slot [src] of my region
        word = torch.zeros(rows, n, dtype=torch.bfloat16)
        word[:, rank * 2 * ps : (rank + 1) * 2 * ps] = parts[src].bfloat16()[:, rank * 2 * ps : (rank + 1) * 2 * ps]
        word[:, src * 2 * ps : (src + 1) * 2 * ps] = want[:, src * 2 * ps : (src + 1) * 2 * ps]
        pair = word.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        full = torch.zeros(rows, pairs, dtype=torch.int64)  # columns of other slices keep tag 0: never read
        for sl in (rank, src):
            full[:, sl * ps : (sl + 1) * ps] = pair[:, sl * ps : (sl + 1) * ps] | (tag << 32)
        R.slot(R.regions[rank], parity, src)[:rows] = full.to(DEV)
    R.launch(rows, mine.to(DEV), out, residual.to(DEV), site, rsag=1)
    torch.cuda.synchronize()
    rc, words = ops.guard_read(R.guard)
    assert rc == 0, f"guard words {words}"
    assert torch.equal(out[:rows].cpu(), want), "the rs + ag form must give the all-to-all form's bits"
    my_pair = parts[rank].bfloat16().contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    fin_pair = want.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    for dst in range(world):
        if dst == rank:
            continue
        got = R.slot(R.regions[dst], parity, rank)[:rows].cpu()
        assert torch.equal(got[:, dst * ps : (dst + 1) * ps], my_pair[:, dst * ps : (dst + 1) * ps] | (tag << 32)), "partial of dst's slice"
        assert torch.equal(got[:, rank * ps : (rank + 1) * ps], fin_pair[:, rank * ps : (rank + 1) * ps] | (tag << 32)), "finished slice"
        rest = [c for c in range(world) if c not in (dst, rank)]
        for c in rest:
            assert not bool(got[:, c * ps : (c + 1) * ps].any()), "nothing else is sent: half the bytes per link"
    # refused where the slices do not divide
    a = L.ReduceArgs()
    a.rows, a.n, a.partial, a.nsum, a.ld, a.sum_stride = 1, 1000, mine.to(DEV).data_ptr(), 1, 1000, ROWS_MAX * 1000
    a.out, a.world, a.rank, a.peer_ptrs, a.deadline_ns, a.guard, a.rsag = out.data_ptr(), 8, 0, R.ptrs.data_ptr(), 10**9, R.guard.data_ptr(), 1
    assert L.load().mono_reduce_launch(C.byref(a), torch.cuda.current_stream().cuda_stream) == -1  # MONO_E_ARG


def test_a_wait_that_runs_out_sets_the_words_flags_the_peers_and_later_launches_drain():
    world, rank, n, rows, site = 4, 1, 512, 3, 6
    R = OneDeviceRanks(world, rank, n)
    g = torch.Generator().manual_seed(5)
    R.guard[0] = 2  # epoch 2: parity 0
    tag = _tag(2, site)
    part = torch.zeros(1, ROWS_MAX, n, device=DEV)
    residual = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(ROWS_MAX, n, dtype=torch.bfloat16, device=DEV)
    # ranks 0 and 3 publish this launch's words; rank 2's slot still holds the words of epoch 0 (same
    # parity, stale tag).  Were a stale tag taken for a current one, the launch would succeed.
    R.publish(0, 0, torch.randn(rows, n, generator=g).bfloat16(), tag)
    R.publish(0, 3, torch.randn(rows, n, generator=g).bfloat16(), tag)
    R.publish(0, 2, torch.randn(rows, n, generator=g).bfloat16(), _tag(0, site))
    t0 = time.perf_counter()
    R.launch(rows, part, out, residual, site, deadline_s=0.05)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert dt < 2.0, f"the launch took {dt:.2f} s: the deadline did not bound the wait"
    rc, words = ops.guard_read(R.guard)
    assert rc == -4, f"mono_guard_read returned {rc}, wants MONO_E_GUARD"
    assert words[0] == site + 1, f"deadline word {words[0]}, wants site + 1 = {site + 1}"
    for peer in range(world):
        flag = int(R.guards[peer][L.GUARD_FLAGS + rank])
        assert flag == (0 if peer == rank else 1), f"flag word of rank {rank} at rank {peer}: {flag}"
    # every later wait returns at once: a second launch with nothing published drains immediately
    t0 = time.perf_counter()
    R.launch(rows, part, out, residual, site + 1, deadline_s=30.0)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0, "a launch after a failure must not wait"
    rc, words2 = ops.guard_read(R.guard)
    assert words2[0] == site + 1, "the first failure's site stays in the sticky word"


def test_a_peer_flag_stops_this_rank():
    world, rank, n, rows = 2, 0, 256, 2
    R = OneDeviceRanks(world, rank, n)
    R.guard[L.GUARD_FLAGS + 1] = 1  # rank 1 has failed and raised its flag here
    part = torch.zeros(1, ROWS_MAX, n, device=DEV)
    residual = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(ROWS_MAX, n, dtype=torch.bfloat16, device=DEV)
    t0 = time.perf_counter()
    R.launch(rows, part, out, residual, 0, deadline_s=20.0)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0, "the flag, not the deadline, must end the wait"
    rc, words = ops.guard_read(R.guard)
    assert rc != 0 and words[1] == 2 and words[0] == 0, f"peer word {words}: wants rank 1 + 1 in the peer word only"


def _chained_ffn(deadline_s):
    import synth
    from sgl_amd_mono_b200.config import CFG_TINY
    from sgl_amd_mono_b200.moe import MoeFfn
    from dataclasses import replace

    cfg = replace(CFG_TINY, n_heads=0, index_heads=0, inter=256)
    w = synth.layer_weights(cfg, 0, DEV)
    os.environ["MONO_MOE_CHAINED"] = "1"
    try:
        ffn = MoeFfn(cfg, w, DEV, deadline_s=deadline_s)
    finally:
        del os.environ["MONO_MOE_CHAINED"]
    assert ffn.chained is not None
    x = torch.randn(4, cfg.hidden, generator=torch.Generator().manual_seed(3)).bfloat16().to(DEV)
    return ffn, x


def test_a_ready_stamp_that_never_comes_gives_up_and_the_next_launch_is_clean():
    """Chained expert launch: one slot's task counter is pre-loaded so that its "last task" count is never
    reached and its ready stamp never written.  The down job's bounded wait on that stamp gives up after
    the launch's wait limit, the launch drains with the deadline word set (TMEM freed: the next launch
    allocates it again), and once the host clears the words and counters the same op computes the
    same result as an undisturbed one."""
    ffn, x = _chained_ffn(deadline_s=0.05)
    good = ffn(x).clone()
    torch.cuda.synchronize()
    rc, words = ops.guard_read(ffn.guard)
    assert rc == 0, words
    assert ffn.chained.args.wait_ns == 50_000_000
    # the routed up job's counters: [slots]; slot 0 can never reach its count from -1000
    done = ffn.chained._chain_words[-2]
    assert done.numel() == ffn.max_expert
    done[0] = -1000
    t0 = time.perf_counter()
    ffn(x)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert dt < 2.0, f"the launch took {dt:.2f} s: the wait limit did not bound the wait"
    rc, words = ops.guard_read(ffn.guard)
    assert rc != 0 and words[0] == 102, f"guard words {words}: wants the GEMV's deadline code 102 (site 101 + 1)"
    assert int(done.abs().sum()) == 0, "the last CTA to leave a failed launch puts the counters back to zero"
    # host-side recovery, then a clean launch with the same bits as before
    ffn.guard.zero_()
    ffn.chained.reset_chain()
    again = ffn(x).clone()
    torch.cuda.synchronize()
    rc, words = ops.guard_read(ffn.guard)
    assert rc == 0, words
    assert torch.equal(again, good)


def test_fault_injection_switch_is_host_side(monkeypatch):
    """``MONO_FAULT_INJECT=rank:site[:after]`` (reference ``SGLANG_AMD_MONO_FAULT_INJECT``,
    ``common/guard.py:79-88``) makes the HOST of that rank skip the launch that would publish at
    ``site`` from its ``after``-th step on, so the other ranks' waits at that site run out.  Here rank 1
    of 2 is the injected one; rank 0 (this process) sees the deadline at that site."""
    from sgl_amd_mono_b200.common import guard as G

    monkeypatch.setenv("MONO_FAULT_INJECT", "1:4:2")
    assert G.fault_injection(0) is None
    assert G.fault_injection(1) == (4, 2)
    inj = G.FaultInjector(1)
    assert [inj.skip(4) for _ in range(3)] == [False, False, True]  # the third step at site 4 and later ones
    assert not inj.skip(5)
    world, n, rows, site = 2, 256, 2, 4
    R = OneDeviceRanks(world, 0, n)
    part = torch.zeros(1, ROWS_MAX, n, device=DEV)
    residual = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(ROWS_MAX, n, dtype=torch.bfloat16, device=DEV)
    peer = G.FaultInjector(1)
    for step in range(3):
        R.guard[0] = step
        if not peer.skip(site):  # the peer's host publishes unless the switch tells it to skip
            R.publish(step & 1, 1, torch.ones(rows, n).bfloat16(), _tag(step, site))
        R.launch(rows, part, out, residual, site, deadline_s=0.05)
        torch.cuda.synchronize()
        rc, words = ops.guard_read(R.guard)
        assert (rc == 0) == (step < 2), f"step {step}: {words}"
    assert words[0] == site + 1


def test_max_resident_ctas_and_the_refusal_of_an_oversized_chained_grid():
    ffn, x = _chained_ffn(deadline_s=1.0)
    res = ffn.chained.max_resident_ctas()
    assert res == L.load().mono_sm_count(), "the tcgen05 GEMV keeps one CTA per SM resident"
    ffn.chained.args.max_ctas = res + 1
    with pytest.raises(RuntimeError, match="resident"):
        ffn(x)
    ffn.chained.args.max_ctas = 0
    ffn(x)
    torch.cuda.synchronize()
    assert ops.guard_read(ffn.guard)[0] == 0


@pytest.mark.parametrize("world,rank,nsum", [(1, 0, 3), (2, 1, 1), (4, 0, 2), (8, 5, 1)])
def test_logits_all_gather_on_one_device(world, rank, nsum):
    """The LM-head tail's K-split sum and all-gather (``glm53_flash/gfx950/kernel.py:3700-3770``): this rank's
    f32 partial sums are added in order, rounded to bf16 and pushed to every rank's logits region; the other
    ranks' words (written by the host here) are widened to f32 ``[rows, vocab]``."""
    rows, nl = 6, 1280
    vocab = world * nl
    g = torch.Generator().manual_seed(7 * world + rank)
    words = 2 * ROWS_MAX * (vocab // 2)
    regions = [torch.zeros(words, dtype=torch.int64, device=DEV) for _ in range(world)]
    guards = [torch.zeros(L.GUARD_WORDS, dtype=torch.int32, device=DEV) for _ in range(world)]
    ptrs = torch.tensor([t.data_ptr() for t in regions], dtype=torch.int64, device=DEV)
    gptrs = torch.tensor([t.data_ptr() for t in guards], dtype=torch.int64, device=DEV)
    out = torch.full((ROWS_MAX, vocab), float("nan"), device=DEV)
    for epoch in range(3):
        guards[rank][0] = epoch
        tag, parity = _tag(epoch, 254), epoch & 1
        shares = [torch.randn(rows, nl, generator=g) * 3 for _ in range(world)]
        mine = torch.zeros(nsum, ROWS_MAX, nl)
        mine[:, :rows] = torch.randn(nsum, rows, nl, generator=g)
        acc = torch.zeros(rows, nl)
        for s in range(nsum):
            acc = acc + mine[s, :rows]
        shares[rank] = acc
        slot = regions[rank][parity * ROWS_MAX * (vocab // 2) : (parity + 1) * ROWS_MAX * (vocab // 2)].view(ROWS_MAX, vocab // 2)
        for src in range(world):
            if src != rank:
                pair = shares[src].bfloat16().contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
                slot[:rows, src * nl // 2 : (src + 1) * nl // 2] = (pair | (tag << 32)).to(DEV)
        a = L.LogitsGatherArgs()
        part = mine.to(DEV)
        a.rows, a.n_local, a.partial, a.nsum, a.ld, a.sum_stride = rows, nl, part.data_ptr(), nsum, nl, ROWS_MAX * nl
        a.out, a.out_ld, a.world, a.rank = out.data_ptr(), vocab, world, rank
        a.peer_ptrs, a.peer_guards = ptrs.data_ptr(), gptrs.data_ptr()
        a.tag, a.parity, a.deadline_ns, a.site, a.guard = 0, 0, int(5e9), 254, guards[rank].data_ptr()
        L.check(L.load().mono_logits_gather_launch(C.byref(a), torch.cuda.current_stream().cuda_stream), "mono_logits_gather_launch")
        torch.cuda.synchronize()
        assert ops.guard_read(guards[rank])[0] == 0
        want = torch.cat(shares, 1) if world == 1 else torch.cat([x.bfloat16().float() for x in shares], 1)
        assert torch.equal(out[:rows].cpu(), want), f"epoch {epoch}"
        if world > 1:  # this rank's share arrived at every other rank with this launch's tag
            pair = shares[rank].bfloat16().contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
            for dst in range(world):
                if dst == rank:
                    continue
                got = regions[dst][parity * ROWS_MAX * (vocab // 2) : (parity + 1) * ROWS_MAX * (vocab // 2)]
                got = got.view(ROWS_MAX, vocab // 2)[:rows, rank * nl // 2 : (rank + 1) * nl // 2].cpu()
                assert torch.equal(got, pair | (tag << 32)), f"epoch {epoch}: push to rank {dst}"


def test_lm_head_wide_step_sums_k_splits_in_a_kernel():
    """More than 8 rows: the head's K is split, and the gather launch (not a torch op) adds the splits."""
    from sgl_amd_mono_b200.tail import LmHeadOp

    g = torch.Generator().manual_seed(11)
    hidden, vocab, rows = 1024, 5000, 13
    w = (torch.randn(vocab, hidden, generator=g) * 0.02).bfloat16()
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
    h = torch.randn(rows, hidden, generator=g).bfloat16()
    op = LmHeadOp(hidden, w.to(DEV), gamma.to(DEV), 1e-6, DEV)
    got = op(h.to(DEV))
    torch.cuda.synchronize()
    _, buf, ns = op.gemv[True]
    if ns > 1:
        want = torch.zeros_like(buf[0, :rows])
        for s in range(ns):
            want = want + buf[s, :rows]
        assert got.data_ptr() == op.gathered.data_ptr()
        assert torch.equal(got, want), "the K splits are added in order"
    ref = S.tail_logits(h, gamma, 1e-6, w)
    assert float((got.cpu() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("world,rank,n", [(1, 0, 2048), (2, 1, 7168), (8, 3, 1024), (4, 0, 512)])
def test_reduce_fused_with_the_norm_staging_matches_the_two_launches(world, rank, n):
    """``mono_reduce_norm_launch``: the reduction (+ all-reduce over host-written peer words + residual) and the RMSNorm
    staging of its output in one launch.  The reduced rows are the bits of ``mono_reduce_launch`` (live and pad rows,
    pushes at every peer); the staged values follow ``mono_act_prep_launch`` up to the last bit of the reciprocal root
    (a row's sum of squares is added per CTA of its cluster, then in CTA order)."""
    rows, nsum, site = 4, 11, 5
    g = torch.Generator().manual_seed(31 * world + rank)
    parts = [torch.randn(rows, n, generator=g) * 4 for _ in range(world)]
    for p in parts:
        p[2] = 0  # row 2 is a pad row on every rank
    mine = torch.zeros(nsum, ROWS_MAX, n)
    mine[:, :rows] = torch.randn(nsum, rows, n, generator=g)
    residual = torch.randn(rows, n, generator=g).bfloat16().to(DEV)
    gamma = (1 + 0.1 * torch.randn(n, generator=g)).bfloat16().to(DEV)
    slots = torch.tensor([5, 9, -1, 77], dtype=torch.int64, device=DEV)
    part = mine.to(DEV)
    got = {}
    for fused in (False, True):
        R = OneDeviceRanks(max(world, 1), rank, n)
        R.guard[0] = 3
        for src in range(world):
            if src != rank:
                R.publish(1, src, parts[src].bfloat16(), _tag(3, site))
        out = torch.zeros(ROWS_MAX, n, dtype=torch.bfloat16, device=DEV)
        dst = ops.ActBuf(L.ACT_HILO, n, DEV)
        xbf = torch.zeros(ROWS_MAX, n, dtype=torch.bfloat16, device=DEV)
        peer = None
        if world > 1:
            peer = type("P", (), {"world": world, "rank": rank, "guard_table": R.gptrs, "region_table": lambda self, s: R.ptrs})()
        pend = ops.PendingReduce(rows, n, part, nsum, out, residual, slots, peer, site, R.guard, 5.0)
        if fused:
            ops.reduce_norm(pend, dst, gamma=gamma, eps=1e-6, out_bf16=xbf)
        else:
            pend.launch()
            ops.act_prep(rows, n, dst, src_bf16=out[:rows], gamma=gamma, eps=1e-6, out_bf16=xbf)
        torch.cuda.synchronize()
        assert ops.guard_read(R.guard)[0] == 0
        got[fused] = (out.clone(), xbf.clone(), dst,
                      [R.slot(R.regions[d], 1, rank)[:rows].cpu().clone() for d in range(max(world, 1))])
    assert torch.equal(got[False][0], got[True][0]) and bool(got[True][0].float().abs().sum() > 0)
    assert torch.equal(got[True][0][2], residual[2]), "a pad row's partial sums count as zero"
    a, b = got[False][1].float(), got[True][1].float()
    assert float((a - b).abs().max()) <= 2.0**-7 * float(a.abs().max()), "normalised rows: at most one bf16 ulp apart"
    assert float((a != b).float().mean()) < 0.01
    # the planes hold hi + lo = the bf16 value / scale
    d = got[True][2]
    val = (Q.e4m3_from_bytes(d.planes[0, 0, :rows, :n].cpu()) + Q.e4m3_from_bytes(d.planes[0, 1, :rows, :n].cpu()))
    val = val.reshape(rows, n // 128, 128) * d.scale_f32[0, :rows, : n // 128].cpu()[..., None]
    x = got[True][1][:rows].float().cpu()
    # exact for values within 2^12 of their 128-chunk's largest; the smallest lose their last bits
    assert float((val.reshape(rows, n) - x).abs().max()) <= 2.0**-11 * float(x.abs().max())
    assert float((val.reshape(rows, n) == x).float().mean()) > 0.95
    if world > 1:
        for a, b in zip(got[False][3], got[True][3]):
            assert torch.equal(a, b) and bool((a >> 32 == _tag(3, site)).all())
