"""The peer-buffer handshake and the rank-ordered all-reduce arithmetic on CPU ranks
(gloo, world size 2 and 3) with a fake IPC backend: every rank ends with the same
address table, a failing rank makes all ranks refuse together, and the emulated
push / rank-ordered sum gives bit-identical results on every rank and matches the oracle."""

import os
import socket
import struct

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import stages as S


class FakeBackend:
    """Addresses are (rank + 1) << 32; handles carry the owner's address."""

    def __init__(self, rank, fail_alloc=False, fail_open_of=None):
        self.rank, self.fail_alloc, self.fail_open_of = rank, fail_alloc, fail_open_of
        self.closed, self.freed = [], []

    def alloc(self, nbytes):
        if self.fail_alloc:
            raise RuntimeError("out of memory (injected)")
        return (self.rank + 1) << 32

    def export(self, ptr):
        return struct.pack("<Q", ptr).ljust(64, b"\0")

    def open(self, handle):
        addr = struct.unpack("<Q", handle[:8])[0]
        if self.fail_open_of is not None and addr == (self.fail_open_of + 1) << 32:
            raise RuntimeError("cannot map the peer (injected)")
        return addr + 0x1000  # a mapping differs from the owner's own address

    def close(self, ptr):
        self.closed.append(ptr)

    def free(self, ptr):
        self.freed.append(ptr)

    def table(self, values, device):
        return torch.tensor(values, dtype=torch.int64)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sgl_amd_mono_b200.common.peer import GUARD_BYTES, PeerBuffer, region_bytes

    try:
        if mode == "ok":
            pb = PeerBuffer(1024, rank, world, dist.group.WORLD, "cpu", backend=FakeBackend(rank))
            want = [((r + 1) << 32) + (0 if r == rank else 0x1000) for r in range(world)]
            assert pb.guard_table.tolist() == want
            assert pb.region_table(0).tolist() == [p + GUARD_BYTES for p in want]
            assert pb.region_table(3).tolist() == [p + GUARD_BYTES + region_bytes(1024, world) for p in want]
            assert pb.guard.data_ptr() == (rank + 1) << 32
            # the all-reduce arithmetic: every rank pushes its bf16 partial, sums in rank order
            g = torch.Generator().manual_seed(100 + rank)
            part = torch.randn(4, 1024, generator=g)
            parts = [torch.empty(4, 1024, dtype=torch.bfloat16) for _ in range(world)]
            dist.all_gather(parts, part.bfloat16())  # stands in for the in-kernel pushes
            res = torch.zeros(4, 1024)
            got = S.allreduce_rank_order([p.float() for p in parts], res)
            ref = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(ref, got)
            assert all(torch.equal(ref[0], r) for r in ref), "ranks must agree bit for bit"
            # the reduce-scatter + all-gather form: the owner of a column slice sums the partials it was sent in
            # rank order, adds the residual, and everybody takes the finished slice from its owner
            res = torch.randn(4, 1024, generator=torch.Generator().manual_seed(7)).bfloat16()
            want = S.allreduce_rank_order([p.float() for p in parts], res)
            sl = 1024 // world if 1024 % world == 0 else None
            if sl is not None:
                mine = S.allreduce_rank_order([p.float()[:, rank * sl : (rank + 1) * sl] for p in parts], res[:, rank * sl : (rank + 1) * sl])
                slices = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(slices, mine.contiguous())  # stands in for the owners' pushes of finished words
                assert torch.equal(torch.cat(slices, 1), want), "rs + ag must give the all-to-all form's bits"
            out.put((rank, "ok"))
        else:
            be = FakeBackend(rank, fail_alloc=(mode == "alloc" and rank == 1),
                             fail_open_of=(0 if mode == "open" and rank == world - 1 else None))
            try:
                PeerBuffer(1024, rank, world, dist.group.WORLD, "cpu", backend=be)
                out.put((rank, "built"))
            except RuntimeError as e:
                assert "every rank" in str(e)
                assert ("injected" in str(e))
                out.put((rank, "refused"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(2, "ok"), (3, "ok"), (2, "alloc"), (3, "open")])
def test_peer_handshake(world, mode):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = dict(out.get(timeout=10) for _ in range(world))
    want = "ok" if mode == "ok" else "refused"
    assert got == {r: want for r in range(world)}


def test_rs_ag_switch(monkeypatch):
    """``ops.rsag_wanted``: off by default at every row count; ``MONO_AR_RSAG=1`` from 12 rows (the reference's switch
    point, ``minimax_m3/gfx950/layout.py:33-34``) where the column slices divide evenly; ``always`` for every step."""
    from sgl_amd_mono_b200 import ops

    monkeypatch.delenv("MONO_AR_RSAG", raising=False)
    assert not ops.rsag_wanted(16, 7168, 8)
    monkeypatch.setenv("MONO_AR_RSAG", "1")
    assert ops.rsag_wanted(12, 7168, 8) and ops.rsag_wanted(16, 6144, 4) and not ops.rsag_wanted(11, 7168, 8)
    assert not ops.rsag_wanted(16, 7168, 1), "one rank has nothing to scatter"
    assert not ops.rsag_wanted(16, 1000, 8), "1000 / 2 pairs do not split into 8 even slices of whole pairs"
    monkeypatch.setenv("MONO_AR_RSAG", "always")
    assert ops.rsag_wanted(1, 7168, 2)
