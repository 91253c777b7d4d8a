"""Symmetric peer memory for the in-kernel tensor-parallel all-reduces.

Reference counterpart: ``common/peer.py:118-165`` (``PeerBuffer``): every rank
allocates one zeroed device buffer, the ranks exchange IPC handles over the host-side
process group (gloo), each opens every peer's buffer, and a device table of the mapped
addresses is what kernels push through.  All ranks refuse together when any rank fails
(``common/peer.py:129-154``).  Here the IPC calls are the library's ``mono_peer_*``
(CUDA IPC); the layout is ``[guard words 256 B][region 0][region 1]`` where a region
holds ``[parity][src rank][16 rows][n/2]`` 8-byte (bf16 pair, tag) words
(``glm53/gfx950/layout.py:224-240``).  Region 0 serves the attention all-reduce,
region 1 the MoE all-reduce (site % 2).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

GUARD_BYTES = 256
N_REGIONS = 2


class CudaIpcBackend:
    """The real backend: ``mono_peer_*`` over CUDA IPC."""

    def __init__(self):
        from .. import _lib as L

        self.L, self.lib = L, L.load()

    def alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.L.check(self.lib.mono_peer_alloc(nbytes, C.byref(p)), "mono_peer_alloc")
        return p.value

    def export(self, ptr: int) -> bytes:
        h = (C.c_ubyte * 64)()
        self.L.check(self.lib.mono_peer_export(ptr, C.byref(h)), "mono_peer_export")
        return bytes(h)

    def open(self, handle: bytes) -> int:
        h = (C.c_ubyte * 64).from_buffer_copy(handle)
        p = C.c_void_p()
        self.L.check(self.lib.mono_peer_open(C.byref(h), C.byref(p)), "mono_peer_open")
        return p.value

    def close(self, ptr: int) -> None:
        self.lib.mono_peer_close(ptr)

    def free(self, ptr: int) -> None:
        self.lib.mono_peer_free(ptr)

    def table(self, values: list[int], device):
        import torch

        return torch.tensor(values, dtype=torch.int64, device=device)


@dataclass
class _Ptr:
    """A raw device address with the ``data_ptr()`` face the launch wrappers use."""

    addr: int

    def data_ptr(self) -> int:
        return self.addr


def region_bytes(n: int, world: int, rows: int = 16) -> int:
    return 2 * world * rows * (n // 2) * 8


class PeerBuffer:
    """Collective constructor: every rank of ``group`` must call it with the same sizes."""

    def __init__(self, n: int, rank: int, world: int, group, device, backend=None, logits_local: int = 0):
        """``logits_local``: this rank's share of the vocabulary when the buffer also carries the LM-head
        tail's logits all-gather (two parity slots of ``[16 rows][vocab / 2]`` words after the two
        all-reduce regions; ``glm53_flash/gfx950/layout.py:193-215``)."""
        import torch.distributed as dist

        self.rank, self.world, self.n, self.device = rank, world, n, device
        self.backend = backend if backend is not None else CudaIpcBackend()
        self.region = region_bytes(n, world)
        self.logits_bytes = 2 * 16 * (world * logits_local // 2) * 8
        self.nbytes = GUARD_BYTES + N_REGIONS * self.region + self.logits_bytes
        self.local = 0
        self.opened: list[int] = []
        ok, handle, why = 1, b"", ""
        try:
            self.local = self.backend.alloc(self.nbytes)
            handle = self.backend.export(self.local)
        except Exception as e:  # every rank must reach the collectives below
            ok, why = 0, f"rank {rank}: {e}"
        infos: list = [None] * world
        dist.all_gather_object(infos, (ok, handle, self.nbytes, why), group=group)
        reasons = [i[3] for i in infos if not i[0]]
        sizes = {i[2] for i in infos}
        if len(sizes) != 1:
            reasons.append(f"ranks disagree on the peer buffer size: {sorted(sizes)}")
        self.ptrs: list[int] = [0] * world
        if not reasons:
            try:
                for r, (_, h, _, _) in enumerate(infos):
                    if r == rank:
                        self.ptrs[r] = self.local
                    else:
                        self.ptrs[r] = self.backend.open(h)
                        self.opened.append(self.ptrs[r])
            except Exception as e:
                reasons.append(f"rank {rank}: {e}")
        # all ranks refuse together: a second round carries late failures (open) to everyone
        late: list = [None] * world
        dist.all_gather_object(late, reasons, group=group)
        all_reasons = sorted({x for lst in late for x in lst})
        if all_reasons:
            self.release()
            raise RuntimeError("peer buffer handshake failed on every rank: " + "; ".join(all_reasons))
        self.guard = _Ptr(self.local)
        self.guard_table = self.backend.table(self.ptrs, device)
        self._regions = [self.backend.table([p + GUARD_BYTES + i * self.region for p in self.ptrs], device)
                         for i in range(N_REGIONS)]
        self.logits_table = None
        if self.logits_bytes:
            self.logits_table = self.backend.table([p + GUARD_BYTES + N_REGIONS * self.region for p in self.ptrs], device)

    def region_table(self, site: int):
        return self._regions[site % N_REGIONS]

    def snapshot(self):
        """This rank's buffer as int64 words on the host (blocking): ``[guard 32 words][region 0][region 1]...``."""
        return _snapshot(self.local, self.nbytes)

    def release(self) -> None:
        for p in self.opened:
            self.backend.close(p)
        self.opened = []
        if self.local:
            self.backend.free(self.local)
            self.local = 0


def _snapshot(ptr: int, nbytes: int):
    import torch

    from .. import _lib as L

    out = torch.empty(nbytes // 8, dtype=torch.int64)
    L.check(L.load().mono_peer_read(out.data_ptr(), ptr, out.numel() * 8), "mono_peer_read")
    return out


class MulticastPeerBuffer:
    """The same buffer over NVLS: symmetric memory bound to an NVLink multicast object, so that a rank's push is one
    ``multimem.st`` that the switch delivers to every rank's copy (the reads, the waits and the rank-ordered sum do
    not change; ``north_star``: "P2P and NVLS-multicast stores").  The allocation, the handle exchange and the
    multicast binding are torch's symmetric memory (``torch.distributed._symmetric_memory``): plumbing, as the
    reference's is HIP IPC.  Collective: every rank of ``group`` builds it with the same sizes; all ranks refuse
    together when the multicast address is missing on any of them (no NVSwitch, or NVLS off)."""

    def __init__(self, n: int, rank: int, world: int, group, device, logits_local: int = 0):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world, self.n, self.device = rank, world, n, device
        self.region = region_bytes(n, world)
        self.logits_bytes = 2 * 16 * (world * logits_local // 2) * 8
        self.nbytes = GUARD_BYTES + N_REGIONS * self.region + self.logits_bytes
        name = group.group_name if hasattr(group, "group_name") else group
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize()
        self.handle = symm_mem.rendezvous(self.buf, name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        oks: list = [None] * world
        dist.all_gather_object(oks, mc != 0, group=group)
        if not all(oks):
            raise RuntimeError(f"NVLS multicast is not available on ranks {[r for r, ok in enumerate(oks) if not ok]}: "
                               "the all-reduce keeps its P2P stores (PeerBuffer)")
        self.mc = mc
        self.local = self.ptrs[rank]
        self.guard = _Ptr(self.local)
        self.guard_table = torch.tensor(self.ptrs, dtype=torch.int64, device=device)
        self._regions = [torch.tensor([p + GUARD_BYTES + i * self.region for p in self.ptrs], dtype=torch.int64, device=device)
                         for i in range(N_REGIONS)]
        self.logits_table = None
        if self.logits_bytes:
            self.logits_table = torch.tensor([p + GUARD_BYTES + N_REGIONS * self.region for p in self.ptrs], dtype=torch.int64,
                                             device=device)

    def region_table(self, site: int):
        return self._regions[site % N_REGIONS]

    def snapshot(self):
        return _snapshot(self.local, self.nbytes)

    def mc_region(self, site: int) -> int:
        """The multicast address of the region ``site`` pushes into."""
        return self.mc + GUARD_BYTES + (site % N_REGIONS) * self.region

    def release(self) -> None:
        self.handle = None
        self.buf = None


def make_peer_buffer(n: int, rank: int, world: int, group, device, logits_local: int = 0, multicast=None):
    """The all-reduce's peer buffer: P2P stores over CUDA IPC, or ``multimem.st`` over NVLS when ``multicast`` is true
    (default: the environment's ``MONO_AR_MULTICAST=1``).  There is no silent fallback: asking for multicast where the
    ranks have none raises on every rank."""
    import os

    if multicast is None:
        multicast = os.environ.get("MONO_AR_MULTICAST") == "1"
    if multicast:
        return MulticastPeerBuffer(n, rank, world, group, device, logits_local=logits_local)
    return PeerBuffer(n, rank, world, group, device, logits_local=logits_local)
