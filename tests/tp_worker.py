"""One rank of the tensor-parallel layer test (run as a child process by test_gpu_tp.py):
python tests/tp_worker.py RANK WORLD PORT ROWS CTX OUTDIR"""

import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main(rank, world, port, rows, ctx, outdir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import synth
        from sgl_amd_mono_b200 import ops
        from sgl_amd_mono_b200.common.peer import make_peer_buffer
        from sgl_amd_mono_b200.config import CFG_TINY
        from sgl_amd_mono_b200.layer import MlaLayerOp, StepTables

        dev = f"cuda:{rank}"
        cfg = CFG_TINY.with_tp(world)
        # MONO_AR_MULTICAST=1: the pushes go out as multimem.st through the switch instead of one store per peer
        peer = make_peer_buffer(cfg.hidden, rank, world, dist.group.WORLD, dev)
        w = synth.layer_weights(cfg, rank, dev)
        step = synth.decode_step(cfg, rows, ctx)
        t = lambda x: x.to(dev)  # noqa: E731
        tables = StepTables(t(step.positions), t(step.slots), t(step.page_table), t(step.kv_pages), t(step.idx_pages),
                            t(step.cos), t(step.sin))
        h = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(1)).bfloat16()
        op = MlaLayerOp(cfg, w, dev, max_ctx=-(-ctx // 64) * 64, peer=peer, guard=peer.guard, deadline_s=10.0)
        outs = []
        for _ in range(4):  # replays: the epoch word advances, tags and parity slots change
            dist.barrier()
            outs.append(op.launch(t(h), tables).clone())
            ops.epoch_advance(op.guard)
            torch.cuda.synchronize()
        rc, words = ops.guard_read(op.guard)
        dist.barrier()
        torch.save(dict(rc=rc, words=words, outs=[o.cpu() for o in outs], w={k: v.cpu() for k, v in w.items()},
                        h1=op.h1[:rows].cpu(), topk=op.topk_slots[:rows].cpu(), ids=op.ffn.ids[:rows].cpu(),
                        scores=op.ffn.scores[:rows].cpu()),
                   Path(outdir) / f"rank{rank}.pt")
        dist.barrier()
        peer.release()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = sys.argv[1:]
    main(int(a[0]), int(a[1]), int(a[2]), int(a[3]), int(a[4]), a[5])
