"""One rank of the tensor-parallel stack test (run as a child process by test_gpu_tp.py):
python tests/tp_stack_worker.py RANK WORLD PORT LAYERS ROWS CTX OUTDIR"""

import os
import sys
from dataclasses import replace
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main(rank, world, port, n_layers, rows, ctx, outdir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import synth
        from sgl_amd_mono_b200 import ops
        from sgl_amd_mono_b200.common.peer import GUARD_BYTES, make_peer_buffer
        from sgl_amd_mono_b200.config import CFG_TINY
        from sgl_amd_mono_b200.layer import StepTables
        from sgl_amd_mono_b200.stack import DecoderStack

        dev = f"cuda:{rank}"
        cfg = replace(CFG_TINY, name="tiny_flash", index_heads=0, vocab=5120).with_tp(world)
        peer = make_peer_buffer(cfg.hidden, rank, world, dist.group.WORLD, dev, logits_local=cfg.vocab // world)
        ws = [synth.layer_weights(cfg if i == n_layers - 1 else replace(cfg, vocab=0), rank, dev, layer=i) for i in range(n_layers)]
        t = lambda x: x.to(dev)  # noqa: E731
        tables = []
        for i in range(n_layers):
            s = synth.verify_step(cfg, rows, 1, ctx, layer=i)
            tables.append(StepTables(t(s.positions), t(s.slots), t(s.page_table), t(s.kv_pages), None, t(s.cos), t(s.sin)))
        st = DecoderStack(cfg, ws, dev, max_ctx=-(-ctx // 64) * 64, peer=peer, deadline_s=10.0)
        h = t(torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(3)).bfloat16())
        dist.barrier()
        x0, logits0 = st.step(h, tables)
        x0, logits0 = x0.clone(), logits0.clone()
        torch.cuda.synchronize()
        dist.barrier()
        st.capture(h, tables)
        same = True
        for _ in range(3):
            dist.barrier()
            x, logits = st.replay()
            torch.cuda.synchronize()
            same = same and torch.equal(x, x0) and torch.equal(logits, logits0)
        rc, words = ops.guard_read(st.guard)
        dist.barrier()
        snap = peer.snapshot()
        torch.save(dict(rc=rc, words=words, same=same, x=x0.cpu(), logits=logits0.cpu(), snap=snap, region=peer.region,
                        guard_bytes=GUARD_BYTES, n=cfg.hidden, rows=rows, world=world, n_layers=n_layers),
                   Path(outdir) / f"stack_rank{rank}.pt")
        dist.barrier()
        peer.release()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = sys.argv[1:]
    main(int(a[0]), int(a[1]), int(a[2]), int(a[3]), int(a[4]), int(a[5]), a[6])
