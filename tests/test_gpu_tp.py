"""Tensor parallel layer on 2+ GPUs: both all-reduces run inside the reduce kernel over
IPC-mapped peer buffers (pushes of (bf16 pair, tag) words, rank-ordered local sum).
Checks: error words clean, every rank's output bit-equal, replays bit-equal, and the
result against the CPU oracle over all ranks' weights.  Skipped with fewer than 2 GPUs."""

import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(world, rows, ctx, outdir, env=None):
    import os

    here = Path(__file__).resolve().parent
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, str(here / "tp_worker.py"), str(r), str(world), str(port), str(rows),
                               str(ctx), str(outdir)], env={**os.environ, **(env or {})}) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    got = []
    for r in range(world):
        got.append(torch.load(outdir / f"rank{r}.pt", weights_only=False))
        (outdir / f"rank{r}.pt").unlink()
    return got


@pytest.mark.parametrize("world,rows,ctx", [(2, 5, 350)])
def test_tp_multicast_pushes_give_the_bits_of_the_peer_stores(world, rows, ctx):
    """The NVLS variant (one multimem.st per word, delivered to every rank by the switch) against the P2P variant
    (one st.relaxed.sys per peer): same waits, same local reads, same rank-ordered sum, so the same bits."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    outdir = Path(__file__).resolve().parent / "_tp_out"
    outdir.mkdir(exist_ok=True)
    p2p = _run_ranks(world, rows, ctx, outdir, {"MONO_AR_MULTICAST": "0"})
    mc = _run_ranks(world, rows, ctx, outdir, {"MONO_AR_MULTICAST": "1"})
    for r in range(world):
        assert p2p[r]["rc"] == 0 and mc[r]["rc"] == 0, (p2p[r]["words"], mc[r]["words"])
        for a, b in zip(p2p[r]["outs"], mc[r]["outs"]):
            assert torch.equal(a, b), f"rank {r}: multicast pushes changed the result"
        assert torch.equal(p2p[r]["h1"], mc[r]["h1"])


@pytest.mark.parametrize("world,rows,ctx", [(2, 13, 300)])
def test_tp_reduce_scatter_all_gather_gives_the_bits_of_the_all_to_all_form(world, rows, ctx):
    """13 rows: from 12 rows ``MONO_AR_RSAG=1`` switches both all-reduces of the layer to reduce-scatter + all-gather."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    outdir = Path(__file__).resolve().parent / "_tp_out"
    outdir.mkdir(exist_ok=True)
    a2a = _run_ranks(world, rows, ctx, outdir, {"MONO_AR_RSAG": "0"})
    rsag = _run_ranks(world, rows, ctx, outdir, {"MONO_AR_RSAG": "1"})
    for r in range(world):
        assert a2a[r]["rc"] == 0 and rsag[r]["rc"] == 0, (a2a[r]["words"], rsag[r]["words"])
        for x, y in zip(a2a[r]["outs"], rsag[r]["outs"]):
            assert torch.equal(x, y), f"rank {r}: the rs + ag form changed the result"
        assert torch.equal(a2a[r]["h1"], rsag[r]["h1"])


@pytest.mark.parametrize("world,rows,ctx", [(2, 4, 400), (2, 13, 300), (4, 6, 320)])
def test_tp_layer_ranks_agree_and_match_oracle(world, rows, ctx):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from oracle import layers as OL
    import synth
    from sgl_amd_mono_b200.config import CFG_TINY

    here = Path(__file__).resolve().parent
    outdir = here / "_tp_out"
    outdir.mkdir(exist_ok=True)
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, str(here / "tp_worker.py"), str(r), str(world), str(port), str(rows),
                               str(ctx), str(outdir)]) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    got = {}
    for r in range(world):
        d = torch.load(outdir / f"rank{r}.pt", weights_only=False)
        got[r] = (d["rc"], d["words"], d["outs"], d["w"], d)
        (outdir / f"rank{r}.pt").unlink()
    for r in range(world):
        assert got[r][0] == 0, f"rank {r} guard words {got[r][1]}"
    ref_out = got[0][2]
    for r in range(1, world):
        for a, b in zip(ref_out, got[r][2]):
            assert torch.equal(a, b), f"rank {r} differs from rank 0"
    for o in ref_out[1:]:
        assert torch.equal(o, ref_out[0]), "replays must be bit-equal"
    cfg = CFG_TINY.with_tp(world)
    step = synth.decode_step(cfg, rows, ctx)
    h = torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(1)).bfloat16()
    ws = [got[r][3] for r in range(world)]
    # stage isolation as in test_gpu_layer.py: attention on the kernel's own selection, the MoE
    # half on the kernel's own h1 (a borderline key or expert may fall differently in the oracle)
    from oracle import stages as S
    from util import assert_close_hidden

    d0 = got[0][4]
    for r in range(1, world):
        assert torch.equal(got[r][4]["topk"], d0["topk"]) and torch.equal(got[r][4]["ids"], d0["ids"])
        assert torch.equal(got[r][4]["h1"], d0["h1"])
    live = step.slots >= 0
    parts = []
    for w in ws:
        kvp, ixp = step.kv_pages.clone(), step.idx_pages.clone()
        fr = OL.attn_front(cfg, w, h, step.positions, step.slots, step.cos, step.sin, kvp, ixp)
        parts.append(OL.attn_back(cfg, w, fr, d0["topk"], kvp) * live[:, None])
    h1_ref = S.allreduce_rank_order(parts, h)
    assert_close_hidden(d0["h1"], h1_ref, "h1 after the attention all-reduce",
                        scale=float((h1_ref.float() - h.float()).abs().max()), max_abs=4e-2)
    mparts = []
    for w in ws:
        mp_, ids_o, _, _ = OL.moe_partial(cfg, w, d0["h1"], live)
        mparts.append(mp_)
    assert torch.equal(ids_o, d0["ids"]), "a near-tie flipped between the f32 logit sums: pick another seed"
    ref = S.allreduce_rank_order(mparts, d0["h1"])
    assert_close_hidden(ref_out[0], ref, "layer output after the MoE all-reduce",
                        scale=float((ref.float() - d0["h1"].float()).abs().max()), max_abs=4e-2)


@pytest.mark.parametrize("world,n_layers,rows,ctx", [(2, 6, 7, 130)])
def test_tp_stack_under_one_graph_ranks_agree_and_every_word_carries_its_launchs_tag(world, n_layers, rows, ctx):
    """Six layers + LM head at TP 2 from one CUDA graph, replayed: 13 reductions a step share two regions and one
    parity.  Ranks agree bit for bit, replays repeat the eager step, the guard words stay clean, and afterwards every
    (value, tag) word of the live rows in the slots of the step's parity carries the tag of the LAST launch that uses
    its region (attention sites are even, FFN sites odd: ``tag = epoch * 256 + site + 1``), in every source slot: no
    word of an earlier or later launch is left where a reader of the last one looked."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import os

    here = Path(__file__).resolve().parent
    outdir = here / "_tp_out"
    outdir.mkdir(exist_ok=True)
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, str(here / "tp_stack_worker.py"), str(r), str(world), str(port), str(n_layers),
                               str(rows), str(ctx), str(outdir)], env=dict(os.environ)) for r in range(world)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    got = []
    for r in range(world):
        got.append(torch.load(outdir / f"stack_rank{r}.pt", weights_only=False))
        (outdir / f"stack_rank{r}.pt").unlink()
    for r in range(world):
        assert got[r]["rc"] == 0, f"rank {r} guard words {got[r]['words']}"
        assert got[r]["same"], f"rank {r}: a replay differs from the eager step"
        assert torch.equal(got[r]["x"], got[0]["x"]) and torch.equal(got[r]["logits"], got[0]["logits"])
    assert got[0]["logits"].shape[-1] == 5120 and torch.isfinite(got[0]["logits"]).all()
    # the step ran 1 eager + 1 capture warm-up(s) + 3 replays; the epoch word says how many steps the device saw
    d = got[0]
    n, region_words, gw = d["n"], d["region"] // 8, d["guard_bytes"] // 8
    pairs = n // 2
    for r in range(world):
        snap = got[r]["snap"]
        epoch_now = int(snap[0] & 0xFFFFFFFF)   # guard word 0 (int32) sits in the low half of the first int64
        last_epoch = epoch_now - 1              # the last step's launches read the epoch before its advance
        parity = last_epoch & 1
        for region, site in ((0, 2 * (n_layers - 1)), (1, 2 * (n_layers - 1) + 1)):
            want = last_epoch * 256 + site + 1
            base = gw + region * region_words
            for src in range(world):
                off = base + (parity * world + src) * 16 * pairs
                tags = (snap[off : off + rows * pairs] >> 32) & 0xFFFFFFFF
                assert bool((tags == want).all()), (f"rank {r} region {region} src {src}: tags {sorted(set(tags.tolist()))[:4]}, "
                                                    f"want {want} (epoch {last_epoch}, site {site})")
