"""CPU restatement of the decoder-layer monokernel arithmetic (TEST INFRASTRUCTURE ONLY).

This package is the parity oracle: plain PyTorch on CPU, fp32 math with bf16 / FP8 / FP4
rounding wherever the reference's device code rounds.  It is never imported by the
product package; only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s
``cpu_baseline`` / ``--impl reference`` legs may use it, and only as the checker or
as the timed CPU baseline.

Pinning.  The reference's kernels (FlyDSL -> gfx950) cannot be built or imported
without FlyDSL, AITER, SGLang and an AMD GPU, so the device arithmetic is restated
from the cited source lines.  The parts of the reference that are pure host Python
(``glm53/check.py`` radix keys, ``deepseek_v41/gfx950/weights.py`` E8M0 / MXFP8
helpers and rope table, ``glm53_flash/check.py`` tail, ``minimax_m3/metadata.py``
causal rows, ``glm53/gfx950/layout.py`` select slices) were imported and run to
generate the fixtures under ``tests/golden/`` (see ``tests/golden/make_golden.py``);
the oracle is checked against those.  Everything that the reference only states as
device code is "parity unpinned" against the reference's binaries and pinned to the
cited formulas instead.
"""
