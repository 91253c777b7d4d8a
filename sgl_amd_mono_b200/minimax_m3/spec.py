"""Refuses until the GQA block-sparse attention stages exist (reference: ``minimax_m3/spec.py``)."""

from __future__ import annotations

from ..registry import DeviceLimits, MonoSpec, Numerics, NumericsKind, Requirements
from ..spec_common import ISA, ROWS, SM_COUNT, TP_SIZES

REASON = "minimax_m3: the GQA block-sparse attention stages are not built for " + ISA + " yet"

SPEC = MonoSpec(
    name="minimax_m3_" + ISA,
    devices={ISA: DeviceLimits(widths=ROWS, tp_sizes=(4,), resident_blocks=SM_COUNT)},
    features=frozenset(), requires=Requirements(), numerics=Numerics(NumericsKind.TOLERANCE, {}),
    model_disable_reasons=lambda model, hf_config, copies: [REASON],
    build=lambda model, hf_config, ctx: (_ for _ in ()).throw(RuntimeError(REASON)),
    api_version=1, config_disable_reasons=lambda cfg, hf_config: [REASON],
)
