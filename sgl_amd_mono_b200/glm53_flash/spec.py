"""A registered spec that refuses every configuration with its reason (reference:
``glm53_flash/spec.py``; the model-specific stages listed in the package docstring are not built)."""

from __future__ import annotations

from ..registry import DeviceLimits, MonoSpec, Numerics, NumericsKind, Requirements
from ..spec_common import ISA, ROWS, SM_COUNT, TP_SIZES

REASON = "glm53_flash: this model's layer stages are not built for " + ISA + " in this library"


def _build(model, hf_config, ctx):
    raise RuntimeError(REASON)


SPEC = MonoSpec(
    name="glm53_flash_" + ISA,
    devices={ISA: DeviceLimits(widths=ROWS, tp_sizes=TP_SIZES, resident_blocks=SM_COUNT)},
    features=frozenset(),
    requires=Requirements(),
    numerics=Numerics(NumericsKind.TOLERANCE, {}),
    model_disable_reasons=lambda model, hf_config, copies: [REASON],
    build=_build,
    api_version=1,
    config_disable_reasons=lambda cfg, hf_config: [REASON],
)
