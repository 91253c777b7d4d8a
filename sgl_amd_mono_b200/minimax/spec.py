"""The dispatcher spec of ``MiniMaxM3Sparse*`` (reference: ``minimax/spec.py:59-99``)."""

from __future__ import annotations

from dataclasses import replace

from ..minimax_m3 import spec as m3
from ..minimax_m31 import spec as m31
from ..spec_common import ISA


def _pick(hf_config):
    return m31.SPEC if m31.is_m31(hf_config) else m3.SPEC


SPEC = replace(
    m31.SPEC,
    name="minimax_" + ISA,
    config_disable_reasons=lambda cfg, hf_config: _pick(hf_config).config_disable_reasons(cfg, hf_config),
    model_disable_reasons=lambda model, hf_config, copies: _pick(hf_config).model_disable_reasons(model, hf_config, copies),
    build=lambda model, hf_config, ctx: _pick(hf_config).build(model, hf_config, ctx),
)
