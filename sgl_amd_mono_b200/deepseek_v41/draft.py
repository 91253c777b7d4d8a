"""The draft model's spec (reference: ``deepseek_v41/draft.py:245-264``): one MLA + MoE
layer served by the same layer op; its steps carry ``tokens_per_request`` draft rows."""

from __future__ import annotations

from dataclasses import replace

from . import spec as target

SPEC = replace(target.SPEC, name="deepseek_v41_draft_" + target.ISA)
