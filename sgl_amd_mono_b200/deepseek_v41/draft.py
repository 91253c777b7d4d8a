"""The draft model's spec (reference: ``deepseek_v41/draft.py``): each stage is the target's layer on the draft's
route and window.  The draft routes 128 experts top-3 (``draft.py:34``) and attends a 128-token window plus the keys of
its own block of rows, without an index source or a top-k (``draft.py:35``, ``:225-227``); its steps carry
``tokens_per_request`` rows a request, run as a verify batch (``draft.py:175-209``)."""

from __future__ import annotations

from dataclasses import replace

from ..registry import DeviceLimits, MonoSpec
from ..spec_common import ISA, SM_COUNT, build_layers
from . import spec as target

EXPERTS, TOPK = 128, 3  # the draft's route
WINDOW = 128            # a row's window, before the block's own keys
MAX_BLOCK = 16          # rows of one step (the block's keys a row may also see)


def layer_config(hf_config, tp: int):
    """The target's layer shapes with the draft's route and a window of WINDOW + MAX_BLOCK keys."""
    c = target.layer_config(hf_config, tp)
    return replace(c, name="deepseek_v41_draft_" + ISA, n_experts=EXPERTS, top_k=TOPK, index_heads=0, window=WINDOW + MAX_BLOCK,
                   vocab=0)


def _build(model, hf_config, ctx):
    from ..layer import MlaLayerOp

    c = layer_config(hf_config, ctx.tp_size)
    peer = None
    if ctx.tp_size > 1:
        from ..common.peer import PeerBuffer

        peer = PeerBuffer(c.hidden, ctx.tp_rank, ctx.tp_size, ctx.cpu_group, ctx.device)

    def make(i, w):
        return MlaLayerOp(c, w, ctx.device, max_ctx=ctx.max_context, peer=peer, guard=peer.guard if peer else None,
                          layer=i, deadline_s=ctx.deadline_s, max_rows=max(ctx.widths), copies=ctx.copies)

    stages = getattr(model, "stages", None)
    n = len(stages) if stages is not None else hf_config.num_hidden_layers
    return build_layers(model, c, ctx, list(range(n)), make)


SPEC = MonoSpec(
    name="deepseek_v41_draft_" + ISA,
    # the draft runs where its target does; the reference serves it at TP 2 and 4 (draft.py:249-253)
    devices={ISA: DeviceLimits(widths=target.SPEC.devices[ISA].widths, tp_sizes=(1, 2, 4), resident_blocks=SM_COUNT)},
    features=target.SPEC.features,
    requires=target.SPEC.requires,
    numerics=target.NUMERICS,
    model_disable_reasons=target._model_disable_reasons,
    build=_build,
    api_version=1,
    config_disable_reasons=target._config_disable_reasons,
    tokens_per_request=target._tokens_per_request,
)
