"""The FFN-only spec (reference: ``minimax_m31/spec.py:441-455``)."""

from __future__ import annotations

from ..config import LayerConfig
from ..registry import DeviceLimits, Feature, MonoSpec, Numerics, NumericsKind, Requirements
from ..spec_common import ISA, ROWS, SM_COUNT, TP_SIZES, Built, config_reasons, log

NUMERICS = Numerics(NumericsKind.TOLERANCE, {"ffn.out.cosine": 0.999, "ffn.out.max_abs": 2e-2, "ffn.ids.max_abs": 0.0})


def nvfp4_experts(hf_config) -> bool:
    """MiniMax-M3.1-Flash's checkpoint: NVFP4 experts (``moe_quant_algo``; reference: minimax_m31/spec.py:116-121).
    The reference hands those experts to SGLang's MoE runner; here they are a weight kind of the expert launches
    (E2M1 values ``w13`` / ``w2``, E4M3 scale bytes per 16 ``w13_s`` / ``w2_s``, f32 scales per expert ``w13_g`` / ``w2_g``)."""
    quant = getattr(hf_config, "quantization_config", None) or {}
    return isinstance(quant, dict) and str(quant.get("moe_quant_algo", "")).upper() == "NVFP4"


def layer_config(hf_config, tp: int) -> LayerConfig:
    g = lambda k: getattr(hf_config, k)  # noqa: E731
    return LayerConfig(name="minimax_m31_" + ISA, hidden=g("hidden_size"), n_experts=g("n_routed_experts"),
                       top_k=g("num_experts_per_tok"), inter=g("moe_intermediate_size"),
                       route_scale=g("routed_scaling_factor"), expert_fmt="nvfp4" if nvfp4_experts(hf_config) else "mxfp4",
                       shared_fmt=getattr(hf_config, "shared_expert_format", "bf16"), router_dtype="f32",
                       eps=g("rms_norm_eps"), tp=tp)


def is_m31(hf_config) -> bool:
    """M3.1 checkpoints carry 4-bit routed experts: MXFP4, or NVFP4 (reference: minimax_m31/spec.py:116-121)."""
    quant = getattr(hf_config, "quantization_config", None) or {}
    return quant.get("quant_method") in ("mxfp4", "mxfp4_mxfp8") or nvfp4_experts(hf_config)


def _config_disable_reasons(cfg, hf_config) -> list[str]:
    reasons = config_reasons("the FFN kernels", {"scoring_func": "sigmoid"}, cfg, hf_config)
    if getattr(hf_config, "hidden_size", 0) % 256 or getattr(hf_config, "moe_intermediate_size", 0) % 256:
        reasons.append("4-bit expert tiles need hidden and intermediate sizes that are multiples of 256")
    if getattr(cfg, "moe_ep_size", 1) != 1:
        reasons.append("expert parallelism is not served (reference: minimax_m3/spec.py:262-266)")
    return reasons


def _build(model, hf_config, ctx):
    from .runner import FfnRunner

    c = layer_config(hf_config, ctx.tp_size)
    ops = {i: FfnRunner(c, layer.weights, ctx.device, deadline_s=ctx.deadline_s, copies=ctx.copies, layer=i)
           for i, layer in enumerate(model.layers)}
    log.info("%s: %d FFN launches, widths %s", c.name, len(ops), ctx.widths)
    return Built(model, c, ops, max(ctx.widths), ctx.max_context - 1)


SPEC = MonoSpec(
    name="minimax_m31_" + ISA,
    devices={ISA: DeviceLimits(widths=ROWS, tp_sizes=TP_SIZES, resident_blocks=SM_COUNT)},
    features=frozenset({Feature.SPECULATIVE_DECODING, Feature.EAGLE3_HIDDEN_STATES}),
    requires=Requirements(dtypes=frozenset({"bfloat16"})),
    numerics=NUMERICS,
    model_disable_reasons=lambda model, hf_config, copies: [],
    build=_build,
    api_version=1,
    config_disable_reasons=_config_disable_reasons,
)
