"""The spec of the flash-sized MLA + MoE model (reference: ``deepseek_v41/spec.py:1207-1258``)."""

from __future__ import annotations

from ..config import LayerConfig
from ..registry import DeviceLimits, Feature, MonoSpec, Numerics, NumericsKind, Requirements
from ..spec_common import ISA, ROWS, SM_COUNT, TP_SIZES, build_layers, config_reasons
from . import HF_CONFIG

NUMERICS = Numerics(NumericsKind.TOLERANCE, {
    "layer.streams.cosine": 0.999, "layer.streams.max_abs": 2e-2, "layer.kv.bytes.max_abs": 0.0,
    "layer.router_ids.max_abs": 0.0,
})


def layer_config(hf_config, tp: int) -> LayerConfig:
    g = lambda k: getattr(hf_config, k)  # noqa: E731
    return LayerConfig(
        name="deepseek_v41_" + ISA, hidden=g("hidden_size"), n_heads=g("num_attention_heads"), q_lora=g("q_lora_rank"),
        nope=g("qk_nope_head_dim"), rope=g("qk_rope_head_dim"), v_head=g("v_head_dim"), index_heads=0,
        n_experts=g("n_routed_experts"), top_k=g("num_experts_per_tok"), inter=g("moe_intermediate_size"),
        route_scale=g("routed_scaling_factor"), expert_fmt="fp8_block", shared_fmt="fp8_block",
        eps=g("rms_norm_eps"), tp=tp, vocab=getattr(hf_config, "vocab_size", 0))


def _config_disable_reasons(cfg, hf_config) -> list[str]:
    keys = {k: HF_CONFIG[k] for k in ("kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "scoring_func")}
    return config_reasons("the MLA kernels", keys, cfg, hf_config)


def _model_disable_reasons(model, hf_config, copies: dict) -> list[str]:
    return []


def _tokens_per_request(model) -> int:
    return getattr(model, "tokens_per_request", 1)


def _build(model, hf_config, ctx):
    from ..layer import MlaLayerOp

    c = layer_config(hf_config, ctx.tp_size)
    peer = None
    if ctx.tp_size > 1:
        from ..common.peer import PeerBuffer

        peer = PeerBuffer(c.hidden, ctx.tp_rank, ctx.tp_size, ctx.cpu_group, ctx.device)

    def make(i, w):
        return MlaLayerOp(c, w, ctx.device, max_ctx=ctx.max_context, peer=peer, guard=peer.guard if peer else None,
                          layer=i, deadline_s=ctx.deadline_s, max_rows=max(ctx.widths))

    return build_layers(model, c, ctx, list(range(hf_config.num_hidden_layers)), make)


SPEC = MonoSpec(
    name="deepseek_v41_" + ISA,
    devices={ISA: DeviceLimits(widths=ROWS, tp_sizes=TP_SIZES, resident_blocks=SM_COUNT)},
    features=frozenset({Feature.SPECULATIVE_DECODING, Feature.RAGGED_VERIFY}),
    requires=Requirements(dtypes=frozenset({"bfloat16"}), server_args={"kv_cache_dtype": frozenset({"fp8_e4m3"})}),
    numerics=NUMERICS,
    model_disable_reasons=_model_disable_reasons,
    build=_build,
    api_version=1,
    config_disable_reasons=_config_disable_reasons,
    tokens_per_request=_tokens_per_request,
)
