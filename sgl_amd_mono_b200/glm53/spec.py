"""The spec of the MLA + DSA + MoE model and its build (reference: ``glm53/spec.py``)."""

from __future__ import annotations

from ..config import CFG_V3, LayerConfig
from ..registry import DeviceLimits, Feature, MonoSpec, Numerics, NumericsKind, Requirements
from ..spec_common import ISA, ROWS, SM_COUNT, TP_SIZES, build_layers, config_reasons, weight_reasons
from . import HF_CONFIG

TOPK = 2048
PAGE_SIZE = 64

# bounds of a covered layer against the model's own layer (reference: glm53/spec.py:154-165)
NUMERICS = Numerics(NumericsKind.TOLERANCE, {
    "layer.streams.cosine": 0.999,
    "layer.streams.max_abs": 2e-2,
    "layer.kv.bytes.max_abs": 0.0,
    "layer.index.bytes.max_abs": 0.0,
    "layer.topk_exact.max_abs": 0.0,
    "layer.router_ids.max_abs": 0.0,
})


def layer_config(hf_config, tp: int) -> LayerConfig:
    g = lambda k: getattr(hf_config, k)  # noqa: E731
    return LayerConfig(
        name="glm53_" + ISA, hidden=g("hidden_size"), n_heads=g("num_attention_heads"), q_lora=g("q_lora_rank"),
        kv_lora=g("kv_lora_rank"), nope=g("qk_nope_head_dim"), rope=g("qk_rope_head_dim"), v_head=g("v_head_dim"),
        index_heads=g("index_n_heads"), index_topk=g("index_topk"), n_experts=g("n_routed_experts"),
        top_k=g("num_experts_per_tok"), inter=g("moe_intermediate_size"), route_scale=g("routed_scaling_factor"),
        expert_fmt="fp8_block", shared_fmt="fp8_block", eps=g("rms_norm_eps"), tp=tp)


def _covered_layers(hf_config) -> list[int]:
    """The MoE layers (reference: glm53/spec.py:168-170)."""
    return list(range(getattr(hf_config, "first_k_dense_replace", 0), hf_config.num_hidden_layers))


def _config_disable_reasons(cfg, hf_config) -> list[str]:
    shape_keys = {k: v for k, v in HF_CONFIG.items() if k in (
        "kv_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "scoring_func", "index_head_dim",
        "rope_interleave", "hidden_act")}
    reasons = config_reasons("the MLA kernels", shape_keys, cfg, hf_config, PAGE_SIZE)
    quant = getattr(hf_config, "quantization_config", None) or {}
    if quant.get("quant_method") != "fp8" or list(quant.get("weight_block_size") or ()) != [128, 128]:
        reasons.append(f"needs the FP8 block-128 checkpoint, got {quant.get('quant_method')!r} "
                       f"{quant.get('weight_block_size')!r}")
    if getattr(hf_config, "index_n_heads", 0) > 64:
        reasons.append("the index scorer serves at most 64 index heads")
    if getattr(cfg, "speculative_algorithm", None) is not None and getattr(cfg, "speculative_eagle_topk", 1) != 1:
        reasons.append("verify steps need one draft chain per request (topk 1)")
    return reasons


def _bound(model, hf_config, tp: int, copies: dict, i: int) -> dict:
    """Layer i's tensors: bound to SGLang's modules (``weights.layer_weights``), or the ``weights`` dict a
    stand-alone synthetic model carries."""
    from ..spec_common import model_layers
    from .weights import layer_weights

    layer = model_layers(model)[i]
    if isinstance(getattr(layer, "weights", None), dict):
        return layer.weights
    return layer_weights(layer, i, layer_config(hf_config, tp), copies)


def _model_disable_reasons(model, hf_config, copies: dict) -> list[str]:
    """Every reason the loaded model cannot be read in place (reference: ``glm53/spec.py:215-251``): each covered
    layer's tensors go through the binding's checks, and a failed check is a reason naming the layer and the tensor."""
    import torch

    tp = getattr(model, "tp_size", 1)
    c = layer_config(hf_config, tp)
    hl, il, h = c.heads_local, c.inter_local, c.hidden
    u8, f32, bf = torch.uint8, torch.float32, torch.bfloat16
    reasons = []
    for i in _covered_layers(hf_config):
        try:
            w = _bound(model, hf_config, tp, {}, i)  # a dry run: its copies are dropped
        except (ValueError, AttributeError) as e:
            reasons.append(f"layer {i}: {e}")
            continue
        reasons += weight_reasons(i, w, {
            "qkv_a": (u8, (c.q_lora + 576, h)), "qkv_a_s": (f32, (-(-(c.q_lora + 576) // 128), h // 128)),
            "q_b": (u8, (hl * 192, c.q_lora)), "kv_b": (u8, (hl * 256, 512)), "kv_b_s": (f32, (hl * 2, 4)),
            "o_proj": (u8, (h, hl * 128)), "router": (bf, (c.n_experts, h)),
            "w13": (u8, (c.n_experts, 2 * il, h)), "w2": (u8, (c.n_experts, h, il)),
        })
    return reasons


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

    return build_layers(model, c, ctx, _covered_layers(hf_config), make,
                        bind=lambda i: _bound(model, hf_config, ctx.tp_size, ctx.copies, i), numerics=NUMERICS)


SPEC = MonoSpec(
    name="glm53_" + ISA,
    devices={ISA: DeviceLimits(widths=ROWS, tp_sizes=TP_SIZES, resident_blocks=SM_COUNT)},
    features=frozenset({Feature.SPECULATIVE_DECODING}),
    requires=Requirements(
        dtypes=frozenset({"bfloat16"}),
        attention_backends=frozenset({"dsa"}),
        server_args={"kv_cache_dtype": frozenset({"fp8_e4m3"}), "enable_hisparse": frozenset({False})},
        env={"SGLANG_DSA_FUSE_TOPK": True},
    ),
    numerics=NUMERICS,
    model_disable_reasons=_model_disable_reasons,
    build=_build,
    api_version=1,
    config_disable_reasons=_config_disable_reasons,
)
