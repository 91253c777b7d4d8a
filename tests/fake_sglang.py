"""Stand-ins for the SGLang modules the weight binding reads (``glm53.weights.SGLANG_READS``), built from a synthetic
weight dict: the attribute names, dtypes and layouts SGLang's loaded DeepSeek-V2-family layer exposes
(reference: ``glm53/gfx950/weights.py:20-60``; ``test/unit/test_contract.py`` pins the same names)."""

from types import SimpleNamespace as NS

import torch

FP8 = torch.float8_e4m3fn


def _lin(w, s):
    return NS(weight=w.view(FP8), weight_scale_inv=s)


def layer_from_weights(cfg, w: dict, kv_scale: float = 0.03125, rope_positions: int = 256):
    """An SGLang-like decoder layer whose tensors are those of ``w`` (FP8 bytes viewed as float8).  W_UK / W_UV are
    presented as SGLang keeps them: ``w_kc [heads, nope, 512]``, ``w_vc [heads, 512, v]`` with one scalar ``w_scale``."""
    hl = cfg.heads_local
    kv_b = w["kv_b"].view(hl, cfg.nope + cfg.v_head, cfg.kv_lora)
    j = torch.arange(32, dtype=torch.float64)
    ang = torch.arange(rope_positions, dtype=torch.float64)[:, None] * 10000.0 ** (-2.0 * j / 64)
    cache = torch.cat([ang.cos(), ang.sin()], 1).float()
    rotary = NS(cos_sin_cache=cache)
    attn = NS(
        fused_qkv_a_proj_with_mqa=_lin(w["qkv_a"], w["qkv_a_s"]),
        q_a_layernorm=NS(weight=w["q_a_norm"]), kv_a_layernorm=NS(weight=w["kv_a_norm"]),
        q_b_proj=_lin(w["q_b"], w["q_b_s"]), o_proj=_lin(w["o_proj"], w["o_proj_s"]),
        w_kc=kv_b[:, : cfg.nope].contiguous().view(FP8), w_vc=kv_b[:, cfg.nope :].transpose(1, 2).contiguous().view(FP8),
        w_scale=torch.tensor(kv_scale), rotary_emb=rotary, indexer=None,
    )
    if cfg.index_heads:
        attn.indexer = NS(wk=_lin(w["idx_wk"], w["idx_wk_s"]), wq_b=_lin(w["idx_wq_b"], w["idx_wq_b_s"]),
                          weights_proj=NS(weight=w["idx_wproj"]),
                          k_norm=NS(weight=w["idx_k_norm_w"].bfloat16(), bias=w["idx_k_norm_b"].bfloat16()), rotary_emb=rotary)
    cat = lambda a, b: torch.cat([a, b[None]], 0).contiguous()  # noqa: E731  the shared expert appended
    experts = NS(w13_weight=cat(w["w13"], w["sh13"]).view(FP8), w13_weight_scale_inv=cat(w["w13_s"], w["sh13_s"]),
                 w2_weight=cat(w["w2"], w["sh2"]).view(FP8), w2_weight_scale_inv=cat(w["w2_s"], w["sh2_s"]))
    mlp = NS(experts=experts, gate=NS(weight=w["router"], e_score_correction_bias=w["router_bias"]))
    return NS(self_attn=attn, mlp=mlp, input_layernorm=NS(weight=w["input_norm"]),
              post_attention_layernorm=NS(weight=w["post_norm"]))
