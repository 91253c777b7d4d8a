"""Binding a covered layer's tensors from SGLang's modules (CPU): in-place views, the recorded copies, and the
refusals that name the tensor (reference contract: ``glm53/gfx950/weights.py:207-310``, ``glm53/spec.py:499-581``)."""

from types import SimpleNamespace as NS

import pytest
import torch

from fake_sglang import layer_from_weights
import synth
from sgl_amd_mono_b200.config import CFG_TINY
from sgl_amd_mono_b200.glm53 import weights as W


def _bound():
    cfg = CFG_TINY
    w = synth.layer_weights(cfg, 0, "cpu")
    layer = layer_from_weights(cfg, w)
    copies = {}
    return cfg, w, layer, copies, W.layer_weights(layer, 3, cfg, copies)


def test_projections_and_experts_are_views_of_sglangs_storage():
    cfg, w, layer, copies, got = _bound()
    for name in ("qkv_a", "qkv_a_s", "q_b", "q_b_s", "o_proj", "o_proj_s", "idx_wk", "idx_wq_b", "idx_wproj", "input_norm",
                 "post_norm", "q_a_norm", "kv_a_norm", "router", "router_bias"):
        assert got[name].data_ptr() == w[name].data_ptr(), f"{name} must be read in place"
        assert torch.equal(got[name], w[name])
    ex = layer.mlp.experts
    assert got["w13"].data_ptr() == ex.w13_weight.data_ptr() and got["w13"].shape[0] == cfg.n_experts
    assert got["sh13"].data_ptr() == ex.w13_weight[cfg.n_experts].data_ptr(), "the shared expert is row E of the fused tensor"
    assert torch.equal(got["w13"], w["w13"]) and torch.equal(got["sh2"], w["sh2"]) and torch.equal(got["w2_s"], w["w2_s"])


def test_the_copies_are_recorded_for_the_startup_log():
    cfg, w, layer, copies, got = _bound()
    keys = set(copies)
    assert ("W_UK | W_UV in one tensor", 3, "kv_b") in keys and ("W_UK | W_UV in one tensor", 3, "kv_b_s") in keys
    assert ("indexer k LayerNorm f32", 3, "weight") in keys and ("indexer k LayerNorm f32", 3, "bias") in keys
    assert len(keys) == 4, f"nothing else is copied: {keys}"
    # w_vc was transposed back into the [v, latent] rows the W_UV GEMV reads; W_UK rows are w_kc's
    assert torch.equal(got["kv_b"], w["kv_b"])
    assert got["kv_b_s"].shape == (cfg.heads_local * 2, 4) and bool((got["kv_b_s"] == 0.03125).all())
    assert got["idx_k_norm_w"].dtype == torch.float32
    cos, sin = W.rope_tables([layer], copies)
    assert cos.dtype == torch.bfloat16 and cos.shape == (256, 32) and ("rope table bf16", "cos") in copies


def test_a_mismatch_is_refused_with_the_tensors_name():
    cfg, w, layer, copies, _ = _bound()
    layer.self_attn.q_b_proj.weight = layer.self_attn.q_b_proj.weight[:-128]
    with pytest.raises(ValueError, match="q_b_proj.weight"):
        W.layer_weights(layer, 0, cfg, {})
    cfg, w, layer, copies, _ = _bound()
    layer.self_attn.o_proj.is_shuffled = True
    with pytest.raises(ValueError, match="row-major"):
        W.layer_weights(layer, 0, cfg, {})
    cfg, w, layer, copies, _ = _bound()
    layer.self_attn.w_scale = torch.ones(4)
    with pytest.raises(ValueError, match="scalar w_scale"):
        W.layer_weights(layer, 0, cfg, {})
    cfg, w, layer, copies, _ = _bound()
    layer.mlp.experts.w13_weight = layer.mlp.experts.w13_weight[:-1]
    with pytest.raises(ValueError, match="shared expert appended"):
        W.layer_weights(layer, 0, cfg, {})
    cfg, w, layer, copies, _ = _bound()
    layer.mlp.gate.weight = (layer.mlp.gate.weight.float() + 1e-4)
    with pytest.raises(ValueError, match="representable in bf16"):
        W.layer_weights(layer, 0, cfg, {})


def test_the_spec_lists_binding_failures_as_reasons_by_layer():
    from sgl_amd_mono_b200.glm53 import spec as glm53
    from sgl_amd_mono_b200.glm53 import HF_CONFIG

    cfg = CFG_TINY
    hf = NS(**{**HF_CONFIG, "hidden_size": cfg.hidden, "num_attention_heads": cfg.n_heads, "q_lora_rank": cfg.q_lora,
               "index_n_heads": cfg.index_heads, "index_topk": cfg.index_topk, "n_routed_experts": cfg.n_experts,
               "num_experts_per_tok": cfg.top_k, "moe_intermediate_size": cfg.inter, "num_hidden_layers": 2,
               "first_k_dense_replace": 0, "rms_norm_eps": cfg.eps})
    good = layer_from_weights(cfg, synth.layer_weights(cfg, 0, "cpu"))
    bad = layer_from_weights(cfg, synth.layer_weights(cfg, 0, "cpu", layer=1))
    bad.self_attn.fused_qkv_a_proj_with_mqa.weight_scale_inv = None
    model = NS(model=NS(layers=[good, bad]), tp_size=1)
    reasons = glm53.SPEC.model_disable_reasons(model, hf, {})
    assert len(reasons) == 1 and reasons[0].startswith("layer 1:") and "fused_qkv_a_proj_with_mqa.weight_scale_inv" in reasons[0]
