"""The plugin surface on CPU: registration by (architecture, model type), lookup by ISA,
refusal reasons, graph-key routing and the step tables (the reference's
test/unit/test_glm53_spec.py and test_deepseek_v4_spec.py are the model)."""

from types import SimpleNamespace

import torch

import sgl_amd_mono_b200 as pkg
from sgl_amd_mono_b200 import registry
from sgl_amd_mono_b200.glm53 import HF_CONFIG as GLM_HF
from sgl_amd_mono_b200.glm53 import spec as glm53
from sgl_amd_mono_b200.minimax import spec as minimax
from sgl_amd_mono_b200.spec_common import Built, step_tables

FP8 = dict(quant_method="fp8", weight_block_size=[128, 128])


def _hf(**over):
    d = dict(GLM_HF, num_hidden_layers=5, first_k_dense_replace=3, quantization_config=FP8)
    d.update(over)
    return SimpleNamespace(**d)


CFG = SimpleNamespace(page_size=None, speculative_algorithm=None, tp_size=8)


def test_the_plugin_registers_every_spec_by_architecture_and_model_type():
    pkg.register_specs()
    found, why = registry.find_spec(backend=pkg.BACKEND, architectures=["GlmMoeDsaForCausalLM"], isa="sm_100a")
    assert found is glm53.SPEC, why
    found, why = registry.find_spec(backend=pkg.BACKEND, architectures=["GlmMoeDsaForCausalLM"], isa="gfx950")
    assert found is None and "gfx950" in why
    # two specs share one architecture and differ by model type
    a, _ = registry.find_spec(backend=pkg.BACKEND, architectures=["DeepseekV4ForCausalLM"], isa="sm_100a", model_type="deepseek_v4")
    b, _ = registry.find_spec(backend=pkg.BACKEND, architectures=["DeepseekV4ForCausalLM"], isa="sm_100a", model_type="deepseek_v41")
    assert a.name.startswith("deepseek_v4_") and b.name.startswith("deepseek_v41_")
    assert registry.spec_registered(backend=pkg.BACKEND, architectures=["MiniMaxM3SparseForCausalLM"])
    assert not registry.spec_registered(backend="amd", architectures=["GlmMoeDsaForCausalLM"])
    none, why = registry.find_spec(backend=pkg.BACKEND, architectures=["LlamaForCausalLM"], isa="sm_100a")
    assert none is None and "LlamaForCausalLM" in why


def test_the_spec_declares_widths_tp_sizes_and_one_cta_per_sm():
    lim = glm53.SPEC.devices["sm_100a"]
    assert glm53.SPEC.widths("sm_100a") == tuple(range(1, 17))
    assert lim.tp_sizes == (1, 2, 4, 8) and lim.resident_blocks == 148
    assert glm53.SPEC.api_version == 1
    assert glm53.SPEC.numerics.bound("layer.topk_exact.max_abs") == 0.0


def test_a_supported_config_has_no_reasons_and_each_mismatch_is_listed():
    assert glm53.SPEC.config_disable_reasons(CFG, _hf()) == []
    reasons = glm53.SPEC.config_disable_reasons(
        SimpleNamespace(page_size=16, speculative_algorithm=None, tp_size=3),
        _hf(kv_lora_rank=256, quantization_config=dict(quant_method="awq")))
    text = " | ".join(reasons)
    assert "kv_lora_rank" in text and "--page-size 16" in text and "--tp-size 3" in text and "FP8 block-128" in text
    assert len(reasons) == 4


def test_covered_layers_are_the_moe_layers():
    assert glm53._covered_layers(_hf()) == [3, 4]


def test_the_minimax_dispatcher_picks_by_checkpoint_quantisation():
    m31 = SimpleNamespace(hidden_size=2048, n_routed_experts=64, num_experts_per_tok=4, moe_intermediate_size=768,
                          routed_scaling_factor=1.0, scoring_func="sigmoid", rms_norm_eps=1e-6,
                          quantization_config=dict(quant_method="mxfp4"))
    assert minimax.SPEC.config_disable_reasons(CFG, m31) == []
    m3 = SimpleNamespace(**{**vars(m31), "quantization_config": dict(quant_method="fp8")})
    assert any("block-sparse" in r for r in minimax.SPEC.config_disable_reasons(CFG, m3))
    odd = SimpleNamespace(**{**vars(m31), "moe_intermediate_size": 384})
    assert any("multiples of 256" in r for r in minimax.SPEC.config_disable_reasons(CFG, odd))
    # M3.1-Flash's checkpoint: NVFP4 experts next to MXFP8 dense layers (the reference's own test config:
    # test/unit/test_minimax_m31_spec.py:16)
    from sgl_amd_mono_b200.minimax_m31 import spec as m31_spec

    nv = SimpleNamespace(**{**vars(m31), "quantization_config": dict(quant_method="mxfp8", moe_quant_algo="NVFP4")})
    assert m31_spec.is_m31(nv) and minimax.SPEC.config_disable_reasons(CFG, nv) == []
    assert m31_spec.layer_config(nv, 4).expert_fmt == "nvfp4" and m31_spec.layer_config(m31, 4).expert_fmt == "mxfp4"


def test_the_m3_spec_lists_every_reason_and_accepts_the_block_sparse_layout():
    from sgl_amd_mono_b200.minimax_m3 import spec as m3

    hf = SimpleNamespace(hidden_size=6144, num_attention_heads=48, num_key_value_heads=8, head_dim=128,
                         scoring_func="sigmoid", sparse_block_size=64, sparse_topk_blocks=16, n_routed_experts=256,
                         num_experts_per_tok=8, moe_intermediate_size=1536, rms_norm_eps=1e-6,
                         quantization_config=dict(quant_method="mxfp4"))
    cfg4 = SimpleNamespace(page_size=64, speculative_algorithm=None, tp_size=4)
    assert m3.SPEC.config_disable_reasons(cfg4, hf) == []
    g = m3.gqa_config(hf, 4)
    assert (g.q_local, g.kv_local, g.qkv_rows) == (12, 2, 18 * 128)
    assert m3.moe_config(hf, 4).inter_local == 384 and m3.moe_config(hf, 4).expert_fmt == "mxfp4"
    bad = SimpleNamespace(**{**vars(hf), "sparse_block_size": 128, "num_key_value_heads": 6})
    text = "\n".join(m3.SPEC.config_disable_reasons(SimpleNamespace(page_size=16, speculative_algorithm="NGRAM", tp_size=4), bad))
    for piece in ("sparse_block_size", "--page-size 16", "whole kv heads", "NGRAM"):
        assert piece in text, piece
    # loaded tensors: every mismatch is reported, by layer and name
    layer = SimpleNamespace(weights={"in_norm": torch.zeros(6144, dtype=torch.bfloat16), "k_scale": 0.05, "v_scale": -1.0})
    model = SimpleNamespace(layers=[SimpleNamespace(weights=None), layer], tp_size=4)
    reasons = m3.SPEC.model_disable_reasons(model, hf, [])
    assert any("layer 1: qkv is missing" in r for r in reasons) and any("v_scale" in r for r in reasons)
    assert not any("in_norm" in r or "k_scale" in r for r in reasons)


def test_step_tables_are_built_once_a_step_with_pads_and_clamped_positions():
    plan = registry.Plan(registry.ShapeKey("target_verify", batch_size=1, tokens_per_request=4))
    assert plan.key.rows == 4
    fb = SimpleNamespace(out_cache_loc=torch.tensor([70, 71, 0, 73, 99]), page_table=torch.arange(20, dtype=torch.int32).reshape(5, 4))
    st = step_tables(plan, torch.tensor([10, 11, 12, 5000, 7]), fb, 4, max_position=4095)
    assert st.slots.tolist() == [70, 71, -1, 73]
    assert st.positions.tolist() == [10, 11, 0, 4095]
    assert st.page_table.shape == (4, 4)
    assert step_tables(plan, None, None, 4, 0) is st  # the second launch of the step reuses it


def test_a_graph_key_wider_than_the_spec_runs_the_models_own_forward():
    class Lm:
        def __init__(self):
            self.ran = []
            self.layers = []

        def forward(self, input_ids, positions, forward_batch, input_embeds=None):
            self.ran.append(input_ids)
            return "own"

    lm = Lm()
    built = Built(lm, None, {}, max_rows=8, max_position=100)
    plan = registry.Plan(registry.ShapeKey("decode", batch_size=12))
    assert built.forward(plan, "ids", None, None) == "own" and lm.ran == ["ids"]
