"""Decoder-layer monokernels for SGLang on NVIDIA B200 (sm_100a).

Keeps the plugin surface of the reference (``sgl_amd_mono/__init__.py:15-54``): SGLang
loads the package through the ``sglang.srt.plugins`` entry point, which calls
``register_specs()``; every spec registers by (HF architecture, model type) under one
backend name, and its module is imported only when a server runs this backend.  Behind
the specs sit Python host runners over a C-ABI library of hand-written CUDA kernels
(``include/mono_b200.h``, ``csrc/``).
"""

__version__ = "0.1.0.dev0"

# one backend name for all of this package's specs: SGLang selects them with it
BACKEND = "monokernel"
# where each spec lives, keyed by the checkpoint's architecture string and its model type (None: whatever the type)
SPECS = {
    ("DeepseekV4ForCausalLM", "deepseek_v4"): "sgl_amd_mono_b200.deepseek_v4.spec:SPEC",
    ("DeepseekV4ForCausalLM", "deepseek_v41"): "sgl_amd_mono_b200.deepseek_v41.spec:SPEC",
    ("DeepseekV4ForCausalLMDSpark", "deepseek_v41"): "sgl_amd_mono_b200.deepseek_v41.draft:SPEC",
    ("Glm5NextForConditionalGeneration", None): "sgl_amd_mono_b200.glm53_flash.spec:SPEC",
    ("GlmMoeDsaForCausalLM", None): "sgl_amd_mono_b200.glm53.spec:SPEC",
    ("MiniMaxM3SparseForCausalLM", None): "sgl_amd_mono_b200.minimax.spec:SPEC",
    ("MiniMaxM3SparseForConditionalGeneration", None): "sgl_amd_mono_b200.minimax.spec:SPEC",
}


def register_specs() -> None:
    """The plugin entry point, which SGLang runs in every process: cheap, imports no kernels."""
    from .registry import register

    for (architecture, model_type), path in SPECS.items():
        register(backend=BACKEND, architecture=architecture, path=path, model_type=model_type)
