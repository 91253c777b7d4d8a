"""Layer shapes the kernels are launched with.

The reference bakes each model's shapes into compile-time constants
(``glm53/__init__.py:11-40`` ``HF_CONFIG``, ``glm53/gfx950/config.py``); the sm_100a
kernels take them as launch arguments instead, so one library serves every spec.
``tp`` shards heads and each expert's intermediate dimension; the q_a|kv_a
projection, the indexer, the router, norms and caches are replicated
(``glm53/gfx950/config.py:207-218``).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

PAGE = 64  # tokens per KV / index page
KV_DIM = 576  # 512 latent + 64 rope values per cached token
KV_PAGE_BYTES = PAGE * KV_DIM + PAGE * 4  # E4M3 values, then one f32 scale per token
IDX_DIM = 128
IDX_PAGE_BYTES = PAGE * (IDX_DIM // 2) + PAGE * (IDX_DIM // 32)  # E2M1 values, then E8M0 codes
MAX_ROWS = 16


@dataclass(frozen=True)
class LayerConfig:
    name: str
    hidden: int
    # attention (MLA); n_heads = 0 for an FFN-only block
    n_heads: int = 0
    q_lora: int = 0
    kv_lora: int = 512
    nope: int = 128
    rope: int = 64
    v_head: int = 128
    index_heads: int = 0
    index_topk: int = 2048
    window: int = 0  # > 0 (and no indexer): a row attends its last `window` keys only (a draft model's attention)
    # MoE
    n_experts: int = 0
    top_k: int = 0
    inter: int = 0  # global expert intermediate size
    route_scale: float = 1.0
    expert_fmt: str = "fp8_block"  # "fp8_block" | "mxfp4" | "nvfp4"
    shared_fmt: str = "fp8_block"  # "fp8_block" | "mxfp4" | "nvfp4" | "bf16" | "none"
    router_dtype: str = "bf16"  # "bf16" | "f32"
    eps: float = 1e-6
    tp: int = 1
    vocab: int = 0

    @property
    def heads_local(self) -> int:
        return self.n_heads // self.tp

    @property
    def inter_local(self) -> int:
        return self.inter // self.tp

    def with_tp(self, tp: int) -> "LayerConfig":
        return replace(self, tp=tp)


# BASELINE config 1: MoE FFN block (minimax_m31-style), TP1.
CFG_FFN_MXFP4 = LayerConfig(
    name="ffn_mxfp4_2048", hidden=2048, n_experts=64, top_k=4, inter=768, route_scale=1.0,
    expert_fmt="mxfp4", shared_fmt="bf16", router_dtype="f32", eps=1e-6,
)
# BASELINE config 3: DeepSeek-V3-shaped MLA + indexer + MoE layer.
CFG_V3 = LayerConfig(
    name="v3_mla_dsa_moe", hidden=7168, n_heads=128, q_lora=1536, nope=128, rope=64, v_head=128,
    index_heads=64, index_topk=2048, n_experts=256, top_k=8, inter=2048, route_scale=2.5,
    expert_fmt="fp8_block", shared_fmt="fp8_block", eps=1e-6,
)
# BASELINE config 5: flash-sized MLA + MoE layer (no indexer; q_lora / nope / v_head as V3).
CFG_FLASH = LayerConfig(
    name="flash_mla_moe", hidden=4096, n_heads=64, q_lora=1536, nope=128, rope=64, v_head=128,
    index_heads=0, n_experts=256, top_k=6, inter=1024, route_scale=1.5,
    expert_fmt="fp8_block", shared_fmt="fp8_block", eps=1e-6, vocab=129280,
)
# A small layer with every feature, for parity tests the CPU oracle finishes in seconds.
CFG_TINY = LayerConfig(
    name="tiny_mla_dsa_moe", hidden=1024, n_heads=8, q_lora=512, nope=128, rope=64, v_head=128,
    index_heads=8, index_topk=256, n_experts=16, top_k=4, inter=512, route_scale=2.5,
    expert_fmt="fp8_block", shared_fmt="fp8_block", eps=1e-6,
)
# The same block with NVFP4 experts (the expert format of MiniMax-M3.1-Flash's checkpoint), shared expert included.
CFG_TINY_FFN_NVFP4 = LayerConfig(
    name="tiny_ffn_nvfp4", hidden=512, n_experts=8, top_k=2, inter=256, route_scale=1.0,
    expert_fmt="nvfp4", shared_fmt="nvfp4", router_dtype="f32", eps=1e-6,
)
CFG_TINY_FFN = LayerConfig(
    name="tiny_ffn_mxfp4", hidden=512, n_experts=8, top_k=2, inter=256, route_scale=1.0,
    expert_fmt="mxfp4", shared_fmt="bf16", router_dtype="f32", eps=1e-6,
)
