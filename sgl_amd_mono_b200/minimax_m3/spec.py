"""MiniMax-M3: GQA block-sparse attention + MoE layers (reference: ``minimax_m3/spec.py``).

Every sparse layer runs as one attention half (input norm, fused q | k | v | index q | index k
projection, head norms + RoPE + cache insert, block scores, top-16 block selection, attention,
o_proj, all-reduce) and one MoE half.  The checks list every reason the configuration or the
loaded tensors cannot be served (``minimax_m3/spec.py:230-300``, ``weights.py:88-98``).
"""

from __future__ import annotations

import torch

from ..config import LayerConfig
from ..gqa import BLOCK, HEAD_DIM, GqaConfig, GqaLayerOp, GqaTables
from ..registry import DeviceLimits, Feature, MonoSpec, Numerics, NumericsKind, Plan, Requirements
from ..spec_common import ISA, ROWS, SM_COUNT, TP_SIZES, config_reasons, log, step_tables, weight_reasons

NUMERICS = Numerics(NumericsKind.TOLERANCE, {
    "layer.out.cosine": 0.999, "layer.out.max_abs": 2e-2,
    "cache.k.max_abs": 0.0, "cache.v.max_abs": 0.0, "cache.index.max_abs": 0.0,  # bytes, bit-exact
    "select.blocks.max_abs": 0.0, "moe.ids.max_abs": 0.0,                         # integers, bit-exact
})


def gqa_config(hf_config, tp: int) -> GqaConfig:
    g = lambda k, d=None: getattr(hf_config, k, d)  # noqa: E731
    return GqaConfig(name="minimax_m3_" + ISA, hidden=g("hidden_size"), q_heads=g("num_attention_heads"),
                     kv_heads=g("num_key_value_heads"), tp=tp, eps=g("rms_norm_eps", 1e-6),
                     init_blocks=g("sparse_init_blocks", 1), local_blocks=g("sparse_local_blocks", 2),
                     rope_theta=g("rope_theta", 1.0e6))


def moe_config(hf_config, tp: int) -> LayerConfig:
    g = lambda k, d=None: getattr(hf_config, k, d)  # noqa: E731
    quant = (g("quantization_config") or {}).get("quant_method")
    return LayerConfig(name="minimax_m3_" + ISA, hidden=g("hidden_size"), n_experts=g("n_routed_experts"),
                       top_k=g("num_experts_per_tok"), inter=g("moe_intermediate_size"),
                       route_scale=g("routed_scaling_factor", 1.0),
                       expert_fmt="mxfp4" if quant in ("mxfp4", "mxfp4_mxfp8") else "fp8_block",
                       shared_fmt=g("shared_expert_format", "none"), router_dtype=g("router_dtype", "bf16"),
                       eps=g("rms_norm_eps", 1e-6), tp=tp)


def _config_disable_reasons(cfg, hf_config) -> list[str]:
    reasons = config_reasons("the block-sparse GQA kernels", {"head_dim": HEAD_DIM, "scoring_func": "sigmoid",
                                                              "sparse_block_size": BLOCK, "sparse_topk_blocks": 16},
                             cfg, hf_config)
    tp = getattr(cfg, "tp_size", 1)
    nq, nkv = getattr(hf_config, "num_attention_heads", 0), getattr(hf_config, "num_key_value_heads", 0)
    if not nq or not nkv or nq % tp or nkv % tp or (nq // tp) % max(nkv // tp, 1) or (nq // max(nkv, 1)) > 8:
        reasons.append(f"{nq} q / {nkv} kv heads at --tp-size {tp}: every rank needs whole kv heads with at most 8 q heads each")
    if getattr(hf_config, "hidden_size", 0) % 256:
        reasons.append("the weight tiles need a hidden size that is a multiple of 256")
    if (getattr(hf_config, "moe_intermediate_size", 0) // max(tp, 1)) % 128:
        reasons.append("the expert intermediate size per rank must be a multiple of 128")
    if getattr(cfg, "moe_ep_size", 1) != 1:
        reasons.append("expert parallelism is not served (reference: minimax_m3/spec.py:262-266)")
    if getattr(cfg, "speculative_algorithm", None) not in (None, "EAGLE3"):
        reasons.append(f"--speculative-algorithm {cfg.speculative_algorithm}: only plain decode and EAGLE3 verify rows are served")
    return reasons


def _expected(g: GqaConfig) -> dict:
    h = g.hidden
    return {
        "in_norm": (torch.bfloat16, (h,)),
        "qkv": (torch.uint8, (g.qkv_rows, h)), "qkv_s": (torch.float32, (g.qkv_rows // 128, h // 128)),
        "o": (torch.uint8, (h, g.q_local * HEAD_DIM)), "o_s": (torch.float32, (h // 128, g.q_local)),
        "g_q": (torch.bfloat16, (HEAD_DIM,)), "g_k": (torch.bfloat16, (HEAD_DIM,)),
        "g_iq": (torch.bfloat16, (HEAD_DIM,)), "g_ik": (torch.bfloat16, (HEAD_DIM,)),
    }


def _model_disable_reasons(model, hf_config, copies) -> list[str]:
    tp = getattr(model, "tp_size", 1)
    g = gqa_config(hf_config, tp)
    reasons = []
    for i, layer in enumerate(model.layers):
        w = getattr(layer, "weights", None)
        if w is None:
            continue  # a dense layer runs the model's own code
        reasons += weight_reasons(i, w, _expected(g))
        for k in ("k_scale", "v_scale"):
            if not (isinstance(w.get(k), float) and w[k] > 0):
                reasons.append(f"layer {i}: {k} must be the layer's positive scalar cache scale")
    return reasons


class _Built:
    """The routed forward: covered layers on the monokernels, the rest on the model's own code."""

    def __init__(self, model, ops_by_layer: dict, max_rows: int, max_position: int, token_rows: dict | None = None):
        self.model, self.ops, self.max_rows, self.max_position = model, ops_by_layer, max_rows, max_position
        self.token_rows = token_rows or {}  # width -> metadata.TokenRows (buffers allocated at build)

    def _block_table(self, forward_batch, rows: int, fallback):
        """The rows' block table: made on the device from SGLang's per-request tables when the batch carries them
        (``minimax_m3/metadata.py:7-42``; inside the graph when captured), else the page table handed over."""
        pool = getattr(getattr(forward_batch, "req_to_token_pool", None), "req_to_token", None)
        tr = self.token_rows.get(rows)
        if pool is None or tr is None:
            return fallback
        n_req = forward_batch.req_pool_indices.shape[0]
        mode = getattr(forward_batch, "forward_mode", None)
        verify = bool(mode is not None and mode.is_target_verify())
        table, _ = tr(pool, forward_batch.req_pool_indices, forward_batch.seq_lens, forward_batch.out_cache_loc, rows // n_req, verify)
        return table

    def forward(self, plan: Plan, input_ids, positions, forward_batch, input_embeds=None, *args, **kw):
        rows = plan.key.rows
        if rows > self.max_rows:
            return type(self.model).forward(self.model, input_ids, positions, forward_batch, input_embeds, *args, **kw)
        st = step_tables(plan, positions, forward_batch, rows, self.max_position)
        st.page_table = self._block_table(forward_batch, rows, st.page_table)
        h = input_embeds if input_embeds is not None else self.model.embed(input_ids)
        h = h[:rows]
        for i, layer in enumerate(self.model.layers):
            op = self.ops.get(i)
            if op is None:
                h = layer.forward(h, positions, forward_batch)
                continue
            c = forward_batch.caches[i]
            tables = GqaTables(st.positions, st.slots, st.page_table, c.k, c.v, c.index, forward_batch.cos, forward_batch.sin)
            h = op.launch(h, tables)
        return self.model.finish(h, forward_batch) if hasattr(self.model, "finish") else h


def _build(model, hf_config, ctx):
    g, m = gqa_config(hf_config, ctx.tp_size), moe_config(hf_config, ctx.tp_size)
    ops_by_layer = {}
    for i, layer in enumerate(model.layers):  # in layer order on every rank: building is a collective when tp_size > 1
        if getattr(layer, "weights", None) is not None:
            ops_by_layer[i] = GqaLayerOp(g, m, layer.weights, ctx.device, ctx.max_context, peer=getattr(ctx, "peer", None),
                                         deadline_s=ctx.deadline_s)
    log.info("%s: %d layers on the monokernels, widths %s, TP %d", g.name, len(ops_by_layer), ctx.widths, ctx.tp_size)
    from .metadata import TokenRows

    token_rows = {w: TokenRows(w, ctx.max_context, ctx.device, block_tokens=64) for w in ctx.widths}
    return _Built(model, ops_by_layer, max(ctx.widths), ctx.max_context - 1, token_rows)


SPEC = MonoSpec(
    name="minimax_m3_" + ISA,
    devices={ISA: DeviceLimits(widths=ROWS, tp_sizes=TP_SIZES, resident_blocks=SM_COUNT)},
    features=frozenset({Feature.SPECULATIVE_DECODING, Feature.EAGLE3_HIDDEN_STATES}),
    requires=Requirements(dtypes=frozenset({"bfloat16"})),
    numerics=NUMERICS,
    model_disable_reasons=_model_disable_reasons,
    build=_build,
    api_version=1,
    config_disable_reasons=_config_disable_reasons,
)
