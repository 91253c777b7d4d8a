"""A covered layer's tensors as the sm_100a kernels read them, from SGLang's loaded modules.

Reference counterpart: ``glm53/gfx950/weights.py`` (``layer_weights`` ``:207-310``, ``_uk_uv``
``:141-178``, ``_indexer`` ``:181-204``, ``rope_tables`` ``:313-345``, the names it reads from
SGLang ``:20-60``).  The contract is the reference's: projections and experts are SGLang's FP8
tensors READ IN PLACE after exhaustive shape / dtype / layout checks (a mismatch raises with the
tensor's name), and the few tensors that have to be re-laid-out are copied once and recorded in
``copies`` (key tuple -> tensor) for SGLang's startup log.

What differs from the gfx950 build is which tensors need a copy.  The TMA descriptors read
SGLang's row-major ``[N, K]`` FP8 weights and ``[N/128, K/128]`` f32 scales as they are, so there
is no tile repack of the projections, the router or the indexer's ``weights_proj`` (the
reference packs those three for its MFMA lanes).  Copies that remain:

  W_UK | W_UV   SGLang keeps ``w_kc [heads, 128, 512]`` and ``w_vc [heads, 512, 128]`` as
                per-tensor FP8 with a scalar ``w_scale``.  The absorb stage and the W_UV GEMV
                read one tensor ``[heads, 256, 512]`` (rows 0..127 = W_UK, rows 128..255 = W_UV
                with the latent dimension contiguous) and block scales ``[heads * 2, 4]``:
                ``w_vc`` is transposed into it (8.4 MB a layer at TP 1, as the reference copies both)
  k LayerNorm   the indexer's weight and bias as f32
  rope tables   bf16 ``[positions, 32]`` cos and sin from SGLang's f32 ``cos_sin_cache``

SGLang appends the shared expert to the routed ones (``w13_weight [257, ...]``): the shared
expert's tensors are views of row 256, the routed experts' views of rows 0..255.
"""

from __future__ import annotations

import torch

from ..config import KV_DIM, LayerConfig

# the SGLang attribute names this module reads, by the SGLang file that defines them
SGLANG_READS = {
    "srt/models/deepseek_v2.py": (
        "self_attn", "mlp", "input_layernorm", "post_attention_layernorm", "fused_qkv_a_proj_with_mqa", "q_a_layernorm",
        "kv_a_layernorm", "q_b_proj", "o_proj", "w_kc", "w_vc", "w_scale", "indexer", "rotary_emb", "gate",
        "e_score_correction_bias", "experts",
    ),
    "srt/layers/attention/dsa/dsa_indexer.py": ("wq_b", "wk", "weights_proj", "k_norm"),
    "srt/layers/rotary_embedding/base.py": ("cos_sin_cache",),
    "srt/layers/quantization/fp8.py": ("weight_scale_inv", "w13_weight", "w13_weight_scale_inv", "w2_weight", "w2_weight_scale_inv"),
}

FP8 = torch.float8_e4m3fn


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


def need(name: str, t, shape: tuple, dtypes: tuple) -> torch.Tensor:
    """The tensor, or a ``ValueError`` that names it and says what it must be."""
    if not isinstance(t, torch.Tensor) or tuple(t.shape) != tuple(shape) or t.dtype not in dtypes or not t.is_contiguous():
        got = f"{t.dtype} {tuple(t.shape)} strides {tuple(t.stride())}" if isinstance(t, torch.Tensor) else type(t).__name__
        raise ValueError(f"needs {name} as contiguous {'/'.join(map(str, dtypes))} {tuple(shape)}, got {got}")
    return t


def _bytes(t: torch.Tensor) -> torch.Tensor:
    """An FP8 tensor as the uint8 tensor the launch wrappers take (a view: same storage)."""
    return t.view(torch.uint8)


def linear(name: str, mod, rows: int, cols: int):
    """A block-FP8 linear read in place: (E4M3 bytes [rows, cols], f32 scales [rows/128, cols/128])."""
    w = need(f"{name}.weight", mod.weight, (rows, cols), (FP8,))
    s = need(f"{name}.weight_scale_inv", getattr(mod, "weight_scale_inv", None), (_cdiv(rows, 128), _cdiv(cols, 128)), (torch.float32,))
    if getattr(mod, "is_shuffled", False) or getattr(mod, "aiter_bpreshuffled", False):
        raise ValueError(f"needs {name}.weight row-major: the TMA descriptors read SGLang's own layout, not a pre-shuffled one")
    return _bytes(w), s


def uk_uv(attn, heads: int, cfg: LayerConfig, idx: int, copies: dict):
    """``kv_b [heads * 256, 512]`` E4M3 bytes and its block scales ``[heads * 2, 4]`` from ``w_kc`` / ``w_vc``."""
    nope, v, lat = cfg.nope, cfg.v_head, cfg.kv_lora
    w_kc, w_vc, w_scale = getattr(attn, "w_kc", None), getattr(attn, "w_vc", None), getattr(attn, "w_scale", None)
    if w_kc is None or w_vc is None or w_kc.dtype != FP8 or w_scale is None or w_scale.numel() != 1:
        raise ValueError(f"needs w_kc / w_vc as per-tensor FP8 E4M3 with a scalar w_scale, got "
                         f"{None if w_kc is None else w_kc.dtype} and {None if w_scale is None else tuple(w_scale.shape)}")
    if tuple(w_kc.shape) != (heads, nope, lat) or tuple(w_vc.shape) != (heads, lat, v):
        raise ValueError(f"needs w_kc [{heads}, {nope}, {lat}] and w_vc [{heads}, {lat}, {v}], got {tuple(w_kc.shape)} and {tuple(w_vc.shape)}")
    kv_b = torch.empty(heads, nope + v, lat, dtype=torch.uint8, device=w_kc.device)
    kv_b[:, :nope] = _bytes(w_kc)
    kv_b[:, nope:] = _bytes(w_vc).transpose(1, 2)
    kv_b = kv_b.reshape(heads * (nope + v), lat)
    kv_b_s = torch.full((heads * (nope + v) // 128, lat // 128), float(w_scale.float().item()), dtype=torch.float32, device=w_kc.device)
    copies["W_UK | W_UV in one tensor", idx, "kv_b"] = kv_b
    copies["W_UK | W_UV in one tensor", idx, "kv_b_s"] = kv_b_s
    return kv_b, kv_b_s


def indexer(attn, cfg: LayerConfig, idx: int, copies: dict) -> dict:
    ind = attn.indexer
    w = {}
    w["idx_wk"], w["idx_wk_s"] = linear("indexer.wk", ind.wk, 128, cfg.hidden)
    w["idx_wq_b"], w["idx_wq_b_s"] = linear("indexer.wq_b", ind.wq_b, cfg.index_heads * 128, cfg.q_lora)
    w["idx_wproj"] = need("indexer.weights_proj", ind.weights_proj.weight, (cfg.index_heads, cfg.hidden), (torch.bfloat16,))
    w["idx_k_norm_w"] = ind.k_norm.weight.detach().float().contiguous()
    w["idx_k_norm_b"] = ind.k_norm.bias.detach().float().contiguous()
    copies["indexer k LayerNorm f32", idx, "weight"] = w["idx_k_norm_w"]
    copies["indexer k LayerNorm f32", idx, "bias"] = w["idx_k_norm_b"]
    return w


def experts_reason(moe, cfg: LayerConfig) -> str | None:
    """Why this layer's experts cannot be read in place, or None."""
    ex = getattr(moe, "experts", None)
    if ex is None or getattr(ex, "w13_weight", None) is None:
        return "the MoE layer has no fused w13_weight / w2_weight tensors"
    if ex.w13_weight.dtype != FP8 or getattr(ex, "w13_weight_scale_inv", None) is None:
        return f"needs block-FP8 experts (w13_weight {ex.w13_weight.dtype}, scales {'present' if getattr(ex, 'w13_weight_scale_inv', None) is not None else 'missing'})"
    if ex.w13_weight.shape[0] != cfg.n_experts + 1:
        return f"needs the shared expert appended to the routed ones ({cfg.n_experts + 1} experts), got {ex.w13_weight.shape[0]}"
    return None


def layer_weights(layer, idx: int, cfg: LayerConfig, copies: dict) -> dict:
    """The dict of this rank's tensors that ``MlaLayerOp`` takes, bound to ``layer``'s storage."""
    attn, moe = layer.self_attn, layer.mlp
    h, hl, il = cfg.hidden, cfg.heads_local, cfg.inter_local
    bf = (torch.bfloat16,)
    w = {
        "input_norm": need("input_layernorm", layer.input_layernorm.weight, (h,), bf),
        "post_norm": need("post_attention_layernorm", layer.post_attention_layernorm.weight, (h,), bf),
        "q_a_norm": need("q_a_layernorm", attn.q_a_layernorm.weight, (cfg.q_lora,), bf),
        "kv_a_norm": need("kv_a_layernorm", attn.kv_a_layernorm.weight, (cfg.kv_lora,), bf),
    }
    w["qkv_a"], w["qkv_a_s"] = linear("fused_qkv_a_proj_with_mqa", attn.fused_qkv_a_proj_with_mqa, cfg.q_lora + KV_DIM, h)
    w["q_b"], w["q_b_s"] = linear("q_b_proj", attn.q_b_proj, hl * (cfg.nope + cfg.rope), cfg.q_lora)
    w["o_proj"], w["o_proj_s"] = linear("o_proj", attn.o_proj, h, hl * cfg.v_head)
    w["kv_b"], w["kv_b_s"] = uk_uv(attn, hl, cfg, idx, copies)
    if getattr(attn, "indexer", None) is not None:
        w.update(indexer(attn, cfg, idx, copies))
    why = experts_reason(moe, cfg)
    if why is not None:
        raise ValueError(why)
    ex, E = moe.experts, cfg.n_experts
    w13 = need("w13_weight", ex.w13_weight, (E + 1, 2 * il, h), (FP8,))
    s13 = need("w13_weight_scale_inv", ex.w13_weight_scale_inv, (E + 1, _cdiv(2 * il, 128), h // 128), (torch.float32,))
    w2 = need("w2_weight", ex.w2_weight, (E + 1, h, il), (FP8,))
    s2 = need("w2_weight_scale_inv", ex.w2_weight_scale_inv, (E + 1, h // 128, _cdiv(il, 128)), (torch.float32,))
    w["w13"], w["w13_s"], w["w2"], w["w2_s"] = _bytes(w13)[:E], s13[:E], _bytes(w2)[:E], s2[:E]
    w["sh13"], w["sh13_s"], w["sh2"], w["sh2_s"] = _bytes(w13)[E], s13[E], _bytes(w2)[E], s2[E]
    gate = moe.gate
    router = need("gate", gate.weight, (E, h), (torch.bfloat16, torch.float32))
    if router.dtype != torch.bfloat16:
        if not torch.equal(router.to(torch.bfloat16).float(), router):
            # SGLang routes an f32 gate in f32; the router stage reads bf16 (glm53/gfx950/weights.py:278-283)
            raise ValueError("needs router weights exactly representable in bf16")
        router = router.to(torch.bfloat16).contiguous()
        copies["router as bf16", idx] = router
    w["router"] = router
    w["router_bias"] = need("e_score_correction_bias", gate.e_score_correction_bias, (E,), (torch.float32,))
    return w


def rope_tables(layers: list, copies: dict):
    """bf16 (cos, sin) ``[positions, 32]`` that every covered layer's rotaries read, from the first layer's
    f32 ``cos_sin_cache [positions, 64]`` (cos, then sin); each indexer's table must equal it
    (``glm53/gfx950/weights.py:313-345``)."""
    def cos_sin(rotary):
        c = rotary.cos_sin_cache
        return c[:, : c.shape[1] // 2], c[:, c.shape[1] // 2 :]

    cos, sin = cos_sin(layers[0].self_attn.rotary_emb)
    for layer in layers:
        ind = getattr(layer.self_attn, "indexer", None)
        if ind is None:
            continue
        c2, s2 = cos_sin(ind.rotary_emb)
        if c2.shape != cos.shape or not torch.equal(c2, cos) or not torch.equal(s2, sin):
            raise ValueError("needs the indexer's rotary table equal to the attention's")
    cos, sin = cos.to(torch.bfloat16).contiguous(), sin.to(torch.bfloat16).contiguous()
    copies["rope table bf16", "cos"] = cos
    copies["rope table bf16", "sin"] = sin
    return cos, sin
