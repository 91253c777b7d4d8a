"""Stage arithmetic of the decode path, restated on CPU (test infrastructure only).

One function per stage of the layer kernels; each cites the reference lines it
follows (paths relative to the reference project).  fp32 math, bf16 / FP8 rounding
where the device code rounds.  The approximate hardware rcp / rsq / exp2 of the
reference are exact here; the parity tolerance absorbs the difference.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import quant as Q

PAGE = 64  # tokens per KV / index page
KV_DIM = 576  # 512 latent + 64 rope values per token
KV_PAGE_BYTES = PAGE * KV_DIM + PAGE * 4  # values, then one f32 scale per token
IDX_DIM = 128
IDX_PAGE_BYTES = PAGE * (IDX_DIM // 2) + PAGE * (IDX_DIM // 32)  # E2M1 values, then E8M0


# ---------------------------------------------------------------- norms, rope, hadamard
def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """y = bf16(x * rsqrt(mean(x^2) + eps) * gamma), fp32 math.

    glm53/gfx950/kernel.py:1367-1414.
    """
    x = x.float()
    r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return Q.bf(x * r * gamma.float())


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float = 1e-6):
    """(x - mean) * rstd * w + b over the last dim, fp32 (glm53/gfx950/kernel.py:2121-2133)."""
    x = x.float()
    mean = x.mean(-1, keepdim=True)
    var = (x - mean).pow(2).mean(-1, keepdim=True)
    return (x - mean) * torch.rsqrt(var + eps) * w.float() + b.float()


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """GPT-J rotary on the last dim (pairs 2j, 2j+1): p0 = x0 c - x1 s, p1 = x0 s + x1 c.

    cos / sin are [rows, dim/2] (already gathered at each row's position), broadcast
    over any middle dims.  glm53/gfx950/kernel.py:2014-2016,2072.
    """
    x = x.float()
    x0, x1 = x[..., 0::2], x[..., 1::2]
    while cos.dim() < x0.dim():
        cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
    c, s = cos.float(), sin.float()
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).flatten(-2)


def rope_table(positions: int, dim: int = 64, theta: float = 10000.0):
    """bf16 cos / sin tables [positions, dim/2] (angle = pos * theta^(-2j/dim)).

    test/kernels/deepseek_v41/check_k1.py:73-78 builds the same angles in fp64.
    """
    j = torch.arange(dim // 2, dtype=torch.float64)
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * theta ** (-2.0 * j / dim)
    return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)


def fwht128(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal Sylvester-order Hadamard over the last 128 dims, fp32.

    glm53/gfx950/kernel.py:556-566: butterflies, then * 128^-0.5.
    """
    x = x.float()
    n = x.shape[-1]
    h = 1
    while h < n:
        y = x.reshape(*x.shape[:-1], n // (2 * h), 2, h)
        x = torch.stack([y[..., 0, :] + y[..., 1, :], y[..., 0, :] - y[..., 1, :]], -2)
        x = x.reshape(*x.shape[:-3], n)
        h *= 2
    return x * (n**-0.5)


# ---------------------------------------------------------------- GEMVs
def gemv_fp8_block(x: torch.Tensor, w: torch.Tensor, scale: torch.Tensor):
    """y = x @ dequant(w).T in fp32 for bf16 activations and block-FP8 weights.

    glm53/gfx950/kernel.py:1061-1172 (FP8 widened exactly, fp32 accumulate, block scale).
    """
    return x.float() @ Q.fp8_block_dequant(w, scale).T


def gemv_fp8_block_a8(x: torch.Tensor, w: torch.Tensor, scale: torch.Tensor):
    """FP8 x FP8 unit: activations quantised per 128 first (kernel.py:1440-1450)."""
    q, s = Q.act_quant_128(x)
    xq = (q.reshape(*x.shape[:-1], -1, 128) * s[..., None]).reshape(x.shape)
    return xq @ Q.fp8_block_dequant(w, scale).T


# ---------------------------------------------------------------- KV cache rows
def kv_row_encode(latent_bf: torch.Tensor, rope_bf: torch.Tensor):
    """One token's cache row from its bf16 latent [.., 512] and rope part [.., 64].

    Values = E4M3(v / scale), scale = token_pow2_scale(amax over all 576 values)
    (quant.token_pow2_scale).  Returns (bytes uint8 [.., 576], scale f32 [..]).
    Bit-exact rule: power-of-two division is exact, the E4M3 cast is RNE.
    """
    v = torch.cat([latent_bf.float(), rope_bf.float()], -1)
    scale = Q.token_pow2_scale(v.abs().amax(-1))
    return Q.e4m3_bytes(v / scale[..., None]), scale


def kv_pages_write(pages: torch.Tensor, slots: torch.Tensor, row_bytes, scales) -> None:
    """Store rows into uint8 pages [n_pages, KV_PAGE_BYTES] at global slots (< 0: pad, no write).

    glm53/gfx950/kernel.py:2049-2100 (slot addressing); glm53/spec.py:15-17 (pads).
    """
    sc = pages[:, PAGE * KV_DIM :].view(torch.float32)
    for i, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        p, o = divmod(slot, PAGE)
        pages[p, o * KV_DIM : (o + 1) * KV_DIM] = row_bytes[i]
        sc[p, o] = scales[i]


def kv_rows_gather(pages: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """Dequantised rows bf16(e4m3 * scale) as f32 [n, 576] for global slots (>= 0)."""
    p, o = slots.long() // PAGE, slots.long() % PAGE
    vals = pages[:, : PAGE * KV_DIM].reshape(-1, PAGE, KV_DIM)[p, o]
    sc = pages[:, PAGE * KV_DIM :].view(torch.float32)[p, o]
    return Q.bf(Q.e4m3_from_bytes(vals) * sc[:, None])


# ---------------------------------------------------------------- index keys (FP4)
def index_key_encode(k: torch.Tensor):
    """FP4 index key of one token from the 128 f32 values after LayerNorm/RoPE/FWHT.

    deepseek_v4/gfx950/kernels/stages/indexer.py:143-151: per 32 values
    sc = pow2_ceil(max(amax, 6 * 2^-126) / 6), q = clamp(v / sc) -> E2M1.
    Returns (packed uint8 [.., 64], E8M0 codes uint8 [.., 4]).
    """
    return Q.mxfp4_quant(k.reshape(-1, IDX_DIM))


def index_pages_write(pages, slots, packed, codes) -> None:
    vals = pages[:, : PAGE * 64]
    sc = pages[:, PAGE * 64 :]
    for i, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        p, o = divmod(slot, PAGE)
        vals[p, o * 64 : (o + 1) * 64] = packed[i]
        sc[p, o * 4 : (o + 1) * 4] = codes[i]


def index_keys_gather(pages: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """Dequantised index keys f32 [n, 128] at global slots."""
    p, o = slots.long() // PAGE, slots.long() % PAGE
    vals = pages[:, : PAGE * 64].reshape(-1, PAGE, 64)[p, o]
    sc = pages[:, PAGE * 64 :].reshape(-1, PAGE, 4)[p, o]
    return Q.mxfp4_dequant(vals, sc)


def index_scores(q: torch.Tensor, w: torch.Tensor, keys: torch.Tensor) -> torch.Tensor:
    """score[k] = sum_h relu(q_h . key_k) * w_h, f32.

    q [heads, 128] (bf16 values), w [heads] f32, keys [n, 128] f32 (exact FP4 values).
    glm53/gfx950/kernel.py:2770-2842.
    """
    dots = q.float() @ keys.float().T  # [heads, n]
    return (F.relu(dots) * w.float()[:, None]).sum(0)


# ---------------------------------------------------------------- exact top-k
def radix_key(bits: torch.Tensor) -> torch.Tensor:
    """Monotone unsigned image of f32 score bits (int64 holding a uint32).

    glm53/gfx950/kernel.py:2698-2699; glm53/check.py:94-97.
    """
    b = bits.to(torch.int64)
    return torch.where(b >= 0, b + (1 << 31), ~b & 0xFFFFFFFF)


def exact_topk_positions(scores: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """Positions the kernel selects for one row of ``n`` scored keys.

    Rows with n <= k keep every key in order.  Otherwise: all keys strictly above the
    k-th largest key in position order, then the first ``remain`` ties in position
    order (glm53/gfx950/kernel.py:3381-3402; ties go to the lowest position).
    """
    if n <= k:
        return torch.arange(n, dtype=torch.int64)
    keys = radix_key(scores[:n].contiguous().view(torch.int32))
    thr = torch.sort(keys, descending=True).values[k - 1]
    above = (keys > thr).nonzero().flatten()
    ties = (keys == thr).nonzero().flatten()[: k - above.numel()]
    return torch.cat([above, ties])


def slots_of_positions(page_row: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Global KV slots page_table[pos / 64] * 64 + pos % 64 (kernel.py:3341-3346)."""
    return page_row.long()[pos // PAGE] * PAGE + pos % PAGE


# ---------------------------------------------------------------- sparse MLA
def sparse_mla_row(q: torch.Tensor, kv: torch.Tensor, sm_scale: float, split: int = 64):
    """One row's sparse MLA over its selected keys.

    q [heads, 576] bf16 values (512 absorbed latent dims then 64 rope), kv [n, 576]
    dequantised rows.  Per split of ``split`` keys: s = (q . kv) * scale, split-local
    m / l, p rounded to bf16 before P.V, the partial accumulator rounded to bf16;
    merge w_j = e^(m_j - M) / sum_j l_j e^(m_j - M); result bf16 [heads, 512].
    glm53/gfx950/kernel.py:3883-3972 (split), :4026-4075 (merge).
    """
    heads = q.shape[0]
    n = kv.shape[0]
    if n == 0:
        return torch.zeros(heads, 512)
    qf, kvf = q.float(), kv.float()
    accs, ms, ls = [], [], []
    for j0 in range(0, n, split):
        k = kvf[j0 : j0 + split]
        s = (qf @ k.T) * sm_scale
        m = s.amax(1)
        p = torch.exp(s - m[:, None])
        ls.append(p.sum(1))
        ms.append(m)
        accs.append(Q.bf(Q.bf(p) @ k[:, :512]))
    m, l, acc = torch.stack(ms), torch.stack(ls), torch.stack(accs)
    big = m.amax(0)
    e = torch.exp(m - big)
    den = (l * e).sum(0)
    w = torch.where(den > 0, e / den, torch.zeros_like(e))
    return Q.bf((acc * w[..., None]).sum(0))


def sparse_mla(q, kv_pages, topk, sm_scale: float) -> torch.Tensor:
    """[S, heads, 576] bf16 query, uint8 KV pages, int32 [S, n] selected slots (-1: none).

    Invalid entries are skipped (they contribute nothing, as a masked key does).
    """
    out = torch.zeros(q.shape[0], q.shape[1], 512)
    for s in range(q.shape[0]):
        sl = topk[s]
        sl = sl[sl >= 0]
        out[s] = sparse_mla_row(q[s], kv_rows_gather(kv_pages, sl), sm_scale)
    return out.to(torch.bfloat16)


# ---------------------------------------------------------------- router
def route(logits: torch.Tensor, bias, k: int, route_scale: float):
    """Sigmoid router: ids by (score + bias) descending, ties to the lower expert id;
    weight = score_k / sum(score of the k picks) * route_scale, in pick order.

    glm53/gfx950/kernel.py:1575-1629; minimax_m31/ffn.py:654-723;
    test/kernels/test_minimax_m31_ffn.py:146-151.
    """
    sc = torch.sigmoid(logits.float())
    return route_from_scores(sc, bias, k, route_scale)


def route_from_scores(sc: torch.Tensor, bias, k: int, route_scale: float):
    key = sc if bias is None else sc + bias.float()
    # stable descending sort = ties to the lower id
    ids = torch.sort(key, dim=-1, descending=True, stable=True).indices[..., :k]
    w = sc.gather(-1, ids)
    w = w * (route_scale / w.sum(-1, keepdim=True).clamp_min(1e-20))
    return ids.to(torch.int32), w


# ---------------------------------------------------------------- experts
def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """mid = g * 1/(1+exp(-g)) * u, no clamp, f32 (glm53/gfx950/kernel.py:4396-4415)."""
    return F.silu(g.float()) * u.float()


def expert_fp8(x, w13, s13, w2, s2):
    """One block-FP8 expert on rows x [n, H] (bf16 values): FP8 x FP8 units.

    up/gate on the per-128 quantised x, mid = swiglu kept f32, mid re-quantised per
    128, down (glm53/gfx950/kernel.py:4352-4999, :5001-5187).  w13 rows = gate then up.
    """
    h = gemv_fp8_block_a8(x, w13, s13)
    inter = h.shape[-1] // 2
    mid = swiglu(h[..., :inter], h[..., inter:])
    return gemv_fp8_block_a8(mid, w2, s2)


def expert_mxfp4(x, w13, c13, w2, c2):
    """One MXFP4 expert on MXFP8 activations (W4A8), bf16 mid.

    glm53_flash/gfx950/kernel.py:4025-4392 (MXFP4 x MXFP8 scaled MMA);
    test/kernels/deepseek_v41/check_ffn.py:208-229 (golden).  No clamp: BASELINE
    config 1 asks for plain SwiGLU.
    """
    q, c = Q.mxfp8_quant(x)
    h = Q.mxfp8_dequant(q, c) @ Q.mxfp4_dequant(w13, c13).T
    inter = h.shape[-1] // 2
    mid = Q.bf(swiglu(h[..., :inter], h[..., inter:]))
    q2, cc2 = Q.mxfp8_quant(mid)
    return Q.mxfp8_dequant(q2, cc2) @ Q.mxfp4_dequant(w2, c2).T


def expert_nvfp4(x, w13, s13, g13, w2, s2, g2):
    """One NVFP4 expert on NVFP4 activations (W4A4: the only operand pairing Blackwell's block-scaled FP4 tensor-core
    kind takes; both operands E2M1 with an E4M3 scale per 16, the weights' f32 tensor scale applied to the f32 sum),
    bf16 mid, plain SwiGLU.  ``g13`` / ``g2``: this expert's f32 tensor scales."""
    xq, xs = Q.nvfp4_act_quant(x)
    h = Q.nvfp4_dequant(xq, xs, 1.0) @ Q.nvfp4_dequant(w13, s13, 1.0).T * float(g13)
    inter = h.shape[-1] // 2
    mid = Q.bf(swiglu(h[..., :inter], h[..., inter:]))
    mq, ms = Q.nvfp4_act_quant(mid)
    return Q.nvfp4_dequant(mq, ms, 1.0) @ Q.nvfp4_dequant(w2, s2, 1.0).T * float(g2)


def expert_bf16(x, w13, w2):
    """bf16 shared expert: bf16 weights and activations, f32 accumulate, bf16 mid."""
    h = x.float() @ w13.float().T
    inter = h.shape[-1] // 2
    mid = Q.bf(swiglu(h[..., :inter], h[..., inter:]))
    return mid @ w2.float().T


# ---------------------------------------------------------------- all-reduce
def allreduce_rank_order(partials, residual=None) -> torch.Tensor:
    """Each rank's partial rounded to bf16, summed in rank order in f32 from 0.0,
    then the residual is added and the result rounded to bf16.

    glm53/gfx950/kernel.py:1631-1688; test/kernels/deepseek_v41/check_ffn.py:251-258.
    """
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:
        acc = acc + Q.bf(p.float())
    if residual is not None:
        acc = acc + residual.float()
    return acc.to(torch.bfloat16)


def tail_logits(h, gamma, eps: float, w_head) -> torch.Tensor:
    """Final RMSNorm + LM-head rows of this rank: f32 logits [S, vocab/W].

    glm53_flash/gfx950/kernel.py:3626-3770; golden glm53_flash/check.py:284-302 (without
    the hyper-connection streams, which BASELINE's configs do not have).
    """
    x = h.float()
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()
    return x @ w_head.float().T


def sm_scale_mla(nope: int, rope: int) -> float:
    """(nope + rope)^-0.5 (glm53/gfx950/config.py:179-181)."""
    return 1.0 / math.sqrt(nope + rope)
