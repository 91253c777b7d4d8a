"""CPU restatement of the GQA block-sparse attention path (test infrastructure only).

Nothing under ``sgl_amd_mono_b200`` may import this module: it is the checker the GPU
kernels are compared with, never a fallback.  Parity is unpinned: the reference's
kernels for this path are JIT-compiled gfx950 programs that cannot run here and its
tests hold no golden vectors for it, so every function restates the formula of the
cited reference lines.

Reference (``sgl_amd_mono/minimax_m3/gfx950``):

* per-head Gemma RMSNorm and partial NeoX RoPE, K / V to the FP8 cache with the layer's
  fixed scale, index key to the index cache as E4M3 with unit scale: ``pre_attn.py:8-19``;
* block score = max over a block's causal keys of (index_q . index_k) times
  fp32(sm_scale * log2 e): ``index_score.py:1-12,60-62``;
* selection: top 16 blocks by (score, block id) descending, the first ``init_blocks``
  pinned to 1e30 and the last ``local_blocks`` to 1e29, rank by counting, full blocks in
  rank order and the tail block last: ``post_attn.py:466-592``, ``select.py:1-56``;
* attention over the selected keys with split-local softmax and a merge:
  ``post_attn.py:706-979``.

Block = page = 64 tokens (the BASELINE configuration; the reference's own build uses
128-token blocks of 16-token pages, ``config.py:37-42``).
"""

from __future__ import annotations

import math
import struct

import torch

from . import quant as Q

BLOCK = 64
TOPK_BLOCKS = 16
HEAD_DIM = 128
ROTARY = 64
LOG2E = 1.4426950408889634


def _f32(x: float) -> float:
    return struct.unpack("f", struct.pack("f", x))[0]


def index_scale_log2e(sm_scale: float) -> float:
    """fp32(fp32(sm_scale) * fp32(log2 e)) (``index_score.py:59-62``)."""
    return _f32(_f32(sm_scale) * _f32(LOG2E))


def head_norm_rope(x: torch.Tensor, gamma: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, eps: float,
                   rope: bool = True) -> torch.Tensor:
    """One head [128] f32 -> bf16-rounded f32: Gemma RMSNorm (weight 1 + gamma), then NeoX
    rotation of dims (i, i + 32), i < 32, with cos/sin [32] (``pre_attn.py:14-16``)."""
    x = x.float()
    rstd = torch.rsqrt((x * x).mean() + eps)
    y = Q.bf(x * rstd * (1.0 + gamma.float()))
    if not rope:
        return y
    out = y.clone()
    a, b = y[:32], y[32:64]
    c, s = cos.float(), sin.float()
    out[:32] = Q.bf(a * c - b * s)
    out[32:64] = Q.bf(b * c + a * s)
    return out


def neox_table(positions: int, rotary: int = ROTARY, theta: float = 1.0e6):
    """bf16 cos / sin tables [positions, rotary / 2]."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary, 2, dtype=torch.float64) / rotary))
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cos(ang).float().bfloat16(), torch.sin(ang).float().bfloat16()


def fp8_scaled_bytes(x_bf: torch.Tensor, scale: float) -> torch.Tensor:
    """E4M3 bytes of x / scale, saturating (the layer's fixed K or V scale)."""
    return Q.e4m3_bytes((x_bf.float() / scale).clamp(-448.0, 448.0))


def block_scores(iq_bf: torch.Tensor, index_keys: torch.Tensor, seq_len: int, sm_scale: float) -> torch.Tensor:
    """Score of every block of one row.  ``iq_bf`` [128] bf16 values, ``index_keys``
    [ctx, 128] decoded E4M3 index keys in position order.  f32 [n_blk]."""
    n_blk = (seq_len + BLOCK - 1) // BLOCK
    dots = index_keys[:seq_len].float() @ iq_bf.float()
    out = torch.full((n_blk,), float("-inf"))
    scale = torch.tensor(index_scale_log2e(sm_scale), dtype=torch.float32)
    for b in range(n_blk):
        out[b] = dots[b * BLOCK : min((b + 1) * BLOCK, seq_len)].max() * scale
    return out


def index_key(score_bits: int, b: int, n_blk: int, init_blocks: int, local_blocks: int) -> int:
    """Signed 32-bit sort key of block b (``post_attn.py:466-477``): pinned blocks first, then an
    integer ordered like the float (-0 == 0, NaN below -inf)."""
    sc = struct.unpack("f", struct.pack("I", score_bits & 0xFFFFFFFF))[0]
    if b < init_blocks:
        sc = 1e30
    if b >= n_blk - local_blocks:
        sc = 1e29
    bits = struct.unpack("i", struct.pack("f", sc))[0]
    if bits == -(2**31):
        bits = 0
    key = bits ^ 0x7FFFFFFF if bits < 0 else bits
    if (bits & 0x7FFFFFFF) > 0x7F800000:
        key = -(2**31)
    return key


def select_blocks(scores: torch.Tensor, seq_len: int, init_blocks: int, local_blocks: int):
    """-> (block ids in slot order, sparse context length).  A context of at most 16 blocks
    keeps every block in order; otherwise the 16 best by (key, block id) descending, full
    blocks by rank and the tail block last (``post_attn.py:540-592``)."""
    n_blk = (seq_len + BLOCK - 1) // BLOCK
    tail = n_blk - 1
    if n_blk <= TOPK_BLOCKS:
        keys = [(-b, b) for b in range(n_blk)]  # unscored: blocks rank by id (post_attn.py:531)
    else:
        bits = scores.contiguous().view(torch.int32).tolist()
        keys = [(index_key(bits[b], b, n_blk, init_blocks, local_blocks), b) for b in range(n_blk)]
    order = sorted(keys, key=lambda kb: (kb[0], kb[1]), reverse=True)
    n_sel = min(n_blk, TOPK_BLOCKS)
    chosen = [b for _, b in order[:n_sel]]
    tail_sel = tail in chosen
    full = [b for b in chosen if b != tail]
    slots = full + ([tail] if tail_sel else [])
    if tail_sel:
        n_ctx = len(full) * BLOCK + seq_len - tail * BLOCK
    else:
        n_ctx = min(n_sel * BLOCK, seq_len)
    return slots, n_ctx


def sparse_attention_row(q_bf: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_scale: float, v_scale: float,
                         n_ctx: int, sm_scale: float) -> torch.Tensor:
    """One row, one kv head.  q_bf [G, 128] (the group's q heads, bf16 values); k, v
    [slots * 64, 128] decoded E4M3 keys / values in slot order; the first n_ctx are live.
    Per 64-key block: s = (q . k) * k_scale * sm_scale, local max / sum, p rounded to bf16,
    PV in f32; blocks merged with w_j = exp(m_j - M) (``post_attn.py:801-979``).  bf16 [G, 128]."""
    G = q_bf.shape[0]
    nb = (n_ctx + BLOCK - 1) // BLOCK
    ms, ls, accs = [], [], []
    for b in range(nb):
        lo, hi = b * BLOCK, min((b + 1) * BLOCK, n_ctx)
        s = (q_bf.float() @ k[lo:hi].float().T) * torch.tensor(k_scale * sm_scale, dtype=torch.float32)
        m = s.max(dim=1).values
        p = torch.exp(s - m[:, None])
        ls.append(p.sum(dim=1))
        accs.append(Q.bf(p) @ v[lo:hi].float())
        ms.append(m)
    M = torch.stack(ms).max(dim=0).values
    num = torch.zeros(G, HEAD_DIM)
    den = torch.zeros(G)
    for m, l, a in zip(ms, ls, accs):
        w = torch.exp(m - M)
        num += a * w[:, None]
        den += l * w
    return Q.bf(num / den[:, None] * torch.tensor(v_scale, dtype=torch.float32))


def sm_scale_gqa(head_dim: int = HEAD_DIM) -> float:
    return 1.0 / math.sqrt(head_dim)


def attention_half(cfg, w: dict, x: torch.Tensor, positions, slots, page_table, caches, cos, sin) -> torch.Tensor:
    """One rank's attention half of a layer for ``x`` [rows, hidden] bf16 (``pre_attn.py:8-19`` then
    ``post_attn.py:466-1003``): input RMSNorm, fused projection, head norms + RoPE, cache insert
    (``caches`` = [k, v, index] uint8 tensors, modified in place), block scores, selection,
    attention, o_proj, residual.  Single rank: the all-reduce is the identity.  bf16 [rows, hidden]."""
    from . import stages as S

    k_cache, v_cache, index_cache = caches
    nq, nk = cfg.q_local, cfg.kv_local
    G = nq // nk
    xn = S.rmsnorm(x, w["in_norm"], cfg.eps)
    qkv = S.gemv_fp8_block(xn, w["qkv"], w["qkv_s"]).reshape(x.shape[0], -1, HEAD_DIM)
    attn = torch.zeros(x.shape[0], nq * HEAD_DIM)
    for r in range(x.shape[0]):
        pos, slot = int(positions[r]), int(slots[r])
        if slot < 0:
            continue
        c, s = cos[pos], sin[pos]
        q = torch.stack([head_norm_rope(qkv[r, h], w["g_q"], c, s, cfg.eps) for h in range(nq)])
        iq = head_norm_rope(qkv[r, nq + 2 * nk], w["g_iq"], c, s, cfg.eps)
        page, off = slot // BLOCK, slot % BLOCK
        for h in range(nk):
            k_cache[page, off, h] = fp8_scaled_bytes(head_norm_rope(qkv[r, nq + h], w["g_k"], c, s, cfg.eps), w["k_scale"])
            v_cache[page, off, h] = fp8_scaled_bytes(Q.bf(qkv[r, nq + nk + h]), w["v_scale"])
        index_cache[page, off] = Q.e4m3_bytes(head_norm_rope(qkv[r, nq + 2 * nk + 1], w["g_ik"], c, s, cfg.eps))
        seq = pos + 1
        n_blk = (seq + BLOCK - 1) // BLOCK
        pt = page_table[r].long()
        scores = block_scores(iq, Q.e4m3_from_bytes(index_cache[pt[:n_blk]].reshape(-1, HEAD_DIM)), seq, cfg.sm_scale)
        blocks, n_ctx = select_blocks(scores, seq, cfg.init_blocks, cfg.local_blocks)
        for h in range(nk):
            kk = Q.e4m3_from_bytes(k_cache[pt[blocks], :, h].reshape(-1, HEAD_DIM))
            vv = Q.e4m3_from_bytes(v_cache[pt[blocks], :, h].reshape(-1, HEAD_DIM))
            o = sparse_attention_row(q[h * G : (h + 1) * G], kk, vv, w["k_scale"], w["v_scale"], n_ctx, cfg.sm_scale)
            attn[r, h * G * HEAD_DIM : (h + 1) * G * HEAD_DIM] = o.reshape(-1)
    o_proj = S.gemv_fp8_block(attn, w["o"], w["o_s"])
    out = Q.bf(x.float() + Q.bf(o_proj))
    live = torch.as_tensor(slots) >= 0
    return torch.where(live[:, None], out, x.float()).bfloat16()
