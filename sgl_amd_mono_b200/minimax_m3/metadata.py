"""The step's per-row tables, made on the device inside the captured graph.

Reference counterpart: ``minimax_m3/metadata.py:7-42`` (``prepare_token_rows``).  SGLang hands a step over per
REQUEST (``req_pool_indices``, ``seq_lens``) and the launches want it per ROW: a decode step has one row per request,
a linear verify step ``query_len`` rows per request, and row j of a request may see the request's accepted prefix plus
its own j + 1 tokens and nothing later.  Everything here is index arithmetic on tensors that already live on the
device, written into buffers allocated at build: it can be captured into a CUDA graph and gives fresh tables on every
replay.  Rows whose cache slot is 0 (the allocator's graph padding) or negative (no cache write) come out with zero
keys and a zero table, so that they attend nothing and join no expert union.
"""

from __future__ import annotations

import torch


def prepare_token_rows(req_to_token, req_pool_indices, seq_lens, block_columns, out_block_table, out_seq_lens,
                       slot_mapping, query_len: int, is_verify: bool, max_context_len: int, block_tokens: int = 128):
    """Fills ``out_block_table`` [rows, len(block_columns)] and ``out_seq_lens`` [rows] in place and returns them.

    ``req_to_token`` [pool, tokens]: a request's token slots; ``block_columns``: the token column that starts each
    block (``arange(0, max_context, block_tokens)``); a block's id is its first slot // ``block_tokens`` (the
    reference's blocks hold 128 tokens, this library's GQA caches 64: pass 64 there).  In a verify step SGLang's
    ``seq_lens`` hold the accepted prefix, so row j sees prefix + j + 1 keys, clamped to ``max_context_len`` (rows the
    scheduler drops past the context limit only have to stay in bounds).
    """
    rows = out_seq_lens.shape[0]
    if query_len < 1 or rows % query_len:
        raise ValueError(f"prepare_token_rows: {rows} rows are not whole requests of {query_len} rows")
    if out_block_table.shape != (rows, block_columns.shape[0]):
        raise ValueError(f"prepare_token_rows: block table {tuple(out_block_table.shape)}, needs "
                         f"{(rows, block_columns.shape[0])}")
    dev = seq_lens.device
    row = torch.arange(rows, dtype=torch.int64, device=dev)
    req = row // query_len                              # the request a row belongs to
    pool_row = req_pool_indices.index_select(0, req).to(torch.int64)
    first_slot = req_to_token.index_select(0, pool_row).index_select(1, block_columns.to(torch.int64))
    out_block_table.copy_(torch.div(first_slot, block_tokens, rounding_mode="floor"))
    keys = seq_lens.index_select(0, req)
    if is_verify:
        keys = torch.clamp(keys + (row - req * query_len + 1).to(keys.dtype), max=max_context_len)
    live = slot_mapping[:rows] > 0
    out_seq_lens.copy_(torch.where(live, keys, torch.zeros_like(keys)))
    out_block_table.mul_(live.to(out_block_table.dtype).unsqueeze(1))
    return out_block_table, out_seq_lens


class TokenRows:
    """The producer with its buffers: one per graph width, allocated at build (nothing is allocated in a step)."""

    def __init__(self, rows: int, max_context: int, device, block_tokens: int = 64):
        self.rows, self.max_context, self.block_tokens = rows, max_context, block_tokens
        self.block_columns = torch.arange(0, max_context, block_tokens, dtype=torch.int64, device=device)
        self.block_table = torch.zeros(rows, self.block_columns.numel(), dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros(rows, dtype=torch.int32, device=device)

    def __call__(self, req_to_token, req_pool_indices, seq_lens, slot_mapping, query_len: int, is_verify: bool):
        return prepare_token_rows(req_to_token, req_pool_indices, seq_lens, self.block_columns, self.block_table,
                                  self.seq_lens, slot_mapping, query_len, is_verify, self.max_context, self.block_tokens)
