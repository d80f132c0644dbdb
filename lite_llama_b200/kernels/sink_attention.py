"""Soft-capped attention with a per-head sink over the token-granular KV pool, for ragged steps
(csrc/attention_sink.cu).  The reference's attention ops (lite_llama/kernels/flashattention2_nopad.py,
flashdecoding.py) have neither cap nor sink, one head size for K and V, and no prompt portions with a cached prefix."""

from __future__ import annotations

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle, workspace


@torch.no_grad()
def attn_prepare(qkv: torch.Tensor, kv_pool: torch.Tensor, kv_rows: torch.Tensor, positions: torch.Tensor,
                 q_cols: int, k_cols: int, v_cols: int, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None,
                 eps: float, gain_coef: float = 0.0, gain_every: float = 0.0, v_first_in: torch.Tensor | None = None,
                 v_first_out: torch.Tensor | None = None, v_lambda: torch.Tensor | None = None) -> None:
    """Whole-row q / k norms, query gain, value mixing and the K|V cache write for the tokens of a step; q is
    normalised in place inside ``qkv [tokens, q_cols + k_cols + v_cols]``."""
    require_cuda(qkv, kv_pool, kv_rows, positions)
    check(lib().b2l_attn_prepare(qkv.data_ptr(), qkv.stride(0), kv_pool.data_ptr(), kv_pool.stride(0), kv_rows.data_ptr(),
                                 positions.data_ptr(), ptr(q_norm), ptr(k_norm), ptr(v_first_in), ptr(v_first_out),
                                 ptr(v_lambda), qkv.shape[0], q_cols, k_cols, v_cols, float(eps), float(gain_coef),
                                 float(gain_every), float_code(qkv, "qkv"), stream_handle()))


@torch.no_grad()
def sink_attention(out: torch.Tensor, q: torch.Tensor, kv_pool: torch.Tensor, table: torch.Tensor, seq_start, seq_ctx,
                   seq_slot, seq_list: torch.Tensor | None, num_seqs: int, max_q_len: int, sink: torch.Tensor | None,
                   heads: int, kv_heads: int, head_dim: int, v_head_dim: int, scale: float, softcap: float,
                   num_splits: int = 0, split_keys: int = 0, window: int = 0, v_col0: int = -1, block: int = 0,
                   v_head_stride: int = -1, v_blocks: int = 1) -> None:
    """Writes ``out [tokens, heads * v_head_dim]`` for the tokens of the listed sequences.  ``num_splits == 0``: tiled
    kernel (prompt portions); ``> 0``: one new token per sequence, its visible keys cut into ranges of ``split_keys``.
    ``window > 0``: a token at position p sees keys p - window + 1 .. p; ``block > 0`` (no window): keys
    ``floor(p / block) * block .. p`` (a block-diagonal causal mask).  ``v_col0 >= 0``: the values start at that
    column of a pool row instead of after the keys (0: the values are the keys' leading columns).  ``v_head_stride >= 0``:
    kv head g's values start ``g * v_head_stride`` columns further (default ``v_head_dim``; 0: every kv head reads the
    same ``v_head_dim`` columns, which lets each query head weigh ALL value heads at once as one wide head).
    ``v_blocks > 1`` (single tokens only): that many neighbouring blocks of ``v_head_dim`` value columns in the same two
    launches, ``out [tokens, v_blocks * heads * v_head_dim]``."""
    require_cuda(out, q, kv_pool, table)
    L = lib()
    nbytes = L.b2l_sink_attention_workspace_bytes(num_seqs, heads * max(1, v_blocks), v_head_dim, num_splits)
    ws = workspace(nbytes, q.device)
    check(L.b2l_sink_attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), kv_pool.data_ptr(),
                               kv_pool.stride(0), table.data_ptr(), table.stride(0), seq_start.data_ptr(),
                               seq_ctx.data_ptr(), seq_slot.data_ptr(), ptr(seq_list), num_seqs, max_q_len, ptr(sink),
                               heads, kv_heads, head_dim, v_head_dim, float(scale), float(softcap or 0.0), int(window),
                               int(block), int(v_col0), int(v_head_stride), int(v_blocks), num_splits, split_keys, ptr(ws), nbytes, float_code(q, "q"),
                               stream_handle()))


MIXED_HEAD_MAX_KEYS = 32768      # the weights of one head and sequence stay in a CTA's shared memory


@torch.no_grad()
def mixed_head_attention(out: torch.Tensor, q: torch.Tensor, kv_pool: torch.Tensor, table: torch.Tensor, seq_start,
                         seq_ctx, seq_slot, seq_list: torch.Tensor | None, num_seqs: int, mix: torch.Tensor, heads: int,
                         kv_heads: int, head_dim: int, v_head_dim: int, scale: float, softcap: float, max_keys: int,
                         window: int = 0, block: int = 0, v_col0: int = -1) -> None:
    """One new token per listed sequence: softmax over its visible keys per head, the heads' weights mixed by
    ``mix [heads, heads]`` (``p'_h = sum_g mix[h, g] p_g``), each head's mixed weights applied to its own kv head's
    values; writes ``out [tokens, heads * v_head_dim]`` rows of those tokens.  ``max_keys`` bounds the keys any of the
    tokens sees (at most ``MIXED_HEAD_MAX_KEYS``)."""
    require_cuda(out, q, kv_pool, table, mix)
    if mix.dtype != q.dtype or mix.numel() != heads * heads or not mix.is_contiguous() or not 0 < max_keys <= MIXED_HEAD_MAX_KEYS:
        raise ValueError("mixed_head_attention: bad mixing matrix or key bound")
    L = lib()
    nbytes = L.b2l_mixed_head_attention_workspace_bytes(num_seqs, heads, max_keys)
    ws = workspace(nbytes, q.device)
    check(L.b2l_mixed_head_attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), kv_pool.data_ptr(),
                                     kv_pool.stride(0), table.data_ptr(), table.stride(0), seq_start.data_ptr(),
                                     seq_ctx.data_ptr(), seq_slot.data_ptr(), ptr(seq_list), num_seqs, mix.data_ptr(),
                                     heads, kv_heads, head_dim, v_head_dim, float(scale), float(softcap or 0.0),
                                     int(window), int(block), int(v_col0), int(max_keys), ptr(ws), nbytes,
                                     float_code(q, "q"), stream_handle()))
