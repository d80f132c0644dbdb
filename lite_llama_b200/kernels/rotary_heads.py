"""Rotary positions from a frequency table, and the per-token preparation of attention layers that norm every head on
its own (csrc/rotary_heads.cu).  The reference rotates with one fixed frequency law and the rotate-half pairing
(lite_llama/kernels/rope_emb.py); here the frequencies are data (interpolated variants compute them on the host) and the
pairing is a parameter."""

from __future__ import annotations

import math

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle

PAIRINGS = {"neighbours": 0, "halves": 1}


def rotary_frequencies(dims: int, base: float, factor: float = 1.0, original: float = 0.0, fast: float = 0.0,
                       slow: float = 0.0) -> tuple[list[float], float]:
    """Per-pair angular frequencies ``f_i = base^(-2i/dims)`` and the magnitude that multiplies cos and sin.  With
    ``factor > 1`` (frequency interpolation by parts): a pair that completes more than ``fast`` turns over ``original``
    positions keeps ``f_i``, one that completes fewer than ``slow`` turns gets ``f_i / factor``, a linear ramp over the
    pair index joins them, and the magnitude is ``0.1 ln(factor) + 1``."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if factor == 1.0 or not original:
        return f, 1.0

    def pair_index(turns: float) -> float:              # the (real-valued) pair that completes `turns` turns
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(fast)), 0)
    hi = min(math.ceil(pair_index(slow)), dims - 1)
    width = max(hi - lo, 0.001)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / width, 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@torch.no_grad()
def rope_table_freqs(positions: torch.Tensor, freqs: torch.Tensor, magnitude: float = 1.0) -> torch.Tensor:
    """fp32 ``[T, 2 * len(freqs)]`` = per token ``magnitude * [cos | sin]`` of ``position * freqs[i]``; the frequencies
    are an fp64 tensor and the angles are formed and evaluated in fp64."""
    require_cuda(positions, freqs)
    if freqs.dtype != torch.float64 or positions.dtype != torch.int32 or not freqs.is_contiguous():
        raise ValueError("rope_table_freqs: int32 positions, fp64 frequencies")
    dims = 2 * freqs.numel()
    out = torch.empty((positions.numel(), dims), dtype=torch.float32, device=positions.device)
    check(lib().b2l_rope_table_freqs(out.data_ptr(), positions.data_ptr(), freqs.data_ptr(), positions.numel(), dims,
                                     float(magnitude), stream_handle()))
    return out


@torch.no_grad()
def head_norm_rope_prepare(qkv: torch.Tensor, kv_pool: torch.Tensor, kv_rows: torch.Tensor,
                           cos_sin: torch.Tensor | None, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None,
                           heads: int, kv_heads: int, head_dim: int, v_head_dim: int, rot_dims: int, eps: float,
                           pairing: str = "neighbours") -> None:
    """Per token of ``qkv [T, heads*head_dim + kv_heads*(head_dim + v_head_dim)]``: per-head RMS norm of q and k (one
    ``[head_dim]`` weight each), rotation of the first ``rot_dims`` entries of every head by the token's row of
    ``cos_sin``, q in place, ``[k | v]`` into pool row ``kv_rows[t]``."""
    require_cuda(qkv, kv_pool, kv_rows, cos_sin, q_norm, k_norm)
    if qkv.stride(-1) != 1 or kv_pool.stride(-1) != 1 or kv_pool.shape[1] < kv_heads * (head_dim + v_head_dim):
        raise ValueError("head_norm_rope_prepare: bad layout")
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.shape[1] != rot_dims or not cos_sin.is_contiguous()):
        raise ValueError("head_norm_rope_prepare: cos_sin is fp32 [T, rot_dims]")
    check(lib().b2l_head_norm_rope_prepare(qkv.data_ptr(), qkv.stride(0), kv_pool.data_ptr(), kv_pool.stride(0),
                                           kv_rows.data_ptr(), ptr(cos_sin), ptr(q_norm), ptr(k_norm), qkv.shape[0],
                                           heads, kv_heads, head_dim, v_head_dim, rot_dims if cos_sin is not None else 0,
                                           PAIRINGS[pairing], float(eps), float_code(qkv, "qkv"), stream_handle()))
