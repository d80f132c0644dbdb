"""Ops around an fp32 residual stream (csrc/residual_stream.cu): the residual sum stays in 32 bits while the
projections run in the activation dtype.  No reference counterpart: the reference keeps a 16-bit residual and puts
its norms in front of the sublayers (lite_llama/models/base.py:299-319)."""

from __future__ import annotations

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle


NORM_KINDS = {"rms": 0, "layer": 1}


@torch.no_grad()
def embed_positions(tokens: torch.Tensor, positions: torch.Tensor, embed: torch.Tensor,
                    pos_table: torch.Tensor | None, want_act: bool = True, scale: float = 1.0):
    """``residual[t] = scale * embed[tokens[t]] + pos_table[positions[t]]`` in fp32; also returns the copy in
    ``embed``'s dtype that the next projection reads (``None`` when that dtype is fp32: the residual itself serves)."""
    require_cuda(tokens, positions, embed, pos_table)
    if tokens.dtype != torch.int32 or positions.dtype != torch.int32:
        raise ValueError("embed_positions takes int32 token and position vectors")
    rows, n = tokens.numel(), embed.shape[1]
    resid = torch.empty((rows, n), dtype=torch.float32, device=embed.device)
    act = torch.empty((rows, n), dtype=embed.dtype, device=embed.device) if want_act and embed.dtype != torch.float32 else None
    check(lib().b2l_embed_positions(resid.data_ptr(), ptr(act), tokens.data_ptr(), positions.data_ptr(), embed.data_ptr(),
                                    ptr(pos_table), rows, n, embed.shape[0],
                                    pos_table.shape[0] if pos_table is not None else 1, float(scale),
                                    float_code(embed, "embed"), stream_handle()))
    return resid, act


@torch.no_grad()
def post_norm_residual(residual: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float,
                       weight_offset: float = 1.0, want_act: bool = True, kind: str = "rms",
                       layer_scale: torch.Tensor | None = None, next_weight: torch.Tensor | None = None,
                       next_kind: str = "rms") -> torch.Tensor | None:
    """``residual += norm(y) * (weight_offset + weight) * layer_scale`` in place (fp32; ``kind``: "rms" or "layer").
    Returns the updated residual in ``y``'s dtype for the next projection (``None`` for fp32) -- or, with
    ``next_weight``, the next sublayer's INPUT norm of it, ``norm'(residual) * next_weight`` (always a tensor)."""
    require_cuda(residual, y, weight)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise ValueError("post_norm_residual: the residual stream is a contiguous fp32 tensor")
    rows, n = residual.shape
    if y.shape != residual.shape or y.stride(-1) != 1 or weight.dtype != y.dtype:
        raise ValueError("post_norm_residual: y must match the residual's shape and the weight's dtype")
    for t in (layer_scale, next_weight):
        if t is not None and (t.dtype != y.dtype or t.numel() != n):
            raise ValueError("post_norm_residual: layer scale / next weight must be [n] in y's dtype")
    need = want_act and (y.dtype != torch.float32 or next_weight is not None)
    act = torch.empty((rows, n), dtype=y.dtype, device=y.device) if need else None
    check(lib().b2l_post_norm_residual(residual.data_ptr(), ptr(act), y.data_ptr(), weight.data_ptr(), ptr(layer_scale),
                                       ptr(next_weight) if need else None, rows, n, y.stride(0), float(eps),
                                       float(weight_offset), NORM_KINDS[kind], NORM_KINDS[next_kind],
                                       float_code(y, "y"), stream_handle()))
    return act


@torch.no_grad()
def rmsnorm_from_f32(residual: torch.Tensor, weight: torch.Tensor, eps: float, weight_offset: float = 1.0,
                     rows: torch.Tensor | None = None, kind: str = "rms") -> torch.Tensor:
    """Norm (``kind``: "rms" or "layer") of (selected rows of) the fp32 residual, written in ``weight``'s dtype."""
    require_cuda(residual, weight, rows)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise ValueError("rmsnorm_from_f32: the residual stream is a contiguous fp32 tensor")
    if rows is not None and rows.dtype != torch.int32:
        raise ValueError("rmsnorm_from_f32: rows must be int32")
    count = residual.shape[0] if rows is None else rows.numel()
    n = residual.shape[1]
    out = torch.empty((count, n), dtype=weight.dtype, device=weight.device)
    check(lib().b2l_rmsnorm_from_f32(out.data_ptr(), residual.data_ptr(), ptr(rows), weight.data_ptr(), count, n,
                                     float(eps), float(weight_offset), NORM_KINDS[kind], float_code(weight, "weight"),
                                     stream_handle()))
    return out


@torch.no_grad()
def relu_squared(x: torch.Tensor) -> torch.Tensor:
    require_cuda(x)
    x = x if x.is_contiguous() else x.contiguous()
    out = torch.empty_like(x)
    check(lib().b2l_relu_squared(out.data_ptr(), x.data_ptr(), x.numel(), float_code(x, "x"), stream_handle()))
    return out


@torch.no_grad()
def gelu(x: torch.Tensor, approximate: str = "none") -> torch.Tensor:
    """Exact (erf) GELU, or the tanh form with ``approximate="tanh"``; evaluated in fp32."""
    require_cuda(x)
    x = x if x.is_contiguous() else x.contiguous()
    out = torch.empty_like(x)
    check(lib().b2l_gelu(out.data_ptr(), x.data_ptr(), x.numel(), {"none": 0, "tanh": 1}[approximate],
                         float_code(x, "x"), stream_handle()))
    return out


@torch.no_grad()
def softcap_to_f32(x: torch.Tensor, cap: float, scale: float = 1.0) -> torch.Tensor:
    """``cap * tanh(scale * x / cap)`` as fp32 (``cap <= 0``: ``scale * x``): the logits a scaled, soft-capped head
    hands out."""
    require_cuda(x)
    x = x if x.is_contiguous() else x.contiguous()
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    check(lib().b2l_softcap_to_f32(out.data_ptr(), x.data_ptr(), x.numel(), float(cap or 0.0), float(scale), float_code(x, "x"),
                                   stream_handle()))
    return out
