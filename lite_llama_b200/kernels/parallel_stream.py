"""Ops of layer-list models built from PARALLEL blocks around an fp32 residual stream that keeps every layer's result
(csrc/parallel_stream.cu): the mixer and the feed-forward read two norms of the same input, their outputs join the
residual in one pass, a per-layer token input follows, and a depth-weighted average of all results so far feeds the next
layer.  No reference counterpart: the reference's layers are sequential pre-norm blocks over a 16-bit residual
(lite_llama/models/base.py:299-319)."""

from __future__ import annotations

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle


@torch.no_grad()
def embed_rmsnorm(tokens: torch.Tensor, embed: torch.Tensor, weight: torch.Tensor | None, eps: float,
                  weight_offset: float = 1.0, scale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``unit_rms(scale * embed[tokens]) * (weight_offset + weight)`` (``weight=None``: the unit-RMS rows),
    written to ``out [tokens, n]`` when given."""
    require_cuda(tokens, embed, weight, out)
    if tokens.dtype != torch.int32:
        raise ValueError("embed_rmsnorm takes an int32 token vector")
    rows, n = tokens.numel(), embed.shape[1]
    if out is None:
        out = torch.empty((rows, n), dtype=torch.float32, device=embed.device)
    elif out.dtype != torch.float32 or out.shape != (rows, n) or not out.is_contiguous():
        raise ValueError("embed_rmsnorm: out is a contiguous fp32 [tokens, n] tensor")
    check(lib().b2l_embed_rmsnorm(out.data_ptr(), tokens.data_ptr(), embed.data_ptr(), ptr(weight), rows, n,
                                  embed.shape[0], float(eps), float(weight_offset), float(scale),
                                  float_code(embed, "embed"), stream_handle()))
    return out


@torch.no_grad()
def depth_mix_norms(stack: torch.Tensor, count: int, coef: torch.Tensor | None, w1: torch.Tensor | None,
                    w2: torch.Tensor | None, eps: float, weight_offset: float = 1.0, out: torch.Tensor | None = None,
                    dtype: torch.dtype | None = None):
    """``stack [levels, tokens, n]`` fp32.  ``x = sum_j coef[j] * stack[j]`` over the first ``count`` levels
    (``coef=None``: ``x = stack[count - 1]``), stored in ``out`` (fp32 ``[tokens, n]``; usually the next level of the
    stack); returns ``(unit_rms(x) * (weight_offset + w1), the same with w2)`` in the weights' dtype, ``None`` for a
    weight that is not given."""
    require_cuda(stack, coef, w1, w2, out)
    if stack.dtype != torch.float32 or stack.dim() != 3 or not stack.is_contiguous() or not 1 <= count <= stack.shape[0]:
        raise ValueError("depth_mix_norms: stack is a contiguous fp32 [levels, tokens, n] tensor")
    _, rows, n = stack.shape
    ref = w1 if w1 is not None else (w2 if w2 is not None else coef)
    dt = ref.dtype if ref is not None else (dtype or torch.float32)
    for t in (coef, w1, w2):
        if t is not None and t.dtype != dt:
            raise ValueError("depth_mix_norms: coefficients and weights share one dtype")
    if coef is not None and coef.numel() < count:
        raise ValueError("depth_mix_norms: fewer coefficients than levels")
    if out is None:
        out = torch.empty((rows, n), dtype=torch.float32, device=stack.device)
    h1 = torch.empty((rows, n), dtype=dt, device=stack.device) if w1 is not None else None
    h2 = torch.empty((rows, n), dtype=dt, device=stack.device) if w2 is not None else None
    code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[dt]
    check(lib().b2l_depth_mix_norms(out.data_ptr(), ptr(h1), ptr(h2), stack.data_ptr(), stack.stride(0), ptr(coef), count,
                                    ptr(w1), ptr(w2), rows, n, float(eps), float(weight_offset), code, stream_handle()))
    return out, h1, h2


@torch.no_grad()
def branch_sum_residual(residual: torch.Tensor, a: torch.Tensor, a_weight: torch.Tensor | None = None,
                        b: torch.Tensor | None = None, b_weight: torch.Tensor | None = None,
                        c: torch.Tensor | None = None, eps: float = 0.0, scale: float = 1.0,
                        want_act: bool = True, scale_b: float | None = None,
                        next_weight: torch.Tensor | None = None) -> torch.Tensor | None:
    """``residual += scale * a' + scale_b * b' + c`` in place (fp32), where ``a' = unit_rms(a) * a_weight`` when the
    weight is given, else ``a`` (``b`` likewise; ``b`` and ``c`` optional; ``scale_b`` defaults to ``scale``).  Returns
    the new residual in ``a``'s dtype for the next projection (``None`` for fp32 or ``want_act=False``); with
    ``next_weight`` it returns ``unit_rms(new residual) * next_weight`` instead, the input norm of the block that
    follows, in every dtype."""
    require_cuda(residual, a, a_weight, b, b_weight, c, next_weight)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise ValueError("branch_sum_residual: the residual stream is a contiguous fp32 tensor")
    rows, n = residual.shape
    for t in (a, b, c):
        if t is not None and (t.shape != residual.shape or t.stride(-1) != 1 or t.dtype != a.dtype):
            raise ValueError("branch_sum_residual: the branches match the residual's shape and share one dtype")
    for t in (a_weight, b_weight, next_weight):
        if t is not None and (t.dtype != a.dtype or t.numel() != n):
            raise ValueError("branch_sum_residual: norm weights are [n] in the branches' dtype")
    act = None
    if next_weight is not None or (want_act and a.dtype != torch.float32):
        act = torch.empty((rows, n), dtype=a.dtype, device=a.device)
    check(lib().b2l_branch_sum_residual(residual.data_ptr(), ptr(act), a.data_ptr(), a.stride(0), ptr(a_weight), ptr(b),
                                        b.stride(0) if b is not None else 0, ptr(b_weight), ptr(c),
                                        c.stride(0) if c is not None else 0, ptr(next_weight), rows, n, float(eps),
                                        float(scale), float(scale if scale_b is None else scale_b), float_code(a, "a"),
                                        stream_handle()))
    return act


@torch.no_grad()
def gelu_mul_gather(z: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, col0: int) -> torch.Tensor:
    """``gelu_tanh(z[t, d]) * table[tokens[t], col0 + d]`` for ``z [tokens, dim]``."""
    require_cuda(z, tokens, table)
    rows, dim = z.shape
    if z.stride(-1) != 1 or table.dtype != z.dtype or table.stride(-1) != 1 or tokens.dtype != torch.int32:
        raise ValueError("gelu_mul_gather: bad layout")
    out = torch.empty((rows, dim), dtype=z.dtype, device=z.device)
    check(lib().b2l_gelu_mul_gather(out.data_ptr(), z.data_ptr(), z.stride(0), tokens.data_ptr(), table.data_ptr(),
                                    table.stride(0), table.shape[0], int(col0), dim, rows, float_code(z, "z"),
                                    stream_handle()))
    return out
