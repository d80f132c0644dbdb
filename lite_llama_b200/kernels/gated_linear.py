"""Linear attention with data-dependent gates over ragged steps, and the small ops around it
(csrc/gated_linear_attention.cu).  No reference counterpart: the reference's mixers are softmax attention only."""

from __future__ import annotations

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle

GATED_LINEAR_MODES = {"forget_gate": 0, "delta_rule": 1}


@torch.no_grad()
def gated_linear_scan(mode: str, state: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, seq_start,
                      seq_ctx, seq_slot, heads: int, qk_heads: int, dim: int, vdim: int, c0: torch.Tensor,
                      c1: torch.Tensor | None = None, p0: torch.Tensor | None = None, p1: torch.Tensor | None = None,
                      q_scale: float = 1.0, unit_eps: float = 1e-6) -> torch.Tensor:
    """``y [tokens, heads * vdim]`` fp32; ``state [slots, heads, dim, vdim]`` fp32 advanced in place.  ``q``, ``k``,
    ``v``, ``p0``, ``p1`` are column views of projections (row strides kept).

    ``"forget_gate"``: ``f = c0 + (1 - c0) * sigmoid(k)`` per key channel (``c0`` = lower bounds ``[heads * dim]``),
    ``S[d, :] <- f[d] S[d, :] + (1 - f[d]) v``, ``y = S^T silu(q)``.
    ``"delta_rule"``: ``q``, ``k`` ``[tokens, qk_heads * dim]`` become unit vectors (``unit_eps`` inside the root; ``q``
    times ``q_scale``); ``g = exp(-exp(c1) * softplus(p1 + c0))``, ``beta = sigmoid(p0)`` per head;
    ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; y = S^T q``."""
    require_cuda(state, q, k, v, c0, c1, p0, p1)
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise ValueError("gated_linear_scan: the memory is a contiguous fp32 [slots, heads, dim, vdim] tensor")
    for t in (q, k, v, p0, p1):
        if t is not None and (t.stride(-1) != 1 or t.dtype != q.dtype):
            raise ValueError("gated_linear_scan: the inputs are column views of one dtype")
    tokens = q.shape[0]
    y = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=q.device)
    check(lib().b2l_gated_linear_scan(y.data_ptr(), state.data_ptr(), q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0),
                                      v.data_ptr(), v.stride(0), ptr(p0), p0.stride(0) if p0 is not None else 0, ptr(p1),
                                      p1.stride(0) if p1 is not None else 0, c0.data_ptr(), ptr(c1), seq_start.data_ptr(),
                                      seq_ctx.data_ptr(), seq_slot.data_ptr(), seq_ctx.numel(), heads, qk_heads, dim,
                                      vdim, float(q_scale), float(unit_eps), GATED_LINEAR_MODES[mode],
                                      float_code(q, "q"), stream_handle()))
    return y


@torch.no_grad()
def head_norm_gate(y: torch.Tensor, weight: torch.Tensor, heads: int, eps: float,
                   gate: torch.Tensor | None = None) -> torch.Tensor:
    """``unit_rms(y[t, h, :]) * weight * silu(gate[t, h, :])`` per head (``gate=None``: no gate); ``y`` fp32
    ``[tokens, heads * vdim]``, ``weight [vdim]`` shared by the heads, output in ``weight``'s dtype."""
    require_cuda(y, weight, gate)
    rows, inner = y.shape
    vdim = inner // heads
    if y.dtype != torch.float32 or not y.is_contiguous() or weight.numel() != vdim or heads * vdim != inner or \
            (gate is not None and (gate.stride(-1) != 1 or gate.dtype != weight.dtype)):
        raise ValueError("head_norm_gate: bad layout")
    out = torch.empty((rows, inner), dtype=weight.dtype, device=y.device)
    check(lib().b2l_head_norm_gate(out.data_ptr(), y.data_ptr(), ptr(gate), gate.stride(0) if gate is not None else 0,
                                   weight.data_ptr(), rows, heads, vdim, float(eps), float_code(weight, "weight"),
                                   stream_handle()))
    return out


@torch.no_grad()
def head_mix(wide: torch.Tensor, mix: torch.Tensor, heads: int, kv_heads: int, per_call: int, vdim: int) -> torch.Tensor:
    """``out[t, h, :] = sum_g mix[h, g] * wide[t, g, kv(h), :]`` for ``wide [tokens, calls, heads, per_call, vdim]``
    (contiguous), where ``wide[t, c // per_call, g, c % per_call]`` is query head g's softmax weights applied to kv head
    c's values: mixing the heads' attention weights after the softmax equals mixing these outputs."""
    require_cuda(wide, mix)
    rows = wide.shape[0]
    if not wide.is_contiguous() or wide.numel() != rows * heads * kv_heads * vdim or mix.numel() != heads * heads or \
            mix.dtype != wide.dtype or not mix.is_contiguous():
        raise ValueError("head_mix: bad layout")
    out = torch.empty((rows, heads * vdim), dtype=wide.dtype, device=wide.device)
    check(lib().b2l_head_mix(out.data_ptr(), wide.data_ptr(), heads * kv_heads * vdim, mix.data_ptr(), rows, heads, kv_heads,
                             per_call, vdim, float_code(wide, "wide"), stream_handle()))
    return out


@torch.no_grad()
def swiglu_scaled(gate: torch.Tensor, up: torch.Tensor, in_scale: torch.Tensor | None = None,
                  out_logit: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(s * gate) * (s * up) * sigmoid(z)`` with one fp32 factor ``s = in_scale[r]`` and one logit
    ``z = out_logit[r, 0]`` per row (both optional).  A factor on a gated unit's INPUT passes through its two linear
    maps, so it is applied here, between the products and the activation."""
    require_cuda(gate, up, in_scale, out_logit)
    rows, n = gate.shape
    if up.shape != gate.shape or gate.stride(-1) != 1 or up.stride(-1) != 1 or up.dtype != gate.dtype or \
            (in_scale is not None and (in_scale.dtype != torch.float32 or in_scale.numel() != rows or not in_scale.is_contiguous())) or \
            (out_logit is not None and (out_logit.dtype != gate.dtype or out_logit.shape[0] != rows)):
        raise ValueError("swiglu_scaled: bad layout")
    out = torch.empty((rows, n), dtype=gate.dtype, device=gate.device)
    check(lib().b2l_swiglu_scaled(out.data_ptr(), out.stride(0), gate.data_ptr(), gate.stride(0), up.data_ptr(),
                                  up.stride(0), ptr(in_scale), ptr(out_logit),
                                  out_logit.stride(0) if out_logit is not None else 0, rows, n, float_code(gate, "gate"),
                                  stream_handle()))
    return out
