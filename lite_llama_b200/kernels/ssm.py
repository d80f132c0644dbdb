"""State-space mixer ops over ragged steps (csrc/ssm_scan.cu).  No reference counterpart."""

from __future__ import annotations

import torch

from ._common import check, float_code, lib, ptr, require_cuda, stream_handle


@torch.no_grad()
def causal_conv_silu(proj: torch.Tensor, col: int, channels: int, weight: torch.Tensor, bias: torch.Tensor,
                     tail: torch.Tensor, seq_start: torch.Tensor, seq_ctx: torch.Tensor, seq_slot: torch.Tensor,
                     activation: bool = True):
    """``silu(conv(proj[:, col:col+channels]))`` per channel over a ragged step (``activation=False``: the plain
    convolution); ``tail [slots, taps-1, channels]`` supplies the inputs of earlier steps and is advanced in place."""
    require_cuda(proj, weight, bias, tail, seq_start, seq_ctx, seq_slot)
    tokens = proj.shape[0]
    taps = weight.shape[1]
    out = torch.empty((tokens, channels), dtype=proj.dtype, device=proj.device)
    view = proj[:, col:col + channels]
    check(lib().b2l_causal_conv_silu(out.data_ptr(), view.data_ptr(), proj.stride(0), weight.data_ptr(), bias.data_ptr(),
                                     ptr(tail), seq_start.data_ptr(), seq_ctx.data_ptr(), seq_slot.data_ptr(),
                                     seq_ctx.numel(), tokens, channels, taps, 1 if activation else 0,
                                     float_code(proj, "proj"), stream_handle()))
    return out


@torch.no_grad()
def ssm_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias, a_log, d_skip, state: torch.Tensor,
             seq_start, seq_ctx, seq_slot, heads: int, groups: int, state_size: int, head_dim: int,
             fixed_decay: torch.Tensor | None = None, silu_inputs: bool = False) -> torch.Tensor:
    """``y [tokens, heads*head_dim]`` fp32; ``state [slots, heads, state_size, head_dim]`` fp32 advanced in place.
    ``dt_raw`` is a column view ``[tokens, heads]`` of the input projection (row stride kept).  With ``fixed_decay``
    (fp32 ``[heads]``) the recurrence is a decayed linear attention, ``S <- decay_h S + B x^T``, ``y = S^T C``: no step
    size, no skip term (``dt_raw``, ``dt_bias``, ``a_log``, ``d_skip`` may be ``None``); ``silu_inputs`` applies SiLU
    to x, B and C as the kernel reads them."""
    require_cuda(xbc, dt_raw, state, fixed_decay)
    if fixed_decay is not None and (fixed_decay.dtype != torch.float32 or fixed_decay.numel() != heads):
        raise ValueError("ssm_scan: fixed_decay is fp32 [heads]")
    if state.dtype != torch.float32:
        raise ValueError("ssm_scan: the recurrent state is fp32")
    tokens = xbc.shape[0]
    y = torch.empty((tokens, heads * head_dim), dtype=torch.float32, device=xbc.device)
    check(lib().b2l_ssm_scan(y.data_ptr(), state.data_ptr(), xbc.data_ptr(), xbc.stride(0), ptr(dt_raw),
                             dt_raw.stride(0) if dt_raw is not None else 0, ptr(dt_bias), ptr(a_log), ptr(d_skip),
                             seq_start.data_ptr(), seq_ctx.data_ptr(), seq_slot.data_ptr(), seq_ctx.numel(), heads,
                             groups, state_size, head_dim, ptr(fixed_decay), 1 if silu_inputs else 0,
                             float_code(xbc, "xbc"), stream_handle()))
    return y


@torch.no_grad()
def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """``unit_rms(y * silu(z)) * weight`` with the statistic taken in ``groups`` equal parts; ``y`` fp32, ``z`` a
    column view of the projection, output in ``weight``'s dtype."""
    require_cuda(y, z, weight)
    rows, inner = y.shape
    out = torch.empty((rows, inner), dtype=weight.dtype, device=y.device)
    check(lib().b2l_gated_group_norm(out.data_ptr(), y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(), rows,
                                     inner, groups, float(eps), float_code(weight, "weight"), stream_handle()))
    return out


DECAY_ATTENTION_CHUNK = 64


@torch.no_grad()
def decay_attention(x: torch.Tensor, state: torch.Tensor, decay: torch.Tensor, seq_start, seq_ctx, seq_slot, heads: int,
                    state_size: int, head_dim: int, longest: int) -> torch.Tensor:
    """Decayed linear attention ``S <- decay_h S + k v^T``, ``y = S^T q`` on SiLU'd ``x = [v | k | q]`` columns (a view
    of the fused projection): ``y [tokens, heads*head_dim]`` fp32, ``state [slots, heads, state_size, head_dim]`` fp32
    advanced in place.  Steps whose longest sequence brings at least half a chunk of tokens run chunk by chunk on the
    tensor cores when the geometry allows (16-bit activations, sizes of 32 / 64 / 128); everything else -- single
    tokens, fp32, other sizes -- runs the token-by-token scan (``ssm_scan`` with fixed decays)."""
    require_cuda(x, state, decay)
    if state.dtype != torch.float32 or decay.dtype != torch.float32 or decay.numel() != heads:
        raise ValueError("decay_attention: fp32 state, fp32 decays [heads]")
    L = lib()
    code = float_code(x, "x")
    if longest >= DECAY_ATTENTION_CHUNK // 2 and x.stride(-1) == 1 and \
            L.b2l_decay_attention_mma_ok(x.data_ptr(), x.stride(0), state_size, head_dim, code):
        y = torch.empty((x.shape[0], heads * head_dim), dtype=torch.float32, device=x.device)
        check(L.b2l_decay_attention_mma(y.data_ptr(), state.data_ptr(), x.data_ptr(), x.stride(0), decay.data_ptr(),
                                        seq_start.data_ptr(), seq_ctx.data_ptr(), seq_slot.data_ptr(), seq_ctx.numel(),
                                        heads, state_size, head_dim, code, stream_handle()))
        return y
    return ssm_scan(x, None, None, None, None, state, seq_start, seq_ctx, seq_slot, heads, heads, state_size, head_dim,
                    fixed_decay=decay, silu_inputs=True)


@torch.no_grad()
def norm_sigmoid_gate(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``unit_rms(y) * weight * sigmoid(z)`` over whole rows: the gate acts AFTER the norm (``gated_group_norm`` gates
    first).  ``y`` fp32, ``z`` a column view of a projection, output in ``weight``'s dtype."""
    require_cuda(y, z, weight)
    rows, n = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or z.stride(-1) != 1 or weight.numel() != n:
        raise ValueError("norm_sigmoid_gate: bad layout")
    out = torch.empty((rows, n), dtype=weight.dtype, device=y.device)
    check(lib().b2l_norm_sigmoid_gate(out.data_ptr(), y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(), rows, n,
                                      float(eps), float_code(weight, "weight"), stream_handle()))
    return out


GATED_SCAN_MODES = {"mingru": 0, "rglru": 1}


@torch.no_grad()
def gated_scan(mode: str, state: torch.Tensor, p0: torch.Tensor, p1: torch.Tensor, p2: torch.Tensor, seq_start, seq_ctx,
               seq_slot, p3: torch.Tensor | None = None, bias_r: torch.Tensor | None = None,
               bias_i: torch.Tensor | None = None, lam: torch.Tensor | None = None,
               decay_scale: float = 0.0) -> torch.Tensor:
    """Element-wise gated recurrence ``S_t = a_t S_(t-1) + b_t``, ``out_t = S_t g_t`` over a ragged step; ``state
    [slots, width]`` fp32 is advanced in place.  ``p0 .. p3`` are ``[tokens, width]`` column views of projections.

    ``"mingru"``: ``z = sigmoid(p0)``, candidate ``p1 + 1/2`` where ``p1 >= 0`` else ``sigmoid(p1)``, ``a = 1 - z``,
    ``b = z * candidate``, ``g = silu(p2)``.
    ``"rglru"``: ``r = sigmoid(p1 + bias_r)``, ``i = sigmoid(p2 + bias_i)``, ``a = exp(-decay_scale * r *
    softplus(lam))``, ``b = sqrt(1 - a^2) * i * p0``, ``g = gelu_tanh(p3)``."""
    require_cuda(state, p0, p1, p2, p3, bias_r, bias_i, lam)
    if state.dtype != torch.float32:
        raise ValueError("gated_scan: the recurrent state is fp32")
    tokens, width = p0.shape
    for t in (p0, p1, p2, p3):
        if t is not None and (t.shape != p0.shape or t.stride(-1) != 1 or t.dtype != p0.dtype):
            raise ValueError("gated_scan: the inputs are [tokens, width] column views of one dtype")
    out = torch.empty((tokens, width), dtype=p0.dtype, device=p0.device)
    check(lib().b2l_gated_scan(out.data_ptr(), out.stride(0), state.data_ptr(), p0.data_ptr(), p0.stride(0),
                               p1.data_ptr(), p1.stride(0), p2.data_ptr(), p2.stride(0), ptr(p3),
                               p3.stride(0) if p3 is not None else 0, ptr(bias_r), ptr(bias_i), ptr(lam),
                               float(decay_scale), seq_start.data_ptr(), seq_ctx.data_ptr(), seq_slot.data_ptr(),
                               seq_ctx.numel(), width, GATED_SCAN_MODES[mode], float_code(p0, "p0"), stream_handle()))
    return out
