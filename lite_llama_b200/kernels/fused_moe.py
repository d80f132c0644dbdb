"""Fused MoE: top-k routed experts as grouped tcgen05 GEMMs
(reference: lite_llama/kernels/fused_moe.py:45-99 ``moe_align_block_size``, :352-438 ``fused_moe``;
router: lite_llama/models/qwen3_moe.py:85-100)."""

from __future__ import annotations

import torch

from ._common import check, dtype_code, float_code, index_width, lib, ptr, require_cuda, stream_handle

_KIND_F16, _KIND_FP8, _KIND_INT8 = 0, 1, 2


@torch.no_grad()
def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Sort token slots by expert and pad each expert's run to ``block_size``.

    Returns ``(sorted_token_ids, expert_ids, num_tokens_post_padded)`` with the reference's exact
    protocol: slot ids (``token*top_k + k``) stable-sorted by expert, sentinel ``num_slots`` in the
    padding, one expert id per row block, padded total on the device. One kernel, no host sync.
    """
    require_cuda(topk_ids)
    ids = topk_ids.reshape(-1)
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    ids = ids.contiguous()
    num_slots = ids.numel()
    max_padded = num_slots + num_experts * (block_size - 1)
    max_blocks = (max_padded + block_size - 1) // block_size
    dev = topk_ids.device
    sorted_ids = torch.empty(max_padded, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(max_blocks, dtype=torch.int32, device=dev)
    num_post = torch.empty(1, dtype=torch.int32, device=dev)
    check(
        lib().b2l_moe_align_block_size(
            ids.data_ptr(), index_width(ids, "topk_ids"), num_slots, int(block_size), int(num_experts),
            sorted_ids.data_ptr(), expert_ids.data_ptr(), num_post.data_ptr(), stream_handle(),
        )
    )
    return sorted_ids, expert_ids, num_post


def _quant_kind(weight: torch.Tensor, scale: torch.Tensor | None) -> int:
    if scale is None:
        return _KIND_F16
    if weight.dtype == torch.uint8:
        return _KIND_FP8
    if weight.dtype == torch.int8:
        return _KIND_INT8
    raise ValueError(f"quantised expert weights must be uint8 or int8, got {weight.dtype}")


def _block_size(num_tokens: int, top_k: int = 1, num_experts: int = 1) -> int:
    """Row-block of the grouped GEMM (= UMMA N): 16 / 32 / 64. The reference picks BLOCK_M from the token count
    alone (fused_moe.py:214-222); what a block holds is one expert's slots, so the choice here follows the expected
    slots per expert (tokens * top_k / experts): 32 decode tokens over 128 experts are ~2 slots per expert, and a
    16-row block halves the padded rows and lets two CTAs share an SM (csrc/moe_gemm.cu). The result does not
    depend on the block size (every slot is the same dot product)."""
    per_expert = num_tokens * top_k / max(1, num_experts)
    if num_tokens <= 16 or per_expert <= 8:
        return 16
    if num_tokens <= 64 or per_expert <= 24:
        return 32
    return 64


def _moe_gemm(a, w, c, scale, kind, topk_weights, sorted_ids, expert_ids, num_post, top_k, block, group_n, group_k):
    num_experts, n, k = w.shape
    if w.stride(-1) != 1 or a.stride(-1) != 1:
        raise ValueError("fused_moe: last dims must be contiguous")
    if w.stride(0) != n * w.stride(1):
        w = w.contiguous()
    se = sn = sk = 0
    if scale is not None:
        if scale.dtype != torch.float32:
            scale = scale.float()
        se, sn, sk = scale.stride()
    check(
        lib().b2l_moe_gemm(
            c.data_ptr(), a.data_ptr(), w.data_ptr(), kind, ptr(scale), ptr(topk_weights), sorted_ids.data_ptr(),
            expert_ids.data_ptr(), num_post.data_ptr(), sorted_ids.numel(), c.shape[0], int(top_k), int(block),
            num_experts, n, k, a.stride(0), w.stride(1), c.stride(0), int(group_n or 1), int(group_k or k),
            se, sn, sk, stream_handle(),
        )
    )


@torch.no_grad()
def fused_moe(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    *,
    w1_scale: torch.Tensor | None = None,
    w2_scale: torch.Tensor | None = None,
    group_n: int = 0,
    group_k: int = 0,
) -> torch.Tensor:
    """``sum_k w_k * (silu(x @ W1g.T) * (x @ W1u.T)) @ W2.T`` over the routed experts.

    Same arguments, rounding points (gate_up, activation and the per-slot down output are rounded to
    fp16; the routing weight multiplies in fp32 before that cast; the top-k sum accumulates in fp32)
    and errors as the reference.
    """
    require_cuda(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale)
    if hidden_states.dtype != torch.float16:
        raise ValueError(f"fused_moe activations must be fp16, got {hidden_states.dtype}")
    num_tokens, hidden = hidden_states.shape
    num_experts, two_inter, _ = w1.shape
    intermediate = two_inter // 2
    top_k = topk_ids.shape[1]
    device, dtype = hidden_states.device, hidden_states.dtype
    kind = _quant_kind(w1, w1_scale)
    if kind != _quant_kind(w2, w2_scale):
        raise ValueError("w1 and w2 must use the same quantisation format")
    # the reference asks for multiples of 128 (fused_moe.py:391-394); this kernel closes an accumulator segment every
    # group_k elements and takes any multiple of 16, which is what sub-block tensor-parallel shards need (TP = 4 of
    # Qwen3-30B-A3B: 192 columns per rank -> 64-wide scale groups)
    if kind and group_k % 16 != 0 and group_k < min(hidden, intermediate):
        raise ValueError(f"group_k ({group_k}) must be a multiple of 16 unless it covers K")
    if kind == _KIND_F16 and w1.dtype != dtype:
        raise ValueError("fp16 expert weights must match the activation dtype")
    x = hidden_states if hidden_states.stride(-1) == 1 and hidden_states.stride(0) % 8 == 0 else hidden_states.contiguous()
    flat_weights = topk_weights.reshape(-1).to(dtype).contiguous()
    block = _block_size(num_tokens, top_k, num_experts)
    sorted_ids, expert_ids, num_post = moe_align_block_size(topk_ids, block, num_experts)

    gate_up = torch.empty((num_tokens * top_k, two_inter), device=device, dtype=dtype)
    _moe_gemm(x, w1, gate_up, w1_scale, kind, None, sorted_ids, expert_ids, num_post, top_k, block, group_n, group_k)

    act = torch.empty((num_tokens * top_k, intermediate), device=device, dtype=dtype)
    check(
        lib().b2l_swiglu(
            act.data_ptr(), gate_up.data_ptr(), gate_up[:, intermediate:].data_ptr(), num_tokens * top_k, intermediate,
            gate_up.stride(0), gate_up.stride(0), act.stride(0), dtype_code(act, "act"), stream_handle(),
        )
    )

    expanded = torch.empty((num_tokens * top_k, hidden), device=device, dtype=dtype)
    _moe_gemm(act, w2, expanded, w2_scale, kind, flat_weights, sorted_ids, expert_ids, num_post, 1, block, group_n,
              group_k)

    out = torch.empty((num_tokens, hidden), device=device, dtype=dtype)
    check(lib().b2l_moe_sum(out.data_ptr(), expanded.data_ptr(), None, num_tokens, hidden, top_k,
                            dtype_code(out, "out"), stream_handle()))
    return out


@torch.no_grad()
def route_topk(router_logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """``(weights [T, k] in the logits dtype, ids [T, k] int64)``: fp32 softmax over all experts,
    top-k, optional renormalisation (lite_llama/models/qwen3_moe.py:94-100), one kernel."""
    require_cuda(router_logits)
    if router_logits.stride(-1) != 1:
        router_logits = router_logits.contiguous()
    tokens, num_experts = router_logits.shape
    w = torch.empty((tokens, top_k), dtype=router_logits.dtype, device=router_logits.device)
    ids = torch.empty((tokens, top_k), dtype=torch.int64, device=router_logits.device)
    check(
        lib().b2l_moe_route_topk(
            w.data_ptr(), ids.data_ptr(), router_logits.data_ptr(), router_logits.stride(0), tokens, num_experts,
            int(top_k), 1 if renormalize else 0, dtype_code(router_logits, "router_logits"), stream_handle(),
        )
    )
    return w, ids


@torch.no_grad()
def route_sigmoid_groups(x: torch.Tensor, router_w: torch.Tensor, bias: torch.Tensor | None, top_k: int,
                         groups: int = 1, keep: int = 1, renormalize: bool = True):
    """Sigmoid router with a selection bias and group-limited choice (router product with fp32 results + one selection
    launch; a single launch for shapes no GEMM takes):
    ``s = sigmoid(router_w @ x)`` in fp32; experts compete with ``s + bias``; they form ``groups`` runs of neighbours,
    a group scores the sum of its two best, only the ``keep`` best groups are eligible; the ``top_k`` winners' weights
    are their ``s`` over the winners' sum (``renormalize=False``: their ``s`` as they are).  Returns ``(weights fp32 [T, k], ids int32 [T, k])``.  The reference's
    router is a softmax over all experts (lite_llama/models/qwen3_moe.py:94-100, ``route_topk``)."""
    require_cuda(x, router_w, bias)
    if x.stride(-1) != 1:
        x = x.contiguous()
    if router_w.dtype != x.dtype or (bias is not None and bias.dtype != x.dtype):
        raise ValueError("route_sigmoid_groups: router weight and bias must be in the activation dtype")
    tokens, k = x.shape
    e = router_w.shape[0]
    router_w = router_w.contiguous()
    w = torch.empty((tokens, top_k), dtype=torch.float32, device=x.device)
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device=x.device)
    L, code = lib(), float_code(x, "x")
    # the router product as a GEMM with fp32 results where one fits (tensor cores for aligned 16-bit operands, the
    # CUDA-core GEMM for true fp32); otherwise the selection kernel does the product itself
    logits = None
    if x.dtype == torch.float32:
        from .linear import linear_simt

        logits = linear_simt(x, router_w)
    elif L.b2l_rows_gemm_mma_ok(x.data_ptr(), router_w.data_ptr(), k, x.stride(0), 0, code):
        logits = torch.empty((tokens, e), dtype=torch.float32, device=x.device)
        check(L.b2l_linear_f32out_mma(logits.data_ptr(), x.data_ptr(), router_w.data_ptr(), tokens, e, k, x.stride(0), e,
                                      code, stream_handle()))
    check(L.b2l_moe_route_sigmoid_groups(w.data_ptr(), ids.data_ptr(), x.data_ptr(), x.stride(0), router_w.data_ptr(),
                                         ptr(bias), ptr(logits), tokens, e, k, int(top_k), int(groups), int(keep), 1 if renormalize else 0, code,
                                         stream_handle()))
    return w, ids


def _swiglu_into(mid: torch.Tensor, wide: torch.Tensor, ff: int, in_scale: torch.Tensor | None) -> None:
    """``mid = silu(s * wide[:, :ff]) * (s * wide[:, ff:])`` with the per-slot fp32 factor ``s`` (optional)."""
    check(lib().b2l_swiglu_scaled(mid.data_ptr(), mid.stride(0), wide.data_ptr(), wide.stride(0), wide[:, ff:].data_ptr(),
                                  wide.stride(0), ptr(in_scale), None, 0, mid.shape[0], ff, float_code(mid, "mid"),
                                  stream_handle()))


@torch.no_grad()
def grouped_experts(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, weights: torch.Tensor,
                    ids: torch.Tensor, addend: torch.Tensor | None = None, activation: str = "gelu",
                    gated: bool = False, weight_on_input: bool = False) -> torch.Tensor:
    """``sum_k weights[t, k] * W_down[e] act(W_up[e] x[t]) (+ addend[t])`` over each token's chosen experts
    ``e = ids[t, k]``: ungated two-matrix experts, ``w_up [E, ff, h]``, ``w_down [E, h, ff]``.  Slots are sorted by
    expert (``moe_align_block_size``), both products run grouped (``mma.sync`` tiles for aligned 16-bit operands, the
    CUDA cores for true fp32 and odd shapes) with the activation in the first one's epilogue and the fp32 routing weight
    in the second's.  ``gated`` (``activation="silu"``): ``w_up [E, 2 * ff, h]`` holds every expert's gate rows then its
    up rows, and the unit is ``W_down (silu(W_gate x) * W_up x)``; the activation is a kernel of its own between the
    products.  ``weight_on_input``: the expert sees ``weights[t, k] * x[t]`` and its output is not weighted; the factor
    passes through the first (linear) product and is applied to its fp32-widened results.  The fp16 / fp8 gated experts
    of the reference's family are ``fused_moe``."""
    require_cuda(x, w_up, w_down, weights, ids, addend)
    if (activation, gated) not in (("gelu", False), ("silu", True)) or (weight_on_input and not gated):
        raise ValueError(f"grouped_experts: unknown expert form {activation!r}, gated={gated}")
    if weights.dtype != torch.float32:
        raise ValueError("grouped_experts: routing weights are fp32")
    tokens, hidden = x.shape
    num_experts, up_rows, _ = w_up.shape
    ff = up_rows // 2 if gated else up_rows
    top_k = ids.shape[1]
    L = lib()
    code = float_code(x, "x")
    if x.stride(-1) != 1:
        x = x.contiguous()
    w_up, w_down = w_up.contiguous(), w_down.contiguous()
    slots = tokens * top_k
    mid = torch.empty((slots, ff), dtype=x.dtype, device=x.device)
    wide = torch.empty((slots, up_rows), dtype=x.dtype, device=x.device) if gated else mid
    expanded = torch.empty((slots, hidden), dtype=x.dtype, device=x.device)
    flat_w = weights.reshape(-1).contiguous()
    down_w = None if weight_on_input else flat_w.data_ptr()
    act = 0 if gated else 1
    # 16-bit operands with 16-byte aligned rows run on the tensor cores (blocks of 16, 64 or 128 slots by the expected
    # slots per expert), everything else on the CUDA cores; the result of a slot does not depend on the block size
    tensor = bool(L.b2l_rows_gemm_mma_ok(x.data_ptr(), w_up.data_ptr(), hidden, x.stride(0), 0, code)) and \
        bool(L.b2l_rows_gemm_mma_ok(mid.data_ptr(), w_down.data_ptr(), ff, mid.stride(0), 0, code))
    per_expert = slots / num_experts
    block = (16 if per_expert <= 16 else (64 if per_expert <= 256 else 128)) if tensor else L.b2l_moe_gemm_simt_block()
    sorted_ids, expert_ids, num_post = moe_align_block_size(ids, block, num_experts)
    common = (sorted_ids.data_ptr(), expert_ids.data_ptr(), num_post.data_ptr(), sorted_ids.numel(), slots)

    def between() -> None:
        if gated:
            _swiglu_into(mid, wide, ff, flat_w if weight_on_input else None)

    if tensor:
        check(L.b2l_moe_gemm_mma(wide.data_ptr(), x.data_ptr(), w_up.data_ptr(), None, *common, top_k, block, up_rows,
                                 hidden, x.stride(0), wide.stride(0), act, code, stream_handle()))
        between()
        check(L.b2l_moe_gemm_mma(expanded.data_ptr(), mid.data_ptr(), w_down.data_ptr(), down_w, *common, 1,
                                 block, hidden, ff, mid.stride(0), expanded.stride(0), 0, code, stream_handle()))
    else:
        check(L.b2l_moe_gemm_simt(wide.data_ptr(), x.data_ptr(), w_up.data_ptr(), None, *common, top_k, up_rows, hidden,
                                  x.stride(0), wide.stride(0), act, code, stream_handle()))
        between()
        check(L.b2l_moe_gemm_simt(expanded.data_ptr(), mid.data_ptr(), w_down.data_ptr(), down_w, *common, 1,
                                  hidden, ff, mid.stride(0), expanded.stride(0), 0, code, stream_handle()))
    out = torch.empty((tokens, hidden), dtype=x.dtype, device=x.device)
    check(L.b2l_moe_sum(out.data_ptr(), expanded.data_ptr(), ptr(addend), tokens, hidden, top_k, code, stream_handle()))
    return out
