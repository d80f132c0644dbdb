"""Decoder for layer-list models: each layer = one mixer (looked up in ``MIXERS`` by the layer's kind) + an optional
feed-forward (``FEED_FORWARDS``), around an fp32 residual stream with the norm on the sublayer OUTPUT:

    x <- x + norm(mixer(x));   x <- x + norm(ff(x))          (the sublayers read x itself)

or, for designs with ``pre_norm`` (and ``layer_scale``), norms on both sides of each sublayer:

    x <- x + s1 * norm_b(mixer(norm_a(x)));   x <- x + s2 * norm_d(ff(norm_c(x)))

where the output norm, the residual sum and the NEXT sublayer's input norm are one kernel (``post_norm_residual``).

The forward is a flat op list over the library's kernels, like ``executor.decoder.Decoder`` is for the uniform
rotary decoders (reference: lite_llama/models/base.py:299-319,447-489), but over a RAGGED step (``RaggedBatch``):
prompt portions and single decode tokens of different requests in one flat ``[tokens, hidden]`` batch.  Projections
run in the activation dtype (bf16 / fp16 on tcgen05, or TRUE fp32 on the CUDA cores); norms, softmax, the residual
sum, decays, step sizes and the recurrent state are fp32 in every mode.

Designs registered here:
  * ``Gufotar``: learned absolute positions, Mamba-2 style state-space layers and position-free attention layers
    (whole-row q/k norm, log-position query gain, tanh soft cap, per-head softmax sink, cross-layer value mixing),
    squared-ReLU feed-forward, zero-centred norm weights.
  * ``Pesivik``: scaled embedding, layer norms (weight, no bias) before and after every sublayer with a per-channel
    layer scale, latent attention (low-rank query and key/value latents, a shared rotated key part, sliding window,
    per-head sigmoid output gate), routed experts (sigmoid router with selection bias and group-limited choice, exact
    GELU, a shared expert), layers that share another layer's weights, soft-capped logits.
  * ``Tisosun``: normed embedding; PARALLEL blocks ``x <- x + mixer(norm1(x)) + ff(norm2(x))`` with a gated feed-forward,
    a gated low-rank per-layer token input after the block, and a learned depth-weighted average of all layer results
    in front of every layer and of the output; mixers: a minimal GRU, a real-gated linear recurrent unit behind a
    short convolution, and softmax attention (biased projections, per-head q / k norm, neighbour-paired rotary
    positions with frequency interpolation by parts, soft cap, block-diagonal causal mask) side by side with decayed
    linear attention.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..kernels import (
    attn_prepare,
    branch_sum_residual,
    causal_conv_silu,
    decay_attention,
    depth_mix_norms,
    embed_positions,
    embed_rmsnorm,
    gated_group_norm,
    gated_linear_scan,
    gated_scan,
    gelu,
    gelu_mul_gather,
    grouped_experts,
    head_linear,
    head_mix,
    head_norm_gate,
    head_norm_rope_prepare,
    latent_prepare,
    linear,
    norm_sigmoid_gate,
    post_norm_residual,
    relu_squared,
    rmsnorm_from_f32,
    rope_heads,
    rope_table,
    rope_table_freqs,
    rotary_frequencies,
    route_sigmoid_groups,
    sink_attention,
    mixed_head_attention,
    MIXED_HEAD_MAX_KEYS,
    softcap_to_f32,
    ssm_scan,
    swiglu_forward,
    swiglu_scaled,
)
from .model_config import (BlockAttentionSpec, ConvWindowAttentionSpec, DecayAttentionSpec, DeltaRuleSpec, DenseMlpSpec,
                           ForgetGateAttentionSpec, LatentAttentionSpec, LayeredConfig, LayerSpec, Mamba2Spec,
                           MinGruSpec, MoeMlpSpec, RgLruSpec, SideBySideSpec, SinkAttentionSpec, WindowDeltaPairSpec)
from .ragged_batch import RaggedBatch
from .registry import Architecture, register


# ------------------------------------------------------------------------------------------------------ weights #
@dataclass
class LayeredLayerWeights:
    norm1: torch.Tensor                                  # norm on the mixer's OUTPUT
    mix: dict[str, torch.Tensor]
    norm2: torch.Tensor | None = None                    # norm on the feed-forward's output
    mlp: dict[str, torch.Tensor] | None = None
    pre1: torch.Tensor | None = None                     # input norms and layer scales of pre-norm designs
    pre2: torch.Tensor | None = None
    ls1: torch.Tensor | None = None
    ls2: torch.Tensor | None = None
    side: dict[str, torch.Tensor] | None = None          # per-layer token input: gate, proj, norm
    depth: torch.Tensor | None = None                    # depth-average coefficients over [embedding, layer results]


@dataclass
class LayeredWeights:
    embed: torch.Tensor
    pos: torch.Tensor | None
    final_norm: torch.Tensor
    head: torch.Tensor
    layers: list[LayeredLayerWeights] = field(default_factory=list)
    embed_norm: torch.Tensor | None = None
    side_embed: torch.Tensor | None = None               # [vocab, layers * token_side_dim]

    def nbytes_per_step(self) -> int:
        """Weight bytes one step streams (embedding / position gathers excluded)."""
        total = self.head.numel() * self.head.element_size()
        seen = set()
        for lw in self.layers:
            if id(lw) in seen:                           # a layer that shares another one's weights
                continue
            seen.add(id(lw))
            for d in (lw.mix, lw.mlp or {}, lw.side or {}):
                total += sum(t.numel() * t.element_size() for t in d.values())
        return total


# ------------------------------------------------------------------------------------------------------- mixers #
class StepContext:
    """What the mixers of one forward share: the step's metadata, the caches, and values one layer hands to later
    ones (the first value-mixing layer's values)."""

    def __init__(self, batch: RaggedBatch, kv_buffer: dict[int, torch.Tensor], table: torch.Tensor, states) -> None:
        self.batch = batch
        self.kv_buffer = kv_buffer
        self.table = table
        self.states = states
        self.v_first: torch.Tensor | None = None
        self._rope: dict[tuple, torch.Tensor | None] = {}

    def rope(self, rot_dims: int, rot_base: float) -> torch.Tensor | None:
        """The step's [cos | sin] table for these rotary constants, built once and shared by the layers."""
        key = (rot_dims, rot_base)
        if key not in self._rope:
            self._rope[key] = rope_table(self.batch.positions, rot_dims, rot_base)
        return self._rope[key]

    def rope_freqs(self, freqs: torch.Tensor, magnitude: float) -> torch.Tensor:
        """The step's magnitude * [cos | sin] table for a frequency vector (one per rotary configuration; layers with
        equal constants share the tensor and so the table)."""
        key = (freqs.data_ptr(), magnitude)
        if key not in self._rope:
            self._rope[key] = rope_table_freqs(self.batch.positions, freqs, magnitude)
        return self._rope[key]


@dataclass
class Branches:
    """A mixer's output as up to two branches that the residual kernel norms (plain weights; none: the branch as it
    is) and sums: ``scale * unit_rms(a) * a_weight + scale_b * unit_rms(b) * b_weight``."""

    a: torch.Tensor
    a_weight: torch.Tensor | None
    b: torch.Tensor | None = None
    b_weight: torch.Tensor | None = None
    scale: float = 1.0
    scale_b: float | None = None                       # the second branch's own factor (default: ``scale``)


def mamba2_mixer(li: int, spec: Mamba2Spec, w: dict[str, torch.Tensor], x: torch.Tensor, ctx: StepContext,
                 eps: float) -> torch.Tensor:
    """in-projection -> [z | x B C | dt]; short causal convolution + SiLU on x B C (tail kept per slot); fp32 scan
    against the slot's state; gate, grouped unit-RMS norm, out-projection."""
    b = ctx.batch
    proj = linear(x, w["in"])
    inner = spec.inner
    xbc = causal_conv_silu(proj, inner, spec.conv_channels, w["conv"], w["conv_b"], ctx.states.conv_tail[li],
                           b.seq_start, b.seq_ctx, b.seq_slot)
    dt_raw = proj[:, inner + spec.conv_channels:]
    y = ssm_scan(xbc, dt_raw, w["dt_bias"], w["A_log"], w["D"], ctx.states.ssm_state[li], b.seq_start, b.seq_ctx,
                 b.seq_slot, spec.heads, spec.groups, spec.state, spec.head_dim)
    gated = gated_group_norm(y, proj[:, :inner], w["norm"], spec.norm_groups, eps)
    return linear(gated, w["o"])


_SPLIT_KEYS = 128          # keys per CTA of the single-token attention kernel (4 warps x 32 keys per pass)
_MAX_SPLITS = 128


def sink_attention_mixer(li: int, spec: SinkAttentionSpec, w: dict[str, torch.Tensor], x: torch.Tensor,
                         ctx: StepContext, eps: float) -> torch.Tensor:
    """fused q|k|v projection -> per-token preparation (norms, query gain, value mixing, cache write) -> attention
    over the pool: the tiled kernel for prompt portions, the key-split kernel for single tokens."""
    b = ctx.batch
    qn, kn, vn = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.v_head_dim
    qkv = linear(x, w["qkv"])
    pool = ctx.kv_buffer[li]
    v_in = v_out = None
    if spec.v_mix:
        if ctx.v_first is None:
            ctx.v_first = v_out = torch.empty((b.tokens, vn), dtype=qkv.dtype, device=qkv.device)
        else:
            v_in = ctx.v_first
    attn_prepare(qkv, pool, b.kv_rows, b.positions, qn, kn, vn, w.get("q_norm"), w.get("k_norm"), eps,
                 spec.gain_coef, spec.gain_every, v_in, v_out, w.get("vmix") if v_in is not None else None)
    out = torch.empty((b.tokens, spec.heads * spec.v_head_dim), dtype=qkv.dtype, device=qkv.device)
    common = (spec.heads, spec.kv_heads, spec.head_dim, spec.v_head_dim, spec.scale, spec.softcap)
    if b.num_portions:
        sink_attention(out, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.portion_list, b.num_portions,
                       b.max_portion, w.get("sink"), *common)
    if b.num_singles:
        splits, per = split_plan(b.max_single_ctx + 1)
        sink_attention(out, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.single_list, b.num_singles, 1,
                       w.get("sink"), *common, num_splits=splits, split_keys=per)
    return linear(out, w["o"])


def split_plan(keys: int) -> tuple[int, int]:
    """(ranges, keys per range) of the single-token attention kernel for a token that sees ``keys`` keys."""
    splits = max(1, min(_MAX_SPLITS, -(-keys // _SPLIT_KEYS)))
    per = -(-keys // splits)
    return splits, -(-per // 32) * 32


def latent_attention_mixer(li: int, spec: LatentAttentionSpec, w: dict[str, torch.Tensor], x: torch.Tensor,
                           ctx: StepContext, eps: float) -> torch.Tensor:
    """One fused down-projection [query latent | key/value latent | shared rotated key part | head gates] -> latent
    norms, rotation and the cache write (``latent_prepare``) -> query up-projection -> the queries' unrotated parts
    multiplied into the latent space per head (``W_uk^T q``), their rotated parts turned by the position -> attention
    over the cached rows [latent | rotated key part] as ONE key/value head whose values are the latent itself (sliding
    window) -> per-head value up-projection with the sigmoid gate in its epilogue -> output projection.  Equal to
    expanding per-head keys and values from the latent for every cached token, without doing so."""
    b = ctx.batch
    H, dim, rot, rank = spec.heads, spec.head_dim, spec.rot_dim, spec.kv_rank
    proj = linear(x, w["down"])
    pool = ctx.kv_buffer[li]
    cos_sin = ctx.rope(spec.rot_dims, spec.rot_base)
    latent_prepare(proj, pool, b.kv_rows, cos_sin, w["q_norm"], w["kv_norm"], spec.q_rank, rank, rot, spec.rot_dims, eps)
    q = linear(proj[:, :spec.q_rank], w["uq"])
    D = rank + rot
    qa = torch.empty((b.tokens, H * D), dtype=q.dtype, device=q.device)
    head_linear(qa, D, q, dim + rot, w["uk_t"])
    if rot:
        rope_heads(qa[:, rank:], D, q[:, dim:], dim + rot, cos_sin, H, rot, spec.rot_dims)
    lat = torch.empty((b.tokens, H * rank), dtype=q.dtype, device=q.device)
    common = (H, 1, D, rank, spec.scale, 0.0)
    if b.num_portions:
        sink_attention(lat, qa, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.portion_list, b.num_portions,
                       b.max_portion, None, *common, window=spec.window, v_col0=0)
    if b.num_singles:
        keys = b.max_single_ctx + 1
        splits, per = split_plan(min(keys, spec.window) if spec.window else keys)
        sink_attention(lat, qa, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.single_list, b.num_singles, 1,
                       None, *common, num_splits=splits, split_keys=per, window=spec.window, v_col0=0)
    out = torch.empty((b.tokens, H * spec.v_head_dim), dtype=q.dtype, device=q.device)
    gate = proj[:, spec.q_rank + rank + rot:] if spec.out_gate else None
    head_linear(out, spec.v_head_dim, lat, rank, w["uv"], gate)
    return linear(out, w["o"])


def min_gru_mixer(li: int, spec: MinGruSpec, w: dict[str, torch.Tensor], x: torch.Tensor, ctx: StepContext,
                  eps: float) -> torch.Tensor:
    """One biased projection [update gate | candidate | output gate] -> the element-wise recurrence against the slot's
    fp32 state (gates in fp32, output gate fused) -> out-projection."""
    b, n = ctx.batch, spec.width
    proj = linear(x, w["in"], w["in_b"])
    y = gated_scan("mingru", ctx.states.ssm_state[li], proj[:, :n], proj[:, n:2 * n], proj[:, 2 * n:3 * n], b.seq_start,
                   b.seq_ctx, b.seq_slot)
    return linear(y, w["o"])


def rg_lru_mixer(li: int, spec: RgLruSpec, w: dict[str, torch.Tensor], x: torch.Tensor, ctx: StepContext,
                 eps: float) -> torch.Tensor:
    """One biased projection [GELU branch | recurrence branch] -> causal convolution of the recurrence branch (tail
    kept per slot) -> the two block-diagonal gate projections -> the recurrence (biases, sigmoids, decay, input
    scaling, GELU of the other branch and the product in one kernel, fp32) -> out-projection."""
    b, n = ctx.batch, spec.width
    per = n // spec.blocks
    proj = linear(x, w["in"], w["in_b"])
    u = causal_conv_silu(proj, n, n, w["conv"], w["conv_b"], ctx.states.conv_tail[li], b.seq_start, b.seq_ctx,
                         b.seq_slot, activation=False)
    gates = torch.empty((b.tokens, 2 * n), dtype=u.dtype, device=u.device)
    head_linear(gates[:, :n], per, u, per, w["ra"])
    head_linear(gates[:, n:], per, u, per, w["ri"])
    y = gated_scan("rglru", ctx.states.ssm_state[li], u, gates[:, :n], gates[:, n:], b.seq_start, b.seq_ctx, b.seq_slot,
                   p3=proj[:, :n], bias_r=w["ra_b"], bias_i=w["ri_b"], lam=w["lam"], decay_scale=spec.decay_scale)
    return linear(y, w["o"])


def side_by_side_mixer(li: int, spec: SideBySideSpec, w: dict[str, torch.Tensor], x: torch.Tensor, ctx: StepContext,
                       eps: float) -> Branches:
    """ONE projection for both halves, [q | k | v (biased) | pad || v' | k' | q' | gate'].  Left: per-head norms,
    rotation and the cache write in one kernel, attention over the pool under the block-diagonal mask, out-projection.
    Right: decayed linear attention against the slot's fp32 memory (SiLU applied as the kernel reads its inputs; chunks
    on the tensor cores for prompt portions, the token-by-token scan otherwise), row norm and sigmoid gate,
    out-projection.  The two outputs go to the residual kernel as branches."""
    b, L, R = ctx.batch, spec.left, spec.right
    proj = linear(x, w["in"], w["in_b"])
    # ---- left: softmax attention over the pool
    pool = ctx.kv_buffer[li]
    cos_sin = ctx.rope_freqs(w["freqs"], spec_magnitude(L)) if L.rot_dims else None
    head_norm_rope_prepare(proj, pool, b.kv_rows, cos_sin, w.get("q_norm"), w.get("k_norm"), L.heads, L.kv_heads,
                           L.head_dim, L.v_head_dim, L.rot_dims, eps, L.pairing)
    att = torch.empty((b.tokens, L.heads * L.v_head_dim), dtype=proj.dtype, device=proj.device)
    common = (L.heads, L.kv_heads, L.head_dim, L.v_head_dim, L.scale, L.softcap)
    if b.num_portions:
        sink_attention(att, proj, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.portion_list, b.num_portions,
                       b.max_portion, None, *common, block=L.block)
    if b.num_singles:
        keys = b.max_single_ctx + 1
        splits, per = split_plan(min(keys, L.block) if L.block else keys)
        sink_attention(att, proj, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.single_list, b.num_singles, 1,
                       None, *common, num_splits=splits, split_keys=per, block=L.block)
    left = linear(att, w["left_o"])
    # ---- right: decayed linear attention over the slot's memory
    r0 = -(-(L.heads * L.head_dim + L.kv_heads * (L.head_dim + L.v_head_dim)) // 8) * 8     # padded attention half
    inner = R.heads * R.v_head_dim
    xbc = proj[:, r0:r0 + inner + 2 * R.heads * R.head_dim]
    y = decay_attention(xbc, ctx.states.ssm_state[li], w["decay"], b.seq_start, b.seq_ctx, b.seq_slot, R.heads,
                        R.head_dim, R.v_head_dim, max(b.max_portion, 1))
    gate = proj[:, r0 + inner + 2 * R.heads * R.head_dim:r0 + 2 * inner + 2 * R.heads * R.head_dim]
    right = linear(norm_sigmoid_gate(y, gate, w["right_norm"], eps), w["right_o"])
    return Branches(left, w["left_out"], right, w["right_out"], 0.5)


def forget_gate_mixer(li: int, spec: ForgetGateAttentionSpec, w: dict[str, torch.Tensor], x: torch.Tensor,
                      ctx: StepContext, eps: float) -> torch.Tensor:
    """ONE projection [q | forget-gate logits (biased) | v] -> the recurrence against the slot's fp32 memory (SiLU of q,
    the bounded forget gate and its complement evaluated in fp32 inside the kernel) -> per-head RMS norm ->
    out-projection."""
    b, n = ctx.batch, spec.heads * spec.head_dim
    proj = linear(x, w["in"], w["in_b"])
    y = gated_linear_scan("forget_gate", ctx.states.ssm_state[li], proj[:, :n], proj[:, n:2 * n], proj[:, 2 * n:],
                          b.seq_start, b.seq_ctx, b.seq_slot, spec.heads, spec.heads, spec.head_dim, spec.v_head_dim,
                          c0=w["lower"])
    return linear(head_norm_gate(y, w["norm"], spec.heads, eps), w["o"])


def wide_value_heads(spec: ConvWindowAttentionSpec, tensor_tiles: bool) -> int:
    """How many kv heads' values one attention call reads side by side as one wide value head when the softmax
    weights are mixed across heads: the most that divide ``kv_heads`` and stay inside the kernels' value width (128
    columns on the tensor-core tiles that serve 16-bit prompt portions, 256 on the CUDA-core kernels that serve fp32
    and single tokens)."""
    limit = 128 if tensor_tiles and spec.head_dim % 8 == 0 and spec.v_head_dim % 8 == 0 and spec.head_dim <= 128 else 256
    best = 1
    for c in range(1, spec.kv_heads + 1):
        if spec.kv_heads % c == 0 and c * spec.v_head_dim <= limit:
            best = c
    return best


def conv_window_attention(li: int, spec: ConvWindowAttentionSpec, w: dict[str, torch.Tensor], proj: torch.Tensor,
                          ctx: StepContext, eps: float) -> torch.Tensor:
    """The attention half of ``window_delta_mixer`` from the fused projection's leading columns [q | k | v]: the short
    convolution (tail per slot), unit-RMS of q and k per head and the cache write, attention under the window, the
    head mix.  Mixing the heads' softmax weights is linear in the weights.  For prompt portions it is done on OUTPUTS:
    every query head's weights are applied to the values of every kv head (the value heads of a pool row read side by
    side as one wide head, ``v_head_stride = 0``), and ``head_mix`` forms ``sum_g M[h, g] * out[g, kv(h)]``, so the
    tiled softmax kernels stay as they are.  For single tokens the normalised weights of a token are small
    (``heads x keys``): ``mixed_head_attention`` writes them, mixes them and reads each head's own values once."""
    b, L = ctx.batch, spec
    H, G, D, Dv = L.heads, L.kv_heads, L.head_dim, L.v_head_dim
    pool = ctx.kv_buffer[li]
    qkv = causal_conv_silu(proj, 0, L.channels, w["left_conv"], w["left_conv_b"], ctx.states.named_tail[li]["left"],
                           b.seq_start, b.seq_ctx, b.seq_slot, activation=False)
    ones = w["ones"] if L.qk_unit_rms else None
    head_norm_rope_prepare(qkv, pool, b.kv_rows, None, ones, ones, H, G, D, Dv, 0, eps)
    if not L.head_mix:
        att = torch.empty((b.tokens, H * Dv), dtype=qkv.dtype, device=qkv.device)
        common = (H, G, D, Dv, L.scale, 0.0)
        if b.num_portions:
            sink_attention(att, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.portion_list, b.num_portions,
                           b.max_portion, None, *common, window=L.window)
        if b.num_singles:
            keys = b.max_single_ctx + 1
            splits, per = split_plan(min(keys, L.window) if L.window else keys)
            sink_attention(att, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.single_list, b.num_singles,
                           1, None, *common, num_splits=splits, split_keys=per, window=L.window)
        return linear(att, w["left_o"])
    keys = min(b.max_single_ctx + 1, L.window) if L.window else b.max_single_ctx + 1
    direct = b.num_singles > 0 and keys <= MIXED_HEAD_MAX_KEYS     # single tokens: the WEIGHTS are mixed, two launches
    att = None
    if b.num_portions or (b.num_singles and not direct):
        per_call = wide_value_heads(L, qkv.dtype != torch.float32 and b.num_portions > 0)
        calls, width = G // per_call, per_call * Dv
        wide = torch.empty((b.tokens, calls * H * width), dtype=qkv.dtype, device=qkv.device)
        common = (H, G, D, width, L.scale, 0.0)
        for c in range(calls if b.num_portions else 0):
            sink_attention(wide[:, c * H * width:(c + 1) * H * width], qkv, pool, ctx.table, b.seq_start, b.seq_ctx,
                           b.seq_slot, b.portion_list, b.num_portions, b.max_portion, None, *common, window=L.window,
                           v_col0=G * D + c * width, v_head_stride=0)
        if b.num_singles and not direct:                 # every block of value columns in the same two launches
            splits, per = split_plan(keys)
            sink_attention(wide, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.single_list, b.num_singles,
                           1, None, *common, num_splits=splits, split_keys=per, window=L.window, v_col0=G * D,
                           v_head_stride=0, v_blocks=calls)
        att = head_mix(wide, w["talk"], H, G, per_call, Dv)      # rows of tokens no call wrote are overwritten below
    if direct:
        if att is None:
            att = torch.empty((b.tokens, H * Dv), dtype=qkv.dtype, device=qkv.device)
        mixed_head_attention(att, qkv, pool, ctx.table, b.seq_start, b.seq_ctx, b.seq_slot, b.single_list, b.num_singles,
                             w["talk"], H, G, D, Dv, L.scale, 0.0, keys, window=L.window)
    return linear(att, w["left_o"])


def window_delta_mixer(li: int, spec: WindowDeltaPairSpec, w: dict[str, torch.Tensor], x: torch.Tensor,
                       ctx: StepContext, eps: float) -> Branches:
    """ONE projection for both halves, [q | k | v (biased) | pad || q' | k' | v' | write logits | decay logits | pad ||
    gate'].  Left: ``conv_window_attention``.  Right: convolution + SiLU of q', k', v' (tail per slot), the gated delta
    rule against the slot's fp32 memory (unit norms, write strength and decay in fp32 inside the kernel), per-head RMS
    norm times the SiLU gate, out-projection.  The residual kernel scales and sums the two."""
    b, L, R = ctx.batch, spec.left, spec.right
    proj = linear(x, w["in"], w["in_b"])
    left = conv_window_attention(li, L, w, proj, ctx, eps)
    r0 = -(-L.channels // 8) * 8
    nqk, nv = R.qk_heads * R.head_dim, R.heads * R.v_head_dim
    qkv = causal_conv_silu(proj, r0, R.channels, w["right_conv"], w["right_conv_b"], ctx.states.named_tail[li]["right"],
                           b.seq_start, b.seq_ctx, b.seq_slot)
    p0 = r0 + R.channels
    g0 = r0 + -(-(R.channels + 2 * R.heads) // 8) * 8
    y = gated_linear_scan("delta_rule", ctx.states.ssm_state[li], qkv[:, :nqk], qkv[:, nqk:2 * nqk], qkv[:, 2 * nqk:],
                          b.seq_start, b.seq_ctx, b.seq_slot, R.heads, R.qk_heads, R.head_dim, R.v_head_dim,
                          c0=w["dt_bias"], c1=w["A_log"], p0=proj[:, p0:p0 + R.heads],
                          p1=proj[:, p0 + R.heads:p0 + 2 * R.heads], q_scale=R.head_dim ** -0.5, unit_eps=R.unit_eps)
    right = linear(head_norm_gate(y, w["right_norm"], R.heads, eps, proj[:, g0:g0 + nv]), w["right_o"])
    return Branches(left, None, right, None, spec.left_scale, spec.right_scale)


def spec_magnitude(spec: BlockAttentionSpec) -> float:
    return rotary_frequencies(spec.rot_dims, spec.rot_base, spec.rot_factor, spec.rot_original, spec.rot_fast,
                              spec.rot_slow)[1]


def _activate(kind: str, x: torch.Tensor) -> torch.Tensor:
    if kind == "relu2":
        return relu_squared(x)
    if kind == "gelu":
        return gelu(x)
    if kind == "gelu_tanh":
        return gelu(x, "tanh")
    raise ValueError(f"unknown feed-forward activation {kind!r}")


def dense_feed_forward(spec: DenseMlpSpec, w: dict[str, torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    if spec.gated:                                   # [gate | up] is one product; silu(gate) * up one kernel
        if spec.activation != "silu":
            raise ValueError(f"unknown gated feed-forward activation {spec.activation!r}")
        gu = linear(x, w["gate_up"])
        return linear(swiglu_forward(gu[:, :spec.ff], gu[:, spec.ff:]), w["down"])
    return linear(_activate(spec.activation, linear(x, w["up"])), w["down"])


def moe_feed_forward(spec: MoeMlpSpec, w: dict[str, torch.Tensor], x: torch.Tensor) -> torch.Tensor:
    """Router (product, sigmoid, bias, group-limited top-k: one launch) -> the shared expert as two dense products ->
    the routed experts as two grouped products; the shared expert's output joins the weighted sum in its kernel."""
    weights, ids = route_sigmoid_groups(x, w["router"], w.get("correction"), spec.top, spec.groups, spec.keep,
                                        renormalize=spec.renormalize)
    shared = None
    if spec.gated:
        # gated experts: [gate | up] stacked per expert; the shared expert's [gate | up | token-gate row] is one product
        if spec.shared_ff:
            f = spec.shared_ff
            gu = linear(x, w["shared_gate_up"])
            z = gu[:, 2 * f:2 * f + 1] if spec.shared_gate else None
            shared = linear(swiglu_scaled(gu[:, :f], gu[:, f:2 * f], None, z), w["shared_down"])
        return grouped_experts(x, w["gate_up"], w["down"], weights, ids, addend=shared, activation=spec.activation,
                               gated=True, weight_on_input=spec.weight_on_input)
    if spec.shared_ff:
        shared = linear(_activate(spec.activation, linear(x, w["shared_up"])), w["shared_down"])
    return grouped_experts(x, w["up"], w["down"], weights, ids, addend=shared, activation=spec.activation)


MIXERS = {"mamba2": mamba2_mixer, "attention": sink_attention_mixer, "latent_attention": latent_attention_mixer,
          "mingru": min_gru_mixer, "rglru": rg_lru_mixer, "parallel": side_by_side_mixer,
          "forget_gate": forget_gate_mixer, "window_delta": window_delta_mixer}
FEED_FORWARDS = {"dense": dense_feed_forward, "moe": moe_feed_forward}


class LayeredDecoder:
    def __init__(self, cfg: LayeredConfig, weights: LayeredWeights, device: str = "cuda",
                 dtype: torch.dtype = torch.bfloat16, norm_weight_offset: float | None = None) -> None:
        cfg.validate()
        self.cfg, self.w, self.device, self.dtype = cfg, weights, device, dtype
        self.norm_offset = cfg.norm_weight_offset if norm_weight_offset is None else norm_weight_offset
        self.layer_trace: list[torch.Tensor] | None = None       # set to [] to record the residual after every layer

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, batch: RaggedBatch, kv_buffer: dict[int, torch.Tensor],
                table: torch.Tensor, states, want_rows: torch.Tensor | None = None) -> torch.Tensor:
        """``tokens [T]`` int32 -> logits ``[T or len(want_rows), vocab]`` in the activation dtype (fp32 when the
        design soft-caps its logits)."""
        cfg, eps, off, kind = self.cfg, self.cfg.rms_norm_eps, self.norm_offset, self.cfg.norm_kind
        ctx = StepContext(batch, kv_buffer, table, states)
        if cfg.single_norm:
            return self._forward_single_norm(tokens, ctx, want_rows)
        if cfg.parallel_block:
            return self._forward_parallel(tokens, ctx, want_rows)
        pre = cfg.pre_norm
        resid, act = embed_positions(tokens, batch.positions, self.w.embed, self.w.pos, want_act=not pre,
                                     scale=cfg.embed_scale)
        if pre and cfg.layers:
            act = rmsnorm_from_f32(resid, self.w.layers[0].pre1, eps, off, None, kind)
        count = len(cfg.layers)
        for li, (spec, lw) in enumerate(zip(cfg.layers, self.w.layers)):
            x = resid if act is None else act
            y = MIXERS[spec.kind](li, spec.mixer, lw.mix, x, ctx, eps)
            # the norm the NEXT sublayer reads through (pre-norm designs): this layer's feed-forward, else the next layer
            after = self.w.layers[li + 1].pre1 if li + 1 < count else None
            nxt = (lw.pre2 if spec.mlp is not None else after) if pre else None
            act = post_norm_residual(resid, y, lw.norm1, eps, off, kind=kind, layer_scale=lw.ls1, next_weight=nxt,
                                     next_kind=kind, want_act=not pre or nxt is not None)
            if spec.mlp is not None:
                x = resid if act is None else act
                y = FEED_FORWARDS[spec.mlp.kind](spec.mlp, lw.mlp, x)
                nxt = after if pre else None
                act = post_norm_residual(resid, y, lw.norm2, eps, off, kind=kind, layer_scale=lw.ls2, next_weight=nxt,
                                         next_kind=kind, want_act=not pre or nxt is not None)
            if self.layer_trace is not None:
                self.layer_trace.append(resid.clone())
        if want_rows is not None and want_rows.numel() == 0:
            return torch.empty((0, cfg.vocab_size), dtype=torch.float32 if cfg.logit_softcap else self.dtype,
                               device=resid.device)
        return self._head(resid, want_rows)

    def _head(self, resid: torch.Tensor, want_rows: torch.Tensor | None) -> torch.Tensor:
        cfg = self.cfg
        hidden = rmsnorm_from_f32(resid, self.w.final_norm, cfg.rms_norm_eps, self.norm_offset, want_rows, cfg.norm_kind)
        logits = linear(hidden, self.w.head)
        if cfg.logit_softcap or cfg.logit_scale != 1.0:
            return softcap_to_f32(logits, cfg.logit_softcap, cfg.logit_scale)
        return logits

    def _forward_single_norm(self, tokens: torch.Tensor, ctx: StepContext, want_rows: torch.Tensor | None) -> torch.Tensor:
        """Parallel blocks with one norm: ``h = norm1(x)``; ``x <- x + mixer(h) + ff(h)``.  The residual stays fp32 in
        place; one kernel adds the (scaled) mixer branches and the feed-forward output and hands out the NEXT layer's
        ``h`` from the same pass."""
        cfg, w, eps, off = self.cfg, self.w, self.cfg.rms_norm_eps, self.norm_offset
        if cfg.norm_kind != "rms" or off != 0.0:
            raise ValueError("single-norm parallel blocks use plain RMS norms")
        resid, _ = embed_positions(tokens, ctx.batch.positions, w.embed, w.pos, want_act=False, scale=cfg.embed_scale)
        count = len(cfg.layers)
        h = rmsnorm_from_f32(resid, w.layers[0].pre1, eps, off, None, cfg.norm_kind) if count else None
        for li, (spec, lw) in enumerate(zip(cfg.layers, w.layers)):
            y = MIXERS[spec.kind](li, spec.mixer, lw.mix, h, ctx, eps)
            f = FEED_FORWARDS[spec.mlp.kind](spec.mlp, lw.mlp, h) if spec.mlp is not None else None
            br = y if isinstance(y, Branches) else Branches(y, None)
            nxt = w.layers[li + 1].pre1 if li + 1 < count else None
            h = branch_sum_residual(resid, br.a, br.a_weight, br.b, br.b_weight, f, eps, br.scale, want_act=False,
                                    scale_b=br.scale_b, next_weight=nxt)
            if self.layer_trace is not None:
                self.layer_trace.append(resid.clone())
        if want_rows is not None and want_rows.numel() == 0:
            return torch.empty((0, cfg.vocab_size), dtype=torch.float32, device=tokens.device)
        return self._head(resid, want_rows)

    def _forward_parallel(self, tokens: torch.Tensor, ctx: StepContext, want_rows: torch.Tensor | None) -> torch.Tensor:
        """Parallel blocks over a stack of fp32 results: level 0 is the (normed) embedding, level i + 1 the result of
        layer i.  Per layer: one kernel forms the layer's input (the depth-weighted sum of the levels so far, or the
        last level) IN the next level and both input norms from one statistic; mixer and feed-forward run; one kernel
        adds their (normed, averaged) outputs to the level; the token input (gate product, GELU * table row, projection)
        joins through the output-norm kernel.  The level then holds the layer's result."""
        cfg, w, eps, off = self.cfg, self.w, self.cfg.rms_norm_eps, self.norm_offset
        if cfg.norm_kind != "rms" or cfg.pre_norm or cfg.layer_scale:
            raise ValueError("parallel blocks use RMS input norms only")
        T, n, count = tokens.numel(), cfg.hidden_size, len(cfg.layers)
        levels = count + 2 if cfg.depth_average else 2           # the last level takes the mix the output norm reads
        stack = torch.empty((levels, T, n), dtype=torch.float32, device=tokens.device)
        if cfg.embed_norm:
            embed_rmsnorm(tokens, w.embed, w.embed_norm, eps, off, cfg.embed_scale, out=stack[0])
        else:
            stack[0].copy_(embed_positions(tokens, ctx.batch.positions, w.embed, w.pos, want_act=False,
                                           scale=cfg.embed_scale)[0])
        coef = None
        for li, (spec, lw) in enumerate(zip(cfg.layers, w.layers)):
            # without a depth average two levels alternate: the previous result is the input
            src = stack[:li + 1] if cfg.depth_average else stack[li % 2:li % 2 + 1]
            x = stack[li + 1] if cfg.depth_average else stack[(li + 1) % 2]
            _, h1, h2 = depth_mix_norms(src, src.shape[0], coef, lw.pre1, lw.pre2 if spec.mlp is not None else None, eps,
                                        off, out=x)
            y = MIXERS[spec.kind](li, spec.mixer, lw.mix, h1, ctx, eps)
            f = FEED_FORWARDS[spec.mlp.kind](spec.mlp, lw.mlp, h2) if spec.mlp is not None else None
            br = y if isinstance(y, Branches) else Branches(y, None)
            act = branch_sum_residual(x, br.a, br.a_weight, br.b, br.b_weight, f, eps, br.scale,
                                      want_act=lw.side is not None, scale_b=br.scale_b)
            if lw.side is not None:
                d = cfg.token_side_dim
                z = linear(x if act is None else act, lw.side["gate"])
                g = gelu_mul_gather(z, tokens, w.side_embed, li * d)
                post_norm_residual(x, linear(g, lw.side["proj"]), lw.side["norm"], eps, 0.0, want_act=False)
            coef = lw.depth
            if self.layer_trace is not None:
                self.layer_trace.append(x.clone())
        if cfg.depth_average and coef is not None:
            src, final = stack[:count + 1], stack[count + 1]
            depth_mix_norms(src, count + 1, coef, None, None, eps, off, out=final, dtype=self.dtype)
        else:
            final = stack[count] if cfg.depth_average else stack[count % 2]
        if want_rows is not None and want_rows.numel() == 0:
            return torch.empty((0, cfg.vocab_size), dtype=torch.float32 if cfg.logit_softcap else self.dtype,
                               device=tokens.device)
        return self._head(final, want_rows)


# ---------------------------------------------------------------------------------------------- Gufotar plumbing #
def parse_gufotar_config(raw: dict) -> LayeredConfig:
    layers = []
    for entry in raw["layers"]:
        kind, m = entry["type"], entry["mixer"]
        if kind == "mamba2":
            mixer = Mamba2Spec(heads=m["heads"], head_dim=m["vdim"], state=m["state"], groups=m.get("groups", 1),
                               norm_groups=m.get("norm_groups", 1), conv=m.get("conv", 1))
        elif kind == "attention":
            qt = m.get("q_temp") or {}
            mixer = SinkAttentionSpec(heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]), head_dim=m["dim"],
                                      v_head_dim=m.get("vdim", m["dim"]), scale=float(m["scale"]),
                                      softcap=float(m.get("softcap") or 0.0), gain_coef=float(qt.get("coef", 0.0)),
                                      gain_every=float(qt.get("every", 0.0)) if qt else 0.0, v_mix=bool(m.get("v_mix")))
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        mlp = entry.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(LayerSpec(kind, mixer, DenseMlpSpec(ff=mlp["ff"]) if mlp is not None else None))
    return LayeredConfig(name=raw.get("architecture", "Gufotar"), hidden_size=raw["width"], vocab_size=raw["vocab"],
                         max_seq_len=raw["max_positions"], rms_norm_eps=float(raw["norm"]["eps"]), layers=tuple(layers))


def map_gufotar_weights(cfg: LayeredConfig, tensors: dict[str, torch.Tensor], device: str,
                        dtype: torch.dtype) -> LayeredWeights:
    """Checkpoint names -> the decoder's weights in the activation dtype; q, k and v are row-concatenated so the three
    projections are one GEMM (each output element is the same dot product)."""

    def get(name: str) -> torch.Tensor:
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    out = LayeredWeights(embed=get("embed"), pos=get("pos"), final_norm=get("final.norm"), head=get("head"))
    for i, spec in enumerate(cfg.layers):
        p = f"l{i}.mix."
        if isinstance(spec.mixer, Mamba2Spec):
            mix = {"in": get(p + "in"), "conv": get(p + "conv"), "conv_b": get(p + "conv.b"),
                   "dt_bias": get(p + "dt_bias"), "A_log": get(p + "A_log"), "D": get(p + "D"),
                   "norm": get(p + "norm"), "o": get(p + "o")}
        else:
            mix = {"qkv": torch.cat([get(p + "q"), get(p + "k"), get(p + "v")], dim=0).contiguous(),
                   "q_norm": get(p + "q.norm"), "k_norm": get(p + "k.norm"), "o": get(p + "o")}
            if p + "sink" in tensors:
                mix["sink"] = get(p + "sink")
            if spec.mixer.v_mix and p + "vmix" in tensors:
                mix["vmix"] = get(p + "vmix").reshape(1)
        lw = LayeredLayerWeights(norm1=get(f"l{i}.norm1"), mix=mix)
        if spec.mlp is not None:
            lw.norm2 = get(f"l{i}.norm2")
            lw.mlp = {"up": get(f"l{i}.mlp.up"), "down": get(f"l{i}.mlp.down")}
        out.layers.append(lw)
    return out


def gufotar_tensor_shapes(cfg: LayeredConfig) -> dict[str, tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a configuration (random initialisation, shape checks)."""
    w = cfg.hidden_size
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg.vocab_size, w), "pos": (cfg.max_seq_len, w)}
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", spec.mixer
        shapes[f"l{i}.norm1"] = (w,)
        if isinstance(m, Mamba2Spec):
            shapes.update({p + "in": (m.in_rows, w), p + "conv": (m.conv_channels, m.conv), p + "conv.b": (m.conv_channels,),
                           p + "dt_bias": (m.heads,), p + "A_log": (m.heads,), p + "D": (m.heads,),
                           p + "norm": (m.inner,), p + "o": (w, m.inner)})
        else:
            shapes.update({p + "q": (m.heads * m.head_dim, w), p + "k": (m.kv_heads * m.head_dim, w),
                           p + "v": (m.kv_heads * m.v_head_dim, w), p + "q.norm": (m.heads * m.head_dim,),
                           p + "k.norm": (m.kv_heads * m.head_dim,), p + "vmix": (), p + "sink": (m.heads,),
                           p + "o": (w, m.heads * m.v_head_dim)})
        if spec.mlp is not None:
            shapes.update({f"l{i}.norm2": (w,), f"l{i}.mlp.up": (spec.mlp.ff, w), f"l{i}.mlp.down": (w, spec.mlp.ff)})
    shapes.update({"final.norm": (w,), "head": (cfg.vocab_size, w)})
    return shapes


def random_gufotar_tensors(cfg: LayeredConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    """Seeded random bf16 tensors with checkpoint names (benchmarks; there are no trained checkpoints offline)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in gufotar_tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(shape) == 2 and leaf != "conv":
            t = torch.randn(shape, generator=g) / (shape[1] ** 0.5)
        elif leaf in ("norm", "D"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf in ("dt_bias", "A_log"):
            t = -1.0 + 0.5 * torch.randn(shape, generator=g)
        elif leaf == "vmix":
            t = torch.tensor(0.4)
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        else:
            t = 0.3 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


register(Architecture("Gufotar", parse_gufotar_config, map_gufotar_weights, LayeredDecoder, ragged_steps=True,
                      sources=("gemm_dense", "gemm_simt", "residual_stream", "ssm_scan", "attention_sink", "elementwise")))


# ---------------------------------------------------------------------------------------------- Pesivik plumbing #
def _router_spec(mlp: dict) -> MoeMlpSpec:
    r = mlp["router"]
    g = r.get("groups") or {}
    shared = mlp.get("shared") or {}
    return MoeMlpSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]),
                      groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))),
                      shared_ff=int(shared.get("ff", 0)), activation="gelu")


def parse_pesivik_config(raw: dict) -> LayeredConfig:
    layers = []
    for entry in raw["layers"]:
        kind, m = entry["type"], entry["mixer"]
        if kind != "latent_attention":
            raise ValueError(f"unknown layer type {kind!r}")
        rot = m.get("rot") or {}
        rot_dim = int(m.get("rot_dim", 0))
        mixer = LatentAttentionSpec(heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=rot_dim,
                                    v_head_dim=int(m.get("vdim", m["dim"])), q_rank=int(m["q_rank"]),
                                    kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                                    rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)),
                                    window=int((m.get("mask") or {}).get("size", 0)), out_gate=True)
        mlp = entry.get("mlp")
        if mlp is not None and mlp.get("kind", "moe") != "moe":
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(LayerSpec(kind, mixer, _router_spec(mlp) if mlp is not None else None,
                                weights_of=entry.get("weights_of")))
    # a layer may name a layer that itself names another: every layer points at the one that owns the tensors
    for i, spec in enumerate(layers):
        j, hops = spec.weights_of, 0
        while j is not None and 0 <= j < len(layers) and layers[j].weights_of is not None:
            j, hops = layers[j].weights_of, hops + 1
            if hops > len(layers):
                raise ValueError(f"layer {i}: 'weights_of' runs in a circle")
        if j != spec.weights_of:
            layers[i] = LayerSpec(spec.kind, spec.mixer, spec.mlp, weights_of=j)
    return LayeredConfig(name=raw.get("architecture", "Pesivik"), hidden_size=int(raw["width"]),
                         vocab_size=int(raw["vocab"]), max_seq_len=0, rms_norm_eps=float(raw["norm"]["eps"]),
                         layers=tuple(layers), norm_kind="layer", pre_norm=True, layer_scale=True,
                         norm_weight_offset=0.0, learned_positions=False,
                         embed_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                         logit_softcap=float(raw.get("logit_softcap") or 0.0))


def map_pesivik_weights(cfg: LayeredConfig, tensors: dict[str, torch.Tensor], device: str,
                        dtype: torch.dtype) -> LayeredWeights:
    """Checkpoint names -> the decoder's weights.  The three projections that read the mixer input (query latent,
    key/value latent + rotated key part, head gates) are row-concatenated into one GEMM weight, padded with zero rows
    to a multiple of 8; the key up-projection is stored transposed per head (the queries are multiplied into the latent
    space); the experts are stacked.  A layer with ``weights_of`` gets the very object of the layer it names."""

    def get(name: str) -> torch.Tensor:
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    out = LayeredWeights(embed=get("embed"), pos=None, final_norm=get("final.norm"), head=get("head"))
    built: dict[int, LayeredLayerWeights] = {}
    for i, spec in enumerate(cfg.layers):
        if spec.weights_of is not None:
            continue
        m, p = spec.mixer, f"l{i}.mix."
        down = torch.cat([get(p + "dq"), get(p + "dkv"), get(p + "g")], dim=0)
        pad = -down.shape[0] % 8
        if pad:
            down = torch.cat([down, down.new_zeros((pad, down.shape[1]))], dim=0)
        uk = get(p + "uk").view(m.heads, m.head_dim, m.kv_rank)
        mix = {"down": down.contiguous(), "q_norm": get(p + "dq.norm"), "kv_norm": get(p + "dkv.norm"),
               "uq": get(p + "uq"), "uk_t": uk.transpose(1, 2).contiguous(),
               "uv": get(p + "uv").view(m.heads, m.v_head_dim, m.kv_rank).contiguous(), "o": get(p + "o")}
        lw = LayeredLayerWeights(norm1=get(f"l{i}.norm1b"), mix=mix, pre1=get(f"l{i}.norm1"), ls1=get(f"l{i}.ls1"))
        if spec.mlp is not None:
            q = f"l{i}.mlp."
            lw.pre2, lw.norm2, lw.ls2 = get(f"l{i}.norm2"), get(f"l{i}.norm2b"), get(f"l{i}.ls2")
            lw.mlp = {"router": get(q + "router"),
                      "up": torch.stack([get(f"{q}e{e}.up") for e in range(spec.mlp.experts)]).contiguous(),
                      "down": torch.stack([get(f"{q}e{e}.down") for e in range(spec.mlp.experts)]).contiguous()}
            if q + "correction" in tensors:
                lw.mlp["correction"] = get(q + "correction")
            if spec.mlp.shared_ff:
                lw.mlp["shared_up"], lw.mlp["shared_down"] = get(q + "shared.up"), get(q + "shared.down")
        built[i] = lw
    out.layers = [built[i if s.weights_of is None else s.weights_of] for i, s in enumerate(cfg.layers)]
    return out


def pesivik_tensor_shapes(cfg: LayeredConfig) -> dict[str, tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a configuration (random initialisation, shape checks)."""
    w = cfg.hidden_size
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg.vocab_size, w)}
    for i, spec in enumerate(cfg.layers):
        if spec.weights_of is not None:
            continue
        p, m = f"l{i}.mix.", spec.mixer
        for n in ("norm1", "norm1b", "ls1"):
            shapes[f"l{i}.{n}"] = (w,)
        shapes.update({p + "dq": (m.q_rank, w), p + "dq.norm": (m.q_rank,), p + "uq": (m.heads * (m.head_dim + m.rot_dim), m.q_rank),
                       p + "dkv": (m.kv_rank + m.rot_dim, w), p + "dkv.norm": (m.kv_rank,),
                       p + "uk": (m.heads * m.head_dim, m.kv_rank), p + "uv": (m.heads * m.v_head_dim, m.kv_rank),
                       p + "g": (m.heads, w), p + "o": (w, m.heads * m.v_head_dim)})
        if spec.mlp is not None:
            q = f"l{i}.mlp."
            for n in ("norm2", "norm2b", "ls2"):
                shapes[f"l{i}.{n}"] = (w,)
            for e in range(spec.mlp.experts):
                shapes[f"{q}e{e}.up"], shapes[f"{q}e{e}.down"] = (spec.mlp.ff, w), (w, spec.mlp.ff)
            shapes[q + "router"], shapes[q + "correction"] = (spec.mlp.experts, w), (spec.mlp.experts,)
            if spec.mlp.shared_ff:
                shapes[q + "shared.up"], shapes[q + "shared.down"] = (spec.mlp.shared_ff, w), (w, spec.mlp.shared_ff)
    shapes.update({"final.norm": (w,), "head": (cfg.vocab_size, w)})
    return shapes


def random_pesivik_tensors(cfg: LayeredConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    """Seeded random bf16 tensors with checkpoint names (benchmarks and tests; no trained checkpoints exist offline)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in pesivik_tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(shape) == 2:
            t = torch.randn(shape, generator=g) / (shape[1] ** 0.5)
        elif leaf == "correction":
            t = 0.1 * torch.randn(shape, generator=g)
        elif leaf in ("ls1", "ls2"):
            t = 0.5 + 0.1 * torch.randn(shape, generator=g)
        else:                                              # norm weights
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


_PESIVIK_SOURCES = ("gemm_dense", "gemm_simt", "gemm_rows_mma", "residual_stream", "attention_sink", "latent_attention",
                    "moe_routing", "elementwise")
register(Architecture("Pesivik", parse_pesivik_config, map_pesivik_weights, LayeredDecoder, ragged_steps=True,
                      sources=_PESIVIK_SOURCES))


# ---------------------------------------------------------------------------------------------- Tisosun plumbing #
def _block_attention_spec(m: dict) -> BlockAttentionSpec:
    rot = m.get("rot") or {}
    sc = rot.get("scaling") or {}
    return BlockAttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), head_dim=int(m["dim"]),
                              v_head_dim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]),
                              softcap=float(m.get("softcap") or 0.0), block=int((m.get("mask") or {}).get("size", 0)),
                              rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                              rot_factor=float(sc.get("factor", 1.0)), rot_original=float(sc.get("original", 0.0)),
                              rot_fast=float(sc.get("fast", 0.0)), rot_slow=float(sc.get("slow", 0.0)))


def parse_tisosun_config(raw: dict) -> LayeredConfig:
    layers = []
    for entry in raw["layers"]:
        kind, m = entry["type"], entry["mixer"]
        if kind == "mingru":
            mixer = MinGruSpec(width=int(m["width"]))
        elif kind == "rglru":
            mixer = RgLruSpec(width=int(m["width"]), blocks=int(m.get("blocks", 1)), conv=int(m.get("conv", 1)))
        elif kind == "parallel":
            r = m["right"]
            mixer = SideBySideSpec(_block_attention_spec(m["left"]),
                                   DecayAttentionSpec(heads=int(r["heads"]), head_dim=int(r["dim"]),
                                                      v_head_dim=int(r.get("vdim", r["dim"])),
                                                      decay=tuple(float(d) for d in r["decay"])))
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        mlp = entry.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(LayerSpec(kind, mixer, DenseMlpSpec(ff=int(mlp["ff"]), activation="silu", gated=True)
                                if mlp is not None else None))
    return LayeredConfig(name=raw.get("architecture", "Tisosun"), hidden_size=int(raw["width"]),
                         vocab_size=int(raw["vocab"]), max_seq_len=0, rms_norm_eps=float(raw["norm"]["eps"]),
                         layers=tuple(layers), norm_weight_offset=1.0, learned_positions=False, parallel_block=True,
                         embed_norm=True, token_side_dim=int((raw.get("token_side") or {}).get("dim", 0)),
                         depth_average=True)


def _pad_rows(t: torch.Tensor, multiple: int) -> torch.Tensor:
    pad = -t.shape[0] % multiple
    return torch.cat([t, t.new_zeros((pad, *t.shape[1:]))], dim=0) if pad else t


def map_tisosun_weights(cfg: LayeredConfig, tensors: dict[str, torch.Tensor], device: str,
                        dtype: torch.dtype) -> LayeredWeights:
    """Checkpoint names -> the decoder's weights.  Every mixer's input projections are row-concatenated into one GEMM
    weight with one bias vector (zeros where a projection has none); the attention half is padded with zero rows to a
    multiple of 8 so that the linear-attention half starts on a 16-byte boundary, and its columns are ordered
    [values | keys | queries | gate], the layout the scan kernel reads.  Decays are fp32, rotary frequencies fp64."""

    def get(name: str) -> torch.Tensor:
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    def zeros(n: int) -> torch.Tensor:
        return torch.zeros(n, dtype=dtype, device=device)

    out = LayeredWeights(embed=get("embed"), pos=None, final_norm=get("final.norm"), head=get("head"),
                         embed_norm=get("embed.norm"), side_embed=get("side.embed") if cfg.token_side_dim else None)
    freq_cache: dict[tuple, torch.Tensor] = {}
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", spec.mixer
        if isinstance(m, MinGruSpec):
            mix = {"in": torch.cat([get(p + "z"), get(p + "x"), get(p + "g")], dim=0).contiguous(),
                   "in_b": torch.cat([get(p + "z.b"), get(p + "x.b"), zeros(m.width)]), "o": get(p + "o")}
        elif isinstance(m, RgLruSpec):
            mix = {"in": torch.cat([get(p + "y"), get(p + "x")], dim=0).contiguous(),
                   "in_b": torch.cat([get(p + "y.b"), get(p + "x.b")]), "conv": get(p + "conv"),
                   "conv_b": get(p + "conv.b"), "ra": get(p + "ra"), "ri": get(p + "ri"),
                   "ra_b": get(p + "ra.b").reshape(-1), "ri_b": get(p + "ri.b").reshape(-1), "lam": get(p + "lam"),
                   "o": get(p + "o")}
        else:
            L, R = m.left, m.right
            lq = _pad_rows(torch.cat([get(p + "left.q"), get(p + "left.k"), get(p + "left.v")], dim=0), 8)
            lb = _pad_rows(torch.cat([get(p + "left.q.b"), get(p + "left.k.b"), get(p + "left.v.b")]), 8)
            rq = torch.cat([get(p + "right.v"), get(p + "right.k"), get(p + "right.q"), get(p + "right.g")], dim=0)
            key = (L.rot_dims, L.rot_base, L.rot_factor, L.rot_original, L.rot_fast, L.rot_slow)
            if L.rot_dims and key not in freq_cache:
                freq_cache[key] = torch.tensor(rotary_frequencies(*key)[0], dtype=torch.float64).to(device=device)
            mix = {"in": torch.cat([lq, rq], dim=0).contiguous(), "in_b": torch.cat([lb, zeros(rq.shape[0])]),
                   "q_norm": get(p + "left.q.norm"), "k_norm": get(p + "left.k.norm"), "left_o": get(p + "left.o"),
                   "right_norm": get(p + "right.norm"), "right_o": get(p + "right.o"), "left_out": get(p + "left.out"),
                   "right_out": get(p + "right.out"),
                   "decay": torch.tensor(R.decay, dtype=torch.float64).to(device=device, dtype=torch.float32)}
            if L.rot_dims:
                mix["freqs"] = freq_cache[key]
        lw = LayeredLayerWeights(norm1=None, mix=mix, pre1=get(f"l{i}.norm1"))
        if spec.mlp is not None:
            lw.pre2 = get(f"l{i}.norm2")
            lw.mlp = {"gate_up": torch.cat([get(f"l{i}.mlp.gate"), get(f"l{i}.mlp.up")], dim=0).contiguous(),
                      "down": get(f"l{i}.mlp.down")}
        if cfg.token_side_dim:
            lw.side = {"gate": get(f"l{i}.side.gate"), "proj": get(f"l{i}.side.proj"), "norm": get(f"l{i}.side.norm")}
        if cfg.depth_average and f"l{i}.dwa" in tensors:      # a layer without coefficients hands its result on as it is
            lw.depth = get(f"l{i}.dwa")
        out.layers.append(lw)
    return out


def tisosun_tensor_shapes(cfg: LayeredConfig) -> dict[str, tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a configuration (random initialisation, shape checks)."""
    w, d = cfg.hidden_size, cfg.token_side_dim
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg.vocab_size, w), "embed.norm": (w,)}
    if d:
        shapes["side.embed"] = (cfg.vocab_size, d * len(cfg.layers))
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", spec.mixer
        shapes[f"l{i}.norm1"] = (w,)
        if isinstance(m, MinGruSpec):
            shapes.update({p + "z": (m.width, w), p + "z.b": (m.width,), p + "x": (m.width, w), p + "x.b": (m.width,),
                           p + "g": (m.width, w), p + "o": (w, m.width)})
        elif isinstance(m, RgLruSpec):
            per = m.width // m.blocks
            shapes.update({p + "y": (m.width, w), p + "y.b": (m.width,), p + "x": (m.width, w), p + "x.b": (m.width,),
                           p + "conv": (m.width, m.conv), p + "conv.b": (m.width,), p + "ra": (m.blocks, per, per),
                           p + "ra.b": (m.blocks, per), p + "ri": (m.blocks, per, per), p + "ri.b": (m.blocks, per),
                           p + "lam": (m.width,), p + "o": (w, m.width)})
        else:
            L, R = m.left, m.right
            shapes.update({p + "left.q": (L.heads * L.head_dim, w), p + "left.q.b": (L.heads * L.head_dim,),
                           p + "left.k": (L.kv_heads * L.head_dim, w), p + "left.k.b": (L.kv_heads * L.head_dim,),
                           p + "left.v": (L.kv_heads * L.v_head_dim, w), p + "left.v.b": (L.kv_heads * L.v_head_dim,),
                           p + "left.q.norm": (L.head_dim,), p + "left.k.norm": (L.head_dim,),
                           p + "left.o": (w, L.heads * L.v_head_dim),
                           p + "right.q": (R.heads * R.head_dim, w), p + "right.k": (R.heads * R.head_dim, w),
                           p + "right.v": (R.heads * R.v_head_dim, w), p + "right.g": (R.heads * R.v_head_dim, w),
                           p + "right.o": (w, R.heads * R.v_head_dim), p + "right.norm": (R.heads * R.v_head_dim,),
                           p + "left.out": (w,), p + "right.out": (w,)})
        if spec.mlp is not None:
            shapes.update({f"l{i}.norm2": (w,), f"l{i}.mlp.gate": (spec.mlp.ff, w), f"l{i}.mlp.up": (spec.mlp.ff, w),
                           f"l{i}.mlp.down": (w, spec.mlp.ff)})
        if cfg.depth_average:
            shapes[f"l{i}.dwa"] = (i + 2,)
        if d:
            shapes.update({f"l{i}.side.gate": (d, w), f"l{i}.side.proj": (w, d), f"l{i}.side.norm": (w,)})
    shapes.update({"final.norm": (w,), "head": (cfg.vocab_size, w)})
    return shapes


def random_tisosun_tensors(cfg: LayeredConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    """Seeded random bf16 tensors with checkpoint names (benchmarks and tests; no trained checkpoints exist offline)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tisosun_tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "dwa":                                     # mostly the newest result, some of every older one
            t = 0.15 * torch.randn(shape, generator=g)
            t[-1] += 0.8
        elif leaf == "conv":
            t = 0.4 * torch.randn(shape, generator=g)
        elif name.endswith("side.embed"):
            t = torch.randn(shape, generator=g)
        elif len(shape) >= 2:
            t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5)
        elif leaf == "lam":
            t = -1.0 + 0.7 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.2 * torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2") or name in ("embed.norm", "final.norm"):
            t = 0.1 * torch.randn(shape, generator=g)         # stored as the distance from one
        else:                                                 # plain norm weights
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


_TISOSUN_SOURCES = ("gemm_dense", "gemm_simt", "gemm_rows_mma", "residual_stream", "parallel_stream", "gated_recurrence",
                    "rotary_heads", "ssm_scan", "decay_attention_mma", "attention_sink", "elementwise")
register(Architecture("Tisosun", parse_tisosun_config, map_tisosun_weights, LayeredDecoder, ragged_steps=True,
                      sources=_TISOSUN_SOURCES))


# ---------------------------------------------------------------------------------------------- Gofezen plumbing #
def _gofezen_mlp(mlp: dict | None) -> DenseMlpSpec | MoeMlpSpec | None:
    if mlp is None:
        return None
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return DenseMlpSpec(ff=int(mlp["ff"]), activation="silu", gated=True)
    if kind != "moe":
        raise ValueError(f"unknown feed-forward kind {kind!r}")
    r = mlp["router"]
    shared = mlp.get("shared") or {}
    return MoeMlpSpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]),
                      shared_ff=int(shared.get("ff", 0)), activation="silu", gated=True, renormalize=False,
                      weight_on_input=True, shared_gate=bool(shared))


def parse_gofezen_config(raw: dict) -> LayeredConfig:
    layers = []
    for entry in raw["layers"]:
        kind, m = entry["type"], entry["mixer"]
        if kind == "hgrn2":
            key, mixer = "forget_gate", ForgetGateAttentionSpec(heads=int(m["heads"]), head_dim=int(m["dim"]),
                                                                v_head_dim=int(m.get("vdim", m["dim"])))
        elif kind == "parallel":
            l, r = m["left"], m["right"]
            left = ConvWindowAttentionSpec(heads=int(l["heads"]), kv_heads=int(l.get("kv_heads", l["heads"])),
                                           head_dim=int(l["dim"]), v_head_dim=int(l.get("vdim", l["dim"])),
                                           scale=float(l["scale"]), window=int((l.get("mask") or {}).get("size", 0)),
                                           conv=int(l.get("conv", 1)))
            right = DeltaRuleSpec(heads=int(r["heads"]), qk_heads=int(r.get("kv_heads", r["heads"])),
                                  head_dim=int(r["dim"]), v_head_dim=int(r.get("vdim", r["dim"])),
                                  conv=int(r.get("conv", 1)))
            key, mixer = "window_delta", WindowDeltaPairSpec(left, right, float(m.get("left_scale", 1.0)),
                                                             float(m.get("right_scale", 1.0)))
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        layers.append(LayerSpec(key, mixer, _gofezen_mlp(entry.get("mlp"))))
    return LayeredConfig(name=raw.get("architecture", "Gofezen"), hidden_size=int(raw["width"]),
                         vocab_size=int(raw["vocab"]), max_seq_len=int(raw["max_positions"]),
                         rms_norm_eps=float(raw["norm"]["eps"]), layers=tuple(layers), norm_weight_offset=0.0,
                         embed_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                         logit_softcap=float(raw.get("logit_softcap") or 0.0), parallel_block=True, single_norm=True,
                         logit_scale=float(raw.get("logit_scale", 1.0)))


def map_gofezen_weights(cfg: LayeredConfig, tensors: dict[str, torch.Tensor], device: str,
                        dtype: torch.dtype) -> LayeredWeights:
    """Checkpoint names -> the decoder's weights.  Every mixer's input projections are row-concatenated into one GEMM
    weight with one bias vector (zeros where a projection has none); parts that a kernel reads with 16-byte accesses
    start on a multiple of 8 rows.  The convolutions' tap tables are stacked in the same order as their channels.
    Experts are stacked with each expert's gate rows before its up rows; the shared expert's token-gate row rides at
    the end of its [gate | up] weight."""

    def get(name: str) -> torch.Tensor:
        if name not in tensors:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    def zeros(*shape: int) -> torch.Tensor:
        return torch.zeros(shape, dtype=dtype, device=device)

    out = LayeredWeights(embed=get("embed"), pos=get("pos"), final_norm=get("final.norm"), head=get("head"))
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", spec.mixer
        if isinstance(m, ForgetGateAttentionSpec):
            n = m.heads * m.head_dim
            mix = {"in": torch.cat([get(p + "q"), get(p + "f"), get(p + "v")], dim=0).contiguous(),
                   "in_b": torch.cat([zeros(n), get(p + "f.b"), zeros(m.heads * m.v_head_dim)]),
                   "lower": get(p + "lower"), "norm": get(p + "norm"), "o": get(p + "o")}
        else:
            L, R = m.left, m.right
            lq = _pad_rows(torch.cat([get(p + "left.q"), get(p + "left.k"), get(p + "left.v")], dim=0), 8)
            lb = _pad_rows(torch.cat([get(p + "left.q.b"), get(p + "left.k.b"), get(p + "left.v.b")]), 8)
            rq = _pad_rows(torch.cat([get(p + "right.q"), get(p + "right.k"), get(p + "right.v"), get(p + "right.b"),
                                      get(p + "right.a")], dim=0), 8)
            rg = _pad_rows(get(p + "right.g"), 8)
            mix = {"in": torch.cat([lq, rq, rg], dim=0).contiguous(),
                   "in_b": torch.cat([lb, zeros(rq.shape[0] + rg.shape[0])]),
                   "left_conv": torch.cat([get(p + "left.q.conv"), get(p + "left.k.conv"), get(p + "left.v.conv")],
                                          dim=0).contiguous(),
                   "left_conv_b": zeros(L.channels), "ones": torch.ones(L.head_dim, dtype=dtype, device=device),
                   "left_o": get(p + "left.o"),
                   "right_conv": torch.cat([get(p + "right.q.conv"), get(p + "right.k.conv"), get(p + "right.v.conv")],
                                           dim=0).contiguous(),
                   "right_conv_b": zeros(R.channels), "A_log": get(p + "right.A_log"), "dt_bias": get(p + "right.dt_bias"),
                   "right_norm": get(p + "right.norm"), "right_o": get(p + "right.o")}
            if L.head_mix:
                mix["talk"] = get(p + "left.talk")
        lw = LayeredLayerWeights(norm1=None, mix=mix, pre1=get(f"l{i}.norm1"))
        q = f"l{i}.mlp."
        if isinstance(spec.mlp, DenseMlpSpec):
            lw.mlp = {"gate_up": torch.cat([get(q + "gate"), get(q + "up")], dim=0).contiguous(), "down": get(q + "down")}
        elif isinstance(spec.mlp, MoeMlpSpec):
            e = range(spec.mlp.experts)
            lw.mlp = {"router": get(q + "router"),
                      "gate_up": torch.stack([torch.cat([get(f"{q}e{j}.gate"), get(f"{q}e{j}.up")], dim=0) for j in e]).contiguous(),
                      "down": torch.stack([get(f"{q}e{j}.down") for j in e]).contiguous()}
            if spec.mlp.shared_ff:
                parts = [get(q + "shared.gate"), get(q + "shared.up")]
                if spec.mlp.shared_gate:
                    parts.append(get(q + "shared.sg").reshape(1, -1))
                lw.mlp["shared_gate_up"] = _pad_rows(torch.cat(parts, dim=0), 8).contiguous()
                lw.mlp["shared_down"] = get(q + "shared.down")
        out.layers.append(lw)
    return out


def gofezen_tensor_shapes(cfg: LayeredConfig) -> dict[str, tuple[int, ...]]:
    """Checkpoint tensor names and shapes of a configuration (random initialisation, shape checks)."""
    w = cfg.hidden_size
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg.vocab_size, w), "pos": (cfg.max_seq_len, w)}
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", spec.mixer
        shapes[f"l{i}.norm1"] = (w,)
        if isinstance(m, ForgetGateAttentionSpec):
            n, nv = m.heads * m.head_dim, m.heads * m.v_head_dim
            shapes.update({p + "q": (n, w), p + "f": (n, w), p + "f.b": (n,), p + "lower": (n,), p + "v": (nv, w),
                           p + "norm": (m.v_head_dim,), p + "o": (w, nv)})
        else:
            L, R = m.left, m.right
            lq, lk, lv = L.heads * L.head_dim, L.kv_heads * L.head_dim, L.kv_heads * L.v_head_dim
            rq, rv = R.qk_heads * R.head_dim, R.heads * R.v_head_dim
            shapes.update({p + "left.q": (lq, w), p + "left.q.b": (lq,), p + "left.k": (lk, w), p + "left.k.b": (lk,),
                           p + "left.v": (lv, w), p + "left.v.b": (lv,), p + "left.q.conv": (lq, L.conv),
                           p + "left.k.conv": (lk, L.conv), p + "left.v.conv": (lv, L.conv),
                           p + "left.talk": (L.heads, L.heads), p + "left.o": (w, L.heads * L.v_head_dim),
                           p + "right.q": (rq, w), p + "right.q.conv": (rq, R.conv), p + "right.k": (rq, w),
                           p + "right.k.conv": (rq, R.conv), p + "right.v": (rv, w), p + "right.v.conv": (rv, R.conv),
                           p + "right.b": (R.heads, w), p + "right.A_log": (R.heads,), p + "right.norm": (R.v_head_dim,),
                           p + "right.a": (R.heads, w), p + "right.dt_bias": (R.heads,), p + "right.g": (rv, w),
                           p + "right.o": (w, rv)})
        q = f"l{i}.mlp."
        if isinstance(spec.mlp, DenseMlpSpec):
            shapes.update({q + "gate": (spec.mlp.ff, w), q + "up": (spec.mlp.ff, w), q + "down": (w, spec.mlp.ff)})
        elif isinstance(spec.mlp, MoeMlpSpec):
            for e in range(spec.mlp.experts):
                shapes.update({f"{q}e{e}.gate": (spec.mlp.ff, w), f"{q}e{e}.up": (spec.mlp.ff, w),
                               f"{q}e{e}.down": (w, spec.mlp.ff)})
            shapes[q + "router"] = (spec.mlp.experts, w)
            if spec.mlp.shared_ff:
                f = spec.mlp.shared_ff
                shapes.update({q + "shared.gate": (f, w), q + "shared.up": (f, w), q + "shared.down": (w, f),
                               q + "shared.sg": (1, w)})
    shapes.update({"final.norm": (w,), "head": (cfg.vocab_size, w)})
    return shapes


def random_gofezen_tensors(cfg: LayeredConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    """Seeded random bf16 tensors with checkpoint names (benchmarks and tests; no trained checkpoints exist offline)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in gofezen_tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "conv":
            t = 0.4 * torch.randn(shape, generator=g)
        elif leaf == "talk":                                  # mostly the head itself, some of every other head
            t = 0.2 * torch.randn(shape, generator=g) + 0.8 * torch.eye(shape[0])
        elif leaf == "lower":
            t = torch.rand(shape, generator=g) * 0.9
        elif name == "pos":
            t = 0.5 * torch.randn(shape, generator=g)
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) / (shape[1] ** 0.5)
        elif leaf in ("A_log", "dt_bias"):
            t = -1.0 + 0.7 * torch.randn(shape, generator=g)
        elif leaf == "b" and name.endswith((".q.b", ".k.b", ".v.b", ".f.b")):
            t = 0.3 * torch.randn(shape, generator=g)
        else:                                                 # plain norm weights
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


_GOFEZEN_SOURCES = ("gemm_dense", "gemm_simt", "gemm_rows_mma", "residual_stream", "parallel_stream", "ssm_scan",
                    "gated_linear_attention", "rotary_heads", "attention_sink", "moe_routing", "elementwise")
register(Architecture("Gofezen", parse_gofezen_config, map_gofezen_weights, LayeredDecoder, ragged_steps=True,
                      sources=_GOFEZEN_SOURCES))
