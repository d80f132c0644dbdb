"""Model geometry for the decoder families the reference serves (LLaMA / Qwen2 / Qwen3 dense).

The reference wraps HF ``AutoConfig`` (lite_llama/models/config.py:48-218); no checkpoints or network
exist in this environment, so the public HF geometries are written down here.
"""

from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class ModelConfig:
    name: str
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    qkv_bias: bool = False
    use_qk_norm: bool = False
    tie_word_embeddings: bool = False
    max_seq_len: int = 2048
    # routed-expert FFN (reference: lite_llama/models/qwen3_moe.py:48-122); 0 experts = dense SwiGLU MLP
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def validate(self) -> None:
        if self.head_dim % 8 != 0:
            raise ValueError(f"head_dim {self.head_dim} must be a multiple of 8")
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)


PRESETS: dict[str, ModelConfig] = {
    "llama-3-8b": ModelConfig("llama-3-8b", 4096, 32, 32, 8, 128, 14336, 128256, rope_theta=5e5, rms_norm_eps=1e-5),
    "qwen2.5-7b": ModelConfig("qwen2.5-7b", 3584, 28, 28, 4, 128, 18944, 152064, rope_theta=1e6, rms_norm_eps=1e-6,
                              qkv_bias=True),
    "qwen2.5-0.5b": ModelConfig("qwen2.5-0.5b", 896, 24, 14, 2, 64, 4864, 151936, rope_theta=1e6, rms_norm_eps=1e-6,
                                qkv_bias=True, tie_word_embeddings=True),
    "qwen3-8b": ModelConfig("qwen3-8b", 4096, 36, 32, 8, 128, 12288, 151936, rope_theta=1e6, rms_norm_eps=1e-6,
                            use_qk_norm=True),
    "qwen3-30b-a3b": ModelConfig("qwen3-30b-a3b", 2048, 48, 32, 4, 128, 6144, 151936, rope_theta=1e6, rms_norm_eps=1e-6,
                                 use_qk_norm=True, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768),
    # small geometries for tests (same code paths, seconds on CPU for the oracle)
    "tiny-llama": ModelConfig("tiny-llama", 256, 2, 8, 2, 32, 512, 1000, rope_theta=1e4),
    "tiny-qwen3": ModelConfig("tiny-qwen3", 256, 2, 8, 4, 32, 512, 1000, rope_theta=1e4, qkv_bias=False,
                              use_qk_norm=True, rms_norm_eps=1e-6),
    "tiny-qwen3-moe": ModelConfig("tiny-qwen3-moe", 256, 2, 8, 4, 32, 512, 1000, rope_theta=1e4, use_qk_norm=True,
                                  rms_norm_eps=1e-6, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128),
    "tiny-qwen2": ModelConfig("tiny-qwen2", 256, 2, 8, 2, 32, 512, 1000, rope_theta=1e4, qkv_bias=True,
                              rms_norm_eps=1e-6),
}


# ---------------------------------------------------------------------------------------------------------------
# Layer-list models: every layer names its own mixer (attention or a recurrent one) and feed-forward, so the
# geometry is a tuple of layer specs instead of one set of sizes.  The reference has no such family (its configs
# are uniform decoders, lite_llama/models/config.py:48-218); the specs below are what the executor asks about one.
# ---------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Mamba2Spec:
    """Scalar-decay state-space mixer: ``heads`` heads of ``head_dim`` channels, ``state`` rows of state per head,
    B / C shared by ``groups`` groups of heads, output norm in ``norm_groups`` parts, ``conv`` convolution taps."""

    heads: int
    head_dim: int
    state: int
    groups: int = 1
    norm_groups: int = 1
    conv: int = 4

    @property
    def inner(self) -> int:
        return self.heads * self.head_dim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state

    @property
    def in_rows(self) -> int:                       # [z | x | B | C | dt]
        return 2 * self.inner + 2 * self.groups * self.state + self.heads

    @property
    def state_shape(self) -> tuple[int, ...]:       # per request slot, fp32
        return (self.heads, self.state, self.head_dim)

    @property
    def conv_tail_shape(self) -> tuple[int, int] | None:      # per request slot, activation dtype
        return (max(self.conv - 1, 1), self.conv_channels)

    def validate(self) -> None:
        if self.heads % self.groups or self.inner % self.norm_groups or self.conv < 1 or self.state > 768:
            raise ValueError(f"unsupported state-space mixer geometry: {self}")


@dataclass(frozen=True)
class SinkAttentionSpec:
    """Position-free attention: whole-row q / k norms, a query gain that grows with the logarithm of the position
    (``1 + gain_coef * ln(floor((p + 1) / gain_every) + 1)``; ``gain_every == 0``: none), ``tanh`` soft cap
    (0: none), a learned per-head sink in the softmax denominator, value mixing across the layers that ask for it."""

    heads: int
    kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    softcap: float = 0.0
    gain_coef: float = 0.0
    gain_every: float = 0.0
    v_mix: bool = False

    def validate(self) -> None:
        if self.heads % self.kv_heads or self.v_head_dim > 256:
            raise ValueError(f"unsupported attention geometry: {self}")

    @property
    def cache_row_width(self) -> int:                  # one token's pool row: all K heads, then all V heads
        return self.kv_heads * (self.head_dim + self.v_head_dim)


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention through low-rank latents: queries ``h -> q_rank -> heads x (head_dim + rot_dim)``; keys / values
    ``h -> kv_rank`` (the cached latent) ``-> heads x head_dim`` keys and ``heads x v_head_dim`` values, plus one
    ``rot_dim``-wide rotated key part shared by all heads (cached beside the latent).  Rotary positions act on the
    first ``rot_dims`` entries of the rotated parts (rotate-half pairing, base ``rot_base``).  ``window`` > 0: a token
    sees itself and the ``window - 1`` tokens before it.  ``out_gate``: a per-head sigmoid gate on the head outputs."""

    heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float = 10000.0
    window: int = 0
    out_gate: bool = True

    def validate(self) -> None:
        if min(self.heads, self.head_dim, self.v_head_dim, self.q_rank, self.kv_rank) < 1 or self.rot_dim < 0 or \
                self.rot_dims % 2 or not 0 <= self.rot_dims <= self.rot_dim or self.window < 0 or self.kv_rank > 256:
            raise ValueError(f"unsupported latent attention geometry: {self}")

    @property
    def cache_row_width(self) -> int:                  # [latent | rotated key part], padded to 16-byte vectors
        return -(-(self.kv_rank + self.rot_dim) // 8) * 8


@dataclass(frozen=True)
class MinGruSpec:
    """Minimal gated recurrent unit: ``width`` channels, one fp32 state value per channel; update gate, candidate
    and output gate read the current token only."""

    width: int

    @property
    def state_shape(self) -> tuple[int, ...]:
        return (self.width,)

    conv_tail_shape = None

    def validate(self) -> None:
        if self.width < 1:
            raise ValueError(f"unsupported recurrent mixer geometry: {self}")


@dataclass(frozen=True)
class RgLruSpec:
    """Recurrent block around a real-gated linear recurrent unit: a GELU branch and a recurrence branch of ``width``
    channels each; the recurrence branch passes a ``conv``-tap causal convolution (no activation), its two gates are
    block-diagonal projections in ``blocks`` parts, the decay is ``exp(-decay_scale * r * softplus(lam))``."""

    width: int
    blocks: int
    conv: int
    decay_scale: float = 8.0

    @property
    def state_shape(self) -> tuple[int, ...]:
        return (self.width,)

    @property
    def conv_tail_shape(self) -> tuple[int, int] | None:
        return (max(self.conv - 1, 1), self.width)

    def validate(self) -> None:
        if self.width < 1 or self.blocks < 1 or self.width % self.blocks or self.conv < 1:
            raise ValueError(f"unsupported recurrent mixer geometry: {self}")


@dataclass(frozen=True)
class BlockAttentionSpec:
    """Softmax attention with biased projections, a per-head RMS norm of q and k (one ``[head_dim]`` weight each,
    shared by the heads), rotary positions on the first ``rot_dims`` entries of every head (``pairing``: "neighbours"
    = entries 2i, 2i+1; "halves" = i, i + rot_dims/2) with frequency interpolation by parts (``rot_factor`` > 1: see
    ``kernels.rotary_frequencies``), a ``tanh`` soft cap (0: none) and a block-diagonal causal mask: position p sees
    the positions of its own run of ``block`` that are not after it (0: plain causal)."""

    heads: int
    kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    softcap: float = 0.0
    block: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_factor: float = 1.0
    rot_original: float = 0.0
    rot_fast: float = 0.0
    rot_slow: float = 0.0
    pairing: str = "neighbours"

    def validate(self) -> None:
        if min(self.heads, self.kv_heads, self.head_dim, self.v_head_dim) < 1 or self.heads % self.kv_heads or \
                self.v_head_dim > 256 or self.rot_dims % 2 or not 0 <= self.rot_dims <= self.head_dim or self.block < 0 \
                or self.pairing not in ("neighbours", "halves"):
            raise ValueError(f"unsupported attention geometry: {self}")

    @property
    def cache_row_width(self) -> int:                  # all K heads, then all V heads, padded to 16-byte vectors
        return -(-self.kv_heads * (self.head_dim + self.v_head_dim) // 8) * 8


@dataclass(frozen=True)
class DecayAttentionSpec:
    """Linear attention with one fixed decay per head: q, k (``heads x head_dim``) and v (``heads x v_head_dim``)
    pass SiLU, the memory ``S_h <- decay_h S_h + k v^T`` (fp32, ``head_dim x v_head_dim``) answers ``S_h^T q``; the
    joined heads are RMS-normed as one row, gated by a sigmoid projection and projected out."""

    heads: int
    head_dim: int
    v_head_dim: int
    decay: tuple[float, ...]

    @property
    def state_shape(self) -> tuple[int, ...]:
        return (self.heads, self.head_dim, self.v_head_dim)

    conv_tail_shape = None

    def validate(self) -> None:
        if min(self.heads, self.head_dim, self.v_head_dim) < 1 or len(self.decay) != self.heads or self.head_dim > 768 \
                or not all(0.0 <= d <= 1.0 for d in self.decay):
            raise ValueError(f"unsupported linear attention geometry: {self}")


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input: softmax attention over the KV pool (``left``) and decayed linear
    attention over a state slot (``right``); each output is RMS-normed over the model width with its own weight and
    the two are averaged."""

    left: BlockAttentionSpec
    right: DecayAttentionSpec

    def validate(self) -> None:
        self.left.validate()
        self.right.validate()

    @property
    def cache_row_width(self) -> int:
        return self.left.cache_row_width

    @property
    def state_shape(self) -> tuple[int, ...]:
        return self.right.state_shape

    conv_tail_shape = None


@dataclass(frozen=True)
class ForgetGateAttentionSpec:
    """Linear attention whose forget gate also decides what is written: per head an fp32 memory ``head_dim x
    v_head_dim``; per key channel ``f = l + (1 - l) sigmoid(.)`` with a learned lower bound ``l``;
    ``S <- diag(f) S + (1 - f) v^T``, read-out ``S^T silu(q)``, per-head RMS norm (one ``[v_head_dim]`` weight)."""

    heads: int
    head_dim: int
    v_head_dim: int

    @property
    def state_shape(self) -> tuple[int, ...]:
        return (self.heads, self.head_dim, self.v_head_dim)

    conv_tail_shape = None

    def validate(self) -> None:
        if min(self.heads, self.head_dim, self.v_head_dim) < 1 or self.head_dim > 256:
            raise ValueError(f"unsupported linear attention geometry: {self}")


@dataclass(frozen=True)
class ConvWindowAttentionSpec:
    """Position-free softmax attention: biased projections, a ``conv``-tap causal convolution on q, k and v (no
    activation), a weightless per-head unit-RMS of q and k (``qk_unit_rms``), a sliding ``window`` (0: plain causal)
    and, with ``head_mix``, a ``heads x heads`` matrix that mixes the heads' softmax weights before they meet the
    values (every head keeps reading its own key/value head)."""

    heads: int
    kv_heads: int
    head_dim: int
    v_head_dim: int
    scale: float
    window: int = 0
    conv: int = 1
    head_mix: bool = True
    qk_unit_rms: bool = True

    @property
    def channels(self) -> int:                         # q | k | v side by side: what the convolution runs over
        return self.heads * self.head_dim + self.kv_heads * (self.head_dim + self.v_head_dim)

    @property
    def cache_row_width(self) -> int:                  # all K heads, then all V heads, padded to 16-byte vectors
        return -(-self.kv_heads * (self.head_dim + self.v_head_dim) // 8) * 8

    def validate(self) -> None:
        if min(self.heads, self.kv_heads, self.head_dim, self.v_head_dim, self.conv) < 1 or self.heads % self.kv_heads \
                or self.v_head_dim > 256 or self.window < 0:
            raise ValueError(f"unsupported attention geometry: {self}")


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Gated delta rule: q, k (``qk_heads x head_dim``) and v (``heads x v_head_dim``) pass a ``conv``-tap causal
    convolution and SiLU; q, k become unit vectors (``unit_eps`` inside the root), q times ``head_dim^-1/2``; per head a
    write strength ``sigmoid(.)`` and a decay ``exp(-exp(A_log) softplus(. + dt_bias))``;
    ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``; per-head RMS norm, SiLU gate."""

    heads: int
    qk_heads: int
    head_dim: int
    v_head_dim: int
    conv: int = 1
    unit_eps: float = 1e-6

    @property
    def channels(self) -> int:
        return 2 * self.qk_heads * self.head_dim + self.heads * self.v_head_dim

    @property
    def state_shape(self) -> tuple[int, ...]:
        return (self.heads, self.head_dim, self.v_head_dim)

    def validate(self) -> None:
        if min(self.heads, self.qk_heads, self.head_dim, self.v_head_dim, self.conv) < 1 or self.heads % self.qk_heads \
                or self.head_dim > 256:
            raise ValueError(f"unsupported delta-rule geometry: {self}")


@dataclass(frozen=True)
class WindowDeltaPairSpec:
    """Two mixers that read the same input: convolved sliding-window attention over the KV pool (``left``) and a gated
    delta rule over a state slot (``right``); the result is ``left_scale * left + right_scale * right``.  Each side
    keeps the last inputs of its own convolution per slot (``conv_tails``)."""

    left: ConvWindowAttentionSpec
    right: DeltaRuleSpec
    left_scale: float = 1.0
    right_scale: float = 1.0

    def validate(self) -> None:
        self.left.validate()
        self.right.validate()

    @property
    def cache_row_width(self) -> int:
        return self.left.cache_row_width

    @property
    def window(self) -> int:
        return self.left.window

    @property
    def state_shape(self) -> tuple[int, ...]:
        return self.right.state_shape

    conv_tail_shape = None

    @property
    def conv_tails(self) -> dict[str, tuple[int, int]]:       # per request slot, activation dtype
        return {"left": (max(self.left.conv - 1, 1), self.left.channels),
                "right": (max(self.right.conv - 1, 1), self.right.channels)}


@dataclass(frozen=True)
class DenseMlpSpec:
    ff: int
    activation: str = "relu2"                          # "relu2" | "gelu" | "gelu_tanh"; gated: "silu"
    kind: str = "dense"                                # key of executor.layered_decoder.FEED_FORWARDS
    gated: bool = False                                # W_down (act(W_gate h) * (W_up h)) instead of W_down act(W_up h)


@dataclass(frozen=True)
class MoeMlpSpec:
    """Routed experts ``W_down act(W_up h)`` (``gated``: ``W_down (act(W_gate h) * W_up h)``) + an optional shared one
    that every token uses.  Sigmoid router scores; the choice adds a per-expert selection bias; ``groups`` runs of
    neighbouring experts compete with the sum of their two best choice scores and only the ``keep`` best groups are
    eligible; the ``top`` winners' weights are their scores over the winners' sum, or (``renormalize=False``) the
    scores themselves.  ``weight_on_input``: an expert sees the token TIMES its weight instead of having its output
    weighted.  ``shared_gate``: the shared expert's output is scaled by one logistic number per token."""

    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0
    activation: str = "gelu"
    kind: str = "moe"
    gated: bool = False
    renormalize: bool = True
    weight_on_input: bool = False
    shared_gate: bool = False

    def validate(self) -> None:
        if self.experts < 1 or not 1 <= self.top <= self.experts or self.groups < 1 or self.experts % self.groups or \
                not 1 <= self.keep <= self.groups or self.keep * (self.experts // self.groups) < self.top:
            raise ValueError(f"unsupported expert routing: {self}")


@dataclass(frozen=True)
class LayerSpec:
    kind: str                                          # key of executor.layered_decoder.MIXERS
    mixer: "Mamba2Spec | SinkAttentionSpec | LatentAttentionSpec | MinGruSpec | RgLruSpec | SideBySideSpec"
    mlp: DenseMlpSpec | MoeMlpSpec | None = None
    weights_of: int | None = None                      # the layer whose tensors this one uses (cache / state are its own)


@dataclass(frozen=True)
class LayeredConfig:
    name: str
    hidden_size: int
    vocab_size: int
    max_seq_len: int                                   # learned position table length; 0 = bounded by the KV pool only
    rms_norm_eps: float
    layers: tuple[LayerSpec, ...] = ()
    norm_kind: str = "rms"                             # "rms" | "layer" (layer norm with a weight, no bias)
    pre_norm: bool = False                             # sublayers read norm(x) (with norms on their outputs as well)
    layer_scale: bool = False                          # per-channel scale on each sublayer's normed output
    norm_weight_offset: float = 1.0                    # 1: norm weights stored around zero; 0: plain weights
    learned_positions: bool = True
    embed_scale: float = 1.0
    logit_softcap: float = 0.0
    # parallel blocks: x <- x + mixer(norm1(x)) + ff(norm2(x)), both norms of the same x (else the sublayers follow
    # one another); embed_norm: the embedding passes the model's norm; token_side_dim > 0: after the block every layer
    # adds a gated low-rank input looked up by the token id; depth_average: the next layer (and the output) reads a
    # learned weighted sum of the embedding output and every layer result so far
    parallel_block: bool = False
    embed_norm: bool = False
    token_side_dim: int = 0
    depth_average: bool = False
    # single_norm: a parallel block with ONE input norm that both sublayers read, x <- x + mixer(h) + ff(h), h = norm1(x)
    single_norm: bool = False
    logit_scale: float = 1.0                           # the head's output times this, before the soft cap

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def attention_layers(self) -> list[int]:
        """Layers that keep rows in the KV pool (their mixer spec names the row width)."""
        return [i for i, l in enumerate(self.layers) if hasattr(l.mixer, "cache_row_width")]

    def recurrent_layers(self) -> list[int]:
        """Layers that keep a fixed-size state per request slot (their mixer spec names its shape)."""
        return [i for i, l in enumerate(self.layers) if hasattr(l.mixer, "state_shape")]

    def validate(self) -> None:
        for i, l in enumerate(self.layers):
            l.mixer.validate()
            if isinstance(l.mlp, MoeMlpSpec):
                l.mlp.validate()
            if l.weights_of is not None:
                j = l.weights_of
                if not 0 <= j < len(self.layers) or j == i or self.layers[j].weights_of is not None:
                    raise ValueError(f"layer {i} shares the weights of layer {j}, which has none of its own")
                if (self.layers[j].kind, self.layers[j].mixer, self.layers[j].mlp) != (l.kind, l.mixer, l.mlp):
                    raise ValueError(f"layer {i} shares the weights of layer {j} but differs from it")
        shared = {l.mixer.kv_heads * l.mixer.v_head_dim for l in self.layers
                  if isinstance(l.mixer, SinkAttentionSpec) and l.mixer.v_mix}
        if len(shared) > 1:
            raise ValueError(f"value-mixing layers must agree on the width of their values, got {sorted(shared)}")

    def with_(self, **kw) -> "LayeredConfig":
        return replace(self, **kw)
