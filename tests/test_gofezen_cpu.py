"""Host side of the Gofezen design: configuration parser, registry, weight mapping, cache and state shapes, and the
restatement's own invariants.  No GPU."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import gofezen_oracle as O
from lite_llama_b200.executor.layered_decoder import (gofezen_tensor_shapes, map_gofezen_weights, parse_gofezen_config,
                                                      random_gofezen_tensors, wide_value_heads)
from lite_llama_b200.executor.model_config import (ConvWindowAttentionSpec, DenseMlpSpec, ForgetGateAttentionSpec, MoeMlpSpec,
                                                   WindowDeltaPairSpec)
from lite_llama_b200.executor.registry import lookup
from lite_llama_b200.executor.state_manager import RecurrentStateManager


def _config():
    left = O.left_entry(heads=4, kv_heads=2, dim=6, vdim=5, size=16, conv=2, scale=0.7)
    return O.make_config([O.hgrn2_layer(), O.pair_layer(left, O.right_entry(heads=3, kv_heads=3, dim=5, vdim=3, conv=4), 1.3, 0.4),
                          O.hgrn2_layer(heads=3, dim=5, vdim=4, mlp=None), O.pair_layer(mlp=O.moe_mlp(3, 3, 4, 0))],
                         width=24, vocab=50, embed_scale=3.0, logit_scale=0.7, softcap=12.0, max_positions=99)


def test_every_size_and_constant_comes_from_the_configuration():
    arch = lookup("gofezen")
    cfg = arch.parse_config(_config())
    cfg.validate()
    assert (cfg.hidden_size, cfg.vocab_size, cfg.max_seq_len, cfg.embed_scale, cfg.logit_scale, cfg.logit_softcap) == \
        (24, 50, 99, 3.0, 0.7, 12.0)
    assert cfg.single_norm and cfg.parallel_block and cfg.norm_weight_offset == 0.0 and cfg.rms_norm_eps == 1e-5
    assert [l.kind for l in cfg.layers] == ["forget_gate", "window_delta", "forget_gate", "window_delta"]
    a, b = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert isinstance(a, ForgetGateAttentionSpec) and a.state_shape == (2, 4, 6)
    assert isinstance(b, WindowDeltaPairSpec) and (b.left_scale, b.right_scale, b.window) == (1.3, 0.4, 16)
    assert b.left.channels == 4 * 6 + 2 * (6 + 5) and b.cache_row_width == 24 and b.state_shape == (3, 5, 3)
    assert b.conv_tails == {"left": (1, 46), "right": (3, 2 * 15 + 9)}
    assert isinstance(cfg.layers[0].mlp, DenseMlpSpec) and cfg.layers[0].mlp.gated and cfg.layers[2].mlp is None
    moe = cfg.layers[1].mlp
    assert isinstance(moe, MoeMlpSpec) and (moe.experts, moe.top, moe.ff, moe.shared_ff) == (5, 2, 6, 7)
    assert moe.gated and moe.weight_on_input and moe.shared_gate and not moe.renormalize
    assert cfg.layers[3].mlp.shared_ff == 0 and not cfg.layers[3].mlp.shared_gate
    assert cfg.attention_layers() == [1, 3] and cfg.recurrent_layers() == [0, 1, 2, 3]


def test_unknown_layers_and_feed_forwards_are_refused():
    raw = _config()
    raw["layers"][0]["type"] = "lstm"
    with pytest.raises(ValueError):
        parse_gofezen_config(raw)
    raw = _config()
    raw["layers"][0]["mlp"]["kind"] = "maxout"
    with pytest.raises(ValueError):
        parse_gofezen_config(raw)
    raw = _config()
    raw["layers"][1]["mixer"]["left"]["kv_heads"] = 3                 # 4 heads on 3 kv heads
    with pytest.raises(ValueError):
        parse_gofezen_config(raw).validate()


def test_weight_mapping_fuses_the_input_projections_and_stacks_the_experts():
    raw = _config()
    cfg = parse_gofezen_config(raw)
    tensors = O.random_model(raw, seed=3)
    assert {k: tuple(v.shape) for k, v in tensors.items()} == gofezen_tensor_shapes(cfg)
    assert set(random_gofezen_tensors(cfg)) == set(tensors)
    w = map_gofezen_weights(cfg, tensors, "cpu", torch.float32)
    a = w.layers[0].mix
    assert a["in"].shape == (2 * 8 + 12, 24) and torch.equal(a["in"][8:16], tensors["l0.mix.f"])
    assert torch.equal(a["in_b"][8:16], tensors["l0.mix.f.b"]) and a["in_b"][:8].abs().sum() == 0
    b, m = w.layers[1].mix, cfg.layers[1].mixer
    r0 = -(-m.left.channels // 8) * 8
    g0 = r0 + -(-(m.right.channels + 2 * m.right.heads) // 8) * 8
    assert b["in"].shape[0] == g0 + -(-m.right.heads * m.right.v_head_dim // 8) * 8
    assert torch.equal(b["in"][24:36], tensors["l1.mix.left.k"]) and torch.equal(b["in"][r0:r0 + 15], tensors["l1.mix.right.q"])
    assert torch.equal(b["in"][r0 + m.right.channels:r0 + m.right.channels + 3], tensors["l1.mix.right.b"])
    assert torch.equal(b["in"][g0:g0 + 9], tensors["l1.mix.right.g"]) and b["in"][m.left.channels:r0].abs().sum() == 0
    assert torch.equal(b["left_conv"][24:36], tensors["l1.mix.left.k.conv"]) and b["right_conv"].shape == (39, 4)
    assert torch.equal(b["in_b"][:24], tensors["l1.mix.left.q.b"]) and b["in_b"][r0:].abs().sum() == 0
    moe = w.layers[1].mlp
    assert moe["gate_up"].shape == (5, 12, 24) and torch.equal(moe["gate_up"][2, 6:], tensors["l1.mlp.e2.up"])
    assert moe["down"].shape == (5, 24, 6) and moe["shared_gate_up"].shape == (16, 24)
    assert torch.equal(moe["shared_gate_up"][14], tensors["l1.mlp.shared.sg"][0]) and moe["shared_gate_up"][15].abs().sum() == 0
    assert "shared_gate_up" not in w.layers[3].mlp and w.layers[2].mlp is None
    assert torch.equal(w.layers[0].mlp["gate_up"][14:], tensors["l0.mlp.up"])


def test_state_slots_hold_a_memory_and_one_tail_per_convolution():
    cfg = parse_gofezen_config(_config())
    st = RecurrentStateManager(cfg, 3, torch.bfloat16, device="cpu")
    assert st.ssm_state[0].shape == (3, 2, 4, 6) and st.ssm_state[1].shape == (3, 3, 5, 3)
    assert st.named_tail[1]["left"].shape == (3, 1, 46) and st.named_tail[1]["right"].shape == (3, 3, 39)
    assert 0 not in st.named_tail and not st.conv_tail and st.ssm_state[0].dtype == torch.float32
    assert st.nbytes() > 0


def test_value_heads_read_side_by_side_fit_the_attention_kernels():
    spec = lambda kv, vdim, dim=64: ConvWindowAttentionSpec(heads=kv * 2, kv_heads=kv, head_dim=dim, v_head_dim=vdim, scale=1.0)
    assert wide_value_heads(spec(2, 64), True) == 2 and wide_value_heads(spec(4, 64), True) == 2
    assert wide_value_heads(spec(4, 64), False) == 4 and wide_value_heads(spec(3, 64), True) == 1
    assert wide_value_heads(spec(8, 16), True) == 8 and wide_value_heads(spec(2, 144), True) == 1
    assert wide_value_heads(spec(6, 40, dim=20), True) == 6           # odd head size: the CUDA-core kernel's 256 columns


def test_restatement_mixing_heads_by_the_identity_is_plain_attention_and_the_window_counts_the_token_itself():
    m = O.left_entry(heads=2, kv_heads=1, dim=4, vdim=3, size=3, conv=1, scale=0.5)
    g = np.random.default_rng(0)
    cols = 2 * 4 + 4 + 3
    h = g.standard_normal((9, cols))
    eye = lambda a, b: np.eye(cols)[a:b]
    w = {"q": eye(0, 8), "k": eye(8, 12), "v": eye(12, 15), "q.b": np.zeros(8), "k.b": np.zeros(4), "v.b": np.zeros(3),
         "q.conv": np.ones((8, 1)), "k.conv": np.ones((4, 1)), "v.conv": np.ones((3, 1)), "talk": np.eye(2), "o": np.eye(6)}
    out = O.window_attention(h, m, w, 1e-6)
    t = 8
    q = O.unit_rms(h[t, 4:8], 1e-6)
    sc = np.array([q @ O.unit_rms(h[j, 8:12], 1e-6) for j in (6, 7, 8)]) * 0.5       # itself and the two before it
    p = np.exp(sc - sc.max()) / np.exp(sc - sc.max()).sum()
    assert np.allclose(out[t, 3:], p @ h[6:9, 12:15])
    w["talk"] = np.array([[0.0, 1.0], [1.0, 0.0]])                                    # the heads trade their weights
    assert np.allclose(O.window_attention(h, m, w, 1e-6)[t, :3], out[t, 3:])


def test_restatement_delta_rule_overwrites_what_a_key_held():
    """With full write strength and no decay, writing twice under one unit key leaves the second value only."""
    S = np.zeros((3, 2))
    k = np.array([0.6, 0.8, 0.0])
    for v in (np.array([1.0, 2.0]), np.array([-3.0, 5.0])):
        S = S + np.outer(k, 1.0 * (v - S.T @ k))
    assert np.allclose(S.T @ k, [-3.0, 5.0])
