"""Host side of the Tisosun design: configuration parser, registry entry, weight mapping (fused input projections,
padded attention half, fp32 decays and frequencies), cache and state geometry, interpolated rotary frequencies, and
the plain restatement's own mask and recurrences on hand-made cases."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import tisosun_oracle as O


def _config():
    other = O.attention_entry(heads=4, kv_heads=2, dim=6, vdim=5, rot_dims=6, chunk=16, softcap=0.0, base=50.0, scaling=None)
    return O.make_config([O.parallel_layer(), O.rglru_layer(), O.mingru_layer(ff=None), O.parallel_layer(other, O.decay_entry(3, 4, 5, (0.9, 1.0, 0.3)))])


def test_config_parser_reads_every_size_and_constant():
    from lite_llama_b200.executor import BlockAttentionSpec, MinGruSpec, RgLruSpec, SideBySideSpec
    from lite_llama_b200.executor.registry import lookup, names

    assert "Tisosun" in names()
    cfg = lookup("tisosun").parse_config(_config())
    cfg.validate()
    assert (cfg.hidden_size, cfg.vocab_size, cfg.rms_norm_eps, cfg.token_side_dim) == (20, 50, 1e-5, 3)
    assert cfg.parallel_block and cfg.embed_norm and cfg.depth_average and cfg.norm_weight_offset == 1.0
    assert cfg.attention_layers() == [0, 3] and cfg.recurrent_layers() == [0, 1, 2, 3]
    m = cfg.layers[0].mixer
    assert isinstance(m, SideBySideSpec) and isinstance(m.left, BlockAttentionSpec)
    L = m.left
    assert (L.heads, L.kv_heads, L.head_dim, L.v_head_dim, L.block, L.softcap, L.rot_dims, L.rot_base) == \
        (3, 1, 8, 10, 7, 15.0, 4, 10000.0)
    assert (L.rot_factor, L.rot_original, L.rot_fast, L.rot_slow, L.pairing) == (3.0, 64.0, 16.0, 1.0, "neighbours")
    assert math.isclose(L.scale, 1 / math.sqrt(8)) and m.cache_row_width == 24 and m.state_shape == (2, 8, 6)
    assert m.right.decay == (0.6, 0.97)
    L2 = cfg.layers[3].mixer.left
    assert (L2.rot_factor, L2.softcap, L2.block, L2.kv_heads) == (1.0, 0.0, 16, 2) and cfg.layers[3].mixer.cache_row_width == 24
    r = cfg.layers[1].mixer
    assert isinstance(r, RgLruSpec) and (r.width, r.blocks, r.conv, r.decay_scale) == (12, 3, 3, 8.0)
    assert r.state_shape == (12,) and r.conv_tail_shape == (2, 12)
    g = cfg.layers[2].mixer
    assert isinstance(g, MinGruSpec) and g.width == 14 and g.conv_tail_shape is None and cfg.layers[2].mlp is None
    f = cfg.layers[0].mlp
    assert f.gated and f.activation == "silu" and f.ff == 12


def test_bad_configurations_are_refused():
    from lite_llama_b200.executor.registry import lookup

    parse = lookup("Tisosun").parse_config
    raw = _config()
    raw["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        parse(raw)
    raw = _config()
    raw["layers"][1]["mixer"]["blocks"] = 5                       # 12 channels in 5 blocks
    with pytest.raises(ValueError):
        parse(raw).validate()
    raw = _config()
    raw["layers"][0]["mixer"]["right"]["decay"] = [0.5]           # two heads, one decay
    with pytest.raises(ValueError):
        parse(raw).validate()
    raw = _config()
    raw["layers"][0]["mixer"]["left"]["rot"]["dims"] = 10         # more rotated entries than the head has
    with pytest.raises(ValueError):
        parse(raw).validate()


def test_weight_mapping_fuses_the_input_projections():
    from lite_llama_b200.executor.layered_decoder import tisosun_tensor_shapes
    from lite_llama_b200.executor.registry import lookup

    arch = lookup("Tisosun")
    raw = _config()
    cfg = arch.parse_config(raw)
    w = O.random_model(raw, seed=3)
    assert {k: tuple(v.shape) for k, v in w.items()} == tisosun_tensor_shapes(cfg)
    wt = arch.map_weights(cfg, w, "cpu", torch.float32)
    assert torch.equal(wt.embed_norm, w["embed.norm"]) and wt.side_embed.shape == (50, 12) and wt.pos is None
    mix = wt.layers[0].mix
    # attention half: 24 + 8 + 10 = 42 rows padded to 48; then [values | keys | queries | gate] of the linear half
    assert mix["in"].shape == (48 + 12 + 16 + 16 + 12, 20) and mix["in_b"].shape == (104,)
    assert torch.equal(mix["in"][:24], w["l0.mix.left.q"]) and torch.equal(mix["in"][32:42], w["l0.mix.left.v"])
    assert not mix["in"][42:48].any() and not mix["in_b"][42:].any()
    assert torch.equal(mix["in_b"][24:32], w["l0.mix.left.k.b"])
    assert torch.equal(mix["in"][48:60], w["l0.mix.right.v"]) and torch.equal(mix["in"][60:76], w["l0.mix.right.k"])
    assert torch.equal(mix["in"][76:92], w["l0.mix.right.q"]) and torch.equal(mix["in"][92:], w["l0.mix.right.g"])
    assert mix["decay"].dtype == torch.float32 and mix["decay"].tolist() == [np.float32(0.6), np.float32(0.97)]
    ref_f, _ = O.yarn_frequencies(4, 10000.0, raw["layers"][0]["mixer"]["left"]["rot"]["scaling"])
    assert mix["freqs"].dtype == torch.float64 and np.allclose(mix["freqs"].numpy(), ref_f, rtol=1e-14)
    r = wt.layers[1].mix
    assert r["in"].shape == (24, 20) and torch.equal(r["in"][12:], w["l1.mix.x"]) and torch.equal(r["in_b"][:12], w["l1.mix.y.b"])
    assert r["ra"].shape == (3, 4, 4) and r["ra_b"].shape == (12,) and torch.equal(r["ri_b"][4:8], w["l1.mix.ri.b"][1])
    g = wt.layers[2].mix
    assert g["in"].shape == (42, 20) and torch.equal(g["in"][28:], w["l2.mix.g"]) and not g["in_b"][28:].any()
    assert wt.layers[2].mlp is None and wt.layers[2].pre2 is None and wt.layers[0].mlp["gate_up"].shape == (24, 20)
    assert [lw.depth.numel() for lw in wt.layers] == [2, 3, 4, 5] and wt.layers[3].side["proj"].shape == (20, 3)
    assert wt.nbytes_per_step() > 0


def test_random_initialisation_has_every_checkpoint_tensor():
    from lite_llama_b200.executor.layered_decoder import random_tisosun_tensors, tisosun_tensor_shapes
    from lite_llama_b200.executor.registry import lookup

    cfg = lookup("Tisosun").parse_config(_config())
    t = random_tisosun_tensors(cfg, seed=1)
    assert {k: tuple(v.shape) for k, v in t.items()} == tisosun_tensor_shapes(cfg)
    assert all(v.dtype == torch.bfloat16 for v in t.values())


def test_state_slots_follow_the_mixers_shapes():
    from lite_llama_b200.executor import RecurrentStateManager
    from lite_llama_b200.executor.registry import lookup

    cfg = lookup("Tisosun").parse_config(_config())
    sm = RecurrentStateManager(cfg, 3, torch.bfloat16, device="cpu")
    assert {i: tuple(t.shape) for i, t in sm.ssm_state.items()} == {0: (3, 2, 8, 6), 1: (3, 12), 2: (3, 14), 3: (3, 3, 4, 5)}
    assert {i: tuple(t.shape) for i, t in sm.conv_tail.items()} == {1: (3, 2, 12)}
    assert all(t.dtype == torch.float32 for t in sm.ssm_state.values()) and sm.conv_tail[1].dtype == torch.bfloat16
    a, b = sm.acquire(), sm.acquire()
    sm.release(a)
    assert sm.acquire() == a and sm.free_slots == 1 and b != a


def test_interpolated_frequencies():
    from lite_llama_b200.kernels.rotary_heads import rotary_frequencies

    f, mag = rotary_frequencies(8, 100.0)
    assert mag == 1.0 and np.allclose(f, [100.0 ** (-i / 4) for i in range(4)])
    # pairs that turn fast are kept, slow ones divided by the factor, and the magnitude grows with its logarithm
    f, mag = rotary_frequencies(16, 10000.0, factor=4.0, original=128.0, fast=8.0, slow=1.0)
    plain = [10000.0 ** (-i / 8) for i in range(8)]
    assert math.isclose(f[0], plain[0]) and math.isclose(f[-1], plain[-1] / 4.0) and math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    assert all(p / 4.0 - 1e-15 <= v <= p + 1e-15 for v, p in zip(f, plain))
    ref, rmag = O.yarn_frequencies(16, 10000.0, {"factor": 4.0, "original": 128, "fast": 8.0, "slow": 1.0})
    assert np.allclose(f, ref, rtol=1e-14) and math.isclose(mag, rmag)


def test_mask_and_recurrences_in_the_restatement():
    # the block mask: position 7 starts a new block of 7 and sees only itself
    m = O.attention_entry(heads=1, kv_heads=1, dim=4, vdim=4, rot_dims=0, chunk=7, scaling=None)
    rng = np.random.default_rng(0)
    w = {"q": rng.normal(size=(4, 6)), "k": rng.normal(size=(4, 6)), "v": rng.normal(size=(4, 6)), "q.b": np.zeros(4),
         "k.b": np.zeros(4), "v.b": np.zeros(4), "q.norm": np.ones(4), "k.norm": np.ones(4), "o": np.eye(4)}
    h = rng.normal(size=(9, 6))
    out = O.chunk_attention(h, list(range(9)), m, w, 1e-6)
    assert np.allclose(out[7], w["v"] @ h[7]) and np.allclose(out[0], w["v"] @ h[0])
    assert not np.allclose(out[8], w["v"] @ h[8])
    # the minimal GRU with an open update gate copies the candidate; with a closed one it keeps the state
    g = {"z": np.zeros((2, 3)), "z.b": np.array([40.0, -40.0]), "x": np.zeros((2, 3)), "x.b": np.array([1.0, 1.0]),
         "g": np.zeros((2, 3)), "o": np.eye(2)}
    g["g"][:, 0] = 1.0
    hh = np.ones((3, 3)) * 50.0                                   # silu(50) = 50
    out = O.min_gru(hh, {"width": 2}, g)
    assert np.allclose(out[:, 0], 1.5 * 50.0) and np.allclose(out[:, 1], 0.0, atol=1e-12)
    # the candidate is continuous at zero and positive below it
    g2 = dict(g, **{"x.b": np.array([-3.0, 0.0]), "z.b": np.array([40.0, 40.0])})
    out = O.min_gru(hh[:1], {"width": 2}, g2)
    assert np.allclose(out[0], [50.0 / (1 + math.exp(3.0)), 25.0])
