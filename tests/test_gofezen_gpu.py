"""The Gofezen path on the GPU against the plain restatement in ``gofezen_oracle`` (float64, token loops): every
mechanism alone through its kernels, then whole models through ``ModelRunner.forward_ragged`` and the engine -- whole
prompts against token-by-token decoding, portions down to two tokens, unequal batches against each request alone,
pool rows and slots that change hands, keys just inside and just outside the window in prompts and in decoding, the
first tokens, long decoding, sizes that differ from one another.  fp32 runs are held to 1e-4 of the logits' spread;
bf16 runs to a few bf16 roundings."""

from __future__ import annotations

import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import gofezen_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]
DEV = "cuda"


def _i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def _close(got, ref, tol):
    got = got.double().cpu()
    ref = torch.as_tensor(np.asarray(ref)).double()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = (got - ref).abs().max().item()
    spread = max(ref.abs().max().item(), 1e-6)
    assert err <= tol * spread, f"max abs err {err:.3e} on values up to {spread:.3e} (tol {tol})"


def _ragged(seqs):
    """``seqs = [(new tokens, cached tokens, slot)]`` -> (seq_start, seq_ctx, seq_slot) on the device."""
    starts = [0]
    for n, _, _ in seqs:
        starts.append(starts[-1] + n)
    return _i32(starts), _i32(c for _, c, _ in seqs), _i32(s for _, _, s in seqs)


def _select(rows_of, width):
    """A projection matrix that picks the given input columns (so a mixer of the restatement reads raw columns)."""
    m = np.zeros((len(rows_of), width))
    for r, c in enumerate(rows_of):
        m[r, c] = 1.0
    return m


PLAN = [[(0, 0, 40), (1, 0, 9)], [(1, 9, 11), (0, 40, 110)], [(0, 110, 111)], [(0, 111, 113), (1, 11, 12)],
        [(1, 12, 50), (0, 113, 114)], [(0, 114, 130)]]          # (sequence, from, to) per step: portions and single tokens


# ------------------------------------------------------------------------------------------- mechanisms alone #
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 8, 6), (4, 32, 96), (1, 5, 1), (3, 24, 40), (2, 80, 72), (1, 200, 16),
                                            (2, 128, 130)])
def test_forget_gate_memory_over_portions_and_single_tokens(dtype, tol, heads, dim, vdim):
    from lite_llama_b200.kernels import gated_linear_scan, head_norm_gate

    n, nv = heads * dim, heads * vdim
    cols = 2 * n + nv
    g = torch.Generator().manual_seed(dim + vdim)
    xs = [(1.5 * torch.randn(L, cols, generator=g)).to(dtype) for L in (130, 50)]
    low = (0.9 * torch.rand(n, generator=g)).to(dtype)
    nw = (1 + 0.2 * torch.randn(vdim, generator=g)).to(dtype)
    w = {"q": _select(range(0, n), cols), "f": _select(range(n, 2 * n), cols), "f.b": np.zeros(n),
         "v": _select(range(2 * n, cols), cols), "lower": O.f64(low), "norm": O.f64(nw), "o": np.eye(nv)}
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    refs = [O.hgrn2(O.f64(x), m, w, 1e-5) for x in xs]
    state = torch.full((3, heads, dim, vdim), 4.0, device=DEV)       # stale contents: a new sequence never reads them
    got = {0: [], 1: []}
    for step in PLAN:
        part = torch.cat([xs[i][a:b] for i, a, b in step]).to(DEV)
        meta = _ragged([(b - a, a, i + 1) for i, a, b in step])
        y = gated_linear_scan("forget_gate", state, part[:, :n], part[:, n:2 * n], part[:, 2 * n:], *meta, heads, heads,
                              dim, vdim, c0=low.to(DEV))
        out = head_norm_gate(y, nw.to(DEV), heads, 1e-5)
        at = 0
        for i, a, b in step:
            got[i].append(out[at:at + b - a])
            at += b - a
    for i in (0, 1):
        _close(torch.cat(got[i]), refs[i], tol)
    assert (state[0] == 4.0).all()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("heads,qk,dim,vdim,taps", [(2, 1, 8, 6, 2), (4, 2, 32, 48, 4), (1, 1, 5, 1, 1), (3, 3, 24, 40, 3),
                                                    (6, 2, 64, 72, 5), (1, 1, 200, 16, 2), (2, 2, 128, 128, 4)])
def test_delta_rule_with_its_convolution_gates_and_output_norm(dtype, tol, heads, qk, dim, vdim, taps):
    from lite_llama_b200.kernels import causal_conv_silu, gated_linear_scan, head_norm_gate

    nq, nv = qk * dim, heads * vdim
    conv_cols = 2 * nq + nv
    cols = conv_cols + 2 * heads + nv                              # q | k | v | write logits | decay logits | gate
    g = torch.Generator().manual_seed(dim + vdim + taps)
    xs = [torch.randn(L, cols, generator=g).to(dtype) for L in (130, 50)]
    cw = (0.5 * torch.randn(conv_cols, taps, generator=g)).to(dtype)
    a_log = (-1 + 0.8 * torch.randn(heads, generator=g)).to(dtype)
    dtb = (-1 + 0.8 * torch.randn(heads, generator=g)).to(dtype)
    nw = (1 + 0.2 * torch.randn(vdim, generator=g)).to(dtype)
    sel = lambda a, b: _select(range(a, b), cols)
    w = {"q": sel(0, nq), "k": sel(nq, 2 * nq), "v": sel(2 * nq, conv_cols), "q.conv": O.f64(cw[:nq]),
         "k.conv": O.f64(cw[nq:2 * nq]), "v.conv": O.f64(cw[2 * nq:]), "b": sel(conv_cols, conv_cols + heads),
         "a": sel(conv_cols + heads, conv_cols + 2 * heads), "g": sel(conv_cols + 2 * heads, cols), "A_log": O.f64(a_log),
         "dt_bias": O.f64(dtb), "norm": O.f64(nw), "o": np.eye(nv)}
    m = {"heads": heads, "kv_heads": qk, "dim": dim, "vdim": vdim, "conv": taps}
    refs = [O.gated_delta(O.f64(x), m, w, 1e-5) for x in xs]
    state = torch.full((3, heads, dim, vdim), -3.0, device=DEV)
    tail = torch.full((3, max(taps - 1, 1), conv_cols), 9.0, dtype=dtype, device=DEV)
    zero_b = torch.zeros(conv_cols, dtype=dtype, device=DEV)
    got = {0: [], 1: []}
    for step in PLAN:
        part = torch.cat([xs[i][a:b] for i, a, b in step]).to(DEV)
        meta = _ragged([(b - a, a, i + 1) for i, a, b in step])
        qkv = causal_conv_silu(part, 0, conv_cols, cw.to(DEV), zero_b, tail, *meta)
        y = gated_linear_scan("delta_rule", state, qkv[:, :nq], qkv[:, nq:2 * nq], qkv[:, 2 * nq:], *meta, heads, qk, dim,
                              vdim, c0=dtb.to(DEV), c1=a_log.to(DEV), p0=part[:, conv_cols:conv_cols + heads],
                              p1=part[:, conv_cols + heads:conv_cols + 2 * heads], q_scale=dim ** -0.5, unit_eps=1e-6)
        out = head_norm_gate(y, nw.to(DEV), heads, 1e-5, part[:, conv_cols + 2 * heads:])
        at = 0
        for i, a, b in step:
            got[i].append(out[at:at + b - a])
            at += b - a
    for i in (0, 1):
        _close(torch.cat(got[i]), refs[i], tol)
    assert (state[0] == -3.0).all()


def _attention_case(m, seqs_plan, dtype, x_by_seq, talk, conv_w):
    """Run ``conv_window_attention`` over a step plan on raw [q | k | v] columns; returns per-sequence outputs."""
    from lite_llama_b200.executor.layered_decoder import StepContext, conv_window_attention
    from lite_llama_b200.executor.model_config import ConvWindowAttentionSpec
    from lite_llama_b200.executor.ragged_batch import RaggedBatch

    spec = ConvWindowAttentionSpec(heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                   scale=m["scale"], window=m["mask"]["size"], conv=m["conv"])
    nseq, longest = len(x_by_seq), max(x.shape[0] for x in x_by_seq)
    pool = torch.full((nseq * longest + 7, spec.cache_row_width), 5.0, dtype=dtype, device=DEV)
    table = torch.zeros((nseq + 1, longest), dtype=torch.int32, device=DEV)
    tails = {0: {"left": torch.full((nseq + 1, max(spec.conv - 1, 1), spec.channels), 7.0, dtype=dtype, device=DEV)}}
    w = {"left_conv": conv_w.to(dtype).to(DEV), "left_conv_b": torch.zeros(spec.channels, dtype=dtype, device=DEV),
         "ones": torch.ones(spec.head_dim, dtype=dtype, device=DEV), "talk": talk.to(dtype).to(DEV),
         "left_o": torch.eye(spec.heads * spec.v_head_dim, dtype=dtype, device=DEV)}
    free = list(range(pool.shape[0]))
    random.Random(3).shuffle(free)                                 # rows in no particular order
    got = {i: [] for i in range(nseq)}
    for step in seqs_plan:
        lens, ctxs, slots, rows = [], [], [], []
        for i, a, b in step:
            lens.append(b - a); ctxs.append(a); slots.append(i + 1)
            mine = [free.pop() for _ in range(b - a)]
            table[i + 1, a:b] = _i32(mine)
            rows += mine
        batch = RaggedBatch.build(lens, ctxs, slots, _i32(rows), DEV)
        ctx = StepContext(batch, {0: pool}, table, SimpleNamespace(named_tail=tails))
        part = torch.cat([x_by_seq[i][a:b] for i, a, b in step]).to(dtype).to(DEV)
        out = conv_window_attention(0, spec, w, part, ctx, 1e-5)
        at = 0
        for i, a, b in step:
            got[i].append(out[at:at + b - a])
            at += b - a
    return [torch.cat(got[i]) for i in range(nseq)]


def _attention_weights(m, cols, talk, conv_w):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    nq, nk = H * D, G * D
    return {"q": _select(range(0, nq), cols), "k": _select(range(nq, nq + nk), cols), "v": _select(range(nq + nk, cols), cols),
            "q.b": np.zeros(nq), "k.b": np.zeros(nk), "v.b": np.zeros(G * V), "q.conv": O.f64(conv_w[:nq]),
            "k.conv": O.f64(conv_w[nq:nq + nk]), "v.conv": O.f64(conv_w[nq + nk:]), "talk": O.f64(talk),
            "o": np.eye(H * V)}


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", [dict(heads=3, kv_heads=1, dim=6, vdim=5, size=9, conv=3),
                                  dict(heads=4, kv_heads=2, dim=64, vdim=32, size=70, conv=3),
                                  dict(heads=8, kv_heads=4, dim=32, vdim=64, size=33, conv=2),     # two calls of two value heads
                                  dict(heads=2, kv_heads=2, dim=16, vdim=144, size=128, conv=4),   # one value head per call
                                  dict(heads=6, kv_heads=1, dim=8, vdim=8, size=1, conv=1),
                                  dict(heads=8, kv_heads=2, dim=16, vdim=24, size=20, conv=2),     # four heads per kv head
                                  dict(heads=8, kv_heads=1, dim=8, vdim=16, size=40, conv=1),      # eight
                                  dict(heads=2, kv_heads=1, dim=40, vdim=24, size=1000, conv=5)])
def test_convolved_window_attention_with_mixed_heads_in_portions_and_single_tokens(dtype, tol, geom):
    m = O.left_entry(scale=2.0 / geom["dim"] ** 0.5, **geom)        # scores of a few units: a pointed softmax
    cols = m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"])
    g = torch.Generator().manual_seed(geom["dim"])
    xs = [torch.randn(L, cols, generator=g).to(dtype).float() for L in (130, 50)]
    talk = (0.4 * torch.randn(m["heads"], m["heads"], generator=g) + torch.eye(m["heads"])).to(dtype).float()
    cw = (0.6 * torch.randn(cols, m["conv"], generator=g)).to(dtype).float()
    refs = [O.window_attention(O.f64(x), m, _attention_weights(m, cols, talk, cw), 1e-5) for x in xs]
    got = _attention_case(m, PLAN, dtype, xs, talk, cw)
    for i in (0, 1):
        _close(got[i], refs[i], tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("geom", [dict(heads=8, kv_heads=4, dim=32, vdim=64, size=33, conv=2),
                                  dict(heads=4, kv_heads=2, dim=16, vdim=144, size=50, conv=1),    # fp32 lanes pass twice
                                  dict(heads=5, kv_heads=1, dim=7, vdim=3, size=300, conv=3)])
def test_single_tokens_with_mixed_outputs_instead_of_mixed_weights(monkeypatch, dtype, tol, geom):
    """Steps of single tokens mix the heads' WEIGHTS (two launches); a window too long for that falls back to weighing
    every value head and mixing the outputs.  Both are the same sum: the fallback is forced here."""
    import lite_llama_b200.executor.layered_decoder as LD
    m = O.left_entry(scale=2.0 / geom["dim"] ** 0.5, **geom)
    cols = m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"])
    g = torch.Generator().manual_seed(geom["vdim"])
    xs = [torch.randn(L, cols, generator=g).to(dtype).float() for L in (130, 50)]
    talk = (0.4 * torch.randn(m["heads"], m["heads"], generator=g) + torch.eye(m["heads"])).to(dtype).float()
    cw = (0.6 * torch.randn(cols, m["conv"], generator=g)).to(dtype).float()
    refs = [O.window_attention(O.f64(x), m, _attention_weights(m, cols, talk, cw), 1e-5) for x in xs]
    direct = _attention_case(m, PLAN, dtype, xs, talk, cw)
    monkeypatch.setattr(LD, "MIXED_HEAD_MAX_KEYS", 0)
    fallback = _attention_case(m, PLAN, dtype, xs, talk, cw)
    for i in (0, 1):
        _close(direct[i], refs[i], tol)
        _close(fallback[i], refs[i], tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("new", [1, 2, 40])
@pytest.mark.parametrize("size", [1, 7, 64, 65, 130, 200])
def test_a_key_at_the_window_edge_is_seen_and_the_one_before_it_is_not(dtype, new, size):
    """One key is made to stand out for the last query (aligned with it, everything else orthogonal noise): at distance
    ``size - 1`` its value fills the output, at distance ``size`` it leaves no trace.  The last token comes in a
    portion of ``new`` tokens after a cached prefix."""
    m = O.left_entry(heads=2, kv_heads=1, dim=16, vdim=8, size=size, conv=1, scale=40.0)
    H, D, V = 2, 16, 8
    cols = H * D + D + V
    total = 260
    talk, cw = torch.eye(H), torch.ones(cols, 1)
    for dist, seen in ((size - 1, True), (size, False)):
        g = torch.Generator().manual_seed(size)
        x = 0.05 * torch.randn(total, cols, generator=g)
        x[:, H * D + D:] = 0.0                                      # all values zero ...
        mark = total - 1 - dist
        x[total - 1, :H * D] = 0.0
        x[total - 1, 0] = x[total - 1, D] = 1.0                     # both query heads point along channel 0
        x[:, H * D] = 0.0                                           # no other key has any of channel 0
        x[mark, H * D:H * D + D] = 0.0
        x[mark, H * D] = 1.0
        x[mark, H * D + D:] = 1.0                                   # ... except the marked key's
        if dist == 0:
            x[mark, 0] = x[mark, D] = 1.0
        x = x.to(dtype).float()
        plan = [[(0, 0, total - new)], [(0, total - new, total)]]
        got = _attention_case(m, plan, dtype, [x], talk, cw)[0][-1].float().cpu()
        ref = O.window_attention(O.f64(x), m, _attention_weights(m, cols, talk, cw), 1e-5)[-1]
        assert abs(float(ref.mean()) - (1.0 if seen else 0.0)) < 0.05
        assert abs(got.mean().item() - (1.0 if seen else 0.0)) < 0.05


def _moe_weights(cfg_mlp, width, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    r = cfg_mlp["router"]
    w = {"router": 3.0 * torch.randn(r["experts"], width, generator=g) / width ** 0.5}
    f = cfg_mlp["expert"]["ff"]
    for e in range(r["experts"]):
        w[f"e{e}.gate"] = torch.randn(f, width, generator=g) / width ** 0.5
        w[f"e{e}.up"] = torch.randn(f, width, generator=g) / width ** 0.5
        w[f"e{e}.down"] = torch.randn(width, f, generator=g) / f ** 0.5
    if cfg_mlp.get("shared"):
        s = cfg_mlp["shared"]["ff"]
        w.update({"shared.gate": torch.randn(s, width, generator=g) / width ** 0.5,
                  "shared.up": torch.randn(s, width, generator=g) / width ** 0.5,
                  "shared.down": torch.randn(width, s, generator=g) / s ** 0.5,
                  "shared.sg": torch.randn(1, width, generator=g) / width ** 0.5})
    return {k: v.to(dtype).float() for k, v in w.items()}


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("experts,top,ff,shared,width", [(5, 2, 6, 7, 24), (10, 1, 80, 112, 192), (1, 1, 8, 0, 16),
                                                         (7, 7, 5, 3, 20), (16, 4, 64, 64, 128)])
def test_routed_gated_experts_weigh_their_input_with_unnormalised_scores(dtype, tol, experts, top, ff, shared, width):
    from lite_llama_b200.executor.layered_decoder import _gofezen_mlp, map_gofezen_weights, moe_feed_forward, parse_gofezen_config

    mlp = O.moe_mlp(experts, top, ff, shared)
    cfg = O.make_config([O.hgrn2_layer(mlp=mlp)], width=width)
    w = _moe_weights(mlp, width, experts * 10 + top, dtype)
    g = torch.Generator().manual_seed(1)
    x = (1.5 * torch.randn(70, width, generator=g)).to(dtype).float()
    scores = O.logistic(O.f64(x) @ O.f64(w["router"]).T)
    keep = [t for t in range(70) if experts == top or
            np.sort(scores[t])[::-1][top - 1] - np.sort(scores[t])[::-1][min(top, experts - 1)] > 0.02]   # no close calls
    x = x[keep]
    ref = O.routed_ff(O.f64(x), mlp, {k: O.f64(v) for k, v in w.items()})
    tensors = O.random_model(cfg, 0)
    tensors.update({f"l0.mlp.{k}": v for k, v in w.items()})
    conf = parse_gofezen_config(cfg)
    lw = map_gofezen_weights(conf, tensors, DEV, dtype).layers[0].mlp
    got = moe_feed_forward(_gofezen_mlp(mlp), lw, x.to(dtype).to(DEV))
    _close(got, ref, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("n", [44, 256, 1100])
def test_scaled_branches_join_the_residual_and_hand_out_the_next_norm(dtype, tol, n):
    from lite_llama_b200.kernels import branch_sum_residual, softcap_to_f32

    T, eps = 6, 1e-4
    r0 = 3 * torch.randn(T, n)
    a, b, c = (torch.randn(T, n + 8).to(dtype) for _ in range(3))
    wn = (1 + 0.3 * torch.randn(n)).to(dtype)
    r = r0.clone().to(DEV)
    act = branch_sum_residual(r, a.to(DEV)[:, :n], None, b.to(DEV)[:, 4:n + 4], None, c.to(DEV)[:, 8:], eps, 0.7,
                              want_act=False, scale_b=1.3, next_weight=wn.to(DEV))
    ref = O.f64(r0) + 0.7 * O.f64(a)[:, :n] + 1.3 * O.f64(b)[:, 4:n + 4] + O.f64(c)[:, 8:]
    _close(r, ref, 3e-6)
    _close(act, np.stack([O.unit_rms(x, eps) for x in ref]) * O.f64(wn), tol)
    r = r0.clone().to(DEV)
    assert branch_sum_residual(r, a.to(DEV)[:, :n], None, None, None, None, eps, 1.0, want_act=False) is None
    _close(r, O.f64(r0) + O.f64(a)[:, :n], 3e-6)
    z = torch.randn(5, 33).to(dtype)
    _close(softcap_to_f32(z.to(DEV), 12.0, 0.75), 12.0 * np.tanh(0.75 * O.f64(z) / 12.0), 3e-6)
    _close(softcap_to_f32(z.to(DEV), 0.0, 0.25), 0.25 * O.f64(z), 3e-6)


# ------------------------------------------------------------------------------------------------- whole models #
def _small():
    # nothing a multiple of 8, three query heads on one kv head, a window shorter than a portion, two experts per token
    other = O.left_entry(heads=4, kv_heads=2, dim=6, vdim=5, size=16, conv=2, scale=0.7)
    return O.make_config([O.hgrn2_layer(), O.pair_layer(), O.hgrn2_layer(heads=3, dim=5, vdim=4, mlp=O.moe_mlp(4, 1, 5, 0)),
                          O.pair_layer(other, O.right_entry(heads=3, kv_heads=3, dim=5, vdim=3, conv=4), 1.3, 0.4, mlp=None),
                          O.hgrn2_layer(mlp=O.moe_mlp(3, 3, 4, 6))])


def _aligned():
    # sizes in steps of 8: the tensor-core tiles in bf16; a window longer than a 64-key tile, one of exactly two tiles
    a = O.left_entry(heads=6, kv_heads=1, dim=32, vdim=24, size=70, conv=3, scale=0.25)
    b = O.left_entry(heads=4, kv_heads=2, dim=64, vdim=64, size=128, conv=4, scale=0.11)
    return O.make_config([O.pair_layer(a, O.right_entry(heads=4, kv_heads=2, dim=32, vdim=16, conv=4), mlp=O.moe_mlp(8, 2, 32, 48)),
                          O.hgrn2_layer(heads=2, dim=32, vdim=64, mlp=O.dense_mlp(96)),
                          O.hgrn2_layer(heads=4, dim=16, vdim=16, mlp=O.moe_mlp(6, 1, 24, 16)),
                          O.pair_layer(b, O.right_entry(heads=2, kv_heads=1, dim=64, vdim=32, conv=2), 0.5, 1.1, mlp=O.dense_mlp(64))],
                         width=64, vocab=128)


def _ones():
    # one head, one expert, one tap, a window of one position, sizes of one
    a = O.left_entry(heads=1, kv_heads=1, dim=4, vdim=1, size=1, conv=1, scale=1.0)
    b = O.left_entry(heads=2, kv_heads=2, dim=2, vdim=3, size=2, conv=1, scale=1.0)
    return O.make_config([O.pair_layer(a, O.right_entry(1, 1, 1, 1, 1), 1.0, 1.0, mlp=O.moe_mlp(1, 1, 1, 1)),
                          O.hgrn2_layer(heads=1, dim=1, vdim=1, mlp=None),
                          O.pair_layer(b, O.right_entry(1, 1, 3, 2, 1), 2.0, 0.0, mlp=O.dense_mlp(5))],
                         width=10, vocab=17, embed_scale=1.0, logit_scale=1.0, softcap=0.0)


CONFIGS = {"small": _small, "aligned": _aligned, "ones": _ones}


def _runner(cfg, w, dtype=torch.float32, max_tokens=512, max_requests=4):
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.registry import lookup

    arch = lookup(cfg["architecture"])
    conf = arch.parse_config(cfg)
    return ModelRunner(conf, arch.map_weights(conf, w, DEV, dtype), max_tokens, device=DEV, dtype=dtype,
                       max_requests=max_requests)


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _feed(runner, req, toks, cuts):
    """Feed ``toks`` in portions of the given sizes (the rest one by one); logits of every position."""
    out, at = [], 0
    for n in list(cuts) + [1] * len(toks):
        if at >= len(toks):
            break
        part = toks[at:at + n]
        out.append(runner.forward_ragged([(req, part)], list(range(len(part)))))
        at += len(part)
    return torch.cat(out)


@pytest.mark.parametrize("name,length", [("small", 45), ("aligned", 150), ("ones", 20)])
def test_whole_prompt_portions_and_decoding_agree_with_the_restatement(name, length):
    cfg = CONFIGS[name]()
    w = O.random_model(cfg, seed=1)
    toks = _tokens(cfg, length, 2)
    ref = O.forward(cfg, w, toks)
    runner = _runner(cfg, w)
    for cuts in ([length], [length - 15], [], [2, 2, 3, 17, 2, 5], [1, length - 1], [7, 1, 1, 20], [64, 2, 63]):
        req = runner.open_request()
        _close(_feed(runner, req, toks, cuts), ref, 1e-4)
        runner.close_request(req)
    assert runner.kv_cache_manager.can_use_mem_size == runner.kv_cache_manager.max_num_tokens
    assert runner.state_manager.free_slots == 4


@pytest.mark.parametrize("layers", ["recurrent_only", "pairs_only"])
def test_models_without_a_cache_or_with_nothing_else(layers):
    if layers == "recurrent_only":
        cfg = O.make_config([O.hgrn2_layer(), O.hgrn2_layer(mlp=None), O.hgrn2_layer(heads=1, dim=7, vdim=3)])
    else:
        cfg = O.make_config([O.pair_layer(mlp=None), O.pair_layer(O.left_entry(size=1000))])
    w = O.random_model(cfg, seed=15)
    toks = _tokens(cfg, 50, 4)
    ref = O.forward(cfg, w, toks)
    runner = _runner(cfg, w, max_tokens=64)
    req = runner.open_request()
    _close(_feed(runner, req, toks, [20, 2]), ref, 1e-4)
    runner.close_request(req)
    assert runner.kv_cache_manager.can_use_mem_size == 64


def test_layer_results_match_one_by_one():
    cfg = CONFIGS["small"]()
    w = O.random_model(cfg, seed=5)
    toks = _tokens(cfg, 12, 6)
    _, layers = O.forward(cfg, w, toks, return_layers=True)
    runner = _runner(cfg, w)
    runner.model.layer_trace = []
    runner.forward_ragged([(runner.open_request(), toks)])
    assert len(runner.model.layer_trace) == len(layers) == 5
    for got, ref in zip(runner.model.layer_trace, layers):
        _close(got, ref, 2e-5)


def test_unequal_batches_match_each_request_alone_and_reuse_rows_and_slots():
    """Six requests through four slots and a pool smaller than their sum: portions beside single tokens, requests
    leaving and joining, rows and slots changing hands; every logit equals the request's own restatement."""
    cfg = CONFIGS["small"]()
    w = O.random_model(cfg, seed=7)
    lens = [40, 3, 25, 1, 31, 18]
    toks = [_tokens(cfg, n, 10 + i) for i, n in enumerate(lens)]
    refs = [O.forward(cfg, w, t) for t in toks]
    runner = _runner(cfg, w, max_tokens=96, max_requests=4)
    plan = {0: [5, 2, 1, 1, 9, 1, 1, 1, 1, 1, 1, 16], 1: [2, 1], 2: [1, 1, 20, 1, 1, 1], 3: [1],
            4: [16, 2, 2, 1, 1, 1, 1, 1, 6], 5: [3, 3, 3, 3, 3, 3]}
    waiting, live, fed, got = [0, 1, 2, 3, 4, 5], {}, {i: 0 for i in plan}, {i: [] for i in plan}
    steps, seen_rows, seen_slots = 0, set(), []
    while waiting or live:
        while waiting and len(live) < 4 and runner.kv_cache_manager.can_use_mem_size >= sum(
                lens[i] - fed[i] for i in live) + lens[waiting[0]]:
            live[waiting.pop(0)] = runner.open_request()
            seen_slots.append(live[max(live)].slot)
        order = sorted(live, key=lambda i: (i * 7 + steps) % 5)               # the batch order changes every step
        entries, want, at, shape = [], [], 0, []
        for i in order:
            n = plan[i].pop(0) if plan[i] else 1
            n = min(n, lens[i] - fed[i])
            entries.append((live[i], toks[i][fed[i]:fed[i] + n]))
            want += list(range(at, at + n))
            at += n
            shape.append((i, n))
        logits = runner.forward_ragged(entries, want)
        at = 0
        for i, n in shape:
            got[i].append(logits[at:at + n])
            at += n
            fed[i] += n
            if fed[i] == lens[i]:
                seen_rows.update(live[i].rows)
                runner.close_request(live.pop(i))
        steps += 1
    for i in plan:
        _close(torch.cat(got[i]), refs[i], 1e-4)
    assert runner.kv_cache_manager.can_use_mem_size == 96 and sum(lens) > 96 >= len(seen_rows)
    assert len(seen_slots) == 6 and len(set(seen_slots)) <= 4                # state slots changed hands too


def test_long_decoding_passes_the_window_and_key_range_edges():
    """320 tokens decoded one by one after a prompt of 100: windows of 150 (one and two key ranges of the single-token
    kernel) and of 33 pass over decoded tokens; a request longer than the pool keeps running because every cached
    layer has a window and unseen rows go back."""
    a = O.left_entry(heads=2, kv_heads=1, dim=8, vdim=8, size=150, conv=3, scale=0.5)
    b = O.left_entry(heads=2, kv_heads=2, dim=8, vdim=4, size=33, conv=2, scale=0.5)
    cfg = O.make_config([O.pair_layer(a, O.right_entry(2, 1, 8, 8, 3), mlp=None), O.hgrn2_layer(heads=2, dim=8, vdim=8),
                         O.pair_layer(b, mlp=O.dense_mlp(8))], width=16, vocab=40)
    w = O.random_model(cfg, seed=9)
    toks = _tokens(cfg, 420, 3)
    ref = O.forward(cfg, w, toks)
    runner = _runner(cfg, w, max_tokens=448)
    _close(_feed(runner, runner.open_request(), toks, [100]), ref, 1e-4)
    runner = _runner(cfg, w, max_tokens=320)                       # fewer rows than tokens
    req = runner.open_request()
    _close(_feed(runner, req, toks, [100]), ref, 1e-4)
    assert runner.rows_held(req) < 320


def test_the_first_tokens_of_a_sequence_reach_a_late_position_through_the_memories_only():
    """Changing token 0 moves the logits 200 positions later (the memories carry it) although every window has long
    passed; with the recurrent outputs silenced (zero out-projections) it no longer does."""
    a = O.left_entry(heads=2, kv_heads=1, dim=8, vdim=8, size=16, conv=3, scale=0.5)
    cfg = O.make_config([O.pair_layer(a, O.right_entry(2, 1, 8, 8, 2), mlp=O.dense_mlp(8)), O.hgrn2_layer(heads=2, dim=8, vdim=8)],
                        width=16, vocab=40)
    w = O.random_model(cfg, seed=4)
    w["l0.mix.right.A_log"] = w["l0.mix.right.A_log"] - 6.0        # both memories forget slowly
    w["l1.mix.lower"] = torch.full_like(w["l1.mix.lower"], 0.98)
    toks = _tokens(cfg, 201, 8)
    other = [(toks[0] + 1) % 40] + toks[1:]

    def last(weights, seq, cuts):
        runner = _runner(cfg, weights)
        return _feed(runner, runner.open_request(), seq, cuts)[-1].double().cpu()

    for cuts in ([201], [190], [64, 2, 100]):
        assert (last(w, toks, cuts) - last(w, other, cuts)).abs().max().item() > 1e-4
    quiet = dict(w)
    quiet["l0.mix.right.o"] = torch.zeros_like(w["l0.mix.right.o"])
    quiet["l1.mix.o"] = torch.zeros_like(w["l1.mix.o"])
    for cuts in ([201], [64, 2, 100]):
        _close(last(quiet, other, cuts), last(quiet, toks, cuts), 1e-6)
    _close(last(w, toks, [190]), O.forward(cfg, w, toks)[-1], 1e-4)


@pytest.mark.parametrize("name,length,cuts", [("small", 40, [13, 2, 9]), ("aligned", 150, [70, 3, 66])])
def test_bf16_serving_precision_stays_within_a_few_roundings(name, length, cuts):
    cfg = CONFIGS[name]()
    w = O.random_model(cfg, seed=11)
    toks = _tokens(cfg, length, 12)
    ref = torch.as_tensor(O.forward(cfg, w, toks))
    for plan in (cuts, [length]):
        runner = _runner(cfg, w, dtype=torch.bfloat16)
        got = _feed(runner, runner.open_request(), toks, plan)
        d = got.double().cpu() - ref
        rel = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / ref.std()
        assert rel.median().item() < 0.03, rel.median().item()
        assert rel.quantile(0.9).item() < 0.1, rel.quantile(0.9).item()      # a token may take another expert in bf16


def test_captured_decode_steps_equal_eager_ones():
    cfg = CONFIGS["aligned"]()
    w = O.random_model(cfg, seed=21)
    prompts = [_tokens(cfg, n, 30 + n) for n in (70, 5, 33)]
    tails = [_tokens(cfg, 12, 40 + i) for i in range(3)]
    outs = []
    for graphs in (False, True):
        runner = _runner(cfg, w, max_tokens=256, max_requests=3)
        if graphs:
            runner.enable_ragged_decode_graphs(ctx_buckets=(64, 256))
            assert runner._ragged_graphs
        reqs = [runner.open_request() for _ in prompts]
        got = [runner.forward_ragged([(r, p) for r, p in zip(reqs, prompts)])]
        for step in range(12):
            live = [i for i in range(3) if not (i == 1 and step >= 6)]          # request 1 leaves half way
            if step == 6:
                runner.close_request(reqs[1])
            got.append(runner.forward_ragged([(reqs[i], [tails[i][step]]) for i in live]).clone())
        outs.append(torch.cat(got).float().cpu())
    _close(outs[1], outs[0], 1e-5)
    ref = O.forward(cfg, w, prompts[0] + tails[0])
    _close(outs[1][[0] + [3 + 3 * k for k in range(6)]], ref[[69] + [70 + k for k in range(6)]], 1e-4)


def test_checkpoint_directory_and_greedy_generation_through_the_engine(tmp_path):
    import json

    from lite_llama_b200.engine import Engine
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.checkpoint import write_safetensors

    cfg = CONFIGS["small"]()
    w = O.random_model(cfg, seed=13, spread=4.0)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    runner = ModelRunner.from_checkpoint(tmp_path, dtype=torch.float32, max_tokens=160, max_requests=3)
    prompts = [_tokens(cfg, n, 20 + n) for n in (9, 1, 30, 4, 17)]
    new = 12
    engine = Engine(runner, max_step_tokens=16, max_portion=7)        # portions of 7 beside decoding requests
    outs = engine.generate(prompts, new)
    for p, out in zip(prompts, outs):
        seq = list(p)
        for t in out:
            logits = torch.as_tensor(O.forward(cfg, w, seq)[-1])
            top2 = logits.topk(2).values
            if (top2[0] - top2[1]).item() < 1e-3:
                break                                                  # undecidable at fp32: stop comparing this one
            assert t == int(logits.argmax()), "greedy token differs from the restatement"
            seq.append(t)
    assert engine.steps > 12 and runner.state_manager.free_slots == 3
    assert runner.kv_cache_manager.can_use_mem_size == 160


# ------------------------------------------------------------------------------------- random models and schedules #
def _random_config(rng, odd):
    def left():
        dim = rng.choice([6, 10, 20] if odd else [8, 16, 32, 64])
        kv = rng.choice([1, 2, 3, 4])
        return O.left_entry(heads=kv * rng.choice([1, 2, 3]), kv_heads=kv, dim=dim,
                            vdim=rng.choice([3, 10, 33] if odd else [8, 24, 64, 80]),
                            size=rng.choice([1, 2, 5, 16, 33, 64, 65, 100, 128, 130, 200, 1000]), conv=rng.choice([1, 2, 3, 4]),
                            scale=rng.choice([0.1, 0.5, 1.0]))

    def right():
        qk = rng.choice([1, 2])
        return O.right_entry(heads=qk * rng.choice([1, 2, 3]), kv_heads=qk, dim=rng.choice([3, 9] if odd else [8, 32, 64]),
                             vdim=rng.choice([5, 7] if odd else [8, 16, 40]), conv=rng.choice([1, 2, 3, 4]))

    def ff():
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return O.dense_mlp(rng.choice([7, 24, 40]))
        experts = rng.choice([1, 3, 8, 12])
        return O.moe_mlp(experts, rng.randint(1, min(experts, 3)), rng.choice([5, 9] if odd else [8, 24]),
                         rng.choice([0, 6, 16]))

    layers = []
    for _ in range(rng.randint(2, 6)):
        if rng.random() < 0.5:
            layers.append(O.pair_layer(left(), right(), rng.choice([0.3, 0.7, 1.0]), rng.choice([0.8, 1.0, 1.5]), ff()))
        else:
            layers.append(O.hgrn2_layer(rng.choice([1, 2, 4]), rng.choice([5, 31] if odd else [8, 32, 48]),
                                        rng.choice([3, 17] if odd else [8, 64]), ff()))
    return O.make_config(layers, width=rng.choice([50, 92, 37, 129] if odd else [16, 40, 72, 144, 200]),
                         vocab=rng.choice([33, 1001] if odd else [17, 64, 300]), eps=rng.choice([1e-5, 1e-6, 1e-3]),
                         embed_scale=rng.choice([1.0, 4.0, 8.0]), logit_scale=rng.choice([0.75, 1.0, 2.0]),
                         softcap=rng.choice([0.0, 10.0, 30.0]), max_positions=256)


@pytest.mark.parametrize("seed", range(8))
def test_random_models_under_random_mixed_schedules(seed):
    """Random sizes (odd widths, head sizes and vocabularies on the odd seeds), layer orders, windows from 1 to beyond
    the sequences; up to four requests fed in random portions beside one another through a pool of exactly their size,
    the tails token by token.  fp32 logits equal the restatement; the bf16 run stays within a few roundings."""
    rng = random.Random(seed)
    cfg = _random_config(rng, odd=seed % 2 == 1)
    w = O.random_model(cfg, seed=seed)
    lens = [rng.choice([1, 5, 23, 60, 97, 150])] + [rng.choice([30, 90, 130]) for _ in range(rng.randint(1, 3))]
    toks = [_tokens(cfg, n, seed * 10 + i) for i, n in enumerate(lens)]
    refs = [O.forward(cfg, w, t) for t in toks]
    plan, fed = [], [0] * len(lens)
    while any(f < n for f, n in zip(fed, lens)):
        step = []
        for i, n in enumerate(lens):
            if fed[i] < n and rng.random() < 0.8:
                left = n - fed[i]
                c = 1 if left <= 20 else min(left - 20, rng.choice([1, 2, 3, 7, 16, 29, 64, 66, 128]))
                step.append((i, c))
                fed[i] += c
        if step:
            plan.append(step)
    pool = -(-sum(lens) // 64) * 64
    for dtype in (torch.float32, torch.bfloat16):
        runner = _runner(cfg, w, dtype=dtype, max_tokens=pool)
        got, reqs, fed = [[] for _ in lens], {}, [0] * len(lens)
        for step in plan:
            entries, want, at = [], [], 0
            for i, c in step:
                if i not in reqs:
                    reqs[i] = runner.open_request()
                entries.append((reqs[i], toks[i][fed[i]:fed[i] + c]))
                want += list(range(at, at + c))
                at += c
            logits = runner.forward_ragged(entries, want).float().cpu()
            at = 0
            for i, c in step:
                got[i].append(logits[at:at + c])
                at += c
                fed[i] += c
                if fed[i] == lens[i]:
                    runner.close_request(reqs.pop(i))
        assert runner.kv_cache_manager.can_use_mem_size == pool
        for i in range(len(lens)):
            if dtype == torch.float32:
                _close(torch.cat(got[i]), refs[i], 1e-4)
            else:
                d = torch.cat(got[i]).double() - torch.as_tensor(refs[i])
                rel = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / max(float(refs[i].std()), 1e-9)
                assert rel.median().item() < 0.08, rel.median().item()
