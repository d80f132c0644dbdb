"""``bench.py --design gufotar | pesivik | tisosun | gofezen``: prefill and decode throughput of a layer-list design at a few sizes that resemble
a real model's layers (random weights, synthetic ids), beside the closest existing model of the framework (the
uniform rotary decoder: same width, layer count, attention geometry and feed-forward width; for Tisosun the Gufotar
layer-list model, the other design with recurrent layers beside attention layers; for Gofezen the Tisosun model, the
other design of parallel blocks), plus every kernel of the
new path timed alone against its like kernel with the fraction of the measured roofline each reaches.

Timing: CUDA events on the launching stream, >= 3 warm-up runs, a 256 MiB write between timed runs (larger than the
126 MB L2), median of the timed runs.  Step figures include the host work of a step (metadata build, allocation);
prefill steps are eager, decode steps replay each model's captured graph.
"""

from __future__ import annotations

import gc
import json
import math
import statistics
import time

import torch

SIZES = {
    # name: width, layers, heads, kv_heads, head_dim, ff, vocab | state-space: heads, head_dim, state, groups
    "1b": dict(width=2048, layers=8, heads=16, kv_heads=4, head_dim=128, ff=8192, vocab=32000,
               s_heads=64, s_dim=64, s_state=128, s_groups=8),
    "8b": dict(width=4096, layers=8, heads=32, kv_heads=8, head_dim=128, ff=14336, vocab=32000,
               s_heads=128, s_dim=64, s_state=128, s_groups=8),
    "small": dict(width=1024, layers=4, heads=16, kv_heads=4, head_dim=64, ff=4096, vocab=32000,
                  s_heads=32, s_dim=64, s_state=64, s_groups=4),
}


def _flush_buffer(dev):
    return torch.empty(256 << 20, dtype=torch.uint8, device=dev)


def timed(fn, flush, warmup=3, reps=7) -> float:
    """Median device milliseconds of ``fn()``."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return statistics.median(ts)


def gufotar_config(sz: dict, max_positions: int) -> dict:
    layers = []
    for i in range(sz["layers"]):
        if i % 2 == 0:
            layers.append({"type": "mamba2", "mlp": None,
                           "mixer": {"conv": 4, "groups": sz["s_groups"], "heads": sz["s_heads"], "norm_groups": sz["s_groups"],
                                     "state": sz["s_state"], "vdim": sz["s_dim"]}})
        else:
            layers.append({"type": "attention", "mlp": {"ff": sz["ff"], "kind": "dense"},
                           "mixer": {"dim": sz["head_dim"], "heads": sz["heads"], "kv_heads": sz["kv_heads"],
                                     "q_temp": {"coef": 0.5, "every": 64}, "scale": 1.0 / math.sqrt(sz["head_dim"]),
                                     "softcap": 30.0, "v_mix": True, "vdim": sz["head_dim"]}})
    return {"architecture": "Gufotar", "layers": layers, "max_positions": max_positions, "norm": {"eps": 1e-5},
            "vocab": sz["vocab"], "width": sz["width"]}


def build_gufotar(sz, batch, max_positions, dev, dtype, every_ff=False):
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.layered_decoder import map_gufotar_weights, parse_gufotar_config, random_gufotar_tensors

    raw = gufotar_config(sz, max_positions)
    if every_ff:                              # a feed-forward in every layer, as the designs it is compared with have
        for layer in raw["layers"]:
            layer["mlp"] = {"ff": sz["ff"], "kind": "dense"}
    conf = parse_gufotar_config(raw)
    conf.validate()
    weights = map_gufotar_weights(conf, random_gufotar_tensors(conf, seed=0), dev, dtype)
    return ModelRunner(conf, weights, batch * max_positions, device=dev, dtype=dtype, max_requests=batch)


def build_uniform(sz, batch, max_positions, dev, dtype):
    from lite_llama_b200.executor import ModelConfig, ModelRunner

    cfg = ModelConfig("uniform-" + str(sz["width"]), sz["width"], sz["layers"], sz["heads"], sz["kv_heads"],
                      sz["head_dim"], sz["ff"], sz["vocab"])
    return ModelRunner.build(cfg, max_seq_len=max_positions, max_gpu_num_blocks=batch * max_positions, device=dev,
                             dtype=dtype, seed=0)


def step_throughput(sz, batch, prompt, dev, dtype, flush) -> dict:
    """tokens/s of a whole-prompt step (batch x prompt tokens) and of a decode step (batch x 1) for both models."""
    max_pos = prompt + 64
    out = {}
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, sz["vocab"], (batch, prompt), generator=gen)
    # ---- the layer-list design: ragged steps through ModelRunner.forward_ragged
    r = build_gufotar(sz, batch, max_pos, dev, dtype)
    r.enable_ragged_decode_graphs(widths=(batch,), ctx_buckets=(max_pos,))     # decode steps replay a captured graph
    reqs = []

    def g_prefill():
        for q in reqs:
            r.close_request(q)
        reqs[:] = [r.open_request() for _ in range(batch)]
        return r.forward_ragged([(q, ids[i].tolist()) for i, q in enumerate(reqs)])

    pre = timed(g_prefill, flush, warmup=2, reps=3)
    tok = [[int(t)] for t in torch.randint(0, sz["vocab"], (batch,), generator=gen)]
    state = {"n": 0}

    def g_decode():
        if state["n"] >= 48:                      # stay inside the position table: start over from the prompt
            g_prefill()
            state["n"] = 0
        state["n"] += 1
        return r.forward_ragged([(q, tok[i]) for i, q in enumerate(reqs)])

    dec = timed(g_decode, flush, warmup=3, reps=9)
    out["gufotar"] = {"prefill_ms": pre, "prefill_tok_s": batch * prompt / pre * 1e3, "decode_ms": dec,
                      "decode_tok_s": batch / dec * 1e3, "weight_bytes_per_step": r.model.w.nbytes_per_step()}
    del r, reqs
    gc.collect()
    torch.cuda.empty_cache()
    # ---- the closest existing model: uniform rotary decoder, padded-rectangle prefill + one-token decode
    u = build_uniform(sz, batch, max_pos, dev, dtype)
    u.enable_cuda_graph(batch_sizes=(batch,), seq_len_buckets=(max_pos,))      # likewise
    lens = torch.full((batch,), prompt, dtype=torch.int64, device=dev)
    idx = torch.arange(batch, dtype=torch.int64, device=dev)
    pos = torch.arange(prompt, device=dev).repeat(batch, 1)
    dids = ids.to(dev)

    def u_prefill():
        u.kv_cache_manager.free_all()
        u.prefill_alloc_kv_cache(prompt, lens.clone(), idx)
        return u.forward(dids, pos, last_token_index=lens - 1)

    pre = timed(u_prefill, flush, warmup=2, reps=3)
    one = dids[:, :1].contiguous()
    ustate = {"n": 0}

    def u_decode():
        if ustate["n"] >= 48:
            u_prefill()
            ustate["n"] = 0
        ustate["n"] += 1
        u.decode_alloc_kv_cache(batch)
        return u.forward(one, (u.atten_info.b_seq_len - 1).view(batch, 1))

    dec = timed(u_decode, flush, warmup=3, reps=9)
    out["uniform_decoder"] = {"prefill_ms": pre, "prefill_tok_s": batch * prompt / pre * 1e3, "decode_ms": dec,
                              "decode_tok_s": batch / dec * 1e3, "weight_bytes_per_step": u.model.w.nbytes_per_step()}
    del u
    gc.collect()
    torch.cuda.empty_cache()
    return out


def kernel_table(sz, batch, prompt, dev, dtype, flush, hbm_gbs, tflops) -> list[dict]:
    """Every kernel of the new path alone, at the size's shapes, beside its like kernel of the uniform decoder.
    ``frac`` = achieved / measured peak (HBM copy bandwidth for the bandwidth-bound ones, cuBLAS bf16 for attention
    over prompts); ``bytes`` / ``flops`` are the algorithmic minimum of one launch."""
    import lite_llama_b200.kernels as K

    es = 2
    W, H, G, D, ff = sz["width"], sz["heads"], sz["kv_heads"], sz["head_dim"], sz["ff"]
    SH, SP, SN, SG = sz["s_heads"], sz["s_dim"], sz["s_state"], sz["s_groups"]
    inner, gn = SH * SP, SG * SN
    T, ctx = batch * prompt, prompt
    rows: list[dict] = []

    def i32(v):
        return torch.tensor(list(v), dtype=torch.int32, device=dev)

    def rnd(*shape, dt=dtype, s=1.0):
        return (torch.randn(*shape, device=dev) * s).to(dt)

    def add(name, like, fn, nbytes=0, flops=0, like_fn=None, like_bytes=None, like_flops=None):
        ms = timed(fn, flush)
        row = {"kernel": name, "us": ms * 1e3}
        if flops:
            row.update(tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tflops, bound="tensor")
        else:
            row.update(gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / hbm_gbs, bound="hbm")
        if like_fn is not None:
            lms = timed(like_fn, flush)
            lf = (like_flops if like_flops is not None else flops)
            lb = (like_bytes if like_bytes is not None else nbytes)
            lfrac = lf / lms / 1e9 / tflops if flops else lb / lms / 1e6 / hbm_gbs
            row.update(like=like, like_us=lms * 1e3, like_frac=lfrac, distance_ratio=(lfrac / row["frac"]) if row["frac"] else None)
        rows.append(row)

    # ---------------- per-sequence metadata for a prompt step and for a decode step
    p_start, p_ctx, p_slot = i32(range(0, T + 1, prompt)), i32([0] * batch), i32(range(batch))
    d_start, d_ctx = i32(range(batch + 1)), i32([ctx] * batch)
    # ---------------- residual stream
    resid = torch.randn(T, W, device=dev)
    y, wn = rnd(T, W), rnd(W, s=0.1)
    xh, res16 = rnd(T, W), rnd(T, W)
    add("post_norm_residual", "skip_rmsnorm", lambda: K.post_norm_residual(resid, y, wn, 1e-5),
        nbytes=T * W * (4 + 4 + es + es), like_fn=lambda: K.skip_rmsnorm(xh, res16, wn, 1e-5), like_bytes=T * W * 4 * es)
    up = rnd(T, ff)
    gu = rnd(T, 2 * ff)
    add("relu_squared", "swiglu_forward", lambda: K.relu_squared(up), nbytes=T * ff * 2 * es,
        like_fn=lambda: K.swiglu_forward(gu[:, :ff], gu[:, ff:]), like_bytes=T * ff * 3 * es)
    # ---------------- state-space mixer
    proj = rnd(T, 2 * inner + 2 * gn + SH)
    cw, cb = rnd(inner + 2 * gn, 4, s=0.5), rnd(inner + 2 * gn, s=0.1)
    tail = torch.zeros(batch, 3, inner + 2 * gn, dtype=dtype, device=dev)
    add("causal_conv_silu (prompts)", None, lambda: K.causal_conv_silu(proj, inner, inner + 2 * gn, cw, cb, tail, p_start, p_ctx, p_slot),
        nbytes=T * (inner + 2 * gn) * 2 * es)
    xbc = rnd(T, inner + 2 * gn, s=0.5)
    dtb, alog, dsk = rnd(SH), rnd(SH, s=0.5), rnd(SH)
    st = torch.zeros(batch, SH, SN, SP, device=dev)
    dt_view = proj[:, 2 * inner + 2 * gn:]
    scan_bytes = T * ((inner + 2 * gn) * es + SH * es + inner * 4)
    add("ssm_scan (prompts)", None, lambda: K.ssm_scan(xbc, dt_view, dtb, alog, dsk, st, p_start, p_ctx, p_slot, SH, SG, SN, SP),
        nbytes=scan_bytes + batch * SH * SP * SN * 4)
    add("ssm_scan (decode)", None, lambda: K.ssm_scan(xbc[:batch], dt_view[:batch], dtb, alog, dsk, st, d_start, d_ctx, p_slot, SH, SG, SN, SP),
        nbytes=batch * SH * SP * SN * 8)
    yf = torch.randn(T, inner, device=dev)
    add("gated_group_norm", "skip_rmsnorm", lambda: K.gated_group_norm(yf, proj[:, :inner], rnd(inner), SG, 1e-5),
        nbytes=T * inner * (4 + es + es), like_fn=lambda: K.skip_rmsnorm(xh, res16, wn, 1e-5), like_bytes=T * W * 4 * es)
    # ---------------- attention: pool shared by both kernels, [K heads | V heads] per row
    kvw = G * 2 * D
    pool = rnd(batch * (ctx + 1), kvw, s=0.5)
    table = torch.arange(batch * (ctx + 1), dtype=torch.int32, device=dev).view(batch, ctx + 1)
    qkv = rnd(T, (H + 2 * G) * D, s=0.5)
    qw, kw = rnd(H * D, s=0.1) + 1, rnd(G * D, s=0.1) + 1
    rows_p = (table[:, :ctx]).reshape(-1).contiguous()
    pos_p = i32(list(range(prompt)) * batch)
    cos = rnd(batch, prompt, D)
    add("attn_prepare", "rope_kv_write", lambda: K.attn_prepare(qkv, pool, rows_p, pos_p, H * D, G * D, G * D, qw, kw, 1e-5, 0.5, 64.0),
        nbytes=T * ((2 * H + 2 * G) * D * es + 2 * G * D * es),
        like_fn=lambda: K.rope_kv_write(qkv[:, :H * D].view(T, H, D), qkv[:, H * D:(H + G) * D].view(T, G, D),
                                        qkv[:, (H + G) * D:].view(T, G, D), cos, cos, rows_p, pool.view(-1, 2 * G, D), batch, prompt))
    sink = rnd(H)
    out = torch.empty(T, H * D, dtype=dtype, device=dev)
    att_flops = 4 * batch * H * D * prompt * (prompt + 1) / 2
    scale = 1.0 / math.sqrt(D)
    q3, k3, v3 = qkv[:, :H * D].view(T, H, D), qkv[:, H * D:(H + G) * D].view(T, G, D), qkv[:, (H + G) * D:].view(T, G, D)
    lens = torch.full((batch,), prompt, dtype=torch.int32, device=dev)
    add("sink_attention (prompts)", "flash_attention2_no_pad",
        lambda: K.sink_attention(out, qkv, pool, table, p_start, p_ctx, p_slot, None, batch, prompt, sink, H, G, D, D, scale, 30.0),
        flops=att_flops,
        like_fn=lambda: K.flash_attention2_no_pad(q3, k3, v3, scale * 1.4426950408889634, p_start[:batch], lens, prompt))
    splits = max(1, min(128, -(-(ctx + 1) // 128)))
    per = -(-(-(-(ctx + 1) // splits)) // 32) * 32
    dec_bytes = batch * (ctx + 1) * kvw * es
    seq1 = torch.full((batch,), ctx + 1, dtype=torch.int32, device=dev)
    add("sink_attention (decode)", "flash_decoding",
        lambda: K.sink_attention(out, qkv, pool, table, d_start, d_ctx, p_slot, None, batch, 1, sink, H, G, D, D, scale, 30.0,
                                 num_splits=splits, split_keys=per),
        nbytes=dec_bytes,
        like_fn=lambda: K.flash_decoding(q3[:batch], pool.view(-1, 2 * G, D)[:, :G], pool.view(-1, 2 * G, D)[:, G:], scale,
                                         table, p_slot, seq1, ctx + 1))
    return rows


# ------------------------------------------------------------------------------------------------------ Pesivik #
P_SIZES = {
    # latent attention: the cached row (kv_rank + rot_dim) is 128 wide, the widest the tensor-core attention tiles take
    "small": dict(width=1024, layers=4, heads=16, dim=64, rot_dim=32, vdim=64, q_rank=384, kv_rank=96, window=256,
                  experts=16, top=4, groups=4, keep=2, ff=512, shared_ff=1024, vocab=32000),
    "1b": dict(width=2048, layers=8, heads=16, dim=128, rot_dim=32, vdim=128, q_rank=768, kv_rank=96, window=256,
               experts=32, top=4, groups=4, keep=2, ff=1024, shared_ff=2048, vocab=32000),
    "8b": dict(width=4096, layers=8, heads=32, dim=128, rot_dim=32, vdim=128, q_rank=1536, kv_rank=96, window=256,
               experts=64, top=8, groups=8, keep=4, ff=1024, shared_ff=2048, vocab=32000),
}


def pesivik_config(sz: dict) -> dict:
    layer = {"type": "latent_attention",
             "mixer": {"dim": sz["dim"], "heads": sz["heads"], "kv_rank": sz["kv_rank"], "mask": {"size": sz["window"]},
                       "q_rank": sz["q_rank"], "rot": {"base": 1.0e6, "dims": sz["rot_dim"]}, "rot_dim": sz["rot_dim"],
                       "scale": 1.0 / math.sqrt(sz["dim"] + sz["rot_dim"]), "vdim": sz["vdim"]},
             "mlp": {"expert": {"ff": sz["ff"]}, "kind": "moe", "shared": {"ff": sz["shared_ff"]},
                     "router": {"experts": sz["experts"], "top": sz["top"],
                                "groups": {"count": sz["groups"], "keep": sz["keep"]}}}}
    return {"architecture": "Pesivik", "embedding": {"scale": 1.0}, "layers": [dict(layer) for _ in range(sz["layers"])],
            "logit_softcap": 50.0, "norm": {"eps": 1e-6}, "vocab": sz["vocab"], "width": sz["width"]}


def build_pesivik(sz, batch, max_positions, dev, dtype):
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.layered_decoder import map_pesivik_weights, parse_pesivik_config, random_pesivik_tensors

    conf = parse_pesivik_config(pesivik_config(sz))
    conf.validate()
    weights = map_pesivik_weights(conf, random_pesivik_tensors(conf, seed=0), dev, dtype)
    return ModelRunner(conf, weights, batch * max_positions, device=dev, dtype=dtype, max_requests=batch)


def build_uniform_moe(sz, batch, max_positions, dev):
    """The closest existing model: the uniform rotary decoder with routed SwiGLU experts (softmax router), same width,
    depth, head count, expert count, experts per token and expert width; head size = dim + rot_dim, 4 query heads per
    kv head.  Its expert kernels are fp16-only, so it runs in fp16 (same bytes as bf16)."""
    from lite_llama_b200.executor import ModelConfig, ModelRunner

    cfg = ModelConfig("uniform-moe-" + str(sz["width"]), sz["width"], sz["layers"], sz["heads"], max(1, sz["heads"] // 4),
                      128 if sz["dim"] + sz["rot_dim"] > 96 else 64, sz["ff"], sz["vocab"], num_experts=sz["experts"],
                      num_experts_per_tok=sz["top"], moe_intermediate_size=sz["ff"])
    return ModelRunner.build(cfg, max_seq_len=max_positions, max_gpu_num_blocks=batch * max_positions, device=dev,
                             dtype=torch.float16, seed=0)


def pesivik_step_throughput(sz, batch, prompt, dev, dtype, flush) -> dict:
    max_pos = prompt + 64
    out = {}
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, sz["vocab"], (batch, prompt), generator=gen)
    r = build_pesivik(sz, batch, max_pos, dev, dtype)
    r.enable_ragged_decode_graphs(widths=(batch,), ctx_buckets=(max_pos,))
    reqs = []

    def p_prefill():
        for q in reqs:
            r.close_request(q)
        reqs[:] = [r.open_request() for _ in range(batch)]
        return r.forward_ragged([(q, ids[i].tolist()) for i, q in enumerate(reqs)])

    pre = timed(p_prefill, flush, warmup=2, reps=3)
    tok = [[int(t)] for t in torch.randint(0, sz["vocab"], (batch,), generator=gen)]
    state = {"n": 0}

    def p_decode():
        if state["n"] >= 48:
            p_prefill()
            state["n"] = 0
        state["n"] += 1
        return r.forward_ragged([(q, tok[i]) for i, q in enumerate(reqs)])

    dec = timed(p_decode, flush, warmup=3, reps=9)
    out["pesivik"] = {"prefill_ms": pre, "prefill_tok_s": batch * prompt / pre * 1e3, "decode_ms": dec,
                      "decode_tok_s": batch / dec * 1e3, "weight_bytes_per_step": r.model.w.nbytes_per_step()}
    del r, reqs
    gc.collect()
    torch.cuda.empty_cache()
    u = build_uniform_moe(sz, batch, max_pos, dev)
    u.enable_cuda_graph(batch_sizes=(batch,), seq_len_buckets=(max_pos,))
    lens = torch.full((batch,), prompt, dtype=torch.int64, device=dev)
    idx = torch.arange(batch, dtype=torch.int64, device=dev)
    pos = torch.arange(prompt, device=dev).repeat(batch, 1)
    dids = ids.to(dev)

    def u_prefill():
        u.kv_cache_manager.free_all()
        u.prefill_alloc_kv_cache(prompt, lens.clone(), idx)
        return u.forward(dids, pos, last_token_index=lens - 1)

    pre = timed(u_prefill, flush, warmup=2, reps=3)
    one = dids[:, :1].contiguous()
    ustate = {"n": 0}

    def u_decode():
        if ustate["n"] >= 48:
            u_prefill()
            ustate["n"] = 0
        ustate["n"] += 1
        u.decode_alloc_kv_cache(batch)
        return u.forward(one, (u.atten_info.b_seq_len - 1).view(batch, 1))

    dec = timed(u_decode, flush, warmup=3, reps=9)
    out["uniform_moe_decoder"] = {"prefill_ms": pre, "prefill_tok_s": batch * prompt / pre * 1e3, "decode_ms": dec,
                                  "decode_tok_s": batch / dec * 1e3, "dtype": "fp16"}
    del u
    gc.collect()
    torch.cuda.empty_cache()
    return out


def pesivik_kernel_table(sz, batch, prompt, dev, dtype, flush, hbm_gbs, tflops) -> list[dict]:
    """Every kernel of the Pesivik path alone at the size's shapes beside its like kernel of the uniform MoE decoder
    (fp16 inputs for those), with the fraction of the measured roofline each reaches."""
    import lite_llama_b200.kernels as K

    es = 2
    W, H, dim, rot, vdim, qr, kr = sz["width"], sz["heads"], sz["dim"], sz["rot_dim"], sz["vdim"], sz["q_rank"], sz["kv_rank"]
    E, top, ff, sff, win = sz["experts"], sz["top"], sz["ff"], sz["shared_ff"], sz["window"]
    D = kr + rot
    T, ctx = batch * prompt, prompt
    G = max(1, H // 4)
    UD = 128 if dim + rot > 96 else 64
    rows: list[dict] = []

    def i32(v):
        return torch.tensor(list(v), dtype=torch.int32, device=dev)

    def rnd(*shape, dt=dtype, s=1.0):
        return (torch.randn(*shape, device=dev) * s).to(dt)

    def add(name, like, fn, nbytes=0, flops=0, like_fn=None, like_bytes=None, like_flops=None):
        ms = timed(fn, flush)
        row = {"kernel": name, "us": ms * 1e3}
        if flops:
            row.update(tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tflops, bound="tensor")
        else:
            row.update(gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / hbm_gbs, bound="hbm")
        if like_fn is not None:
            lms = timed(like_fn, flush)
            lf = like_flops if like_flops is not None else flops
            lb = like_bytes if like_bytes is not None else nbytes
            lfrac = lf / lms / 1e9 / tflops if flops else lb / lms / 1e6 / hbm_gbs
            row.update(like=like, like_us=lms * 1e3, like_frac=lfrac,
                       distance_ratio=(lfrac / row["frac"]) if row["frac"] else None)
        rows.append(row)

    f16 = torch.float16
    p_start, p_ctx, p_slot = i32(range(0, T + 1, prompt)), i32([0] * batch), i32(range(batch))
    d_start, d_ctx = i32(range(batch + 1)), i32([ctx] * batch)
    # ---------------- residual stream: output norm + layer scale + residual + the next input norm in one launch
    resid = torch.randn(T, W, device=dev)
    y, wn, ls, wnext = rnd(T, W), rnd(W, s=0.1) + 1, rnd(W, s=0.1) + 0.5, rnd(W, s=0.1) + 1
    xh, res16, wn16 = rnd(T, W, dt=f16), rnd(T, W, dt=f16), rnd(W, dt=f16, s=0.1)
    add("post_norm_residual (layer norm, scale, next norm)", "skip_rmsnorm",
        lambda: K.post_norm_residual(resid, y, wn, 1e-5, 0.0, kind="layer", layer_scale=ls, next_weight=wnext, next_kind="layer"),
        nbytes=T * W * (4 + 4 + es + es), like_fn=lambda: K.skip_rmsnorm(xh, res16, wn16, 1e-5), like_bytes=T * W * 4 * es)
    mid = rnd(T, sff)
    gu = rnd(T, 2 * sff, dt=f16)
    add("gelu", "swiglu_forward", lambda: K.gelu(mid), nbytes=T * sff * 2 * es,
        like_fn=lambda: K.swiglu_forward(gu[:, :sff], gu[:, sff:]), like_bytes=T * sff * 3 * es)
    # ---------------- latent preparation beside the rotary cache write
    cols = -(-(qr + kr + rot + H) // 8) * 8
    proj = rnd(T, cols, s=0.5)
    pool = rnd(batch * (ctx + 1), D, s=0.5)
    table = torch.arange(batch * (ctx + 1), dtype=torch.int32, device=dev).view(batch, ctx + 1)
    rows_p = table[:, :ctx].reshape(-1).contiguous()
    pos_p = i32(list(range(prompt)) * batch)
    wq, wkv = rnd(qr, s=0.1) + 1, rnd(kr, s=0.1) + 1
    cs = K.rope_table(pos_p, rot, 1.0e6)
    add("rope_table (once per step)", None, lambda: K.rope_table(pos_p, rot, 1.0e6), nbytes=T * (4 + rot * 4))
    upool = rnd(batch * (ctx + 1), 2 * G * UD, dt=f16, s=0.5)
    uqkv = rnd(T, (H + 2 * G) * UD, dt=f16, s=0.5)
    cos = rnd(batch, prompt, UD, dt=f16)
    add("latent_prepare", "rope_kv_write",
        lambda: K.latent_prepare(proj, pool, rows_p, cs, wq, wkv, qr, kr, rot, rot, 1e-5),
        nbytes=T * ((2 * qr + kr + rot) * es + D * es),
        like_fn=lambda: K.rope_kv_write(uqkv[:, :H * UD].view(T, H, UD), uqkv[:, H * UD:(H + G) * UD].view(T, G, UD),
                                        uqkv[:, (H + G) * UD:].view(T, G, UD), cos, cos, rows_p, upool.view(-1, 2 * G, UD), batch, prompt),
        like_bytes=T * ((2 * H + 2 * G) * UD * es + 2 * G * UD * es))
    # ---------------- per-head products beside the dense GEMM at equal FLOPs
    q = rnd(T, H * (dim + rot), s=0.5)
    qa = torch.empty(T, H * D, dtype=dtype, device=dev)
    ukt = rnd(H, kr, dim, s=0.1)
    dense_x, dense_w = rnd(T, dim), rnd(H * kr, dim, s=0.1)
    add("head_linear (queries into the latent space)", "linear (one GEMM of equal FLOPs)",
        lambda: K.head_linear(qa, D, q, dim + rot, ukt), flops=2 * T * H * kr * dim,
        like_fn=lambda: K.linear(dense_x, dense_w))
    add("rope_heads (queries' rotated parts)", None,
        lambda: K.rope_heads(qa[:, kr:], D, q[:, dim:], dim + rot, cs, H, rot, rot), nbytes=T * H * rot * 2 * es)
    lat = rnd(T, H * kr, s=0.5)
    o = torch.empty(T, H * vdim, dtype=dtype, device=dev)
    uv = rnd(H, vdim, kr, s=0.1)
    dense_x2, dense_w2 = rnd(T, kr), rnd(H * vdim, kr, s=0.1)
    add("head_linear (values out of the latent, gated)", "linear (one GEMM of equal FLOPs)",
        lambda: K.head_linear(o, vdim, lat, kr, uv, proj[:, qr + kr + rot:]), flops=2 * T * H * vdim * kr,
        like_fn=lambda: K.linear(dense_x2, dense_w2))
    # ---------------- attention over the latent rows (one kv head of width D, values = its first kr columns)
    scale = 1.0 / math.sqrt(dim + rot)
    qa = rnd(T, H * D, s=0.5)
    seen = sum(min(t + 1, win) for t in range(prompt))
    att_flops = 2 * batch * H * (D + kr) * seen
    q3, k3, v3 = (uqkv[:, :H * UD].view(T, H, UD), uqkv[:, H * UD:(H + G) * UD].view(T, G, UD),
                  uqkv[:, (H + G) * UD:].view(T, G, UD))
    lens = torch.full((batch,), prompt, dtype=torch.int32, device=dev)
    add("attention over latent rows (prompts, window %d)" % win, "flash_attention2_no_pad (full causal)",
        lambda: K.sink_attention(lat, qa, pool, table, p_start, p_ctx, p_slot, None, batch, prompt, None, H, 1, D, kr, scale,
                                 0.0, window=win, v_col0=0),
        flops=att_flops,
        like_fn=lambda: K.flash_attention2_no_pad(q3, k3, v3, scale * 1.4426950408889634, p_start[:batch], lens, prompt),
        like_flops=4 * batch * H * UD * prompt * (prompt + 1) / 2)
    keys = min(ctx + 1, win)
    splits = max(1, min(128, -(-keys // 128)))
    per = -(-(-(-keys // splits)) // 32) * 32
    seq1 = torch.full((batch,), ctx + 1, dtype=torch.int32, device=dev)
    uout = torch.empty(T, H * UD, dtype=f16, device=dev)
    add("attention over latent rows (decode, window %d)" % win, "flash_decoding (context %d)" % (ctx + 1),
        lambda: K.sink_attention(lat, qa, pool, table, d_start, d_ctx, p_slot, None, batch, 1, None, H, 1, D, kr, scale, 0.0,
                                 num_splits=splits, split_keys=per, window=win, v_col0=0),
        nbytes=batch * keys * D * es,
        like_fn=lambda: K.flash_decoding(q3[:batch], upool.view(-1, 2 * G, UD)[:, :G], upool.view(-1, 2 * G, UD)[:, G:], scale,
                                         table, p_slot, seq1, ctx + 1),
        like_bytes=batch * (ctx + 1) * 2 * G * UD * es)
    # the same at a long context without a window: 8 sequences x 8193 keys
    lctx = 8192
    lpool = rnd(batch * (lctx + 1), D, s=0.5)
    ltable = torch.arange(batch * (lctx + 1), dtype=torch.int32, device=dev).view(batch, lctx + 1)
    l_ctx = i32([lctx] * batch)
    lsplits = max(1, min(128, -(-(lctx + 1) // 128)))
    lper = -(-(-(-(lctx + 1) // lsplits)) // 32) * 32
    lupool = rnd(batch * (lctx + 1), 2 * G * UD, dt=f16, s=0.5)
    lseq = torch.full((batch,), lctx + 1, dtype=torch.int32, device=dev)
    add("attention over latent rows (decode, %d keys, no window)" % (lctx + 1), "flash_decoding (context %d)" % (lctx + 1),
        lambda: K.sink_attention(lat, qa, lpool, ltable, d_start, l_ctx, p_slot, None, batch, 1, None, H, 1, D, kr, scale, 0.0,
                                 num_splits=lsplits, split_keys=lper, window=0, v_col0=0),
        nbytes=batch * (lctx + 1) * D * es,
        like_fn=lambda: K.flash_decoding(q3[:batch], lupool.view(-1, 2 * G, UD)[:, :G], lupool.view(-1, 2 * G, UD)[:, G:], scale,
                                         ltable, p_slot, lseq, lctx + 1),
        like_bytes=batch * (lctx + 1) * 2 * G * UD * es)
    del lpool, lupool
    # ---------------- router and experts
    x = rnd(T, W, s=0.5)
    rw, rb = rnd(E, W, s=0.05), rnd(E, s=0.1)
    x16, rw16 = x.to(f16), rw.to(f16)
    add("route_sigmoid_groups (product + choice)", "linear + route_topk",
        lambda: K.route_sigmoid_groups(x, rw, rb, top, sz["groups"], sz["keep"]), nbytes=T * W * es + E * W * es,
        like_fn=lambda: K.route_topk(K.linear(x16, rw16), top))
    wts, ids = K.route_sigmoid_groups(x, rw, rb, top, sz["groups"], sz["keep"])
    up, down = rnd(E, ff, W, s=0.03), rnd(E, W, ff, s=0.03)
    w1, w2 = rnd(E, 2 * ff, W, dt=f16, s=0.03), rnd(E, W, ff, dt=f16, s=0.03)
    tw, tid = K.route_topk(K.linear(x16, rw16), top)
    add("grouped_experts (prompts)", "fused_moe", lambda: K.grouped_experts(x, up, down, wts, ids),
        flops=2 * T * top * 2 * ff * W, like_fn=lambda: K.fused_moe(x16, w1, w2, tw, tid),
        like_flops=2 * T * top * 3 * ff * W)
    xd, xd16 = x[:batch].contiguous(), x16[:batch].contiguous()
    wd, idd, twd, tidd = wts[:batch].contiguous(), ids[:batch].contiguous(), tw[:batch].contiguous(), tid[:batch].contiguous()
    active = len(set(idd.flatten().tolist()))
    active_u = len(set(tidd.flatten().tolist()))
    add("grouped_experts (decode)", "fused_moe", lambda: K.grouped_experts(xd, up, down, wd, idd),
        nbytes=active * 2 * ff * W * es, like_fn=lambda: K.fused_moe(xd16, w1, w2, twd, tidd),
        like_bytes=active_u * 3 * ff * W * es)
    logits = rnd(batch, sz["vocab"], s=8.0)
    add("softcap_to_f32 (logits)", None, lambda: K.softcap_to_f32(logits, 50.0), nbytes=batch * sz["vocab"] * (es + 4))
    return rows


# ------------------------------------------------------------------------------------------------------ Tisosun #
T_SIZES = {
    # attention half: heads x head_dim on kv_heads, blocks of `chunk` positions; linear-attention half: r_heads memories
    # of r_dim x r_vdim; recurrent layers of the model width; gated feed-forward; 64-wide token input
    "small": dict(width=1024, layers=4, heads=16, kv_heads=4, head_dim=64, chunk=1024, r_heads=16, r_dim=64, r_vdim=64,
                  ff=2048, side=64, vocab=32000, s_heads=32, s_dim=64, s_state=64, s_groups=4),
    "1b": dict(width=2048, layers=8, heads=16, kv_heads=4, head_dim=128, chunk=1024, r_heads=16, r_dim=128, r_vdim=128,
               ff=4096, side=64, vocab=32000, s_heads=64, s_dim=64, s_state=128, s_groups=8),
    "8b": dict(width=4096, layers=8, heads=32, kv_heads=8, head_dim=128, chunk=1024, r_heads=32, r_dim=128, r_vdim=128,
               ff=7168, side=64, vocab=32000, s_heads=128, s_dim=64, s_state=128, s_groups=8),
}


def tisosun_config(sz: dict) -> dict:
    """Layers in the order parallel, real-gated LRU, parallel, minimal GRU, ... with a gated feed-forward each."""
    par = {"type": "parallel", "mlp": {"ff": sz["ff"], "kind": "dense"},
           "mixer": {"left": {"dim": sz["head_dim"], "heads": sz["heads"], "kv_heads": sz["kv_heads"],
                              "mask": {"size": sz["chunk"]},
                              "rot": {"base": 10000.0, "dims": sz["head_dim"] // 2,
                                      "scaling": {"factor": 8.0, "fast": 32.0, "original": 4096, "slow": 1.0}},
                              "scale": 1.0 / math.sqrt(sz["head_dim"]), "softcap": 30.0, "vdim": sz["head_dim"]},
                     "right": {"decay": [1.0 - 2.0 ** (-2 - 6 * h / sz["r_heads"]) for h in range(sz["r_heads"])],
                               "dim": sz["r_dim"], "heads": sz["r_heads"], "vdim": sz["r_vdim"]}}}
    lru = {"type": "rglru", "mlp": {"ff": sz["ff"], "kind": "dense"},
           "mixer": {"blocks": sz["heads"], "conv": 4, "width": sz["width"]}}
    gru = {"type": "mingru", "mlp": {"ff": sz["ff"], "kind": "dense"}, "mixer": {"width": sz["width"]}}
    order = [par, lru, par, gru]
    return {"architecture": "Tisosun", "layers": [dict(order[i % 4]) for i in range(sz["layers"])], "norm": {"eps": 1e-6},
            "token_side": {"dim": sz["side"]}, "vocab": sz["vocab"], "width": sz["width"]}


def build_tisosun(sz, batch, max_positions, dev, dtype):
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.layered_decoder import map_tisosun_weights, parse_tisosun_config, random_tisosun_tensors

    conf = parse_tisosun_config(tisosun_config(sz))
    conf.validate()
    weights = map_tisosun_weights(conf, random_tisosun_tensors(conf, seed=0), dev, dtype)
    return ModelRunner(conf, weights, batch * max_positions, device=dev, dtype=dtype, max_requests=batch)


def tisosun_step_throughput(sz, batch, prompt, dev, dtype, flush) -> dict:
    """tokens/s of a whole-prompt step and of a decode step: Tisosun beside the Gufotar layer-list model of the same
    width, depth, attention geometry and feed-forward width (its feed-forward in every layer here; ungated, so the
    gated one of Tisosun is given 2/3 of its width: equal feed-forward weights)."""
    max_pos = prompt + 64
    out = {}
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, sz["vocab"], (batch, prompt), generator=gen)
    tok = [[int(t)] for t in torch.randint(0, sz["vocab"], (batch,), generator=gen)]
    like = dict(sz, ff=sz["ff"] * 3 // 2)
    for name, build in (("tisosun", lambda: build_tisosun(sz, batch, max_pos, dev, dtype)),
                        ("gufotar", lambda: build_gufotar(like, batch, max_pos, dev, dtype, every_ff=True))):
        r = build()
        r.enable_ragged_decode_graphs(widths=(batch,), ctx_buckets=(max_pos,))
        reqs = []

        def prefill():
            for q in reqs:
                r.close_request(q)
            reqs[:] = [r.open_request() for _ in range(batch)]
            return r.forward_ragged([(q, ids[i].tolist()) for i, q in enumerate(reqs)])

        pre = timed(prefill, flush, warmup=2, reps=3)
        state = {"n": 0}

        def decode():
            if state["n"] >= 48:
                prefill()
                state["n"] = 0
            state["n"] += 1
            return r.forward_ragged([(q, tok[i]) for i, q in enumerate(reqs)])

        dec = timed(decode, flush, warmup=3, reps=9)
        out[name] = {"prefill_ms": pre, "prefill_tok_s": batch * prompt / pre * 1e3, "decode_ms": dec,
                     "decode_tok_s": batch / dec * 1e3, "weight_bytes_per_step": r.model.w.nbytes_per_step()}
        del r, reqs, prefill, decode
        gc.collect()
        torch.cuda.empty_cache()
    return out


def tisosun_kernel_table(sz, batch, prompt, dev, dtype, flush, hbm_gbs, tflops) -> list[dict]:
    """Every kernel of the Tisosun path alone at the size's shapes beside its like kernel of the Gufotar path (the
    closest existing model), with the fraction of the measured roofline each reaches."""
    import lite_llama_b200.kernels as K

    es = 2
    W, H, G, D, ff, side = sz["width"], sz["heads"], sz["kv_heads"], sz["head_dim"], sz["ff"], sz["side"]
    RH, RD, RV, chunk = sz["r_heads"], sz["r_dim"], sz["r_vdim"], sz["chunk"]
    SH, SP, SN, SG = sz["s_heads"], sz["s_dim"], sz["s_state"], sz["s_groups"]
    T, ctx, levels = batch * prompt, prompt, sz["layers"] // 2 + 1
    rows: list[dict] = []

    def i32(v):
        return torch.tensor(list(v), dtype=torch.int32, device=dev)

    def rnd(*shape, dt=dtype, s=1.0):
        return (torch.randn(*shape, device=dev) * s).to(dt)

    def add(name, like, fn, nbytes=0, flops=0, like_fn=None, like_bytes=None, like_flops=None):
        ms = timed(fn, flush)
        row = {"kernel": name, "us": ms * 1e3}
        if flops:
            row.update(tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tflops, bound="tensor")
        else:
            row.update(gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / hbm_gbs, bound="hbm")
        if like_fn is not None:
            lms = timed(like_fn, flush)
            lf = like_flops if like_flops is not None else flops
            lb = like_bytes if like_bytes is not None else nbytes
            lfrac = lf / lms / 1e9 / tflops if flops else lb / lms / 1e6 / hbm_gbs
            row.update(like=like, like_us=lms * 1e3, like_frac=lfrac,
                       distance_ratio=(lfrac / row["frac"]) if row["frac"] else None)
        rows.append(row)

    p_start, p_ctx, p_slot = i32(range(0, T + 1, prompt)), i32([0] * batch), i32(range(batch))
    d_start, d_ctx = i32(range(batch + 1)), i32([ctx] * batch)
    toks = torch.randint(0, sz["vocab"], (T,), device=dev, dtype=torch.int32)
    pos_p = i32(list(range(prompt)) * batch)
    # ---------------- residual stack
    embed, wn = rnd(sz["vocab"], W), rnd(W, s=0.1)
    stack = torch.randn(levels + 1, T, W, device=dev)
    add("embed_rmsnorm", "embed_positions", lambda: K.embed_rmsnorm(toks, embed, wn, 1e-6, out=stack[0]),
        nbytes=T * W * (es + 4), like_fn=lambda: K.embed_positions(toks, pos_p, embed, None), like_bytes=T * W * (es + 4 + es))
    coef, w1, w2 = rnd(levels, s=0.3), rnd(W, s=0.1), rnd(W, s=0.1)
    y = rnd(T, W)
    resid = torch.randn(T, W, device=dev)
    like_norm = lambda: K.post_norm_residual(resid, y, wn, 1e-5)
    like_norm_bytes = T * W * (4 + 4 + es + es)
    add("depth_mix_norms (%d levels -> next level + two input norms)" % levels, "post_norm_residual",
        lambda: K.depth_mix_norms(stack[:levels], levels, coef, w1, w2, 1e-6, out=stack[levels]),
        nbytes=T * W * (4 * levels + 4 + 2 * es), like_fn=like_norm, like_bytes=like_norm_bytes)
    a, b, c = rnd(T, W), rnd(T, W), rnd(T, W)
    add("branch_sum_residual (two normed branches + feed-forward)", "post_norm_residual",
        lambda: K.branch_sum_residual(resid, a, w1, b, w2, c, 1e-6, 0.5), nbytes=T * W * (4 + 4 + 3 * es + es),
        like_fn=like_norm, like_bytes=like_norm_bytes)
    z, table = rnd(T, side), rnd(sz["vocab"], side * sz["layers"])
    up = rnd(T, ff)
    add("gelu_mul_gather (token input)", "relu_squared", lambda: K.gelu_mul_gather(z, toks, table, side),
        nbytes=T * side * 3 * es, like_fn=lambda: K.relu_squared(up), like_bytes=T * ff * 2 * es)
    gu = rnd(T, 2 * ff)
    add("swiglu_forward (gated feed-forward)", "relu_squared", lambda: K.swiglu_forward(gu[:, :ff], gu[:, ff:]),
        nbytes=T * ff * 3 * es, like_fn=lambda: K.relu_squared(up), like_bytes=T * ff * 2 * es)
    # ---------------- attention half
    kvw = G * 2 * D
    pool = rnd(batch * (ctx + 1), kvw, s=0.5)
    tab = torch.arange(batch * (ctx + 1), dtype=torch.int32, device=dev).view(batch, ctx + 1)
    qkv = rnd(T, (H + 2 * G) * D, s=0.5)
    rows_p = tab[:, :ctx].reshape(-1).contiguous()
    rot = D // 2
    f, mag = K.rotary_frequencies(rot, 10000.0, 8.0, 4096.0, 32.0, 1.0)
    freqs = torch.tensor(f, dtype=torch.float64, device=dev)
    cs = K.rope_table_freqs(pos_p, freqs, mag)
    add("rope_table_freqs (once per step)", "rope_table", lambda: K.rope_table_freqs(pos_p, freqs, mag),
        nbytes=T * (4 + rot * 4), like_fn=lambda: K.rope_table(pos_p, rot, 10000.0))
    qn, kn = rnd(D, s=0.1) + 1, rnd(D, s=0.1) + 1
    qw, kw = rnd(H * D, s=0.1) + 1, rnd(G * D, s=0.1) + 1
    prep_bytes = T * ((2 * H + 2 * G) * D * es + 2 * G * D * es)
    add("head_norm_rope_prepare", "attn_prepare",
        lambda: K.head_norm_rope_prepare(qkv, pool, rows_p, cs, qn, kn, H, G, D, D, rot, 1e-6), nbytes=prep_bytes + T * rot * 4,
        like_fn=lambda: K.attn_prepare(qkv, pool, rows_p, pos_p, H * D, G * D, G * D, qw, kw, 1e-5, 0.5, 64.0),
        like_bytes=prep_bytes)
    out = torch.empty(T, H * D, dtype=dtype, device=dev)
    scale = 1.0 / math.sqrt(D)
    sink = rnd(H)
    seen = sum(t % chunk + 1 for t in range(prompt))
    add("block-masked attention (prompts, blocks of %d)" % chunk, "sink_attention (full causal, sink)",
        lambda: K.sink_attention(out, qkv, pool, tab, p_start, p_ctx, p_slot, None, batch, prompt, None, H, G, D, D, scale, 30.0,
                                 block=chunk),
        flops=4 * batch * H * D * seen,
        like_fn=lambda: K.sink_attention(out, qkv, pool, tab, p_start, p_ctx, p_slot, None, batch, prompt, sink, H, G, D, D, scale, 30.0),
        like_flops=4 * batch * H * D * prompt * (prompt + 1) / 2)
    keys = min(ctx + 1, ctx % chunk + 1)
    splits = max(1, min(128, -(-min(ctx + 1, chunk) // 128)))
    per = -(-(-(-min(ctx + 1, chunk) // splits)) // 32) * 32
    fs = max(1, min(128, -(-(ctx + 1) // 128)))
    fper = -(-(-(-(ctx + 1) // fs)) // 32) * 32
    add("block-masked attention (decode, %d of %d keys seen)" % (keys, ctx + 1), "sink_attention (decode, all keys)",
        lambda: K.sink_attention(out, qkv, pool, tab, d_start, d_ctx, p_slot, None, batch, 1, None, H, G, D, D, scale, 30.0,
                                 num_splits=splits, split_keys=per, block=chunk),
        nbytes=batch * keys * kvw * es,
        like_fn=lambda: K.sink_attention(out, qkv, pool, tab, d_start, d_ctx, p_slot, None, batch, 1, sink, H, G, D, D, scale, 30.0,
                                         num_splits=fs, split_keys=fper),
        like_bytes=batch * (ctx + 1) * kvw * es)
    # ---------------- linear-attention half beside the state-space scan
    rin = RH * RV
    rproj = rnd(T, 2 * rin + 2 * RH * RD, s=0.5)
    dec = torch.tensor([1.0 - 2.0 ** (-2 - 6 * h / RH) for h in range(RH)], dtype=torch.float32, device=dev)
    rst = torch.zeros(batch, RH, RD, RV, device=dev)
    inner, gn = SH * SP, SG * SN
    xbc = rnd(T, inner + 2 * gn, s=0.5)
    sproj = rnd(T, SH)
    dtb, alog, dsk = rnd(SH), rnd(SH, s=0.5), rnd(SH)
    sst = torch.zeros(batch, SH, SN, SP, device=dev)
    xr = rproj[:, :rin + 2 * RH * RD]
    add("ssm_scan, fixed decay (prompts; the fp32 and odd-size path)", "ssm_scan (state-space, prompts)",
        lambda: K.ssm_scan(xr, None, None, None, None, rst, p_start, p_ctx, p_slot, RH, RH, RD, RV, fixed_decay=dec, silu_inputs=True),
        nbytes=T * ((rin + 2 * RH * RD) * es + rin * 4) + batch * RH * RD * RV * 4,
        like_fn=lambda: K.ssm_scan(xbc, sproj, dtb, alog, dsk, sst, p_start, p_ctx, p_slot, SH, SG, SN, SP),
        like_bytes=T * ((inner + 2 * gn) * es + SH * es + inner * 4) + batch * SH * SP * SN * 4)
    add("decay_attention (prompts, 64-token chunks on the tensor cores)", "ssm_scan (state-space, prompts)",
        lambda: K.decay_attention(xr, rst, dec, p_start, p_ctx, p_slot, RH, RD, RV, prompt),
        nbytes=T * ((rin + 2 * RH * RD) * es + rin * 4) + batch * RH * RD * RV * 4,
        like_fn=lambda: K.ssm_scan(xbc, sproj, dtb, alog, dsk, sst, p_start, p_ctx, p_slot, SH, SG, SN, SP),
        like_bytes=T * ((inner + 2 * gn) * es + SH * es + inner * 4) + batch * SH * SP * SN * 4)
    add("ssm_scan, fixed decay (decode)", "ssm_scan (state-space, decode)",
        lambda: K.ssm_scan(xr[:batch], None, None, None, None, rst, d_start, d_ctx, p_slot, RH, RH, RD, RV, fixed_decay=dec, silu_inputs=True),
        nbytes=batch * RH * RD * RV * 8,
        like_fn=lambda: K.ssm_scan(xbc[:batch], sproj[:batch], dtb, alog, dsk, sst, d_start, d_ctx, p_slot, SH, SG, SN, SP),
        like_bytes=batch * SH * SP * SN * 8)
    yf = torch.randn(T, rin, device=dev)
    yg = torch.randn(T, inner, device=dev)
    nw, gw = rnd(rin, s=0.1) + 1, rnd(inner, s=0.1) + 1
    zz = rnd(T, inner)
    add("norm_sigmoid_gate", "gated_group_norm", lambda: K.norm_sigmoid_gate(yf, rproj[:, rin + 2 * RH * RD:], nw, 1e-6),
        nbytes=T * rin * (4 + es + es), like_fn=lambda: K.gated_group_norm(yg, zz, gw, SG, 1e-5), like_bytes=T * inner * (4 + es + es))
    # ---------------- element-wise recurrences
    gproj = rnd(T, 3 * W)
    gst = torch.zeros(batch, W, device=dev)
    scan_like = lambda: K.ssm_scan(xbc, sproj, dtb, alog, dsk, sst, p_start, p_ctx, p_slot, SH, SG, SN, SP)
    scan_like_bytes = T * ((inner + 2 * gn) * es + SH * es + inner * 4) + batch * SH * SP * SN * 4
    add("gated_scan, minimal GRU (prompts)", "ssm_scan (state-space, prompts)",
        lambda: K.gated_scan("mingru", gst, gproj[:, :W], gproj[:, W:2 * W], gproj[:, 2 * W:], p_start, p_ctx, p_slot),
        nbytes=T * W * 4 * es, like_fn=scan_like, like_bytes=scan_like_bytes)
    add("gated_scan, minimal GRU (decode)", "ssm_scan (state-space, decode)",
        lambda: K.gated_scan("mingru", gst, gproj[:batch, :W], gproj[:batch, W:2 * W], gproj[:batch, 2 * W:], d_start, d_ctx, p_slot),
        nbytes=batch * W * (4 * es + 8),
        like_fn=lambda: K.ssm_scan(xbc[:batch], sproj[:batch], dtb, alog, dsk, sst, d_start, d_ctx, p_slot, SH, SG, SN, SP),
        like_bytes=batch * SH * SP * SN * 8)
    lproj = rnd(T, 2 * W)
    cw, cb = rnd(W, 4, s=0.5), rnd(W, s=0.1)
    tail = torch.zeros(batch, 3, W, dtype=dtype, device=dev)
    gcw, gcb = rnd(inner + 2 * gn, 4, s=0.5), rnd(inner + 2 * gn, s=0.1)
    gtail = torch.zeros(batch, 3, inner + 2 * gn, dtype=dtype, device=dev)
    gp = rnd(T, 2 * inner + 2 * gn + SH)
    add("causal convolution without activation (prompts)", "causal_conv_silu",
        lambda: K.causal_conv_silu(lproj, W, W, cw, cb, tail, p_start, p_ctx, p_slot, activation=False), nbytes=T * W * 2 * es,
        like_fn=lambda: K.causal_conv_silu(gp, inner, inner + 2 * gn, gcw, gcb, gtail, p_start, p_ctx, p_slot),
        like_bytes=T * (inner + 2 * gn) * 2 * es)
    u = rnd(T, W, s=0.5)
    per_b = W // H
    gw2 = rnd(H, per_b, per_b, s=0.1)
    gates = torch.empty(T, 2 * W, dtype=dtype, device=dev)
    dx, dw = rnd(T, per_b), rnd(W, per_b, s=0.1)
    add("head_linear (block-diagonal gate projection)", "linear (one GEMM of equal FLOPs)",
        lambda: K.head_linear(gates[:, :W], per_b, u, per_b, gw2), flops=2 * T * W * per_b, like_fn=lambda: K.linear(dx, dw))
    br, bi, lam = rnd(W, s=0.3), rnd(W, s=0.3), rnd(W) - 2
    add("gated_scan, real-gated LRU (prompts)", "ssm_scan (state-space, prompts)",
        lambda: K.gated_scan("rglru", gst, u, gates[:, :W], gates[:, W:], p_start, p_ctx, p_slot, p3=lproj[:, :W], bias_r=br,
                             bias_i=bi, lam=lam, decay_scale=8.0),
        nbytes=T * W * 5 * es, like_fn=scan_like, like_bytes=scan_like_bytes)
    return rows


G_SIZES = {
    # attention half: heads x head_dim on kv_heads under a sliding window; delta-rule half: r_heads memories of r_dim x
    # r_vdim on r_qk query/key heads; forget-gate layers: f_heads memories of f_dim x f_vdim; a dense gated feed-forward in
    # the forget-gate layers, routed experts (+ a shared one) in the side-by-side layers.  The Tisosun columns are its
    # own geometry at equal width, depth, attention shape and dense feed-forward width.
    "small": dict(width=1024, layers=4, heads=16, kv_heads=4, head_dim=64, window=256, r_heads=16, r_qk=4, r_dim=64,
                  r_vdim=64, f_heads=8, f_dim=128, f_vdim=128, ff=2048, experts=16, top=2, e_ff=512, shared=1024,
                  vocab=32000, chunk=1024, side=64, s_heads=32, s_dim=64, s_state=64, s_groups=4),
    "1b": dict(width=2048, layers=8, heads=16, kv_heads=4, head_dim=128, window=256, r_heads=16, r_qk=4, r_dim=128,
               r_vdim=128, f_heads=16, f_dim=128, f_vdim=128, ff=4096, experts=32, top=4, e_ff=512, shared=2048,
               vocab=32000, chunk=1024, side=64, s_heads=64, s_dim=64, s_state=128, s_groups=8),
    "8b": dict(width=4096, layers=8, heads=32, kv_heads=8, head_dim=128, window=256, r_heads=32, r_qk=8, r_dim=128,
               r_vdim=128, f_heads=32, f_dim=128, f_vdim=128, ff=7168, experts=64, top=4, e_ff=1024, shared=3072,
               vocab=32000, chunk=1024, side=64, s_heads=128, s_dim=64, s_state=128, s_groups=8),
}


def gofezen_config(sz: dict, max_positions: int) -> dict:
    """Layers in the order forget-gate (dense feed-forward), side-by-side (routed experts), ..."""
    par = {"type": "parallel",
           "mlp": {"kind": "moe", "router": {"experts": sz["experts"], "top": sz["top"]}, "expert": {"ff": sz["e_ff"]},
                   "shared": {"ff": sz["shared"]}},
           "mixer": {"left": {"conv": 3, "dim": sz["head_dim"], "heads": sz["heads"], "kv_heads": sz["kv_heads"],
                              "mask": {"size": sz["window"]}, "scale": 1.0 / math.sqrt(sz["head_dim"]), "vdim": sz["head_dim"]},
                     "left_scale": 0.6,
                     "right": {"conv": 4, "dim": sz["r_dim"], "heads": sz["r_heads"], "kv_heads": sz["r_qk"], "vdim": sz["r_vdim"]},
                     "right_scale": 0.9}}
    fg = {"type": "hgrn2", "mlp": {"kind": "dense", "ff": sz["ff"]},
          "mixer": {"dim": sz["f_dim"], "heads": sz["f_heads"], "vdim": sz["f_vdim"]}}
    return {"architecture": "Gofezen", "embedding": {"scale": 8.0}, "layers": [dict((fg, par)[i % 2]) for i in range(sz["layers"])],
            "logit_scale": 0.5, "logit_softcap": 30.0, "max_positions": max_positions, "norm": {"eps": 1e-6},
            "vocab": sz["vocab"], "width": sz["width"]}


def build_gofezen(sz, batch, max_positions, dev, dtype):
    from lite_llama_b200.executor import ModelRunner
    from lite_llama_b200.executor.layered_decoder import map_gofezen_weights, parse_gofezen_config, random_gofezen_tensors

    conf = parse_gofezen_config(gofezen_config(sz, max_positions))
    conf.validate()
    weights = map_gofezen_weights(conf, random_gofezen_tensors(conf, seed=0), dev, dtype)
    return ModelRunner(conf, weights, batch * max_positions, device=dev, dtype=dtype, max_requests=batch)


def gofezen_step_throughput(sz, batch, prompt, dev, dtype, flush) -> dict:
    """tokens/s of a whole-prompt step and of a decode step: Gofezen beside the Tisosun model (the other design of
    parallel blocks with recurrent layers and attention side by side with linear attention) of the same width, depth,
    attention geometry and dense feed-forward width."""
    max_pos = prompt + 64
    out = {}
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, sz["vocab"], (batch, prompt), generator=gen)
    tok = [[int(t)] for t in torch.randint(0, sz["vocab"], (batch,), generator=gen)]
    for name, build in (("gofezen", lambda: build_gofezen(sz, batch, max_pos, dev, dtype)),
                        ("tisosun", lambda: build_tisosun(sz, batch, max_pos, dev, dtype))):
        r = build()
        r.enable_ragged_decode_graphs(widths=(batch,), ctx_buckets=(max_pos,))
        reqs = []

        def prefill():
            for q in reqs:
                r.close_request(q)
            reqs[:] = [r.open_request() for _ in range(batch)]
            return r.forward_ragged([(q, ids[i].tolist()) for i, q in enumerate(reqs)])

        pre = timed(prefill, flush, warmup=2, reps=3)
        state = {"n": 0}

        def decode():
            if state["n"] >= 48:
                prefill()
                state["n"] = 0
            state["n"] += 1
            return r.forward_ragged([(q, tok[i]) for i, q in enumerate(reqs)])

        dec = timed(decode, flush, warmup=3, reps=9)
        out[name] = {"prefill_ms": pre, "prefill_tok_s": batch * prompt / pre * 1e3, "decode_ms": dec,
                     "decode_tok_s": batch / dec * 1e3, "weight_bytes_per_step": r.model.w.nbytes_per_step()}
        del r, reqs, prefill, decode
        gc.collect()
        torch.cuda.empty_cache()
    return out


def gofezen_kernel_table(sz, batch, prompt, dev, dtype, flush, hbm_gbs, tflops) -> list[dict]:
    """Every kernel of the Gofezen path alone at the size's shapes beside its like kernel of the Tisosun path (the
    closest existing model; for the routed experts the ungated grouped experts of the Pesivik path), with the fraction
    of the measured roofline each reaches."""
    import lite_llama_b200.kernels as K
    from lite_llama_b200.executor.layered_decoder import split_plan

    es = 2
    W, H, G, D, ff, win = sz["width"], sz["heads"], sz["kv_heads"], sz["head_dim"], sz["ff"], sz["window"]
    RH, RQ, RD, RV = sz["r_heads"], sz["r_qk"], sz["r_dim"], sz["r_vdim"]
    FH, FD, FV = sz["f_heads"], sz["f_dim"], sz["f_vdim"]
    E, top, eff = sz["experts"], sz["top"], sz["e_ff"]
    T, ctx = batch * prompt, prompt
    rows: list[dict] = []

    def i32(v):
        return torch.tensor(list(v), dtype=torch.int32, device=dev)

    def rnd(*shape, dt=dtype, s=1.0):
        return (torch.randn(*shape, device=dev) * s).to(dt)

    def add(name, like, fn, nbytes=0, flops=0, like_fn=None, like_bytes=None, like_flops=None):
        ms = timed(fn, flush)
        row = {"kernel": name, "us": ms * 1e3}
        if flops:
            row.update(tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tflops, bound="tensor")
        else:
            row.update(gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / hbm_gbs, bound="hbm")
        if like_fn is not None:
            lms = timed(like_fn, flush)
            lf = like_flops if like_flops is not None else flops
            lb = like_bytes if like_bytes is not None else nbytes
            lfrac = lf / lms / 1e9 / tflops if flops else lb / lms / 1e6 / hbm_gbs
            row.update(like=like, like_us=lms * 1e3, like_frac=lfrac,
                       distance_ratio=(lfrac / row["frac"]) if row["frac"] else None)
        rows.append(row)

    p_start, p_ctx, p_slot = i32(range(0, T + 1, prompt)), i32([0] * batch), i32(range(batch))
    d_start, d_ctx = i32(range(batch + 1)), i32([ctx] * batch)
    # ---------------- residual stream: scaled branches + feed-forward + the next layer's input norm in one pass
    resid = torch.randn(T, W, device=dev)
    a, b, c, w1, w2 = rnd(T, W), rnd(T, W), rnd(T, W), rnd(W, s=0.1) + 1, rnd(W, s=0.1) + 1
    add("branch_sum_residual (two scaled branches + feed-forward + next input norm)",
        "branch_sum_residual (two normed branches + feed-forward)",
        lambda: K.branch_sum_residual(resid, a, None, b, None, c, 1e-6, 0.6, want_act=False, scale_b=0.9, next_weight=w1),
        nbytes=T * W * (4 + 4 + 3 * es + es),
        like_fn=lambda: K.branch_sum_residual(resid, a, w1, b, w2, c, 1e-6, 0.5), like_bytes=T * W * (4 + 4 + 3 * es + es))
    lg = rnd(batch, sz["vocab"])
    add("softcap_to_f32 (scaled, capped logits of a decode step)", None, lambda: K.softcap_to_f32(lg, 30.0, 0.5),
        nbytes=batch * sz["vocab"] * (es + 4))
    # ---------------- attention half: convolution, unit-RMS + cache write, window attention over wide values, head mix
    ch = H * D + 2 * G * D
    proj = rnd(T, ch, s=0.5)
    cw, cb = rnd(ch, 3, s=0.5), torch.zeros(ch, dtype=dtype, device=dev)
    tail = torch.zeros(batch, 2, ch, dtype=dtype, device=dev)
    SH, SP, SN, SG = sz["s_heads"], sz["s_dim"], sz["s_state"], sz["s_groups"]
    lproj, lw, lb = rnd(T, 2 * W), rnd(W, 4, s=0.5), rnd(W, s=0.1)
    ltail = torch.zeros(batch, 3, W, dtype=dtype, device=dev)
    add("causal convolution of q | k | v (prompts, 3 taps, no activation)", "causal convolution without activation (gated LRU)",
        lambda: K.causal_conv_silu(proj, 0, ch, cw, cb, tail, p_start, p_ctx, p_slot, activation=False), nbytes=T * ch * 2 * es,
        like_fn=lambda: K.causal_conv_silu(lproj, W, W, lw, lb, ltail, p_start, p_ctx, p_slot, activation=False),
        like_bytes=T * W * 2 * es)
    kvw = G * 2 * D
    pool = rnd(batch * (ctx + 1), kvw, s=0.5)
    tab = torch.arange(batch * (ctx + 1), dtype=torch.int32, device=dev).view(batch, ctx + 1)
    rows_p = tab[:, :ctx].reshape(-1).contiguous()
    pos_p = i32(list(range(prompt)) * batch)
    ones = torch.ones(D, dtype=dtype, device=dev)
    rot = D // 2
    f, mag = K.rotary_frequencies(rot, 10000.0, 8.0, 4096.0, 32.0, 1.0)
    cs = K.rope_table_freqs(pos_p, torch.tensor(f, dtype=torch.float64, device=dev), mag)
    prep_bytes = T * ((2 * H + 2 * G) * D * es + 2 * G * D * es)
    add("head_norm_rope_prepare (unit-RMS of q and k, no rotation, cache write)", "head_norm_rope_prepare (weights, rotation)",
        lambda: K.head_norm_rope_prepare(proj, pool, rows_p, None, ones, ones, H, G, D, D, 0, 1e-6), nbytes=prep_bytes,
        like_fn=lambda: K.head_norm_rope_prepare(proj, pool, rows_p, cs, ones, ones, H, G, D, D, rot, 1e-6),
        like_bytes=prep_bytes + T * rot * 4)
    per_call = max(c for c in range(1, G + 1) if G % c == 0 and (c * D <= 128 or c == 1))
    calls, width = G // per_call, per_call * D
    wide = torch.empty(T, calls * H * width, dtype=dtype, device=dev)
    out = torch.empty(T, H * D, dtype=dtype, device=dev)
    scale = 1.0 / math.sqrt(D)
    seen = sum(min(t + 1, win) for t in range(prompt))
    chunk = sz["chunk"]
    like_seen = sum(t % chunk + 1 for t in range(prompt))

    def mixed_prompt():
        for cidx in range(calls):
            K.sink_attention(wide[:, cidx * H * width:(cidx + 1) * H * width], proj, pool, tab, p_start, p_ctx, p_slot, None,
                             batch, prompt, None, H, G, D, width, scale, 0.0, window=win, v_col0=G * D + cidx * width,
                             v_head_stride=0)

    add("window attention, every value head under every query head's weights (prompts, window %d, %d calls)" % (win, calls),
        "block-masked attention (prompts, blocks of %d)" % chunk, mixed_prompt,
        flops=batch * H * seen * (2 * D + 2 * G * D),
        like_fn=lambda: K.sink_attention(out, proj, pool, tab, p_start, p_ctx, p_slot, None, batch, prompt, None, H, G, D, D,
                                         scale, 30.0, block=chunk),
        like_flops=4 * batch * H * D * like_seen)
    talk = rnd(H, H, s=0.2)
    add("head_mix (weights mixed across heads, on the outputs)", None,
        lambda: K.head_mix(wide, talk, H, G, per_call, D), nbytes=T * H * D * (G + 1) * es)
    keys = min(ctx + 1, win)
    splits, per = split_plan(keys)
    # a step of single tokens mixes the WEIGHTS: softmax weights per head, then mixed weights times each head's own values

    def mixed_decode():
        K.mixed_head_attention(out, proj, pool, tab, d_start, d_ctx, p_slot, None, batch, talk, H, G, D, D, scale, 0.0, keys,
                               window=win)

    lkeys = min(ctx + 1, ctx % chunk + 1)
    lsplits, lper = split_plan(min(ctx + 1, chunk))
    add("window attention, weights mixed across heads (decode, %d of %d keys seen, 2 launches)" % (keys, ctx + 1),
        "block-masked attention (decode, %d keys seen)" % lkeys, mixed_decode, nbytes=batch * keys * kvw * es,
        like_fn=lambda: K.sink_attention(out, proj, pool, tab, d_start, d_ctx, p_slot, None, batch, 1, None, H, G, D, D, scale,
                                         30.0, num_splits=lsplits, split_keys=lper, block=chunk),
        like_bytes=batch * lkeys * kvw * es)
    # ---------------- the two memories beside Tisosun's linear attention (token scan and tensor-core chunks)
    rin = RH * RV
    tproj = rnd(T, 2 * rin + 2 * RH * RD, s=0.5)
    dec = torch.tensor([1.0 - 2.0 ** (-2 - 6 * h / RH) for h in range(RH)], dtype=torch.float32, device=dev)
    tst = torch.zeros(batch, RH, RD, RV, device=dev)
    tx = tproj[:, :rin + 2 * RH * RD]
    like_scan = lambda: K.ssm_scan(tx, None, None, None, None, tst, p_start, p_ctx, p_slot, RH, RH, RD, RV, fixed_decay=dec, silu_inputs=True)
    like_chunk = lambda: K.decay_attention(tx, tst, dec, p_start, p_ctx, p_slot, RH, RD, RV, prompt)
    like_dec = lambda: K.ssm_scan(tx[:batch], None, None, None, None, tst, d_start, d_ctx, p_slot, RH, RH, RD, RV, fixed_decay=dec, silu_inputs=True)
    like_bytes = T * ((rin + 2 * RH * RD) * es + rin * 4) + batch * RH * RD * RV * 4
    dch = 2 * RQ * RD + RH * RV
    dproj = rnd(T, dch + 2 * RH, s=0.5)
    dst = torch.zeros(batch, RH, RD, RV, device=dev)
    dtb, alog = rnd(RH) - 1, rnd(RH, s=0.5) - 1
    dq, dk, dv = dproj[:, :RQ * RD], dproj[:, RQ * RD:2 * RQ * RD], dproj[:, 2 * RQ * RD:dch]
    p0, p1 = dproj[:, dch:dch + RH], dproj[:, dch + RH:]

    def delta(n, start, cx):
        return K.gated_linear_scan("delta_rule", dst, dq[:n], dk[:n], dv[:n], start, cx, p_slot, RH, RQ, RD, RV, c0=dtb, c1=alog,
                                   p0=p0[:n], p1=p1[:n], q_scale=RD ** -0.5)

    d_bytes = T * ((dch + 2 * RH) * es + rin * 4) + batch * RH * RD * RV * 4
    add("gated_linear_scan, delta rule (prompts)", "ssm_scan, fixed decay (prompts, token by token)",
        lambda: delta(T, p_start, p_ctx), nbytes=d_bytes, like_fn=like_scan, like_bytes=like_bytes)
    rows.append(dict(rows[-1], like="decay_attention (prompts, 64-token chunks on the tensor cores)"))
    lms = timed(like_chunk, flush)
    rows[-1].update(like_us=lms * 1e3, like_frac=like_bytes / lms / 1e6 / hbm_gbs,
                    distance_ratio=like_bytes / lms / 1e6 / hbm_gbs / rows[-1]["frac"])
    add("gated_linear_scan, delta rule (decode)", "ssm_scan, fixed decay (decode)", lambda: delta(batch, d_start, d_ctx),
        nbytes=batch * RH * RD * RV * 8, like_fn=like_dec, like_bytes=batch * RH * RD * RV * 8)
    fproj = rnd(T, 2 * FH * FD + FH * FV, s=0.5)
    fst = torch.zeros(batch, FH, FD, FV, device=dev)
    low = torch.rand(FH * FD, device=dev).to(dtype) * 0.9
    fq, fk, fv = fproj[:, :FH * FD], fproj[:, FH * FD:2 * FH * FD], fproj[:, 2 * FH * FD:]

    def forget(n, start, cx):
        return K.gated_linear_scan("forget_gate", fst, fq[:n], fk[:n], fv[:n], start, cx, p_slot, FH, FH, FD, FV, c0=low)

    f_bytes = T * ((2 * FH * FD + FH * FV) * es + FH * FV * 4) + batch * FH * FD * FV * 4
    add("gated_linear_scan, forget gate (prompts)", "ssm_scan, fixed decay (prompts, token by token)",
        lambda: forget(T, p_start, p_ctx), nbytes=f_bytes, like_fn=like_scan, like_bytes=like_bytes)
    add("gated_linear_scan, forget gate (decode)", "ssm_scan, fixed decay (decode)", lambda: forget(batch, d_start, d_ctx),
        nbytes=batch * FH * FD * FV * 8, like_fn=like_dec, like_bytes=batch * RH * RD * RV * 8)
    yf = torch.randn(T, rin, device=dev)
    nw, nv = rnd(rin, s=0.1) + 1, rnd(RV, s=0.1) + 1
    gate = rnd(T, rin)
    add("head_norm_gate (per-head norm, SiLU gate)", "norm_sigmoid_gate", lambda: K.head_norm_gate(yf, nv, RH, 1e-6, gate),
        nbytes=T * rin * (4 + es + es), like_fn=lambda: K.norm_sigmoid_gate(yf, gate, nw, 1e-6))
    rcw, rcb = rnd(dch, 4, s=0.5), torch.zeros(dch, dtype=dtype, device=dev)
    rtail = torch.zeros(batch, 3, dch, dtype=dtype, device=dev)
    add("causal convolution + SiLU of q' | k' | v' (prompts, 4 taps)", "causal convolution without activation (gated LRU)",
        lambda: K.causal_conv_silu(dproj, 0, dch, rcw, rcb, rtail, p_start, p_ctx, p_slot), nbytes=T * dch * 2 * es,
        like_fn=lambda: K.causal_conv_silu(lproj, W, W, lw, lb, ltail, p_start, p_ctx, p_slot, activation=False),
        like_bytes=T * W * 2 * es)
    # ---------------- feed-forwards
    gu = rnd(T, 2 * ff)
    zrow = rnd(T, 8)
    add("swiglu_scaled (shared expert: SiLU * up * logistic token gate)", "swiglu_forward",
        lambda: K.swiglu_scaled(gu[:, :ff], gu[:, ff:], None, zrow[:, :1]), nbytes=T * ff * 3 * es,
        like_fn=lambda: K.swiglu_forward(gu[:, :ff], gu[:, ff:]))
    x = rnd(T, W, s=0.5)
    router = rnd(E, W, s=W ** -0.5)
    add("route_sigmoid_groups (scores kept as they are)", "route_sigmoid_groups (renormalised)",
        lambda: K.route_sigmoid_groups(x, router, None, top, 1, 1, renormalize=False), flops=2 * T * E * W,
        like_fn=lambda: K.route_sigmoid_groups(x, router, None, top, 1, 1))
    wts, ids = K.route_sigmoid_groups(x, router, None, top, 1, 1, renormalize=False)
    wgu, wdn = rnd(E, 2 * eff, W, s=W ** -0.5), rnd(E, W, eff, s=eff ** -0.5)
    wup = rnd(E, 2 * eff, W, s=W ** -0.5)                            # ungated experts of equal weight bytes and FLOPs
    wdn2 = rnd(E, W, 2 * eff, s=eff ** -0.5)
    add("grouped_experts, gated, weight on the input (prompts)", "grouped_experts, ungated GELU (equal first product)",
        lambda: K.grouped_experts(x, wgu, wdn, wts, ids, activation="silu", gated=True, weight_on_input=True),
        flops=2 * T * top * 3 * eff * W, like_fn=lambda: K.grouped_experts(x, wup, wdn2, wts, ids),
        like_flops=2 * T * top * 4 * eff * W)
    xd, wd, idd = x[:batch], wts[:batch].contiguous(), ids[:batch].contiguous()
    add("grouped_experts, gated, weight on the input (decode)", "grouped_experts, ungated GELU (equal first product)",
        lambda: K.grouped_experts(xd, wgu, wdn, wd, idd, activation="silu", gated=True, weight_on_input=True),
        nbytes=min(E, batch * top) * 3 * eff * W * es, like_fn=lambda: K.grouped_experts(xd, wup, wdn2, wd, idd),
        like_bytes=min(E, batch * top) * 4 * eff * W * es)
    return rows


def run(args) -> None:
    from bench import ClockSampler, peaks

    dev = "cuda:0"
    torch.cuda.set_device(0)
    dtype = torch.bfloat16
    hbm_gbs, tflops, src = peaks()
    flush = _flush_buffer(dev)
    sizes = [s for s in (args.design_sizes or "small,1b,8b").split(",") if s]
    table, steps, kernels = {"pesivik": (P_SIZES, pesivik_step_throughput, pesivik_kernel_table),
                             "tisosun": (T_SIZES, tisosun_step_throughput, tisosun_kernel_table),
                             "gofezen": (G_SIZES, gofezen_step_throughput, gofezen_kernel_table)}.get(
        args.design, (SIZES, step_throughput, kernel_table))
    result = {"design": args.design, "dtype": "bf16", "data": "synthetic ids, random weights", "peaks": {"hbm_gbs": hbm_gbs, "bf16_tflops": tflops, "source": src},
              "batch": args.batch, "prompt_len": args.prompt_len, "l2_policy": "256 MiB written between timed runs", "sizes": {}}
    t0 = time.time()
    with ClockSampler(0) as clocks:
        for name in sizes:
            sz = table[name]
            entry = {"geometry": sz}
            entry["steps"] = steps(sz, args.batch, args.prompt_len, dev, dtype, flush)
            torch.cuda.empty_cache()
            entry["kernels"] = kernels(sz, args.batch, args.prompt_len, dev, dtype, flush, hbm_gbs, tflops)
            torch.cuda.empty_cache()
            result["sizes"][name] = entry
    result["clocks"] = clocks.summary()
    result["seconds"] = round(time.time() - t0, 1)
    print(json.dumps(result))
