"""Plain float64 restatement of the Tisosun design, one function per mechanism, token loops instead of batched
kernels.  Shares no code with the package: the tests compare the CUDA path with this.

A model is ``(config, tensors)``: ``config`` is the dict form of ``config.json`` (keys ``width``, ``vocab``,
``norm.eps``, ``token_side.dim``, ``layers``), ``tensors`` maps checkpoint names to arrays.

Notation: ``n(x) = x / sqrt(mean(x^2) + eps)`` is the unit-RMS form of a vector, ``s(z)`` the logistic function.
"""

from __future__ import annotations

import math

import numpy as np


def f64(t) -> np.ndarray:
    if hasattr(t, "detach"):
        t = t.detach().cpu().double().numpy()
    return np.asarray(t, dtype=np.float64)


# ------------------------------------------------------------------------------------------------- small pieces #
def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / math.sqrt(float(np.mean(x * x)) + eps)


def norm_plain(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return unit_rms(x, eps) * w


def norm_centred(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """The model's norm: its weight is stored as the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def logistic(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * logistic(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


# ------------------------------------------------------------------------------------------------- rotation #
def yarn_frequencies(dims: int, base: float, scaling: dict | None) -> tuple[np.ndarray, float]:
    """Per-pair angular frequencies and the factor on cos / sin.  Without ``scaling`` the plain ``base^(-2i/dims)``.
    With it, pairs that turn fast keep their frequency, pairs that turn slowly are slowed by ``factor``, and a linear
    ramp over the pair index joins the two."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_index_of(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(vec: np.ndarray, pos: int, dims: int, freqs: np.ndarray, mag: float) -> np.ndarray:
    """Neighbouring entries (2i, 2i+1) of the first ``dims`` are turned by ``pos * freqs[i]``; the rest is untouched."""
    out = vec.copy()
    for i in range(dims // 2):
        a = pos * freqs[i]
        c, s = math.cos(a) * mag, math.sin(a) * mag
        u, v = vec[2 * i], vec[2 * i + 1]
        out[2 * i] = u * c - v * s
        out[2 * i + 1] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------- mixers #
def min_gru(h: np.ndarray, m: dict, w: dict) -> np.ndarray:
    """``h [T, width]`` -> ``[T, width]``.  Gates read the current token only."""
    T = h.shape[0]
    state = np.zeros(m["width"])
    out = np.zeros((T, w["o"].shape[0]))
    for t in range(T):
        z = logistic(w["z"] @ h[t] + w["z.b"])
        u = w["x"] @ h[t] + w["x.b"]
        cand = np.where(u >= 0.0, u + 0.5, logistic(u))
        state = (1.0 - z) * state + z * cand
        out[t] = w["o"] @ (state * silu(w["g"] @ h[t]))
    return out


def rg_lru(h: np.ndarray, m: dict, w: dict) -> np.ndarray:
    T = h.shape[0]
    width, blocks, taps = m["width"], m["blocks"], m["conv"]
    per = width // blocks
    pre = np.stack([w["x"] @ h[t] + w["x.b"] for t in range(T)])          # convolution input
    state = np.zeros(width)
    out = np.zeros((T, w["o"].shape[0]))
    sp = softplus(w["lam"])
    for t in range(T):
        y = gelu_tanh(w["y"] @ h[t] + w["y.b"])
        u = w["conv.b"].copy()
        for j in range(taps):                      # column taps-1 multiplies the current token
            src = t - (taps - 1 - j)
            if src >= 0:
                u = u + w["conv"][:, j] * pre[src]
        r = np.zeros(width)
        i_gate = np.zeros(width)
        for b in range(blocks):
            sl = slice(b * per, (b + 1) * per)
            r[sl] = logistic(w["ra"][b] @ u[sl] + w["ra.b"][b])
            i_gate[sl] = logistic(w["ri"][b] @ u[sl] + w["ri.b"][b])
        a = np.exp(-8.0 * r * sp)
        state = a * state + np.sqrt(1.0 - a * a) * i_gate * u
        out[t] = w["o"] @ (state * y)
    return out


def chunk_attention(h: np.ndarray, positions: list[int], m: dict, w: dict, eps: float) -> np.ndarray:
    """Softmax attention whose mask is block-diagonal: a query sees the keys of its own block of ``mask.size``
    positions that are not after it."""
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    rdims = int(rot.get("dims", 0))
    freqs, mag = yarn_frequencies(rdims, float(rot.get("base", 10000.0)), rot.get("scaling")) if rdims else (None, 1.0)
    size = int((m.get("mask") or {}).get("size", 0))
    cap = float(m.get("softcap") or 0.0)
    T = h.shape[0]
    qs, ks, vs = [], [], []
    for t in range(T):
        q = (w["q"] @ h[t] + w["q.b"]).reshape(H, dim)
        k = (w["k"] @ h[t] + w["k.b"]).reshape(G, dim)
        v = (w["v"] @ h[t] + w["v.b"]).reshape(G, vdim)
        q = np.stack([norm_plain(q[i], w["q.norm"], eps) for i in range(H)])
        k = np.stack([norm_plain(k[i], w["k.norm"], eps) for i in range(G)])
        if rdims:
            q = np.stack([rotate_pairs(q[i], positions[t], rdims, freqs, mag) for i in range(H)])
            k = np.stack([rotate_pairs(k[i], positions[t], rdims, freqs, mag) for i in range(G)])
        qs.append(q), ks.append(k), vs.append(v)
    out = np.zeros((T, w["o"].shape[0]))
    for t in range(T):
        heads = []
        for i in range(H):
            g = i // (H // G)
            seen = [j for j in range(t + 1)
                    if not size or positions[j] // size == positions[t] // size]
            sc = np.array([float(qs[t][i] @ ks[j][g]) * float(m["scale"]) for j in seen])
            if cap:
                sc = cap * np.tanh(sc / cap)
            p = np.exp(sc - sc.max())
            p = p / p.sum()
            heads.append(sum(p[n] * vs[j][g] for n, j in enumerate(seen)))
        out[t] = w["o"] @ np.concatenate(heads)
    return out


def decay_attention(h: np.ndarray, m: dict, w: dict, eps: float) -> np.ndarray:
    """Linear attention with a fixed decay per head: a ``dim x vdim`` memory per head, no softmax."""
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    mem = np.zeros((H, dim, vdim))
    out = np.zeros((T, w["o"].shape[0]))
    for t in range(T):
        q = silu(w["q"] @ h[t]).reshape(H, dim)
        k = silu(w["k"] @ h[t]).reshape(H, dim)
        v = silu(w["v"] @ h[t]).reshape(H, vdim)
        o = np.zeros((H, vdim))
        for i in range(H):
            mem[i] = float(m["decay"][i]) * mem[i] + np.outer(k[i], v[i])
            o[i] = mem[i].T @ q[i]
        o = norm_plain(o.reshape(-1), w["norm"], eps) * logistic(w["g"] @ h[t])
        out[t] = w["o"] @ o
    return out


def side_by_side(h: np.ndarray, positions: list[int], m: dict, w: dict, eps: float) -> np.ndarray:
    left = chunk_attention(h, positions, m["left"], {k[5:]: v for k, v in w.items() if k.startswith("left.")}, eps)
    right = decay_attention(h, m["right"], {k[6:]: v for k, v in w.items() if k.startswith("right.")}, eps)
    return np.stack([0.5 * (norm_plain(left[t], w["left.out"], eps) + norm_plain(right[t], w["right.out"], eps))
                     for t in range(h.shape[0])])


def gated_ff(h: np.ndarray, w: dict) -> np.ndarray:
    return np.stack([w["down"] @ (silu(w["gate"] @ x) * (w["up"] @ x)) for x in h])


# ------------------------------------------------------------------------------------------------- the model #
def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: f64(v) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False):
    """Logits ``[T, vocab]`` of one whole sequence (positions 0 .. T-1); with ``return_layers`` also every layer's
    result before the depth average."""
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    positions = list(range(T))
    embed = f64(tensors["embed"])
    x = np.stack([norm_centred(embed[t], f64(tensors["embed.norm"]), eps) for t in tokens])
    side_dim = int((config.get("token_side") or {}).get("dim", 0))
    history = [x]
    results = []
    for li, layer in enumerate(config["layers"]):
        p = f"l{li}."
        h1 = np.stack([norm_centred(v, f64(tensors[p + "norm1"]), eps) for v in x])
        w = sub(tensors, p + "mix.")
        kind, m = layer["type"], layer["mixer"]
        if kind == "mingru":
            y = min_gru(h1, m, w)
        elif kind == "rglru":
            y = rg_lru(h1, m, w)
        elif kind == "parallel":
            y = side_by_side(h1, positions, m, w, eps)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            h2 = np.stack([norm_centred(v, f64(tensors[p + "norm2"]), eps) for v in x])
            y = y + gated_ff(h2, sub(tensors, p + "mlp."))
        x = x + y
        if side_dim:
            table = f64(tensors["side.embed"])
            gate, proj, nw = f64(tensors[p + "side.gate"]), f64(tensors[p + "side.proj"]), f64(tensors[p + "side.norm"])
            for t in range(T):
                e = table[tokens[t], li * side_dim:(li + 1) * side_dim]
                x[t] = x[t] + norm_plain(proj @ (gelu_tanh(gate @ x[t]) * e), nw, eps)
        history.append(x)
        results.append(x)
        if p + "dwa" in tensors:
            mix = f64(tensors[p + "dwa"])
            x = sum(mix[j] * history[j] for j in range(li + 2))
    final = np.stack([norm_centred(v, f64(tensors["final.norm"]), eps) for v in x])
    logits = final @ f64(tensors["head"]).T
    return (logits, results) if return_layers else logits


# ------------------------------------------------------------------------------------- configurations for tests #
def attention_entry(heads=3, kv_heads=1, dim=8, vdim=10, rot_dims=4, base=10000.0, chunk=7, softcap=15.0,
                    scaling="default", scale=None) -> dict:
    if scaling == "default":
        scaling = {"factor": 3.0, "fast": 16.0, "original": 64, "slow": 1.0}
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk}, "rot": rot,
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim), "softcap": softcap, "vdim": vdim}


def decay_entry(heads=2, dim=8, vdim=6, decay=(0.6, 0.97)) -> dict:
    return {"decay": list(decay), "dim": dim, "heads": heads, "vdim": vdim}


def layer_entry(kind: str, mixer: dict, ff: int | None = 12) -> dict:
    return {"type": kind, "mixer": mixer, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def parallel_layer(left: dict | None = None, right: dict | None = None, ff: int | None = 12) -> dict:
    return layer_entry("parallel", {"left": left or attention_entry(), "right": right or decay_entry()}, ff)


def mingru_layer(width=14, ff: int | None = 12) -> dict:
    return layer_entry("mingru", {"width": width}, ff)


def rglru_layer(width=12, blocks=3, conv=3, ff: int | None = 12) -> dict:
    return layer_entry("rglru", {"blocks": blocks, "conv": conv, "width": width}, ff)


def make_config(layers: list[dict], width=20, vocab=50, eps=1e-5, side_dim=3) -> dict:
    return {"architecture": "Tisosun", "layers": layers, "norm": {"eps": eps}, "token_side": {"dim": side_dim},
            "vocab": vocab, "width": width}


def random_model(config: dict, seed: int = 0, spread: float = 1.0):
    """Random tensors with checkpoint names, already rounded to bfloat16 values (returned as float32 torch tensors)."""
    import torch

    g = torch.Generator().manual_seed(seed)
    w, d = config["width"], config["token_side"]["dim"]
    count = len(config["layers"])

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain * spread / math.sqrt(cols))

    def vec(n, centre, dev):
        return centre + dev * torch.randn(n, generator=g)

    t = {"embed": torch.randn(config["vocab"], w, generator=g), "embed.norm": vec(w, 0.0, 0.2),
         "side.embed": torch.randn(config["vocab"], d * count, generator=g), "final.norm": vec(w, 0.0, 0.2),
         "head": mat(config["vocab"], w, 3.0)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        t[f"l{i}.norm1"] = vec(w, 0.0, 0.2)
        if layer["type"] == "mingru":
            n = m["width"]
            t.update({p + "z": mat(n, w, 2.0), p + "z.b": vec(n, 0.0, 0.5), p + "x": mat(n, w, 2.0), p + "x.b": vec(n, 0.0, 0.5),
                      p + "g": mat(n, w, 2.0), p + "o": mat(w, n)})
        elif layer["type"] == "rglru":
            n, b = m["width"], m["blocks"]
            per = n // b
            t.update({p + "y": mat(n, w, 2.0), p + "y.b": vec(n, 0.0, 0.3), p + "x": mat(n, w, 2.0), p + "x.b": vec(n, 0.0, 0.3),
                      p + "conv": 0.5 * torch.randn(n, m["conv"], generator=g), p + "conv.b": vec(n, 0.0, 0.2),
                      p + "ra": torch.randn(b, per, per, generator=g) / math.sqrt(per), p + "ra.b": vec(b * per, 0.0, 0.5).view(b, per),
                      p + "ri": torch.randn(b, per, per, generator=g) / math.sqrt(per), p + "ri.b": vec(b * per, 0.0, 0.5).view(b, per),
                      p + "lam": vec(n, -2.0, 1.0), p + "o": mat(w, n)})
        else:
            L, R = m["left"], m["right"]
            H, G, D, Dv = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
            t.update({p + "left.q": mat(H * D, w, 2.0), p + "left.q.b": vec(H * D, 0.0, 0.3), p + "left.k": mat(G * D, w, 2.0),
                      p + "left.k.b": vec(G * D, 0.0, 0.3), p + "left.v": mat(G * Dv, w), p + "left.v.b": vec(G * Dv, 0.0, 0.3),
                      p + "left.q.norm": vec(D, 1.0, 0.2), p + "left.k.norm": vec(D, 1.0, 0.2), p + "left.o": mat(w, H * Dv),
                      p + "left.out": vec(w, 1.0, 0.2), p + "right.out": vec(w, 1.0, 0.2)})
            h, dr, dv = R["heads"], R["dim"], R["vdim"]
            t.update({p + "right.q": mat(h * dr, w, 2.0), p + "right.k": mat(h * dr, w, 2.0), p + "right.v": mat(h * dv, w, 2.0),
                      p + "right.g": mat(h * dv, w, 2.0), p + "right.norm": vec(h * dv, 1.0, 0.2), p + "right.o": mat(w, h * dv)})
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            t.update({f"l{i}.norm2": vec(w, 0.0, 0.2), f"l{i}.mlp.gate": mat(ff, w, 2.0), f"l{i}.mlp.up": mat(ff, w, 2.0),
                      f"l{i}.mlp.down": mat(w, ff)})
        mix = 0.2 * torch.randn(i + 2, generator=g)
        mix[-1] += 0.8
        t[f"l{i}.dwa"] = mix
        t.update({f"l{i}.side.gate": mat(d, w, 2.0), f"l{i}.side.proj": mat(w, d), f"l{i}.side.norm": vec(w, 0.5, 0.1)})
    return {k: v.to(torch.bfloat16).float() for k, v in t.items()}
