"""Plain float64 restatement of the Gofezen design, one function per mechanism, token loops instead of batched
kernels.  Shares no code with the package: the tests compare the CUDA path with this.

A model is ``(config, tensors)``: ``config`` is the dict form of ``config.json`` (keys ``width``, ``vocab``,
``norm.eps``, ``embedding.scale``, ``logit_scale``, ``logit_softcap``, ``layers``), ``tensors`` maps checkpoint names
to arrays.

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


def logistic(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * logistic(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def short_conv(u: np.ndarray, taps_w: np.ndarray) -> np.ndarray:
    """``u [T, C]``, ``taps_w [C, taps]`` -> ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)``; inputs before the first
    token are zero; the last column multiplies the current token."""
    T, taps = u.shape[0], taps_w.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                y[t] += taps_w[:, j] * u[src]
    return y


# ------------------------------------------------------------------------------------------------- mixers #
def hgrn2(h: np.ndarray, m: dict, w: dict, eps: float) -> np.ndarray:
    """Linear attention whose forget gate is also the complement of its write gate.  Per head a ``dim x vdim`` memory:
    ``S <- diag(f) S + (1 - f) v^T``, read-out ``S^T q``; ``f = l + (1 - l) s(W_f h + b)`` with a lower bound ``l``."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, D)
    v = (h @ w["v"].T).reshape(T, H, V)
    low = w["lower"]
    f = (low + (1.0 - low) * logistic(h @ w["f"].T + w["f.b"])).reshape(T, H, D)
    S = np.zeros((H, D, V))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            S[a] = f[t, a][:, None] * S[a] + np.outer(1.0 - f[t, a], v[t, a])
            o[t, a] = unit_rms(S[a].T @ q[t, a], eps) * w["norm"]
    return o.reshape(T, H * V) @ w["o"].T


def window_attention(h: np.ndarray, m: dict, w: dict, eps: float) -> np.ndarray:
    """Softmax attention without positions: biased projections, a short convolution on q, k, v, weightless per-head
    unit-RMS of q and k, a sliding window, and the heads' softmax weights mixed by a ``heads x heads`` matrix before
    they meet the values (head ``a`` keeps reading the values of its own key/value head)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = int(m["mask"]["size"]) if m.get("mask") else 0
    q = short_conv(h @ w["q"].T + w["q.b"], w["q.conv"]).reshape(T, H, D)
    k = short_conv(h @ w["k"].T + w["k.b"], w["k.conv"]).reshape(T, G, D)
    v = short_conv(h @ w["v"].T + w["v.b"], w["v.conv"]).reshape(T, G, V)
    per = H // G
    out = np.zeros((T, H, V))
    for t in range(T):
        lo = max(0, t - size + 1) if size else 0
        probs = np.zeros((H, t + 1 - lo))
        for a in range(H):
            qa = unit_rms(q[t, a], eps)
            sc = np.array([float(qa @ unit_rms(k[j, a // per], eps)) for j in range(lo, t + 1)]) * m["scale"]
            e = np.exp(sc - sc.max())
            probs[a] = e / e.sum()
        mixed = w["talk"] @ probs
        for a in range(H):
            out[t, a] = mixed[a] @ v[lo:t + 1, a // per]
    return out.reshape(T, H * V) @ w["o"].T


def gated_delta(h: np.ndarray, m: dict, w: dict, eps: float) -> np.ndarray:
    """Gated delta rule.  q, k (``kv_heads x dim``) and v (``heads x vdim``) pass a short convolution and SiLU; q, k
    become unit vectors (q also times ``dim^-1/2``).  Per head, with write strength ``beta`` and decay ``g``:
    ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``.  The read-out is unit-RMS'd, weighted and gated."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, V)
    beta = logistic(h @ w["b"].T)
    decay = np.exp(-np.exp(w["A_log"]) * softplus(h @ w["a"].T + w["dt_bias"]))
    gate = silu(h @ w["g"].T).reshape(T, H, V)
    per = H // G
    S = np.zeros((H, D, V))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            c = a // per
            qa = q[t, c] / math.sqrt(float(q[t, c] @ q[t, c]) + 1e-6) * D ** -0.5
            ka = k[t, c] / math.sqrt(float(k[t, c] @ k[t, c]) + 1e-6)
            S[a] *= decay[t, a]
            u = beta[t, a] * (v[t, a] - S[a].T @ ka)
            S[a] += np.outer(ka, u)
            o[t, a] = unit_rms(S[a].T @ qa, eps) * w["norm"] * gate[t, a]
    return o.reshape(T, H * V) @ w["o"].T


def side_by_side(h: np.ndarray, m: dict, w: dict, eps: float) -> np.ndarray:
    left = window_attention(h, m["left"], {k[5:]: v for k, v in w.items() if k.startswith("left.")}, eps)
    right = gated_delta(h, m["right"], {k[6:]: v for k, v in w.items() if k.startswith("right.")}, eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ------------------------------------------------------------------------------------------------- feed-forwards #
def gated_ff(x: np.ndarray, w: dict, prefix: str = "") -> np.ndarray:
    return w[prefix + "down"] @ (silu(w[prefix + "gate"] @ x) * (w[prefix + "up"] @ x))


def dense_ff(h: np.ndarray, m: dict, w: dict) -> np.ndarray:
    return np.stack([gated_ff(x, w) for x in h])


def routed_ff(h: np.ndarray, m: dict, w: dict) -> np.ndarray:
    """Sigmoid router; the ``top`` best experts each see the token TIMES their score (not renormalised); a shared
    expert, scaled by one logistic number per token, joins."""
    top = int(m["router"]["top"])
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    for t, x in enumerate(h):
        s = logistic(w["router"] @ x)
        for e in np.argsort(-s, kind="stable")[:top]:
            out[t] += gated_ff(s[e] * x, w, f"e{e}.")
        if m.get("shared"):
            out[t] += logistic(float(w["shared.sg"][0] @ x)) * gated_ff(x, w, "shared.")
    return out


# ------------------------------------------------------------------------------------------------- whole model #
def layer_tensors(tensors: dict, i: int, part: str) -> dict:
    p = f"l{i}.{part}."
    return {k[len(p):]: f64(v) for k, v in tensors.items() if k.startswith(p)}


def forward(config: dict, tensors: dict, tokens, trace: list | None = None, return_layers: bool = False):
    """``tokens`` of ONE sequence -> logits ``[T, vocab]``; ``trace`` collects the residual after every layer
    (``return_layers``: returned beside the logits)."""
    if return_layers:
        layers: list = []
        return forward(config, tensors, tokens, layers), layers
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    x = f64(tensors["embed"])[list(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    x = x + f64(tensors["pos"])[:T]
    for i, layer in enumerate(config["layers"]):
        nw = f64(tensors[f"l{i}.norm1"])
        h = np.stack([unit_rms(r, eps) * nw for r in x])
        mw = layer_tensors(tensors, i, "mix")
        if layer["type"] == "hgrn2":
            y = hgrn2(h, layer["mixer"], mw, eps)
        elif layer["type"] == "parallel":
            y = side_by_side(h, layer["mixer"], mw, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            fw = layer_tensors(tensors, i, "mlp")
            y = y + (dense_ff(h, mlp, fw) if mlp["kind"] == "dense" else routed_ff(h, mlp, fw))
        x = x + y
        if trace is not None:
            trace.append(x.copy())
    fn = f64(tensors["final.norm"])
    z = np.stack([unit_rms(r, eps) * fn for r in x]) @ f64(tensors["head"]).T * float(config.get("logit_scale", 1.0))
    cap = float(config.get("logit_softcap") or 0.0)
    return cap * np.tanh(z / cap) if cap else z


# ------------------------------------------------------------------------------------------- test model builders #
def left_entry(heads=3, kv_heads=1, dim=6, vdim=5, size=9, conv=3, scale=0.4) -> dict:
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "conv": conv,
            "scale": scale}


def right_entry(heads=2, kv_heads=1, dim=4, vdim=6, conv=2) -> dict:
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense_mlp(ff=14) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=5, top=2, ff=6, shared_ff=7) -> dict:
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        out["shared"] = {"ff": shared_ff}
    return out


def hgrn2_layer(heads=2, dim=4, vdim=6, mlp="dense") -> dict:
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim},
            "mlp": dense_mlp() if mlp == "dense" else mlp}


def pair_layer(left=None, right=None, left_scale=0.7, right_scale=1.2, mlp="moe") -> dict:
    return {"type": "parallel", "mixer": {"left": left or left_entry(), "right": right or right_entry(),
                                          "left_scale": left_scale, "right_scale": right_scale},
            "mlp": moe_mlp() if mlp == "moe" else mlp}


def make_config(layers, width=24, vocab=50, eps=1e-5, embed_scale=3.0, logit_scale=0.7, softcap=12.0,
                max_positions=512) -> dict:
    return {"architecture": "Gofezen", "width": width, "vocab": vocab, "max_positions": max_positions,
            "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "logit_scale": logit_scale,
            "logit_softcap": softcap, "layers": list(layers)}


def tensor_shapes(config: dict) -> dict:
    w = config["width"]
    out = {"embed": (config["vocab"], w), "pos": (config["max_positions"], w), "final.norm": (w,),
           "head": (config["vocab"], w)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        out[f"l{i}.norm1"] = (w,)
        if layer["type"] == "hgrn2":
            n, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({p + "q": (n, w), p + "f": (n, w), p + "f.b": (n,), p + "lower": (n,), p + "v": (nv, w),
                        p + "norm": (m["vdim"],), p + "o": (w, nv)})
        else:
            a, b = m["left"], m["right"]
            for name, rows in (("q", a["heads"] * a["dim"]), ("k", a["kv_heads"] * a["dim"]), ("v", a["kv_heads"] * a["vdim"])):
                out.update({f"{p}left.{name}": (rows, w), f"{p}left.{name}.b": (rows,), f"{p}left.{name}.conv": (rows, a["conv"])})
            out.update({p + "left.talk": (a["heads"], a["heads"]), p + "left.o": (w, a["heads"] * a["vdim"])})
            for name, rows in (("q", b["kv_heads"] * b["dim"]), ("k", b["kv_heads"] * b["dim"]), ("v", b["heads"] * b["vdim"])):
                out.update({f"{p}right.{name}": (rows, w), f"{p}right.{name}.conv": (rows, b["conv"])})
            out.update({p + "right.b": (b["heads"], w), p + "right.a": (b["heads"], w), p + "right.A_log": (b["heads"],),
                        p + "right.dt_bias": (b["heads"],), p + "right.norm": (b["vdim"],),
                        p + "right.g": (b["heads"] * b["vdim"], w), p + "right.o": (w, b["heads"] * b["vdim"])})
        mlp, q = layer.get("mlp"), f"l{i}.mlp."
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out.update({q + "gate": (mlp["ff"], w), q + "up": (mlp["ff"], w), q + "down": (w, mlp["ff"])})
        else:
            f = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out.update({f"{q}e{e}.gate": (f, w), f"{q}e{e}.up": (f, w), f"{q}e{e}.down": (w, f)})
            out[q + "router"] = (mlp["router"]["experts"], w)
            if mlp.get("shared"):
                f = mlp["shared"]["ff"]
                out.update({q + "shared.gate": (f, w), q + "shared.up": (f, w), q + "shared.down": (w, f),
                            q + "shared.sg": (1, w)})
    return out


def random_model(config: dict, seed: int = 0, spread: float = 1.0) -> dict:
    """Random tensors (torch, fp32 holding bf16-exact values) with checkpoint names; ``spread`` widens the head so
    that greedy choices are decided by more than rounding."""
    import torch

    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "talk":
            t = 0.3 * torch.randn(shape, generator=g) + 0.7 * torch.eye(shape[0])
        elif leaf == "lower":
            t = 0.9 * torch.rand(shape, generator=g)
        elif name == "pos":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "head":
            t = spread * torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif leaf == "router":
            t = 3.0 * torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif leaf in ("A_log", "dt_bias"):
            t = -1.0 + 0.8 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16).float()
    return out
