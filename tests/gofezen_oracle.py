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


def forward(config: dict, tensors: dict, tokens, trace: list | None = None) -> np.ndarray:
    """``tokens`` of ONE sequence -> logits ``[T, vocab]``; ``trace`` collects the residual after every layer."""
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
