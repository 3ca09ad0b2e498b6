"""Plain float64 implementation of the Kokolorn decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, numpy only; it shares no code
with the package.  ``weights`` maps tensor names to arrays, ``config`` is the parsed config.json.

    x0 = E[token] * s                                   (s = embedding.scale)
    layers before the loop, then ``times`` passes over layers start..stop-1 (same tensors), then the rest;
    at the head of pass t:  x <- Win [x; x0] + step[t]
    a layer:  x <- x + mixer(n1(x));  x <- x + ff(n2(x))     n(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
    logits = E n_final(x)

Mixers: "attention" (softmax attention whose values are the keys as projected, before the keys' norm; a
temperature on the queries that grows with the position), "delta" (the gated delta rule on a matrix state),
"parallel" (half the sum of a softmax attention with a bias by distance and a state-space recurrence, each
normalised over the width).  Feed-forwards: a clamped gated one, or a mixture of small experts with one that
every token uses.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np

F = np.float64


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """The plain weight."""
    return unit_rms(x.astype(F), eps) * weight.astype(F)


def layer_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """A layer's norm: its weight is stored around zero."""
    return unit_rms(x.astype(F), eps) * (1.0 + weight.astype(F))


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1.0 + np.exp(-z))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z: np.ndarray) -> np.ndarray:
    return np.logaddexp(0.0, z)


def short_conv(u: np.ndarray, w: np.ndarray, bias: Optional[np.ndarray] = None) -> np.ndarray:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j) (+ bias), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=F), u.astype(F)], axis=0)
    y = np.zeros((T, C), dtype=F)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j].astype(F)[None, :]
    if bias is not None:
        y += bias.astype(F)[None, :]
    return y


def query_temperature(positions: np.ndarray, coef: float, every: int) -> np.ndarray:
    """1 + coef * ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * np.log(np.floor((positions.astype(F) + 1.0) / every) + 1.0)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Distances below rows/2 have a row each; beyond, rows are spaced evenly in the logarithm up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def softmax_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                      bias: Optional[np.ndarray] = None, far: float = 0.0) -> np.ndarray:
    """q [T, H, d], k [T, G, d], v [T, G, dv]; causal; ``bias`` [rows, H] is looked up by the bucket of i - j and is
    not scaled.  Returns [T, H * dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), dtype=F)
    if bias is not None:                                   # by_distance[h, n]: the bias of the key n positions back
        by_distance = np.array([[bias[distance_bucket(n, bias.shape[0], far), h] for n in range(T)] for h in range(H)], dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, h]) * scale
            if bias is not None:
                s = s + by_distance[h, i::-1]
            w = np.exp(s - s.max())
            out[i, h] = (w / w.sum()) @ v[:i + 1, g]
    return out.reshape(T, -1)


def attention_mixer(h: np.ndarray, W: Dict[str, np.ndarray], p: str, m: dict, eps: float) -> np.ndarray:
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[p + "q"].astype(F).T + W[p + "q.b"].astype(F)).reshape(T, H, d)
    k = (h @ W[p + "k"].astype(F).T + W[p + "k.b"].astype(F)).reshape(T, G, d)
    v = k.copy()                                           # the values are the keys as projected
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    if m.get("q_temp") is not None:
        q = q * query_temperature(np.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    a = softmax_attention(q, k, v, m["scale"])
    return a @ W[p + "o"].astype(F).T


def delta_rule(q: np.ndarray, k: np.ndarray, v: np.ndarray, beta: np.ndarray, g: np.ndarray) -> np.ndarray:
    """One head: q, k [T, d], v [T, dv], beta, g [T].  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]), dtype=F)
    out = np.zeros((T, v.shape[1]), dtype=F)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h: np.ndarray, W: Dict[str, np.ndarray], p: str, m: dict, eps: float) -> np.ndarray:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].astype(F).T, W[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ W[p + "k"].astype(F).T, W[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ W[p + "v"].astype(F).T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].astype(F).T)
    g = np.exp(-np.exp(W[p + "A_log"].astype(F)) * softplus(h @ W[p + "a"].astype(F).T + W[p + "dt_bias"].astype(F)))
    gate = silu(h @ W[p + "g"].astype(F).T).reshape(T, H, dv)
    o = np.zeros((T, H, dv), dtype=F)
    for n in range(H):
        j = n // (H // G)
        o[:, n] = delta_rule(q[:, j], k[:, j], v[:, n], beta[:, n], g[:, n])
    o = unit_rms(o, eps) * W[p + "norm"].astype(F) * gate
    return o.reshape(T, -1) @ W[p + "o"].astype(F).T


def state_space(x: np.ndarray, B: np.ndarray, C: np.ndarray, dt: np.ndarray, a: float, D: float) -> np.ndarray:
    """One head: x [T, dv], B, C [T, N], dt [T].  S_t = exp(-a dt_t) S_(t-1) + dt_t B_t x_t^T; y_t = S_t^T C_t + D x_t."""
    T, dv = x.shape
    S = np.zeros((B.shape[1], dv), dtype=F)
    y = np.zeros((T, dv), dtype=F)
    for t in range(T):
        S = math.exp(-a * dt[t]) * S + dt[t] * np.outer(B[t], x[t])
        y[t] = S.T @ C[t] + D * x[t]
    return y


def state_space_mixer(h: np.ndarray, W: Dict[str, np.ndarray], p: str, m: dict, eps: float) -> np.ndarray:
    T = h.shape[0]
    H, dv, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * dv
    rows = h @ W[p + "in"].astype(F).T
    z = rows[:, :inner]
    xbc = silu(short_conv(rows[:, inner:2 * inner + 2 * G * N], W[p + "conv"], W[p + "conv.b"]))
    dt = softplus(rows[:, 2 * inner + 2 * G * N:] + W[p + "dt_bias"].astype(F))
    x = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    y = np.zeros((T, H, dv), dtype=F)
    for n in range(H):
        j = n // (H // G)
        y[:, n] = state_space(x[:, n], B[:, j], C[:, j], dt[:, n], math.exp(float(W[p + "A_log"][n])), float(W[p + "D"][n]))
    y = y.reshape(T, inner) * silu(z)                      # the gate comes before the norm
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"].astype(F)
    return y @ W[p + "o"].astype(F).T


def biased_attention_mixer(h: np.ndarray, W: Dict[str, np.ndarray], p: str, m: dict) -> np.ndarray:
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[p + "q"].astype(F).T + W[p + "q.b"].astype(F)).reshape(T, H, d)
    k = (h @ W[p + "k"].astype(F).T + W[p + "k.b"].astype(F)).reshape(T, G, d)
    if m.get("q_temp") is not None:
        q = q * query_temperature(np.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    a = softmax_attention(q, k, k, m["scale"], bias=W[p + "rel"].astype(F), far=float(m["bias_max"]))
    return a @ W[p + "o"].astype(F).T + W[p + "o.b"].astype(F)


def parallel_mixer(h: np.ndarray, W: Dict[str, np.ndarray], p: str, m: dict, eps: float) -> np.ndarray:
    left = biased_attention_mixer(h, W, p + "left.", m["left"])
    right = state_space_mixer(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


def dense_ff(h: np.ndarray, W: Dict[str, np.ndarray], p: str, limit: float) -> np.ndarray:
    g = np.minimum(h @ W[p + "gate"].astype(F).T, limit)
    u = np.clip(h @ W[p + "up"].astype(F).T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].astype(F).T


def expert(h: np.ndarray, W: Dict[str, np.ndarray], p: str) -> np.ndarray:
    return np.maximum(h @ W[p + "up"].astype(F).T, 0.0) ** 2 @ W[p + "down"].astype(F).T


def route(h: np.ndarray, W: Dict[str, np.ndarray], p: str, top: int, margins: Optional[list] = None):
    """(chosen experts [T, top], weights [T, top]): the largest logits, softmax over them alone.  ``margins`` collects,
    per token, how far the last chosen logit lies above the first one left out."""
    z = h @ W[p + "router"].astype(F).T + W[p + "router.b"].astype(F)
    ids = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    if margins is not None:
        ordered = -np.sort(-z, axis=-1)
        margins.append(ordered[:, top - 1] - ordered[:, top] if z.shape[1] > top else np.full(z.shape[0], np.inf))
    zs = np.take_along_axis(z, ids, axis=-1)
    w = np.exp(zs - zs.max(-1, keepdims=True))
    return ids, w / w.sum(-1, keepdims=True)


def moe_ff(h: np.ndarray, W: Dict[str, np.ndarray], p: str, mlp: dict, margins: Optional[list] = None) -> np.ndarray:
    ids, w = route(h, W, p, mlp["router"]["top"], margins)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]), dtype=F)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            out[t] += w[t, j] * expert(h[t:t + 1], W, f"{p}e{ids[t, j]}.")[0]
    if mlp.get("shared") is not None:
        out += expert(h, W, p + "shared.")
    return out


def run_order(config: dict) -> List[tuple]:
    """(layer, pass or None when the layer opens no pass) in the order the layers run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(n, None) for n in range(count)]
    order = [(n, None) for n in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(n, t if n == loop["start"] else None) for n in range(loop["start"], loop["stop"])]
    return order + [(n, None) for n in range(loop["stop"], count)]


def layer_forward(x: np.ndarray, W: Dict[str, np.ndarray], n: int, layer: dict, eps: float,
                  margins: Optional[list] = None) -> np.ndarray:
    p = f"l{n}."
    h = layer_norm(x, W[p + "norm1"], eps)
    kind = layer["type"]
    if kind == "attention":
        x = x + attention_mixer(h, W, p + "mix.", layer["mixer"], eps)
    elif kind == "delta":
        x = x + delta_mixer(h, W, p + "mix.", layer["mixer"], eps)
    elif kind == "parallel":
        x = x + parallel_mixer(h, W, p + "mix.", layer["mixer"], eps)
    else:
        raise ValueError(kind)
    mlp = layer.get("mlp")
    if mlp is None:
        return x
    h = layer_norm(x, W[p + "norm2"], eps)
    if mlp["kind"] == "dense":
        return x + dense_ff(h, W, p + "mlp.", mlp["limit"])
    return x + moe_ff(h, W, p + "mlp.", mlp, margins)


def forward(config: dict, W: Dict[str, np.ndarray], tokens, streams: Optional[list] = None,
            margins: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence; ``streams`` collects the stream after every layer run, ``margins`` every
    routed layer run's distances from another choice of experts."""
    eps = config["norm"]["eps"]
    E = W["embed"].astype(F)
    x0 = E[np.asarray(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    x = x0.copy()
    for n, opens in run_order(config):
        if opens is not None:
            x = np.concatenate([x, x0], axis=-1) @ W["loop.in"].astype(F).T + W["loop.step"].astype(F)[opens]
        x = layer_forward(x, W, n, config["layers"][n], eps, margins)
        if streams is not None:
            streams.append(x.copy())
    return layer_norm(x, W["final.norm"], eps) @ E.T
