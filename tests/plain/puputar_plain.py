"""A plain, slow Puputar decoder in numpy float64: whole sequences, no cache, one function per mechanism.

It is the oracle of the Puputar tests and shares no code with the package.  ``config`` is the dictionary that
config.json holds, ``weights`` maps tensor names to float64 arrays.

The design, in this file's notation.  The stream starts as ``x = gn(E[token]) * w_embed`` with ``gn`` the RMS
norm taken separately over ``G`` equal consecutive parts of a row.  Layer ``l``:

    a   = gn(x) * w1            b = gn(x) * w2
    a~  = a + (a_prev - a) * mu           (a_prev: the previous token's ``a``, zeros for the first token)
    x  <- x + mixer(a~) + ff(b)

Mixer (latent attention): ``cq = rms(Wdq a~) * gq``, ``q = Wuq cq`` (per head ``[dim | rot_dim]``);
``[c_raw | kr] = Wdkv a~``, ``c = rms(c_raw) * gkv``; per head ``k = Wuk c``, ``v = Wuv c``; the ``rot_dim`` parts
of q and the one shared ``kr`` are rotated in neighbouring pairs; ``s_ij = scale (q_i . k_j + qr_i . kr_j)`` for
``j <= i``, softmax, ``o_i = sum_j p_ij v_j``; the heads' outputs are gated by ``sigmoid(Wg a~)`` (one gate per
head, or one per element) and multiplied by ``Wo``.  A layer may read the ``c`` and rotated ``kr`` of an earlier
layer instead of making its own.

Feed-forward: ``Wdown act(Wup b + bup) + bdown`` with the two-parameter activation of :func:`xielu`, or a mixture
of small experts ``Wdown relu(Wup b)^2`` chosen by :func:`route`, of which the last ``identity`` are the input itself.
"""
from __future__ import annotations

import numpy as np


# ----------------------------------------------------------------------------------------------- norms
def rms_norm(x, weight, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def group_norm(x, weight, groups, eps):
    """Each of ``groups`` equal consecutive parts of a row over its own root mean square; then the weight."""
    x = np.asarray(x, dtype=np.float64)
    parts = x.reshape(x.shape[:-1] + (groups, x.shape[-1] // groups))
    parts = parts / np.sqrt(np.mean(parts * parts, axis=-1, keepdims=True) + eps)
    return parts.reshape(x.shape) * weight


# ----------------------------------------------------------------------------------------------- token shift
def token_shift(h, mu):
    """Row t becomes h_t + (h_(t-1) - h_t) * mu, with zeros before the first row."""
    before = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (before - h) * mu


# ----------------------------------------------------------------------------------------------- rotation
def rotate_pairs(x, positions, base, dims):
    """x [T, ..., D]: elements 2i and 2i+1 (i < dims/2) are turned by the angle position * base^(-2i/dims)."""
    x = np.array(x, dtype=np.float64)
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    cos, sin = np.cos(angle).reshape(shape), np.sin(angle).reshape(shape)
    u, v = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = u * cos - v * sin
    x[..., 1:dims:2] = v * cos + u * sin
    return x


# ----------------------------------------------------------------------------------------------- attention
def causal_softmax_attention(q, k, v, scale):
    """q [T, H, D], k [T, H, D], v [T, H, V] -> [T, H, V]; row i sees rows j <= i."""
    tokens = q.shape[0]
    scores = np.einsum("ihd,jhd->hij", q, k) * scale
    mask = np.tril(np.ones((tokens, tokens), dtype=bool))
    scores = np.where(mask[None], scores, -np.inf)
    scores = scores - scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p = p / p.sum(axis=-1, keepdims=True)
    return np.einsum("hij,jhv->ihv", p, v)


def latent_kv(h, w, prefix, m, eps, positions):
    """The latent c [T, kv_rank] and the rotated shared key part [T, rot_dim] of a layer that makes its own."""
    rank = m["kv_rank"]
    down = h @ w[prefix + "dkv"].T
    c = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    shared = rotate_pairs(down[:, rank:], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, shared


def latent_attention(h, w, prefix, m, eps, positions, gate, kv):
    """``gate``: "head" (one logistic gate per head) or "element" (one per output element); ``kv``: (c, rotated
    shared key part), this layer's own or an earlier layer's."""
    tokens = h.shape[0]
    heads, dim, rot, vdim = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, shared = kv
    cq = rms_norm(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps)
    q = (cq @ w[prefix + "uq"].T).reshape(tokens, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[prefix + "uk"].T).reshape(tokens, heads, dim)
    v = (c @ w[prefix + "uv"].T).reshape(tokens, heads, vdim)
    k = np.concatenate([k_plain, np.broadcast_to(shared[:, None, :], (tokens, heads, rot))], axis=-1)
    o = causal_softmax_attention(np.concatenate([q_plain, q_rot], axis=-1), k, v, m["scale"])
    g = 1.0 / (1.0 + np.exp(-(h @ w[prefix + "g"].T)))
    if gate == "head":
        o = o * g[:, :, None]
    else:
        o = o * g.reshape(tokens, heads, vdim)
    return o.reshape(tokens, heads * vdim) @ w[prefix + "o"].T


# ----------------------------------------------------------------------------------------------- feed-forward
def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - z) + 0.5 * z
    return np.where(z > 0, pos, neg)


def dense_ff(h, w, prefix):
    p, q = w[prefix + "act"]
    inner = xielu(h @ w[prefix + "up"].T + w[prefix + "up.b"], p, q)
    return inner @ w[prefix + "down"].T + w[prefix + "down.b"]


def route(h, router, correction, top, group_count, group_keep):
    """-> (ids [T, top], weights [T, top]).  Softmax over all router outputs; the choice looks at score +
    correction, only inside the ``group_keep`` groups whose best such value is largest; the weights are the chosen
    experts' plain scores over their sum."""
    z = h @ router.T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    choice = s + correction
    tokens, outputs = choice.shape
    per = outputs // group_count
    best = choice.reshape(tokens, group_count, per).max(axis=-1)
    ids = np.zeros((tokens, top), dtype=np.int64)
    weights = np.zeros((tokens, top))
    for t in range(tokens):
        kept = np.argsort(-best[t], kind="stable")[:group_keep]
        allowed = np.full(outputs, -np.inf)
        for g in kept:
            allowed[g * per:(g + 1) * per] = choice[t, g * per:(g + 1) * per]
        ids[t] = np.argsort(-allowed, kind="stable")[:top]
        weights[t] = s[t, ids[t]] / (s[t, ids[t]].sum() + 1e-20)
    return ids, weights


def route_margin(h, router, correction, top, group_count, group_keep):
    """[T]: how far each row's choice is from another one: the smallest of (the last chosen value minus the best value
    left inside the kept groups) and (the last kept group's value minus the best group left out)."""
    z = h @ router.T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    choice = s / s.sum(axis=-1, keepdims=True) + correction
    tokens, outputs = choice.shape
    per = outputs // group_count
    ids, _ = route(h, router, correction, top, group_count, group_keep)
    out = np.full(tokens, np.inf)
    for t in range(tokens):
        best = np.sort(choice[t].reshape(group_count, per).max(axis=-1))[::-1]
        if group_keep < group_count:
            out[t] = best[group_keep - 1] - best[group_keep]
        kept = np.argsort(-choice[t].reshape(group_count, per).max(axis=-1), kind="stable")[:group_keep]
        left = [choice[t, i] for g in kept for i in range(g * per, (g + 1) * per) if i not in ids[t]]
        if left:
            out[t] = min(out[t], choice[t, ids[t]].min() - max(left))
    return out


def moe_ff(h, w, prefix, mlp, margins=None):
    """``margins``: a list that receives this layer's :func:`route_margin` (for tests that must know which rows a
    rounding could route elsewhere)."""
    r = mlp["router"]
    experts, identity = r["experts"], r.get("identity", 0)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    ids, weights = route(h, w[prefix + "router"], w[prefix + "correction"], r["top"], groups["count"], groups["keep"])
    if margins is not None:
        margins.append(route_margin(h, w[prefix + "router"], w[prefix + "correction"], r["top"], groups["count"], groups["keep"]))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(ids[t], weights[t]):
            if e >= experts:                       # one of the last ``identity`` outputs: the input itself
                out[t] += weight * h[t]
            else:
                inner = np.maximum(h[t] @ w[f"{prefix}e{e}.up"].T, 0.0) ** 2
                out[t] += weight * (inner @ w[f"{prefix}e{e}.down"].T)
    return out


# ----------------------------------------------------------------------------------------------- the model
def forward(config, w, tokens, return_layers=False, margins=None, shift=True):
    """Logits [T, vocab] of a whole sequence (and, on request, the stream after every layer [L, T, width]).
    ``margins``: a list that receives every routed layer's :func:`route_margin`; ``shift`` False leaves the token
    shift out (for tests of the tests)."""
    eps, groups = config["norm"]["eps"], config["norm"].get("groups", 1)
    positions = np.arange(len(tokens))
    x = group_norm(w["embed"][np.asarray(tokens)], w["embed.norm"], groups, eps)
    kept = {}
    streams = []
    for n, layer in enumerate(config["layers"]):
        p = f"l{n}."
        m = layer["mixer"]
        a = group_norm(x, w[p + "norm1"], groups, eps)
        if shift:
            a = token_shift(a, w[p + "shift"])
        mlp = layer.get("mlp")
        b = group_norm(x, w[p + "norm2"], groups, eps) if mlp is not None else None
        if m.get("kv_from") is None:
            kept[n] = latent_kv(a, w, p + "mix.", m, eps, positions)
            kv = kept[n]
        else:
            kv = kept[m["kv_from"]]
        gate = {"latent_attention": "head", "latent_attention_2": "element"}[layer["type"]]
        mixed = latent_attention(a, w, p + "mix.", m, eps, positions, gate, kv)
        if mlp is None:
            fed = 0.0
        elif mlp["kind"] == "dense":
            fed = dense_ff(b, w, p + "mlp.")
        else:
            fed = moe_ff(b, w, p + "mlp.", mlp, margins)
        x = x + (mixed + fed)
        streams.append(x.copy())
    logits = group_norm(x, w["final.norm"], groups, eps) @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
