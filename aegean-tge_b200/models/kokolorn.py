"""The Kokolorn decoder as a ModelSpec, and its random weights.

Every layer is pre-norm, x <- x + mixer(n1(x)); x <- x + mlp(n2(x)), the norms' weights stored around zero
(``rmsnorm`` with ``unit_offset``).  The embedding is scaled; the head reads the same table unscaled.  A run of
layers may be passed through several times: the later passes are layers that run an earlier layer's parts with a
cache and state of their own (``LayerSpec.weights_from``), and the layer that opens a pass has an ``entry``, the
stream step ``reinject`` (x <- Win [x; x0] + step[t], x0 the embedding output).

Mixers: "attention" is ``gqa_attention`` with ``values: "keys"`` (the values are the keys as projected, before the
keys' norm), a per-head norm of q and k, a temperature on the queries and no rotation; "delta" is
``gated_delta_rule``; "parallel" is ``mixer_sum`` with ``normalize`` (each branch's output over its root mean
square, times a weight, times 1/2) of a ``gqa_attention`` with a learned bias by distance and a ``state_space``
mixer.  Feed-forwards: ``clamped_glu``, or ``routed_experts`` with a router bias and a ``dense_mlp`` every token uses.

Checkpoint tensor names: ``embed``, ``final.norm``, ``loop.in``, ``loop.step``; per layer i ``l<i>.norm1``,
``l<i>.norm2``; attention ``l<i>.mix.{q,k,o}``, ``l<i>.mix.{q,k}.b``, ``l<i>.mix.{q,k}.norm``; delta
``l<i>.mix.{q,k,v,g,b,a,o}``, ``l<i>.mix.{q,k,v}.conv``, ``l<i>.mix.{A_log,dt_bias,norm}``; parallel
``l<i>.mix.left.{q,k,o}``, ``l<i>.mix.left.{q,k,o}.b``, ``l<i>.mix.left.rel``, ``l<i>.mix.right.{in,conv,conv.b,dt_bias,
A_log,D,norm,o}``, ``l<i>.mix.{left,right}.out``; dense ``l<i>.mlp.{gate,up,down}``; experts ``l<i>.mlp.e<j>.{up,down}``,
``l<i>.mlp.router``, ``l<i>.mlp.router.b``, ``l<i>.mlp.shared.{up,down}``.
"""
from __future__ import annotations

from typing import Dict, Iterator, Optional, Tuple

from ..config.kokolorn import (ARCHITECTURE, DeltaMixer, DenseFF, ExpertsFF, KeyedAttention, KokolornConfig, ParallelMixer,
                               StateSpaceMixer)
from ..config.model_spec import LayerSpec, ModelSpec, PartSpec
from ..registry import Architecture, register_architecture
from ..weights.draws import Draw, normal, uniform

NO_POSITION_LIMIT = 2 ** 31 - 1      # the design states no longest sequence
SWISH_ALPHA = 1.702                  # the dense feed-forward's gate is g sigmoid(1.702 g)
UNIT_EPS = 1e-6                      # q and k of the delta rule: x / sqrt(sum x^2 + 1e-6)
def rel_rows(bias_max: float) -> int:
    """Rows of the bias by distance in models drawn at random (a checkpoint's table brings its own count)."""
    return 32 if bias_max >= 64.0 else 16


def _norm(config: KokolornConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"size": config.width, "eps": config.eps, "unit_offset": True}, {"weight": name})


def _keyed_attention(config: KokolornConfig, m: KeyedAttention, prefix: str) -> PartSpec:
    params = {"hidden_size": config.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "scale": m.scale,
              "qkv_bias": True, "values": "keys", "position": PartSpec("none")}
    weights = {"q.weight": prefix + "q", "q.bias": prefix + "q.b", "k.weight": prefix + "k", "k.bias": prefix + "k.b",
               "o.weight": prefix + "o"}
    if m.q_temp is not None:
        params["q_temp"] = {"coef": m.q_temp.coef, "every": m.q_temp.every}
    if m.bias_max is None:
        params.update(o_bias=False, qk_norm={"scope": "head", "eps": config.eps})
        weights.update({"q_norm.weight": prefix + "q.norm", "k_norm.weight": prefix + "k.norm"})
    else:
        params.update(o_bias=True, distance_bias={"far": m.bias_max})     # the table's own shape gives its rows
        weights.update({"o.bias": prefix + "o.b", "rel": prefix + "rel"})
    return PartSpec("gqa_attention", params, weights)


def _delta(config: KokolornConfig, m: DeltaMixer, prefix: str) -> PartSpec:
    params = {"hidden_size": config.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
              "taps": m.conv, "eps": config.eps, "unit_eps": UNIT_EPS}
    weights = {f"{t}.weight": prefix + t for t in ("q", "k", "v", "g", "b", "a", "o")}
    weights.update({f"{t}.conv.weight": f"{prefix}{t}.conv" for t in ("q", "k", "v")})
    weights.update({"A_log": prefix + "A_log", "dt_bias": prefix + "dt_bias", "norm.weight": prefix + "norm"})
    return PartSpec("gated_delta_rule", params, weights)


def _state_space(config: KokolornConfig, m: StateSpaceMixer, prefix: str) -> PartSpec:
    params = {"hidden_size": config.width, "heads": m.heads, "value_dim": m.vdim, "state": m.state, "groups": m.groups,
              "norm_groups": m.norm_groups, "taps": m.conv, "eps": config.eps}
    weights = {"in.weight": prefix + "in", "conv.weight": prefix + "conv", "conv.bias": prefix + "conv.b",
               "dt_bias": prefix + "dt_bias", "A_log": prefix + "A_log", "D": prefix + "D", "norm.weight": prefix + "norm",
               "o.weight": prefix + "o"}
    return PartSpec("state_space", params, weights)


def _mixer(config: KokolornConfig, n: int) -> PartSpec:
    layer, prefix = config.layers[n], f"l{n}.mix."
    if layer.kind == "attention":
        return _keyed_attention(config, layer.mixer, prefix)
    if layer.kind == "delta":
        return _delta(config, layer.mixer, prefix)
    left = _keyed_attention(config, layer.mixer.left, prefix + "left.")
    right = _state_space(config, layer.mixer.right, prefix + "right.")
    weights = {f"left.{k}": v for k, v in left.weights.items()}
    weights.update({f"right.{k}": v for k, v in right.weights.items()})
    weights.update({"left.out_norm.weight": prefix + "left.out", "right.out_norm.weight": prefix + "right.out"})
    return PartSpec("mixer_sum", {"branches": (("left", left, 0.5), ("right", right, 0.5)),
                                  "normalize": {"eps": config.eps, "hidden_size": config.width}}, weights)


def _feed_forward(config: KokolornConfig, n: int) -> Optional[PartSpec]:
    mlp, prefix = config.layers[n].mlp, f"l{n}.mlp."
    if mlp is None:
        return None
    if isinstance(mlp, DenseFF):
        return PartSpec("clamped_glu", {"hidden_size": config.width, "intermediate_size": mlp.ff, "limit": mlp.limit,
                                        "alpha": SWISH_ALPHA, "up_offset": 1.0},
                        {"gate.weight": prefix + "gate", "up.weight": prefix + "up", "down.weight": prefix + "down"})
    assert isinstance(mlp, ExpertsFF)
    weights = {"router.weight": prefix + "router", "router.bias": prefix + "router.b"}
    for e in range(mlp.experts):
        weights[f"experts.{e}.up.weight"] = f"{prefix}e{e}.up"
        weights[f"experts.{e}.down.weight"] = f"{prefix}e{e}.down"
    shared = None
    if mlp.shared_ff is not None:
        shared = PartSpec("dense_mlp", {"hidden_size": config.width, "intermediate_size": mlp.shared_ff,
                                        "activation": "relu_squared", "bias": False})
        weights.update({"shared.up.weight": prefix + "shared.up", "shared.down.weight": prefix + "shared.down"})
    return PartSpec("routed_experts", {"hidden_size": config.width, "intermediate_size": mlp.ff, "experts": mlp.experts,
                                       "top": mlp.top, "activation": "relu_squared", "correction": False,
                                       "router_bias": True, "shared": shared}, weights)


def build_spec(config: KokolornConfig) -> ModelSpec:
    width = config.width
    layers, schedule = [], []
    own = [(_mixer(config, n), _feed_forward(config, n)) for n in range(len(config.layers))]
    def layer_spec(n: int, entry: Optional[PartSpec], source: Optional[int]) -> LayerSpec:
        mixer, ffn = own[n]
        norm2 = _norm(config, f"l{n}.norm2") if ffn is not None else None
        return LayerSpec("pre_norm", mixer, ffn, _norm(config, f"l{n}.norm1"), norm2, weights_from=source, entry=entry)
    entries = {}
    for n, opens in config.run_order():
        if opens is not None:
            entries[(n, opens)] = PartSpec("reinject", {"hidden_size": width, "index": opens, "count": config.loop.times},
                                           {"weight": "loop.in", "step": "loop.step"})
    # every layer's first visit is the layer itself, in the file's order; later passes follow as borrowed layers
    passes_seen: Dict[int, int] = {}
    for n in range(len(config.layers)):
        opens = 0 if (config.loop is not None and n == config.loop.start) else None
        layers.append(layer_spec(n, entries.get((n, opens)) if opens is not None else None, None))
    for n, opens in config.run_order():
        visit = passes_seen.get(n, 0)
        passes_seen[n] = visit + 1
        if visit == 0:
            schedule.append(n)
            continue
        layers.append(layer_spec(n, entries.get((n, opens)) if opens is not None else None, n))
        schedule.append(len(layers) - 1)
    sizes = {"vocab_size": config.vocab, "hidden_size": width}
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=config.vocab, max_positions=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(schedule),
        embedding=PartSpec("token_embedding", {**sizes, "scale": config.embedding_scale}, {"weight": "embed"}),
        final_norm=_norm(config, "final.norm"),
        head=PartSpec("linear_head", sizes, {"weight": "embed"}))


def random_plan(config: KokolornConfig) -> Iterator[Tuple[str, Tuple[int, ...], str, Draw]]:
    """(name, shape, role, draw) of every checkpoint tensor.  Projections N(0, 1/sqrt(fan-in)), the layers' norm weights
    U(-0.1, 0.1) (they are stored around zero), plain norm weights 1 + U(-0.1, 0.1), convolution taps U(-0.5, 0.5),
    decay logarithms U(-3, -1), step biases U(-1, 1), the bias by distance N(0, 0.5)."""
    w = config.width
    yield "embed", (config.vocab, w), "matrix", normal(1.0)
    if config.loop is not None:
        yield "loop.in", (w, 2 * w), "matrix", normal((2 * w) ** -0.5)
        yield "loop.step", (config.loop.times, w), "vector", normal(0.1)
    for n, layer in enumerate(config.layers):
        p, m = f"l{n}.", layer.mixer
        yield p + "norm1", (w,), "vector", uniform(-0.1, 0.1)
        if layer.mlp is not None:
            yield p + "norm2", (w,), "vector", uniform(-0.1, 0.1)
        if isinstance(m, KeyedAttention) or isinstance(m, ParallelMixer):
            a = m if isinstance(m, KeyedAttention) else m.left
            q = p + ("mix." if isinstance(m, KeyedAttention) else "mix.left.")
            yield q + "q", (a.heads * a.dim, w), "matrix", normal(w ** -0.5)
            yield q + "q.b", (a.heads * a.dim,), "vector", normal(0.1)
            yield q + "k", (a.kv_heads * a.dim, w), "matrix", normal(w ** -0.5)
            yield q + "k.b", (a.kv_heads * a.dim,), "vector", normal(0.1)
            yield q + "o", (w, a.heads * a.vdim), "matrix", normal((a.heads * a.vdim) ** -0.5)
            if a.bias_max is None:
                yield q + "q.norm", (a.dim,), "vector", uniform(0.9, 1.1)
                yield q + "k.norm", (a.dim,), "vector", uniform(0.9, 1.1)
            else:
                yield q + "o.b", (w,), "vector", normal(0.1)
                yield q + "rel", (rel_rows(a.bias_max), a.heads), "vector", normal(0.5)
        if isinstance(m, DeltaMixer):
            q = p + "mix."
            for t, rows in (("q", m.kv_heads * m.dim), ("k", m.kv_heads * m.dim), ("v", m.heads * m.vdim)):
                yield q + t, (rows, w), "matrix", normal(w ** -0.5)
                yield f"{q}{t}.conv", (rows, m.conv), "vector", uniform(-0.5, 0.5)
            yield q + "g", (m.heads * m.vdim, w), "matrix", normal(w ** -0.5)
            yield q + "b", (m.heads, w), "matrix", normal(w ** -0.5)
            yield q + "a", (m.heads, w), "matrix", normal(w ** -0.5)
            yield q + "A_log", (m.heads,), "vector", uniform(-3.0, -1.0)
            yield q + "dt_bias", (m.heads,), "vector", uniform(-1.0, 1.0)
            yield q + "norm", (m.vdim,), "vector", uniform(0.9, 1.1)
            yield q + "o", (w, m.heads * m.vdim), "matrix", normal((m.heads * m.vdim) ** -0.5)
        if isinstance(m, ParallelMixer):
            r, q = m.right, p + "mix.right."
            inner, channels = r.heads * r.vdim, r.heads * r.vdim + 2 * r.groups * r.state
            yield q + "in", (inner + channels + r.heads, w), "matrix", normal(w ** -0.5)
            yield q + "conv", (channels, r.conv), "vector", uniform(-0.5, 0.5)
            yield q + "conv.b", (channels,), "vector", normal(0.1)
            yield q + "dt_bias", (r.heads,), "vector", uniform(-1.0, 1.0)
            yield q + "A_log", (r.heads,), "vector", uniform(-3.0, -1.0)
            yield q + "D", (r.heads,), "vector", uniform(0.5, 1.5)
            yield q + "norm", (inner,), "vector", uniform(0.9, 1.1)
            yield q + "o", (w, inner), "matrix", normal(inner ** -0.5)
            yield p + "mix.left.out", (w,), "vector", uniform(0.9, 1.1)
            yield p + "mix.right.out", (w,), "vector", uniform(0.9, 1.1)
        if isinstance(layer.mlp, DenseFF):
            yield p + "mlp.gate", (layer.mlp.ff, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.up", (layer.mlp.ff, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.down", (w, layer.mlp.ff), "matrix", normal(layer.mlp.ff ** -0.5)
        elif isinstance(layer.mlp, ExpertsFF):
            r = layer.mlp
            yield p + "mlp.router", (r.experts, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.router.b", (r.experts,), "vector", normal(0.1)
            for e in range(r.experts):
                yield f"{p}mlp.e{e}.up", (r.ff, w), "matrix", normal(w ** -0.5)
                yield f"{p}mlp.e{e}.down", (w, r.ff), "matrix", normal(r.ff ** -0.5)
            if r.shared_ff is not None:
                yield p + "mlp.shared.up", (r.shared_ff, w), "matrix", normal(w ** -0.5)
                yield p + "mlp.shared.down", (w, r.shared_ff), "matrix", normal(r.shared_ff ** -0.5)
    yield "final.norm", (w,), "vector", uniform(-0.1, 0.1)


register_architecture(Architecture(name=ARCHITECTURE, parse_config=KokolornConfig.from_dict, build_spec=build_spec,
                                   random_plan=random_plan))
