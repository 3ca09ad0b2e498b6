"""The Puputar decoder as a ModelSpec, and its random weights.

The stream starts from normalised embeddings, x = gn(E[token]) w_e, with gn the RMS norm taken in groups.  Every
layer is a parallel block with two norms of the same x: x <- x + mixer(shift(gn(x) w1)) + ff(gn(x) w2).  The mixer
reads its rows blended with the previous token's (token shift, a row of per-request state per layer) and is
attention over a latent cache with one logistic output gate per head (``latent_attention``) or per element
(``latent_attention_2``); a layer may read the cache entries of an earlier layer.  The feed-forward is dense with
biases and the two-parameter xIELU activation, a mixture of small squared-ReLU experts with identity experts, or
absent.  All of it is built from the engine's shared parts.

Checkpoint tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``head``, and per layer i ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.shift``, ``l<i>.mix.{dq,uq,dkv,uk,uv,g,o}``, ``l<i>.mix.{dq,dkv}.norm`` (no ``dkv`` tensors in
a layer that reads another's entries), ``l<i>.mlp.{up,down}`` with ``.b`` biases and ``l<i>.mlp.act``, or
``l<i>.mlp.router``, ``l<i>.mlp.correction`` and ``l<i>.mlp.e<k>.{up,down}``.
"""
from __future__ import annotations

from typing import Iterator, Tuple

from ..config.model_spec import LayerSpec, ModelSpec, PartSpec
from ..config.puputar import ARCHITECTURE, GATES, DenseFF, PuputarConfig, RoutedFF
from ..registry import Architecture, register_architecture
from ..weights.draws import Draw, normal, uniform

NO_POSITION_LIMIT = 2 ** 31 - 1      # the design states no longest sequence


def _norm(config: PuputarConfig, tensor: str, optional: bool = False) -> PartSpec:
    params = {"size": config.width, "eps": config.eps, "groups": config.groups}
    if optional:
        params["optional"] = True
    return PartSpec("group_rmsnorm", params, {"weight": tensor})


def _mixer(config: PuputarConfig, n: int) -> PartSpec:
    layer = config.layers[n]
    m = layer.mixer
    prefix = f"l{n}.mix."
    shared = m.kv_from is not None
    position = PartSpec("rope_interleaved", {"head_dim": m.rot_dim, "theta": m.rot_base, "rotary_dim": m.rot_dims}) \
        if m.rot_dim else PartSpec("none")
    weights = {"dq.weight": prefix + "dq", "dq_norm.weight": prefix + "dq.norm", "uq.weight": prefix + "uq",
               "uk.weight": prefix + "uk", "uv.weight": prefix + "uv", "g.weight": prefix + "g", "o.weight": prefix + "o"}
    if not shared:
        weights.update({"dkv.weight": prefix + "dkv", "dkv_norm.weight": prefix + "dkv.norm"})
    attention = PartSpec(
        "latent_attention",
        {"hidden_size": config.width, "heads": m.heads, "head_dim": m.dim, "rope_dim": m.rot_dim, "value_dim": m.vdim,
         "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": config.eps, "gate": GATES[layer.kind],
         "position": position, "shared_kv": shared},
        weights)
    wrapped = {"shift": f"l{n}.shift"}
    wrapped.update({f"inner.{local}": name for local, name in weights.items()})
    return PartSpec("shifted_mixer", {"hidden_size": config.width, "inner": attention}, wrapped)


def _feed_forward(config: PuputarConfig, n: int):
    mlp = config.layers[n].mlp
    prefix = f"l{n}.mlp."
    if mlp is None:
        return None
    if isinstance(mlp, DenseFF):
        return PartSpec("dense_mlp", {"hidden_size": config.width, "intermediate_size": mlp.ff, "activation": "xielu",
                                      "bias": True},
                        {"up.weight": prefix + "up", "up.bias": prefix + "up.b", "down.weight": prefix + "down",
                         "down.bias": prefix + "down.b", "act": prefix + "act"})
    assert isinstance(mlp, RoutedFF)
    weights = {"router.weight": prefix + "router", "correction": prefix + "correction"}
    for e in range(mlp.experts):
        weights[f"experts.{e}.up.weight"] = f"{prefix}e{e}.up"
        weights[f"experts.{e}.down.weight"] = f"{prefix}e{e}.down"
    return PartSpec("routed_experts",
                    {"hidden_size": config.width, "intermediate_size": mlp.ff, "experts": mlp.experts, "top": mlp.top,
                     "identity": mlp.identity, "group_count": mlp.group_count, "group_keep": mlp.group_keep,
                     "activation": "relu_squared", "correction": True},
                    weights)


def build_spec(config: PuputarConfig) -> ModelSpec:
    layers = []
    for n, layer in enumerate(config.layers):
        ffn = _feed_forward(config, n)
        # a layer without feed-forward has nothing that reads a second norm; a checkpoint may hold one all the same
        norm2 = _norm(config, f"l{n}.norm2", optional=ffn is None)
        layers.append(LayerSpec("parallel", _mixer(config, n), ffn, _norm(config, f"l{n}.norm1"), norm2,
                                cache_from=layer.mixer.kv_from))
    sizes = {"vocab_size": config.vocab, "hidden_size": config.width}
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=config.width, vocab_size=config.vocab, max_positions=NO_POSITION_LIMIT,
        layers=tuple(layers), schedule=tuple(range(len(layers))),
        embedding=PartSpec("token_embedding", {**sizes, "norm": _norm(config, "embed.norm")},
                           {"weight": "embed", "norm.weight": "embed.norm"}),
        final_norm=_norm(config, "final.norm"),
        head=PartSpec("linear_head", sizes, {"weight": "head"}))


def random_plan(config: PuputarConfig) -> Iterator[Tuple[str, Tuple[int, ...], str, Draw]]:
    """(name, shape, role, draw) of every checkpoint tensor.  Projections N(0, 1/sqrt(fan-in)), norm weights
    1 + U(-0.1, 0.1), shift weights U(0, 1), activation numbers U(-1, 1), router corrections U(-0.1, 0.1)."""
    w = config.width
    yield "embed", (config.vocab, w), "matrix", normal(1.0)
    yield "embed.norm", (w,), "vector", uniform(0.9, 1.1)
    for n, layer in enumerate(config.layers):
        p, m = f"l{n}.", layer.mixer
        yield p + "norm1", (w,), "vector", uniform(0.9, 1.1)
        if layer.mlp is not None:
            yield p + "norm2", (w,), "vector", uniform(0.9, 1.1)
        yield p + "shift", (w,), "vector", uniform(0.0, 1.0)
        yield p + "mix.dq", (m.q_rank, w), "matrix", normal(w ** -0.5)
        yield p + "mix.dq.norm", (m.q_rank,), "vector", uniform(0.9, 1.1)
        yield p + "mix.uq", (m.heads * (m.dim + m.rot_dim), m.q_rank), "matrix", normal(m.q_rank ** -0.5)
        if m.kv_from is None:
            yield p + "mix.dkv", (m.kv_rank + m.rot_dim, w), "matrix", normal(w ** -0.5)
            yield p + "mix.dkv.norm", (m.kv_rank,), "vector", uniform(0.9, 1.1)
        yield p + "mix.uk", (m.heads * m.dim, m.kv_rank), "matrix", normal(m.kv_rank ** -0.5)
        yield p + "mix.uv", (m.heads * m.vdim, m.kv_rank), "matrix", normal(m.kv_rank ** -0.5)
        gates = m.heads if GATES[layer.kind] == "head" else m.heads * m.vdim
        yield p + "mix.g", (gates, w), "matrix", normal(w ** -0.5)
        yield p + "mix.o", (w, m.heads * m.vdim), "matrix", normal((m.heads * m.vdim) ** -0.5)
        if isinstance(layer.mlp, DenseFF):
            yield p + "mlp.up", (layer.mlp.ff, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.up.b", (layer.mlp.ff,), "vector", normal(0.1)
            yield p + "mlp.down", (w, layer.mlp.ff), "matrix", normal(layer.mlp.ff ** -0.5)
            yield p + "mlp.down.b", (w,), "vector", normal(0.1)
            yield p + "mlp.act", (2,), "vector", uniform(-1.0, 1.0)
        elif isinstance(layer.mlp, RoutedFF):
            r = layer.mlp
            yield p + "mlp.router", (r.experts + r.identity, w), "matrix", normal(w ** -0.5)
            yield p + "mlp.correction", (r.experts + r.identity,), "vector", uniform(-0.1, 0.1)
            for e in range(r.experts):
                yield f"{p}mlp.e{e}.up", (r.ff, w), "matrix", normal(w ** -0.5)
                yield f"{p}mlp.e{e}.down", (w, r.ff), "matrix", normal(r.ff ** -0.5)
    yield "final.norm", (w,), "vector", uniform(0.9, 1.1)
    yield "head", (config.vocab, w), "matrix", normal(w ** -0.5)


register_architecture(Architecture(name=ARCHITECTURE, parse_config=PuputarConfig.from_dict, build_spec=build_spec,
                                   random_plan=random_plan))
