"""Typed configuration of the Kokolorn decoder, read from config.json.

A Kokolorn model is a list of pre-norm layers, x <- x + mixer(norm1(x)); x <- x + mlp(norm2(x)), with norm weights
stored around zero.  A run of the layers may be passed through several times with the same tensors; at the head of
every pass the stream is mixed with the embedding output again.  Everything that may differ between two models of
the design is in config.json::

    architecture        "Kokolorn"
    vocab, width        vocabulary and residual width
    norm.eps            epsilon of every RMS norm
    embedding.scale     factor on the looked-up rows (the output head reads the table without it)
    loop                absent, or {start, stop, times}: layers start..stop-1 run ``times`` times in a row
    layers[i].type      "attention", "delta" or "parallel"
    layers[i].mixer     attention: heads, kv_heads, dim, vdim, scale, q_temp {coef, every}
                        delta:     heads, kv_heads, dim, vdim, conv (taps)
                        parallel:  left  {heads, kv_heads, dim, vdim, scale, q_temp {coef, every}, bias_max}
                                   right {heads, vdim, state, groups, norm_groups, conv (taps)}
    layers[i].mlp       null; {"kind": "dense", "ff", "limit"}; or {"kind": "moe", "expert": {"ff"},
                        "router": {"experts", "top"}, "shared": {"ff"} (absent or null: none)}

The design states no longest sequence: the engine's ``context`` alone bounds a request.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .common import ConfigError
from .lepizen import _int, _number

ARCHITECTURE = "Kokolorn"
MAX_TAPS = 16


@dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: int

    def to_dict(self) -> Dict[str, Any]:
        return {"coef": self.coef, "every": self.every}


@dataclass(frozen=True)
class KeyedAttention:
    """Softmax attention whose values are its keys as projected; ``bias_max`` (the left branch of a parallel mixer):
    the distance at which the learned bias by distance reaches its last row."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[QueryTemperature]
    bias_max: Optional[float] = None

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                               "scale": self.scale}
        if self.q_temp is not None:
            out["q_temp"] = self.q_temp.to_dict()
        if self.bias_max is not None:
            out["bias_max"] = self.bias_max
        return out


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class StateSpaceMixer:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "norm_groups": self.norm_groups, "conv": self.conv}


@dataclass(frozen=True)
class ParallelMixer:
    left: KeyedAttention
    right: StateSpaceMixer

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class DenseFF:
    ff: int
    limit: float

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class ExpertsFF:
    ff: int
    experts: int
    top: int
    shared_ff: Optional[int]

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int

    def to_dict(self) -> Dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class KokolornLayer:
    kind: str                   # "attention", "delta" or "parallel"
    mixer: Any
    mlp: Any                    # None, DenseFF or ExpertsFF


def _object(where: str, raw: Dict[str, Any], key: str) -> Dict[str, Any]:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: missing object {where}'{key}'")
    return value


def _taps(where: str, m: Dict[str, Any]) -> int:
    taps = _int(where, m, "conv")
    if taps > MAX_TAPS:
        raise ConfigError(f"config.json: {where}'conv' has {taps} taps; at most {MAX_TAPS}")
    return taps


def _keyed_attention(where: str, m: Dict[str, Any], biased: bool) -> KeyedAttention:
    heads, kv_heads = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv_heads} kv_heads")
    dim, vdim = _int(where, m, "dim"), _int(where, m, "vdim")
    if vdim != dim:
        raise ConfigError(f"config.json: {where}the values are the keys, so 'vdim' {vdim} must equal 'dim' {dim}")
    temp = None
    if m.get("q_temp") is not None:
        t = _object(where, m, "q_temp")
        temp = QueryTemperature(coef=_number(where + "q_temp.", t, "coef", positive=False), every=_int(where + "q_temp.", t, "every"))
    bias_max = None
    if biased:
        bias_max = _number(where, m, "bias_max")
    return KeyedAttention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_number(where, m, "scale"), q_temp=temp,
                          bias_max=bias_max)


def _delta(where: str, m: Dict[str, Any]) -> DeltaMixer:
    heads, kv_heads = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv_heads} kv_heads")
    dim = _int(where, m, "dim")
    if dim > 256:
        raise ConfigError(f"config.json: {where}'dim' {dim}: the recurrence takes keys of up to 256 numbers")
    return DeltaMixer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_int(where, m, "vdim"), conv=_taps(where, m))


def _state_space(where: str, m: Dict[str, Any], width: int) -> StateSpaceMixer:
    heads, groups, parts = _int(where, m, "heads"), _int(where, m, "groups"), _int(where, m, "norm_groups")
    vdim, state = _int(where, m, "vdim"), _int(where, m, "state")
    if heads % groups:
        raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {groups} groups")
    if (heads * vdim) % parts:
        raise ConfigError(f"config.json: {where}{parts} norm_groups do not divide the inner width {heads * vdim}")
    if state > 256:
        raise ConfigError(f"config.json: {where}'state' {state}: the recurrence takes states of up to 256 rows")
    return StateSpaceMixer(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=parts, conv=_taps(where, m))


def _mlp(where: str, mlp: Any) -> Any:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}'mlp' must be null or an object")
    kind = mlp.get("kind")
    if kind == "dense":
        return DenseFF(ff=_int(where + "mlp.", mlp, "ff"), limit=_number(where + "mlp.", mlp, "limit"))
    if kind == "moe":
        router = _object(where + "mlp.", mlp, "router")
        experts, top = _int(where + "mlp.router.", router, "experts"), _int(where + "mlp.router.", router, "top")
        if top > experts:
            raise ConfigError(f"config.json: {where}mlp.router takes {top} of {experts} experts")
        if experts > 1024:
            raise ConfigError(f"config.json: {where}mlp.router.experts {experts}: the router takes up to 1024")
        shared = mlp.get("shared")
        shared_ff = None if shared is None else _int(where + "mlp.shared.", _object(where + "mlp.", mlp, "shared"), "ff")
        return ExpertsFF(ff=_int(where + "mlp.expert.", _object(where + "mlp.", mlp, "expert"), "ff"), experts=experts,
                         top=top, shared_ff=shared_ff)
    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' or 'moe', got {kind!r}")


@dataclass(frozen=True)
class KokolornConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[KokolornLayer, ...]
    loop: Optional[Loop]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def run_order(self) -> Tuple[Tuple[int, Optional[int]], ...]:
        """(layer, the pass it opens or None) in the order the layers run."""
        count = len(self.layers)
        if self.loop is None:
            return tuple((n, None) for n in range(count))
        order = [(n, None) for n in range(self.loop.start)]
        for t in range(self.loop.times):
            order += [(n, t if n == self.loop.start else None) for n in range(self.loop.start, self.loop.stop)]
        return tuple(order + [(n, None) for n in range(self.loop.stop, count)])

    @staticmethod
    def from_dict(raw: Dict[str, Any]) -> "KokolornConfig":
        vocab = _int("", raw, "vocab")
        if vocab >= 2 ** 31:
            raise ConfigError(f"config.json: vocab {vocab} does not fit 32-bit token ids")
        width = _int("", raw, "width")
        eps = _number("norm.", _object("", raw, "norm"), "eps")
        scale = 1.0
        if raw.get("embedding") is not None:
            scale = _number("embedding.", _object("", raw, "embedding"), "scale", positive=False)
        listed = raw.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{index}] must be an object")
            kind = entry.get("type")
            m = _object(where, entry, "mixer")
            if kind == "attention":
                mixer: Any = _keyed_attention(where + "mixer.", m, biased=False)
            elif kind == "delta":
                mixer = _delta(where + "mixer.", m)
            elif kind == "parallel":
                mixer = ParallelMixer(left=_keyed_attention(where + "mixer.left.", _object(where + "mixer.", m, "left"), biased=True),
                                      right=_state_space(where + "mixer.right.", _object(where + "mixer.", m, "right"), width))
            else:
                raise ConfigError(f"config.json: {where}'type' must be 'attention', 'delta' or 'parallel', got {kind!r}")
            layers.append(KokolornLayer(kind=kind, mixer=mixer, mlp=_mlp(where, entry.get("mlp"))))
        loop = None
        if raw.get("loop") is not None:
            lp = _object("", raw, "loop")
            loop = Loop(start=_int("loop.", lp, "start", minimum=0), stop=_int("loop.", lp, "stop"), times=_int("loop.", lp, "times"))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop runs layers {loop.start}..{loop.stop - 1} of {len(layers)}")
        return KokolornConfig(vocab=vocab, width=width, eps=eps, embedding_scale=scale, layers=tuple(layers), loop=loop)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                               "embedding": {"scale": self.embedding_scale},
                               "layers": [{"type": layer.kind, "mixer": layer.mixer.to_dict(),
                                           "mlp": None if layer.mlp is None else layer.mlp.to_dict()} for layer in self.layers]}
        if self.loop is not None:
            out["loop"] = self.loop.to_dict()
        return out
