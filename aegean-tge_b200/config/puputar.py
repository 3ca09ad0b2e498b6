"""Typed configuration of the Puputar decoder, read from config.json.

A Puputar model is a list of parallel layers with two norms, x <- x + mixer(shift(norm1(x))) + mlp(norm2(x)): the
norms are RMS norms taken in groups, the mixer's input is blended with the previous token's (token shift), the mixer
is attention over a latent cache, and the feed-forward is dense or a mixture of experts.  Everything that may differ
between two models of the design is in config.json::

    architecture        "Puputar"
    vocab, width        vocabulary and residual width
    norm.eps            epsilon of every RMS norm (the layers', the embedding's, the final one, the latents')
    norm.groups         parts a row is cut into, each normalised on its own (absent: 1)
    layers[i].type      "latent_attention" (one output gate per head) or "latent_attention_2" (one per element)
    layers[i].mixer     heads, dim (plain query/key numbers per head), rot_dim (rotated ones), vdim, q_rank, kv_rank,
                        scale (multiplies q . k), rot {base, dims (rotated numbers of the rot_dim part)},
                        kv_from (optional: index of the layer whose cached latents and shared key part this one reads)
    layers[i].mlp       null; {"kind": "dense", "ff": inner width}; or {"kind": "moe", "expert": {"ff": inner width},
                        "router": {"experts", "top", "identity" (absent: 0), "groups": {"count", "keep"} (absent: none)}}

The design states no longest sequence: the engine's ``context`` alone bounds a request.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .common import ConfigError
from .lepizen import _int, _number

ARCHITECTURE = "Puputar"
GATES = {"latent_attention": "head", "latent_attention_2": "element"}


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                               "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale,
                               "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class DenseFF:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class RoutedFF:
    ff: int
    experts: int
    top: int
    identity: int = 0
    group_count: int = 1
    group_keep: int = 1

    def to_dict(self) -> Dict[str, Any]:
        router: Dict[str, Any] = {"experts": self.experts, "top": self.top, "identity": self.identity}
        if self.group_count > 1:
            router["groups"] = {"count": self.group_count, "keep": self.group_keep}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": router}


@dataclass(frozen=True)
class PuputarLayer:
    kind: str                     # "latent_attention" | "latent_attention_2"
    mixer: LatentMixer
    mlp: Any                      # None | DenseFF | RoutedFF

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.kind, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


def _mixer(where: str, raw: Any) -> LatentMixer:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where}'mixer' must be an object")
    w = where + "mixer."
    rot = raw.get("rot")
    rot_dim = _int(w, raw, "rot_dim", minimum=0)
    if rot_dim and not isinstance(rot, dict):
        raise ConfigError(f"config.json: {w}'rot' must be an object with base and dims")
    base, dims = (1.0, 0) if not rot_dim else (_number(w + "rot.", rot, "base"), _int(w + "rot.", rot, "dims", minimum=0))
    if dims % 2 or dims > rot_dim:
        raise ConfigError(f"config.json: {w}rot.'dims' must be even and at most rot_dim {rot_dim}, got {dims}")
    kv_from = raw.get("kv_from")
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
        raise ConfigError(f"config.json: {w}'kv_from' must be a layer index, got {kv_from!r}")
    return LatentMixer(heads=_int(w, raw, "heads"), dim=_int(w, raw, "dim"), rot_dim=rot_dim, vdim=_int(w, raw, "vdim"),
                       q_rank=_int(w, raw, "q_rank"), kv_rank=_int(w, raw, "kv_rank"), scale=_number(w, raw, "scale"),
                       rot_base=base, rot_dims=dims, kv_from=kv_from)


def _mlp(where: str, raw: Any):
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where}'mlp' must be null or an object")
    w = where + "mlp."
    kind = raw.get("kind")
    if kind == "dense":
        return DenseFF(ff=_int(w, raw, "ff"))
    if kind != "moe":
        raise ConfigError(f"config.json: {w}'kind' must be 'dense' or 'moe', got {kind!r}")
    expert, router = raw.get("expert"), raw.get("router")
    if not isinstance(expert, dict) or not isinstance(router, dict):
        raise ConfigError(f"config.json: {w}'expert' and 'router' must be objects")
    experts = _int(w + "router.", router, "experts", minimum=0)
    identity = _int(w + "router.", router, "identity", minimum=0) if "identity" in router else 0
    top = _int(w + "router.", router, "top")
    count = keep = 1
    groups = router.get("groups")
    if groups is not None:
        if not isinstance(groups, dict):
            raise ConfigError(f"config.json: {w}router.'groups' must be an object with count and keep")
        count, keep = _int(w + "router.groups.", groups, "count"), _int(w + "router.groups.", groups, "keep")
    outputs = experts + identity
    if outputs <= 0 or outputs % count or keep > count:
        raise ConfigError(f"config.json: {w}router: {count} groups ({keep} kept) do not divide {outputs} router outputs")
    if top > (outputs // count) * keep:
        raise ConfigError(f"config.json: {w}router: {top} choices do not fit {keep} groups of {outputs // count}")
    return RoutedFF(ff=_int(w + "expert.", expert, "ff"), experts=experts, top=top, identity=identity, group_count=count,
                    group_keep=keep)


@dataclass(frozen=True)
class PuputarConfig:
    vocab: int
    width: int
    eps: float
    groups: int
    layers: Tuple[PuputarLayer, ...]

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PuputarConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with eps")
        width = _int("", raw, "width")
        groups = _int("norm.", norm, "groups") if "groups" in norm else 1
        if width % groups:
            raise ConfigError(f"config.json: norm.'groups' {groups} does not divide the width {width}")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for n, entry in enumerate(entries):
            where = f"layers[{n}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{n}] must be an object")
            kind = entry.get("type")
            if kind not in GATES:
                raise ConfigError(f"config.json: {where}'type' must be one of {', '.join(sorted(GATES))}, got {kind!r}")
            mixer = _mixer(where, entry.get("mixer"))
            if mixer.kv_from is not None:
                if mixer.kv_from >= n:
                    raise ConfigError(f"config.json: {where}mixer.'kv_from' {mixer.kv_from} must name an earlier layer")
                source = layers[mixer.kv_from].mixer
                if source.kv_from is not None:
                    raise ConfigError(f"config.json: {where}mixer.'kv_from' names layer {mixer.kv_from}, which keeps no "
                                      f"entries of its own")
                if (source.kv_rank, source.rot_dim, source.rot_base, source.rot_dims) != \
                        (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                    raise ConfigError(f"config.json: {where}mixer reads the entries of layer {mixer.kv_from}, whose kv_rank, "
                                      f"rot_dim or rotation differ")
            layers.append(PuputarLayer(kind=kind, mixer=mixer, mlp=_mlp(where, entry.get("mlp"))))
        return cls(vocab=_int("", raw, "vocab"), width=width, eps=_number("norm.", norm, "eps"), groups=groups,
                   layers=tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps, "groups": self.groups}, "layers": [layer.to_dict() for layer in self.layers]}
