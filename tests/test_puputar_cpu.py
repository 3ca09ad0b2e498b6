"""Puputar without a GPU: its configuration, its model description and tensor names, the oracle's own functions, and
the cache and state the design asks of the cache manager (one entry per token per layer that keeps its own, none for
a layer that reads another's; a shift row per layer in every request's slot)."""
import copy

import numpy as np
import pytest

from aegean_tge_b200 import ConfigError, architecture_of
from aegean_tge_b200.cache import CacheManager
from aegean_tge_b200.config.model_spec import expected_tensors
from aegean_tge_b200.parts.base import PagedCacheSpec, StateSpec
from plain import puputar_plain as plain

MIXER = {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 10, "kv_rank": 12, "scale": 0.3, "rot": {"base": 100.0, "dims": 4}}
DENSE = {"type": "latent_attention", "mixer": MIXER, "mlp": {"kind": "dense", "ff": 40}}
ROUTED = {"type": "latent_attention_2", "mixer": dict(MIXER, heads=2, vdim=8, kv_from=0),
          "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 4, "top": 2, "identity": 2, "groups": {"count": 3, "keep": 2}}}}
BARE = {"type": "latent_attention_2", "mixer": dict(MIXER, kv_rank=20, rot={"base": 7.0, "dims": 2}), "mlp": None}
CONFIG = {"architecture": "Puputar", "vocab": 50, "width": 24, "norm": {"eps": 1e-5, "groups": 3}, "layers": [DENSE, ROUTED, BARE]}


def _parse(raw):
    arch = architecture_of(raw)
    return arch, arch.parse_config(raw)


def test_config_round_trip_and_description():
    arch, config = _parse(CONFIG)
    assert config.to_dict() == CONFIG
    spec = arch.build_spec(config)
    spec.validate()
    assert [layer.cache_from for layer in spec.layers] == [None, 0, None]
    assert [layer.block for layer in spec.layers] == ["parallel"] * 3
    assert [layer.mixer.kind for layer in spec.layers] == ["shifted_mixer"] * 3
    assert [layer.mixer.params["inner"].params["gate"] for layer in spec.layers] == ["head", "element", "element"]
    assert spec.layers[1].mixer.params["inner"].params["shared_kv"] and not spec.layers[0].mixer.params["inner"].params["shared_kv"]
    assert spec.layers[2].feed_forward is None and spec.layers[2].ffn_norm.params["optional"]
    assert spec.embedding.params["norm"].kind == "group_rmsnorm" and spec.final_norm.params["groups"] == 3
    names = set(expected_tensors(spec))
    assert {"embed.norm", "l0.shift", "l0.mix.dkv.norm", "l0.mlp.up.b", "l0.mlp.act", "l1.mlp.router", "l1.mlp.correction",
            "l1.mlp.e3.down", "l2.mix.dkv"} <= names
    assert not any(name.startswith("l1.mix.dkv") for name in names) and "l1.mlp.e4.up" not in names
    planned = {name: shape for name, shape, _role, _draw in arch.random_plan(config)}
    assert set(planned) == names - {"l2.norm2"}          # a layer without feed-forward may, but need not, bring a second norm
    assert planned["l0.mix.g"] == (3, 24) and planned["l1.mix.g"] == (16, 24) and planned["l0.mix.uq"] == (36, 10)
    assert planned["l0.mix.dkv"] == (16, 24) and planned["l1.mlp.router"] == (6, 24) and planned["l2.mix.dkv"] == (24, 24)


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "attention"), (("layers", 0, "mixer", "rot", "dims"), 3), (("layers", 0, "mixer", "rot", "dims"), 6),
    (("layers", 0, "mixer", "rot"), None), (("layers", 0, "mixer", "heads"), 0), (("layers", 0, "mixer", "scale"), "big"),
    (("layers", 1, "mixer", "kv_from"), 1), (("layers", 1, "mixer", "kv_from"), 2), (("layers", 1, "mixer", "kv_rank"), 16),
    (("layers", 1, "mixer", "rot"), {"base": 5.0, "dims": 4}), (("layers", 1, "mlp", "kind"), "gated"),
    (("layers", 1, "mlp", "router", "groups"), {"count": 4, "keep": 2}), (("layers", 1, "mlp", "router", "groups"), {"count": 3, "keep": 4}),
    (("layers", 1, "mlp", "router", "top"), 5), (("layers", 1, "mlp", "expert"), None), (("norm",), {}), (("norm",), {"eps": 1e-5, "groups": 5}),
    (("layers",), []), (("width",), None)])
def test_config_errors_name_the_key(path, value):
    raw = copy.deepcopy(CONFIG)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        _parse(raw)
    assert str(path[-1]) in str(error.value) or "layer" in str(error.value) or "router" in str(error.value)


def test_a_reader_of_a_reader_is_refused():
    raw = copy.deepcopy(CONFIG)
    raw["layers"].append(copy.deepcopy(ROUTED))
    raw["layers"][3]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError):
        _parse(raw)


def test_what_a_model_may_leave_out():
    raw = copy.deepcopy(CONFIG)
    del raw["norm"]["groups"]
    del raw["layers"][1]["mlp"]["router"]["groups"], raw["layers"][1]["mlp"]["router"]["identity"]
    arch, config = _parse(raw)
    assert config.groups == 1 and config.layers[1].mlp.identity == 0 and config.layers[1].mlp.group_count == 1
    spec = arch.build_spec(config)
    assert spec.layers[1].feed_forward.params["identity"] == 0
    assert dict(expected_tensors(spec))["l1.mlp.router"]
    assert {name: shape for name, shape, _r, _d in arch.random_plan(config)}["l1.mlp.router"] == (4, 24)


def test_cache_and_state_the_design_declares():
    """Layers 0 and 2 keep one entry of kv_rank + rot_dim numbers per token; layer 1 keeps none; every layer has a
    shift row in the request's slot, zeroed for each taker."""
    manager = CacheManager(4, 2)
    entry = lambda size: PagedCacheSpec((("kv", (1, size)),), None)
    shift = StateSpec((("shift", (24,)),))
    manager.add_layer(0, entry(16), shift)
    manager.add_layer(1, None, shift)
    manager.add_layer(2, entry(24), shift)
    assert len(manager.groups) == 1                      # both keep every token: one group, one block table


# ---------------------------------------------------------------------------
# the oracle's own functions
def test_oracle_norm_shift_and_rotation():
    x = np.array([[3.0, 4.0, 0.0, 0.0, 6.0, 8.0]])
    got = plain.group_norm(x, np.ones(6), 3, 0.0 + 1e-12)
    assert np.allclose(got, [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5), 0, 0, 6 / np.sqrt(50), 8 / np.sqrt(50)]], atol=1e-5)
    assert np.allclose(plain.group_norm(x, np.ones(6), 1, 1e-12), x / np.sqrt((x ** 2).mean()))
    h = np.arange(6.0).reshape(3, 2)
    assert np.allclose(plain.token_shift(h, np.array([1.0, 0.5])), [[0.0, 0.5], [0.0, 2.0], [2.0, 4.0]])
    v = np.array([[[1.0, 0.0, 0.0, 2.0, 5.0]]])
    turned = plain.rotate_pairs(v, [1], np.e, 4)           # frequencies 1 and e^-1/2... pairs (0,1) and (2,3)
    a, b = 1.0, np.e ** -0.5
    assert np.allclose(turned[0, 0], [np.cos(a), np.sin(a), -2 * np.sin(b), 2 * np.cos(b), 5.0])
    assert np.allclose(plain.rotate_pairs(v, [0], 10.0, 4), v)


def test_oracle_router_and_activation():
    correction = np.array([0.0, 0.0, 0.0, 0.0, 0.3, 0.0])
    logits = np.log(np.array([[0.30, 0.05, 0.05, 0.25, 0.05, 0.30]]))
    ids, weights = plain.route(logits, np.eye(6), correction, 2, 3, 1)
    # groups (0,1) (2,3) (4,5): best choice values 0.30, 0.25, 0.35 -> the last group; inside it 0.35 (output 4) and 0.30
    assert ids.tolist() == [[4, 5]] and np.allclose(weights, [[0.05 / 0.35, 0.30 / 0.35]])
    ids, _ = plain.route(logits, np.eye(6), -1.0 + 0 * correction, 2, 3, 1)
    assert ids.tolist() == [[0, 1]]                      # all choice values negative: the groups left out are not 0
    assert plain.route_margin(logits, np.eye(6), correction, 2, 3, 1)[0] == pytest.approx(0.05)
    z = np.array([-2.0, 0.0, 1.5])
    sp = lambda t: np.log1p(np.exp(t))
    assert np.allclose(plain.xielu(z, 0.3, -0.7), [(0.5 + sp(-0.7)) * (np.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, sp(0.3) * 2.25 + 0.75])
    h = np.array([[1.0, -2.0]])
    w = {"p.router": np.zeros((3, 2)), "p.correction": np.array([0.0, -1.0, 0.0]),
         "p.e0.up": np.array([[1.0, 0.0], [0.0, 1.0]]), "p.e0.down": np.array([[2.0, 0.0], [0.0, 2.0]]),
         "p.e1.up": np.zeros((2, 2)), "p.e1.down": np.zeros((2, 2))}
    out = plain.moe_ff(h, w, "p.", {"router": {"experts": 2, "identity": 1, "top": 2}})
    # equal scores; outputs 0 and 2 are chosen, each with weight 1/2: expert 0 gives 2 relu(h)^2, output 2 gives h itself
    assert np.allclose(out, [[0.5 * 2.0 + 0.5 * 1.0, 0.5 * 0.0 + 0.5 * -2.0]])
