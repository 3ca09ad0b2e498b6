"""Kokolorn without a GPU: its configuration, its model description and tensor names (the passes over a run of layers
as borrowed layers with entries), the rows of the bias by distance, parameters whose length the tensor decides, and
the oracle's own functions."""
import copy
import math

import numpy as np
import pytest

from aegean_tge_b200 import ConfigError, architecture_of
from aegean_tge_b200.config.model_spec import expected_tensors
from aegean_tge_b200.parts.attention import GQAttention
from aegean_tge_b200.parts.base import ParamSpec
from plain import kokolorn_plain as plain

ATT = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.4, "q_temp": {"coef": 0.2, "every": 16}},
       "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 20}}}
DELTA = {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3}, "mlp": {"kind": "dense", "ff": 40, "limit": 2.5}}
PAR = {"type": "parallel", "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25,
                                              "q_temp": {"coef": 0.1, "every": 8}, "bias_max": 50.0},
                                     "right": {"heads": 3, "vdim": 8, "state": 6, "groups": 1, "norm_groups": 2, "conv": 2}},
       "mlp": None}
CONFIG = {"architecture": "Kokolorn", "vocab": 60, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
          "layers": [DELTA, ATT, PAR, DELTA], "loop": {"start": 1, "stop": 3, "times": 3}}


def _parse(raw):
    arch = architecture_of(raw)
    return arch, arch.parse_config(raw)


def test_config_round_trip_and_description():
    arch, config = _parse(CONFIG)
    assert config.to_dict() == CONFIG
    spec = arch.build_spec(config)
    spec.validate()
    # layers 1 and 2 run three times: the first visit is the layer itself, the later ones borrow its parts
    assert config.run_order() == ((0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None))
    assert spec.schedule == (0, 1, 2, 4, 5, 6, 7, 3)
    assert [layer.weights_from for layer in spec.layers] == [None, None, None, None, 1, 2, 1, 2]
    assert [None if layer.entry is None else layer.entry.params["index"] for layer in spec.layers] == [None, 0, None, None, 1, None, 2, None]
    assert [layer.mixer.kind for layer in spec.layers[:4]] == ["gated_delta_rule", "gqa_attention", "mixer_sum", "gated_delta_rule"]
    assert spec.layers[1].mixer.params["values"] == "keys" and spec.layers[1].mixer.params["qk_norm"]["scope"] == "head"
    left = spec.layers[2].mixer.params["branches"][0][1]
    assert left.params["distance_bias"] == {"far": 50.0} and left.params["o_bias"] and "qk_norm" not in left.params
    assert spec.layers[2].feed_forward is None and spec.layers[2].ffn_norm is None
    assert spec.layers[1].feed_forward.params["shared"].params["activation"] == "relu_squared"
    assert spec.embedding.params["scale"] == 1.5 and spec.head.weights["weight"] == "embed"
    assert spec.final_norm.params["unit_offset"]
    names = set(expected_tensors(spec))
    assert {"embed", "final.norm", "loop.in", "loop.step", "l0.mix.q.conv", "l0.mix.A_log", "l0.mix.b", "l1.mix.q.b", "l1.mix.k.norm",
            "l1.mlp.router.b", "l1.mlp.e4.down", "l1.mlp.shared.up", "l2.mix.left.rel", "l2.mix.left.o.b", "l2.mix.right.conv.b",
            "l2.mix.right.D", "l2.mix.left.out", "l2.mix.right.out", "l3.mlp.gate"} <= names
    assert not any(name.startswith(("l4.", "l1.mix.v", "l2.mix.left.v", "l2.norm2", "l1.mlp.e5")) for name in names)
    planned = {name: shape for name, shape, _role, _draw in arch.random_plan(config)}
    assert set(planned) == names
    assert planned["loop.in"] == (24, 48) and planned["loop.step"] == (3, 24) and planned["l0.mix.v.conv"] == (48, 3)
    assert planned["l2.mix.right.in"] == (2 * 24 + 2 * 6 + 3, 24) and planned["l2.mix.right.conv"] == (24 + 12, 2)
    assert planned["l2.mix.left.rel"][1] == 2 and planned["l0.mix.norm"] == (12,)


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "retention"), (("layers", 0, "mixer", "conv"), 0), (("layers", 0, "mixer", "conv"), 17),
    (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "dim"), 300), (("layers", 0, "mlp", "limit"), 0.0),
    (("layers", 0, "mlp", "kind"), "gated"), (("layers", 1, "mixer", "vdim"), 4), (("layers", 1, "mixer", "scale"), None),
    (("layers", 1, "mixer", "q_temp"), {"coef": 0.2, "every": 0}), (("layers", 1, "mlp", "router", "top"), 6),
    (("layers", 1, "mlp", "expert"), None), (("layers", 1, "mlp", "shared"), {"ff": 0}), (("layers", 2, "mixer", "left", "bias_max"), None),
    (("layers", 2, "mixer", "right", "norm_groups"), 5), (("layers", 2, "mixer", "right", "groups"), 2),
    (("layers", 2, "mixer", "right"), None), (("loop", "stop"), 5), (("loop", "start"), 3), (("loop", "times"), 0),
    (("norm",), {}), (("embedding",), {"scale": "big"}), (("layers",), []), (("width",), None)])
def test_config_errors_name_the_key(path, value):
    raw = copy.deepcopy(CONFIG)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        _parse(raw)
    assert str(path[-1]) in str(error.value) or "layer" in str(error.value) or "loop" in str(error.value)


def test_what_a_model_may_leave_out():
    raw = copy.deepcopy(CONFIG)
    del raw["loop"], raw["embedding"], raw["layers"][1]["mlp"]["shared"], raw["layers"][1]["mixer"]["q_temp"]
    arch, config = _parse(raw)
    assert config.loop is None and config.embedding_scale == 1.0 and config.layers[1].mlp.shared_ff is None
    spec = arch.build_spec(config)
    assert spec.schedule == (0, 1, 2, 3) and all(layer.entry is None for layer in spec.layers)
    names = set(expected_tensors(spec))
    assert "loop.in" not in names and "l1.mlp.shared.up" not in names
    assert "q_temp" not in spec.layers[1].mixer.params and spec.layers[1].feed_forward.params["shared"] is None
    # one pass is still a pass: the stream is mixed with the embedding once
    raw["loop"] = {"start": 0, "stop": 4, "times": 1}
    arch, config = _parse(raw)
    spec = arch.build_spec(config)
    assert spec.schedule == (0, 1, 2, 3) and spec.layers[0].entry.params == {"hidden_size": 24, "index": 0, "count": 1}


@pytest.mark.parametrize("rows,far", [(32, 120.0), (8, 100.0), (16, 16.5), (2, 40.0), (64, 4096.0), (32, 128.0), (7, 30.0)])
def test_rows_of_the_bias_by_distance(rows, far):
    import torch
    for n in range(0, int(far) + 40):
        assert GQAttention.distance_row(n, rows, far) == plain.distance_bucket(n, rows, far), n
    rel = torch.arange(rows * 3, dtype=torch.float32).reshape(rows, 3)
    table = GQAttention.expand_distance_bias(rel, far)
    span = table.shape[1]
    assert table.shape[0] == 3 and span <= math.ceil(far) + 1
    assert plain.distance_bucket(span - 1, rows, far) == rows - 1 and (span == 1 or plain.distance_bucket(span - 2, rows, far) < rows - 1)
    for n in (0, 1, rows // 2 - 1, rows // 2, span - 1):
        if 0 <= n < span:
            assert table[:, n].tolist() == rel[plain.distance_bucket(n, rows, far)].tolist()
    with pytest.raises(ValueError):
        GQAttention.expand_distance_bias(rel[:1], far)
    with pytest.raises(ValueError):
        GQAttention.expand_distance_bias(rel, float(rows // 2))


def test_a_parameter_may_leave_an_extent_to_the_tensor():
    spec = ParamSpec((-1, 4), role="vector")
    assert spec.takes((32, 4)) and spec.takes((2, 4)) and not spec.takes((32, 5)) and not spec.takes((32,))
    assert ParamSpec((3, 4)).takes((3, 4)) and not ParamSpec((3, 4)).takes((4, 4))


# ---------------------------------------------------------------------------
# the oracle's own functions
def test_oracle_delta_rule_writes_corrects_and_forgets():
    d, dv = 4, 3
    e = np.eye(d)
    # three orthogonal unit keys; full strength, no decay: each readout returns the value written under its key
    k = np.stack([e[0], e[1], e[2], e[0]])
    v = np.arange(12, dtype=float).reshape(4, dv)
    q = np.stack([e[0], e[0], e[1], e[0]])
    o = plain.delta_rule(q, k, v, np.ones(4), np.ones(4))
    assert np.allclose(o[0], v[0]) and np.allclose(o[1], v[0]) and np.allclose(o[2], v[1])
    assert np.allclose(o[3], v[3])                       # the same key again: the old value is replaced, not added to
    half = plain.delta_rule(q, k, v, np.full(4, 0.5), np.ones(4))
    assert np.allclose(half[3], 0.5 * v[0] + 0.5 * (v[3] - 0.5 * v[0]))
    decayed = plain.delta_rule(q, k, v, np.ones(4), np.array([1.0, 0.5, 0.5, 1.0]))
    assert np.allclose(decayed[1], 0.5 * v[0]) and np.allclose(decayed[2], 0.5 * v[1])     # what was written fades with every later decay


def test_oracle_state_space_and_short_convolution():
    x = np.array([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    B = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])
    C = np.array([[1.0, 0.0], [1.0, 1.0], [0.0, 1.0]])
    dt = np.array([0.5, 1.0, 2.0])
    y = plain.state_space(x, B, C, dt, a=0.0, D=0.25)     # no decay: S_t is a running sum of dt B x^T
    assert np.allclose(y[0], 0.5 * x[0] + 0.25 * x[0])
    assert np.allclose(y[1], 0.5 * x[0] + 1.0 * x[1] + 0.25 * x[1])
    assert np.allclose(y[2], 1.0 * x[1] + 2.0 * x[2] + 0.25 * x[2])
    y = plain.state_space(x, B, C, dt, a=math.log(2.0), D=0.0)
    assert np.allclose(y[1], 0.5 * 0.5 * x[0] + x[1])
    u = np.arange(8, dtype=float).reshape(4, 2)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    got = plain.short_conv(u, w, bias=np.array([0.5, 0.0]))
    assert np.allclose(got[:, 1], u[:, 1])                # the last tap is the current token's
    assert np.allclose(got[:, 0], [0.5, 200 + 0.5, 400 + 20 + 0.5, 600 + 40 + 2 + 0.5])


def test_oracle_temperature_buckets_router_and_feed_forward():
    t = plain.query_temperature(np.array([0, 6, 7, 8, 23]), 0.5, 8)
    assert np.allclose(t, [1.0, 1.0, 1.0 + 0.5 * math.log(2), 1.0 + 0.5 * math.log(2), 1.0 + 0.5 * math.log(4)])
    assert [plain.distance_bucket(n, 8, 64.0) for n in (0, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == [0, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]
    W = {"m.router": np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]]), "m.router.b": np.array([0.0, 0.0, -1.5])}
    ids, w = plain.route(np.array([[2.0, 1.0]]), W, "m.", 2)
    assert ids.tolist() == [[0, 2]] and np.allclose(w, [[1 / (1 + math.exp(-0.5)), 1 / (1 + math.exp(0.5))]])
    W = {"f.gate": np.array([[1.0], [1.0]]), "f.up": np.array([[1.0], [-1.0]]), "f.down": np.eye(2)}
    out = plain.dense_ff(np.array([[5.0]]), W, "f.", 2.0)
    g = 2.0 / (1 + math.exp(-1.702 * 2.0))
    assert np.allclose(out, [[g * 3.0, g * -1.0]])
    assert plain.run_order({"layers": [0, 1, 2], "loop": {"start": 1, "stop": 2, "times": 2}}) == [(0, None), (1, 0), (1, 1), (2, None)]
