"""The Kokolorn design in the engine against its plain implementation (tests/plain/kokolorn_plain.py).

First every mechanism alone through its kernel (the recurrence in both forms with its state in slots, what readies its
inputs with the convolution's tail, the gate before the norm, the normalised sum of branches, the clamped gate, the
queries' temperature with the store of keys and values, the bias by distance), with inputs made so that a lost state, a
key one position off or a wrong row of the bias shows; then whole models of five small configurations that differ in
every size, order and option, cut and batched in every way, in both number formats.
"""
import json
import os
import random

import numpy as np
import pytest
import torch

from helpers import batch_index, paged_cache, rel_error
from plain import kokolorn_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_TOL = {"float32": 2e-5, "bfloat16": 2e-2}
MODEL_TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def _att(heads, kv_heads, dim, scale, temp=None, bias_max=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if temp is not None:
        out["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if bias_max is not None:
        out["bias_max"] = bias_max
    return out


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _ssm(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, experts, top, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _config(vocab, width, eps, layers, loop=None, scale=None):
    out = {"architecture": "Kokolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    if scale is not None:
        out["embedding"] = {"scale": scale}
    return out


def _configs():
    return {
        # every kind of layer, a run of two layers passed through twice after a layer of its own, a layer without
        # feed-forward at the end; sharp softmaxes so that one lost key changes a row
        "A": _config(210, 96, 1e-5, [
            _layer("delta", _delta(4, 2, 32, 48, 4), _dense(128, 1.5)),
            _layer("attention", _att(6, 3, 16, 0.6, temp=(0.4, 16)), _moe(32, 6, 2, shared=48)),
            _layer("parallel", {"left": _att(4, 2, 32, 0.3, temp=(0.3, 32), bias_max=70.0), "right": _ssm(6, 16, 24, 2, 3, 3)},
                   _moe(48, 4, 3, shared=32)),
            _layer("attention", _att(2, 1, 48, 0.4, temp=(0.2, 7)), None)], loop=(1, 3, 2), scale=0.7),
        # what other models keep apart is equal or 1 here: as many kv heads as heads, one tap, one expert chosen of two and
        # no shared one, one group per head, one norm group, one pass over everything, no temperature, no embedding scale
        "B": _config(128, 64, 1e-6, [
            _layer("parallel", {"left": _att(2, 2, 32, 0.18, bias_max=33.0), "right": _ssm(2, 32, 16, 2, 1, 1)}, _moe(64, 2, 1)),
            _layer("delta", _delta(2, 2, 16, 16, 1), _dense(64, 7.0)),
            _layer("attention", _att(1, 1, 64, 0.125), _moe(32, 3, 3))], loop=(0, 3, 1)),
        # nothing a multiple of 8; the looped run in the middle, three passes; a delta layer inside the loop
        "C": _config(97, 100, 2e-5, [
            _layer("attention", _att(3, 1, 20, 0.5, temp=(0.5, 5)), _dense(70, 0.8)),
            _layer("delta", _delta(6, 3, 12, 10, 3), _moe(18, 5, 2, shared=30)),
            _layer("parallel", {"left": _att(5, 5, 12, 0.4, temp=(0.1, 3), bias_max=17.5), "right": _ssm(5, 6, 10, 1, 5, 2)}, None)],
            loop=(1, 2, 3), scale=1.3),
        # large heads and states (the tensor-core attention where the design allows it), many experts, no loop at all
        "D": _config(300, 128, 1e-6, [
            _layer("attention", _att(8, 2, 64, 0.2, temp=(0.3, 64)), _moe(64, 24, 4, shared=64)),
            _layer("delta", _delta(4, 2, 128, 128, 4), _dense(192, 1.0)),
            _layer("parallel", {"left": _att(4, 1, 128, 0.1, temp=(0.5, 128), bias_max=200.0), "right": _ssm(4, 64, 128, 1, 2, 4)},
                   _dense(128, 2.0))]),
        # many query heads to a kv head, head sizes that only the mma.sync kernels take (96, 80), keys of 64 for the
        # recurrence, two taps, many experts with several chosen, three passes from the first layer on, a layer after them
        "E": _config(250, 160, 1e-6, [
            _layer("attention", _att(16, 2, 96, 0.15, temp=(0.25, 48)), _moe(40, 32, 6, shared=56)),
            _layer("delta", _delta(8, 2, 64, 32, 2), None),
            _layer("parallel", {"left": _att(8, 1, 80, 0.2, temp=(0.4, 20), bias_max=40.0), "right": _ssm(8, 24, 64, 4, 4, 2)},
                   _dense(96, 3.0))], loop=(0, 2, 3), scale=0.9),
    }


CONFIGS = _configs()
SEEDS = {"A": 41, "B": 42, "C": 43, "D": 44, "E": 45}


@pytest.fixture(scope="module")
def ops():
    from aegean_tge_b200 import ops as module
    module.core()
    return module


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from aegean_tge_b200 import write_random_model
    out = {}
    for name, config in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"kokolorn_{name}")
        write_random_model(str(folder), config, seed=SEEDS[name], dtype="float32")
        out[name] = str(folder)
    return out


def _read_weights(folder):
    with open(os.path.join(folder, "model.safetensors"), "rb") as handle:
        size = int.from_bytes(handle.read(8), "little")
        header = json.loads(handle.read(size))
        data = handle.read()
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        assert entry["dtype"] == "F32", (name, entry["dtype"])
        begin, end = entry["data_offsets"]
        out[name] = np.frombuffer(data[begin:end], dtype="<f4").reshape(entry["shape"]).copy()
    return out


def _to_bfloat16(array):
    return torch.from_numpy(np.ascontiguousarray(array)).to(torch.bfloat16).float().numpy()


_WEIGHTS = {}


def _weights(folders, name, dtype):
    if (name, dtype) not in _WEIGHTS:
        from aegean_tge_b200 import architecture_of
        arch = architecture_of(CONFIGS[name])
        matrices = {tensor for tensor, _shape, role, _draw in arch.random_plan(arch.parse_config(CONFIGS[name])) if role == "matrix"}
        w = _read_weights(folders[name])
        if dtype == "bfloat16":         # matrices are held in bfloat16, vectors (taps, biases, tables, norms) in float32
            w = {k: (_to_bfloat16(v) if k in matrices else v) for k, v in w.items()}
        _WEIGHTS[(name, dtype)] = {k: v.astype(np.float64) for k, v in w.items()}
    return _WEIGHTS[(name, dtype)]


@pytest.fixture(scope="module")
def oracle(folders):
    """oracle(name, dtype, tokens) -> logits; oracle.margin(name, dtype, tokens) -> [T], every row's smallest distance
    from another choice of experts over all routed layer runs."""
    cache = {}

    def both(name, dtype, tokens, config=None):
        key = (name, dtype, tuple(tokens), json.dumps(config, sort_keys=True) if config else "")
        if key not in cache:
            margins = []
            logits = plain.forward(config or CONFIGS[name], _weights(folders, name, dtype), list(tokens), margins=margins)
            smallest = np.min(np.stack(margins), axis=0) if margins else np.full(len(tokens), np.inf)
            cache[key] = (torch.from_numpy(logits).float(), smallest)
        return cache[key]

    def get(name, dtype, tokens, config=None):
        return both(name, dtype, tokens, config)[0]
    get.margin = lambda name, dtype, tokens: both(name, dtype, tokens)[1]
    return get


# In bfloat16 a rounding can send a row to other experts when two router logits lie close together: such a row may
# differ from the oracle by any amount, and so may every later row of the request, which reads it through the caches and
# states.  Rows before the first close call must agree; a request with none must agree everywhere.
CLOSE_CALL = 3e-2


def _agree(got, oracle, name, dtype, tokens, rows=None, where=""):
    """``got``: logits of ``rows`` (default: all) of the sequence ``tokens``."""
    ref = oracle(name, dtype, tokens)
    rows = list(range(len(tokens))) if rows is None else list(rows)
    scale = float(ref.abs().max())
    ref = ref[rows]
    got = got.detach().float().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all()
    error = (got - ref).abs().max(dim=1).values / scale
    if dtype == "float32":
        assert float(error.max()) < MODEL_TOL[dtype], (name, dtype, where, float(error.max()))
        return
    margin = oracle.margin(name, dtype, tokens)
    close = np.nonzero(margin < CLOSE_CALL)[0]
    clear_until = int(close[0]) if len(close) else len(tokens)
    for r, e in zip(rows, error.tolist()):
        if r < clear_until:
            assert e < MODEL_TOL[dtype], (name, dtype, where, r, e)


def _tokens(name, count, salt=0):
    rnd = random.Random(SEEDS[name] * 1000 + salt)
    return [rnd.randrange(CONFIGS[name]["vocab"]) for _ in range(count)]


def _engine(folders, name, dtype, **kw):
    from aegean_tge_b200 import Engine
    kw.setdefault("context", 512)
    kw.setdefault("max_tokens", 1024)
    kw.setdefault("max_requests", 8)
    return Engine(folders[name], dtype=dtype, **kw)


def _portion(request, tokens, want=None):
    from aegean_tge_b200.engine import Portion
    return Portion(request, tokens, list(range(len(tokens))) if want is None else want)


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def _f32(array):
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).to(DEV)


# ---------------------------------------------------------------------------
# mechanisms, one by one
def _unit(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def _run_scan(ops, qk, v, gates, heads, dim, vdim, lengths, cuts, delta, skip=None):
    """Feeds requests of the given lengths through the scan in steps: ``cuts[i]`` lists, per step, (request, count).  The
    slots are out of order and every other slot holds junk.  Returns each request's rows."""
    slots_total = len(lengths) + 3
    state = torch.full((slots_total, heads, dim, vdim), 7.5, device=DEV)
    slot_of = {r: (2 * r + 1) % slots_total for r in range(len(lengths))}
    for r in slot_of:
        state[slot_of[r]].zero_()
    starts = np.concatenate([[0], np.cumsum(lengths)])
    done = [0] * len(lengths)
    out = [[] for _ in lengths]
    for step in cuts:
        rows = np.concatenate([np.arange(starts[r] + done[r], starts[r] + done[r] + n) for r, n in step])
        q_start = _i32(np.concatenate([[0], np.cumsum([n for _, n in step])]).tolist())
        slots = _i32([slot_of[r] for r, _ in step])
        got = ops.gated_rule_scan(_f32(qk[rows]), _f32(v[rows]), _f32(gates[rows]), state, slots, q_start, len(step), delta=delta,
                                  skip=None if skip is None else _f32(skip))
        at = 0
        for r, n in step:
            out[r].append(got[at:at + n].cpu())
            at += n
            done[r] += n
    assert done == list(lengths)
    assert float(state[0].min()) == 7.5 or 0 in slot_of.values()
    return [torch.cat(rows) for rows in out]


@pytest.mark.parametrize("delta", [True, False])
@pytest.mark.parametrize("heads,groups,dim,vdim", [(4, 2, 32, 48), (3, 1, 12, 10), (2, 2, 100, 7), (2, 1, 128, 128), (1, 1, 256, 17),
                                                 (4, 2, 64, 40)])
def test_recurrence_in_portions_batches_and_slots(ops, delta, heads, groups, dim, vdim):
    rng = np.random.default_rng(heads * 1000 + dim + int(delta))
    lengths = [37, 5, 64]
    total = sum(lengths)
    q = _unit(rng.standard_normal((total, groups, dim))) * (dim ** -0.5 if delta else 1.0)
    k = _unit(rng.standard_normal((total, groups, dim)))
    v = rng.standard_normal((total, heads, vdim))
    decay = rng.uniform(0.6, 1.0, (total, heads))
    strength = rng.uniform(0.1, 1.0, (total, heads)) if delta else rng.uniform(0.1, 2.0, (total, heads))
    skip = None if delta else rng.standard_normal(heads)
    qk = np.stack([q, k], axis=2)
    gates = np.stack([decay, strength], axis=2)
    cuts = [[(0, 20), (1, 1), (2, 2)], [(2, 1), (0, 1), (1, 2)], [(1, 2), (0, 16)], [(2, 61)]]
    got = _run_scan(ops, qk, v.reshape(total, -1), gates, heads, dim, vdim, lengths, cuts, delta, skip)
    starts = np.concatenate([[0], np.cumsum(lengths)])
    for r, n in enumerate(lengths):
        lo = starts[r]
        ref = np.zeros((n, heads, vdim))
        for h in range(heads):
            g = h // (heads // groups)
            if delta:
                ref[:, h] = plain.delta_rule(q[lo:lo + n, g], k[lo:lo + n, g], v[lo:lo + n, h], strength[lo:lo + n, h], decay[lo:lo + n, h])
            else:
                # with a = 1 the decay exp(-a dt) is handed over as the number itself: dt = -ln(decay) would tie the two
                ref[:, h] = _state_space_with(q[lo:lo + n, g], k[lo:lo + n, g], v[lo:lo + n, h], strength[lo:lo + n, h],
                                              decay[lo:lo + n, h], skip[h])
        assert rel_error(got[r], torch.from_numpy(ref.reshape(n, -1))) < KERNEL_TOL["float32"], (r, n)


def _state_space_with(C, B, x, dt, decay, D):
    S = np.zeros((B.shape[1], x.shape[1]))
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        S = decay[t] * S + dt[t] * np.outer(B[t], x[t])
        y[t] = S.T @ C[t] + D * x[t]
    return y


def test_recurrence_keeps_what_nothing_overwrites(ops):
    """No decay, full strength, orthogonal keys: a value written at the first token is read back exactly 300 tokens later,
    token by token through the state; the delta rule replaces a value written under the same key, the other form adds."""
    dim, vdim, n = 32, 8, 301
    e = np.eye(dim)
    k = np.stack([e[0]] + [e[1 + t % (dim - 1)] for t in range(n - 2)] + [e[0]])[:, None, :]
    q = np.stack([e[0]] * n)[:, None, :]
    v = np.arange(n * vdim, dtype=float).reshape(n, 1, vdim) / 100.0
    gates = np.ones((n, 1, 2))
    qk = np.stack([q, k], axis=2)
    for delta in (True, False):
        got = _run_scan(ops, qk, v.reshape(n, -1), gates, 1, dim, vdim, [n], [[(0, 100)]] + [[(0, 1)]] * 200 + [[(0, 1)]], delta)[0]
        assert torch.allclose(got[n - 2], torch.from_numpy(v[0, 0]).float(), atol=1e-6)
        want_last = v[n - 1, 0] if delta else v[0, 0] + v[n - 1, 0]
        assert torch.allclose(got[n - 1], torch.from_numpy(want_last).float(), atol=1e-5)


@pytest.mark.parametrize("mode", ["delta", "state_space"])
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_what_the_recurrence_takes_with_the_convolutions_tail(ops, mode, taps):
    """The rows after the input product: convolution (its tail carried per request through portions of one and two
    tokens), SiLU, unit vectors, decays and strengths."""
    rng = np.random.default_rng(taps * 10 + len(mode))
    heads, groups, dim, vdim = 4, 2, 12, 10
    qkw, vw = groups * dim, heads * vdim
    channels = 2 * qkw + vw
    lengths = [9, 23]
    total = sum(lengths)
    width = channels + vw + 2 * heads if mode == "delta" else vw + channels + heads
    raw = rng.standard_normal((total, width))
    conv_w = rng.uniform(-0.5, 0.5, (channels, taps))
    conv_b = None if mode == "delta" else rng.standard_normal(channels) * 0.1
    a_log, dt_bias = rng.uniform(-2, 0, heads), rng.uniform(-1, 1, heads)
    slots_total = 4
    tails = torch.full((slots_total, max(taps - 1, 1), channels), 3.25, device=DEV) if taps > 1 else None
    slot_of = {0: 2, 1: 0}
    if tails is not None:
        tails[2].zero_()
        tails[0].zero_()
    starts = [0, lengths[0]]
    cuts = [[(0, 1), (1, 2)], [(1, 1), (0, 2)], [(0, 1), (1, 1)], [(0, 5), (1, 19)]]
    done = [0, 0]
    got_qk, got_v, got_g = {}, {}, {}
    for step in cuts:
        rows = np.concatenate([np.arange(starts[r] + done[r], starts[r] + done[r] + n) for r, n in step])
        counts = [n for _, n in step]
        q_start = _i32(np.concatenate([[0], np.cumsum(counts)]).tolist())
        seq = _i32([s for s, n in enumerate(counts) for _ in range(n)])
        qk, v, gates = ops.gated_prepare(_f32(raw[rows]), ops.GATED_DELTA if mode == "delta" else ops.GATED_STATE_SPACE, groups, heads,
                                         dim, vdim, taps, _f32(conv_w), None if conv_b is None else _f32(conv_b), tails,
                                         _i32([slot_of[r] for r, _ in step]), q_start, seq, len(step), _f32(a_log), _f32(dt_bias),
                                         q_scale=dim ** -0.5 if mode == "delta" else 1.0)
        for i, row in enumerate(rows):
            got_qk[row], got_v[row], got_g[row] = qk[i].cpu(), v[i].cpu(), gates[i].cpu()
        for r, n in step:
            done[r] += n
    for r, n in enumerate(lengths):
        lo = starts[r]
        part = raw[lo:lo + n]
        if mode == "delta":
            conv = plain.silu(plain.short_conv(part[:, :channels], conv_w))
            q = _unit(conv[:, :qkw].reshape(n, groups, dim)) * dim ** -0.5
            k = _unit(conv[:, qkw:2 * qkw].reshape(n, groups, dim))
            v = conv[:, 2 * qkw:]
            strength = plain.sigmoid(part[:, channels + vw:channels + vw + heads])
            decay = np.exp(-np.exp(a_log) * plain.softplus(part[:, channels + vw + heads:] + dt_bias))
        else:
            conv = plain.silu(plain.short_conv(part[:, vw:vw + channels], conv_w, conv_b))
            v = conv[:, :vw]
            k = conv[:, vw:vw + qkw].reshape(n, groups, dim)
            q = conv[:, vw + qkw:].reshape(n, groups, dim)
            strength = plain.softplus(part[:, vw + channels:] + dt_bias)
            decay = np.exp(-np.exp(a_log) * strength)
        for t in range(n):
            assert rel_error(got_qk[lo + t], torch.from_numpy(np.stack([q[t], k[t]], axis=1))) < KERNEL_TOL["float32"], (r, t)
            assert rel_error(got_v[lo + t], torch.from_numpy(v[t])) < KERNEL_TOL["float32"], (r, t)
            assert rel_error(got_g[lo + t], torch.from_numpy(np.stack([decay[t], strength[t]], axis=1))) < KERNEL_TOL["float32"], (r, t)
    if tails is not None:
        assert float(tails[1].min()) == 3.25 and float(tails[3].max()) == 3.25          # other requests' slots untouched


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_before_the_norm_in_parts(ops, dtype):
    rng = np.random.default_rng(5)
    y, z, w = rng.standard_normal((11, 60)) * 3, rng.standard_normal((11, 60)), rng.uniform(0.5, 1.5, 60)
    for parts in (1, 3, 5):
        gated = y * plain.silu(z)
        ref = plain.unit_rms(gated.reshape(11, parts, 60 // parts), 1e-5).reshape(11, 60) * w
        got = ops.gated_norm(_f32(y), _f32(z), _f32(w), parts, 1e-5, sigmoid=False, gate_first=True, out_dtype=TORCH[dtype])
        assert got.dtype == TORCH[dtype] and rel_error(got, torch.from_numpy(ref)) < KERNEL_TOL[dtype]
        after = plain.unit_rms(y.reshape(11, parts, 60 // parts), 1e-5).reshape(11, 60) * w * plain.silu(z)
        assert rel_error(torch.from_numpy(after), torch.from_numpy(ref)) > 0.05          # the order matters


def test_branches_normalised_over_the_width_and_added(ops):
    rng = np.random.default_rng(6)
    x, y, w = rng.standard_normal((7, 100)), rng.standard_normal((7, 100)) * 30, rng.uniform(0.5, 1.5, 100)
    stream = _f32(x)
    ops.norm_scale_add(stream, _f32(y), _f32(w), 1e-5, alpha=0.5)
    assert rel_error(stream, torch.from_numpy(x + 0.5 * plain.rms_norm(y, w, 1e-5))) < KERNEL_TOL["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_clamped_gate(ops, dtype):
    rng = np.random.default_rng(7)
    g, u = rng.standard_normal((9, 35)) * 3, rng.standard_normal((9, 35)) * 3
    rows = np.stack([g, u], axis=2).reshape(9, 70)
    for limit in (0.8, 2.0, 100.0):
        gc, uc = np.minimum(g, limit), np.clip(u, -limit, limit)
        ref = gc * plain.sigmoid(1.702 * gc) * (uc + 1.0)
        got = ops.gated_clamp_act(_f32(rows), limit, 1.702, 1.0, TORCH[dtype])
        assert rel_error(got, torch.from_numpy(ref)) < KERNEL_TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,width,inner", [(5, 64, 48), (150, 96, 200), (300, 128, 1024), (3, 100, 35)])
def test_clamped_gate_as_the_products_epilogue(ops, dtype, tokens, width, inner):
    """The feed-forward part with the design's constants clamps and gates in the epilogue of its first product (the
    tensor-core product, its sums over cuts along k, and the CUDA-core product), with other constants in a kernel of
    its own: both are the plain formula."""
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import FEED_FORWARDS, build_part
    from aegean_tge_b200.parts.base import BuildEnv
    rng = np.random.default_rng(tokens)
    W = {"f.gate": rng.standard_normal((inner, width)) * 0.3, "f.up": rng.standard_normal((inner, width)) * 0.3,
         "f.down": rng.standard_normal((width, inner)) * inner ** -0.5}
    h = rng.standard_normal((tokens, width))
    if dtype == "bfloat16":
        W = {k: _to_bfloat16(v.astype(np.float32)).astype(np.float64) for k, v in W.items()}
        h = _to_bfloat16(h.astype(np.float32)).astype(np.float64)
    env = BuildEnv(dtype=TORCH[dtype], device=DEV, hidden_size=width, max_positions=64, page_size=16, ops=ops)
    for alpha, limit in ((1.702, 0.9), (1.702, 50.0), (1.3, 0.9)):
        part = build_part(FEED_FORWARDS, PartSpec("clamped_glu", {"hidden_size": width, "intermediate_size": inner, "limit": limit,
                                                                  "alpha": alpha}), env)
        part.load({f"{t}.weight": torch.from_numpy(W[f"f.{t}"]).to(DEV, TORCH[dtype]) for t in ("gate", "up", "down")})
        got = part.forward(torch.from_numpy(h).to(DEV, TORCH[dtype]), None)
        g = np.minimum(h @ W["f.gate"].T, limit)
        u = np.clip(h @ W["f.up"].T, -limit, limit)
        ref = (g * plain.sigmoid(alpha * g) * (u + 1.0)) @ W["f.down"].T
        if alpha == 1.702:
            assert rel_error(torch.from_numpy(ref), torch.from_numpy(plain.dense_ff(h, W, "f.", limit))) < 1e-12
        assert rel_error(got, torch.from_numpy(ref)) < 1.5 * KERNEL_TOL[dtype], (alpha, limit)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,normed,every", [(4, 2, 16, True, 4), (3, 3, 20, False, 7), (8, 1, 64, True, 64), (2, 2, 12, True, 0)])
def test_temperature_norm_and_store_of_keys_and_values(ops, dtype, heads, kv_heads, dim, normed, every):
    """q normalised and heated by position, the keys normalised into their pages, the values the keys as they arrived."""
    rng = np.random.default_rng(dim)
    page, n, first = 16, 37, 59                     # positions 59..95 straddle multiples of every and page borders
    rows = torch.from_numpy(rng.standard_normal((n, (heads + kv_heads) * dim)) * 2).to(TORCH[dtype])
    raw = rows.float().numpy().astype(np.float64)
    qw, kw = (rng.uniform(0.5, 1.5, dim), rng.uniform(0.5, 1.5, dim)) if normed else (None, None)
    pages = 8
    k_pages = torch.zeros(pages, kv_heads, page, dim, dtype=TORCH[dtype], device=DEV)
    v_pages = torch.zeros_like(k_pages)
    table = _i32([[5, 2, 7, 0, 3, 1, 6]])
    positions, seq = _i32(list(range(first, first + n))), _i32([0] * n)
    qk = rows.to(DEV).clone()
    ops.qk_temp_store(qk, None if qw is None else _f32(qw), None if kw is None else _f32(kw), 1e-5, 0.37, every, positions, seq,
                      table, k_pages, v_pages, heads, kv_heads, dim)
    q = raw[:, :heads * dim].reshape(n, heads, dim)
    k = raw[:, heads * dim:].reshape(n, kv_heads, dim)
    if normed:
        q, kn = plain.rms_norm(q, qw, 1e-5), plain.rms_norm(k, kw, 1e-5)
    else:
        kn = k
    if every:
        q = q * plain.query_temperature(np.arange(first, first + n), 0.37, every)[:, None, None]
    assert rel_error(qk[:, :heads * dim], torch.from_numpy(q.reshape(n, -1))) < KERNEL_TOL[dtype]
    order = table[0].tolist()
    for t in range(n):
        p = first + t
        assert rel_error(k_pages[order[p // page], :, p % page], torch.from_numpy(kn[t])) < KERNEL_TOL[dtype]
        assert torch.equal(v_pages[order[p // page], :, p % page].cpu(), rows[t, heads * dim:].reshape(kv_heads, dim))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,far,page,dim", [(8, 40.0, 16, 16), (32, 120.0, 64, 64), (4, 300.0, 16, 32), (32, 100.0, 64, 128),
                                               (16, 33.0, 64, 48), (32, 100.0, 64, 256), (9, 60.0, 32, 96)])
def test_bias_by_distance_in_the_softmax(ops, dtype, rows, far, page, dim):
    """Every row of the table differs from its neighbours by several units, so a distance one off, a wrong row past the
    middle or a scaled bias changes the result; prompts and single tokens, two requests, shuffled pages."""
    from aegean_tge_b200.parts.attention import GQAttention
    heads, kv_heads, dim, scale = 4, 2, 16, 0.3
    rng = np.random.default_rng(rows)
    rel = rng.permutation(rows * heads).reshape(rows, heads).astype(np.float64) * 1.5 - rows
    table = GQAttention.expand_distance_bias(torch.from_numpy(rel).float(), far).to(DEV)
    lengths = [int(far) + 175, 21]
    k_pages, v_pages, block_table, k_list, _ = paged_cache(lengths, kv_heads, dim, page, TORCH[dtype], DEV, seed=rows)
    for new in ([lengths[0], lengths[1]], [1, 1], [40, 2]):
        starts = [lengths[0] - new[0], lengths[1] - new[1]]
        positions, seq, q_start, start_pos = batch_index(new, starts, DEV)
        q = torch.randn(sum(new), heads * dim, generator=torch.Generator().manual_seed(3)).to(TORCH[dtype])
        got = ops.attention(q.to(DEV), k_pages, k_pages, block_table, q_start, start_pos, positions, seq, 2, max(new), max(lengths),
                            heads, kv_heads, dim, scale, dist_bias=table)
        at = 0
        for s in range(2):
            keys = k_list[s].double().numpy()
            full = np.zeros((lengths[s], heads, dim))
            full[starts[s]:] = q[at:at + new[s]].double().numpy().reshape(new[s], heads, dim)
            ref = plain.softmax_attention(full, keys, keys, scale, bias=rel, far=far)[starts[s]:]
            assert rel_error(got[at:at + new[s]], torch.from_numpy(ref)) < KERNEL_TOL[dtype], (new, s)
            at += new[s]


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds_stands_out(ops, dtype):
    """A key made to dominate its query sits at the first position, at a page's last and first entry, or just behind the
    distance where the bias stops changing: the row is that key (the values are the keys), whatever the bias says."""
    from aegean_tge_b200.parts.attention import GQAttention
    heads, kv_heads, dim, page, n = 2, 1, 32, 16, 400
    rel = torch.linspace(-2.0, 2.0, 16 * heads).reshape(16, heads)
    table = GQAttention.expand_distance_bias(rel, 90.0).to(DEV)
    for place in (0, 15, 16, n - 92, n - 1):
        k_pages, _v, block_table, k_list, _ = paged_cache([n], kv_heads, dim, page, TORCH[dtype], DEV, seed=place)
        key = k_list[0][place, 0].float()
        q = (key * (60.0 / float(key @ key))).repeat(heads)[None].to(TORCH[dtype])
        positions, seq, q_start, start_pos = batch_index([1], [n - 1], DEV)
        got = ops.attention(q.to(DEV), k_pages, k_pages, block_table, q_start, start_pos, positions, seq, 1, 1, n, heads, kv_heads, dim,
                            1.0, dist_bias=table)
        assert rel_error(got[0].float().cpu().reshape(heads, dim), key.repeat(heads, 1)) < 2 * KERNEL_TOL[dtype], place


# ---------------------------------------------------------------------------
# whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_first_tokens(folders, oracle, ops, name, dtype):
    engine = _engine(folders, name, dtype)
    for length in (1, 2, 3, 7, 16, 33, 64, 65, 150):
        tokens = _tokens(name, length, salt=length)
        logits = engine.runner.step([_portion("r", tokens)])
        engine.runner.finish("r")
        _agree(logits, oracle, name, dtype, tokens, where=length)
    ops.check_status()
    engine.cache.check()


def _without(config, change):
    altered = json.loads(json.dumps(config))
    change(altered)
    return altered


def test_each_mechanism_changed_would_show(oracle):
    """The oracle with one mechanism changed differs from itself by far more than the tolerance: so the whole-model
    tests would see a kernel that got that mechanism wrong."""
    tokens = _tokens("A", 90, salt=3)
    ref = oracle("A", "float32", tokens)
    def no_temperature(c): del c["layers"][1]["mixer"]["q_temp"]
    def other_every(c): c["layers"][2]["mixer"]["left"]["q_temp"]["every"] = 31
    def other_far(c): c["layers"][2]["mixer"]["left"]["bias_max"] = 60.0
    def other_scale(c): c["layers"][3]["mixer"]["scale"] *= 1.3
    def one_pass(c): c["loop"]["times"] = 1
    def other_limit(c): c["layers"][0]["mlp"]["limit"] = 1.0
    def other_top(c): c["layers"][1]["mlp"]["router"]["top"] = 3
    def other_parts(c): c["layers"][2]["mixer"]["right"]["norm_groups"] = 1
    def no_embedding_scale(c): del c["embedding"]
    for change in (no_temperature, other_every, other_far, other_scale, one_pass, other_limit, other_top, other_parts, no_embedding_scale):
        assert rel_error(oracle("A", "float32", tokens, config=_without(CONFIGS["A"], change)), ref) > 1e-3, change.__name__


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token_decoding(folders, oracle, name, dtype):
    tokens = _tokens(name, 110, salt=1)
    ref = oracle(name, dtype, tokens)
    engine = _engine(folders, name, dtype)
    rows = [engine.runner.step([_portion("r", tokens[:68])])]
    for t in range(68, len(tokens)):
        rows.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
    got = torch.cat(rows)
    _agree(got, oracle, name, dtype, tokens)
    assert engine.runner.graph_replays > 0
    if dtype == "float32":
        whole = _engine(folders, name, dtype).runner.step([_portion("w", tokens)])
        assert float((got - whole).abs().max()) <= 2e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("page_size", [16, 64])
def test_portions_down_to_two_tokens(folders, oracle, name, dtype, page_size):
    tokens = _tokens(name, 230, salt=2)
    engine = _engine(folders, name, dtype, page_size=page_size)
    cuts = [7, 2, 16, 3, 2, 30, 2, 17, 41, 1, 1, 26, 2, 64, 5, 2, 2, 7]
    assert sum(cuts) == len(tokens)
    rows, pos = [], 0
    for count in cuts:
        rows.append(engine.runner.step([_portion("r", tokens[pos:pos + count])]))
        pos += count
    _agree(torch.cat(rows), oracle, name, dtype, tokens)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("page_size,pool_tokens", [(16, 320), (64, 512)])
def test_unequal_requests_in_one_batch_on_pages_and_slots_that_are_used_again(folders, oracle, ops, name, dtype, page_size,
                                                                            pool_tokens):
    """Up to four live requests in four slots, portions of some beside single tokens of others, a pool so small that
    pages and slots of finished requests serve the next ones; every request's logits are those it gets alone."""
    lengths = {"a": 70, "b": 45, "c": 130, "d": 19, "e": 64, "f": 33, "g": 90}
    tokens = {r: _tokens(name, n, salt=ord(r)) for r, n in lengths.items()}
    engine = _engine(folders, name, dtype, max_tokens=pool_tokens, page_size=page_size, max_requests=4)
    got, done = {r: [] for r in lengths}, {r: 0 for r in lengths}
    holders, slot_users = {}, {}

    def run(step):
        logits = engine.runner.step([_portion(r, tokens[r][done[r]:done[r] + count]) for r, count in step])
        row = 0
        for r, count in step:
            got[r].append(logits[row:row + count])
            row += count
            done[r] += count
            slot_users.setdefault(engine.cache.slot_of(r), set()).add(r)
            for page in engine.cache.groups[0].tables[r]:
                if page >= 0:
                    holders.setdefault(page, set()).add(r)
            if done[r] == lengths[r]:
                engine.runner.finish(r)

    run([("a", 40), ("b", 3)])
    run([("a", 2), ("b", 40), ("c", 64), ("d", 1)])
    run([("a", 28), ("b", 2), ("c", 2), ("d", 16)])          # a and b end
    run([("c", 60), ("d", 2), ("e", 1), ("f", 30)])           # d ends; e and f take over pages and slots
    for _ in range(3):
        run([("c", 1), ("e", 1), ("f", 1)])                   # f ends
    run([("c", 1), ("e", 58), ("g", 2)])
    run([("e", 2), ("g", 64)])                                # c ended before; e ends
    run([("g", 24)])
    ops.check_status()
    engine.cache.check()
    assert any(len(who) > 1 for who in holders.values()) and any(len(who) > 1 for who in slot_users.values())
    assert not engine.cache.live_requests()
    for r in lengths:
        assert done[r] == lengths[r]
        _agree(torch.cat(got[r]), oracle, name, dtype, tokens[r], where=r)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(folders, oracle, name, dtype):
    """Three tokens of prompt, then 330 single tokens through the decode graphs: over many page borders, many
    multiples of the temperature's period, and past the distance where the bias stops changing."""
    tokens = _tokens(name, 333, salt=5)
    engine = _engine(folders, name, dtype, page_size=16)
    rows = [engine.runner.step([_portion("r", tokens[:3])])]
    for t in range(3, len(tokens)):
        rows.append(engine.runner.step([_portion("r", tokens[t:t + 1])]))
    _agree(torch.cat(rows), oracle, name, dtype, tokens)
    assert engine.runner.graph_replays > 0
    engine.cache.check()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_scheduler(folders, oracle, name):
    """``Engine.generate`` (scheduler, portions of 16, sampler, steps queued ahead) gives the plain model's greedy
    continuation."""
    engine = _engine(folders, name, "float32", chunk=16, max_batch_tokens=48)
    prompts = [_tokens(name, n, salt=40 + n) for n in (5, 37, 1, 70)]
    outputs = engine.generate(prompts, n=12)
    for prompt, produced in zip(prompts, outputs):
        sequence = list(prompt)
        for token in produced:
            logits = oracle(name, "float32", sequence)[-1]
            best = int(torch.argmax(logits))
            if token != best:          # only a tie within rounding may differ
                assert float(logits[best] - logits[token]) < 1e-4 * float(logits.abs().max()), (name, len(sequence))
            sequence.append(int(token))
        assert len(produced) == 12
    assert not engine.cache.live_requests()
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_sampled_generation_with_requests_that_come_and_go(folders, dtype):
    """Twelve requests with samplers through six slots, then three: the same seeds give the same tokens whatever shared
    a step with what (no state leaks between a slot's users; steps queued ahead and dropped leave none)."""
    from aegean_tge_b200 import SamplingParams
    prompts = [_tokens("A", 3 + 11 * i, salt=300 + i) for i in range(12)]
    params = [SamplingParams(temperature=0.8, top_k=(0, 20, 50)[i % 3], top_p=(1.0, 0.9)[i % 2], seed=40 + i) for i in range(12)]
    outputs = []
    for slots, budget, chunk in ((6, 64, 16), (3, 256, 64)):
        engine = _engine(folders, "A", dtype, max_requests=slots, max_batch_tokens=budget, chunk=chunk, max_tokens=640)
        outputs.append(engine.generate(prompts, n=10, sampling=params))
        assert not engine.cache.live_requests()
        engine.cache.check()
    if dtype == "float32":
        assert outputs[0] == outputs[1]


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_of_a_kokolorn_model(folders, oracle, tmp_path, dtype):
    """bin/trace_run as a subprocess: two requests, portions and single tokens in one batch, slots given back."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a, b = _tokens("A", 60, salt=90), _tokens("A", 9, salt=91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[40:41], "want": [0]}, {"id": "b", "tokens": b[:7], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [1]}, {"id": "a", "tokens": a[41:], "want": [18]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    run = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["A"], "--dtype", dtype,
                          "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    vocab = CONFIGS["A"]["vocab"]
    read = lambda step: torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, vocab))
    _agree(torch.cat([read(0), read(1), read(2)[1:]]), oracle, "A", dtype, a, rows=[0, 39, 40, 59])
    _agree(read(2)[:1], oracle, "A", dtype, b, rows=[8])


def test_command_line_serves_the_design(folders, capsys):
    from aegean_tge_b200.cli import main
    assert main(["generate", "--model", folders["D"], "--tokens", "5 17 3", "--n", "6", "--print-ids", "--context", "128"]) == 0
    out = capsys.readouterr().out
    assert len(out.split("ids      :")[1].split()) == 6
    common = ["--model", folders["D"], "--context", "512", "--max-requests", "12"]
    assert main(["bench", "decode", *common, "--batch", "3", "--prompt-len", "40", "--n", "4"]) == 0
    assert main(["bench", "prefill", *common, "--prompt-len", "100", "--repeat", "1"]) == 0
    assert main(["plan", "--model", folders["A"], "--context", "256", "--sessions", "2"]) == 0
    capsys.readouterr()
