"""The Puputar design in the engine against its plain implementation (tests/plain/puputar_plain.py).

First every mechanism alone through its kernel or part (the norm in groups, the token shift with its per-request row,
the rotation of neighbouring pairs, attention over the latent cache with both gates and with another layer's
entries, the two-parameter activation, the router with its groups, corrections and identity experts, both ways
through the experts), with inputs made so that a lost key, a lost state or a wrongly masked group shows; then whole
models of five small configurations that differ in every size, order and option, cut and batched in every way, in
both number formats.
"""
import json
import os
import random

import numpy as np
import pytest
import torch

from helpers import rel_error
from plain import puputar_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_TOL = {"float32": 2e-5, "bfloat16": 2e-2}
MODEL_TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def _mixer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims=None, kv_from=None):
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
           "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, identity=None, groups=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _config(vocab, width, eps, groups, layers):
    norm = {"eps": eps}
    if groups is not None:
        norm["groups"] = groups
    return {"architecture": "Puputar", "vocab": vocab, "width": width, "norm": norm, "layers": layers}


LA, LA2 = "latent_attention", "latent_attention_2"


def _configs():
    return {
        # a routed layer first; a layer of each kind reads the entries of a layer of the other kind; a layer without
        # feed-forward; sharp softmaxes (large scales) so that a single lost key changes a row
        "A": _config(210, 96, 1e-5, 3, [
            _layer(LA2, _mixer(4, 32, 16, 32, 48, 48, 0.6, 5000.0), _moe(32, 6, 2, identity=2, groups=(2, 1))),
            _layer(LA, _mixer(3, 16, 16, 48, 40, 32, 0.9, 700.0), _dense(128)),
            _layer(LA, _mixer(2, 48, 16, 16, 24, 48, 0.5, 5000.0, kv_from=0), None),
            _layer(LA2, _mixer(5, 16, 16, 16, 56, 32, 1.2, 700.0, kv_from=1), _moe(48, 4, 3, identity=1)),
            _layer(LA, _mixer(4, 32, 16, 32, 48, 48, 0.3, 100.0), _dense(64))]),
        # what other models keep apart is equal or 1 here: one norm group, one head, one expert chosen, no identity
        # experts, no groups, every size of the mixer the same
        "B": _config(128, 64, 1e-6, None, [
            _layer(LA2, _mixer(1, 32, 32, 32, 32, 32, 0.125, 10000.0), _dense(64)),
            _layer(LA, _mixer(1, 32, 32, 32, 32, 32, 0.125, 10000.0), _moe(64, 4, 1)),
            _layer(LA, _mixer(1, 32, 32, 32, 32, 32, 0.125, 10000.0, kv_from=0), _moe(32, 3, 1, identity=0, groups=(1, 1)))]),
        # nothing a multiple of 8; part of the shared key rotated; every group kept; as many choices as kept outputs
        "C": _config(97, 100, 2e-5, 5, [
            _layer(LA, _mixer(3, 12, 6, 10, 20, 14, 0.4, 50.0, dims=4), _moe(18, 5, 3, identity=1, groups=(3, 2))),
            _layer(LA2, _mixer(5, 6, 10, 12, 14, 22, 0.7, 9.0), _dense(70)),
            _layer(LA2, _mixer(2, 20, 6, 6, 10, 14, 0.3, 50.0, dims=4, kv_from=0), _moe(10, 2, 4, identity=2, groups=(2, 2)))]),
        # large heads and entries, many heads on the one cached entry, many experts
        "D": _config(300, 128, 1e-6, 4, [
            _layer(LA, _mixer(20, 64, 32, 64, 64, 128, 0.1, 500000.0), _moe(64, 24, 4, identity=4, groups=(7, 3))),
            _layer(LA2, _mixer(8, 128, 64, 128, 96, 64, 0.08, 250000.0), _dense(192))]),
        # identity experts alone can be chosen; corrections decide; one layer only reads
        "E": _config(150, 48, 1e-5, 2, [
            _layer(LA2, _mixer(2, 16, 16, 16, 16, 16, 0.7, 1000.0), _moe(16, 1, 2, identity=3, groups=(2, 1))),
            _layer(LA2, _mixer(2, 16, 16, 16, 16, 16, 0.7, 1000.0, kv_from=0), None)]),
    }


CONFIGS = _configs()
SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34, "E": 35}


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
        folder = tmp_path_factory.mktemp(f"puputar_{name}")
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
        w = _read_weights(folders[name])
        if dtype == "bfloat16":         # matrices are held in bfloat16, vectors in float32
            w = {k: (_to_bfloat16(v) if v.ndim == 2 else v) for k, v in w.items()}
        _WEIGHTS[(name, dtype)] = {k: v.astype(np.float64) for k, v in w.items()}
    return _WEIGHTS[(name, dtype)]


@pytest.fixture(scope="module")
def oracle(folders):
    """oracle(name, dtype, tokens) -> logits; oracle.margin(name, dtype, tokens) -> [T], every row's smallest distance
    from another choice of experts over all routed layers."""
    cache = {}

    def both(name, dtype, tokens, config=None, **kw):
        key = (name, dtype, tuple(tokens), json.dumps(config, sort_keys=True) if config else "", json.dumps(kw, sort_keys=True))
        if key not in cache:
            margins = []
            logits = plain.forward(config or CONFIGS[name], _weights(folders, name, dtype), list(tokens), margins=margins, **kw)
            smallest = np.min(np.stack(margins), axis=0) if margins else np.full(len(tokens), np.inf)
            cache[key] = (torch.from_numpy(logits).float(), smallest)
        return cache[key]

    def get(name, dtype, tokens, config=None, **kw):
        return both(name, dtype, tokens, config, **kw)[0]
    get.margin = lambda name, dtype, tokens: both(name, dtype, tokens)[1]
    return get


# In bfloat16 a rounding can send a row to other experts when two choice values lie close together: such a row (and
# the next one, which the token shift blends with it) may differ from the oracle by any amount.  Rows whose choice is
# clear must agree; the others may fail, but only they, and only few of all rows.
CLOSE_CALL = 2e-2


def _agree(got, oracle, name, dtype, tokens, rows=None, where=""):
    """``got``: logits of ``rows`` (default: all) of the sequence ``tokens``."""
    ref = oracle(name, dtype, tokens)
    rows = list(range(len(tokens))) if rows is None else list(rows)
    ref = ref[rows]
    got = got.detach().float().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all()
    error = (got - ref).abs().max(dim=1).values / float(oracle(name, dtype, tokens).abs().max())
    if dtype == "float32":
        assert float(error.max()) < MODEL_TOL[dtype], (name, dtype, where, float(error.max()))
        return
    margin = oracle.margin(name, dtype, tokens)
    unclear = np.array([margin[r] < CLOSE_CALL or (r > 0 and margin[r - 1] < CLOSE_CALL) for r in rows])
    over = (error >= MODEL_TOL[dtype]).numpy()
    assert not (over & ~unclear).any(), (name, dtype, where, [(rows[i], float(error[i])) for i in np.nonzero(over & ~unclear)[0]])
    assert over.sum() <= max(1, len(rows) // 20), (name, dtype, where, int(over.sum()), len(rows))


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


def _index(cuts, starts):
    """Index tensors of one step: portions of the given lengths that start at the given positions."""
    positions, seq, q_start = [], [], [0]
    for s, (n, first) in enumerate(zip(cuts, starts)):
        positions += list(range(first, first + n))
        seq += [s] * n
        q_start.append(q_start[-1] + n)
    return _i32(positions), _i32(seq), _i32(q_start), _i32(list(starts))


# ---------------------------------------------------------------------------
# mechanisms, one by one
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,groups", [(96, 3), (64, 1), (100, 5), (320, 2), (1024, 4), (7, 7)])
def test_norm_in_groups(ops, dtype, width, groups):
    gen = torch.Generator().manual_seed(width + groups)
    x = torch.randn(13, width, generator=gen) * 3
    x[:, : width // groups] *= 40.0            # one part much larger than the others: a norm over the whole row would show
    w = 1 + 0.2 * torch.randn(width, generator=gen)
    ref = torch.from_numpy(plain.group_norm(x.numpy(), w.numpy(), groups, 1e-5))
    got = ops.group_norm(x.to(DEV), w.to(DEV), 1e-5, groups, TORCH[dtype])
    assert rel_error(got, ref) < KERNEL_TOL[dtype]
    rows = _i32([12, 0, 5])
    assert rel_error(ops.group_norm(x.to(DEV), w.to(DEV), 1e-5, groups, TORCH[dtype], rows=rows), ref[[12, 0, 5]]) < KERNEL_TOL[dtype]
    if groups > 1:
        whole = torch.from_numpy(plain.group_norm(x.numpy(), w.numpy(), 1, 1e-5))
        assert rel_error(got.float().cpu(), whole) > 0.1
    # two norms of the same rows that differ in their weights only, from one launch
    w2 = 1 + 0.2 * torch.randn(width, generator=gen)
    first, second = ops.group_norm(x.to(DEV), w.to(DEV), 1e-5, groups, TORCH[dtype], weight2=w2.to(DEV))
    assert torch.equal(first, got)
    assert rel_error(second, torch.from_numpy(plain.group_norm(x.numpy(), w2.numpy(), groups, 1e-5))) < KERNEL_TOL[dtype]
    stream = x.to(DEV)
    assert ops.group_norm(stream, w.to(DEV), 1e-5, groups, torch.float32, out=stream).data_ptr() == stream.data_ptr()
    assert rel_error(stream, ref) < KERNEL_TOL["float32"]


def test_norm_part_in_one_group_can_be_fused():
    from aegean_tge_b200 import ops
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import NORMS, build_part
    from aegean_tge_b200.parts.base import BuildEnv
    env = BuildEnv(dtype=torch.float32, device=DEV, hidden_size=48, max_positions=64, page_size=16, ops=ops)
    one = build_part(NORMS, PartSpec("group_rmsnorm", {"size": 48, "eps": 1e-5}, {"weight": "w"}), env)
    three = build_part(NORMS, PartSpec("group_rmsnorm", {"size": 48, "eps": 1e-5, "groups": 3}, {"weight": "w"}), env)
    w = torch.ones(48, device=DEV)
    one.load({"weight": w})
    three.load({"weight": w})
    assert one.fusable()[1] == 1e-5 and three.fusable() is None
    with pytest.raises(ValueError):
        build_part(NORMS, PartSpec("group_rmsnorm", {"size": 48, "eps": 1e-5, "groups": 5}, {"weight": "w"}), env)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 100, 1500])
@pytest.mark.parametrize("cuts", [[[30]], [[1], [1], [2], [1], [25]], [[9, 1, 12], [2, 1, 1], [1, 1, 1], [18, 27, 16]]])
def test_token_shift_in_portions_and_batches(ops, dtype, width, cuts):
    """Requests cut into portions down to one token and batched, their slots out of order and junk in every slot that no
    request of the step uses; a weight of exactly 1 in some columns makes the row before stand alone there, so a lost
    or stale state shows whole."""
    gen = torch.Generator().manual_seed(width)
    requests = len(cuts[0])
    lengths = [sum(step[r] for step in cuts) for r in range(requests)]
    rows = [torch.randn(n, width, generator=gen).to(TORCH[dtype]) for n in lengths]
    mu = torch.rand(width, generator=gen)
    mu[::3] = 1.0
    mu[1::7] = 0.0
    slots = [5, 2, 7][:requests]
    state = torch.randn(9, width, generator=gen).to(DEV)           # junk everywhere: position 0 must not read it
    done = [0] * requests
    got = [[] for _ in range(requests)]
    for step in cuts:
        live = [r for r in range(requests) if step[r] > 0]
        positions, seq, q_start, start_pos = _index([step[r] for r in live], [done[r] for r in live])
        h = torch.cat([rows[r][done[r]:done[r] + step[r]] for r in live]).to(DEV)
        out = ops.token_shift(h, mu.to(DEV), state, _i32([slots[r] for r in live]), seq, q_start, start_pos, len(live))
        row = 0
        for r in live:
            got[r].append(out[row:row + step[r]])
            row += step[r]
            done[r] += step[r]
    for r in range(requests):
        ref = torch.from_numpy(plain.token_shift(rows[r].double().numpy(), mu.double().numpy()))
        assert rel_error(torch.cat(got[r]), ref) < KERNEL_TOL[dtype], (r, lengths[r])
        assert torch.equal(state[slots[r]].cpu(), rows[r][-1].float())
    ops.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,width,dims,base", [(1, 32, 32, 10000.0), (3, 6, 4, 50.0), (5, 10, 10, 9.0), (8, 64, 16, 250000.0)])
def test_rotation_of_neighbouring_pairs(ops, dtype, heads, width, dims, base):
    from aegean_tge_b200.parts.rope import pair_tables
    gen = torch.Generator().manual_seed(dims)
    positions = [0, 1, 2, 63, 64, 700, 3, 1999]
    stride = width + 5                                 # the runs lie inside wider heads
    src = torch.randn(len(positions), heads * stride, generator=gen).to(TORCH[dtype])
    cos, sin = pair_tables(base, dims, 2000)
    dst = torch.zeros(len(positions), heads * width, dtype=TORCH[dtype], device=DEV)
    ops.rotate_interleaved(src.to(DEV)[:, 5:], stride, dst, width, heads, width, cos.to(DEV), sin.to(DEV), dims, _i32(positions))
    runs = src.double().view(len(positions), heads, stride)[:, :, 5:]
    ref = torch.from_numpy(plain.rotate_pairs(runs.numpy(), positions, base, dims)).reshape(len(positions), heads * width)
    assert rel_error(dst, ref) < KERNEL_TOL[dtype]
    if dims < width:
        assert torch.equal(dst.view(len(positions), heads, width)[:, :, dims:].cpu(), runs[:, :, dims:].to(TORCH[dtype]))
    # the rotated numbers at the end of a run, the plain ones before them copied
    if width > dims:
        lead = width - dims
        moved = torch.cat([runs[..., dims:], runs[..., :dims]], dim=-1).to(TORCH[dtype])
        want = torch.cat([ref.view(len(positions), heads, width)[..., dims:], ref.view(len(positions), heads, width)[..., :dims]], dim=-1)
        back = torch.zeros(len(positions), heads * width, dtype=TORCH[dtype], device=DEV)
        ops.rotate_interleaved(moved.reshape(len(positions), -1).to(DEV), width, back, width, heads, width, cos.to(DEV), sin.to(DEV), dims,
                               _i32(positions), first=lead)
        assert rel_error(back, want.reshape(len(positions), -1)) < KERNEL_TOL[dtype]
    # the halves-paired rotation is another function: it must differ
    half = runs.clone()
    angle = torch.tensor(positions, dtype=torch.float64)[:, None] * base ** (-2.0 * torch.arange(dims // 2) / dims)
    a, b = runs[..., :dims // 2], runs[..., dims // 2:dims]
    half[..., :dims // 2] = a * angle.cos()[:, None] - b * angle.sin()[:, None]
    half[..., dims // 2:dims] = b * angle.cos()[:, None] + a * angle.sin()[:, None]
    if dims > 2:
        assert rel_error(half.reshape(len(positions), -1), ref) > 1e-2
    ops.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_parameter_activation(ops, dtype):
    gen = torch.Generator().manual_seed(3)
    z = (torch.randn(7, 50, generator=gen) * 3).to(TORCH[dtype])
    z[0, :4] = torch.tensor([0.0, -0.0, 1e-3, -1e-3]).to(TORCH[dtype])
    for p, q in ((0.3, -0.7), (-2.0, 1.5), (0.0, 0.0)):
        rows = z.clone().to(DEV)
        wide = torch.zeros(7, 64, dtype=TORCH[dtype], device=DEV)
        wide[:, :50] = rows
        ops.activation(wide[:, :50], ops.ACT_XIELU, torch.tensor([p, q], device=DEV))
        ref = torch.from_numpy(plain.xielu(z.double().numpy(), p, q))
        assert rel_error(wide[:, :50], ref) < KERNEL_TOL[dtype]
        assert float(wide[:, 50:].abs().max()) == 0.0
    squared = z.clone().to(DEV)
    ops.activation(squared, ops.ACT_RELU_SQUARED)
    assert rel_error(squared, z.double().clamp(min=0) ** 2) < KERNEL_TOL[dtype]
    # rows of a multiple of eight numbers inside wider rows (eight at a time in bfloat16)
    y = (torch.randn(9, 48, generator=gen) * 3).to(TORCH[dtype])
    for kind, params, ref in ((ops.ACT_XIELU, torch.tensor([0.3, -0.7], device=DEV), plain.xielu(y.double().numpy(), 0.3, -0.7)),
                              (ops.ACT_RELU_SQUARED, None, (y.double().clamp(min=0) ** 2).numpy())):
        wide = torch.full((9, 64), 2.0, dtype=TORCH[dtype], device=DEV)
        wide[:, :48] = y.to(DEV)
        ops.activation(wide[:, :48], kind, params)
        assert rel_error(wide[:, :48], torch.from_numpy(ref)) < KERNEL_TOL[dtype]
        assert float((wide[:, 48:] - 2.0).abs().max()) == 0.0


# ---------------------------------------------------------------------------
# the router and the experts
def _route_case(ops, logits, correction, top, count, keep):
    ids, weights = ops.router_topk(logits.to(DEV), None if correction is None else correction.to(DEV), top, count, keep)
    zero = np.zeros(logits.shape[1]) if correction is None else correction.double().numpy()
    ref_ids, ref_w = plain.route(logits.double().numpy(), np.eye(logits.shape[1]), zero, top, count, keep)
    assert np.array_equal(ids.cpu().numpy(), ref_ids), (top, count, keep)
    assert rel_error(weights, torch.from_numpy(ref_w)) < 1e-5
    return ids.cpu().numpy()


@pytest.mark.parametrize("outputs,top,count,keep", [(8, 2, 4, 2), (18, 2, 2, 1), (6, 3, 3, 2), (4, 4, 2, 2), (5, 3, 1, 1), (28, 4, 7, 3),
                                                      (3, 1, 1, 1), (64, 8, 8, 4), (130, 6, 10, 3)])
def test_router_choice_in_groups(ops, outputs, top, count, keep):
    """The router alone (the oracle gets the logits through an identity router matrix).  Corrections of every sign:
    when all choice values are negative, a group that is left out must count as minus infinity, not as 0."""
    gen = torch.Generator().manual_seed(outputs * 10 + top)
    logits = torch.randn(50, outputs, generator=gen) * 2
    for correction in (None, torch.randn(outputs, generator=gen) * 0.2, -1.0 - torch.rand(outputs, generator=gen),
                       torch.linspace(-0.5, 0.5, outputs)):
        ids = _route_case(ops, logits, correction, top, count, keep)
        per = outputs // count
        assert all(len({int(e) // per for e in row}) <= keep for row in ids)
        assert all(len(set(row.tolist())) == top for row in ids)


def test_router_correction_steers_the_choice_and_not_the_weights(ops):
    logits = torch.tensor([[3.0, 2.0, 1.0, 0.0, -1.0, -2.0]])
    plainly = _route_case(ops, logits, None, 2, 1, 1)
    steered = _route_case(ops, logits, torch.tensor([0.0, 0.0, 0.0, 0.0, 5.0, 5.0]), 2, 1, 1)
    assert plainly.tolist() == [[0, 1]] and steered.tolist() == [[4, 5]]
    # groups of three: the group with the single best value wins, although the other has the larger sum
    grouped = _route_case(ops, torch.tensor([[2.0, -9.0, -9.0, 1.9, 1.9, 1.9]]), None, 2, 2, 1)
    assert grouped.tolist() == [[0, 1]]


def _experts(gen, experts, ff, width, dtype):
    up = (torch.randn(experts, ff, width, generator=gen) * width ** -0.5).to(TORCH[dtype])
    down = (torch.randn(experts, width, ff, generator=gen) * ff ** -0.5).to(TORCH[dtype])
    return up, down


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,experts,identity,top,count,keep", [(96, 32, 6, 2, 2, 4, 2), (100, 18, 5, 1, 3, 3, 2), (64, 64, 4, 0, 1, 1, 1),
                                                                      (48, 16, 1, 3, 2, 2, 1), (128, 64, 24, 4, 4, 7, 3)])
@pytest.mark.parametrize("tokens", [1, 5, 33, 150])
def test_routed_feed_forward_part(dtype, width, ff, experts, identity, top, count, keep, tokens):
    """The part alone, through both ways (every pair reading its expert directly; pairs grouped by expert and
    multiplied block by block): the weighted sum added into the stream, identity experts giving the input itself."""
    from aegean_tge_b200 import ops
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import FEED_FORWARDS, build_part
    from aegean_tge_b200.parts.base import BuildEnv, StepContext
    env = BuildEnv(dtype=TORCH[dtype], device=DEV, hidden_size=width, max_positions=64, page_size=16, ops=ops)
    names = {"router.weight": "r", "correction": "c"}
    names.update({f"experts.{e}.{t}.weight": f"e{e}{t}" for e in range(experts) for t in ("up", "down")})
    part = build_part(FEED_FORWARDS, PartSpec("routed_experts", {"hidden_size": width, "intermediate_size": ff, "experts": experts,
                                                                 "top": top, "identity": identity, "group_count": count,
                                                                 "group_keep": keep}, names), env)
    gen = torch.Generator().manual_seed(width + tokens)
    up, down = _experts(gen, experts, ff, width, dtype)
    router = (torch.randn(experts + identity, width, generator=gen) * 2 * width ** -0.5).to(TORCH[dtype])
    correction = torch.randn(experts + identity, generator=gen) * 0.1
    tensors = {"router.weight": router.to(DEV), "correction": correction.to(DEV)}
    for e in range(experts):
        tensors[f"experts.{e}.up.weight"], tensors[f"experts.{e}.down.weight"] = up[e].to(DEV), down[e].to(DEV)
    part.load(tensors)
    h = torch.randn(tokens, width, generator=gen).to(TORCH[dtype])
    x = torch.randn(tokens, width, generator=gen)
    w = {"p.router": router.double().numpy(), "p.correction": correction.double().numpy()}
    for e in range(experts):
        w[f"p.e{e}.up"], w[f"p.e{e}.down"] = up[e].double().numpy(), down[e].double().numpy()
    mlp = {"router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": count, "keep": keep}}}
    ref = x.double() + torch.from_numpy(plain.moe_ff(h.double().numpy(), w, "p.", mlp))
    ctx = StepContext(num_tokens=tokens, num_seqs=1, token_ids=None, positions=None, seq_of_token=None, q_start=None, start_pos=None,
                      ctx_len=None, slots=None, block_tables=[], max_q_len=tokens, max_ctx_len=tokens)
    stream = x.to(DEV)
    part.forward_add(h.to(DEV), stream, ctx)
    assert rel_error(stream, ref) < KERNEL_TOL[dtype]
    if tokens > 32:       # the same rows as single tokens take the direct way: same result within rounding
        ctx.max_q_len = 1
        again = x.to(DEV)
        part.forward_add(h.to(DEV), again, ctx)
        assert rel_error(again, ref) < KERNEL_TOL[dtype]
        assert rel_error(again, stream) < (1e-5 if dtype == "float32" else 2e-2)
    ops.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward_with_biases_and_two_parameter_activation(dtype):
    from aegean_tge_b200 import ops
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import FEED_FORWARDS, build_part
    from aegean_tge_b200.parts.base import BuildEnv
    width, ff = 72, 200
    env = BuildEnv(dtype=TORCH[dtype], device=DEV, hidden_size=width, max_positions=64, page_size=16, ops=ops)
    names = {"up.weight": "u", "up.bias": "ub", "down.weight": "d", "down.bias": "db", "act": "a"}
    part = build_part(FEED_FORWARDS, PartSpec("dense_mlp", {"hidden_size": width, "intermediate_size": ff, "activation": "xielu",
                                                            "bias": True}, names), env)
    assert set(part.param_specs()) == set(names)
    gen = torch.Generator().manual_seed(5)
    up = (torch.randn(ff, width, generator=gen) * 0.2).to(TORCH[dtype])
    down = (torch.randn(width, ff, generator=gen) * 0.1).to(TORCH[dtype])
    ub, db, act = torch.randn(ff, generator=gen), torch.randn(width, generator=gen), torch.tensor([0.4, -0.3])
    part.load({"up.weight": up.to(DEV), "down.weight": down.to(DEV), "up.bias": ub.to(DEV), "down.bias": db.to(DEV), "act": act.to(DEV)})
    h = torch.randn(11, width, generator=gen).to(TORCH[dtype])
    w = {"p.up": up.double().numpy(), "p.up.b": ub.double().numpy(), "p.down": down.double().numpy(), "p.down.b": db.double().numpy(),
         "p.act": act.double().numpy()}
    ref = torch.from_numpy(plain.dense_ff(h.double().numpy(), w, "p."))
    assert rel_error(part.forward(h.to(DEV), None), ref) < 2 * KERNEL_TOL[dtype]
    x = torch.randn(11, width, generator=gen)
    stream = x.to(DEV)
    part.forward_add(h.to(DEV), stream, None)
    assert rel_error(stream, x.double() + ref) < 2 * KERNEL_TOL[dtype]


# ---------------------------------------------------------------------------
# attention over the latent cache
class _LatentCase:
    """A latent attention part with weights of its own, pages shuffled over a pool with junk in it, and the plain
    function on whole sequences beside it."""

    def __init__(self, dtype, hidden, heads, dim, rot, vdim, q_rank, kv_rank, scale, base, dims, gate, page_size=16, seed=0,
                 matched=False, expand="never"):
        from aegean_tge_b200 import ops
        from aegean_tge_b200.config import PartSpec
        from aegean_tge_b200.parts import MIXERS, build_part
        from aegean_tge_b200.parts.base import BuildEnv
        self.ops, self.dtype, self.hidden, self.page_size = ops, dtype, hidden, page_size
        self.m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
                  "rot": {"base": base, "dims": dims}}
        self.gate = gate
        self.env = BuildEnv(dtype=TORCH[dtype], device=DEV, hidden_size=hidden, max_positions=2048, page_size=page_size, ops=ops)
        position = PartSpec("rope_interleaved", {"head_dim": rot, "theta": base, "rotary_dim": dims})
        self.params = {"hidden_size": hidden, "heads": heads, "head_dim": dim, "rope_dim": rot, "value_dim": vdim, "q_rank": q_rank,
                       "kv_rank": kv_rank, "scale": scale, "eps": 1e-5, "gate": gate, "position": position, "expand_keys": expand}
        locals_ = ["dq.weight", "dq_norm.weight", "uq.weight", "dkv.weight", "dkv_norm.weight", "uk.weight", "uv.weight", "o.weight"]
        if gate != "none":
            locals_.append("g.weight")
        self.part = build_part(MIXERS, PartSpec("latent_attention", self.params, {n: n for n in locals_}), self.env)
        gen = torch.Generator().manual_seed(seed)
        mk = lambda rows, cols: (torch.randn(rows, cols, generator=gen) * cols ** -0.5).to(TORCH[dtype])
        gates = {"none": 0, "head": heads, "element": heads * vdim}[gate]
        t = {"dq.weight": mk(q_rank, hidden), "uq.weight": mk(heads * (dim + rot), q_rank), "dkv.weight": mk(kv_rank + rot, hidden),
             "uk.weight": mk(heads * dim, kv_rank), "uv.weight": mk(heads * vdim, kv_rank), "o.weight": mk(hidden, heads * vdim),
             "dq_norm.weight": 1 + 0.1 * torch.randn(q_rank, generator=gen), "dkv_norm.weight": 1 + 0.1 * torch.randn(kv_rank, generator=gen)}
        if gates:
            t["g.weight"] = mk(gates, hidden)
        if matched:
            # queries and keys made alike: with equal latents the plain parts of q and k are the same vector, so the
            # score of a query with the key of a row made for it is |k|^2, the largest any key of that length can reach
            assert q_rank == kv_rank
            t["uq.weight"].view(heads, dim + rot, q_rank)[:, :dim] = t["uk.weight"].view(heads, dim, kv_rank)
            t["uq.weight"].view(heads, dim + rot, q_rank)[:, dim:] *= 0.05
            t["dq_norm.weight"] = t["dkv_norm.weight"].clone()
        self.tensors = t
        self.part.load({k: v.to(DEV) for k, v in t.items()})
        self.w = {"p." + k.replace(".weight", "").replace("_norm", ".norm"): v.double().numpy() for k, v in t.items()}
        self.gen = gen

    def row_for(self, h_query):
        """An input row whose kv latent equals the query latent of ``h_query`` (matched weights)."""
        dq, dkv = self.tensors["dq.weight"].double(), self.tensors["dkv.weight"].double()[: self.m["kv_rank"]]
        return (torch.linalg.pinv(dkv) @ (dq @ h_query.double())).to(TORCH[self.dtype])

    def plain(self, h):
        positions = np.arange(h.shape[0])
        rows = h.double().numpy()
        kv = plain.latent_kv(rows, self.w, "p.", self.m, 1e-5, positions)
        if self.gate == "none":
            w = dict(self.w)
            w["p.g"] = np.zeros((self.m["heads"], self.hidden))
            return torch.from_numpy(plain.latent_attention(rows, w, "p.", self.m, 1e-5, positions, "head", kv)) * 2.0
        return torch.from_numpy(plain.latent_attention(rows, self.w, "p.", self.m, 1e-5, positions, self.gate, kv))

    def run(self, sequences, cuts, reader=None):
        """Runs the part over the sequences cut into steps (``cuts[step][request]`` tokens, 0: not in the step) and returns
        every request's rows.  ``reader``: a second part that reads the entries this one stores (after it, in every step)."""
        from aegean_tge_b200.parts import LayerCache
        from aegean_tge_b200.parts.base import StepContext
        ps = self.page_size
        need = [-(-len(s) // ps) for s in sequences]
        pages = sum(need) + 3
        order = list(range(pages))
        random.Random(7).shuffle(order)
        entry = self.m["kv_rank"] + self.m["rot_dim"]
        store = (torch.randn(pages, 1, ps, entry, generator=self.gen) * 3).to(TORCH[self.dtype]).to(DEV)     # junk, finite
        table = torch.full((len(sequences), max(need)), -1, dtype=torch.int32)
        cursor = 0
        for r, n in enumerate(need):
            table[r, :n] = torch.tensor(order[cursor:cursor + n], dtype=torch.int32)
            cursor += n
        done = [0] * len(sequences)
        got = [[] for _ in sequences]
        also = [[] for _ in sequences]
        for step in cuts:
            live = [r for r in range(len(sequences)) if step[r] > 0]
            lens, starts = [step[r] for r in live], [done[r] for r in live]
            positions, seq, q_start, start_pos = _index(lens, starts)
            ctx = StepContext(num_tokens=sum(lens), num_seqs=len(live), token_ids=positions, positions=positions, seq_of_token=seq,
                              q_start=q_start, start_pos=start_pos, ctx_len=_i32([s + n for s, n in zip(starts, lens)]),
                              slots=_i32(list(range(len(live)))), block_tables=[table[live].contiguous().to(DEV)], max_q_len=max(lens),
                              max_ctx_len=max(s + n for s, n in zip(starts, lens)), host_q_lens=lens, host_start_pos=starts,
                              host_slots=list(range(len(live))))
            h = torch.cat([sequences[r][done[r]:done[r] + step[r]] for r in live]).to(DEV)
            out = self.part.forward(h, ctx, LayerCache(paged={"kv": store}, group=0, owner=True))
            more = reader.part.forward(h, ctx, LayerCache(paged={"kv": store}, group=0, owner=False)) if reader is not None else None
            row = 0
            for r in live:
                got[r].append(out[row:row + step[r]])
                if more is not None:
                    also[r].append(more[row:row + step[r]])
                row += step[r]
                done[r] += step[r]
        self.ops.check_status()
        return [torch.cat(g) for g in got], ([torch.cat(a) for a in also] if reader is not None else None)


LATENT_SHAPES = [  # hidden, heads, dim, rot, vdim, q_rank, kv_rank, scale, base, dims, gate
    (96, 4, 32, 16, 32, 48, 48, 0.3, 5000.0, 16, "element"),
    (64, 1, 32, 32, 32, 32, 32, 0.125, 10000.0, 32, "head"),
    (100, 3, 12, 6, 10, 20, 14, 0.4, 50.0, 4, "head"),
    (128, 20, 64, 32, 64, 64, 128, 0.1, 500000.0, 32, "none"),
    (80, 5, 6, 10, 12, 14, 22, 0.7, 9.0, 10, "element"),
]
LATENT_CUTS = [[[70, 45]], [[40, 3], [2, 40], [28, 2]], [[1, 0], [1, 1], [2, 1], [1, 17], [0, 1], [65, 25]]]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", LATENT_SHAPES)
@pytest.mark.parametrize("cuts", LATENT_CUTS)
@pytest.mark.parametrize("page_size", [16, 64])
@pytest.mark.parametrize("expand", ["never", "always"])
def test_latent_attention_part_with_its_cache(dtype, shape, cuts, page_size, expand):
    """``expand``: the entries serve as one key/value head, or every head gets its own keys and values in pages of the
    step's own (what long portions do); the same function either way."""
    case = _LatentCase(dtype, *shape, page_size=page_size, seed=len(cuts), expand=expand)
    assert case.part.cache_spec().entries == (("kv", (1, shape[6] + shape[3])),) and case.part.cache_spec().window is None
    gen = torch.Generator().manual_seed(11)
    lengths = [sum(step[r] for step in cuts) for r in range(2)]
    sequences = [torch.randn(n, shape[0], generator=gen).to(TORCH[dtype]) for n in lengths]
    got, _ = case.run(sequences, cuts)
    for r in range(2):
        assert rel_error(got[r], case.plain(sequences[r])) < 1.5 * KERNEL_TOL[dtype], (r, lengths[r])


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_layer_that_reads_another_layers_entries(dtype):
    """The reader has other heads, sizes, scale and gate, no down projection of its own, and stores nothing."""
    owner = _LatentCase(dtype, 96, 4, 32, 16, 32, 48, 48, 0.3, 5000.0, 16, "element", seed=1)
    reader = _LatentCase(dtype, 96, 3, 16, 16, 48, 40, 48, 0.5, 5000.0, 16, "head", seed=2)
    from aegean_tge_b200.config import PartSpec
    from aegean_tge_b200.parts import MIXERS, build_part
    names = [n for n in reader.tensors if not n.startswith("dkv")]
    part = build_part(MIXERS, PartSpec("latent_attention", {**reader.params, "shared_kv": True}, {n: n for n in names}), reader.env)
    assert not any(n.startswith("dkv") for n in part.param_specs())
    part.load({n: reader.tensors[n].to(DEV) for n in names})
    reader.part = part
    gen = torch.Generator().manual_seed(12)
    sequences = [torch.randn(n, 96, generator=gen).to(TORCH[dtype]) for n in (70, 45)]
    for cuts in LATENT_CUTS:
        _, got = owner.run(sequences, cuts, reader=reader)
        for r in range(2):
            rows = sequences[r].double().numpy()
            positions = np.arange(rows.shape[0])
            kv = plain.latent_kv(rows, owner.w, "p.", owner.m, 1e-5, positions)
            ref = torch.from_numpy(plain.latent_attention(rows, reader.w, "p.", reader.m, 1e-5, positions, "head", kv))
            assert rel_error(got[r], ref) < 1.5 * KERNEL_TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page_size", [16, 64])
@pytest.mark.parametrize("tail", [0, 1, 40])
@pytest.mark.parametrize("expand", ["auto", "always"])
def test_one_far_key_among_hundreds_stands_out(dtype, page_size, tail, expand):
    """Queries and keys are made alike and the softmax sharp, so the last prompt token (or, with a tail, a token decoded
    alone after it) gives nearly all its weight to the one row made for it: the first token, a page's last or first
    entry, or a row hundreds of tokens back.  Without that row the output is another."""
    case = _LatentCase(dtype, 96, 4, 32, 16, 48, 40, 40, 3.0, 5000.0, 16, "head", page_size=page_size, seed=3, matched=True,
                       expand=expand)
    gen = torch.Generator().manual_seed(13)
    length = 600
    for place in (0, 1, page_size - 1, page_size, 63, 64, 65, 300, length - 3):
        h = torch.randn(length + tail, 96, generator=gen).to(TORCH[dtype])
        h[place] = case.row_for(h[-1])
        ref = case.plain(h)
        without = h.clone()
        without[place] = torch.randn(96, generator=gen).to(TORCH[dtype])
        assert rel_error(case.plain(without)[-1:], ref[-1:]) > 0.3, place           # the test's own sharpness
        cuts = [[length]] + [[1]] * tail
        got, _ = case.run([h], cuts)
        assert rel_error(got[0][-1:], ref[-1:]) < 2 * KERNEL_TOL[dtype], (place, tail)
        if dtype == "float32":          # in bfloat16 a sharp softmax lets rows with two close keys differ by more
            assert rel_error(got[0], ref) < 2 * KERNEL_TOL[dtype], (place, tail)


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


@pytest.mark.parametrize("name", ["A", "C"])
def test_each_mechanism_left_out_would_show(oracle, name):
    """The oracle with one mechanism changed differs from itself by far more than the tolerance: so the whole-model
    tests would see a kernel that got that mechanism wrong."""
    tokens = _tokens(name, 90, salt=3)
    ref = oracle(name, "float32", tokens)
    def groups_off(c): c["norm"]["groups"] = 1
    def other_base(c): c["layers"][0]["mixer"]["rot"]["base"] *= 3.0
    def other_scale(c): c["layers"][1]["mixer"]["scale"] *= 1.3
    def other_kind(c): c["layers"][0]["type"], c["layers"][1]["type"] = c["layers"][1]["type"], c["layers"][0]["type"]
    def all_groups(c): c["layers"][0]["mlp"]["router"]["groups"]["keep"] = c["layers"][0]["mlp"]["router"]["groups"]["count"]
    for change in (groups_off, other_base, other_scale, all_groups):
        assert rel_error(oracle(name, "float32", tokens, config=_without(CONFIGS[name], change)), ref) > 1e-3, change.__name__
    assert rel_error(oracle(name, "float32", tokens, shift=False), ref) > 1e-2


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
    ref = oracle(name, dtype, tokens)
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
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_long_decoding(folders, oracle, name, dtype):
    """Three tokens of prompt, then 330 single tokens through the decode graphs, over many page borders."""
    tokens = _tokens(name, 333, salt=5)
    ref = oracle(name, dtype, tokens)
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
    a step with what (no shift row leaks between a slot's users; steps queued ahead and dropped leave none)."""
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
def test_trace_replay_of_a_puputar_model(folders, oracle, tmp_path, dtype):
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
