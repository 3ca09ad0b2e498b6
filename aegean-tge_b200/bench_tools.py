"""Timed prefill and decode steps with their roofline fractions, shared by `tge bench` and bench.py.

Timing is with CUDA events on the launching stream after warm-up, with a
synchronize on both sides.  A decode step reads every weight once (about
15 GB for the 7B shape) plus the cache of the live requests, far more than
the 126 MB L2, so no extra flush is needed between steps; the prefill's
weights are likewise larger than L2.
"""
from __future__ import annotations

import random
from typing import Dict, List

import torch

from . import peaks as _peaks
from .engine.batch import Portion


def _random_tokens(vocab: int, count: int, seed: int) -> List[int]:
    rnd = random.Random(seed)
    return [rnd.randrange(vocab) for _ in range(count)]


def prefill_flops(engine, tokens: int) -> float:
    """Operations of one whole prompt (a multiply-add is two): what the model's parts report for ``tokens``
    tokens under a causal mask, and one row of logits."""
    return engine.model.step_flops(tokens, tokens * (tokens + 1) / 2.0, 1)


def bench_prefill(engine, prompt_len: int, repeat: int = 3, warmup: int = 2, sustain_seconds: float = 0.0) -> Dict[str, float]:
    """A whole prompt in one step, timed on the device: the mean of ``repeat`` runs after ``warmup``.

    A B200 under its power cap runs the first steps after a pause faster than it sustains (a 2,048-token
    prompt of the 7B shape: 20.3 ms for two or three runs, then 22.5-23.5 ms).  With ``sustain_seconds`` > 0 two
    more figures are taken, to be read against the two peaks measured the same ways: ``burst_ms`` (the best of
    three runs after a pause of two seconds; the burst peak is a best of ten) and ``sustained_ms`` (the mean over
    a loop of that many seconds; the sustained peak is a loop of four seconds)."""
    import time
    vocab = engine.spec.vocab_size
    counter = [0]

    def one() -> float:
        tokens = _random_tokens(vocab, prompt_len, seed=100 + counter[0] % 7)
        counter[0] += 1
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.runner.step([Portion("bench-prefill", tokens, [prompt_len - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.runner.finish("bench-prefill")
        return start.elapsed_time(stop)

    for _ in range(warmup):
        one()
    times = [one() for _ in range(repeat)]
    ms = sum(times) / len(times)
    flops = prefill_flops(engine, prompt_len)
    peak, source = _peaks.load()
    tflops = flops / (ms * 1e-3) / 1e12
    out = {"tokens": prompt_len, "ms": ms, "tok_s": prompt_len / (ms * 1e-3), "tflops": tflops,
           "peak_tflops": peak["bf16_tflops"], "frac": tflops / peak["bf16_tflops"], "peak_source": source,
           "flops": flops}
    if sustain_seconds > 0:
        begin = time.perf_counter()
        loop = []
        while time.perf_counter() - begin < sustain_seconds:
            loop.append(one())
        out["sustained_ms"] = sum(loop) / len(loop)
        sustained_peak = peak.get("bf16_tflops_sustained", peak["bf16_tflops"])
        out["sustained_frac"] = flops / (out["sustained_ms"] * 1e-3) / 1e12 / sustained_peak
        time.sleep(2.0)
        out["burst_ms"] = min(one() for _ in range(3))
        out["burst_frac"] = flops / (out["burst_ms"] * 1e-3) / 1e12 / peak["bf16_tflops"]
    return out


def fill_cache(engine, batch: int, prompt_len: int, chunk: int = 2048, prefix: str = "bench") -> List[str]:
    """Prefills ``batch`` requests of ``prompt_len`` random tokens (untimed); returns their ids."""
    vocab = engine.spec.vocab_size
    names = []
    for b in range(batch):
        name = f"{prefix}-{b}"
        tokens = _random_tokens(vocab, prompt_len, seed=1000 + b)
        for begin in range(0, prompt_len, chunk):
            engine.runner.step([Portion(name, tokens[begin:begin + chunk], [])])
        names.append(name)
    return names


def decode_step_bytes(engine, names: List[str]) -> float:
    """Bytes a decode step must move: every weight it uses once, and of each live request the cache entries it may
    read (a window's, where there is one) and the fixed-size state it reads and writes."""
    return engine.model.step_param_bytes(len(names)) + sum(engine.model.decode_cache_bytes(engine.cache.computed(n)) for n in names)


def bench_decode(engine, batch: int, prompt_len: int, steps: int = 64, warmup: int = 3) -> Dict[str, float]:
    """Device-timed decode steps (model and sampling kernels; the sampled ids stay on the device)."""
    from . import ops
    names = fill_cache(engine, batch, prompt_len)
    vocab = engine.spec.vocab_size
    zeros = torch.zeros(batch, dtype=torch.float32, device=engine.device)
    feed = [_random_tokens(vocab, warmup + steps, seed=5000 + b) for b in range(batch)]
    def one(step: int):
        logits = engine.runner.step([Portion(n, [feed[b][step]], [0]) for b, n in enumerate(names)])
        return ops.sample(logits, zeros, zeros)
    for step in range(warmup):
        one(step)
    torch.cuda.synchronize()
    bytes_first = decode_step_bytes(engine, names)
    launches_before = ops.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(warmup, warmup + steps):
        one(step)
    stop.record()
    torch.cuda.synchronize()
    ops.check_status()
    ms = start.elapsed_time(stop) / steps
    bytes_last = decode_step_bytes(engine, names)
    for n in names:
        engine.runner.finish(n)
    step_bytes = (bytes_first + bytes_last) / 2
    peak, source = _peaks.load()
    gbs = step_bytes / (ms * 1e-3) / 1e9
    return {"batch": batch, "ms_per_step": ms, "tok_s": batch / (ms * 1e-3), "step_bytes": step_bytes, "gbs": gbs,
            "peak_gbs": peak["hbm_gbs"], "frac": gbs / peak["hbm_gbs"], "peak_source": source,
            "launches": ops.launches - launches_before, "steps": steps}


def bench_mixed(engine, decodes: int, prompt_len: int, portion: int, repeat: int = 3) -> Dict[str, float]:
    """One step of ``decodes`` single tokens (each request holding ``prompt_len`` tokens) beside one prompt
    portion of ``portion`` tokens, timed on the device: what a scheduler's step looks like while a prompt arrives."""
    names = fill_cache(engine, decodes, prompt_len, prefix="mixed")
    prompt = _random_tokens(engine.spec.vocab_size, portion, seed=31)
    times = []
    for it in range(repeat + 1):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.runner.step([Portion(n, [7 + it], [0]) for n in names] + [Portion("mixed-prompt", prompt, [portion - 1])])
        stop.record()
        torch.cuda.synchronize()
        engine.runner.finish("mixed-prompt")
        if it:
            times.append(start.elapsed_time(stop))
    for n in names:
        engine.runner.finish(n)
    ms = sum(times) / len(times)
    return {"ms": ms, "decodes": decodes, "portion": portion, "tok_s": (decodes + portion) / (ms * 1e-3)}


def step_timeline(engine, batch: int, prompt_len: int, prefill: bool, portion: int = 0) -> List[Dict[str, float]]:
    """Where one step's time goes, by kernel name, from the CUDA activity records of one step after
    warm-up: a prompt of ``prompt_len`` tokens (``prefill``) or one token for each of ``batch`` requests
    that hold ``prompt_len`` tokens, with ``portion`` > 0 beside one prompt portion of that many tokens.

    A kernel launched as the dependent of another starts early and waits, so its own duration says
    little.  What is charged to a kernel here is the time from the end of the kernel that ended before it
    (or from its own start, if later) to its own end: the charges add up to the span of the step less the
    gaps in which nothing ran.
    """
    from torch.profiler import ProfilerActivity, profile
    vocab = engine.spec.vocab_size
    if prefill:
        tokens = _random_tokens(vocab, prompt_len, seed=77)

        def run():
            engine.runner.step([Portion("timeline", tokens, [prompt_len - 1])])
            engine.runner.finish("timeline")
        names = []
    else:
        names = fill_cache(engine, batch, prompt_len, prefix="timeline")
        beside = _random_tokens(vocab, portion, seed=78) if portion > 0 else []

        def run():
            engine.runner.step([Portion(n, [5], [0]) for n in names] +
                               ([Portion("timeline-portion", beside, [portion - 1])] if portion > 0 else []))
            if portion > 0:
                engine.runner.finish("timeline-portion")
    for _ in range(4):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    for n in names:
        engine.runner.finish(n)
    events = [(e.time_range.start, e.time_range.start + e.device_time_total, e.name) for e in prof.events()
              if e.device_time_total > 0]
    events.sort(key=lambda e: e[1])
    first = min(e[0] for e in events)
    by_name: Dict[str, List[float]] = {}
    previous_end = first
    for start, end, raw in events:
        name = raw.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0].strip()
        by_name.setdefault(name, []).append(end - max(previous_end, start))
        previous_end = max(previous_end, end)
    span = previous_end - first
    rows = [{"kernel": name, "launches": len(v), "us": sum(v), "share": sum(v) / span} for name, v in by_name.items()]
    rows.sort(key=lambda r: -r["us"])
    rows.append({"kernel": "span of the step under the profiler", "launches": len(events), "us": span, "share": 1.0})
    return rows


# ----------------------------------------------------------------------------
# two designs side by side at equal size
# ----------------------------------------------------------------------------
def paired_configs(width: int, heads: int, kv_heads: int, head_dim: int, gated_inner: int, layers: int,
                   vocab: int) -> Dict[str, dict]:
    """A Qwen2 and a Lepizen config.json of the same width, heads, layers, vocabulary and parameter count: the
    ungated feed-forward gets one and a half times the gated one's inner width (two matrices instead of three)."""
    qwen2 = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": layers,
             "hidden_size": width, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
             "intermediate_size": gated_inner, "vocab_size": vocab, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
             "tie_word_embeddings": False, "max_position_embeddings": 32768, "use_sliding_window": False,
             "hidden_act": "silu"}
    layer = {"type": "attention",
             "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
                       "v_mix": True},
             "mlp": {"kind": "dense", "ff": gated_inner * 3 // 2}}
    lepizen = {"architecture": "Lepizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
               "logit_scale": 1.0, "logit_softcap": 50.0, "layers": [layer] * layers}
    return {"qwen2": qwen2, "lepizen": lepizen, "mozepel": mozepel_config(width, heads, kv_heads, head_dim, gated_inner, layers, vocab),
            "puputar": puputar_config(width, heads, head_dim, gated_inner, layers, vocab),
            "kokolorn": kokolorn_config(width, heads, kv_heads, head_dim, gated_inner, layers, vocab)}


def kokolorn_config(width: int, heads: int, kv_heads: int, head_dim: int, gated_inner: int, layers: int, vocab: int,
                    experts: int = 16, top: int = 4) -> dict:
    """A Kokolorn config.json with the width, heads, kv heads, head size and layer count of a Qwen2 shape, its layers by
    turns delta (keys and values of ``head_dim``, four taps, the clamped gated feed-forward of the gated inner width),
    attention (the shape's GQA; ``experts`` experts of a quarter of the gated inner width of which ``top`` are used, and
    a shared one of half of it: as many multiplications per token as the dense one), parallel (the shape's GQA with a
    bias by distance up to 2,048 beside a state-space mixer of as many heads, states of 128 rows, four taps) and
    attention again; one pass over all layers, so the stream is mixed with the embedding once."""
    quarter = max(gated_inner // 4 // 64 * 64, 64)
    dense = {"kind": "dense", "ff": gated_inner, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": quarter}, "router": {"experts": experts, "top": top}, "shared": {"ff": 2 * quarter}}
    temp = {"coef": 0.1, "every": 1024}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "q_temp": temp}
    kinds = [
        {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "conv": 4}, "mlp": dense},
        {"type": "attention", "mixer": dict(attention), "mlp": moe},
        {"type": "parallel", "mixer": {"left": dict(attention, bias_max=2048.0),
                                       "right": {"heads": heads, "vdim": head_dim, "state": 128, "groups": kv_heads,
                                                 "norm_groups": kv_heads, "conv": 4}}, "mlp": moe},
        {"type": "attention", "mixer": dict(attention), "mlp": moe}]
    return {"architecture": "Kokolorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": [kinds[n % 4] for n in range(layers)], "loop": {"start": 0, "stop": layers, "times": 1}}


def puputar_config(width: int, heads: int, head_dim: int, gated_inner: int, layers: int, vocab: int, experts: int = 16,
                   top: int = 4) -> dict:
    """A Puputar config.json with the width, heads, head size and layer count of a Qwen2 shape: queries and keys of
    ``head_dim`` numbers (half of them rotated), values of ``head_dim``, a query latent of a quarter of the width, cache
    entries of 192 + head_dim / 2 numbers; layers by turns with the dense feed-forward (two matrices of one and a
    half times the gated inner width) and with ``experts`` small experts and four identity experts, in four groups of
    which two are kept, of which ``top`` are used (together as wide as the dense one); every fourth layer reads the entries of the routed layer before it."""
    rot = head_dim // 2
    mixer = {"heads": heads, "dim": head_dim - rot, "rot_dim": rot, "vdim": head_dim, "q_rank": max(width // 4 // 64 * 64, 64),
             "kv_rank": 192, "scale": head_dim ** -0.5, "rot": {"base": 500000.0, "dims": rot}}
    dense = {"kind": "dense", "ff": gated_inner * 3 // 2}
    routed = {"kind": "moe", "expert": {"ff": max(gated_inner * 3 // 2 // top // 64 * 64, 64)},
              "router": {"experts": experts, "top": top, "identity": 4, "groups": {"count": 4, "keep": 2}}}
    out = []
    for n in range(layers):
        if n % 2 == 0:
            out.append({"type": "latent_attention", "mixer": dict(mixer), "mlp": dense})
        elif n % 4 == 1:
            out.append({"type": "latent_attention_2", "mixer": dict(mixer), "mlp": routed})
        else:
            out.append({"type": "latent_attention_2", "mixer": dict(mixer, kv_from=n - 2), "mlp": routed})
    return {"architecture": "Puputar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6, "groups": 2}, "layers": out}


def mozepel_config(width: int, heads: int, kv_heads: int, head_dim: int, gated_inner: int, layers: int, vocab: int,
                   window: int = 1024, pool: int = 64) -> dict:
    """A Mozepel config.json with the width, heads, head size, inner width and layer count of a Qwen2 shape: three
    retention layers (heads x head_dim keys and values) to one parallel layer (a window of ``window`` tokens with
    blocks of ``pool``, four taps, half of each head rotated; beside it half as many decayed heads with keys of half
    the size), all with the gated feed-forward."""
    decay = lambda n: [1.0 - 2.0 ** (-5.0 - 5.0 * h / max(n - 1, 1)) for h in range(n)]
    mlp = {"kind": "dense", "ff": gated_inner}
    retention = {"type": "retention", "mlp": mlp,
                 "mixer": {"heads": heads, "dim": head_dim, "vdim": head_dim, "decay": decay(heads),
                           "rot": {"base": 1000000.0, "dims": head_dim}}}
    right_heads = max(heads // 2, 1)
    parallel = {"type": "parallel", "mlp": mlp,
                "mixer": {"left_scale": 1.0, "right_scale": 0.5,
                          "left": {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
                                   "conv": 4, "mask": {"size": window, "pool": pool},
                                   "rot": {"base": 500000.0, "dims": head_dim // 2,
                                           "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
                          "right": {"heads": right_heads, "dim": max(head_dim // 2, 1), "vdim": head_dim, "decay": decay(right_heads)}}}
    return {"architecture": "Mozepel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "postln_alpha": 2.0,
            "layers": [parallel if n % 4 == 3 else retention for n in range(layers)]}


def compare_designs(configs: Dict[str, dict], prompt_len: int = 2048, batches=(8, 64), steps: int = 32, warmup: int = 3,
                    page_size: int = 64, timelines: bool = True) -> Dict[str, dict]:
    """Prefill and decode of each config (random weights drawn on the device, bfloat16), one engine at a time:
    a ``prompt_len``-token prompt against the bf16 peak, decode steps of each batch after prompts of that length
    against the copy bandwidth, and where the time of a prefill step and of a decode step of the first batch goes,
    kernel by kernel."""
    import gc
    import time
    from .engine.engine import Engine
    out: Dict[str, dict] = {}
    for name, config in configs.items():
        gc.collect()
        torch.cuda.empty_cache()
        most = max(batches)
        engine = Engine(random_config=config, seed=0, dtype="bfloat16", context=2 * prompt_len, page_size=page_size,
                        max_tokens=most * (prompt_len + steps + warmup + 80) + prompt_len, max_batch_tokens=prompt_len,
                        max_requests=most + 1)
        row: Dict[str, object] = {"weight_gb": round(engine.model.weight_bytes() / 1e9, 3),
                                  "step_param_gb": round(engine.model.step_param_bytes() / 1e9, 3)}
        run = bench_prefill(engine, prompt_len, repeat=3, warmup=2, sustain_seconds=0.5)
        row["prefill"] = {"tokens": prompt_len, "ms": round(run["burst_ms"], 3), "tok_s": round(prompt_len / (run["burst_ms"] * 1e-3), 1),
                          "tflops": round(run["flops"] / (run["burst_ms"] * 1e-3) / 1e12, 1), "frac": round(run["burst_frac"], 4),
                          "sustained_ms": round(run["sustained_ms"], 3), "sustained_frac": round(run["sustained_frac"], 4)}
        for batch in batches:
            torch.cuda.synchronize()
            time.sleep(2.0)
            run = bench_decode(engine, batch, prompt_len, steps=steps, warmup=warmup)
            row[f"decode_b{batch}"] = {"ms_per_step": round(run["ms_per_step"], 4), "tok_s": round(run["tok_s"], 1),
                                      "gbs": round(run["gbs"], 1), "hbm_frac": round(run["frac"], 4),
                                      "launches_per_step": run["launches"] // run["steps"]}
        if timelines:
            keep = lambda rows: [{"kernel": r["kernel"], "launches": r["launches"], "us": round(r["us"], 1),
                                  "share": round(r["share"], 4)} for r in rows[:12] + rows[-1:]]
            row["prefill_kernels"] = keep(step_timeline(engine, 1, prompt_len, prefill=True))
            row["decode_kernels"] = keep(step_timeline(engine, batches[0], prompt_len, prefill=False))
            if len(batches) > 1:
                row[f"decode_kernels_b{batches[-1]}"] = keep(step_timeline(engine, batches[-1], prompt_len, prefill=False))
        out[name] = row
        del engine
    return out
