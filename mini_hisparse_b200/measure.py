"""Measurement of the decode step and of a prompt's prefill: timing, byte and flop counts.

The reference measures only its storage path (experiments/benchmark.py:1, docs/benchmarks.md:88:
"not LLM tokens/s"); generation speed is this engine's own metric.  A decode step is timed on
the device with CUDA events around K consecutive steps of the engine's step function (graph
replay plus the copy of that step's index arrays); the end-to-end number goes through
``Engine.step()`` with host token lists in and out.  Every step reads all weights (far more than
the L2 holds), so no L2 flush is needed between steps.
"""
from __future__ import annotations

import json
import subprocess
import time
from pathlib import Path

import torch

from .kernels import api as K

ROOT = Path(__file__).resolve().parent.parent
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                  "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            out = {"source": "measured"}
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                out[k] = float(d[k]) if k in d else FALLBACK_PEAKS[k]
            return out
        except Exception:   # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if clocks:
            clocks.sort()
            self.result = {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": mx,
                           "reasons": sorted(reasons), "samples": len(clocks)}


# ---- counts -------------------------------------------------------------------------------------
def headline_config(config: dict, *, batch: int, context: int, layers: int, page_size: int) -> dict:
    """The ``config`` of the headline bench line, from the model's config.json keys: both arms of the
    benchmark print the same dictionary for the same shape."""
    heads = config["num_attention_heads"]
    return {
        "model": "Qwen2.5-7B shape", "global_batch": batch, "seq_len": context, "parallelism": "single GPU",
        "layers": layers, "layers_of_config": config["num_hidden_layers"], "hidden": config["hidden_size"],
        "q_heads": heads, "kv_heads": config["num_key_value_heads"],
        "head_dim": config.get("head_dim") or config["hidden_size"] // heads,
        "intermediate": config["intermediate_size"], "vocab": config["vocab_size"], "page_size": page_size,
        "l2": "inputs larger than L2 (all weights are read every step)", "peaks": f"of {peaks()['source']}",
    }


def decode_bytes(model, cache, live_tokens: int) -> int:
    """Bytes a decode step has to read: every weight it uses once (the embedding table is only
    gathered, so it does not count unless it is also the tied head) and the cache of the live
    requests."""
    weights = model.weight_bytes()
    emb = model.embedding.weight
    if model.head.weight.data_ptr() != emb.data_ptr():
        weights -= emb.numel() * emb.element_size()
    kv = 0
    for g in cache.page_groups:
        kv += g.page_bytes() // cache.cfg.page_size * live_tokens
    return weights + kv


def prefill_flops(cfg, layers: int, T: int) -> float:
    """2 flops per weight element per token for the products, 4 nq d per (query, key) pair for
    causal attention (half of T^2 pairs)."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_token = 2 * (H * (q + 2 * kv) + q * H + 3 * H * I)
    attn = 4 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2
    return layers * (per_token * T + attn) + 2 * H * V     # the head runs on the last row only


# ---- building ---------------------------------------------------------------------------------
def build_engine(config: dict, *, batch: int, context: int, dtype="bfloat16", device="cuda:0",
                 page_size=16, weight_seed=0, layers: int | None = None, max_tokens_per_step=2048,
                 extra_pages: int = 0):
    from .engine.engine import Engine, load_model

    config = dict(config)
    if layers is not None:
        config["num_hidden_layers"] = layers
    model = load_model(config, device=device, dtype=dtype, random_seed=weight_seed)
    pages = batch * -(-context // page_size) + extra_pages
    # graph_after=1: the benchmarks time the steady state, and their warm-up is a few steps
    engine = Engine(model, num_pages=pages, page_size=page_size, max_requests=batch,
                    max_tokens_per_step=max_tokens_per_step, graph_after=1)
    return engine


def synthetic_context(engine, batch: int, tokens: int, seed: int = 0) -> list[str]:
    """Open ``batch`` requests that already hold ``tokens`` cached positions each.  The pages are
    filled with random keys and values instead of running prompts through the model: like the
    weights, the cache content is synthetic, and a decode step's cost does not depend on it."""
    cache = engine.cache
    names = []
    gen = torch.Generator(device=cache.cfg.device).manual_seed(seed)
    for g in cache.page_groups:
        g.storage.normal_(0.0, 0.5, generator=gen)
    for i in range(batch):
        name = f"bench{i}"
        cache.open(name)
        cache.ensure(name, tokens)
        cache.advance(name, tokens)
        names.append(name)
    return names


def time_decode(engine, names, steps: int, warmup: int, vocab: int, sampled_warmup: int = 0) -> dict:
    """Device time of ``steps`` decode steps of the step function (one token per request).

    The clocks are sampled every 100 ms (more often disturbs the timing), so a short timed region may
    see no sample: ``sampled_warmup`` further untimed steps of the same load run between the warm-up
    and the timed steps with the sampler already on."""
    from .engine.step import StepEntry

    B = len(names)
    gen = torch.Generator().manual_seed(1)
    def entries():
        toks = torch.randint(0, vocab, (B,), generator=gen).tolist()
        return [StepEntry(n, [t], [0]) for n, t in zip(names, toks)]
    for _ in range(warmup):
        engine.runner.step(entries())
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = K.launches
    with ClockSampler() as clocks:
        for _ in range(sampled_warmup):
            engine.runner.step(entries())
        launches0 = K.launches
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            engine.runner.step(entries())
        end.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    engine.runner.check_status()
    return {"ms_per_step": ms / steps, "tokens_per_s": B * steps / (ms / 1e3),
            "launches": K.launches - launches0, "clocks": clocks.result}


def decode_benchmark(config: dict, *, batch=8, prompt_tokens=1024, steps=20, warmup=3,
                     dtype="bfloat16", device="cuda:0", page_size=16, weight_seed=0,
                     layers: int | None = None) -> dict:
    """What ``bench`` of the command line prints: decode tokens a second at one batch size."""
    engine = build_engine(config, batch=batch, context=prompt_tokens + steps + warmup + 1, dtype=dtype,
                          device=device, page_size=page_size, weight_seed=weight_seed, layers=layers)
    names = synthetic_context(engine, batch, prompt_tokens)
    r = time_decode(engine, names, steps, warmup, engine.model.spec.vocab_size)
    live = batch * (prompt_tokens + warmup + steps // 2)
    nbytes = decode_bytes(engine.model, engine.cache, live)
    p = peaks()
    gbs = nbytes / (r["ms_per_step"] / 1e3) / 1e9
    return {"metric": "decode tokens/s", "batch": batch, "context": prompt_tokens, "dtype": dtype,
            "tokens_per_second": r["tokens_per_s"], "ms_per_step": r["ms_per_step"],
            "bytes_per_step": nbytes, "achieved_gbs": gbs,
            "hbm_fraction": gbs / p["hbm_gbs"], "peak_source": p["source"], "clocks": r["clocks"]}


def prefill_benchmark(config: dict, *, prompt_tokens=2048, max_tokens_per_step=2048, repeats=3, dtype="bfloat16",
                      device="cuda:0", page_size=16, weight_seed=0, layers: int | None = None) -> dict:
    """What ``bench --prefill`` prints: one prompt of ``prompt_tokens`` through ``Engine.step()`` in
    portions of at most ``max_tokens_per_step`` (wall clock, host work included), best of ``repeats``."""
    from .config.registry import resolve

    engine = build_engine(config, batch=1, context=prompt_tokens + 2, dtype=dtype, device=device,
                          page_size=page_size, weight_seed=weight_seed, layers=layers,
                          max_tokens_per_step=max_tokens_per_step, extra_pages=2)
    config = dict(config)
    if layers is not None:
        config["num_hidden_layers"] = layers
    cfg, _ = resolve(config)
    vocab = engine.model.spec.vocab_size
    g = torch.Generator().manual_seed(7)
    times = []
    with ClockSampler() as clocks:
        for i in range(repeats + 1):
            prompt = torch.randint(0, vocab, (prompt_tokens,), generator=g).tolist()
            engine.add_request(f"p{i}", prompt, max_new_tokens=1)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.run()
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
    sec = min(times[1:])
    segs, start = [], 0
    while start < prompt_tokens:
        n = min(max_tokens_per_step, prompt_tokens - start)
        segs.append((start, n))
        start += n
    flops = sum(step_flops(cfg, config["num_hidden_layers"], [sg], 0) for sg in segs) + 2 * cfg.hidden_size * cfg.vocab_size
    p = peaks()
    return {"metric": "prefill tokens/s (one prompt through Engine.step)", "prompt_tokens": prompt_tokens,
            "max_tokens_per_step": max_tokens_per_step, "layers": config["num_hidden_layers"], "dtype": dtype,
            "tokens_per_second": prompt_tokens / sec, "ms": sec * 1e3, "tflops": flops / sec / 1e12,
            "bf16_fraction_of_burst": flops / sec / 1e12 / p["bf16_tflops"],
            "bf16_fraction_of_sustained": flops / sec / 1e12 / p["bf16_tflops_sustained"], "peak_source": p["source"],
            "clocks": clocks.result}


# ---- serving workloads: requests through Engine.step(), host tokens in and out -----------------------
def step_flops(cfg, layers: int, segments: list[tuple[int, int]], logit_rows: int) -> float:
    """Floating-point operations of one step: 2 per weight element and token for the products, 4 d per
    (query head, query, key) pair for attention; ``segments`` holds (cached positions, new tokens)."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_token = 2 * (H * (q + 2 * kv) + q * H + 3 * H * I)
    tokens = sum(n for _, n in segments)
    pairs = sum(n * start + n * (n + 1) // 2 for start, n in segments)
    return layers * (per_token * tokens + 4 * q * pairs) + 2 * H * V * logit_rows


def _percentile(sorted_values, p):
    if not sorted_values:
        return None
    return sorted_values[min(len(sorted_values) - 1, int(p / 100.0 * len(sorted_values)))]


def serving_workload(config: dict, *, prompts: list[list[int]], max_new_tokens: int, max_tokens_per_step: int,
                     context: int, page_size: int = 16, dtype="bfloat16", device="cuda:0", weight_seed: int = 0,
                     layers: int | None = None, num_pages: int | None = None, label: str = "",
                     graph_after: int = 8) -> dict:
    """Run ``prompts`` through the engine as a server would: all requests are queued at once, the
    scheduler cuts the prompts into portions of at most ``max_tokens_per_step`` tokens beside the
    decode tokens of the requests that are already generating, greedy sampling, until every request
    has ``max_new_tokens`` tokens.  Wall-clock times per step (host work included: this is what a
    client sees), and for the whole run the bytes that had to be read (every weight once per step and
    the cache of the step's requests) and the floating-point operations, against the measured peaks.

    ``num_pages`` None sizes the pool for the requests' whole lifetimes; "free" takes what the device
    has left after the weights (less a reserve for the step's workspace)."""
    from .config.registry import resolve
    from .engine.engine import Engine, load_model

    config = dict(config)
    full_layers = config["num_hidden_layers"]
    if layers is not None:
        config["num_hidden_layers"] = layers
    layers = config["num_hidden_layers"]
    cfg, _ = resolve(config)
    model = load_model(config, device=device, dtype=dtype, random_seed=weight_seed)
    need_pages = sum(-(-(len(p) + max_new_tokens) // page_size) for p in prompts)
    probe_engine_pages = need_pages
    if num_pages == "free":
        torch.cuda.synchronize()
        free, _total = torch.cuda.mem_get_info(torch.device(device))
        kv_heads, d = cfg.num_key_value_heads, cfg.head_dim
        page_bytes = layers * 2 * kv_heads * page_size * d * (2 if dtype == "bfloat16" else 4)
        reserve = 6 << 30                       # logits, activations and plans of the largest step
        probe_engine_pages = max(need_pages, int((free - reserve) // page_bytes))
    elif num_pages is not None:
        probe_engine_pages = num_pages
    engine = Engine(model, num_pages=probe_engine_pages, page_size=page_size, max_requests=len(prompts),
                    max_tokens_per_step=max_tokens_per_step, graph_after=graph_after)
    for i, prompt in enumerate(prompts):
        engine.add_request(f"r{i}", prompt, max_new_tokens=max_new_tokens)
    weights = decode_bytes(model, engine.cache, 0)
    kv_per_token = sum(g.page_bytes() // page_size for g in engine.cache.page_groups)
    step_ms, kinds, read_bytes, flops = [], [], 0, 0.0
    generated = prompt_tokens = seen = 0
    torch.cuda.synchronize()
    with ClockSampler() as clocks:
        t_start = time.perf_counter()
        while not engine.scheduler.idle or engine._queued is not None:
            t0 = time.perf_counter()
            emitted = engine.step()
            step_ms.append((time.perf_counter() - t0) * 1e3)
            generated += len(emitted)
            # a call may launch no step, one, or two (a decode step queued behind the one it waits for)
            new = engine.launches - seen
            seen = engine.launches
            kind = "decode"
            for held in list(engine.launch_log)[len(engine.launch_log) - new:] if new else []:
                segs = [(start, n) for _, start, n in held]
                if not all(n == 1 for _, n in segs):
                    kind = "mixed"
                read_bytes += weights + kv_per_token * sum(start + n for start, n in segs)
                flops += step_flops(cfg, layers, segs, sum(1 for _ in segs))
            kinds.append(kind)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t_start
    engine.runner.check_status()
    prompt_tokens = sum(len(p) for p in prompts)
    p = peaks()
    ordered = sorted(step_ms)
    decode_ms = sorted(ms for ms, k in zip(step_ms, kinds) if k == "decode")
    mixed_ms = sorted(ms for ms, k in zip(step_ms, kinds) if k == "mixed")
    gbs, tflops = read_bytes / seconds / 1e9, flops / seconds / 1e12
    hbm_frac, flop_frac = gbs / p["hbm_gbs"], tflops / p["bf16_tflops_sustained"]
    snap = engine.snapshot()
    return {
        "workload": label, "requests": len(prompts), "prompt_tokens": prompt_tokens, "generated_tokens": generated,
        "max_new_tokens": max_new_tokens, "max_tokens_per_step": max_tokens_per_step, "context": context,
        "layers": layers, "layers_of_config": full_layers, "dtype": dtype, "page_size": page_size,
        "seconds": seconds, "generated_tokens_per_s": generated / seconds,
        "tokens_per_s": (generated + prompt_tokens) / seconds, "steps": len(step_ms),
        "step_ms": {"p50": _percentile(ordered, 50), "p90": _percentile(ordered, 90), "p99": _percentile(ordered, 99),
                    "max": ordered[-1] if ordered else None},
        "decode_step_ms": {"steps": len(decode_ms), "p50": _percentile(decode_ms, 50), "p99": _percentile(decode_ms, 99)},
        "mixed_step_ms": {"steps": len(mixed_ms), "p50": _percentile(mixed_ms, 50), "p99": _percentile(mixed_ms, 99)},
        "roofline": {"bound": "hbm" if hbm_frac >= flop_frac else "bf16", "hbm": {"achieved": gbs, "peak": p["hbm_gbs"],
                     "unit": "GB/s", "frac": hbm_frac}, "bf16": {"achieved": tflops, "peak": p["bf16_tflops_sustained"],
                     "unit": "TFLOP/s (sustained)", "frac": flop_frac}, "frac": max(hbm_frac, flop_frac),
                     "peaks": f"of {p['source']}"},
        "clocks": clocks.result, "pages": snap["cache"]["page_groups"][0]["pages_total"],
        "pages_peak": snap["cache"]["page_groups"][0]["pages_peak"], "gpu_launches": K.launches,
        "graph_after": graph_after,
        "graphs": {k: engine.runner.stats[k] for k in ("graph_steps", "graph_captures", "graph_deferred")},
        "data": "synthetic: seeded random weights, uniform-random token ids",
    }


def workload_prompts(name: str, vocab: int, seed: int = 0) -> tuple[list[list[int]], dict]:
    """The token ids and settings of the two named serving workloads."""
    g = torch.Generator().manual_seed(seed)
    if name == "serving14b":
        # 32 requests, prompts of 128 to 4,096 uniform-random tokens, portions of 512 beside decoding
        lengths = torch.randint(128, 4097, (32,), generator=g).tolist()
        settings = dict(max_new_tokens=128, max_tokens_per_step=512, context=8192, num_pages=None)
    elif name == "long32b":
        # 16 requests of 8,192 prompt tokens and 512 generated ones, the pool sized from free memory
        lengths = [8192] * 16
        settings = dict(max_new_tokens=512, max_tokens_per_step=2048, context=16384, num_pages="free")
    else:
        raise ValueError(f"unknown workload {name!r}: serving14b or long32b")
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
    return prompts, settings


# ---- two architectures side by side at equal size -------------------------------------------------------
def koronex_shape(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, layers: int, vocab: int,
                  window: int = 1024, side_dim: int = 64) -> dict:
    """A Koronex config.json of a real model's sizes: groups of four layers (lightning attention, two
    windowed attention layers, a third that reads the second's keys), every layer with a feed-forward."""
    att = dict(heads=heads, kv_heads=kv_heads, dim=head_dim, vdim=head_dim, mask=dict(size=window),
               rot=dict(dims=head_dim // 2, base=10000.0), scale=head_dim ** -0.5)
    out = []
    for i in range(layers):
        mlp = dict(kind="dense", ff=ff)
        if i % 4 == 0:
            decay = [float(1.0 - 2.0 ** (-(3 + 5 * h / max(1, heads - 1)))) for h in range(heads)]
            out.append(dict(type="lightning", mixer=dict(heads=heads, dim=head_dim, vdim=head_dim, decay=decay), mlp=mlp))
        elif i % 4 == 3:
            out.append(dict(type="attention", mixer=dict(att, kv_from=i - 1), mlp=mlp))
        else:
            out.append(dict(type="attention", mixer=dict(att), mlp=mlp))
    return dict(architecture="Koronex", vocab=vocab, width=width, embedding=dict(scale=1.0), norm=dict(eps=1e-5),
                postln_alpha=1.0, token_side=dict(dim=side_dim), layers=out)


def dotivik_shape(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, layers: int, vocab: int,
                  window: int = 1024, kv_rank: int = 96, rot_dim: int = 32) -> dict:
    """A Dotivik config.json of a real model's sizes with ``layers`` layer RUNS: groups of three layers (latent
    attention, attention with two score maps per head, latent attention), of which the middle of the model
    runs twice, every layer with a feed-forward.  Latent layers have ``heads`` heads (head_dim unrotated and
    rot_dim rotated elements, values head_dim wide) over a cache row of kv_rank + rot_dim = 128 numbers; map
    layers have heads / 2 heads with two maps of head_dim / 2 each and values head_dim wide."""
    lat = dict(heads=heads, dim=head_dim, rot_dim=rot_dim, vdim=head_dim, kv_rank=kv_rank,
               scale=(head_dim + rot_dim) ** -0.5, mask=dict(size=window), rot=dict(dims=rot_dim, base=10000.0))
    att = dict(heads=heads // 2, kv_heads=max(1, kv_heads // 2), dim=head_dim // 2, vdim=head_dim,
               scale=(head_dim // 2) ** -0.5, softcap=50.0, diff=0.5, rot=dict(dims=head_dim // 2, base=10000.0))
    repeat = max(1, layers // 4)                       # layers of the run that goes twice
    stored = layers - repeat
    out = [dict(type="attention" if i % 3 == 1 else "latent_attention", mixer=dict(att if i % 3 == 1 else lat),
                mlp=dict(kind="dense", ff=ff)) for i in range(stored)]
    start = (stored - repeat) // 2
    return dict(architecture="Dotivik", vocab=vocab, width=width, norm=dict(eps=1e-5), layers=out,
                loop=dict(start=start, stop=start + repeat, times=2))


def tudasun_shape(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, layers: int, vocab: int,
                  kv_rank: int = 96, rot_dim: int = 32, side_dim: int = 64) -> dict:
    """A Tudasun config.json of a real model's sizes: groups of four layers (HGRN2, gated linear attention, latent
    attention, gated linear attention), the second latent layer of every pair reading the first one's rows.  The
    recurrent layers have ``heads`` heads with states of head_dim x head_dim; latent layers have ``heads`` heads
    (head_dim unrotated and rot_dim rotated elements, values head_dim wide) over a cache row of kv_rank + rot_dim =
    128 numbers.  The first layer's feed-forward is dense (PolyNorm, ``ff`` wide); the others are routed: 14 experts
    and 2 identity experts in 4 groups of which 2 are kept, 2 a token, each ff / 4 wide, beside a shared expert
    ff / 2 wide, so that a token's products are as many as in a gated feed-forward ``ff`` wide."""
    lat = dict(heads=heads, dim=head_dim, rot_dim=rot_dim, vdim=head_dim, kv_rank=kv_rank,
               scale=(head_dim + rot_dim) ** -0.5, rot=dict(dims=rot_dim, base=10000.0))
    rec = dict(heads=heads, dim=head_dim, vdim=head_dim)
    moe = dict(kind="moe", expert=dict(ff=ff // 4), shared=dict(ff=ff // 2),
               router=dict(experts=14, identity=2, top=2, groups=dict(count=4, keep=2)))
    out, owner = [], None
    for i in range(layers):
        mlp = dict(kind="dense", ff=ff) if i == 0 else moe
        if i % 4 == 0:
            out.append(dict(type="hgrn2", mixer=dict(rec), mlp=mlp))
        elif i % 4 == 2:
            mixer = dict(lat)
            if owner is not None:
                mixer["kv_from"], owner = owner, None
            else:
                owner = i
            out.append(dict(type="latent_attention", mixer=mixer, mlp=mlp))
        else:
            out.append(dict(type="gla", mixer=dict(rec, tau=8.0, decay_rank=16), mlp=mlp))
    return dict(architecture="Tudasun", vocab=vocab, width=width, norm=dict(eps=1e-6), logit_softcap=50.0,
                token_side=dict(dim=side_dim), layers=out)


def rizovik_shape(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, layers: int, vocab: int,
                  window: int = 1024, pool: int = 64, keep_first: int = 4) -> dict:
    """A Rizovik config.json of a real model's sizes: groups of three layers (the window with pooled blocks, the window
    with kept first positions and mixed heads, the gated delta rule with states of head_dim x head_dim), the last two
    layer runs using the tensors of the first layer of their kind.  Every layer has a routed
    feed-forward: 16 experts of which a token uses 4, each ff / 4 wide, so that a token's products are as many as in a
    gated feed-forward ``ff`` wide.  The layer that mixes heads applies every head's weights to the values of all its
    KV heads, which its kernel takes up to 512 numbers wide: it gets at most 512 / head_dim KV heads."""
    rot = dict(dims=head_dim // 2, base=10000.0)
    pooled = dict(heads=heads, kv_heads=kv_heads, dim=head_dim, vdim=head_dim, scale=head_dim ** -0.5,
                  mask=dict(size=window, pool=pool), rot=rot)
    kept = dict(heads=heads, kv_heads=min(kv_heads, max(1, 512 // head_dim)), dim=head_dim, vdim=head_dim,
                scale=head_dim ** -0.5, mask=dict(size=window, keep_first=keep_first),
                rot=dict(rot, scaling=dict(factor=8.0)))
    delta = dict(heads=heads, kv_heads=kv_heads, dim=head_dim, vdim=head_dim, conv=4)
    moe = dict(kind="moe", expert=dict(ff=ff // 4), router=dict(experts=16, top=4))
    kinds = [("attention", pooled), ("attention_2", kept), ("delta", delta)]
    out = []
    for i in range(layers):
        kind, mixer = kinds[i % 3]
        entry = dict(type=kind, mixer=dict(mixer), mlp=dict(moe))
        if layers > 3 and i >= layers - 2:
            entry["weights_of"] = i % 3                  # the first layer of its kind
        out.append(entry)
    return dict(architecture="Rizovik", vocab=vocab, width=width, norm=dict(eps=1e-6), residual_mult=0.5, layers=out)


def qwen2_shape(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, layers: int, vocab: int) -> dict:
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=vocab, hidden_size=width,
                intermediate_size=ff, num_hidden_layers=layers, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=head_dim, rms_norm_eps=1e-6, rope_theta=1e6,
                tie_word_embeddings=False, max_position_embeddings=32768)


class KernelTimes:
    """Times every launch made through kernels.api inside the block with CUDA events, by function name
    (eager steps only: a replayed graph makes no calls here)."""

    SKIP = {"stream_scope", "dtype_code", "stream_k_scratch", "gemm_tc_wait_limit", "KernelError",
            "attention_decode_supports", "attention_tma_supports", "gemm_tc_qkv_rope_supports",
            "attention_decode_max_clusters", "lightning_chunk_smem", "attention_mma_ext_supports",
            "lightning_chunked_tc_supports"}

    def __enter__(self):
        self.saved, self.events = {}, []
        for name, fn in list(vars(K).items()):
            if callable(fn) and not name.startswith("_") and name not in self.SKIP and getattr(fn, "__module__", "") == K.__name__:
                self.saved[name] = fn
                setattr(K, name, self._timed(name, fn))
        return self

    def _timed(self, name, fn):
        def call(*a, **kw):
            if getattr(self, "inside", False):         # a function that calls another: count the outer one
                return fn(*a, **kw)
            self.inside = True
            try:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                r = fn(*a, **kw)
                e.record()
            finally:
                self.inside = False
            shape = tuple(a[0].shape) if a and isinstance(a[0], torch.Tensor) else ()
            self.events.append((name, shape, s, e))
            return r
        return call

    def __exit__(self, *exc):
        for name, fn in self.saved.items():
            setattr(K, name, fn)
        torch.cuda.synchronize()
        self.by_name: dict[str, float] = {}
        self.calls: dict[str, int] = {}
        for name, shape, s, e in self.events:
            self.by_name[name] = self.by_name.get(name, 0.0) + s.elapsed_time(e) * 1e3
            self.calls[name] = self.calls.get(name, 0) + 1

    def table(self) -> dict:
        return {n: {"us": round(t, 1), "calls": self.calls[n]} for n, t in sorted(self.by_name.items(), key=lambda kv: -kv[1])}


def architecture_point(config: dict, *, prefill_tokens=2048, batch=8, context=4096, steps=32, warmup=4,
                       page_size=16, kernels=True) -> dict:
    """Prefill of one prompt and decode at one batch size for any registered architecture, device-timed
    through the step function; with ``kernels`` also one eager prefill step and one eager decode step
    timed launch by launch."""
    import gc

    from .cache.manager import CacheConfig, CacheManager
    from .engine.engine import load_model
    from .engine.step import ModelRunner, StepEntry

    model = load_model(config, device="cuda:0", dtype="bfloat16", random_seed=0)
    vocab = model.spec.vocab_size
    g = torch.Generator().manual_seed(5)
    out = {"weight_bytes": model.weight_bytes()}

    def runner_for(pages, requests, graphs=True):
        cache = CacheManager(model.cache_needs, CacheConfig(num_pages=pages, page_size=page_size, max_requests=requests,
                                                            dtype=model.rt.dtype))
        return ModelRunner(model, cache, use_graphs=graphs), cache

    # prefill
    runner, cache = runner_for(prefill_tokens // page_size + 8, 2)
    times = []
    for i in range(4):
        cache.open(i)
        toks = torch.randint(0, vocab, (prefill_tokens,), generator=g).tolist()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        runner.step([StepEntry(i, toks, [prefill_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        cache.close(i)
    out["prefill"] = {"tokens": prefill_tokens, "ms": min(times[1:]), "tokens_per_s": prefill_tokens / (min(times[1:]) / 1e3)}
    if kernels:
        cache.open("k")
        toks = torch.randint(0, vocab, (prefill_tokens,), generator=g).tolist()
        with KernelTimes() as kt:
            runner.step([StepEntry("k", toks, [prefill_tokens - 1])])
        out["prefill"]["kernels"] = kt.table()
        cache.close("k")
    runner.check_status()
    del runner, cache
    gc.collect()
    torch.cuda.empty_cache()
    # decode
    runner, cache = runner_for(batch * (context // page_size + 1), batch)
    for grp in cache.page_groups:
        grp.storage.normal_(0.0, 0.5)
    names = list(range(batch))
    start_ctx = context - steps - warmup - 2
    for n in names:
        cache.open(n)
        cache.ensure(n, start_ctx)
        cache.advance(n, start_ctx)

    def entries():
        toks = torch.randint(0, vocab, (batch,), generator=g).tolist()
        return [StepEntry(n, [t], [0]) for n, t in zip(names, toks)]
    for _ in range(warmup):
        runner.step(entries())
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler() as clocks:
        a.record()
        for _ in range(steps):
            runner.step(entries())
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    # bytes a decode step must read: the weights once, the keys and values that every layer's window
    # still sees, and every state (read and written)
    kv = 0
    sees = {}            # a mixer that keeps every page but reads a window (and block means, or kept first positions) only
    for block in model.blocks:
        mixer, need = block.mixer, block.cache_need()
        w = getattr(mixer, "window", None)
        if need is not None and w and getattr(need, "window", None) is None:
            far = max(0, context - w)
            pool, kept = getattr(mixer, "pool", 0), getattr(mixer, "keep_first", 0)
            sees[need] = min(context, w) + (far // pool if pool else 0) + min(kept, far)
    for grp in cache.page_groups:
        seen = sees.get(grp.need, context) if grp.window is None else min(context, grp.window)
        kv += grp.page_bytes() // page_size * seen * batch
    state = sum(2 * grp.storage[:, :batch].numel() * grp.storage.element_size() for grp in cache.state_groups)
    emb = model.embedding.weight
    nbytes = model.weight_bytes() - emb.numel() * emb.element_size() + kv + state
    if getattr(model.head, "tied", False):
        nbytes += emb.numel() * emb.element_size()            # the table is the head's weight: read whole
    runs: dict[int, int] = {}
    for e in model.spec.order:                                 # a layer that runs again reads its weights again
        runs[e.layer] = runs.get(e.layer, 0) + 1
    for i, n in runs.items():
        if n > 1:
            nbytes += (n - 1) * sum(p.nbytes() for p in model.blocks[i].parts().values())
    p = peaks()
    out["decode"] = {"batch": batch, "context": context, "ms_per_step": ms, "tokens_per_s": batch / (ms / 1e3),
                     "bytes": nbytes, "gbs": nbytes / (ms / 1e3) / 1e9, "hbm_frac": nbytes / (ms / 1e3) / 1e9 / p["hbm_gbs"],
                     "graph_steps": runner.stats["graph_steps"], "clocks": clocks.result}
    if kernels:
        runner.use_graphs = False
        with KernelTimes() as kt:
            runner.step(entries())
        out["decode"]["kernels"] = kt.table()
    runner.check_status()
    del runner, cache, model
    gc.collect()
    torch.cuda.empty_cache()
    return out


COMPARE_SIZES = {
    # name: width, heads, kv_heads, head_dim, ff, layers, vocab
    "2k": (2048, 16, 4, 128, 8192, 8, 32000),
    "4k": (4096, 32, 8, 128, 14336, 8, 32000),
}


DESIGN_SHAPES = {"koronex": koronex_shape, "dotivik": dotivik_shape, "tudasun": tudasun_shape, "rizovik": rizovik_shape,
                 "qwen2": qwen2_shape}
# the existing model that a design is set beside: Tudasun beside Koronex, the other design with a recurrent mixer over
# a float32 state, softmax attention with a sink, layers that read another layer's rows and a per-layer token input
# Rizovik beside Tudasun: routed feed-forwards, a recurrent mixer over a float32 state, attention over a cache that keeps
# every row
BESIDE = {"koronex": "qwen2", "dotivik": "qwen2", "tudasun": "koronex", "rizovik": "tudasun"}


def compare_architectures(sizes=("2k", "4k"), design: str = "koronex", beside: str | None = None, **kw) -> dict:
    """``design`` (Koronex, Dotivik or Tudasun) beside another model (``beside``; default: the Qwen2 dense model, for
    Tudasun Koronex) at equal width, heads, feed-forward width and count of layer runs."""
    beside = beside or BESIDE[design]
    out = {"peaks": peaks(), "beside": beside, "sizes": {}}
    for name in sizes:
        shape = COMPARE_SIZES[name]
        out["sizes"][name] = {
            "shape": dict(zip(("width", "heads", "kv_heads", "head_dim", "ff", "layers", "vocab"), shape)),
            design: architecture_point(DESIGN_SHAPES[design](*shape), **kw),
            beside: architecture_point(DESIGN_SHAPES[beside](*shape), **kw),
        }
    return out
