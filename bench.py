#!/usr/bin/env python3
"""Decode and prefill throughput of Qwen3-shaped models on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 4b|1.7b|8b] [--check]

The default run (``--config 4b``) is the headline: a step is one decode step of
a batch of 8 sequences at a context of 4,096 tokens.  Prints one JSON line:
``value`` = decoded tokens per second timed on the device over exactly K
graph-replayed steps; ``e2e`` = the same through ``Engine.generate`` with host
token lists in and out; ``prefill`` = one prompt of 2,048 tokens; ``roofline``
= bytes the decode step has to read (every weight once, the cache of the live
sequences) over its time, against the measured copy bandwidth; ``points`` =
decode at batch 1 and 64, at context 2,048, and averaged over the sweep from
2,048 to 4,096 positions.

``--config 1.7b``: 16 sequences with prompt lengths drawn uniformly from
[64, 2048] (seeded), 256 decode steps.  ``--config 8b``: an untied head, 32
prompts of 1,024 tokens, 512 decode steps, a cache of 8,192 tokens per
sequence.  ``--check`` decodes nothing for speed: it runs the same layer
sizes with 2 layers in bfloat16 and in true 32-bit and prints how far the
logits are apart.

``--impl reference`` drives the unmodified engine of IshaanBansal2006/starter
from ``baseline/_ref/engine`` (a plain copy of its ``engine/`` folder) through
its own ``Engine(model_path).generate(input_ids, max_new_tokens)``.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_COMMON = dict(architectures=["Qwen3ForCausalLM"], num_key_value_heads=8, head_dim=128, vocab_size=151936,
               rms_norm_eps=1e-6)
CONFIGS = {
    # name: (config.json, workload)
    "4b": (dict(_COMMON, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32,
                rope_theta=5000000.0, tie_word_embeddings=True),
           dict(model="Qwen3-4B shape", batch=8, context=4096, steps=256, prompts="decode ends at the context")),
    "1.7b": (dict(_COMMON, hidden_size=2048, intermediate_size=6144, num_hidden_layers=28, num_attention_heads=16,
                  rope_theta=1000000.0, tie_word_embeddings=True),
             dict(model="Qwen3-1.7B shape", batch=16, context=2048 + 256, steps=256, prompts="uniform[64,2048]")),
    "8b": (dict(_COMMON, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                rope_theta=1000000.0, tie_word_embeddings=False),
           dict(model="Qwen3-8B shape", batch=32, context=8192, steps=512, prompts="1024 each")),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PREFILL_TOKENS = 2048
LONG_PREFILL_TOKENS = 8192   # a second prefill point, where attention is a third of the work


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            peaks = {k: float(raw[k]) for k in FALLBACK_PEAKS if k in raw}
            if "hbm_gbs" in peaks and "bf16_tflops" in peaks:
                peaks.setdefault("bf16_tflops_sustained", peaks["bf16_tflops"])
                return peaks, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int = 0):
        self.proc = None
        self.lines = []
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, max_mhz, reasons = [], 0, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(int(float(parts[0])))
                max_mhz = max(max_mhz, int(float(parts[1])))
            except ValueError:
                continue
            for name, flag in zip(self.NAMES, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def model_numbers(raw, n_layers):
    """Parameters of one layer's matrices, bytes of the weights a decode step reads (the embedding
    table only where it is the output head as well), and cache bytes per token."""
    H, I, V = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    HQ, HKV, D = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    layer_params = (HQ + 2 * HKV) * D * H + H * HQ * D + 2 * I * H + H * I
    weight_bytes = 2 * (n_layers * (layer_params + 2 * H + 2 * D) + V * H + H)
    kv_bytes_per_token = n_layers * 2 * HKV * D * 2
    return layer_params, weight_bytes, kv_bytes_per_token


def prefill_flops(raw, n_layers, lengths):
    """Flops of a prefill of prompts of these lengths with logits at each prompt's last token."""
    layer_params, _, _ = model_numbers(raw, n_layers)
    D, HQ = raw["head_dim"], raw["num_attention_heads"]
    linear = 2.0 * sum(lengths) * layer_params * n_layers
    attention = sum(4.0 * D * HQ * (t * (t + 1) / 2.0) for t in lengths) * n_layers
    return linear + attention + 2.0 * len(lengths) * raw["vocab_size"] * raw["hidden_size"]


def prefill_point(points, name, raw, n_layers, lengths, ms, peaks):
    """A further prefill measurement as flat numbers: tokens a second under ``name``, its time under
    ``name_ms`` and its flops / time / the sustained bf16 peak under ``name_frac_of_sustained``."""
    points[name] = round(sum(lengths) * 1000.0 / ms, 1)
    points[name + "_ms"] = round(ms, 3)
    points[name + "_frac_of_sustained"] = round(
        prefill_flops(raw, n_layers, lengths) / (ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)


def prompt_lengths(workload, seed=4):
    import torch
    B = workload["batch"]
    if workload["prompts"] == "uniform[64,2048]":
        g = torch.Generator().manual_seed(seed)
        return torch.randint(64, 2049, (B,), generator=g).tolist()
    if workload["prompts"] == "1024 each":
        return [1024] * B
    return [workload["context"] - workload["steps"] - 1] * B


# ---- this library ---------------------------------------------------------------------------------

def time_decode(session, sampling, starts, steps, warmup, torch):
    """Device time per step of exactly ``steps`` decode steps of len(starts) sequences; sequence b
    holds starts[b] tokens when the warm-up begins.  Returns (ms per step, mean context while timed)."""
    from starter_b200.engine.graph import GraphDecoder
    cache = session.cache
    decoder = GraphDecoder(session, sampling)
    batch = len(starts)
    slots = [cache.alloc() for _ in range(batch)]
    try:
        for s, start in zip(slots, starts):
            cache.reserve(s, start + warmup + steps)
            cache.assume_length(s, start)
        bucket = decoder.bucket(batch)
        cache.flush()
        g = torch.Generator().manual_seed(0)
        tokens = torch.randint(0, session.vocab_size, (batch,), generator=g).tolist()
        bucket.load(slots, tokens, list(range(batch)), 0)
        for _ in range(warmup):
            bucket.graph.replay()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            bucket.graph.replay()
        t1.record()
        torch.cuda.synchronize()
        for s in slots:
            cache.advance_host(s, steps + warmup)
        session.stepper.raise_on_status()
        ms = t0.elapsed_time(t1) / steps
        return ms, sum(starts) / batch + warmup + steps / 2.0
    finally:
        for s in slots:
            cache.free(s)


def count_step_launches(session, sampling, batch, torch):
    """Kernels of this library in one decode step (counted on an eager pass over the null slot)."""
    from starter_b200.engine.graph import GraphDecoder
    b = GraphDecoder(session, sampling).new_bucket(batch)
    before = session.runtime.ops.launches
    b.body()
    torch.cuda.synchronize()
    return session.runtime.ops.launches - before


def time_prefill(session, lengths, repeats, torch):
    """Median device time of one step that runs prompts of these lengths, logits at each one's end."""
    from starter_b200.engine.step import StepEntry
    cache = session.cache
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, session.vocab_size, (n,), generator=g).tolist() for n in lengths]
    times = []
    for _ in range(repeats + 1):
        slots = [cache.alloc() for _ in prompts]
        try:
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            session.stepper.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
            t1.record()
            torch.cuda.synchronize()
            times.append(t0.elapsed_time(t1))
        finally:
            for s in slots:
                cache.free(s)
    times = sorted(times[1:])  # the first pass warms libraries up
    return times[len(times) // 2]


def time_e2e(engine, lengths, steps, torch):
    """Decoded tokens per second as a caller of Engine.generate sees them: host token lists in, host
    token lists out.  Returns (tokens/s from the first step's tokens to the last's, seconds from the
    call to the first step's tokens: upload of the prompts, their prefill, the first selection)."""
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, engine.session.vocab_size, (n,), generator=g).tolist() for n in lengths]
    for _ in engine.generate(prompts, 4):  # untimed, the same prompts: the library's first call at these shapes and
        pass                               # the capture of this batch size's decode graph (the reference arm does the same)
    torch.cuda.synchronize()
    t_call = time.perf_counter()
    it = engine.generate(prompts, steps + 1)
    next(it)
    t0 = time.perf_counter()
    n = 0
    for out in it:
        n += 1
    dt = time.perf_counter() - t0
    assert n == steps
    return len(lengths) * steps / dt, t0 - t_call


def run_ours(args, raw, workload) -> int:
    import torch
    from starter_b200.config import config_from_dict
    from starter_b200.engine.engine import Engine
    from starter_b200.engine.session import Session
    from starter_b200.sampling import SamplingParams
    from starter_b200.weights import RandomSource

    peaks, peak_source = load_peaks()
    raw = dict(raw)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_dict(raw)
    n_layers = cfg.num_hidden_layers
    layer_params, weight_bytes, kv_per_token = model_numbers(raw, n_layers)
    batch, context, steps, warmup = args.batch, args.context, args.steps, args.warmup
    torch.cuda.set_device(0)
    source = RandomSource(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    headline = args.config == "4b"
    max_batch = max(batch, 64 if headline and not args.skip_points else 1)
    lengths = prompt_lengths(dict(workload, batch=batch, context=context, steps=steps))
    long_prefill = LONG_PREFILL_TOKENS if headline and not args.skip_points else 0
    session = Session((cfg, source), dtype="bfloat16", max_tokens=max(max_batch * context, PREFILL_TOKENS, long_prefill),
                      max_seqs=max_batch, max_seq_tokens=max(context, PREFILL_TOKENS, long_prefill), device="cuda:0",
                      verbose=True)
    for group in session.cache.groups:  # a context of random keys and values stands in for real prompts
        group.k.normal_()
        group.v.normal_()
    sampling = SamplingParams()
    ops = session.runtime.ops

    # The step that is timed: the workload's own decode steps.  4b: the last `steps` positions before the
    # context's end; the others: the `steps` positions after the prompts.
    starts = [context - steps - warmup] * batch if headline else [n - warmup for n in lengths]
    with ClockSampler() as clocks:
        ms_step, mean_ctx = time_decode(session, sampling, starts, steps, warmup, torch)
    clock_summary = clocks.summary()
    per_step_launches = count_step_launches(session, sampling, batch, torch)
    value = batch * 1000.0 / ms_step
    step_bytes = weight_bytes + batch * mean_ctx * kv_per_token
    achieved_gbs = step_bytes / (ms_step * 1e-3) / 1e9

    def rate(b, ms):
        return round(b * 1000.0 / ms, 1)

    points = {}
    if not args.skip_points:
        if headline:
            for b in (1, 64):
                ms, _ = time_decode(session, sampling, [context - steps - warmup] * b, steps, warmup, torch)
                points[f"decode_b{b}"] = rate(b, ms)
            half = context // 2
            for b in (1, batch, 64):
                ms, _ = time_decode(session, sampling, [half - steps // 2 - warmup] * b, steps, warmup, torch)
                points[f"decode_b{b}_ctx{half}"] = rate(b, ms)
                ms, _ = time_decode(session, sampling, [half - warmup] * b, context - half, warmup, torch)
                points[f"decode_b{b}_sweep_{half}_{context}"] = rate(b, ms)
        else:
            ms, ctx = time_decode(session, sampling, [context - steps - warmup] * batch, steps, warmup, torch)
            points[f"decode_b{batch}_ctx{context}"] = rate(batch, ms)
            points[f"decode_b{batch}_ctx{context}_hbm_frac"] = round(
                (weight_bytes + batch * ctx * kv_per_token) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)

    prefill_ms = time_prefill(session, [PREFILL_TOKENS], repeats=3, torch=torch)
    prefill_frac = prefill_flops(raw, n_layers, [PREFILL_TOKENS]) / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)
    prefill = {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4)}
    if long_prefill:
        ms = time_prefill(session, [long_prefill], repeats=2, torch=torch)
        prefill_point(points, f"prefill_{long_prefill}", raw, n_layers, [long_prefill], ms, peaks)
    if not headline:  # the workload's own prompts, all in one step
        ms = time_prefill(session, lengths, repeats=2, torch=torch)
        prefill_point(points, "prefill_workload", raw, n_layers, lengths, ms, peaks)
        points["prefill_workload_tokens"] = sum(lengths)

    e2e = None
    if not args.skip_e2e:
        engine = Engine.from_session(session)
        e2e_value, first_s = time_e2e(engine, lengths, steps, torch)
        # Timed from the first step's tokens to the last's: inside that region a step's input (the token
        # chosen one step before) is already on the device, so nothing goes up; its tokens come down.
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
               "d2h_bytes_per_step": 4 * batch, "first_tokens_s": round(first_s, 4),
               "prompt_upload_bytes": 4 * (sum(lengths) + 4 * batch),
               "region": "decode steps; prompt upload and prefill are in first_tokens_s"}

    line = {
        "metric": f"decode tok/s at batch {batch}, context {round(mean_ctx + steps / 2.0)} ({workload['model']}, bf16, "
                  "random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0, N(0,0.02)), random token ids, random cache contents",
        "impl": "ours",
        "config": {"model": workload["model"], "layers": n_layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied": cfg.tie_word_embeddings, "global_batch": batch, "seq_len": context,
                   "prompts": workload["prompts"], "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": "each step reads all weights (larger than L2)", "peaks": peak_source,
                   "decode_weight_copy_gb": round(getattr(ops, "_tiled_bytes", 0) / 1e9, 2)},
        "e2e": e2e, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
        "gpu_launches": per_step_launches * steps,
    }
    print(json.dumps(line))
    return 0


def run_check(args, raw, workload) -> int:
    """The 32-bit check path at the benchmark's layer sizes: 2 layers, the shape rules as they are."""
    import torch
    from starter_b200.config import config_from_dict
    from starter_b200.engine.check import compare_dtypes
    cfg = config_from_dict(dict(raw, num_hidden_layers=args.layers or 2))
    report = compare_dtypes(cfg, seed=0, prompt_lengths=(300, 2048), decode_batches=(1, 8, 64), decode_steps=6,
                            device="cuda:0", verbose=True)
    report.update(impl="ours", check="bfloat16 engine against the float32 engine, same weights",
                  config={"model": workload["model"], "layers": cfg.num_hidden_layers,
                          "layers_of_model": raw["num_hidden_layers"]})
    print(json.dumps(report))
    return 0 if report["within_tolerance"] else 1


# ---- the reference --------------------------------------------------------------------------------

# ---- another model family beside the Qwen3 shape of equal size --------------------------------------

def _kudazen_raw(width, ff, layers, latent, wkv, attention, vocab=32000):
    """A Kudazen configuration of ``layers`` layers that cycle through the three mixers."""
    kinds = [
        {"type": "latent_attention", "mixer": dict(latent, scale=(latent["dim"] + latent["rot_dim"]) ** -0.5,
                                                   rot={"base": 10000.0, "dims": latent["rot_dim"]})},
        {"type": "wkv", "mixer": dict(wkv)},
        {"type": "attention", "mixer": dict(attention, scale=attention["dim"] ** -0.5)},
    ]
    entries = [dict(kinds[i % 3], mlp={"kind": "dense", "ff": ff, "limit": 7.0}) for i in range(layers)]
    return {"architecture": "Kudazen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5, "groups": 2}, "layers": entries}


FAMILY_SIZES = {
    # name: (Kudazen configuration, the Qwen3 configuration of the same width, feed-forward, layers and vocabulary)
    "1024": (_kudazen_raw(1024, 4096, 6, dict(heads=8, dim=64, rot_dim=32, vdim=64, q_rank=384, kv_rank=256),
                          dict(heads=16, dim=64, decay_rank=64), dict(heads=16, kv_heads=4, dim=64, vdim=64, mask={"size": 1024})),
             dict(architectures=["Qwen3ForCausalLM"], hidden_size=1024, intermediate_size=4096, num_hidden_layers=6,
                  num_attention_heads=16, num_key_value_heads=4, head_dim=64, vocab_size=32000, rms_norm_eps=1e-6,
                  rope_theta=1000000.0, tie_word_embeddings=True)),
    "2048": (_kudazen_raw(2048, 8192, 6, dict(heads=16, dim=128, rot_dim=64, vdim=128, q_rank=768, kv_rank=512),
                          dict(heads=32, dim=64, decay_rank=64), dict(heads=16, kv_heads=8, dim=128, vdim=128, mask={"size": 2048})),
             dict(architectures=["Qwen3ForCausalLM"], hidden_size=2048, intermediate_size=8192, num_hidden_layers=6,
                  num_attention_heads=16, num_key_value_heads=8, head_dim=128, vocab_size=32000, rms_norm_eps=1e-6,
                  rope_theta=1000000.0, tie_word_embeddings=True)),
}


def _nazulorn_raw(width, layers, gla, attention, experts, expert_ff, top, identity, shared_ff, vocab=32000, streams=2):
    """A Nazulorn configuration of ``layers`` layers that cycle through gla, attention, attention."""
    kinds = [
        {"type": "gla", "mixer": dict(gla, tau=8.0)},
        {"type": "attention", "mixer": dict(attention, scale=attention["dim"] ** -0.5, diff=0.5,
                                            rot={"base": 500000.0, "dims": attention["dim"],
                                                 "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}})},
    ]
    mlp = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top, "scale": 2.0},
           "expert": {"ff": expert_ff, "limit": 7.0}, "shared": {"ff": shared_ff, "limit": 7.0}}
    entries = [dict(kinds[min(i % 3, 1)], mlp=mlp) for i in range(layers)]
    return {"architecture": "Nazulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "residual_mult": 0.5, "streams": streams, "logit_scale": 1.0, "layers": entries}


# Nazulorn beside Kudazen (the closest design the library has: a recurrence with a matrix state, attention with a bounded
# reach, the clamped activation, a 32-bit residual) at the same width, layers, vocabulary and feed-forward work per token:
# four chosen experts and the shared expert together are as wide as Kudazen's dense feed-forward; the two maps of a head
# give the attention kernels Kudazen's number of query and key heads.
NAZULORN_SIZES = {
    "1024": (_nazulorn_raw(1024, 6, dict(heads=8, dim=64, vdim=128, decay_rank=64),
                           dict(heads=8, kv_heads=2, dim=64, vdim=64, mask={"size": 1024}), experts=16, expert_ff=512, top=4,
                           identity=2, shared_ff=2048), FAMILY_SIZES["1024"][0]),
    "2048": (_nazulorn_raw(2048, 6, dict(heads=16, dim=64, vdim=128, decay_rank=64),
                           dict(heads=8, kv_heads=4, dim=128, vdim=128, mask={"size": 2048}), experts=32, expert_ff=1024, top=4,
                           identity=2, shared_ff=4096), FAMILY_SIZES["2048"][0]),
}


def _gulazen_raw(width, layers, attention, ff, experts, expert_ff, top, shared_ff, vocab=32000, taps=4):
    """A Gulazen configuration of ``layers`` layers whose feed-forward alternates between dense and experts."""
    mixer = dict(attention, scale=attention["dim"] ** -0.5, softcap=30.0)
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff}}
    entries = [{"type": "attention", "mixer": mixer, "mlp": moe if i % 2 else dense} for i in range(layers)]
    return {"architecture": "Gulazen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "canon": {"taps": taps}, "layers": entries}


# Gulazen beside Nazulorn (the closest design the library has: attention with a bounded reach and a sink-like extra term in
# the softmax over pages of a ring, experts with a shared expert, a 32-bit residual that the branches change in place) at
# the same width, layers, vocabulary, window and expert sizes; Gulazen's attention has Nazulorn's number of score maps (its
# query heads; Nazulorn's heads carry two maps each) and key/value heads.
GULAZEN_SIZES = {
    "1024": (_gulazen_raw(1024, 6, dict(heads=16, kv_heads=4, dim=64, vdim=64, mask={"size": 1024, "keep_first": 4}), ff=4096,
                          experts=16, expert_ff=512, top=4, shared_ff=2048), NAZULORN_SIZES["1024"][0]),
    "2048": (_gulazen_raw(2048, 6, dict(heads=16, kv_heads=8, dim=128, vdim=128, mask={"size": 2048, "keep_first": 4}), ff=8192,
                          experts=32, expert_ff=1024, top=4, shared_ff=4096), NAZULORN_SIZES["2048"][0]),
}
def _paditar_raw(width, attention, left, right, ff, vocab=32000):
    """A Paditar configuration of four layers (side by side, two maps, side by side, two maps) whose first two run twice:
    six layer runs."""
    two_maps = {"type": "attention", "mixer": dict(attention, scale=attention["dim"] ** -0.5, diff=0.5,
                                                   rot={"base": 500000.0, "dims": attention["dim"] // 2})}
    pair = {"type": "parallel", "mixer": {"left": dict(left, vdim=left["dim"], scale=left["dim"] ** -0.5, conv=4,
                                                       q_temp={"coef": 0.2, "every": 64}),
                                          "right": dict(right, gate_cap=15.0), "left_scale": 1.0, "right_scale": 0.6}}
    mlp = {"kind": "dense", "ff": ff}
    entries = [dict(kind, mlp=mlp) for kind in (pair, two_maps, pair, two_maps)]
    return {"architecture": "Paditar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": entries}


# Paditar beside Nazulorn (the closest design the library has: attention with two score maps per head, a recurrence with
# a matrix state per head, a 32-bit residual) at the same width, layer runs, vocabulary and feed-forward work per token:
# the dense feed-forward is as wide as Nazulorn's four chosen experts and its shared expert together; the two-map
# attention and the matrix memory have the head counts and sizes of Nazulorn's attention and gated linear attention.
PADITAR_SIZES = {
    "1024": (_paditar_raw(1024, dict(heads=8, kv_heads=2, dim=64, vdim=64), dict(heads=8, kv_heads=2, dim=64),
                          dict(heads=8, dim=64, vdim=128), ff=4096), NAZULORN_SIZES["1024"][0]),
    "2048": (_paditar_raw(2048, dict(heads=8, kv_heads=4, dim=128, vdim=128), dict(heads=8, kv_heads=4, dim=128),
                          dict(heads=16, dim=64, vdim=128), ff=8192), NAZULORN_SIZES["2048"][0]),
}
FAMILIES = {"kudazen": (FAMILY_SIZES, "qwen3", "Qwen3ForCausalLM"), "nazulorn": (NAZULORN_SIZES, "kudazen", "Kudazen"),
            "gulazen": (GULAZEN_SIZES, "nazulorn", "Nazulorn"), "paditar": (PADITAR_SIZES, "nazulorn", "Nazulorn")}


class TimedOps:
    """The kernel call table with a pair of CUDA events around every call: per call name, the device time and what
    the call must move or compute at least, from its arguments (the bound is the slower of the two)."""

    def __init__(self, ops, torch, peaks):
        self._ops, self._torch, self._peaks = ops, torch, peaks
        self.records = []      # (name, start event, end event, bytes, flops)
        self.ctx_tokens = 0    # tokens every sequence of the step holds (set by the caller: sizes the attention's work)

    @staticmethod
    def _nbytes(values):
        total = 0
        for v in values:
            if hasattr(v, "element_size") and hasattr(v, "numel"):
                total += v.numel() * v.element_size()
            elif isinstance(v, (tuple, list)):
                total += TimedOps._nbytes(v)
        return total

    def _cost(self, name, args, kwargs, out):
        nbytes = self._nbytes(args) + self._nbytes(kwargs.values()) + self._nbytes([out])
        flops = 0.0
        if name in ("linear", "linear_swiglu", "linear_xielu", "linear_relu2", "linear_bias"):
            a, w = args[0], args[1]
            flops = 2.0 * a.shape[0] * w.shape[0] * w.shape[1]
        elif name == "linear_heads":
            a, w = args[0], args[1]
            flops = 2.0 * a.shape[0] * w.shape[0] * w.shape[1] * w.shape[2]
            nbytes = w.numel() * 2 + 2 * a.shape[0] * w.shape[0] * (w.shape[1] + w.shape[2])
        elif name in ("flex_attention", "attention", "qk_attention", "talking_attention"):
            ctx, q, cache = args[0], args[1], args[2]
            req, group = cache.group.request, cache.group
            v_dim = group.v_dim if group.v_dim else kwargs.get("v_dim", req.head_dim)
            heads = q.shape[1] if name in ("flex_attention", "talking_attention") else args[3]
            reach = self.ctx_tokens
            for r in (kwargs.get("chunk"), kwargs.get("window"), req.window):
                if r:
                    reach = min(reach, r)
            token_bytes = (req.num_kv_heads * req.head_dim + getattr(group, "v_heads", req.num_kv_heads) * (group.v_dim or 0)) * 2
            if ctx.max_q_len == 1:
                pairs = float(ctx.n_rows) * reach
                cache_bytes = ctx.n_seqs * reach * token_bytes
            else:
                t = ctx.n_rows / ctx.n_seqs
                if reach >= t:
                    pairs = ctx.n_seqs * t * (t + 1) / 2.0
                elif kwargs.get("chunk") and reach == kwargs.get("chunk"):
                    pairs = ctx.n_seqs * t * reach / 2.0                                  # blocks of `chunk` positions, each causal inside
                else:
                    pairs = ctx.n_seqs * (reach * (reach + 1) / 2.0 + (t - reach) * reach)   # a sliding window: full reach from position `reach` on
                cache_bytes = ctx.n_rows * token_bytes
            flops = 2.0 * pairs * heads * (req.head_dim + v_dim)
            nbytes = cache_bytes + 2 * self._nbytes([q]) if name != "qk_attention" else cache_bytes + self._nbytes([q])
        elif name == "wkv_scan":
            r, state, heads, dim = args[1], args[11], args[12], args[13]
            flops = 6.0 * r.shape[0] * heads * dim * dim
            nbytes = 2 * args[0].n_seqs * heads * dim * dim * 4 + 6 * r.numel() * 2
        elif name == "gla_scan":
            q, heads, dim, vdim = args[1], args[12], args[13], args[14]
            flops = 6.0 * q.shape[0] * heads * dim * vdim
            nbytes = 2 * args[0].n_seqs * heads * dim * vdim * 4 + q.shape[0] * heads * (2 * dim * 2 + 3 * vdim * 2 + dim * 4)
        elif name == "mlstm_scan":
            q, heads, dim, vdim = args[1], args[15], args[16], args[17]
            flops = 6.0 * q.shape[0] * heads * dim * (vdim + 1)
            nbytes = (2 * args[0].n_seqs * heads * (dim * vdim + dim + 1) * 4 + q.shape[0] * heads * (2 * dim * 2 + 3 * vdim * 2)
                      + q.shape[0] * heads * 8)
        elif name == "conv_qk_store":
            q, k = args[1], args[2]
            nbytes = (2 * q.numel() + 3 * k.numel()) * q.element_size()     # queries in and out, keys in, normed keys and values out
        elif name == "moe_experts":
            h, chosen, w_gu, w_down = args[0], args[1], args[3], args[4]
            pairs = chosen.numel()
            per_expert = (w_gu[0].numel() + w_down[0].numel()) if w_gu is not None else 0
            flops = 2.0 * pairs * per_expert      # an upper bound: pairs of identity outputs do no product
            touched = min(pairs, w_gu.shape[0]) if w_gu is not None else 0
            nbytes = touched * per_expert * 2 + 3 * h.numel() * 2 + pairs * 8
        elif name == "moe_route":
            h, router = args[0], args[1]
            flops = 0.0    # 32-bit dot products on the CUDA cores: bounded by the rows it reads
            nbytes = h.numel() * 2 + router.numel() * 4 + h.shape[0] * args[3] * 8
        elif name == "stream_norm":
            x, pending = args[0], args[2]
            nbytes = x.numel() * 4 * (2 if pending is not None else 1) + (x.numel() // args[1]) * 2 * (2 if pending is not None else 1)
        return nbytes, flops

    def __getattr__(self, name):
        attr = getattr(self._ops, name)
        if not callable(attr) or name in ("prepare_matrix", "folds", "sm_count", "status_into", "set_dependent_launch",
                                          "read_kernel_status", "kernel_status", "uneven_matters"):
            return attr

        def timed(*args, **kwargs):
            t0 = self._torch.cuda.Event(enable_timing=True)
            t1 = self._torch.cuda.Event(enable_timing=True)
            t0.record()
            out = attr(*args, **kwargs)
            t1.record()
            if out is not None or name not in ("qk_attention",):
                label = name
                if name == "flex_attention":   # the two users of this call apart: values inside the key rows (latent) or pages of their own
                    req = args[2].group.request
                    label += ("[latent]" if kwargs.get("values_in_keys") else
                              "[keys as values]" if kwargs.get("sink") is not None and req.v_dim == req.head_dim and args[2].aux is not None else
                              "[latent, narrow form]" if kwargs.get("sink") is not None else
                              "[two maps]" if args[2].group.v_heads != args[2].group.request.num_kv_heads else "[chunked]")
                self.records.append((label, t0, t1) + self._cost(name, args, kwargs, out))
            return out
        return timed

    def table(self):
        """{call name: {calls, us (all calls of one pass), bound_us, frac_of_bound}}, of the records since the last clear."""
        self._torch.cuda.synchronize()
        hbm, tflops = self._peaks["hbm_gbs"] * 1e9, self._peaks["bf16_tflops"] * 1e12
        rows = {}
        for name, t0, t1, nbytes, flops in self.records:
            row = rows.setdefault(name, {"calls": 0, "us": 0.0, "bound_us": 0.0})
            row["calls"] += 1
            row["us"] += t0.elapsed_time(t1) * 1e3
            row["bound_us"] += max(nbytes / hbm, flops / tflops) * 1e6
        for row in rows.values():
            row["frac_of_bound"] = round(row["bound_us"] / row["us"], 4) if row["us"] else None
            row["us"], row["bound_us"] = round(row["us"], 1), round(row["bound_us"], 2)
        return rows


def _family_arm(torch, raw, peaks, prefill_tokens, batch, context, steps, warmup):
    """Prefill and decode throughput of one configuration with random weights, and its kernels' times by call name
    (one eager prefill pass and one eager decode step with events around every call)."""
    from starter_b200.config import config_from_dict
    from starter_b200.engine.session import Session
    from starter_b200.engine.step import StepEntry
    from starter_b200.sampling import SamplingParams
    from starter_b200.weights import RandomSource
    cfg = config_from_dict(raw)
    source = RandomSource(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    session = Session((cfg, source), dtype="bfloat16", max_tokens=max(batch * context, prefill_tokens) + 64 * batch, max_seqs=batch,
                      max_seq_tokens=max(context, prefill_tokens), max_step_tokens=prefill_tokens, max_rows=max(prefill_tokens, 8192),
                      device="cuda:0", verbose=False)
    for group in session.cache.groups:     # a context of random keys, values and states stands in for real prompts
        for name in ("k", "v", "data"):
            t = getattr(group, name, None)
            if t is not None:
                t.normal_(0.0, 0.5)
    out = {}
    ms = time_prefill(session, [prefill_tokens], 5, torch)
    out["prefill_tok_s"], out["prefill_ms"] = round(prefill_tokens * 1000.0 / ms, 1), round(ms, 3)
    ms, _ = time_decode(session, SamplingParams(), [context - steps - warmup] * batch, steps, warmup, torch)
    out["decode_tok_s"], out["decode_ms_per_step"] = round(batch * 1000.0 / ms, 1), round(ms, 4)
    out["decode_launches"] = count_step_launches(session, SamplingParams(), batch, torch)
    # per call name: swap the call table of the runtime (every part reads it there) for the timed one
    timed = TimedOps(session.runtime.ops, torch, peaks)
    parts = [p for p in session.model.parts()] + [getattr(p, "position", None) for p in session.model.parts()]
    holders = [session.runtime] + [p for p in parts if p is not None and hasattr(p, "ops")]
    saved = [h.ops for h in holders]
    for h in holders:
        h.ops = timed
    try:
        g = torch.Generator().manual_seed(3)
        cache = session.cache
        for label, n_seqs, rows, held in (("prefill", 1, prefill_tokens, 0), ("decode", batch, 1, context - 1)):
            best = None
            for _ in range(3):
                slots = [cache.alloc() for _ in range(n_seqs)]
                try:
                    for sl in slots:
                        cache.assume_length(sl, held)
                    cache.flush()
                    timed.records, timed.ctx_tokens = [], held + rows
                    session.stepper.step([StepEntry(sl, torch.randint(0, session.vocab_size, (rows,), generator=g).tolist(), [rows - 1])
                                          for sl in slots])
                    table = timed.table()
                finally:
                    for sl in slots:
                        cache.free(sl)
                if best is None or sum(r["us"] for r in table.values()) < sum(r["us"] for r in best.values()):
                    best = table
            out[label + "_calls"] = best
    finally:
        for h, ops in zip(holders, saved):
            h.ops = ops
    return out


def run_family(args) -> int:
    """--family kudazen | nazulorn | gulazen | paditar: the design at a few sizes that resemble a real model's layers (random weights),
    beside the library's closest model of the same width, feed-forward work per token, layer count and vocabulary (Kudazen
    beside the Qwen3 decoder, Nazulorn beside Kudazen, Gulazen and Paditar beside Nazulorn).  One JSON line."""
    import torch
    peaks, peak_source = load_peaks()
    torch.cuda.set_device(0)
    table, beside_name, beside_arch = FAMILIES[args.family]
    sizes = [s for s in (args.sizes.split(",") if args.sizes else sorted(table)) if s]
    result = {"family": args.family, "beside": beside_arch, "dtype": "bf16", "data": "synthetic, random weights",
              "prefill_tokens": PREFILL_TOKENS, "decode_batch": args.batch, "decode_context": args.context, "steps": args.steps,
              "warmup": args.warmup, "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops")}, "peaks_from": peak_source,
              "timing": "CUDA events; decode through the captured graph; *_calls: one eager pass with events around every call "
                        "(a call's time includes its launch), bound = max(bytes / copy bandwidth, flops / bf16 burst)",
              "sizes": {}}
    with ClockSampler() as clocks:
        for name in sizes:
            if name not in table:
                print(f"unknown size {name!r}; known: {', '.join(sorted(table))}", file=sys.stderr)
                return 1
            ours, beside = table[name]
            result["sizes"][name] = {
                args.family: _family_arm(torch, ours, peaks, PREFILL_TOKENS, args.batch, args.context, args.steps, args.warmup),
                beside_name: _family_arm(torch, beside, peaks, PREFILL_TOKENS, args.batch, args.context, args.steps, args.warmup)}
    result["clocks"] = clocks.summary()
    print(json.dumps(result))
    return 0


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def run_reference(args, raw, workload) -> int:
    """Drive the reference's own Engine from baseline/_ref/engine, unmodified.

    Its switches (engine/engine.py:437-454): ENGINE_RECYCLE=0 turns its speculative decoding off (not
    part of this comparison: both arms decode one token per sequence per step), ENGINE_SELF_CHECK=0
    skips its comparison with the Transformers library.  Every other switch keeps its default, so its
    start-up pickers choose its kernels by timing, as in a stock run.
    """
    ref_engine = os.path.join(ROOT, "baseline", "_ref", "engine")
    if not os.path.isfile(os.path.join(ref_engine, "engine.py")):
        return _unavailable("baseline/_ref/engine/engine.py is absent: copy the reference's engine/ folder there")
    if workload["prompts"] == "uniform[64,2048]":
        return _unavailable("the reference rejects prompts of unequal length (engine/engine.py:584-585: "
                            "'all prompts in a batch must have the same length'), which this workload is made of")
    os.environ.setdefault("ENGINE_RECYCLE", "0")
    os.environ.setdefault("ENGINE_SELF_CHECK", "0")
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device: the reference's kernels need one")
        from starter_b200.config import config_from_dict
        from starter_b200.weights import write_model_folder
    except Exception as exc:  # noqa: BLE001
        return _unavailable(f"set-up failed: {exc!r}")

    peaks, peak_source = load_peaks()
    raw = dict(raw)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    n_layers = raw["num_hidden_layers"]
    _, weight_bytes, kv_per_token = model_numbers(raw, n_layers)
    batch, context, steps, warmup = args.batch, args.context, args.steps, args.warmup
    headline = args.config == "4b"
    lengths = prompt_lengths(dict(workload, batch=batch, context=context, steps=steps))
    T = lengths[0]
    folder = tempfile.mkdtemp(prefix="starter_ref_model_")
    try:
        # Data only: the same kind of folder the reference is given in a stock run, with seeded random weights.
        write_model_folder(config_from_dict(raw), 0, folder, device="cuda:0")
        torch.cuda.empty_cache()
        sys.path.insert(0, ref_engine)
        try:
            from engine import Engine  # the reference's engine/engine.py
        except Exception as exc:  # noqa: BLE001
            return _unavailable(f"importing the reference's engine failed: {exc!r}")

        def fresh_engine():
            # A new engine per measurement: its pickers share one 60 s budget that starts with the object.
            gc.collect()
            torch.cuda.empty_cache()
            eng = Engine(folder)
            if eng.fallback is not None or eng.model is None:
                raise RuntimeError("the reference fell back to its Transformers baseline (its model did not load)")
            return eng

        def generate_timed(eng, B, T, n_new, seed):
            """(tokens/s between the first and the last yield, seconds to the first yield) of one call."""
            g = torch.Generator().manual_seed(seed)
            ids = torch.randint(0, raw["vocab_size"], (B, T), generator=g).tolist()
            for _ in eng.generate(ids, n_new):  # untimed: builds the plan, runs the pickers, captures the graphs
                pass
            if eng.fallback is not None:
                raise RuntimeError("the reference fell back to its Transformers baseline during generate")
            torch.cuda.synchronize()
            t_call = time.perf_counter()
            it = eng.generate(ids, n_new)
            next(it)
            t0 = time.perf_counter()
            n = sum(1 for _ in it)
            dt = time.perf_counter() - t0
            assert n == n_new - 1
            return B * n / dt, t0 - t_call

        def replay_decode(eng, key, start, n_steps):
            """Device time per step of its captured decode graph, the sequences set to ``start`` tokens."""
            plan = eng.plans[key]
            if plan.g_decode is None:
                raise RuntimeError("the reference did not capture its decode graph")
            if start + warmup + n_steps > plan.plan.cap:
                raise RuntimeError(f"its plan holds {plan.plan.cap} tokens per sequence")
            plan.plan.pos.fill_(start)
            for _ in range(warmup):
                plan._step_decode()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(n_steps):
                plan._step_decode()
            t1.record()
            torch.cuda.synchronize()
            return t0.elapsed_time(t1) / n_steps

        try:
            eng = fresh_engine()
            with ClockSampler() as clocks:
                e2e_value, first_s = generate_timed(eng, batch, T, steps + 1, seed=2)
                start = (context - steps - warmup) if headline else T - warmup
                ms_step = replay_decode(eng, (batch, T), start, steps)
            clock_summary = clocks.summary()
            mean_ctx = start + warmup + steps / 2.0
            points = {}
            if not headline:
                points["prefill_workload"] = {"tokens": batch * T, "first_tokens_s": round(first_s, 4)}
            if headline and not args.skip_points:
                for b in (1, 64):
                    del eng
                    eng = fresh_engine()
                    # a short prompt, a plan that holds the whole context; positions are then set on its plan
                    short, n_new = 64, context - 64
                    g = torch.Generator().manual_seed(3)
                    ids = torch.randint(0, raw["vocab_size"], (b, short), generator=g).tolist()
                    it = eng.generate(ids, n_new)
                    for _ in range(4):
                        next(it)
                    it.close()
                    torch.cuda.synchronize()
                    ms = replay_decode(eng, (b, short), context - steps - warmup, steps)
                    points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
                    half = context // 2   # the same plan at half the context, as this library's arm measures it
                    ms = replay_decode(eng, (b, short), half - steps // 2 - warmup, steps)
                    points[f"decode_b{b}_ctx{half}"] = round(b * 1000.0 / ms, 1)
            del eng

            def prefill_ms_of(n_tokens, repeats):
                eng = fresh_engine()
                g = torch.Generator().manual_seed(1)
                ids = torch.randint(0, raw["vocab_size"], (1, n_tokens), generator=g).tolist()
                list(eng.generate(ids, 1))
                plan = eng.plans[(1, n_tokens)]
                times = []
                for _ in range(repeats + 1):
                    torch.cuda.synchronize()
                    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    t0.record()
                    plan._step_prefill()
                    t1.record()
                    torch.cuda.synchronize()
                    times.append(t0.elapsed_time(t1))
                times = sorted(times[1:])
                return times[len(times) // 2]

            prefill_ms = prefill_ms_of(PREFILL_TOKENS, 3)
            if headline and not args.skip_points:
                ms = prefill_ms_of(LONG_PREFILL_TOKENS, 2)
                prefill_point(points, f"prefill_{LONG_PREFILL_TOKENS}", raw, n_layers, [LONG_PREFILL_TOKENS], ms, peaks)
        except Exception as exc:  # noqa: BLE001
            return _unavailable(f"the reference's engine failed on this box: {exc!r}")
    finally:
        shutil.rmtree(folder, ignore_errors=True)

    step_bytes = weight_bytes + batch * mean_ctx * kv_per_token
    achieved_gbs = step_bytes / (ms_step * 1e-3) / 1e9
    prefill_frac = prefill_flops(raw, n_layers, [PREFILL_TOKENS]) / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)
    line = {
        "metric": f"decode tok/s at batch {batch}, context {round(mean_ctx + steps / 2.0)} ({workload['model']}, bf16, "
                  "random weights)",
        "value": round(batch * 1000.0 / ms_step, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0, N(0,0.02)), random token ids",
        "impl": "reference",
        "config": {"model": workload["model"], "layers": n_layers, "layers_of_model": full_layers,
                   "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
                   "tied": raw["tie_word_embeddings"], "global_batch": batch, "seq_len": context,
                   "prompts": workload["prompts"], "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": "each step reads all weights (larger than L2)", "peaks": peak_source,
                   "switches": f"ENGINE_RECYCLE={os.environ['ENGINE_RECYCLE']} ENGINE_SELF_CHECK={os.environ['ENGINE_SELF_CHECK']}",
                   "value_is": "its captured decode graph replayed with plan.pos set; e2e is Engine.generate alone"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 8 * batch, "first_tokens_s": round(first_s, 4),
                "region": "decode steps; prompt upload and prefill are in first_tokens_s"},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps that are timed (default: the workload's)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="4b", choices=sorted(CONFIGS))
    ap.add_argument("--check", action="store_true", help="compare bfloat16 with 32-bit logits at these layer sizes")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--context", type=int, default=0)
    ap.add_argument("--skip-points", action="store_true", help="leave out the further decode points")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--family", default="", choices=["", "kudazen", "nazulorn", "gulazen", "paditar"],
                    help="instead of the default workload: this model family at a few layer sizes, beside the library's closest "
                         "model of equal size (kudazen beside the Qwen3 shape, nazulorn beside kudazen, gulazen and paditar beside "
                         "nazulorn)")
    ap.add_argument("--sizes", default="", help="with --family: sizes to run, with commas between them (default: all)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library does not run on {args.gpus} GPUs")
        return 2
    raw, workload = CONFIGS[args.config]
    args.batch = args.batch or workload["batch"]
    args.context = args.context or workload["context"]
    args.steps = args.steps or workload["steps"]
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args, raw, workload)
    import torch
    if not torch.cuda.is_available():   # no fallback: the library's kernels are the thing measured
        print("bench.py needs a CUDA device (sm_100a) and found none", file=sys.stderr)
        return 1
    if args.check:
        return run_check(args, raw, workload)
    if args.family:
        args.batch = args.batch if "--batch" in sys.argv else 8
        args.context = args.context if "--context" in sys.argv else 2048
        args.steps = args.steps if "--steps" in sys.argv else 64
        return run_family(args)
    return run_ours(args, raw, workload)


if __name__ == "__main__":
    sys.exit(main())
