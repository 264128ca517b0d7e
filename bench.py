#!/usr/bin/env python3
"""Measures generation on one B200: decode tokens a second at batch 8 (the headline), at
batch 1 and 64, and prefill of 2,048 tokens, on the Mistral-7B-v0.3 layer sizes with
random weights and random token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  A step is one decode step of the whole batch.  `value` times K
steps with CUDA events on the launching stream (engine step + token choice; the chosen
tokens stay on the device and feed the next step); `e2e` is the same number through the Python entry point
(`Model.generate`): host token ids in, host token ids out, every step copying its
inputs from pinned host memory and reading its chosen tokens back.  Weights (14.5 GB)
exceed the 126 MB L2, so no L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if d.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.index = index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.out.close()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    p = [x.strip() for x in line.split(",")]
                    if len(p) < 7:
                        continue
                    try:
                        sm.append(float(p[0])); mx.append(float(p[1]))
                    except ValueError:
                        continue
                    for n, v in zip(names, p[3:7]):
                        if v.lower().startswith("active"):
                            reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, n_layers):
    """Bytes a decode step reads and FLOPs a prefill does, from the configuration."""
    hs, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nk, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_layer_params = (nq + 2 * nk) * hd * hs + hs * nq * hd + 3 * I * hs + 2 * hs
    weight_bytes = 2 * (n_layers * per_layer_params + V * hs + hs)          # layers, head, final norm
    kv_bytes_per_token = n_layers * 2 * nk * hd * 2
    return per_layer_params, weight_bytes, kv_bytes_per_token


def prefill_flops(cfg, n_layers, T):
    hs, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nk, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    lin = 2 * T * ((nq + 2 * nk) * hd * hs + hs * nq * hd + 3 * I * hs)
    attn = 2 * 2 * nq * hd * (T * (T + 1) // 2)                             # causal QK^T and PV
    return n_layers * (lin + attn) + 2 * V * hs


def device_timed_decode(engine, sampler_kernels, prompts, steps, warmup):
    """K decode steps of the whole batch, timed with CUDA events; returns (seconds, context at start)."""
    import torch
    slots = [engine.open() for _ in prompts]
    logits = engine.step(list(zip(slots, prompts)), want="last")
    out = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
    sampler_kernels.argmax(logits, out)
    toks = out.tolist()
    for _ in range(warmup):
        logits = engine.step([(s, [t]) for s, t in zip(slots, toks)], want="last")
        sampler_kernels.argmax(logits, out)
    ctx0 = engine.length(slots[0])
    entries = [(s, [0]) for s in slots]                  # placeholders: each step takes its tokens from `out`
    rows = list(range(len(slots)))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = engine.kernels.launches
    e0.record()
    for _ in range(steps):
        logits = engine.step(entries, want="last", device_tokens=(out, rows))
        sampler_kernels.argmax(logits, out)
    e1.record()
    torch.cuda.synchronize()
    engine.check()
    launches = engine.kernels.launches - launches0
    for s in slots:
        engine.close(s)
    return e0.elapsed_time(e1) / 1e3, ctx0, launches


def sm_clock_reader():
    """A function that reads the SM clock in MHz (a query only), or None without NVML."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(0)
        return lambda: int(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
    except Exception:
        return None


def steps_after_a_prefill(engine, prompts, n=40):
    """The first `n` decode steps right after a batch's prefill, one by one: the time of each
    (host clock around a synchronised step) and the SM clock read after it.  Shows how long the
    clocks take to come back after the prefill's power draw, which is the difference between the
    device-timed number (taken after warm-up steps) and the one through the entry point."""
    import torch
    read_mhz = sm_clock_reader()
    slots = [engine.open() for _ in prompts]
    logits = engine.step(list(zip(slots, prompts)), want="last")
    out = torch.empty(len(prompts), dtype=torch.int32, device=engine.device)
    engine.kernels.argmax(logits, out)
    torch.cuda.synchronize()
    ms, mhz = [], []
    entries, rows = [(s, [0]) for s in slots], list(range(len(slots)))
    for _ in range(n):
        t0 = time.perf_counter()
        logits = engine.step(entries, want="last", device_tokens=(out, rows))
        engine.kernels.argmax(logits, out)
        torch.cuda.synchronize()
        ms.append(round((time.perf_counter() - t0) * 1e3, 3))
        mhz.append(read_mhz() if read_mhz else None)
    for s in slots:
        engine.close(s)
    prod = [round(a * b / 1e3, 2) for a, b in zip(ms, mhz)] if read_mhz else None      # ms x GHz: clock-free work
    return {"step_ms": ms, "sm_mhz": mhz, "ms_times_ghz": prod}


def run_ours(args):
    import torch
    from braidinfer_b200.api import Model
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.sampling import SamplingParams

    pk = peaks()
    cfg_dict = preset("mistral_7b_v03")
    full_layers = cfg_dict["num_hidden_layers"]
    if args.quick and not args.layers:
        args.layers = 4
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    n_layers = cfg_dict["num_hidden_layers"]
    B, prompt_len, gen_len, ctx_len = args.batch, 2048, 256, 4096
    steps, warmup = args.steps, max(3, args.warmup)
    t0 = time.time()
    cache_seqs = B if args.quick else 64
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=cache_seqs * ctx_len,
                                max_slots=64, use_graphs=not args.no_graphs, verbose=True)
    cfg = engine.config
    model = Model(engine, max_batch=64)
    g = torch.Generator().manual_seed(0)

    def prompts_for(b, n=prompt_len):
        return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for _ in range(b)]

    _, weight_bytes, kv_per_tok = model_numbers(cfg, n_layers)

    # ---- prefill of 2,048 tokens (one sequence), timed on the device
    p1 = prompts_for(1)
    times = []
    for i in range(3 + 3):
        s = engine.open()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step([(s, p1[0])], want="last")
        e1.record()
        torch.cuda.synchronize()
        engine.close(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    pre_ms = statistics.median(times)
    pre_flops = prefill_flops(cfg, n_layers, prompt_len)
    prefill = {"value": prompt_len / (pre_ms / 1e3), "tokens": prompt_len, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "unit": "tokens/s",
               "peak": f"{pk['bf16_tflops']} TFLOP/s bf16, {pk['source']}"}
    if pk.get("bf16_tflops_sustained"):
        # the step is timed as the median of back-to-back repeats, under the power cap: the library's
        # product measured the same way is the second yardstick
        prefill["frac_of_sustained"] = pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)
    if not args.quick:
        # the same prompt by itself, as one arrives in use: half a second of rest before each of three
        # repeats, so that the step starts below the power cap (the burst peak was measured so)
        rested = []
        for i in range(3):
            time.sleep(0.5)
            s = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([(s, p1[0])], want="last")
            e1.record()
            torch.cuda.synchronize()
            engine.close(s)
            rested.append(e0.elapsed_time(e1))
        r_ms = statistics.median(rested)
        prefill["after_rest"] = {"ms": r_ms, "value": prompt_len / (r_ms / 1e3),
                                 "frac": pre_flops / (r_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode at the headline batch, device-timed, with clocks sampled meanwhile
    with ClockSampler() as cs:
        secs, ctx0, launches = device_timed_decode(engine, engine.kernels, prompts_for(B), steps, warmup)
    clocks = cs.summary()
    value = B * steps / secs
    ms_per_step = secs / steps * 1e3
    avg_ctx = ctx0 + steps / 2
    step_bytes = weight_bytes + B * avg_ctx * kv_per_tok + B * cfg.hidden_size * 2
    achieved = step_bytes / (secs / steps) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"], "bytes_per_step": step_bytes}

    # ---- the same through the Python entry point: host tokens in, host tokens out
    e2e = None
    if not args.quick:
        outs = model.generate(prompts_for(B), SamplingParams.greedy(), stop_tokens=(),
                              max_new_tokens=min(steps, gen_len) + 1)
        st = model.last_stats
        e2e = {"value": st.decode_tokens / st.decode_seconds if st.decode_seconds > 0 else 0.0, "unit": "tokens/s",
               "h2d_bytes_per_step": engine.packer.h2d_bytes_last, "d2h_bytes_per_step": B * 4,
               "prefill_tokens_per_s": st.prompt_tokens / st.prefill_seconds if st.prefill_seconds > 0 else 0.0}

    # ---- other batch sizes, temperature sampling, and the steps right after a prefill
    points = {}
    after_prefill = None
    for b in (() if args.quick else (1, 64)):
        k = min(steps, 64)
        s2, _, _ = device_timed_decode(engine, engine.kernels, prompts_for(b), k, warmup)
        points[f"decode_b{b}"] = b * k / s2
    if not args.quick:
        warm = SamplingParams(temperature=0.8, seed=1)
        model.generate(prompts_for(B, 64), warm, stop_tokens=(), max_new_tokens=4)      # the sampling kernel's first call
        model.generate(prompts_for(B), warm, stop_tokens=(), max_new_tokens=min(steps, gen_len) + 1)
        st = model.last_stats
        points["decode_b8_temperature"] = st.decode_tokens / st.decode_seconds if st.decode_seconds > 0 else 0.0
        # a short prompt by itself (time to its first logits): such steps go through CUDA graphs from the
        # third step of a shape on
        short = prompts_for(1, 64)[0]
        ms = []
        for i in range(6):
            slot = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([(slot, short)], want="last")
            e1.record()
            torch.cuda.synchronize()
            engine.close(slot)
            ms.append(e0.elapsed_time(e1))
        points["prompt_64_tokens_ms"] = statistics.median(ms[3:])
        after_prefill = steps_after_a_prefill(engine, prompts_for(B))

    line = {
        "metric": "decode tokens/s at batch 8, Mistral-7B-v0.3 sizes, bf16 (also batch 1, 64; prefill of 2,048 tokens)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, uniform random token ids",
        "impl": "ours",
        "config": {"model": "Mistral-7B-v0.3 sizes", "layers": n_layers, "layers_of_full_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_theta": cfg.rope_theta, "rms_eps": cfg.rms_norm_eps, "global_batch": B,
                   "seq_len": ctx_len, "prompt_len": prompt_len, "context_at_timing": int(avg_ctx),
                   "cache_tokens": cache_seqs * ctx_len, "parallelism": "single GPU",
                   "l2": "inputs (14.5 GB of weights) exceed L2; no flush"},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill, "roofline": roofline,
        "points": points, "after_prefill": after_prefill, "setup_seconds": time.time() - t0,
    }
    print(json.dumps(line))
    return 0


def run_other_size(args):
    """The other sizes the measurements are quoted on:
    `mistral_7b_v01`: sliding window 4096, context 8192, batch 8, prompts of 6,000-8,000 tokens;
    `mistral_nemo_12b`: head_dim 128 with hidden 5120, vocabulary 131072, context 16384, batch 16, prompts of
    512-8,192 tokens.  One JSON line with the same keys as the default run: `value` is decode tokens a second
    timed on the device, `prefill` the batch's prompt step, `roofline` the bytes a decode step has to read
    (every weight once, and the keys and values that each sequence's window still sees) over its time,
    `e2e` the same batch through `Model.generate`."""
    import random
    import torch
    from braidinfer_b200.api import Model
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    from braidinfer_b200.sampling import SamplingParams
    pk = peaks()
    rng = random.Random(0)
    g = torch.Generator().manual_seed(0)
    if args.preset == "mistral_7b_v01":
        B, ctx, lens = 8, 8192, [rng.randint(6000, 8000) for _ in range(8)]
    else:
        B, ctx, lens = 16, 16384, [rng.randint(512, 8192) for _ in range(16)]
    cfg_dict = preset(args.preset)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    n_layers = cfg_dict["num_hidden_layers"]
    t0 = time.time()
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=B * ctx, max_slots=B)
    cfg = engine.config
    model = Model(engine, max_batch=B)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    steps, warmup = min(args.steps, 128), max(3, args.warmup)
    _, weight_bytes, kv_per_tok = model_numbers(cfg, n_layers)

    # the batch's prompts in one step (unequal lengths), timed on the device after one warm-up run
    pre_ms = None
    for i in range(2):
        slots = [engine.open() for _ in prompts]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step(list(zip(slots, prompts)), want="last")
        e1.record()
        torch.cuda.synchronize()
        pre_ms = e0.elapsed_time(e1)
        for sl in slots:
            engine.close(sl)
    window = cfg.sliding_window
    lin = 2 * ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim * cfg.hidden_size
               + cfg.hidden_size * cfg.num_attention_heads * cfg.head_dim + 3 * cfg.intermediate_size * cfg.hidden_size)
    att = sum(sum(min(p + 1, window) if window else p + 1 for p in range(n)) for n in lens) * 4 * cfg.num_attention_heads * cfg.head_dim
    pre_flops = n_layers * (lin * sum(lens) + att) + 2 * cfg.vocab_size * cfg.hidden_size * B
    prefill = {"value": sum(lens) / (pre_ms / 1e3), "tokens": sum(lens), "ms": pre_ms, "unit": "tokens/s",
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
               "peak": f"{pk['bf16_tflops']} TFLOP/s bf16, {pk['source']}"}

    with ClockSampler() as cs:
        secs, _, launches = device_timed_decode(engine, engine.kernels, prompts, steps, warmup)
    clocks = cs.summary()
    seen = [min(n + warmup + steps / 2, window) if window else n + warmup + steps / 2 for n in lens]
    step_bytes = weight_bytes + sum(seen) * kv_per_tok + B * cfg.hidden_size * 2
    achieved = step_bytes / (secs / steps) / 1e9
    outs = model.generate(prompts, SamplingParams.greedy(), stop_tokens=(), max_new_tokens=steps + 1)
    st = model.last_stats
    engine.check()
    print(json.dumps({
        "metric": f"decode tokens/s at batch {B}, {args.preset} sizes, bf16 (unequal prompts; also their prefill)",
        "value": B * steps / secs, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": secs / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, uniform random token ids", "impl": "ours",
        "config": {"model": args.preset, "layers": n_layers, "layers_of_full_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "sliding_window": window, "global_batch": B, "seq_len": ctx, "prompt_tokens": sum(lens),
                   "prompt_len_min": min(lens), "prompt_len_max": max(lens), "parallelism": "single GPU",
                   "weights_gb": round(engine.weight_bytes / 1e9, 2), "cache_gb": round(engine.cache.nbytes() / 1e9, 2),
                   "l2": "inputs (weights) exceed L2; no flush"},
        "e2e": {"value": st.decode_tokens / st.decode_seconds if st.decode_seconds > 0 else 0.0, "unit": "tokens/s",
                "h2d_bytes_per_step": engine.packer.h2d_bytes_last, "d2h_bytes_per_step": B * 4,
                "prefill_tokens_per_s": st.prompt_tokens / st.prefill_seconds if st.prefill_seconds > 0 else 0.0},
        "gpu_launches": launches, "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"], "bytes_per_step": step_bytes},
        "setup_seconds": time.time() - t0}))
    return 0


def run_sweep(args):
    """Decode at batch 1, 8, 64 over contexts of 512 to 32,768 tokens and prefill of 512 to 16,384
    tokens, on the default sizes: one JSON line with time, achieved bandwidth or FLOP rate, and the
    fraction of the peak, for every point.  Not the headline line."""
    import torch
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    pk = peaks()
    cfg_dict = preset("mistral_7b_v03")
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    n_layers = cfg_dict["num_hidden_layers"]
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=64 * (8192 + 128),
                                max_slots=64, verbose=True)
    cfg = engine.config
    g = torch.Generator().manual_seed(0)
    _, weight_bytes, kv_per_tok = model_numbers(cfg, n_layers)
    decode, prefill = [], []
    for T in (512, 2048, 8192, 16384):
        p = torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist()
        times = []
        for i in range(5):
            s = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([(s, p)], want="last")
            e1.record()
            torch.cuda.synchronize()
            engine.close(s)
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        fl = prefill_flops(cfg, n_layers, T)
        prefill.append({"tokens": T, "ms": round(ms, 3), "tokens_per_s": round(T / ms * 1e3),
                        "tflops": round(fl / ms / 1e9, 1), "frac": round(fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3)})
    for ctx in (512, 2048, 8192, 32768):
        for b in (1, 8, 64):
            if b * (ctx + 128) > engine.max_tokens:
                continue
            prompts = [torch.randint(0, cfg.vocab_size, (ctx,), generator=g).tolist() for _ in range(b)]
            steps = 48
            secs, ctx0, _ = device_timed_decode(engine, engine.kernels, prompts, steps, 24)    # clocks settle after the prompts
            step_bytes = weight_bytes + b * (ctx0 + steps / 2) * kv_per_tok
            gbs = step_bytes / (secs / steps) / 1e9
            decode.append({"batch": b, "context": ctx, "ms_per_step": round(secs / steps * 1e3, 3),
                           "tokens_per_s": round(b * steps / secs, 1), "gb_per_s": round(gbs),
                           "frac": round(gbs / pk["hbm_gbs"], 3)})
    print(json.dumps({"metric": "sweep over batch, context and prompt length, Mistral-7B-v0.3 sizes, bf16", "impl": "ours",
                      "layers": n_layers, "peaks": pk, "prefill": prefill, "decode": decode}))
    return 0


def run_timeline(args):
    """Where a decode step's time goes: one CUDA-graph step of the default sizes under the torch
    profiler (device activity only), printed as one JSON line: for the kernels of one layer in the
    middle of the step, the time from the end of the kernel before to the end of this one (kernels
    overlap their predecessors' tails through programmatic dependent launch, so durations would
    count time twice).  Not the headline line."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    cfg_dict = preset("mistral_7b_v03")
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    B = args.batch
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True, max_tokens=B * 4096, max_slots=B,
                                verbose=True)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, engine.config.vocab_size, (2048,), generator=g).tolist() for _ in range(B)]
    slots = [engine.open() for _ in prompts]
    engine.step(list(zip(slots, prompts)))
    for _ in range(8):
        engine.step([(s, [5]) for s in slots])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            engine.step([(s, [5]) for s in slots])
        torch.cuda.synchronize()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "trace.json")
        prof.export_chrome_trace(path)
        with open(path) as f:
            ev = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
    ev.sort(key=lambda e: e["ts"])
    first = [i for i, e in enumerate(ev) if "embed" in e["name"]][-1]
    step = ev[first:]
    span = step[-1]["ts"] + step[-1]["dur"] - step[0]["ts"]
    # a layer = from one attention kernel to the next
    att = [i for i, e in enumerate(step) if "attn_" in e["name"] and "combine" not in e["name"]]
    mid = len(att) // 2
    start, per_layer = att[mid], att[mid + 1] - att[mid]
    rows, prev_end = [], step[start - 1]["ts"] + step[start - 1]["dur"]
    for e in step[start:start + per_layer]:
        end = e["ts"] + e["dur"]
        rows.append({"kernel": e["name"].split("(")[0][:48], "until_its_end_us": round(end - prev_end, 2)})
        prev_end = end
    print(json.dumps({"metric": "one decode step under the profiler, Mistral-7B-v0.3 sizes, bf16", "impl": "ours",
                      "batch": B, "kernels_in_step": len(step), "step_us": round(span, 1), "kernels_a_layer": per_layer,
                      "layer_us": round(sum(r["until_its_end_us"] for r in rows), 1), "one_layer": rows}))
    return 0


def run_prompt_timeline(args):
    """Where a prompt's time goes, by prompt length: for each length given (--prompt-timeline 256,512,...), one prompt
    step of the default layer sizes (8 layers unless --layers says otherwise) under the torch profiler, and for the
    kernels of one layer in the middle the time from the end of the kernel before to the end of this one, as
    run_timeline does for a decode step.  Lengths up to 256 go through a CUDA graph from the third step on, as they
    do in generation.  One JSON line a length.  Not the headline line."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from braidinfer_b200.config import preset
    from braidinfer_b200.engine import Engine
    cfg_dict = preset("mistral_7b_v03")
    cfg_dict["num_hidden_layers"] = args.layers or 8
    lengths = [int(t) for t in args.prompt_timeline.split(",")]
    engine = Engine.from_random(cfg_dict, seed=0, dtype="bfloat16", on_device=True,
                                max_tokens=2 * max(max(lengths), 4096), max_slots=2, verbose=True)
    c = engine.config
    per_token = 2 * (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                     + c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    pk = peaks()
    g = torch.Generator().manual_seed(0)
    for T in lengths:
        prompt = torch.randint(0, c.vocab_size, (T,), generator=g).tolist()
        for _ in range(3):
            s = engine.open()
            engine.step([(s, prompt)])
            engine.close(s)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            s = engine.open()
            engine.step([(s, prompt)])
            engine.close(s)
            torch.cuda.synchronize()
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "trace.json")
            prof.export_chrome_trace(path)
            with open(path) as f:
                ev = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
        ev.sort(key=lambda e: e["ts"])
        att = [i for i, e in enumerate(ev) if "attn_" in e["name"] and "combine" not in e["name"]]
        mid = len(att) // 2
        start, per_layer = att[mid], att[mid + 1] - att[mid]
        rows, prev_end = [], ev[start - 1]["ts"] + ev[start - 1]["dur"]
        for e in ev[start:start + per_layer]:
            end = e["ts"] + e["dur"]
            rows.append({"kernel": e["name"].split("(")[0][:48], "until_its_end_us": round(end - prev_end, 2)})
            prev_end = end
        layer_us = sum(r["until_its_end_us"] for r in rows)
        print(json.dumps({"metric": "one prompt step under the profiler, Mistral-7B-v0.3 layer sizes, bf16", "impl": "ours",
                          "tokens": T, "layers": cfg_dict["num_hidden_layers"], "layer_us": round(layer_us, 1),
                          "layer_flops_over_burst_peak_us": round(T * per_token / (pk["bf16_tflops"] * 1e12) * 1e6, 1),
                          "frac_of_burst": round(T * per_token / (pk["bf16_tflops"] * 1e12) * 1e6 / layer_us, 3),
                          "step_us": round(ev[-1]["ts"] + ev[-1]["dur"] - ev[0]["ts"], 1), "one_layer": rows}), flush=True)
    return 0


def run_chain(args):
    """What the chain of dependent kernels of a decode step costs, at the default sizes: products alone chained to
    themselves, and product + reducer pairs, each six times over distinct weights in one CUDA graph, timed with
    events (L2 flushed before each replay).  With BRAIDINFER_TRACE=1 in the environment the library is built with
    time stamps at the phase boundaries of the product and of the reduce + norm kernel (csrc/trace.cuh); the
    line then also carries, for the o product + reducer chain, the median over CTAs of every stamp, in
    microseconds from the chain's first entry.  Not the headline line."""
    import ctypes
    import numpy as np
    import torch
    from braidinfer_b200.csrc import build
    from braidinfer_b200.csrc.api import get_kernels, interleave_gate_up
    K = get_kernels(verbose=True)
    dev, B = "cuda", args.batch
    hs, I, nq, nk, hd, NL = 4096, 14336, 32, 8, 128, 6
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *sh: (torch.randn(*sh, device=dev, generator=g) * 0.02).bfloat16()
    W = {"qkv": [rn((nq + 2 * nk) * hd, hs) for _ in range(NL)], "o": [rn(hs, nq * hd) for _ in range(NL)],
         "gate_up": [interleave_gate_up(rn(I, hs), rn(I, hs)) for _ in range(NL)], "down": [rn(hs, I) for _ in range(NL)]}
    X = {"qkv": rn(B, hs), "o": rn(B, nq * hd), "gate_up": rn(B, hs), "down": rn(B, I)}
    wn = torch.ones(hs, device=dev, dtype=torch.bfloat16)
    h = torch.zeros(B, hs, device=dev)
    out = torch.empty(B, hs, device=dev, dtype=torch.bfloat16)
    act = torch.empty(B, I, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)

    def product_only(name):
        def f(l):
            K.gemm_tc_partial(X[name], W[name][l])
            K.pending_partial = None
        return f

    def with_reducer(name):
        def f(l):
            p = K.gemm_tc_partial(X[name], W[name][l])
            if name == "gate_up":
                K.streamk_reduce(p, act, swiglu=True)
            else:
                K.streamk_reduce_norm(p, h, wn, out, 1e-5)
        return f

    def graph_of(fn):
        body = lambda: [fn(l) for l in range(NL)]
        body()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            body()
        K.pending_partial = None
        return gr

    def timed(gr, reps=20):
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); gr.replay(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / NL)
        return round(statistics.median(ts), 2)

    pk = peaks()
    res = {}
    for name in ("o", "qkv", "down", "gate_up"):
        ideal = W[name][0].numel() * 2 / (pk["hbm_gbs"] * 1e3)
        res[name] = {"bytes_over_bandwidth_us": round(ideal, 2), "product_alone_us": timed(graph_of(product_only(name))),
                     "product_and_reducer_us": timed(graph_of(with_reducer(name)))}
    line = {"metric": "chains of decode-step kernels, Mistral-7B-v0.3 layer sizes, bf16", "impl": "ours", "batch": B,
            "peaks": pk, "per_kernel_or_pair": res}
    if build.trace_build():
        gr = graph_of(with_reducer("o"))
        for _ in range(2):
            flush.zero_(); gr.replay()
        traces = {}
        for kname, ctas, names in (("gemm_tc", 160, ["entry", "set_up", "ring_asked", "wait_over", "first_stage_full",
                                                     "last_accumulator", "epilogue_done", "all_done"]),
                                   ("reduce_norm", 64, ["entry", "before_wait", "wait_over", "loaded_and_added",
                                                        "block_sum_done", "stored"])):
            read = getattr(K.lib, f"braid_{kname}_trace_read")
            buf = (ctypes.c_ulonglong * (64 * ctas * 8))()
            read(buf, 1)                                   # forget the warm-up launches
            traces[kname] = (read, buf, ctas, names)
        flush.zero_()
        torch.cuda.synchronize()
        gr.replay()
        torch.cuda.synchronize()
        t0, table = None, {}
        for kname, (read, buf, ctas, names) in traces.items():
            read(buf, 0)
            t = np.frombuffer(buf, dtype=np.uint64).reshape(64, ctas, 8).astype(np.float64)
            if t0 is None:
                t0 = t[0, :, 0][t[0, :, 0] > 0].min()
            rows = []
            for l in range(NL):
                ok = t[l, :, 0] > 0
                if ok.any():
                    rows.append({n: round(float(np.median(t[l, ok, i]) - t0) / 1e3, 2) for i, n in enumerate(names)})
            table[kname] = rows
        line["trace_o_product_and_reducer_us"] = table
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------ the Bidinex decoder beside the dense one
BIDINEX_SIZES = {
    # name: width, heads, dim, rot_dim, vdim, kv_rank, experts, groups, keep, top, expert ff, layers, vocab
    "w2048_e64": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, rank=512, experts=64, groups=8, keep=4, top=6,
                      ff=1408, layers=4, vocab=32768),
    "w4096_e32": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, rank=512, experts=32, groups=4, keep=2, top=4,
                      ff=2048, layers=4, vocab=32768),
    "w1024_e16": dict(width=1024, heads=8, dim=64, rot=32, vdim=64, rank=256, experts=16, groups=1, keep=1, top=2,
                      ff=1024, layers=4, vocab=32768),
}


def bidinex_config(z):
    mixer = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "rot": {"base": 10000.0, "dims": z["rot"]},
             "vdim": z["vdim"], "kv_rank": z["rank"], "scale": (z["dim"] + z["rot"]) ** -0.5}
    mlp = {"kind": "moe", "expert": {"ff": z["ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"], "keep": z["keep"]}}}
    return {"architecture": "Bidinex", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5}, "residual_mult": 1.0, "logit_softcap": 30.0,
            "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": mlp} for _ in range(z["layers"])], "loop": None}


def dense_twin_config(z):
    """The dense decoder of equal size: same width, layers, heads and vocabulary, a head as large as a latent head's
    query (dim + rot_dim, rounded to what the tcgen05 attention is built for), the feed-forward as wide as the
    experts a token uses."""
    hd = 128 if z["dim"] + z["rot"] > 64 else 64
    return {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "torch_dtype": "bfloat16",
            "num_hidden_layers": z["layers"], "hidden_size": z["width"], "num_attention_heads": z["heads"],
            "num_key_value_heads": max(1, z["heads"] // 4), "head_dim": hd, "intermediate_size": z["top"] * z["ff"],
            "vocab_size": z["vocab"], "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "sliding_window": None,
            "tie_word_embeddings": True, "max_position_embeddings": 32768}


def run_bidinex(args):
    """`--bidinex`: prompt and decode throughput of the Bidinex decoder at sizes like a real model's layers (random
    weights, a few layers), beside the dense decoder of equal size, and the new kernels one by one beside the
    dense model's like kernels with their fractions of the measured peaks.  Prints one JSON line of its own; the
    default run and its line are untouched."""
    import torch
    from braidinfer_b200.engine import Engine
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, reps=5, warm=2, graph=False):
        """Median device time of fn() after warm-up, L2 flushed before every call.  `graph`: fn's launches are
        captured once and replayed, so that a kernel of a few microseconds is not timed by the host's launches."""
        for _ in range(warm):
            fn()
        run = fn
        if graph:
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            run = gr.replay
            run()
        ts = []
        for _ in range(reps):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / 1e3)
        return statistics.median(ts)

    def frac(seconds, flops, nbytes):
        """Time the kernel's work takes at the measured peaks (the slower of its FLOPs and its bytes) over its time."""
        return max(flops / (pk["bf16_tflops"] * 1e12), nbytes / (pk["hbm_gbs"] * 1e9)) / seconds

    T, B, C = args.prompt_len, args.batch, args.context
    sizes = [n for n in BIDINEX_SIZES if not args.sizes or n in args.sizes.split(",")]
    out = {"metric": "bidinex_beside_dense_decoder", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic, random weights",
           "prompt_len": T, "decode_batch": B, "decode_context": C, "peaks": pk, "l2": "flushed between timed calls",
           "sizes": {}}
    with ClockSampler() as clocks:
        for name in sizes:
            z = BIDINEX_SIZES[name]
            row = {}
            for label, cfg in (("bidinex", bidinex_config(z)), ("dense", dense_twin_config(z))):
                eng = Engine.from_random(cfg, 1, dtype="bfloat16", on_device=True, max_tokens=max(B * (C + 192), T + 64),
                                         max_slots=B, verbose=False)
                g = torch.Generator().manual_seed(0)
                prompt = torch.randint(0, z["vocab"], (T,), generator=g).tolist()

                def prefill():
                    s = eng.open()
                    eng.step([(s, prompt)], want="last")
                    eng.close(s)
                tp = timed(prefill, reps=3, warm=2)
                prompts = [torch.randint(0, z["vocab"], (C,), generator=g).tolist() for _ in range(B)]
                secs, ctx0, launches = device_timed_decode(eng, eng.kernels, prompts, args.steps, max(args.warmup, 3))
                eng.check()
                row[label] = {"prefill_tokens_per_s": round(T / tp), "prefill_ms": round(tp * 1e3, 3),
                              "decode_tokens_per_s": round(B * args.steps / secs), "decode_ms_per_step": round(secs / args.steps * 1e3, 4),
                              "weight_gb": round(eng.weight_bytes / 1e9, 3), "launches_per_decode_step": launches // args.steps}
                del eng
                torch.cuda.empty_cache()
            row["kernels"] = bidinex_kernels(z, T, B, C, timed, frac)
            out["sizes"][name] = row
    out["clocks"] = clocks.summary()
    print(json.dumps(out))
    return 0


def bidinex_kernels(z, T, B, C, timed, frac):
    """The new kernels alone, each beside the dense decoder's like kernel: seconds, and the fraction of the measured
    peak its algorithmic FLOPs or bytes (whichever bounds it) reach."""
    import torch
    from braidinfer_b200.cache import PAGE_SIZE
    from braidinfer_b200.csrc.api import get_kernels
    K = get_kernels(verbose=False)
    dev, bf = "cuda", torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    H, R, rot, W, E, top, ff = z["heads"], z["rank"], z["rot"], z["width"], z["experts"], z["top"], z["ff"]
    D = R + rot
    hd = 128 if z["dim"] + z["rot"] > 64 else 64
    nkh = max(1, H // 4)
    res = {}

    def paged(n_seqs, length, planes, heads, dim):
        blocks = -(-length // PAGE_SIZE)
        cache = torch.randn(n_seqs * blocks, planes, heads, PAGE_SIZE, dim, device=dev, dtype=bf) * 0.5
        table = torch.arange(n_seqs * blocks, dtype=torch.int32, device=dev).view(n_seqs, blocks)
        return cache, table

    # ---- attention over a prompt of T tokens
    cache, table = paged(1, T, 1, 1, D)
    q = torch.randn(T, H, D, device=dev, dtype=bf) * 0.3
    o = torch.empty(T, H, R, device=dev, dtype=bf)
    seq0 = torch.zeros(T, dtype=torch.int32, device=dev)
    z0, zT = i32([0]), i32([T])
    t = timed(lambda: K.attn_latent_mma(q, o, cache, table, z0, zT, z0, seq0, 1, T, R, None, 0.1), graph=True)
    fl = 2 * H * (D + R) * (T * (T + 1) // 2) * (2 if R > 256 else 1) / (2 if R > 256 else 1)
    res["prompt_attention"] = {"latent_mma_ms": round(t * 1e3, 3), "latent_frac": round(frac(t, fl, 0), 3)}
    dcache, dtable = paged(1, T, 2, nkh, hd)
    qkv = torch.randn(T, (H + 2 * nkh) * hd, device=dev, dtype=bf) * 0.3
    od = torch.empty(T, H * hd, device=dev, dtype=bf)
    t = timed(lambda: K.attn_tc(qkv, od, dcache, dtable, z0, zT, z0, 1, T, H, nkh, hd, None, 0.1), graph=True)
    res["prompt_attention"].update(dense_tcgen05_ms=round(t * 1e3, 3), dense_frac=round(frac(t, 2 * 2 * H * hd * (T * (T + 1) // 2), 0), 3))

    # ---- attention of B decoded tokens over a context of C
    cache, table = paged(B, C, 1, 1, D)
    q = torch.randn(B, H, D, device=dev, dtype=bf) * 0.3
    o = torch.empty(B, H, R, device=dev, dtype=bf)
    seqs = torch.arange(B, dtype=torch.int32, device=dev)
    ones, befores, starts = i32([1] * B), i32([C - 1] * B), i32(list(range(B)))
    n_splits = max(1, min(296 // K.attn_latent_ctas(R, rot, B, 1, H), (C // 32) // 4, 32))
    t = timed(lambda: K.attn_latent_mma(q, o, cache, table, starts, ones, befores, seqs, B, 1, R, None, 0.1, n_splits=n_splits), reps=9, graph=True)
    res["decode_attention"] = {"latent_mma_ms": round(t * 1e3, 4), "latent_frac": round(frac(t, 0, B * C * D * 2), 3), "slices": n_splits}
    dcache, dtable = paged(B, C, 2, nkh, hd)
    qkv = torch.randn(B, (H + 2 * nkh) * hd, device=dev, dtype=bf) * 0.3
    od = torch.empty(B, H * hd, device=dev, dtype=bf)
    g = H // nkh
    sp = max(1, min(K.attn_decode_slots(hd) // (B * nkh * -(-g // 16)), (C // 32) // 4, 64))
    t = timed(lambda: K.attn_mma(qkv, od, dcache, dtable, starts, ones, befores, seqs, B, 1, H, nkh, hd, None, 0.1,
                                 n_splits=sp, few_tokens=True), reps=9, graph=True)
    res["decode_attention"].update(dense_mma_ms=round(t * 1e3, 4), dense_frac=round(frac(t, 0, B * C * 2 * nkh * hd * 2), 3))

    # ---- the feed-forward's products: the experts over sorted rows beside the dense gate+up and down
    for what, rows in (("prompt_experts", T), ("decode_experts", B)):
        x = torch.randn(rows, W, device=dev, dtype=bf) * 0.3
        wg, wu = [torch.randn(E, ff, W, device=dev, dtype=bf) * 0.02 for _ in range(2)]
        wd = torch.randn(E, W, ff, device=dev, dtype=bf) * 0.02
        idx = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(rows)]).to(torch.int32)
        tile = 16 if rows * top <= 16 * E else 64
        plan = K.moe_plan(idx, torch.zeros(rows, dtype=torch.int32, device=dev), E, tile)
        act = torch.empty(plan[4] * tile, ff, device=dev, dtype=bf)
        y = torch.empty(plan[4] * tile, W, device=dev, dtype=bf)
        t1 = timed(lambda: K.moe_gemm_mma(x, wg, wu, act, plan, top, tile), graph=True)
        t2 = timed(lambda: K.moe_gemm_mma(act, wd, None, y, plan, top, tile), graph=True)
        used = int(torch.unique(idx).numel())
        fl1, fl2 = 2 * rows * top * 2 * ff * W, 2 * rows * top * ff * W
        by1, by2 = used * 2 * ff * W * 2, used * ff * W * 2
        res[what] = {"gate_up_ms": round(t1 * 1e3, 4), "gate_up_frac": round(frac(t1, fl1, by1), 3),
                     "down_ms": round(t2 * 1e3, 4), "down_frac": round(frac(t2, fl2, by2), 3), "experts_used": used, "tile": tile}
        del wg, wu, wd
        I = top * ff
        from braidinfer_b200.csrc.api import interleave_gate_up
        from braidinfer_b200.parts.linear import stream_k_pays
        wgu = interleave_gate_up(torch.randn(I, W, device=dev, dtype=bf) * 0.02, torch.randn(I, W, device=dev, dtype=bf) * 0.02)
        wdn = torch.randn(W, I, device=dev, dtype=bf) * 0.02
        a2 = torch.empty(rows, I, device=dev, dtype=bf)
        hres = torch.zeros(rows, W, device=dev, dtype=torch.float32)
        sk1, sk2 = stream_k_pays(rows, wgu.shape[0], W), stream_k_pays(rows, W, I)
        t1 = timed(lambda: K.gemm_tc(x, wgu, a2, swiglu=True, stream_k=sk1), graph=True)
        t2 = timed(lambda: K.gemm_tc(a2, wdn, hres, residual=hres, stream_k=sk2), graph=True)
        res[what].update(dense_gate_up_ms=round(t1 * 1e3, 4), dense_gate_up_frac=round(frac(t1, 2 * rows * 2 * I * W, 2 * I * W * 2), 3),
                         dense_down_ms=round(t2 * 1e3, 4), dense_down_frac=round(frac(t2, 2 * rows * I * W, I * W * 2), 3))
        del wgu, wdn
    # ---- the per-head products of the latent mixer (no like kernel in the dense decoder)
    for what, rows in (("prompt_head_products", T), ("decode_head_products", B)):
        qx = torch.randn(rows, H, z["dim"] + rot, device=dev, dtype=bf)[:, :, :z["dim"]]
        wk = torch.randn(H, R, z["dim"], device=dev, dtype=bf) * 0.05
        ql = torch.empty(rows, H, D, device=dev, dtype=bf)
        qlv = ql[:, :, :R]
        t1 = timed(lambda: K.gemm_heads(qx, wk, qlv), graph=True)
        ol = torch.randn(rows, H, R, device=dev, dtype=bf)
        wv = torch.randn(H, z["vdim"], R, device=dev, dtype=bf) * 0.05
        ov = torch.empty(rows, H, z["vdim"], device=dev, dtype=bf)
        t2 = timed(lambda: K.gemm_heads(ol, wv, ov), graph=True)
        res[what] = {"into_latent_ms": round(t1 * 1e3, 4),
                     "into_latent_frac": round(frac(t1, 2 * rows * H * R * z["dim"], 2 * (rows * H * (z["dim"] + R) + H * R * z["dim"])), 3),
                     "out_of_latent_ms": round(t2 * 1e3, 4),
                     "out_of_latent_frac": round(frac(t2, 2 * rows * H * R * z["vdim"], 2 * (rows * H * (z["vdim"] + R) + H * R * z["vdim"])), 3)}
    return res

# ------------------------------------------------------------------ the Loduzen decoder beside the dense one
LODUZEN_SIZES = {
    # width, attention heads / kv heads / head size / window, linear-attention heads / key / value size,
    # state-space heads / value size / state / groups, feed-forward, side columns, layers (attention and state-space in turn)
    "w2048": dict(width=2048, heads=16, kv=4, dim=128, window=1024, lheads=8, ldk=128, ldv=256, sheads=64, sp=64, sn=128, sg=8,
                  ff=5632, side=256, layers=4, vocab=32768),
    "w4096": dict(width=4096, heads=32, kv=8, dim=128, window=1024, lheads=16, ldk=128, ldv=256, sheads=128, sp=64, sn=128, sg=8,
                  ff=14336, side=256, layers=4, vocab=32768),
    "w1024": dict(width=1024, heads=8, kv=2, dim=64, window=512, lheads=4, ldk=64, ldv=128, sheads=32, sp=64, sn=64, sg=4,
                  ff=2816, side=128, layers=4, vocab=32768),
}


def loduzen_config(z):
    left = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
            "mask": {"size": z["window"]},
            "rot": {"base": 1e6, "dims": z["dim"] // 2, "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
    right = {"heads": z["lheads"], "dim": z["ldk"], "vdim": z["ldv"], "tau": 8.0}
    par = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0},
           "mlp": {"kind": "dense", "ff": z["ff"]}}
    ssm = {"type": "mamba2", "mixer": {"heads": z["sheads"], "vdim": z["sp"], "state": z["sn"], "groups": z["sg"], "conv": 4,
                                       "norm_groups": z["sg"]}, "mlp": {"kind": "dense", "ff": z["ff"]}}
    return {"architecture": "Loduzen", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
            "token_side": {"dim": z["side"]}, "layers": [par if i % 2 == 0 else ssm for i in range(z["layers"])]}


def loduzen_twin_config(z):
    """The dense decoder of equal size: same width, layers, attention heads, head size, window, feed-forward, vocabulary."""
    return {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "torch_dtype": "bfloat16",
            "num_hidden_layers": z["layers"], "hidden_size": z["width"], "num_attention_heads": z["heads"],
            "num_key_value_heads": z["kv"], "head_dim": z["dim"], "intermediate_size": z["ff"], "vocab_size": z["vocab"],
            "rope_theta": 1e6, "rms_norm_eps": 1e-6, "sliding_window": z["window"], "tie_word_embeddings": True,
            "max_position_embeddings": 32768}


def run_loduzen(args):
    """`--loduzen`: prompt and decode throughput of the Loduzen decoder at sizes like a real model's layers (random
    weights, four layers), beside the dense decoder of equal size, and the new kernels one by one beside the dense
    model's like kernels with their fractions of the measured peaks.  Prints one JSON line of its own; the default
    run and its line are untouched."""
    import torch
    from braidinfer_b200.engine import Engine
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, reps=5, warm=2, graph=False):
        for _ in range(warm):
            fn()
        run = fn
        if graph:
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            run = gr.replay
            run()
        ts = []
        for _ in range(reps):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / 1e3)
        return statistics.median(ts)

    def frac(seconds, flops, nbytes):
        return max(flops / (pk["bf16_tflops"] * 1e12), nbytes / (pk["hbm_gbs"] * 1e9)) / seconds

    T, B, C = args.prompt_len, args.batch, args.context
    sizes = [n for n in LODUZEN_SIZES if not args.sizes or n in args.sizes.split(",")]
    out = {"metric": "loduzen_beside_dense_decoder", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic, random weights",
           "prompt_len": T, "decode_batch": B, "decode_context": C, "peaks": pk, "l2": "flushed between timed calls", "sizes": {}}
    with ClockSampler() as clocks:
        for name in sizes:
            z = LODUZEN_SIZES[name]
            row = {}
            for label, cfg in (("loduzen", loduzen_config(z)), ("dense", loduzen_twin_config(z))):
                eng = Engine.from_random(cfg, 1, dtype="bfloat16", on_device=True, max_tokens=max(B * (C + 192), T + 64),
                                         max_slots=B, verbose=False)
                g = torch.Generator().manual_seed(0)
                prompt = torch.randint(0, z["vocab"], (T,), generator=g).tolist()

                def prefill():
                    s = eng.open()
                    eng.step([(s, prompt)], want="last")
                    eng.close(s)
                tp = timed(prefill, reps=3, warm=2)
                prompts = [torch.randint(0, z["vocab"], (C,), generator=g).tolist() for _ in range(B)]
                secs, ctx0, launches = device_timed_decode(eng, eng.kernels, prompts, args.steps, max(args.warmup, 3))
                eng.check()
                row[label] = {"prefill_tokens_per_s": round(T / tp), "prefill_ms": round(tp * 1e3, 3),
                              "decode_tokens_per_s": round(B * args.steps / secs), "decode_ms_per_step": round(secs / args.steps * 1e3, 4),
                              "weight_gb": round(eng.weight_bytes / 1e9, 3), "state_mb_per_sequence": round(sum(
                                  s.shape[1] for s in eng.cache.state if s is not None) / 1e6, 3),
                              "launches_per_decode_step": launches // args.steps}
                del eng
                torch.cuda.empty_cache()
            row["kernels"] = loduzen_kernels(z, T, B, C, timed, frac)
            out["sizes"][name] = row
    out["clocks"] = clocks.summary()
    print(json.dumps(out))
    return 0


def loduzen_kernels(z, T, B, C, timed, frac):
    """The new kernels alone, each beside the dense decoder's like kernel where it has one: seconds, and the fraction
    of the measured peak that its algorithmic FLOPs or bytes (whichever bounds it) reach.  The recurrences run on the
    ordinary float32 pipes: their `frac` is of the copy bandwidth (the bytes they must move), and `tflops` says what
    they compute."""
    import torch
    from types import SimpleNamespace
    from braidinfer_b200.cache import PAGE_SIZE
    from braidinfer_b200.csrc.api import get_kernels
    K = get_kernels(verbose=False)
    dev, bf = "cuda", torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    H, nkh, hd, Wd, win = z["heads"], z["kv"], z["dim"], z["width"], z["window"]
    res = {}

    def paged(n_seqs, length):
        blocks = -(-length // PAGE_SIZE)
        cache = torch.randn(n_seqs * blocks, 2, nkh, PAGE_SIZE, hd, device=dev, dtype=bf) * 0.5
        table = torch.arange(n_seqs * blocks, dtype=torch.int32, device=dev).view(n_seqs, blocks)
        return cache, table

    def steps_of(n_seqs, each, before):
        rows = n_seqs * each
        return SimpleNamespace(rows=rows, n_tokens=rows, n_seqs=n_seqs, q_start=i32([i * each for i in range(n_seqs)]),
                               q_len=i32([each] * n_seqs), kv_before=i32([before] * n_seqs), slot_ids=i32(list(range(n_seqs))), max_q_len=each,
                               token_seq=torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(each),
                               positions=(torch.arange(each, dtype=torch.int32, device=dev) + before).repeat(n_seqs))

    # ---- attention over a prompt of T tokens: the kernel with the sink beside the dense model's
    cache, table = paged(1, T)
    st = steps_of(1, T, 0)
    q = torch.randn(T, (H + nkh) * hd, device=dev, dtype=bf) * 0.3
    o = torch.empty(T, H * hd, device=dev, dtype=bf)
    visible = sum(min(p + 1, win) for p in range(T))
    fl = 2 * 2 * H * hd * visible
    t = timed(lambda: K.attn_mma(q, o, cache, table, st.q_start, st.q_len, st.kv_before, st.token_seq, 1, T, H, nkh, hd, win,
                                 hd ** -0.5, sink=0.0, out_scale=1.2), graph=True)
    res["prompt_attention"] = {"sink_mma_ms": round(t * 1e3, 3), "sink_mma_frac": round(frac(t, fl, 0), 3)}
    if K.attn_tc_supports(hd):
        for label, sink in (("sink_tcgen05", 0.0), ("dense_tcgen05", None)):
            t = timed(lambda: K.attn_tc(q, o, cache, table, st.q_start, st.q_len, st.kv_before, 1, T, H, nkh, hd, win, hd ** -0.5,
                                        sink=sink, out_scale=1.2 if sink is not None else 1.0), graph=True)
            res["prompt_attention"].update({label + "_ms": round(t * 1e3, 3), label + "_frac": round(frac(t, fl, 0), 3)})

    # ---- attention of B decoded tokens over a context of C
    cache, table = paged(B, C)
    sd = steps_of(B, 1, C - 1)
    q = torch.randn(B, (H + nkh) * hd, device=dev, dtype=bf) * 0.3
    o = torch.empty(B, H * hd, device=dev, dtype=bf)
    g = H // nkh
    span = min(C, win)
    sp = max(1, min(K.attn_decode_slots(hd) // (B * nkh * -(-g // 16)), (span // 32) // 4, 64))
    by = B * span * 2 * nkh * hd * 2
    for label, sink in (("sink", 0.0), ("dense", None)):
        t = timed(lambda: K.attn_mma(q, o, cache, table, sd.q_start, sd.q_len, sd.kv_before, sd.token_seq, B, 1, H, nkh, hd, win,
                                     hd ** -0.5, n_splits=sp, few_tokens=True, sink=sink), reps=9, graph=True)
        res.setdefault("decode_attention", {"slices": sp}).update({label + "_mma_ms": round(t * 1e3, 4), label + "_frac": round(frac(t, 0, by), 3)})

    # ---- norm of heads + rotation + cache write (one kernel) beside the dense model's rotation + cache write
    inv = torch.rand(hd // 4, device=dev)
    wn = torch.ones(hd, device=dev, dtype=bf)
    for what, stp, n_seqs, length in (("prompt_prep", st, 1, T), ("decode_prep", sd, B, C)):
        cache, table = paged(n_seqs, length)
        rows = stp.rows
        qk = torch.randn(rows, (H + nkh) * hd, device=dev, dtype=bf)
        qkv = torch.randn(rows, (H + 2 * nkh) * hd, device=dev, dtype=bf)
        t1 = timed(lambda: K.head_norm_rope_kv(qk, wn, wn, inv, stp.positions, stp.token_seq, table, cache, H, nkh, hd, hd // 2, True,
                                               True, PAGE_SIZE, 1e-6, 1.1), reps=9, graph=True)
        t2 = timed(lambda: K.rope_kv_write(qkv, inv, stp.positions, stp.token_seq, table, cache, H, nkh, hd, hd // 2, True, PAGE_SIZE),
                   reps=9, graph=True)
        by1 = rows * hd * 2 * (2 * (H + nkh) + 2 * nkh)
        res[what] = {"norm_rope_ms": round(t1 * 1e3, 4), "norm_rope_frac": round(frac(t1, 0, by1), 3),
                     "dense_rope_ms": round(t2 * 1e3, 4), "dense_frac": round(frac(t2, 0, by1), 3)}

    # ---- the recurrences: gated linear attention (a decay per channel) and the state-space layer (a decay per head)
    for what, stp in (("prompt", st), ("decode", sd)):
        rows, n_seqs = stp.rows, stp.n_seqs
        for kind, heads, groups, dk, dv in (("linear_attention", z["lheads"], z["lheads"], z["ldk"], z["ldv"]),
                                            ("state_space", z["sheads"], z["sg"], z["sn"], z["sp"])):
            qq = torch.randn(rows, groups * dk, device=dev, dtype=bf) * 0.1
            kk = torch.randn(rows, groups * dk, device=dev, dtype=bf) * 0.1
            vv = torch.randn(rows, heads * dv, device=dev, dtype=bf)
            oo = torch.empty(rows, heads * dv, device=dev, dtype=torch.float32)
            state = torch.zeros(n_seqs, heads * dk * dv * 4, dtype=torch.uint8, device=dev)
            if kind == "linear_attention":
                gate = torch.rand(rows, heads * dk, device=dev) * 0.1 + 0.9     # the decays themselves in a long step
                bias = torch.zeros(heads * dk, device=dev, dtype=bf)
                fn = lambda: K.linear_scan(qq, kk, vv, gate, bias, oo, state, 0, stp, heads, groups, dk, dv, "channel",
                                           q_scale=dk ** -0.5, inv_tau=1 / 8, gate_is_decay=rows > 64)
                gbytes = rows * heads * dk * 4
            else:
                gate = torch.randn(rows, heads, device=dev, dtype=bf)
                bias = torch.zeros(heads, device=dev, dtype=bf)
                al = torch.zeros(heads, device=dev, dtype=bf)
                fn = lambda: K.linear_scan(qq, kk, vv, gate, bias, oo, state, 0, stp, heads, groups, dk, dv, "head", a_log=al, skip=al)
                gbytes = rows * heads * 2
            t = timed(fn, reps=5, graph=True)
            by = rows * (2 * groups * dk * 2 + heads * dv * 2 + heads * dv * 4) + gbytes + 2 * n_seqs * heads * dk * dv * 4
            fl = 4 * rows * heads * dk * dv
            res[f"{what}_{kind}_scan"] = {"ms": round(t * 1e3, 4), "frac_of_bandwidth": round(by / (t * 1e9) / peaks()["hbm_gbs"], 3),
                                          "tflops_fp32": round(fl / t / 1e12, 2), "mb": round(by / 1e6, 2)}
        # the gated norms and the convolution that go with them
        inner = z["sheads"] * z["sp"]
        ch = inner + 2 * z["sg"] * z["sn"]
        x = torch.randn(rows, ch, device=dev, dtype=bf)
        y = torch.empty(rows, ch, device=dev, dtype=bf)
        cw, cb = torch.randn(ch, 4, device=dev, dtype=bf), torch.zeros(ch, device=dev, dtype=bf)
        cstate = torch.zeros(n_seqs, 3 * ch * 4, dtype=torch.uint8, device=dev)
        t = timed(lambda: K.causal_conv(x, y, cw, cb, cstate, 0, stp), reps=9, graph=True)
        res[f"{what}_convolution"] = {"ms": round(t * 1e3, 4), "frac": round(frac(t, 0, rows * ch * 4 + n_seqs * 3 * ch * 8), 3)}
        yy = torch.randn(rows, inner, device=dev)
        gt = torch.randn(rows, inner, device=dev, dtype=bf)
        wv = torch.ones(inner, device=dev, dtype=bf)
        ob = torch.empty(rows, inner, device=dev, dtype=bf)
        t = timed(lambda: K.gated_norm(yy, gt, wv, ob, stp.token_seq, inner // z["sg"], True, 1e-6), reps=9, graph=True)
        res[f"{what}_gated_norm"] = {"ms": round(t * 1e3, 4), "frac": round(frac(t, 0, rows * inner * 8), 3)}
        hres = torch.zeros(rows, Wd, device=dev)
        t = timed(lambda: K.rmsnorm_add(hres, hres, torch.ones(Wd, device=dev, dtype=bf), 1e-6), reps=9, graph=True)
        res[f"{what}_side_norm_add"] = {"ms": round(t * 1e3, 4), "frac": round(frac(t, 0, rows * Wd * 12), 3)}
        xb = torch.empty(rows, Wd, device=dev, dtype=bf)
        t = timed(lambda: K.rmsnorm(hres, torch.ones(Wd, device=dev, dtype=bf), xb, 1e-6), reps=9, graph=True)
        res[f"{what}_side_norm_add"].update(dense_rmsnorm_ms=round(t * 1e3, 4), dense_frac=round(frac(t, 0, rows * Wd * 6), 3))
    return res


# ------------------------------------------------------------------ the Birepel decoder beside the Loduzen one
def birepel_config(z):
    """Attention and matrix-memory layers in turn at the sizes of `LODUZEN_SIZES`: the attention heads of the other
    model's attention, the memory heads of its linear attention, its feed-forward (clamped here), and in the second
    layer eight experts of which two serve a token, sized so that a token's products equal the dense unit's."""
    att = {"heads": z["heads"], "kv_heads": z["kv"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
           "q_temp": {"coef": 0.1, "every": 1024}}
    mem = {"heads": z["lheads"], "dim": z["ldk"], "vdim": z["ldv"], "gate_cap": 15.0}
    dense = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": (3 * z["ff"] // 4) // 64 * 64}, "router": {"experts": 8, "top": 2}}
    layers = []
    for i in range(z["layers"]):
        layers.append({"type": "attention", "mixer": att, "mlp": dense} if i % 2 == 0 else
                      {"type": "mlstm", "mixer": mem, "mlp": moe if i == 1 else dense})
    return {"architecture": "Birepel", "vocab": z["vocab"], "width": z["width"], "max_positions": 16384, "norm": {"eps": 1e-6},
            "layers": layers}


def run_birepel(args):
    """`--birepel`: prompt and decode throughput of the Birepel decoder at sizes like a real model's layers (random
    weights, four layers), beside the Loduzen decoder of equal size (the closest model here: attention with a sink
    beside recurrent layers with a matrix of state), and the new kernels one by one beside that model's like kernels
    with their fractions of the measured peaks.  Prints one JSON line of its own; the default run and its line are
    untouched."""
    import torch
    from braidinfer_b200.engine import Engine
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, reps=5, warm=2, graph=False):
        for _ in range(warm):
            fn()
        run = fn
        if graph:
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            run = gr.replay
            run()
        ts = []
        for _ in range(reps):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / 1e3)
        return statistics.median(ts)

    def frac(seconds, flops, nbytes):
        return max(flops / (pk["bf16_tflops"] * 1e12), nbytes / (pk["hbm_gbs"] * 1e9)) / seconds

    T, B, C = args.prompt_len, args.batch, args.context
    sizes = [n for n in LODUZEN_SIZES if not args.sizes or n in args.sizes.split(",")]
    out = {"metric": "birepel_beside_loduzen_decoder", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic, random weights",
           "prompt_len": T, "decode_batch": B, "decode_context": C, "peaks": pk, "l2": "flushed between timed calls", "sizes": {}}
    with ClockSampler() as clocks:
        for name in sizes:
            z = LODUZEN_SIZES[name]
            row = {}
            for label, cfg in (("birepel", birepel_config(z)), ("loduzen", loduzen_config(z))):
                eng = Engine.from_random(cfg, 1, dtype="bfloat16", on_device=True, max_tokens=max(B * (C + 192), T + 64),
                                         max_slots=B, verbose=False)
                g = torch.Generator().manual_seed(0)
                prompt = torch.randint(0, z["vocab"], (T,), generator=g).tolist()

                def prefill():
                    s = eng.open()
                    eng.step([(s, prompt)], want="last")
                    eng.close(s)
                tp = timed(prefill, reps=3, warm=2)
                prompts = [torch.randint(0, z["vocab"], (C,), generator=g).tolist() for _ in range(B)]
                secs, ctx0, launches = device_timed_decode(eng, eng.kernels, prompts, args.steps, max(args.warmup, 3))
                eng.check()
                row[label] = {"prefill_tokens_per_s": round(T / tp), "prefill_ms": round(tp * 1e3, 3),
                              "decode_tokens_per_s": round(B * args.steps / secs), "decode_ms_per_step": round(secs / args.steps * 1e3, 4),
                              "weight_gb": round(eng.weight_bytes / 1e9, 3), "state_mb_per_sequence": round(sum(
                                  s.shape[1] for s in eng.cache.state if s is not None) / 1e6, 3),
                              "launches_per_decode_step": launches // args.steps}
                del eng
                torch.cuda.empty_cache()
            row["kernels"] = birepel_kernels(z, T, B, C, timed, frac)
            out["sizes"][name] = row
    out["clocks"] = clocks.summary()
    print(json.dumps(out))
    return 0


def birepel_kernels(z, T, B, C, timed, frac):
    """The new kernels alone, each beside the Loduzen decoder's like kernel: seconds, and the fraction of the measured
    peak that its algorithmic FLOPs or bytes (whichever bounds it) reach.  The recurrences run on the ordinary float32
    pipes: their `frac` is of the copy bandwidth (the bytes they must move), and `tflops` says what they compute."""
    import torch
    from types import SimpleNamespace
    from braidinfer_b200.cache import PAGE_SIZE
    from braidinfer_b200.csrc.api import get_kernels
    K = get_kernels(verbose=False)
    dev, bf = "cuda", torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    H, nkh, hd, Wd, win = z["heads"], z["kv"], z["dim"], z["width"], z["window"]
    hbm = peaks()["hbm_gbs"]
    res = {}

    def paged(n_seqs, length):
        blocks = -(-length // PAGE_SIZE)
        cache = torch.randn(n_seqs * blocks, 2, nkh, PAGE_SIZE, hd, device=dev, dtype=bf) * 0.5
        table = torch.arange(n_seqs * blocks, dtype=torch.int32, device=dev).view(n_seqs, blocks)
        return cache, table

    def steps_of(n_seqs, each, before):
        rows = n_seqs * each
        return SimpleNamespace(rows=rows, n_tokens=rows, n_seqs=n_seqs, q_start=i32([i * each for i in range(n_seqs)]),
                               q_len=i32([each] * n_seqs), kv_before=i32([before] * n_seqs), slot_ids=i32(list(range(n_seqs))), max_q_len=each,
                               token_seq=torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(each),
                               positions=(torch.arange(each, dtype=torch.int32, device=dev) + before).repeat(n_seqs))

    st, sd = steps_of(1, T, 0), steps_of(B, 1, C - 1)
    sinks = torch.randn(H, device=dev)

    # ---- attention over a prompt of T tokens: a sink and a gate a head (no window) beside one sink for all (windowed)
    cache, table = paged(1, T)
    q = torch.randn(T, H * hd + 64, device=dev, dtype=bf) * 0.3
    gate = q[:, H * hd:H * hd + H]
    o = torch.empty(T, H * hd, device=dev, dtype=bf)
    fl_full = 2 * 2 * H * hd * (T * (T + 1) // 2)
    fl_win = 2 * 2 * H * hd * sum(min(p + 1, win) for p in range(T))
    row = {}
    for label, kw, w, fl in (("birepel", dict(head_sinks=sinks, head_gate=gate), None, fl_full),
                             ("loduzen", dict(sink=0.0, out_scale=1.2), win, fl_win)):
        t = timed(lambda: K.attn_mma(q, o, cache, table, st.q_start, st.q_len, st.kv_before, st.token_seq, 1, T, H, nkh, hd, w,
                                     hd ** -0.5, **kw), graph=True)
        row.update({label + "_mma_ms": round(t * 1e3, 3), label + "_mma_frac": round(frac(t, fl, 0), 3)})
        if K.attn_tc_supports(hd):
            t = timed(lambda: K.attn_tc(q, o, cache, table, st.q_start, st.q_len, st.kv_before, 1, T, H, nkh, hd, w, hd ** -0.5, **kw),
                      graph=True)
            row.update({label + "_tcgen05_ms": round(t * 1e3, 3), label + "_tcgen05_frac": round(frac(t, fl, 0), 3)})
    res["prompt_attention"] = row

    # ---- attention of B decoded tokens over a context of C (Loduzen's window caps what it reads)
    cache, table = paged(B, C)
    qd = torch.randn(B, H * hd + 64, device=dev, dtype=bf) * 0.3
    gd = qd[:, H * hd:H * hd + H]
    od = torch.empty(B, H * hd, device=dev, dtype=bf)
    g = H // nkh
    row = {}
    for label, kw, w in (("birepel", dict(head_sinks=sinks, head_gate=gd), None), ("loduzen", dict(sink=0.0), win)):
        span = min(C, w) if w else C
        sp = max(1, min(K.attn_decode_slots(hd) // (B * nkh * -(-g // 16)), (span // 32) // 4, 64))
        by = B * span * 2 * nkh * hd * 2
        t = timed(lambda: K.attn_mma(qd, od, cache, table, sd.q_start, sd.q_len, sd.kv_before, sd.token_seq, B, 1, H, nkh, hd, w,
                                     hd ** -0.5, n_splits=sp, few_tokens=True, **kw), reps=9, graph=True)
        row.update({label + "_ms": round(t * 1e3, 4), label + "_frac": round(frac(t, 0, by), 3), label + "_slices": sp})
    res["decode_attention"] = row

    # ---- unit heads + temperature + cache write (one kernel) beside Loduzen's norm of heads + rotation + cache write
    inv = torch.rand(hd // 4, device=dev)
    wn = torch.ones(hd, device=dev, dtype=bf)
    for what, stp, n_seqs, length in (("prompt_prep", st, 1, T), ("decode_prep", sd, B, C)):
        cache, table = paged(n_seqs, length)
        rows = stp.rows
        src = torch.randn(rows, (H + 2 * nkh) * hd + 64, device=dev, dtype=bf)
        qo = torch.empty(rows, H * hd, device=dev, dtype=bf)
        qk = torch.randn(rows, (H + nkh) * hd, device=dev, dtype=bf)
        t1 = timed(lambda: K.head_prep_kv(src, qo, stp.positions, stp.token_seq, table, cache, H, nkh, hd, hd, hd, True, 1e-6, 0.1, 1024),
                   reps=9, graph=True)
        t2 = timed(lambda: K.head_norm_rope_kv(qk, wn, wn, inv, stp.positions, stp.token_seq, table, cache, H, nkh, hd, hd // 2, True,
                                               True, PAGE_SIZE, 1e-6, 1.1), reps=9, graph=True)
        by1 = rows * hd * 2 * (2 * H + 4 * nkh)                  # heads read, queries and two cache planes written
        by2 = rows * hd * 2 * (2 * (H + nkh) + 2 * nkh)
        res[what] = {"birepel_ms": round(t1 * 1e3, 4), "birepel_frac": round(frac(t1, 0, by1), 3),
                     "loduzen_ms": round(t2 * 1e3, 4), "loduzen_frac": round(frac(t2, 0, by2), 3)}

    # ---- the recurrences: the matrix memory (decays and key factors given, a normaliser as one more column) beside
    # gated linear attention (a decay per channel) at the same heads and sizes; with them the gates and the read-outs
    heads, dk, dv = z["lheads"], z["ldk"], z["ldv"]
    for what, stp in (("prompt", st), ("decode", sd)):
        rows, n_seqs = stp.rows, stp.n_seqs
        qq = torch.randn(rows, heads * dk, device=dev, dtype=bf) * 0.1
        kk = torch.randn(rows, heads * dk, device=dev, dtype=bf) * 0.1
        vv = torch.randn(rows, heads * dv, device=dev, dtype=bf)
        bias = torch.zeros(heads * dk, device=dev, dtype=bf)
        # the memory
        m_off = heads * dk * (dv + 1) * 4
        state = torch.zeros(n_seqs, m_off + heads * 4, dtype=torch.uint8, device=dev)
        zz = torch.randn(rows, 2 * heads, device=dev) * 2
        zz[:, heads:] += 4.0
        gates = torch.empty(rows, 3 * heads, device=dev)
        bi = torch.zeros(heads, device=dev, dtype=bf)
        t = timed(lambda: K.mlstm_gates(zz, bi, bi, gates, state, m_off, stp, heads, 15.0), reps=9, graph=True)
        res[f"{what}_memory_gates"] = {"ms": round(t * 1e3, 4), "mb": round(rows * heads * 20 / 1e6, 3),
                                       "frac": round(frac(t, 0, rows * heads * 20), 4)}
        K.mlstm_gates(zz, bi, bi, gates, state, m_off, stp, heads, 15.0)
        oo = torch.empty(rows, heads * (dv + 1), device=dev)
        t = timed(lambda: K.linear_scan(qq, kk, vv, gates[:, :heads], bi, oo, state, 0, stp, heads, heads, dk, dv + 1, "given",
                                        q_scale=dk ** -0.5, kappa=gates[:, heads:2 * heads], v_cols=dv), reps=5, graph=True)
        by = rows * (2 * heads * dk * 2 + heads * dv * 2 + heads * (dv + 1) * 4 + heads * 8) + 2 * n_seqs * heads * dk * (dv + 1) * 4
        fl = 4 * rows * heads * dk * (dv + 1)
        res[f"{what}_memory_scan"] = {"ms": round(t * 1e3, 4), "frac_of_bandwidth": round(by / (t * 1e9) / hbm, 3),
                                      "tflops_fp32": round(fl / t / 1e12, 2), "mb": round(by / 1e6, 2)}
        # Loduzen's gated linear attention
        state2 = torch.zeros(n_seqs, heads * dk * dv * 4, dtype=torch.uint8, device=dev)
        gate = torch.rand(rows, heads * dk, device=dev) * 0.1 + 0.9
        o2 = torch.empty(rows, heads * dv, device=dev)
        t = timed(lambda: K.linear_scan(qq, kk, vv, gate, bias, o2, state2, 0, stp, heads, heads, dk, dv, "channel",
                                        q_scale=dk ** -0.5, inv_tau=1 / 8, gate_is_decay=rows > 64), reps=5, graph=True)
        by = rows * (2 * heads * dk * 2 + heads * dv * 2 + heads * dv * 4 + heads * dk * 4) + 2 * n_seqs * heads * dk * dv * 4
        fl = 4 * rows * heads * dk * dv
        res[f"{what}_memory_scan"].update(loduzen_ms=round(t * 1e3, 4), loduzen_frac_of_bandwidth=round(by / (t * 1e9) / hbm, 3),
                                          loduzen_tflops_fp32=round(fl / t / 1e12, 2))
        # the read-outs: floor, unit norm a head, weight and gate beside Loduzen's gated norm
        inner = heads * dv
        gt = torch.randn(rows, inner, device=dev, dtype=bf)
        wv = torch.ones(inner, device=dev, dtype=bf)
        ob = torch.empty(rows, inner, device=dev, dtype=bf)
        t1 = timed(lambda: K.mlstm_out(oo, gates[:, 2 * heads:], gt, wv, ob, stp.token_seq, heads, dv, 1e-6), reps=9, graph=True)
        yy = torch.randn(rows, inner, device=dev)
        t2 = timed(lambda: K.gated_norm(yy, gt, wv, ob, stp.token_seq, dv, True, 1e-6), reps=9, graph=True)
        res[f"{what}_memory_read_out"] = {"birepel_ms": round(t1 * 1e3, 4), "birepel_frac": round(frac(t1, 0, rows * (inner * 8 + heads * 8)), 3),
                                          "loduzen_ms": round(t2 * 1e3, 4), "loduzen_frac": round(frac(t2, 0, rows * inner * 8), 3)}
        # the clamped gated unit beside the plain one
        I = z["ff"]
        gu = torch.randn(rows, 2 * I, device=dev, dtype=bf)
        ao = torch.empty(rows, I, device=dev, dtype=bf)
        t1 = timed(lambda: K.glu_clamp(gu, ao, 7.0, 1.702), reps=9, graph=True)
        t2 = timed(lambda: K.silu_mul(gu, ao), reps=9, graph=True)
        res[f"{what}_gated_unit"] = {"birepel_ms": round(t1 * 1e3, 4), "birepel_frac": round(frac(t1, 0, rows * I * 6), 3),
                                     "loduzen_ms": round(t2 * 1e3, 4), "loduzen_frac": round(frac(t2, 0, rows * I * 6), 3)}
        # the norm of what a sublayer returned, added to the stream (zero-centred weight) beside Loduzen's norm and sum
        hres, ysub = torch.zeros(rows, Wd, device=dev), torch.randn(rows, Wd, device=dev)
        w1 = torch.zeros(Wd, device=dev, dtype=bf)
        t1 = timed(lambda: K.rmsnorm_add(hres, ysub, w1, 1e-6, w_offset=1.0), reps=9, graph=True)
        t2 = timed(lambda: K.rmsnorm_add(hres, ysub, w1, 1e-6), reps=9, graph=True)
        res[f"{what}_norm_add"] = {"birepel_ms": round(t1 * 1e3, 4), "birepel_frac": round(frac(t1, 0, rows * Wd * 12), 3),
                                   "loduzen_ms": round(t2 * 1e3, 4), "loduzen_frac": round(frac(t2, 0, rows * Wd * 12), 3)}
        # embedding with a learned position beside the embedding alone
        tab = torch.randn(z["vocab"], Wd, device=dev, dtype=bf)
        ptab = torch.randn(max(T, C) + 8, Wd, device=dev, dtype=bf)
        ids = torch.randint(0, z["vocab"], (rows,), device=dev, dtype=torch.int32)
        eo = torch.empty(rows, Wd, device=dev)
        t1 = timed(lambda: K.embed(tab, ids, eo, 1.0, pos_table=ptab, positions=stp.positions), reps=9, graph=True)
        t2 = timed(lambda: K.embed(tab, ids, eo, 1.0), reps=9, graph=True)
        res[f"{what}_embedding"] = {"birepel_ms": round(t1 * 1e3, 4), "birepel_frac": round(frac(t1, 0, rows * Wd * 8), 3),
                                    "loduzen_ms": round(t2 * 1e3, 4), "loduzen_frac": round(frac(t2, 0, rows * Wd * 6), 3)}
        # experts without gates (squared relu) beside gated experts on the same plan: the first product of both
        E, top, J = 8, 2, (3 * z["ff"] // 4) // 64 * 64
        x = torch.randn(rows, Wd, device=dev, dtype=bf) * 0.1
        wu = torch.randn(E, J, Wd, device=dev, dtype=bf) * 0.02
        wg = torch.randn(E, J, Wd, device=dev, dtype=bf) * 0.02
        lg = torch.randn(rows, E, device=dev)
        idx = torch.empty(rows, top, dtype=torch.int32, device=dev)
        wgt = torch.empty(rows, top, device=dev)
        K.moe_route(lg, idx, wgt, 1, 1)
        tile = 16 if rows * top <= 16 * E else 64
        plan = K.moe_plan(idx, stp.token_seq, E, tile)
        act = torch.empty(plan[4] * tile, J, device=dev, dtype=bf)
        t1 = timed(lambda: K.moe_gemm_mma(x, wu, None, act, plan, top, tile, relu2=True), reps=5, graph=True)
        t2 = timed(lambda: K.moe_gemm_mma(x, wg, wu, act, plan, top, tile), reps=5, graph=True)
        used = min(E, rows * top)
        res[f"{what}_experts_first_product"] = {
            "birepel_ms": round(t1 * 1e3, 4), "birepel_frac": round(frac(t1, 2 * rows * top * J * Wd, used * J * Wd * 2), 3),
            "gated_ms": round(t2 * 1e3, 4), "gated_frac": round(frac(t2, 4 * rows * top * J * Wd, 2 * used * J * Wd * 2), 3)}
    K.check_device_errors()
    return res


# ------------------------------------------------------------------ the Ludazen decoder beside the Bidinex one
def ludazen_config(z):
    """Attention and latent layers in turn at the sizes of `BIDINEX_SIZES`: the latent layers are the other model's
    (behind a window, without gates), the second of them reads the first one's latent; the attention layers have its
    head count, a kv head for four heads, heads as large as a latent head's query, a window of 1,024 with four kept
    tokens; the experts are the other model's (chosen by sigmoid scores, beside a shared one of an expert's size), the
    dense feed-forward is as wide as the experts a token uses."""
    hd = 128 if z["dim"] + z["rot"] > 64 else 64
    att = {"heads": z["heads"], "kv_heads": max(1, z["heads"] // 4), "dim": hd, "vdim": hd, "scale": hd ** -0.5,
           "rot": {"base": 10000.0, "dims": hd, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
           "mask": {"size": 1024, "keep_first": 4}}
    lat = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "rot": {"base": 10000.0, "dims": z["rot"]},
           "vdim": z["vdim"], "kv_rank": z["rank"], "scale": (z["dim"] + z["rot"]) ** -0.5, "mask": {"size": 1024}}
    moe = {"kind": "moe", "expert": {"ff": z["ff"]}, "router": {"experts": z["experts"], "top": z["top"]}, "shared": {"ff": z["ff"]}}
    dense = {"kind": "dense", "ff": z["top"] * z["ff"]}
    layers, owner = [], None
    for i in range(z["layers"]):
        if i % 2 == 0:
            layers.append({"type": "attention", "mixer": att, "mlp": dense if i % 4 == 0 else moe})
        else:
            layers.append({"type": "latent_attention", "mixer": dict(lat, **({"kv_from": owner} if owner is not None else {})),
                           "mlp": moe if owner is None else dense})
            owner = i if owner is None else owner
    return {"architecture": "Ludazen", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "layers": layers}


def run_ludazen(args):
    """`--ludazen`: prompt and decode throughput of the Ludazen decoder at sizes like a real model's layers (random
    weights, four layers), beside the Bidinex decoder of equal size (the closest model here: latent attention and a
    mixture of experts), and the new kernels and kernel options one by one beside the like kernels that the other
    models run, with their fractions of the measured peaks.  Prints one JSON line of its own; the default run and
    its line are untouched."""
    import torch
    from braidinfer_b200.engine import Engine
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, reps=5, warm=2, graph=False):
        for _ in range(warm):
            fn()
        run = fn
        if graph:
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            run = gr.replay
            run()
        ts = []
        for _ in range(reps):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / 1e3)
        return statistics.median(ts)

    def frac(seconds, flops, nbytes):
        return max(flops / (pk["bf16_tflops"] * 1e12), nbytes / (pk["hbm_gbs"] * 1e9)) / seconds

    T, B, C = args.prompt_len, args.batch, args.context
    sizes = [n for n in BIDINEX_SIZES if not args.sizes or n in args.sizes.split(",")]
    out = {"metric": "ludazen_beside_bidinex_decoder", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic, random weights",
           "prompt_len": T, "decode_batch": B, "decode_context": C, "peaks": pk, "l2": "flushed between timed calls", "sizes": {}}
    with ClockSampler() as clocks:
        for name in sizes:
            z = BIDINEX_SIZES[name]
            row = {}
            for label, cfg in (("ludazen", ludazen_config(z)), ("bidinex", bidinex_config(z))):
                eng = Engine.from_random(cfg, 1, dtype="bfloat16", on_device=True, max_tokens=max(B * (C + 192), T + 64),
                                         max_slots=B, verbose=False)
                g = torch.Generator().manual_seed(0)
                prompt = torch.randint(0, z["vocab"], (T,), generator=g).tolist()

                def prefill():
                    s = eng.open()
                    eng.step([(s, prompt)], want="last")
                    eng.close(s)
                tp = timed(prefill, reps=3, warm=2)
                prompts = [torch.randint(0, z["vocab"], (C,), generator=g).tolist() for _ in range(B)]
                secs, ctx0, launches = device_timed_decode(eng, eng.kernels, prompts, args.steps, max(args.warmup, 3))
                eng.check()
                row[label] = {"prefill_tokens_per_s": round(T / tp), "prefill_ms": round(tp * 1e3, 3),
                              "decode_tokens_per_s": round(B * args.steps / secs), "decode_ms_per_step": round(secs / args.steps * 1e3, 4),
                              "weight_gb": round(eng.weight_bytes / 1e9, 3), "cache_mb": round(eng.cache.nbytes() / 1e6, 1),
                              "launches_per_decode_step": launches // args.steps}
                del eng
                torch.cuda.empty_cache()
            row["kernels"] = ludazen_kernels(z, T, B, C, timed, frac)
            out["sizes"][name] = row
    out["clocks"] = clocks.summary()
    print(json.dumps(out))
    return 0


def ludazen_kernels(z, T, B, C, timed, frac):
    """The new kernels and options alone, each beside the like kernel of another model: seconds, and the fraction of
    the measured peak that its algorithmic FLOPs or bytes (whichever bounds it) reach.  The attention whose heads'
    probabilities are mixed is charged with the FLOPs of the design (scores and values once a head); what its kernels
    compute beyond that (the values of every kv head a query head) shows as a lower fraction."""
    import torch
    from types import SimpleNamespace
    from braidinfer_b200.cache import PAGE_SIZE
    from braidinfer_b200.csrc.api import get_kernels
    K = get_kernels(verbose=False)
    dev, bf = "cuda", torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)        # noqa: E731
    H, Wd, E, top, ff, R, rot = z["heads"], z["width"], z["experts"], z["top"], z["ff"], z["rank"], z["rot"]
    hd = 128 if z["dim"] + z["rot"] > 64 else 64
    nkh, win, keep, D = max(1, H // 4), 1024, 4, R + rot
    res = {}

    def paged(n_seqs, length, planes, heads, dim):
        blocks = -(-length // PAGE_SIZE)
        cache = torch.randn(n_seqs * blocks, planes, heads, PAGE_SIZE, dim, device=dev, dtype=bf) * 0.5
        table = torch.arange(n_seqs * blocks, dtype=torch.int32, device=dev).view(n_seqs, blocks)
        return cache, table

    def steps_of(n_seqs, each, before):
        return SimpleNamespace(q_start=i32([i * each for i in range(n_seqs)]), q_len=i32([each] * n_seqs),
                               kv_before=i32([before] * n_seqs),
                               token_seq=torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(each))

    temp, talk = torch.rand(H, device=dev) + 0.5, (torch.randn(H, H, device=dev) * 0.3).to(bf)
    # ---- attention over a prompt and of decoded tokens: heads mixed after the softmax (every query head over the values
    # of every kv head, then the mix) beside the plain windowed attention of the same heads
    for what, n_seqs, each, before in (("prompt_attention", 1, T, 0), ("decode_attention", B, 1, C - 1)):
        st = steps_of(n_seqs, each, before)
        rows = n_seqs * each
        cache, table = paged(n_seqs, before + each, 2, nkh, hd)
        q = torch.randn(rows, (H + 2 * nkh) * hd, device=dev, dtype=bf) * 0.3
        wide = torch.empty(rows, H * nkh * hd, device=dev, dtype=bf)
        o = torch.empty(rows, H * hd, device=dev, dtype=bf)
        few = each <= 8
        seen = sum(min(p + 1, win) + min(keep, max(p + 1 - win, 0)) for p in range(before, before + each)) * n_seqs
        fl = 2 * 2 * H * hd * seen
        nbytes = n_seqs * min(before + each, win + keep) * nkh * 2 * hd * 2
        sp = sp1 = 1
        if few:
            ctas = n_seqs * nkh * -(-(H // nkh) // 16)
            tiles = max(1, (min(before + each, win + keep)) // 32)
            sp = max(1, min(K.attn_decode_slots(hd, nkh) // (ctas * (nkh // K.attn_value_heads_a_launch(hd, nkh))), tiles // 4, 64))
            sp1 = max(1, min(K.attn_decode_slots(hd) // ctas, tiles // 4, 64))

        def mixed():
            K.attn_mma(q, wide, cache, table, st.q_start, st.q_len, st.kv_before, st.token_seq, n_seqs, each, H, nkh, hd, win,
                       hd ** -0.5, n_splits=sp, few_tokens=few, keep_first=keep, head_scale=temp, value_heads=nkh)
            K.head_mix(wide, talk, o, st.token_seq, H, nkh, hd, hd)
        t1 = timed(mixed, graph=True)
        t1a = timed(lambda: K.head_mix(wide, talk, o, st.token_seq, H, nkh, hd, hd), graph=True)
        t2 = timed(lambda: K.attn_mma(q, o, cache, table, st.q_start, st.q_len, st.kv_before, st.token_seq, n_seqs, each, H, nkh, hd,
                                      win, hd ** -0.5, n_splits=sp1, few_tokens=few), graph=True)
        res[what] = {"mixed_heads_ms": round(t1 * 1e3, 4), "mixed_heads_frac": round(frac(t1, fl, nbytes), 3),
                     "of_which_mix_ms": round(t1a * 1e3, 4),
                     "mix_frac": round(frac(t1a, 0, rows * (H * nkh * hd + H * hd) * 2), 3),
                     "plain_window_ms": round(t2 * 1e3, 4), "plain_window_frac": round(frac(t2, fl, nbytes), 3),
                     "groups_of_value_heads": nkh // K.attn_value_heads_a_launch(hd, nkh), "slices": sp}
    # ---- latent attention behind a window beside the same kernel over the whole context (the Bidinex layer)
    for what, n_seqs, each, before in (("prompt_latent_attention", 1, T, 0), ("decode_latent_attention", B, 1, C - 1)):
        st = steps_of(n_seqs, each, before)
        rows = n_seqs * each
        cache, table = paged(n_seqs, before + each, 1, 1, D)
        q = torch.randn(rows, H, D, device=dev, dtype=bf) * 0.3
        o = torch.empty(rows, H, R, device=dev, dtype=bf)
        row = {}
        for label, w in (("window", win), ("whole", None)):
            span = min(before + each, w) if w else before + each
            sp = 1
            if each <= 8:
                sp = max(1, min(296 // K.attn_latent_ctas(R, rot, n_seqs, each, H), (span // 32) // 4, 32))
            t = timed(lambda: K.attn_latent_mma(q, o, cache, table, st.q_start, st.q_len, st.kv_before, st.token_seq, n_seqs, each, R, w,
                                                0.1, n_splits=sp), graph=True)
            seen = sum(min(p + 1, w) if w else p + 1 for p in range(before, before + each)) * n_seqs
            row.update({label + "_ms": round(t * 1e3, 4), label + "_frac": round(frac(t, 2 * H * (D + R) * seen, n_seqs * span * D * 2), 3)})
        res[what] = row
    # ---- the experts' first products with the weight on their input beside the same without, and routing
    for what, rows in (("prompt_experts", T), ("decode_experts", B)):
        x = torch.randn(rows, Wd, device=dev, dtype=bf) * 0.3
        wg, wu = [torch.randn(E, ff, Wd, device=dev, dtype=bf) * 0.02 for _ in range(2)]
        logits = torch.randn(rows, E, device=dev)
        idx = torch.empty(rows, top, dtype=torch.int32, device=dev)
        wgt = torch.empty(rows, top, dtype=torch.float32, device=dev)
        tr1 = timed(lambda: K.moe_route(logits, idx, wgt, 1, 1, sigmoid=True), graph=True)
        tr2 = timed(lambda: K.moe_route(logits, idx, wgt, 1, 1), graph=True)
        tile = 16 if rows * top <= 16 * E else 64
        plan = K.moe_plan(idx, torch.zeros(rows, dtype=torch.int32, device=dev), E, tile)
        act = torch.empty(plan[4] * tile, ff, device=dev, dtype=bf)
        t1 = timed(lambda: K.moe_gemm_mma(x, wg, wu, act, plan, top, tile, in_wgt=wgt), graph=True)
        t2 = timed(lambda: K.moe_gemm_mma(x, wg, wu, act, plan, top, tile), graph=True)
        used = int(torch.unique(idx).numel())
        fl1, by1 = 2 * rows * top * 2 * ff * Wd, used * 2 * ff * Wd * 2
        res[what] = {"weighted_input_ms": round(t1 * 1e3, 4), "weighted_input_frac": round(frac(t1, fl1, by1), 3),
                     "weighted_output_ms": round(t2 * 1e3, 4), "weighted_output_frac": round(frac(t2, fl1, by1), 3),
                     "route_sigmoid_ms": round(tr1 * 1e3, 4), "route_softmax_ms": round(tr2 * 1e3, 4), "experts_used": used, "tile": tile}
        del wg, wu
    # ---- bias + two-piece activation (with the ones column) beside the gated unit's activation kernel
    I = top * ff
    for what, rows in (("prompt_activation", T), ("decode_activation", B)):
        zz = torch.randn(rows, 2 * I, device=dev, dtype=bf)
        bias, pq = torch.randn(I, device=dev, dtype=bf), torch.tensor([0.3, -0.2], device=dev, dtype=bf)
        a1 = torch.empty(rows, I + 8, device=dev, dtype=bf)
        a2 = torch.empty(rows, I, device=dev, dtype=bf)
        t1 = timed(lambda: K.bias_xielu(zz[:, :I], bias, pq, a1, I), graph=True)
        t2 = timed(lambda: K.act_mul(zz, a2, "silu"), graph=True)
        res[what] = {"bias_xielu_ms": round(t1 * 1e3, 4), "bias_xielu_frac": round(frac(t1, 0, rows * I * 4), 3),
                     "gated_silu_ms": round(t2 * 1e3, 4), "gated_silu_frac": round(frac(t2, 0, rows * I * 6), 3)}
    return res


def run_reference(args):
    print(json.dumps({"impl": "reference", "unavailable":
                      "mcelrath/braidinfer is Rust + HIP for AMD RDNA3: pip finds neither setup.py nor pyproject.toml, "
                      "and this image has no cargo, rustc, hipcc or ROCm"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--quick", action="store_true",
                    help="a small case for profilers: 4 layers unless --layers says otherwise, a cache for this batch "
                         "only, no batch-1/64 points and no end-to-end run; the number it prints is not a bench value")
    ap.add_argument("--no-graphs", action="store_true", help="launch every step kernel by kernel")
    ap.add_argument("--preset", default="mistral_7b_v03",
                    choices=["mistral_7b_v03", "mistral_7b_v01", "mistral_nemo_12b"],
                    help="the default is the headline run; the other two print their own line (see run_other_size)")
    ap.add_argument("--sweep", action="store_true",
                    help="decode over batch and context, prefill over prompt length; prints its own line (see run_sweep)")
    ap.add_argument("--chain", action="store_true",
                    help="what chains of decode-step kernels cost, with phase time stamps under BRAIDINFER_TRACE=1 "
                         "(see run_chain)")
    ap.add_argument("--prompt-timeline", default="", metavar="T1,T2,...",
                    help="a prompt step of each length under the torch profiler: a layer's kernels with their share "
                         "(see run_prompt_timeline)")
    ap.add_argument("--timeline", action="store_true",
                    help="one decode step under the torch profiler: a layer's kernels with their share (see run_timeline)")
    ap.add_argument("--bidinex", action="store_true",
                    help="the Bidinex decoder at sizes like a real model's layers beside the dense decoder of equal size, "
                         "and its kernels one by one; prints its own line (see run_bidinex)")
    ap.add_argument("--loduzen", action="store_true",
                    help="the Loduzen decoder (attention beside linear attention, state-space layers) beside the dense "
                         "decoder of equal size, and its kernels one by one; prints its own line (see run_loduzen)")
    ap.add_argument("--birepel", action="store_true",
                    help="another measurement: the Birepel decoder at sizes like a real model's layers beside the Loduzen "
                         "decoder of equal size, and its kernels one by one; prints its own line (see run_birepel)")
    ap.add_argument("--ludazen", action="store_true",
                    help="another measurement: the Ludazen decoder at sizes like a real model's layers beside the Bidinex "
                         "decoder of equal size, and its kernels one by one; prints its own line (see run_ludazen)")
    ap.add_argument("--sizes", default="", help="with --bidinex / --loduzen / --birepel / --ludazen: names of the sizes, with commas (default: all)")
    ap.add_argument("--prompt-len", type=int, default=2048, help="with --bidinex: tokens of the timed prompt")
    ap.add_argument("--context", type=int, default=2048, help="with --bidinex: context of the timed decode steps")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.bidinex:
        return run_bidinex(args)
    if args.loduzen:
        return run_loduzen(args)
    if args.birepel:
        return run_birepel(args)
    if args.ludazen:
        return run_ludazen(args)
    if args.sweep:
        return run_sweep(args)
    if args.prompt_timeline:
        return run_prompt_timeline(args)
    if args.timeline:
        return run_timeline(args)
    if args.chain:
        return run_chain(args)
    if args.preset != "mistral_7b_v03":
        return run_other_size(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
