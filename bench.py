#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

    python bench.py --shape tinyllama|llama2-7b|llama3-8b [--layers L]

    python bench.py --design murilorn [--size 2k,4k]    (likewise for the third architecture)
    python bench.py --design luvapel [--size 2k,4k]     (the fourth, beside the third)
    python bench.py --design midulorn [--size 2k,4k]    (the fifth, beside the third)
    python bench.py --design kavenex [--size 2k,4k]     (a JSON line of its own: the second architecture
                                                         beside Llama at equal sizes, kernel beside like kernel)

A step is one decode step: every live request advances by one token. The default
run has the layer sizes of TinyLlama-1.1B with random weights, 8 requests and a
context of 2,048 tokens; ``--shape`` chooses another of the reference's published
shapes. Times are taken with CUDA events on the launching stream, after warm-up,
with a synchronize on both sides of the timed region and an event after every
step inside it (so that the median step is known beside the mean). Nothing
flushes L2 between steps: a decode step reads every weight once (gigabytes), far
more than L2 holds. The end-to-end figure goes through ``Engine.generate`` with
token ids coming from and going back to the host every step. Fractions are
given against the peaks measured on this pool (``MEASURED_PEAKS.json``) and
against the nominal ones. The reference itself runs on the CPU only and cannot be
built here; what stands in for its "CPU seconds" is the plain implementation of
the tests on the smallest published configuration.
"""
from __future__ import annotations

import argparse
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

LLAMA = dict(architectures=["LlamaForCausalLM"], model_type="llama", rms_norm_eps=1e-5, tie_word_embeddings=False)
# layer sizes of the reference's published configurations; `context`: the benchmark's context length
SHAPES = {
    "tinyllama": dict(name="TinyLlama-1.1B shape", context=2048, layers_default=22, config=dict(
        LLAMA, hidden_size=2048, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
        intermediate_size=5632, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=2048)),
    # the larger shapes run with a quarter of their layers by default (the layers are alike; writing and
    # loading 13 to 15 GB of random weights would take minutes): `config` names both numbers
    "llama2-7b": dict(name="Llama-2-7B shape", context=4096, layers_default=8, config=dict(
        LLAMA, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=32, head_dim=128,
        intermediate_size=11008, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096)),
    "llama3-8b": dict(name="Llama-3-8B shape", context=8192, layers_default=8, config=dict(
        LLAMA, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=8192)),
}
# ``--design kavenex``: the Kavenex design beside the Llama decoder at equal width, heads, head size,
# feed-forward size and depth (random weights). Four layers each: Kavenex's are dense, routed, dense,
# routed (a token's `top` experts together as large as the dense feed-forward, plus a shared one).
DESIGN_SIZES = {
    "2k": dict(width=2048, heads=32, dim=32, rot_dim=32, vdim=64, kv_rank=256, ff=5632, experts=16, top=4,
               expert_ff=1408, shared_ff=1408, side=64, vocab=32000, llama_kv_heads=4, scale=0.125),
    "4k": dict(width=4096, heads=32, dim=64, rot_dim=64, vdim=128, kv_rank=512, ff=11008, experts=16, top=4,
               expert_ff=2752, shared_ff=2752, side=64, vocab=32000, llama_kv_heads=8, scale=0.088),
}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
NOMINAL = {"hbm_gbs": 7700.0, "bf16_tflops": 2250.0}     # HBM3e of the HGX B200; dense bfloat16 tensor rate


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])), "measured"
    except Exception:
        return FALLBACK_PEAKS["hbm_gbs"], FALLBACK_PEAKS["bf16_tflops"], "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        """Call at the start and at the end of the timed region."""
        self.marks = getattr(self, "marks", []) + [time.time()]

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        marks = getattr(self, "marks", [])
        lo, hi = (marks[0], marks[-1]) if len(marks) >= 2 else (0.0, float("inf"))

        def collect(inside):
            sm, mx, reasons = [], [], set()
            for when, line in self.lines:
                # a sample is printed up to one period after it was taken
                if inside and not (lo <= when <= hi + 0.06):
                    continue
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, v in zip(names, parts[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            return sorted(sm), mx, reasons

        sm, mx, reasons = collect(True)
        window = "timed region"
        if not sm:       # the region was shorter than the sampling period: the samples around it
            sm, mx, reasons = collect(False)
            window = "decode phase around the timed region"
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def model_bytes_and_flops(cfg, layers, batch, kv_len, itemsize=2):
    d, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (q + 2 * kv) + q * d + 3 * d * ff
    weight_bytes = (layers * per_layer + V * d) * itemsize          # every matrix once; norms are negligible
    cache_bytes = batch * kv_len * layers * 2 * kv * itemsize
    return per_layer, weight_bytes, cache_bytes


def run_ours(args) -> dict:
    import numpy as np
    import torch
    from garuda_b200 import Engine, SamplingParams, StepEntry
    from garuda_b200.weights import write_random_model

    shape = SHAPES[args.shape]
    full_layers = shape["config"]["num_hidden_layers"]
    layers = args.layers or shape["layers_default"]
    context = shape["context"]
    cfg = dict(shape["config"], num_hidden_layers=layers)
    hbm_peak, tflops_peak, peak_kind = peaks()
    K, W = args.steps, args.warmup
    batch = args.batch
    # the cache: 64 requests at a context of at most 2,048 (the 64-request point), or the headline's
    # requests at the shape's own context, whichever is more
    b64_context = min(context, 2048)
    kv_tokens = max(64 * b64_context, batch * context) + 64 * 32
    tmp = tempfile.mkdtemp(prefix="garuda_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    try:
        t0 = time.time()
        write_random_model(tmp, cfg, seed=0, store_dtype=torch.bfloat16)
        print(f"[bench] wrote random weights in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        engine = Engine(tmp, dtype="bfloat16", context=context, page_size=32, kv_tokens=kv_tokens,
                        max_concurrent=64, queue_capacity=256, max_batch_tokens=PREFILL_TOKENS,
                        prefill_chunk=PREFILL_TOKENS, ignore_eos=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    runner, ops = engine.runner, engine.ops
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    ev = lambda: torch.cuda.Event(enable_timing=True)

    if args.only:
        return run_one_phase(args, engine, cfg, rng, context)

    # ---------------------------------------------------------------- prompts in one step
    def prefill(tokens, at=0):
        """Median milliseconds of a step of `tokens` prompt tokens that start at position `at`."""
        toks = rng.integers(0, V, tokens).tolist()
        before = rng.integers(0, V, at).tolist() if at else None
        times = []
        for i in range(3 + 5):
            rid = 1000 + i
            if before:
                for lo in range(0, at, PREFILL_TOKENS):
                    runner.run([StepEntry(rid, before[lo:lo + PREFILL_TOKENS], [])])
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            runner.run([StepEntry(rid, toks, [tokens - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.end(rid)
            if i >= 3:
                times.append(s.elapsed_time(e))
        return sorted(times)[len(times) // 2]

    per_layer, _, _ = model_bytes_and_flops(cfg, layers, 1, 0)

    def prefill_flops(T, at=0):
        keys = T * at + T * (T + 1) // 2
        return 2 * T * layers * per_layer + 2 * V * cfg["hidden_size"] \
            + layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * keys

    def prefill_record(T, ms, at=0):
        rate = prefill_flops(T, at) / (ms * 1e-3)
        return {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(rate / (tflops_peak * 1e12), 4), "tflops": round(rate / 1e12, 1),
                "frac_nominal": round(rate / (NOMINAL["bf16_tflops"] * 1e12), 4)}

    prefill_ms = prefill(PREFILL_TOKENS)
    prefill_rec = prefill_record(PREFILL_TOKENS, prefill_ms)
    points = {}
    if context > PREFILL_TOKENS:
        # the last 2,048 tokens of a prompt as long as the shape's own context
        ms = prefill(PREFILL_TOKENS, at=context - PREFILL_TOKENS)
        points[f"prefill_last_2048_of_{context}_frac"] = prefill_record(PREFILL_TOKENS, ms, context - PREFILL_TOKENS)["frac"]
        points[f"prefill_last_2048_of_{context}_ms"] = round(ms, 3)
    points["prefill_512_ms"] = round(prefill(512), 3)

    # ---------------------------------------------------------------- decode
    def decode(nreq, steps, warmup, ctx_len, sample_clocks=False, beside=0):
        """Requests prefilled so that the last timed step reaches the full context. `beside`: every
        step also carries a prompt portion of that many tokens of another request (a mixed step)."""
        start_len = ctx_len - steps - warmup
        ids = list(range(nreq))
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.start()          # early: nvidia-smi takes a moment to print its first sample
        for r in ids:
            toks = rng.integers(0, V, start_len).tolist()
            for lo in range(0, start_len, PREFILL_TOKENS):
                runner.run([StepEntry(r, toks[lo:lo + PREFILL_TOKENS], [])])
        feed = rng.integers(0, V, (steps + warmup, nreq))
        extra = rng.integers(0, V, beside * (steps + warmup)).tolist() if beside else None
        out = torch.empty(nreq, dtype=torch.int32, device=engine.device)

        def one(i):
            entries = [StepEntry(r, [int(feed[i, j])], [0]) for j, r in enumerate(ids)]
            if beside:
                entries.append(StepEntry(9000, extra[i * beside:(i + 1) * beside], []))
            logits = runner.run(entries)
            ops.argmax(logits, out)
            if beside:
                runner.end(9000)     # the next step's portion starts a prompt again

        for i in range(warmup):
            one(i)
        launches0 = ops.launches
        marks = [ev() for _ in range(steps + 1)]
        torch.cuda.synchronize()
        if sampler:
            sampler.mark()
        marks[0].record()
        for i in range(warmup, warmup + steps):
            one(i)
            marks[i - warmup + 1].record()
        torch.cuda.synchronize()
        if sampler:
            sampler.mark()
            time.sleep(0.06)         # let the sample taken at the end be printed
        clocks = sampler.stop() if sampler else None
        ms = marks[0].elapsed_time(marks[-1]) / steps
        each = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
        launches = ops.launches - launches0 + runner.graphs.launches_replayed(nreq) * (0 if beside else steps)
        for r in ids:
            runner.end(r)
        return ms, each[len(each) // 2], clocks, launches, ctx_len - steps / 2

    ms_b, med_b, clocks, launches, mean_kv = decode(batch, K, W, context, sample_clocks=True)
    _, wbytes, cbytes = model_bytes_and_flops(cfg, layers, batch, mean_kv)
    achieved = (wbytes + cbytes) / (ms_b * 1e-3) / 1e9
    side = min(K, 64)

    def frac_of(nreq, ms, ctx_len):
        _, wb, cb = model_bytes_and_flops(cfg, layers, nreq, ctx_len - side / 2)
        return round((wb + cb) / (ms * 1e-3) / 1e9 / hbm_peak, 4)

    ms1, _, _, _, _ = decode(1, side, W, context)
    ms64, _, _, _, _ = decode(64, side, W, b64_context)
    mixed_ms, _, _, _, _ = decode(8, min(K, 8), W, min(context, 2048), beside=504)
    ops.tc.check_errors()
    points.update({"decode_b1": round(1 / ms1 * 1e3, 1), "decode_b64": round(64 / ms64 * 1e3, 1),
                   "decode_b1_ms": round(ms1, 4), "decode_b64_ms": round(ms64, 4),
                   "decode_b1_hbm_frac": frac_of(1, ms1, context), "decode_b64_hbm_frac": frac_of(64, ms64, b64_context),
                   "decode_b64_context": b64_context, "mixed_step_8_decode_504_prompt_ms": round(mixed_ms, 3)})

    # ---------------------------------------------------------------- end to end through Engine.generate
    prompts = [rng.integers(0, V, context - K - W - 1).tolist() for _ in range(batch)]

    def steady_rate(stamps):
        """Tokens a second while all requests decode together: from the moment the last request to
        start has had its W warm-up tokens (with long prompts the first requests decode beside the
        others' prompt portions for a while) to the moment the first request ends."""
        per = {}
        for i, when in stamps:
            per.setdefault(i, []).append(when)
        if len(per) < batch or min(len(v) for v in per.values()) <= W:
            return 0.0
        t0 = max(v[W - 1] for v in per.values())
        t1 = min(v[-1] for v in per.values())
        inside = sorted(when for _, when in stamps if t0 <= when <= t1)
        return (len(inside) - 1) / (inside[-1] - inside[0]) if len(inside) > 1 and inside[-1] > inside[0] else 0.0

    stamps = []
    engine.warm_up()      # graphs of the smaller batches, which the run's last rounds use as requests end
    engine.generate(prompts, SamplingParams.greedy(max_tokens=K + W), on_token=lambda i, t: stamps.append((i, time.perf_counter())))
    torch.cuda.synchronize()
    e2e_value = steady_rate(stamps)
    cap = runner.graphs.graphs.get(batch)
    h2d = int(cap.pinned.numel() * 4) if cap is not None else 0
    # the same with sampled requests (the reference's default temperature, top-k and top-p), as a point
    stamps_s = []
    engine.generate(prompts, SamplingParams(temperature=0.8, top_k=40, top_p=0.95, max_tokens=K + W, seed=1),
                    on_token=lambda i, t: stamps_s.append((i, time.perf_counter())))
    torch.cuda.synchronize()
    points["e2e_sampled"] = round(steady_rate(stamps_s), 1)
    engine.check_errors()

    return {
        "metric": f"decode tok/s at batch {batch}, context {context} ({shape['name']}, random weights)",
        "value": round(batch / ms_b * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_b, 4), "ms_per_step_median": round(med_b, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0, 0.02) and uniform random token ids",
        "config": {"model": shape["name"], "layers": layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "rope_theta": cfg["rope_theta"],
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied": False, "global_batch": batch, "seq_len": context,
                   "context_at_first_timed_step": context - K, "page_size": 32, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": f"inputs larger than L2 (weights {wbytes / 1e9:.2f} GB per step)",
                   "peaks": peak_kind},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": batch * 4},
        "gpu_launches": int(launches),
        "prefill": prefill_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4), "peak_nominal": NOMINAL["hbm_gbs"],
                     "frac_nominal": round(achieved / NOMINAL["hbm_gbs"], 4)},
        "points": points,
        "cpu_reference": cpu_reference_seconds(),
        "clocks": clocks,
    }


def design_configs(z):
    mixer = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot_dim"], "vdim": z["vdim"], "kv_rank": z["kv_rank"],
             "scale": z["scale"], "rot": {"base": 10000.0, "dims": z["rot_dim"]}}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["expert_ff"], "limit": 7.0},
           "shared": {"ff": z["shared_ff"], "limit": 7.0}}
    kavenex = {"architecture": "Kavenex", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
               "norm": {"eps": 1e-5}, "residual_mult": 0.5, "token_side": {"dim": z["side"]}, "max_positions": 4096,
               "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": m} for m in (dense, moe, dense, moe)]}
    llama = dict(LLAMA, hidden_size=z["width"], num_hidden_layers=4, num_attention_heads=z["heads"],
                 num_key_value_heads=z["llama_kv_heads"], head_dim=z["dim"] + z["rot_dim"], intermediate_size=z["ff"],
                 vocab_size=z["vocab"], rope_theta=10000.0, max_position_embeddings=4096)
    return kavenex, llama


def run_design(args) -> dict:
    """Prefill and decode throughput of the Kavenex design and of the Llama decoder at equal sizes, and
    the design's kernels beside the like kernels of Llama, each against its roofline (the slower of
    bytes / measured copy rate and FLOPs / measured bfloat16 rate)."""
    import numpy as np
    import torch
    from garuda_b200 import Engine, StepEntry
    from garuda_b200.engine.batch import Workspace
    from garuda_b200.weights import write_random_model

    hbm_peak, tflops_peak, peak_kind = peaks()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than L2: written before every timed run

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        return sorted(times)[len(times) // 2]

    def roof(ms, flops=0.0, nbytes=0.0):
        ideal = max(flops / (tflops_peak * 1e12), nbytes / (hbm_peak * 1e9)) * 1e3
        return {"ms": round(ms, 4), "roofline_ms": round(ideal, 4), "frac": round(ideal / ms, 4)}

    out = {"design": "kavenex", "peaks": peak_kind, "hbm_gbs": hbm_peak, "bf16_tflops": tflops_peak, "dtype": "bf16",
           "data": "synthetic", "timing": "CUDA events, 3 warm-up runs, L2 flushed before every timed run, median", "sizes": {}}
    B, CTX, T = 8, 2048, PREFILL_TOKENS
    for name in (args.size.split(",") if args.size else list(DESIGN_SIZES)):
        z = DESIGN_SIZES[name]
        rec = {}
        engines = {}
        for arch, cfg in zip(("kavenex", "llama"), design_configs(z)):
            tmp = tempfile.mkdtemp(prefix="garuda_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
            try:
                write_random_model(tmp, cfg, seed=0, store_dtype=torch.bfloat16)
                engine = Engine(tmp, dtype="bfloat16", context=4096, page_size=32, kv_tokens=B * CTX + 4096 + 64,
                                max_concurrent=B, max_batch_tokens=T, prefill_chunk=T, ignore_eos=True)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            engines[arch] = engine
            runner, rng, V = engine.runner, np.random.default_rng(0), z["vocab"]
            toks = rng.integers(0, V, T).tolist()
            rid = [0]

            def prefill():
                rid[0] += 1
                runner.run([StepEntry(10_000 + rid[0], toks, [T - 1])])
                runner.end(10_000 + rid[0])

            ms = timed(prefill, reps=5)
            rec[arch] = {"prefill_2048_ms": round(ms, 3), "prefill_tok_s": round(T / ms * 1e3)}
            steps = 48
            for r in range(B):
                runner.run([StepEntry(r, rng.integers(0, V, CTX - steps - 8).tolist(), [])])
            feed = rng.integers(0, V, (steps + 8, B))
            for i in range(8):
                runner.run([StepEntry(r, [int(feed[i, r])], [0]) for r in range(B)])
            marks = [ev() for _ in range(steps + 1)]
            torch.cuda.synchronize()
            marks[0].record()
            for i in range(steps):
                runner.run([StepEntry(r, [int(feed[8 + i, r])], [0]) for r in range(B)])
                marks[i + 1].record()
            torch.cuda.synchronize()
            each = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
            for r in range(B):
                runner.end(r)
            rec[arch].update({"decode_b8_ctx2048_ms": round(each[len(each) // 2], 4),
                              "decode_tok_s": round(B / each[len(each) // 2] * 1e3),
                              "graph_replays": runner.graphs.replays})
            if engine.ops.tc is not None:
                engine.ops.tc.check_errors()
        # ------------------------------------------------------------ kernel beside like kernel
        ops = engines["kavenex"].ops
        bf = torch.bfloat16
        H, rank, rot, dn, dv, W = z["heads"], z["kv_rank"], z["rot_dim"], z["dim"], z["vdim"], z["width"]
        row, hd, Hkv, ps = rank + rot, z["dim"] + z["rot_dim"], z["llama_kv_heads"], 32
        ws = Workspace(dev)

        class Ctx:
            pass
        ctx = Ctx()
        ctx.ws = ws
        ctx.step_cache = {}
        kern = {}

        def paged(nreq, q_len, kv_len, heads, width, pools):
            pages = (kv_len + ps - 1) // ps
            bt = torch.arange(nreq * pages, dtype=torch.int32, device=dev).view(nreq, pages)
            cu = torch.arange(nreq + 1, dtype=torch.int32, device=dev) * q_len
            kvl = torch.full((nreq,), kv_len, dtype=torch.int32, device=dev)
            req = torch.arange(nreq, dtype=torch.int32, device=dev).repeat_interleave(q_len)
            q = torch.randn(nreq * q_len, heads, width, device=dev).to(bf)
            pool = [torch.randn(nreq * pages, kvh, ps, w_, device=dev).to(bf) for kvh, w_ in pools]
            return q, pool, bt, cu, kvl, req

        for label, nreq, q_len, kv_len in (("prefill_2048", 1, T, T), ("decode_b8_ctx2048", B, 1, CTX)):
            keys = nreq * (q_len * (kv_len - q_len) + q_len * (q_len + 1) // 2)
            q, (pool,), bt, cu, kvl, req = paged(nreq, q_len, kv_len, H, row, [(1, row)])
            o = torch.empty(nreq * q_len, H * rank, dtype=bf, device=dev)
            ms = timed(lambda: ops.paged_attention(q, pool, pool, bt, cu, kvl, req, o, 0.1, 0, ps, nreq, q_len, kv_len,
                                                   ws=ws, min_q_len=q_len, value_dim=rank))
            kern[f"latent_attention_{label}"] = roof(ms, 2.0 * H * (row + rank) * keys,
                                                     2.0 * (nreq * kv_len * row + q.numel() + o.numel()))
            q, (kp, vp), bt, cu, kvl, req = paged(nreq, q_len, kv_len, H, hd, [(Hkv, hd), (Hkv, hd)])
            o = torch.empty(nreq * q_len, H * hd, dtype=bf, device=dev)
            ms = timed(lambda: ops.paged_attention(q, kp, vp, bt, cu, kvl, req, o, 0.1, 0, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len))
            kern[f"llama_attention_{label}"] = roof(ms, 4.0 * H * hd * keys,
                                                    2.0 * (2 * nreq * kv_len * Hkv * hd + q.numel() + o.numel()))
        for label, M in (("2048_tokens", T), ("8_tokens", B)):
            h = torch.randn(M, W, device=dev).to(bf)
            x = torch.zeros(M, W, device=dev)
            E, top, F = z["experts"], z["top"], z["expert_ff"]
            wgu = ops.pack_expert_gate_up([(torch.randn(F, W, device=dev) * 0.02).to(bf) for _ in range(E)],
                                          [(torch.randn(F, W, device=dev) * 0.02).to(bf) for _ in range(E)])
            wd = (torch.randn(E, W, F, device=dev) * 0.02).to(bf)
            wr = (torch.randn(E, W, device=dev) * 0.5).to(bf)
            ids = torch.empty(M, top, dtype=torch.int32, device=dev)
            wt = torch.empty(M, top, device=dev)

            def routed():
                ops.route_topk(h, wr, None, top, ids, wt)
                ops.routed_feed_forward(ctx, h, wgu, wd, ids, wt, x, "clamped_swish", 7.0, 0.5)

            ms = timed(routed)
            used = min(E, M * top)
            kern[f"routed_experts_{label}"] = roof(ms, 2.0 * M * top * 3 * F * W, 2.0 * used * 3 * F * W)
            FF = z["ff"]
            g = ops.pack_gate_up((torch.randn(FF, W, device=dev) * 0.02).to(bf), (torch.randn(FF, W, device=dev) * 0.02).to(bf))
            dwn = (torch.randn(W, FF, device=dev) * 0.02).to(bf)
            act = torch.empty(M, FF, dtype=bf, device=dev)

            def dense(kind):
                ops.linear_gated(ctx, h, g, act, kind, 0.0)
                ops.linear(act, dwn, x, accumulate=True, alpha=0.5)

            kern[f"dense_gelu_feed_forward_{label}"] = roof(timed(lambda: dense("gelu_tanh")), 2.0 * M * 3 * FF * W, 2.0 * 3 * FF * W)
            kern[f"llama_silu_feed_forward_{label}"] = roof(timed(lambda: dense("silu")), 2.0 * M * 3 * FF * W, 2.0 * 3 * FF * W)
            del wgu, wd, g, dwn
        qn = torch.randn(T, H, dn, device=dev).to(bf)
        wuk = (torch.randn(H * rank, dn, device=dev) * 0.05).to(bf)
        ql = torch.empty(T, H, row, dtype=bf, device=dev)
        kern["query_into_latent_2048_tokens"] = roof(timed(lambda: ops.head_linear(qn, wuk, ql, rank, dn, False)),
                                                     2.0 * T * H * dn * rank, 2.0 * (qn.numel() + T * H * rank))
        mixed = torch.randn(T, H, rank, device=dev).to(bf)
        wuv = (torch.randn(H * dv, rank, device=dev) * 0.05).to(bf)
        oo = torch.empty(T, H, dv, dtype=bf, device=dev)
        kern["values_out_of_latent_2048_tokens"] = roof(timed(lambda: ops.head_linear(mixed, wuv, oo, dv, rank, False)),
                                                        2.0 * T * H * dv * rank, 2.0 * (mixed.numel() + oo.numel()))
        xr = torch.randn(T, W, device=dev)
        wv, bv = torch.ones(W, dtype=bf, device=dev), torch.zeros(W, dtype=bf, device=dev)
        on = torch.empty(T, W, dtype=bf, device=dev)
        kern["layer_norm_2048_tokens"] = roof(timed(lambda: ops.layernorm(xr, wv, bv, 1e-5, on)), 0, 6.0 * T * W)
        kern["llama_rms_norm_2048_tokens"] = roof(timed(lambda: ops.rmsnorm(xr, wv, 1e-5, on)), 0, 6.0 * T * W)
        rec["kernels"] = kern
        rec["config"] = {k: v for k, v in z.items()}
        out["sizes"][name] = rec
        del engines
        torch.cuda.empty_cache()
    return out


def cpu_reference_seconds() -> dict:
    """The reference is a CPU engine; it cannot be built here, so the nearest thing to its time is
    the plain implementation of the tests (its formulas, numpy, 32-bit, no cache) on the smallest of
    its published configurations: three prompts of up to 48 tokens, whole, and 16 greedy tokens each."""
    try:
        import numpy as np
        from garuda_b200.weights.random_init import random_weights
        from tests.plain import llama_plain
        cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
                   rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=128)
        w = {k: v.float().numpy() for k, v in random_weights(cfg, 0).items()}
        rng = np.random.default_rng(0)
        prompts = [rng.integers(0, 256, n).tolist() for n in (1, 24, 48)]
        t0 = time.perf_counter()
        for p in prompts:
            llama_plain.forward(cfg, w, p)
        t1 = time.perf_counter()
        for p in prompts:
            llama_plain.greedy_generate(cfg, w, p, 16)
        t2 = time.perf_counter()
        return {"what": "plain numpy implementation, Tiny A (2 layers, hidden 64), 3 prompts of 1/24/48 tokens",
                "prefill_seconds": round(t1 - t0, 4), "generate_16_tokens_each_seconds": round(t2 - t1, 4)}
    except Exception as e:      # the tests' plain model is not part of an installed package
        return {"unavailable": f"{type(e).__name__}: {e}"}


def run_one_phase(args, engine, cfg, rng, context) -> dict:
    """One phase only, for profiling: `--only prefill` runs a 2,048-token prompt `steps` times,
    `--only decode` prefills `--batch` requests and runs `steps` decode steps, `--only attention` runs
    the attention kernel alone on the last `--tokens` tokens of one request of `--context` (random
    queries, keys and values in the engine's own cache layout). Prints times, not the benchmark
    record."""
    import torch
    from garuda_b200 import StepEntry
    runner, V = engine.runner, cfg["vocab_size"]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    times = []
    if args.only == "attention":
        T, ctx_len, page = args.tokens, max(args.context or args.tokens, args.tokens), 32
        Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        npages = (ctx_len + page - 1) // page
        dev, ops = engine.device, engine.ops
        k, v = (torch.randn(npages + 1, Hkv, page, hd, device=dev).bfloat16() for _ in range(2))
        q = torch.randn(T, Hq, hd, device=dev).bfloat16()
        out = torch.zeros(T, Hq * hd, device=dev, dtype=torch.bfloat16)
        table = torch.arange(npages, dtype=torch.int32, device=dev).view(1, npages)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        kvl = torch.tensor([ctx_len], dtype=torch.int32, device=dev)
        treq = torch.zeros(T, dtype=torch.int32, device=dev)
        for i in range(args.warmup + args.steps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            ops.paged_attention(q, k, v, table, cu, kvl, treq, out, hd ** -0.5, 0, page, 1, T, ctx_len, min_q_len=T)
            e.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(s.elapsed_time(e))
        ops.tc.check_errors()
        ms = sorted(times)[len(times) // 2]
        flops = 4.0 * Hq * hd * (T * (ctx_len - T) + T * (T + 1) / 2)
        return {"only": "attention", "shape": args.shape, "tokens": T, "context": ctx_len, "heads": Hq, "kv_heads": Hkv,
                "head_dim": hd, "us": round(ms * 1e3, 1), "tflops_causal": round(flops / ms / 1e9, 1)}
    if args.only == "prefill":
        toks = rng.integers(0, V, args.tokens).tolist()
        for i in range(args.warmup + args.steps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            runner.run([StepEntry(i, toks, [args.tokens - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.end(i)
            if i >= args.warmup:
                times.append(s.elapsed_time(e))
    else:
        ids = list(range(args.batch))
        ctx_len = min(context, args.context or context)
        start_len = ctx_len - args.steps - args.warmup
        for r in ids:
            toks = rng.integers(0, V, start_len).tolist()
            for lo in range(0, start_len, PREFILL_TOKENS):
                runner.run([StepEntry(r, toks[lo:lo + PREFILL_TOKENS], [])])
        for i in range(args.warmup + args.steps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            runner.run([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in ids])
            e.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(s.elapsed_time(e))
    engine.ops.tc.check_errors()
    return {"only": args.only, "shape": args.shape, "batch": args.batch, "layers": cfg["num_hidden_layers"],
            "ms": [round(t, 4) for t in times]}


# ``--design murilorn``: the Murilorn design beside the Llama decoder at equal width, heads, head size and
# depth (random weights). Four layers: three delta-rule layers and one of windowed attention, each with
# routed experts (a token's `top` experts together as large as Llama's feed-forward), two streams.
MURILORN_SIZES = {
    "2k": dict(width=2048, heads=32, kv_heads=4, dim=64, window=1024, keep_first=4, softcap=30.0, d_heads=16, d_kv_heads=16,
               d_dim=128, d_vdim=128, taps=4, rank=64, experts=16, top=4, expert_ff=1408, streams=2, vocab=32000),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, window=1024, keep_first=4, softcap=30.0, d_heads=32, d_kv_heads=16,
               d_dim=128, d_vdim=128, taps=4, rank=128, experts=16, top=4, expert_ff=2752, streams=2, vocab=32000),
}


def murilorn_configs(z):
    attn = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                           "scale": z["dim"] ** -0.5, "softcap": z["softcap"],
                                           "mask": {"size": z["window"], "keep_first": z["keep_first"]}}}
    delta = {"type": "channel_delta", "mixer": {"heads": z["d_heads"], "kv_heads": z["d_kv_heads"], "dim": z["d_dim"],
                                                "vdim": z["d_vdim"], "conv": z["taps"], "decay_rank": z["rank"], "gate_rank": z["rank"]}}
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["expert_ff"]}}
    murilorn = {"architecture": "Murilorn", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
                "norm": {"eps": 1e-5}, "streams": z["streams"], "logit_scale": 1.0, "logit_softcap": 30.0, "max_positions": 4096,
                "layers": [dict(m, mlp=moe) for m in (delta, delta, delta, attn)]}
    llama = dict(LLAMA, hidden_size=z["width"], num_hidden_layers=4, num_attention_heads=z["heads"],
                 num_key_value_heads=z["kv_heads"], head_dim=z["dim"], intermediate_size=z["top"] * z["expert_ff"],
                 vocab_size=z["vocab"], rope_theta=10000.0, max_position_embeddings=4096)
    return murilorn, llama


def run_design_murilorn(args) -> dict:
    """Prefill and decode throughput of the Murilorn design and of the Llama decoder at equal sizes, and
    the design's kernels beside the like kernels of Llama, each against its roofline (the slower of
    bytes / measured copy rate and FLOPs / measured bfloat16 rate)."""
    import numpy as np
    import torch
    from garuda_b200 import Engine, StepEntry
    from garuda_b200.engine.batch import Workspace
    from garuda_b200.weights import write_random_model

    hbm_peak, tflops_peak, peak_kind = peaks()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        return sorted(times)[len(times) // 2]

    def roof(ms, flops=0.0, nbytes=0.0):
        ideal = max(flops / (tflops_peak * 1e12), nbytes / (hbm_peak * 1e9)) * 1e3
        return {"ms": round(ms, 4), "roofline_ms": round(ideal, 4), "frac": round(ideal / ms, 4)}

    out = {"design": "murilorn", "peaks": peak_kind, "hbm_gbs": hbm_peak, "bf16_tflops": tflops_peak, "dtype": "bf16",
           "data": "synthetic", "timing": "CUDA events, 3 warm-up runs, L2 flushed before every timed run, median", "sizes": {}}
    B, CTX, T = 8, 2048, PREFILL_TOKENS
    for name in (args.size.split(",") if args.size else list(MURILORN_SIZES)):
        z = MURILORN_SIZES[name]
        rec, engines = {}, {}
        for arch, cfg in zip(("murilorn", "llama"), murilorn_configs(z)):
            tmp = tempfile.mkdtemp(prefix="garuda_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
            try:
                write_random_model(tmp, cfg, seed=0, store_dtype=torch.bfloat16)
                engine = Engine(tmp, dtype="bfloat16", context=4096, page_size=32, kv_tokens=B * CTX + 4096 + 64,
                                max_concurrent=B, max_batch_tokens=T, prefill_chunk=T, ignore_eos=True)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            engines[arch] = engine
            runner, rng, V = engine.runner, np.random.default_rng(0), z["vocab"]
            toks = rng.integers(0, V, T).tolist()
            rid = [0]

            def prefill():
                rid[0] += 1
                runner.run([StepEntry(10_000 + rid[0], toks, [T - 1])])
                runner.end(10_000 + rid[0])

            ms = timed(prefill, reps=5)
            rec[arch] = {"prefill_2048_ms": round(ms, 3), "prefill_tok_s": round(T / ms * 1e3)}
            steps = 48
            for r in range(B):
                runner.run([StepEntry(r, rng.integers(0, V, CTX - steps - 8).tolist(), [])])
            feed = rng.integers(0, V, (steps + 8, B))
            for i in range(8):
                runner.run([StepEntry(r, [int(feed[i, r])], [0]) for r in range(B)])
            marks = [ev() for _ in range(steps + 1)]
            torch.cuda.synchronize()
            marks[0].record()
            for i in range(steps):
                runner.run([StepEntry(r, [int(feed[8 + i, r])], [0]) for r in range(B)])
                marks[i + 1].record()
            torch.cuda.synchronize()
            each = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
            for r in range(B):
                runner.end(r)
            rec[arch].update({"decode_b8_ctx2048_ms": round(each[len(each) // 2], 4),
                              "decode_tok_s": round(B / each[len(each) // 2] * 1e3),
                              "graph_replays": runner.graphs.replays,
                              "kernels_per_decode_step": runner.graphs.launches_replayed(B)})
            if engine.ops.tc is not None:
                engine.ops.tc.check_errors()
        # ------------------------------------------------------------ kernel beside like kernel
        ops = engines["murilorn"].ops
        bf = torch.bfloat16
        H, Hkv, hd, W, ps, win = z["heads"], z["kv_heads"], z["dim"], z["width"], 32, z["window"]
        ws = Workspace(dev)

        class Ctx:
            pass
        ctx = Ctx()
        ctx.ws = ws
        ctx.step_cache = {}
        kern = {}
        for label, nreq, q_len, kv_len in (("prefill_2048", 1, T, T), ("decode_b8_ctx2048", B, 1, CTX)):
            pages = (kv_len + ps - 1) // ps
            bt = torch.arange(nreq * pages, dtype=torch.int32, device=dev).view(nreq, pages)
            cu = torch.arange(nreq + 1, dtype=torch.int32, device=dev) * q_len
            kvl = torch.full((nreq,), kv_len, dtype=torch.int32, device=dev)
            req = torch.arange(nreq, dtype=torch.int32, device=dev).repeat_interleave(q_len)
            q = torch.randn(nreq * q_len, H, hd, device=dev).to(bf)
            kp, vp = (torch.randn(nreq * pages, Hkv, ps, hd, device=dev).to(bf) for _ in range(2))
            o = torch.empty(nreq * q_len, H * hd, dtype=bf, device=dev)
            # keys a query reads: its window (and the kept first positions)
            keys = nreq * sum(min(p + 1, win) + (z["keep_first"] if p + 1 > win else 0) for p in range(kv_len - q_len, kv_len))
            read = nreq * min(kv_len, win + q_len)
            ms = timed(lambda: ops.paged_attention(q, kp, vp, bt, cu, kvl, req, o, hd ** -0.5, win, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len, softcap=z["softcap"], keep_first=z["keep_first"], sink=True))
            kern[f"capped_sink_attention_{label}"] = roof(ms, 4.0 * H * hd * keys, 2.0 * (2 * read * Hkv * hd + q.numel() + o.numel()))
            ms = timed(lambda: ops.paged_attention(q, kp, vp, bt, cu, kvl, req, o, hd ** -0.5, win, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len))
            kern[f"llama_windowed_attention_{label}"] = roof(ms, 4.0 * H * hd * keys, 2.0 * (2 * read * Hkv * hd + q.numel() + o.numel()))
        E, top, F = z["experts"], z["top"], z["expert_ff"]
        for label, M in (("2048_tokens", T), ("8_tokens", B)):
            h = torch.randn(M, W, device=dev).to(bf)
            x = torch.zeros(M, W, device=dev)
            wgu = ops.pack_expert_gate_up([(torch.randn(F, W, device=dev) * 0.02).to(bf) for _ in range(E)],
                                          [(torch.randn(F, W, device=dev) * 0.02).to(bf) for _ in range(E)])
            wd = (torch.randn(E, W, F, device=dev) * 0.02).to(bf)
            wr = (torch.randn(E, W, device=dev) * 0.5).to(bf)
            ids = torch.empty(M, top, dtype=torch.int32, device=dev)
            wt = torch.empty(M, top, device=dev)

            def routed():
                ops.route_topk(h, wr, None, top, ids, wt, score="sigmoid")
                ops.routed_feed_forward(ctx, h, wgu, wd, ids, wt, x, "silu", 0.0, 1.0, scale_input=True)

            used = min(E, M * top)
            kern[f"routed_experts_{label}"] = roof(timed(routed), 2.0 * M * top * 3 * F * W, 2.0 * used * 3 * F * W)
            FF = top * F
            g = ops.pack_gate_up((torch.randn(FF, W, device=dev) * 0.02).to(bf), (torch.randn(FF, W, device=dev) * 0.02).to(bf))
            dwn = (torch.randn(W, FF, device=dev) * 0.02).to(bf)
            act = torch.empty(M, FF, dtype=bf, device=dev)

            def dense():
                ops.linear_gated(ctx, h, g, act, "silu", 0.0)
                ops.linear(act, dwn, x, accumulate=True)

            kern[f"llama_silu_feed_forward_{label}"] = roof(timed(dense), 2.0 * M * 3 * FF * W, 2.0 * 3 * FF * W)
            del wgu, wd, g, dwn
        # the recurrent mixer's own kernels (no counterpart in Llama): bytes are its rows in and out and the state
        dH, dG, dd, dv, taps = z["d_heads"], z["d_kv_heads"], z["d_dim"], z["d_vdim"], z["taps"]
        C = 2 * dG * dd + dH * dv
        conv_w, a_log = torch.randn(C, taps, device=dev) * 0.3, torch.randn(dH, device=dev) * 0.3
        dtb, nw = torch.randn(dH * dd, device=dev), torch.ones(dv, device=dev)
        state = torch.zeros(B, dH * dd * dv + (taps - 1) * C, device=dev)

        class Bt:
            pass
        for label, nreq, q_len in (("prefill_2048", 1, T), ("decode_b8", B, 1)):
            b = Bt()
            b.cu_q = torch.arange(nreq + 1, dtype=torch.int32, device=dev) * q_len
            b.slots = torch.arange(nreq, dtype=torch.int32, device=dev)
            b.token_req = torch.arange(nreq, dtype=torch.int32, device=dev).repeat_interleave(q_len)
            b.num_requests, b.max_q_len = nreq, q_len
            ctx.batch = b
            n = nreq * q_len
            proj, second = torch.randn(n, C + dH, device=dev), torch.randn(n, dH * dd + dH * dv, device=dev)
            o = torch.empty(n, dH * dv, dtype=bf, device=dev)
            ms = timed(lambda: ops.delta_rule(ctx, proj, second, conv_w, a_log, dtb, nw, 1e-5, state, dH, dG, dd, dv, taps, o))
            moved = 4.0 * (proj.numel() + second.numel()) + 2.0 * o.numel() + 2 * 4.0 * nreq * state.shape[1]
            kern[f"delta_rule_{label}"] = roof(ms, 0, moved)
        S = z["streams"]
        xs, y = torch.randn(T, S, W, device=dev), torch.randn(T, W, device=dev)
        a_in, b_out, mix = torch.ones(S, device=dev), torch.ones(S, device=dev), torch.eye(S, device=dev).contiguous()
        wv = torch.ones(W, device=dev)
        on = torch.empty(T, W, dtype=bf, device=dev)
        kern["streams_read_2048_tokens"] = roof(timed(lambda: ops.streams_rmsnorm(xs, a_in, wv, 1e-5, on)), 0, (4.0 * S + 2.0) * T * W)
        kern["streams_write_and_read_2048_tokens"] = roof(
            timed(lambda: ops.streams_update(xs, mix, b_out, y, next_in=a_in, norm_weight=wv, eps=1e-5, normed=on)), 0,
            (8.0 * S + 4.0 + 2.0) * T * W)
        xr = torch.randn(T, W, device=dev)
        kern["llama_rms_norm_2048_tokens"] = roof(timed(lambda: ops.rmsnorm(xr, wv, 1e-5, on)), 0, 6.0 * T * W)
        rec["kernels"] = kern
        rec["config"] = {k: v for k, v in z.items()}
        out["sizes"][name] = rec
        del engines
        torch.cuda.empty_cache()
    return out


# ``--design luvapel``: the Luvapel design beside the Murilorn decoder (the closest of the engine's models: a
# delta rule and windowed attention) at equal width, heads, head sizes and depth (random weights). Four layers:
# generalized delta rule, mixers side by side (windowed attention and a gated delta rule), and again; every
# layer with a dense feed-forward as large as a Murilorn token's experts together.
LUVAPEL_SIZES = {
    "2k": dict(width=2048, heads=32, kv_heads=4, dim=64, window=1024, rot_dims=32, g_heads=32, g_dim=64, rank=64,
               d_heads=16, d_kv_heads=16, d_dim=128, d_vdim=128, taps=4, ff=5632, experts=16, top=4, expert_ff=1408, vocab=32000),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, window=1024, rot_dims=64, g_heads=32, g_dim=128, rank=128,
               d_heads=32, d_kv_heads=16, d_dim=128, d_vdim=128, taps=4, ff=11008, experts=16, top=4, expert_ff=2752, vocab=32000),
}


def luvapel_configs(z):
    ff = {"kind": "dense", "ff": z["ff"]}
    general = {"type": "general_delta", "mixer": {"heads": z["g_heads"], "dim": z["g_dim"], "decay_rank": z["rank"]}, "mlp": ff}
    left = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
            "mask": {"size": z["window"]}, "rot": {"base": 10000.0, "dims": z["rot_dims"]}}
    right = {"heads": z["d_heads"], "kv_heads": z["d_kv_heads"], "dim": z["d_dim"], "vdim": z["d_vdim"], "conv": z["taps"]}
    parallel = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": ff}
    luvapel = {"architecture": "Luvapel", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
               "norm": {"eps": 1e-5}, "max_positions": 4096, "layers": [general, parallel, general, parallel]}
    attn = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                           "scale": z["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": z["window"], "keep_first": 4}}}
    delta = {"type": "channel_delta", "mixer": {"heads": z["d_heads"], "kv_heads": z["d_kv_heads"], "dim": z["d_dim"],
                                                "vdim": z["d_vdim"], "conv": z["taps"], "decay_rank": z["rank"], "gate_rank": z["rank"]}}
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["expert_ff"]}}
    murilorn = {"architecture": "Murilorn", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
                "norm": {"eps": 1e-5}, "streams": 2, "logit_scale": 1.0, "logit_softcap": 30.0, "max_positions": 4096,
                "layers": [dict(m, mlp=moe) for m in (delta, attn, delta, attn)]}
    return luvapel, murilorn


def run_design_luvapel(args) -> dict:
    """Prefill and decode throughput of the Luvapel design and of the Murilorn decoder at equal sizes, and
    the design's kernels beside the like kernels of Murilorn (or of Llama, where those are the like ones),
    each against its roofline (the slower of bytes / measured copy rate and FLOPs / measured bfloat16 rate)."""
    import numpy as np
    import torch
    from garuda_b200 import Engine, StepEntry
    from garuda_b200.engine.batch import Workspace
    from garuda_b200.parts.attention import NormedKeyAttention
    from garuda_b200.weights import write_random_model

    hbm_peak, tflops_peak, peak_kind = peaks()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        return sorted(times)[len(times) // 2]

    def roof(ms, flops=0.0, nbytes=0.0):
        ideal = max(flops / (tflops_peak * 1e12), nbytes / (hbm_peak * 1e9)) * 1e3
        return {"ms": round(ms, 4), "roofline_ms": round(ideal, 4), "frac": round(ideal / ms, 4)}

    out = {"design": "luvapel", "beside": "murilorn", "peaks": peak_kind, "hbm_gbs": hbm_peak, "bf16_tflops": tflops_peak,
           "dtype": "bf16", "data": "synthetic",
           "timing": "CUDA events, 3 warm-up runs, L2 flushed before every timed run, median", "sizes": {}}
    B, CTX, T = 8, 2048, PREFILL_TOKENS
    for name in (args.size.split(",") if args.size else list(LUVAPEL_SIZES)):
        z = LUVAPEL_SIZES[name]
        rec, engines = {}, {}
        for arch, cfg in zip(("luvapel", "murilorn"), luvapel_configs(z)):
            tmp = tempfile.mkdtemp(prefix="garuda_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
            try:
                write_random_model(tmp, cfg, seed=0, store_dtype=torch.bfloat16)
                engine = Engine(tmp, dtype="bfloat16", context=4096, page_size=32, kv_tokens=B * CTX + 4096 + 64,
                                max_concurrent=B, max_batch_tokens=T, prefill_chunk=T, ignore_eos=True)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            engines[arch] = engine
            runner, rng, V = engine.runner, np.random.default_rng(0), z["vocab"]
            toks = rng.integers(0, V, T).tolist()
            rid = [0]

            def prefill():
                rid[0] += 1
                runner.run([StepEntry(10_000 + rid[0], toks, [T - 1])])
                runner.end(10_000 + rid[0])

            ms = timed(prefill, reps=5)
            rec[arch] = {"prefill_2048_ms": round(ms, 3), "prefill_tok_s": round(T / ms * 1e3)}
            steps = 48
            for r in range(B):
                runner.run([StepEntry(r, rng.integers(0, V, CTX - steps - 8).tolist(), [])])
            feed = rng.integers(0, V, (steps + 8, B))
            for i in range(8):
                runner.run([StepEntry(r, [int(feed[i, r])], [0]) for r in range(B)])
            marks = [ev() for _ in range(steps + 1)]
            torch.cuda.synchronize()
            marks[0].record()
            for i in range(steps):
                runner.run([StepEntry(r, [int(feed[8 + i, r])], [0]) for r in range(B)])
                marks[i + 1].record()
            torch.cuda.synchronize()
            each = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
            for r in range(B):
                runner.end(r)
            rec[arch].update({"decode_b8_ctx2048_ms": round(each[len(each) // 2], 4),
                              "decode_tok_s": round(B / each[len(each) // 2] * 1e3),
                              "graph_replays": runner.graphs.replays,
                              "kernels_per_decode_step": runner.graphs.launches_replayed(B)})
            if engine.ops.tc is not None:
                engine.ops.tc.check_errors()
        # ------------------------------------------------------------ kernel beside like kernel
        ops = engines["luvapel"].ops
        bf = torch.bfloat16
        H, Hkv, hd, W, ps, win = z["heads"], z["kv_heads"], z["dim"], z["width"], 32, z["window"]
        ws = Workspace(dev)

        class Ctx:
            pass
        ctx = Ctx()
        ctx.ws = ws
        ctx.step_cache = {}
        kern = {}
        for label, nreq, q_len, kv_len in (("prefill_2048", 1, T, T), ("decode_b8_ctx2048", B, 1, CTX)):
            pages = (kv_len + ps - 1) // ps
            bt = torch.arange(nreq * pages, dtype=torch.int32, device=dev).view(nreq, pages)
            cu = torch.arange(nreq + 1, dtype=torch.int32, device=dev) * q_len
            kvl = torch.full((nreq,), kv_len, dtype=torch.int32, device=dev)
            req = torch.arange(nreq, dtype=torch.int32, device=dev).repeat_interleave(q_len)
            q = torch.randn(nreq * q_len, H, hd, device=dev).to(bf)
            kp, vp = (torch.randn(nreq * pages, Hkv, ps, hd, device=dev).to(bf) for _ in range(2))
            o = torch.empty(nreq * q_len, H * hd, dtype=bf, device=dev)
            keys = nreq * sum(min(p + 1, win) for p in range(kv_len - q_len, kv_len))
            read = nreq * min(kv_len, win + q_len)
            cost = (4.0 * H * hd * keys, 2.0 * (2 * read * Hkv * hd + q.numel() + o.numel()))
            ms = timed(lambda: ops.paged_attention(q, kp, vp, bt, cu, kvl, req, o, hd ** -0.5, win, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len))
            kern[f"windowed_attention_{label}"] = roof(ms, *cost)
            ms = timed(lambda: ops.paged_attention(q, kp, vp, bt, cu, kvl, req, o, hd ** -0.5, win, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len, softcap=30.0, keep_first=4, sink=True))
            kern[f"murilorn_capped_sink_attention_{label}"] = roof(ms, *cost)
            # the projected row into queries and pages: normed and rotated here, biased there
            n = nreq * q_len
            pos = (torch.arange(q_len, dtype=torch.int32, device=dev) + (kv_len - q_len)).repeat(nreq)
            row = torch.randn(n, (H + 3 * Hkv) * hd, device=dev)
            part = NormedKeyAttention(W, H, Hkv, hd, rot_base=10000.0, rot_dims=z["rot_dims"])
            qw, kw = torch.ones(H, hd, device=dev), torch.ones(hd, device=dev)
            moved = 4.0 * n * (H + Hkv) * hd + 2.0 * n * (H + 2 * Hkv) * hd
            ms = timed(lambda: ops.qk_norm_rope_append(row, (0, H * hd, H * hd), q, kp, vp, pos, req, bt, H, Hkv, hd, hd, qw, kw,
                                                       1e-5, part.rotary, ps))
            kern[f"norm_rotate_store_{label}"] = roof(ms, 0, moved)
            bias = torch.zeros((H + 2 * Hkv) * hd, device=dev)
            rowm = torch.randn(n, (H + 2 * Hkv) * hd, device=dev)
            ms = timed(lambda: ops.qkv_bias_append(rowm, bias, q, kp, vp, pos, req, bt, H, Hkv, hd, hd, ps))
            kern[f"murilorn_bias_store_{label}"] = roof(ms, 0, 4.0 * rowm.numel() + 2.0 * rowm.numel())
        # feed-forwards: relu^2 of one product here, SiLU-gate of two in Llama's (the dense like kernel)
        FF = z["ff"]
        for label, M in (("2048_tokens", T), ("8_tokens", B)):
            h = torch.randn(M, W, device=dev).to(bf)
            x = torch.zeros(M, W, device=dev)
            up, dwn = (torch.randn(FF, W, device=dev) * 0.02).to(bf), (torch.randn(W, FF, device=dev) * 0.02).to(bf)
            act, y = torch.empty(M, FF, dtype=bf, device=dev), torch.empty(M, W, device=dev)

            def plain():
                ops.linear_act(ctx, h, up, act, "relu2")
                ops.linear(act, dwn, y)

            kern[f"relu2_feed_forward_{label}"] = roof(timed(plain), 2.0 * M * 2 * FF * W, 2.0 * 2 * FF * W)
            g = ops.pack_gate_up((torch.randn(FF, W, device=dev) * 0.02).to(bf), (torch.randn(FF, W, device=dev) * 0.02).to(bf))

            def dense():
                ops.linear_gated(ctx, h, g, act, "silu", 0.0)
                ops.linear(act, dwn, x, accumulate=True)

            kern[f"llama_silu_feed_forward_{label}"] = roof(timed(dense), 2.0 * M * 3 * FF * W, 2.0 * 3 * FF * W)
            del up, dwn, g, y, act
        # the recurrent mixers: bytes are their rows in and out and the state

        class Bt:
            pass
        dH, dG, dd, dv, taps = z["d_heads"], z["d_kv_heads"], z["d_dim"], z["d_vdim"], z["taps"]
        gH, gd = z["g_heads"], z["g_dim"]
        C = 2 * dG * dd + dH * dv
        conv_w, a_log = torch.randn(C, taps, device=dev) * 0.3, torch.randn(dH, device=dev) * 0.3
        nw = torch.ones(dv, device=dev)
        state = torch.zeros(B, dH * dd * dv + (taps - 1) * C, device=dev)
        gstate = torch.zeros(B, gH * gd * gd, device=dev)
        HD = gH * gd
        w0, a0, gnw = torch.randn(HD, device=dev), torch.randn(HD, device=dev), torch.ones(HD, device=dev)
        for label, nreq, q_len in (("prefill_2048", 1, T), ("decode_b8", B, 1)):
            b = Bt()
            b.cu_q = torch.arange(nreq + 1, dtype=torch.int32, device=dev) * q_len
            b.slots = torch.arange(nreq, dtype=torch.int32, device=dev)
            b.token_req = torch.arange(nreq, dtype=torch.int32, device=dev).repeat_interleave(q_len)
            b.num_requests, b.max_q_len = nreq, q_len
            ctx.batch = b
            n = nreq * q_len
            proj = torch.randn(n, C + dH, device=dev)
            o = torch.empty(n, dH * dv, dtype=bf, device=dev)
            second = torch.randn(n, dH + dH * dv, device=dev)
            dtb = torch.randn(dH, device=dev)
            ms = timed(lambda: ops.delta_rule(ctx, proj, second, conv_w, a_log, dtb, nw, 1e-5, state, dH, dG, dd, dv, taps, o,
                                              decay_per_head=True, gate="silu"))
            kern[f"head_delta_rule_{label}"] = roof(ms, 0, 4.0 * (proj.numel() + second.numel()) + 2.0 * o.numel()
                                                    + 2 * 4.0 * nreq * state.shape[1])
            second = torch.randn(n, dH * dd + dH * dv, device=dev)
            dtb = torch.randn(dH * dd, device=dev)
            ms = timed(lambda: ops.delta_rule(ctx, proj, second, conv_w, a_log, dtb, nw, 1e-5, state, dH, dG, dd, dv, taps, o))
            kern[f"murilorn_channel_delta_rule_{label}"] = roof(ms, 0, 4.0 * (proj.numel() + second.numel()) + 2.0 * o.numel()
                                                                + 2 * 4.0 * nreq * state.shape[1])
            gproj, zdec = torch.randn(n, 5 * HD, device=dev), torch.randn(n, HD, device=dev)
            go = torch.empty(n, HD, dtype=bf, device=dev)
            ms = timed(lambda: ops.general_delta(ctx, gproj, (0, HD, 2 * HD, 3 * HD, 4 * HD), zdec, w0, a0, 0.6, gnw, 1e-5, gstate,
                                                 gH, gd, gd, go))
            kern[f"general_delta_rule_{label}"] = roof(ms, 0, 4.0 * (gproj.numel() + zdec.numel()) + 2.0 * go.numel()
                                                       + 2 * 4.0 * nreq * gstate.shape[1])
        # what joins a sublayer to the residual: two branches, gate, norm and sum here; two streams there
        ys = [torch.randn(T, W, device=dev) for _ in range(2)]
        bw = [torch.ones(W, device=dev) for _ in range(2)]
        gate, gb_, wv = torch.randn(T, W, device=dev), torch.zeros(W, device=dev), torch.ones(W, device=dev)
        xr, hb = torch.randn(T, W, device=dev), torch.empty(T, W, dtype=bf, device=dev)
        kern["branches_gate_norm_add_2048_tokens"] = roof(
            timed(lambda: ops.sublayer_merge(ys, bw, 1e-5, x=xr, gate=gate, gate_bias=gb_, weight=wv, rounded=hb)), 0,
            (4.0 * 5 + 2.0) * T * W)
        kern["gate_norm_add_2048_tokens"] = roof(
            timed(lambda: ops.sublayer_merge(ys[:1], None, 1e-5, x=xr, gate=gate, gate_bias=gb_, weight=wv, rounded=hb)), 0,
            (4.0 * 4 + 2.0) * T * W)
        S = 2
        xs, y = torch.randn(T, S, W, device=dev), torch.randn(T, W, device=dev)
        a_in, b_out, mix = torch.ones(S, device=dev), torch.ones(S, device=dev), torch.eye(S, device=dev).contiguous()
        on = torch.empty(T, W, dtype=bf, device=dev)
        kern["murilorn_streams_write_and_read_2048_tokens"] = roof(
            timed(lambda: ops.streams_update(xs, mix, b_out, y, next_in=a_in, norm_weight=wv, eps=1e-5, normed=on)), 0,
            (8.0 * S + 4.0 + 2.0) * T * W)
        octx = torch.randn(T, H * hd, device=dev).to(bf)
        kern["output_gate_2048_tokens"] = roof(timed(lambda: ops.gate_mul(octx, gate[:, :H * hd], "sigmoid")), 0, (4.0 + 4.0) * T * H * hd)
        rec["kernels"] = kern
        rec["config"] = {k: v for k, v in z.items()}
        out["sizes"][name] = rec
        del engines
        torch.cuda.empty_cache()
    return out


# ``--design midulorn``: the Midulorn design beside the Murilorn decoder (the closest of the engine's models:
# attention with a sink and biases and no position encoding, a recurrence behind short convolutions, routed
# experts) at equal width, heads, head sizes and depth (random weights). Four layers: chunked attention behind
# convolutions with a dense feed-forward, latent attention with experts, a gated recurrence with a dense
# feed-forward, chunked attention with experts.
MIDULORN_SIZES = {
    "2k": dict(width=2048, heads=32, kv_heads=4, dim=64, chunk=1024, taps=4, l_heads=16, l_dim=64, rot_dim=32, l_vdim=64,
               kv_rank=256, gru=4096, ff=5632, experts=16, top=4, expert_ff=1408, vocab=32000,
               d_heads=16, d_kv_heads=16, d_dim=128, d_vdim=128, rank=64),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, chunk=1024, taps=4, l_heads=32, l_dim=64, rot_dim=32, l_vdim=64,
               kv_rank=512, gru=8192, ff=11008, experts=16, top=4, expert_ff=2752, vocab=32000,
               d_heads=32, d_kv_heads=16, d_dim=128, d_vdim=128, rank=128),
}


def midulorn_configs(z):
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["expert_ff"]}}
    att = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                          "scale": z["dim"] ** -0.5, "conv": z["taps"], "mask": {"size": z["chunk"]}, "v_mix": True}}
    lat = {"type": "latent_attention", "mixer": {"heads": z["l_heads"], "dim": z["l_dim"], "rot_dim": z["rot_dim"], "vdim": z["l_vdim"],
                                                 "kv_rank": z["kv_rank"], "scale": (z["l_dim"] + z["rot_dim"]) ** -0.5,
                                                 "rot": {"base": 10000.0, "dims": z["rot_dim"]}}}
    gru = {"type": "mingru", "mixer": {"width": z["gru"]}}
    midulorn = {"architecture": "Midulorn", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
                "norm": {"eps": 1e-5}, "postln_alpha": 2.0, "logit_scale": 1.0, "max_positions": 4096,
                "layers": [dict(att, mlp=dense), dict(lat, mlp=moe), dict(gru, mlp=dense), dict(att, mlp=moe)]}
    attn = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                                           "scale": z["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": z["chunk"], "keep_first": 4}}}
    delta = {"type": "channel_delta", "mixer": {"heads": z["d_heads"], "kv_heads": z["d_kv_heads"], "dim": z["d_dim"],
                                                "vdim": z["d_vdim"], "conv": z["taps"], "decay_rank": z["rank"], "gate_rank": z["rank"]}}
    murilorn = {"architecture": "Murilorn", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
                "norm": {"eps": 1e-5}, "streams": 2, "logit_scale": 1.0, "logit_softcap": 30.0, "max_positions": 4096,
                "layers": [dict(m, mlp=moe) for m in (attn, delta, delta, attn)]}
    return midulorn, murilorn


def run_design_midulorn(args) -> dict:
    """Prefill and decode throughput of the Midulorn design and of the Murilorn decoder at equal sizes, and
    the design's kernels beside the like kernels of the engine's other models, each against its roofline (the
    slower of bytes / measured copy rate and FLOPs / measured bfloat16 rate)."""
    import numpy as np
    import torch
    from garuda_b200 import Engine, StepEntry
    from garuda_b200.engine.batch import Workspace
    from garuda_b200.weights import write_random_model

    hbm_peak, tflops_peak, peak_kind = peaks()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        return sorted(times)[len(times) // 2]

    def roof(ms, flops=0.0, nbytes=0.0):
        ideal = max(flops / (tflops_peak * 1e12), nbytes / (hbm_peak * 1e9)) * 1e3
        return {"ms": round(ms, 4), "roofline_ms": round(ideal, 4), "frac": round(ideal / ms, 4)}

    out = {"design": "midulorn", "beside": "murilorn", "peaks": peak_kind, "hbm_gbs": hbm_peak, "bf16_tflops": tflops_peak,
           "dtype": "bf16", "data": "synthetic",
           "timing": "CUDA events, 3 warm-up runs, L2 flushed before every timed run, median", "sizes": {}}
    B, CTX, T = 8, 2048, PREFILL_TOKENS
    for name in (args.size.split(",") if args.size else list(MIDULORN_SIZES)):
        z = MIDULORN_SIZES[name]
        rec, engines = {}, {}
        for arch, cfg in zip(("midulorn", "murilorn"), midulorn_configs(z)):
            tmp = tempfile.mkdtemp(prefix="garuda_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
            try:
                write_random_model(tmp, cfg, seed=0, store_dtype=torch.bfloat16)
                engine = Engine(tmp, dtype="bfloat16", context=4096, page_size=32, kv_tokens=B * CTX + 4096 + 64,
                                max_concurrent=B, max_batch_tokens=T, prefill_chunk=T, ignore_eos=True)
            finally:
                shutil.rmtree(tmp, ignore_errors=True)
            engines[arch] = engine
            runner, rng, V = engine.runner, np.random.default_rng(0), z["vocab"]
            toks = rng.integers(0, V, T).tolist()
            rid = [0]

            def prefill():
                rid[0] += 1
                runner.run([StepEntry(10_000 + rid[0], toks, [T - 1])])
                runner.end(10_000 + rid[0])

            ms = timed(prefill, reps=5)
            rec[arch] = {"prefill_2048_ms": round(ms, 3), "prefill_tok_s": round(T / ms * 1e3)}
            steps = 48
            for r in range(B):
                runner.run([StepEntry(r, rng.integers(0, V, CTX - steps - 8).tolist(), [])])
            feed = rng.integers(0, V, (steps + 8, B))
            for i in range(8):
                runner.run([StepEntry(r, [int(feed[i, r])], [0]) for r in range(B)])
            marks = [ev() for _ in range(steps + 1)]
            torch.cuda.synchronize()
            marks[0].record()
            for i in range(steps):
                runner.run([StepEntry(r, [int(feed[8 + i, r])], [0]) for r in range(B)])
                marks[i + 1].record()
            torch.cuda.synchronize()
            each = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
            for r in range(B):
                runner.end(r)
            rec[arch].update({"decode_b8_ctx2048_ms": round(each[len(each) // 2], 4),
                              "decode_tok_s": round(B / each[len(each) // 2] * 1e3),
                              "graph_replays": runner.graphs.replays,
                              "kernels_per_decode_step": runner.graphs.launches_replayed(B)})
            if engine.ops.tc is not None:
                engine.ops.tc.check_errors()
        # ------------------------------------------------------------ kernel beside like kernel
        ops = engines["midulorn"].ops
        bf = torch.bfloat16
        H, Hkv, hd, W, ps, chunk = z["heads"], z["kv_heads"], z["dim"], z["width"], 32, z["chunk"]
        ws = Workspace(dev)

        class Ctx:
            pass

        class Bt:
            pass
        ctx = Ctx()
        ctx.ws = ws
        ctx.step_cache = {}
        kern = {}
        for label, nreq, q_len, kv_len in (("prefill_2048", 1, T, T), ("decode_b8_ctx2048", B, 1, CTX)):
            pages = (kv_len + ps - 1) // ps
            n = nreq * q_len
            bt = torch.arange(nreq * pages, dtype=torch.int32, device=dev).view(nreq, pages)
            cu = torch.arange(nreq + 1, dtype=torch.int32, device=dev) * q_len
            kvl = torch.full((nreq,), kv_len, dtype=torch.int32, device=dev)
            req = torch.arange(nreq, dtype=torch.int32, device=dev).repeat_interleave(q_len)
            pos = (torch.arange(q_len, dtype=torch.int32, device=dev) + (kv_len - q_len)).repeat(nreq)
            b = Bt()
            b.cu_q, b.token_req, b.positions, b.kv_lens = cu, req, pos, kvl
            b.slots = torch.arange(nreq, dtype=torch.int32, device=dev)
            b.num_requests, b.max_q_len, b.min_q_len = nreq, q_len, q_len
            ctx.batch = b
            # chunked attention with sinks and the distance term, beside Murilorn's windowed one of as many keys
            q = torch.randn(n, H, hd, device=dev).to(bf)
            kp, vp = (torch.randn(nreq * pages, Hkv, ps, hd, device=dev).to(bf) for _ in range(2))
            o = torch.empty(n, H * hd, dtype=bf, device=dev)
            sinks, r1, r2 = torch.randn(H, device=dev), torch.rand(H, device=dev), torch.rand(H, device=dev)
            seen = [p % chunk + 1 for p in range(kv_len - q_len, kv_len)]
            tiles = -(-max(seen) // 64) * 64 if q_len == 1 else sum(-(-min(c, kv_len) // 64) * 64 for c in (chunk,) * (kv_len // chunk))
            cost = (4.0 * H * hd * nreq * sum(seen), 2.0 * (2 * nreq * min(kv_len, max(seen) if q_len == 1 else kv_len) * Hkv * hd + q.numel() + o.numel()))
            ms = timed(lambda: ops.paged_attention(q, kp, vp, bt, cu, kvl, req, o, hd ** -0.5, 0, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len, sink_values=sinks, distance=(r1, r2), chunk=chunk))
            kern[f"chunked_attention_{label}"] = roof(ms, *cost)
            win = max(seen) if q_len == 1 else chunk
            keys = nreq * sum(min(p + 1, win) for p in range(kv_len - q_len, kv_len))
            cost_w = (4.0 * H * hd * keys, 2.0 * (2 * nreq * min(kv_len, win + q_len) * Hkv * hd + q.numel() + o.numel()))
            ms = timed(lambda: ops.paged_attention(q, kp, vp, bt, cu, kvl, req, o, hd ** -0.5, win, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len, softcap=30.0, keep_first=4, sink=True))
            kern[f"murilorn_capped_sink_attention_{label}"] = roof(ms, *cost_w)
            # latent attention with sinks, beside the same kernel without (Kavenex's)
            LH, rank, rot = z["l_heads"], z["kv_rank"], z["rot_dim"]
            ql = torch.randn(n, LH, rank + rot, device=dev).to(bf)
            pool = torch.randn(nreq * pages, 1, ps, rank + rot, device=dev).to(bf)
            ol = torch.empty(n, LH * rank, dtype=bf, device=dev)
            lsinks = torch.randn(LH, device=dev)
            causal = nreq * sum(p + 1 for p in range(kv_len - q_len, kv_len))
            cost_l = (2.0 * LH * (2 * rank + rot) * causal, 2.0 * (nreq * kv_len * (rank + rot) + ql.numel() + ol.numel()))
            ms = timed(lambda: ops.paged_attention(ql, pool, pool, bt, cu, kvl, req, ol, 0.1, 0, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len, value_dim=rank, sink_values=lsinks))
            kern[f"latent_attention_with_sinks_{label}"] = roof(ms, *cost_l)
            ms = timed(lambda: ops.paged_attention(ql, pool, pool, bt, cu, kvl, req, ol, 0.1, 0, ps, nreq, q_len, kv_len, ws=ws,
                                                   min_q_len=q_len, value_dim=rank))
            kern[f"kavenex_latent_attention_{label}"] = roof(ms, *cost_l)
            # the projected row into queries and pages: convolved and normed here, biased there
            C = (H + 2 * Hkv) * hd
            row, bias = torch.randn(n, C, device=dev), torch.zeros(C, device=dev)
            cw, qw, kw = torch.randn(C, z["taps"], device=dev), torch.ones(hd, device=dev), torch.ones(hd, device=dev)
            cstate = torch.zeros(nreq, (z["taps"] - 1) * C, device=dev)
            vf = torch.randn(n, Hkv * hd, device=dev)
            moved = 4.0 * row.numel() + 2.0 * row.numel() + 4.0 * vf.numel() + 2 * 4.0 * cstate.numel()
            ms = timed(lambda: ops.conv_qkv_append(ctx, row, bias, cw, z["taps"], cstate, q, kp, vp, bt, H, Hkv, hd, hd, qw, kw, 1e-5, ps,
                                                   v_first_in=vf, mix=0.5))
            kern[f"convolve_norm_mix_store_{label}"] = roof(ms, 0, moved)
            ms = timed(lambda: ops.qkv_bias_append(row, bias, q, kp, vp, pos, req, bt, H, Hkv, hd, hd, ps))
            kern[f"murilorn_bias_store_{label}"] = roof(ms, 0, 4.0 * row.numel() + 2.0 * row.numel())
            # the recurrences: bytes are their rows in and out and the state
            G = z["gru"]
            proj = torch.randn(n, 3 * G, device=dev)
            bz, bu = torch.randn(G, device=dev), torch.randn(G, device=dev)
            gstate = torch.zeros(nreq, G, device=dev)
            go = torch.empty(n, G, dtype=bf, device=dev)
            ms = timed(lambda: ops.mingru(ctx, proj, (0, G, 2 * G), bz, bu, gstate, go))
            kern[f"gated_recurrence_{label}"] = roof(ms, 0, 4.0 * proj.numel() + 2.0 * go.numel() + 2 * 4.0 * gstate.numel())
            dH, dG, dd, dv, taps = z["d_heads"], z["d_kv_heads"], z["d_dim"], z["d_vdim"], z["taps"]
            DC = 2 * dG * dd + dH * dv
            conv_w, a_log, nw = torch.randn(DC, taps, device=dev) * 0.3, torch.randn(dH, device=dev) * 0.3, torch.ones(dv, device=dev)
            dstate = torch.zeros(nreq, dH * dd * dv + (taps - 1) * DC, device=dev)
            dproj, second = torch.randn(n, DC + dH, device=dev), torch.randn(n, dH * dd + dH * dv, device=dev)
            dtb, do = torch.randn(dH * dd, device=dev), torch.empty(n, dH * dv, dtype=bf, device=dev)
            ms = timed(lambda: ops.delta_rule(ctx, dproj, second, conv_w, a_log, dtb, nw, 1e-5, dstate, dH, dG, dd, dv, taps, do))
            kern[f"murilorn_channel_delta_rule_{label}"] = roof(ms, 0, 4.0 * (dproj.numel() + second.numel()) + 2.0 * do.numel()
                                                                + 2 * 4.0 * dstate.numel())
            del q, kp, vp, o, ql, pool, ol, row, proj, go, dproj, second, do
        # feed-forwards: xIELU of one product here, SiLU-gate of two in Llama's (the dense like kernel)
        FF = z["ff"]
        for label, M in (("2048_tokens", T), ("8_tokens", B)):
            h = torch.randn(M, W, device=dev).to(bf)
            x = torch.zeros(M, W, device=dev)
            up, dwn = (torch.randn(FF, W, device=dev) * 0.02).to(bf), (torch.randn(W, FF, device=dev) * 0.02).to(bf)
            act = torch.empty(M, FF, dtype=bf, device=dev)

            def plain():
                ops.linear_xielu(ctx, h, up, act, 0.7, 1.2)
                ops.linear(act, dwn, x, accumulate=True, alpha=0.5)

            kern[f"xielu_feed_forward_{label}"] = roof(timed(plain), 2.0 * M * 2 * FF * W, 2.0 * 2 * FF * W)
            g = ops.pack_gate_up((torch.randn(FF, W, device=dev) * 0.02).to(bf), (torch.randn(FF, W, device=dev) * 0.02).to(bf))

            def dense():
                ops.linear_gated(ctx, h, g, act, "silu", 0.0)
                ops.linear(act, dwn, x, accumulate=True)

            kern[f"llama_silu_feed_forward_{label}"] = roof(timed(dense), 2.0 * M * 3 * FF * W, 2.0 * 3 * FF * W)
            del up, dwn, g, act
        # what joins a sublayer to the residual: one pass that norms in place here; two streams written and read there
        wv = torch.ones(W, device=dev)
        xr, hb = torch.randn(T, W, device=dev), torch.empty(T, W, dtype=bf, device=dev)
        kern["norm_after_the_sum_2048_tokens"] = roof(timed(lambda: ops.post_norm(xr, None, 1.0, wv, 1e-5, rounded=hb)), 0,
                                                      (4.0 * 2 + 2.0) * T * W)
        S = 2
        xs, y = torch.randn(T, S, W, device=dev), torch.randn(T, W, device=dev)
        a_in, b_out, mix = torch.ones(S, device=dev), torch.ones(S, device=dev), torch.eye(S, device=dev).contiguous()
        on = torch.empty(T, W, dtype=bf, device=dev)
        kern["murilorn_streams_write_and_read_2048_tokens"] = roof(
            timed(lambda: ops.streams_update(xs, mix, b_out, y, next_in=a_in, norm_weight=wv, eps=1e-5, normed=on)), 0,
            (8.0 * S + 4.0 + 2.0) * T * W)
        LH, rank = z["l_heads"], z["kv_rank"]
        mixed, gl = torch.randn(T, LH * rank, device=dev).to(bf), torch.randn(T, LH, device=dev)
        kern["gate_per_head_2048_tokens"] = roof(timed(lambda: ops.group_gate_mul(mixed, gl, rank)), 0, 4.0 * T * LH * rank)
        rec["kernels"] = kern
        rec["config"] = {k: v for k, v in z.items()}
        out["sizes"][name] = rec
        del engines
        torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="tinyllama", choices=sorted(SHAPES),
                    help="layer sizes: one of the reference's published configurations")
    ap.add_argument("--only", choices=["prefill", "decode", "attention"], help="run one phase only (for profiling)")
    ap.add_argument("--batch", type=int, default=8, help="requests of the timed decode steps")
    ap.add_argument("--tokens", type=int, default=PREFILL_TOKENS, help="prompt tokens with --only prefill")
    ap.add_argument("--context", type=int, default=0, help="context reached with --only decode (default: the shape's); keys with --only attention")
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (reported beside the full number)")
    ap.add_argument("--design", choices=["kavenex", "murilorn", "luvapel", "midulorn"],
                    help="instead of the default workload: this design beside the Llama decoder (luvapel and midulorn: "
                         "beside Murilorn, the closest of the engine's models) at equal sizes")
    ap.add_argument("--size", default="", help="with --design: which of its sizes (2k, 4k; default both)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "hanumanit/garuda is a Rust crate without a Python package; no cargo/rustc here, "
                          "its dependencies are not vendored and there is no network, so it cannot be built"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine does not run on {args.gpus} GPUs")
        return 2
    args.warmup = max(args.warmup, 3)
    args.steps = max(1, min(args.steps, 512))
    if not 1 <= args.batch <= 64:
        print("bench.py: --batch must be 1 to 64")
        return 2
    if args.design:
        run = {"murilorn": run_design_murilorn, "luvapel": run_design_luvapel, "kavenex": run_design,
               "midulorn": run_design_midulorn}[args.design]
        print(json.dumps(run(args)))
        return 0
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
