#!/usr/bin/env python3
"""Decode and prefill throughput of the Gemma-2-2B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 (device-timed with CUDA
events around exactly K single-token steps after W warm-up steps, from 2,048-token prompts, cache
sized for the context length of 8,192).  `e2e` is the same through the Python entry point
(`Generator.generate_batch`): host token lists in, host token lists out, every step copying its
batch description from pinned host memory and reading the sampled tokens back.  `prefill` is one
2,048-token prompt in one step; `points` holds decode at batch 1 and 64; `roofline` compares the
bytes a decode step must read (every weight once, the cache of the live requests) with its time.
A decode step reads 5.2 GB of weights, far more than the 126 MB L2, so nothing stays cached
between timed iterations.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Gemma 2 2B shape
GEMMA2_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 26, "hidden_size": 2304, "num_attention_heads": 8, "num_key_value_heads": 4,
    "head_dim": 256, "intermediate_size": 9216, "vocab_size": 256000, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "sliding_window": 4096, "query_pre_attn_scalar": 256,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "max_position_embeddings": 8192,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "bos_token_id": 2, "eos_token_id": 1,
}
# BASELINE.json configs[3] and [4]: the 9B and 27B shapes
GEMMA2_9B = dict(GEMMA2_2B, num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8,
                 head_dim=256, intermediate_size=14336, query_pre_attn_scalar=256)
GEMMA2_27B = dict(GEMMA2_2B, num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16,
                  head_dim=128, intermediate_size=36864, query_pre_attn_scalar=144)
CONTEXT = 8192
PROMPT = 2048
NEW_TOKENS = 128
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed regions run."""
    FIELDS = ["clocks.sm", "clocks.max.sm", "power.draw", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=" + ",".join(self.FIELDS),
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != len(self.FIELDS):
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:]):
                if val == "Active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(spec, element_size=2):
    total = 0
    for t in spec.tensor_specs().values():
        n = 1
        for s in t.shape:
            n *= s
        total += n * element_size
    return total


def cache_bytes_read(cfg, layers, lengths, element_size=2):
    """Bytes of keys and values a decode step reads for sequences of the given lengths."""
    per_key = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * element_size
    total = 0
    for i in range(layers):
        local = cfg["sliding_window"] is not None and i % 2 == 0
        for n in lengths:
            total += per_key * (min(n, cfg["sliding_window"]) if local else n)
    return total


def prefill_flops(cfg, layers, T):
    H, nh, nkv, hd, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                            cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    linear = 2 * T * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I) * layers
    attn = 0
    for i in range(layers):
        local = cfg["sliding_window"] is not None and i % 2 == 0
        keys = sum(min(p + 1, cfg["sliding_window"]) if local else p + 1 for p in range(T))
        attn += 4 * nh * hd * keys
    return linear + attn + 2 * V * H      # logits at the last row only


def decode_run(engine, batch, steps, warmup, vocab, torch, rng, prompt_len=PROMPT):
    """Prefill `batch` prompts of `prompt_len` tokens, then time `steps` single-token steps on the device."""
    slots = [engine.new_sequence() for _ in range(batch)]
    prompts = [[int(v) for v in rng.integers(0, vocab, size=prompt_len)] for _ in range(batch)]
    engine.step(slots, prompts, [[] for _ in slots])
    feed = [[[int(v)] for v in rng.integers(0, vocab, size=batch)] for _ in range(steps + warmup)]
    from rust_deeplearning_b200.kernels import library
    for k in range(warmup):
        engine.step(slots, feed[k], "last")
    torch.cuda.synchronize()
    launches0 = library.launch_count
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(warmup, warmup + steps):
        engine.step(slots, feed[k], "last")
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    launches = library.launch_count - launches0
    lengths = [engine.length(s) for s in slots]
    for s in slots:
        engine.release(s)
    mid = [n - steps // 2 for n in lengths]
    return ms, launches, mid


def spread(lo, hi, n):
    """n prompt lengths from lo to hi in equal steps."""
    return [lo + (hi - lo) * i // (n - 1) for i in range(n)]


def workload(cfg, prompt_lens, new_tokens, pk, torch, rng, seed=0):
    """One of the larger shapes end to end on the engine: all prompts in one step (device-timed), then
    `new_tokens` single-token steps; the steps around the middle of the run are timed on the device.
    Returns a flat dict of figures."""
    import gc
    from rust_deeplearning_b200 import Engine, random_model
    from rust_deeplearning_b200.config.base import architecture_for
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    model = random_model(cfg, seed=seed, dtype="bfloat16", device="cuda:0")
    torch.cuda.synchronize()
    load_peak = torch.cuda.max_memory_allocated()
    arch = architecture_for(cfg)
    wbytes = weight_bytes(arch.build_spec(arch.parse_config(cfg)))
    V, L = cfg["vocab_size"], cfg["num_hidden_layers"]
    longest = max(prompt_lens) + new_tokens
    per_seq = [-(-(n + new_tokens) // 64) * 64 for n in prompt_lens]
    engine = Engine(model, max_tokens=sum(per_seq), max_seqs=len(prompt_lens), max_context=-(-longest // 64) * 64)
    prompts = [[int(v) for v in rng.integers(0, V, size=n)] for n in prompt_lens]
    slots = [engine.new_sequence() for _ in prompts]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    p0, p1 = ev(), ev()
    torch.cuda.synchronize()
    p0.record()
    engine.step(slots, prompts, "last")
    p1.record()
    torch.cuda.synchronize()
    prefill_ms = p0.elapsed_time(p1)
    first = max(3, new_tokens // 2 - 10)             # the timed steps lie around the middle of the run
    timed = min(20, new_tokens - 1 - first)
    feed = rng.integers(0, V, size=(new_tokens - 1, len(prompts)))
    t0, t1 = ev(), ev()
    for k in range(new_tokens - 1):
        if k == first:
            t0.record()
        if k == first + timed:
            t1.record()
        engine.step(slots, [[int(v)] for v in feed[k]], "last")
    if first + timed >= new_tokens - 1:
        t1.record()
    torch.cuda.synchronize()
    engine.check_status()
    ms = t0.elapsed_time(t1) / timed
    mid = [n + first + timed // 2 for n in prompt_lens]
    step_bytes = wbytes + cache_bytes_read(cfg, L, mid)
    out = {"layers": L, "prompts": f"{len(prompt_lens)} of {min(prompt_lens)}..{max(prompt_lens)} tokens", "new_tokens": new_tokens,
           "decode_tok_s": round(len(prompts) / (ms * 1e-3), 1), "decode_ms_per_step": round(ms, 3),
           "decode_step_gb": round(step_bytes / 1e9, 2),
           "decode_hbm_frac": round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
           "prefill_tokens": sum(prompt_lens), "prefill_ms": round(prefill_ms, 1),
           "prefill_tok_s": round(sum(prompt_lens) / (prefill_ms * 1e-3), 1),
           "weights_gb": round(wbytes / 1e9, 2), "load_peak_gb": round(load_peak / 1e9, 2),
           "cache_gb": round(engine.cache.nbytes() / 1e9, 2)}
    for s in slots:
        engine.release(s)
    del engine, model
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one small case (for profiling) and print a short line instead of the full record")
    ap.add_argument("--batch", type=int, default=8, help="batch of the --only decode case")
    ap.add_argument("--context", type=int, default=PROMPT, help="prompt length of the --only decode case")
    ap.add_argument("--no-large", action="store_true", help="leave out the 9B and 27B shapes and the long contexts")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (no Python package, no GPU code); no cargo/rustc in this image, "
                          "pip install of the reference tree fails: neither setup.py nor pyproject.toml"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library is single-GPU by design (got --gpus {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.steps + args.warmup > NEW_TOKENS - 1:
        args.steps = NEW_TOKENS - 1 - args.warmup

    import numpy as np
    import torch
    from rust_deeplearning_b200 import Engine, Generator, random_model
    from rust_deeplearning_b200.config.base import architecture_for
    from rust_deeplearning_b200.kernels import library

    cfg = dict(GEMMA2_2B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    rng = np.random.default_rng(0)
    torch.cuda.set_device(0)
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    wbytes = weight_bytes(spec)
    V = cfg["vocab_size"]

    if args.only is not None:
        # one case, few steps: what a profiler is pointed at
        engine = Engine(model, max_tokens=args.batch * CONTEXT, max_seqs=args.batch, max_context=CONTEXT)
        if args.only == "decode":
            ms, launches, _ = decode_run(engine, args.batch, args.steps, args.warmup, V, torch, rng, args.context)
            print(json.dumps({"case": "decode", "batch": args.batch, "context": args.context, "layers": layers, "ms_per_step": round(ms, 4),
                              "tokens_per_s": round(args.batch / (ms * 1e-3), 1), "launches": launches}))
        else:
            prompt = [int(v) for v in rng.integers(0, V, size=PROMPT)]
            for _ in range(args.warmup + args.steps):
                slot = engine.new_sequence()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                start.record()
                engine.step([slot], [prompt], "last")
                stop.record()
                host_ms = (time.perf_counter() - t0) * 1e3     # the host's share: validation, batch description, launches
                torch.cuda.synchronize()
                engine.release(slot)
            print(json.dumps({"case": "prefill", "tokens": PROMPT, "layers": layers, "ms": round(start.elapsed_time(stop), 3),
                              "host_ms": round(host_ms, 3)}))
        return 0

    clocks = ClockSampler()
    clocks.start()

    # ---- decode, device-timed: batch 8 (the headline), 1 and 64 ----
    engine = Engine(model, max_tokens=64 * CONTEXT, max_seqs=64, max_context=CONTEXT)
    ms8, launches, mid8 = decode_run(engine, 8, args.steps, args.warmup, V, torch, rng)
    # ---- end to end through the Python entry point: host tokens in and out ----
    # (right after the device-timed run of the same batch, so that both see the same clocks)
    gen = Generator(model, max_cache_tokens=8 * CONTEXT, max_batch=8, max_context=CONTEXT).with_temperature(0.0)
    gen.with_stop_tokens([])
    prompts = [[int(v) for v in rng.integers(0, V, size=PROMPT)] for _ in range(8)]
    marks = {}
    count = [0]
    first, last = 8 * args.warmup, 8 * (args.warmup + args.steps)

    def on_token(_req, _tok):
        count[0] += 1
        if count[0] == first:
            marks["t0"] = time.perf_counter()
        elif count[0] == last:
            marks["t1"] = time.perf_counter()

    gen.generate_batch_results(prompts, args.warmup + args.steps + 1, stream=on_token)
    e2e_tps = 8 * args.steps / (marks["t1"] - marks["t0"])
    h2d = next(iter(gen.engine._graphs.values())).layout.size * 4 if gen.engine._graphs else 0
    del gen
    torch.cuda.empty_cache()

    side = min(args.steps, 50)
    ms1, _, _ = decode_run(engine, 1, side, args.warmup, V, torch, rng)
    ms64, _, mid64 = decode_run(engine, 64, side, args.warmup, V, torch, rng)

    # ---- prefill: one prompt of 2,048 tokens in one step ----
    prompt = [int(v) for v in rng.integers(0, V, size=PROMPT)]
    times = []
    for k in range(3 + 5):
        slot = engine.new_sequence()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([slot], [prompt], "last")
        stop.record()
        torch.cuda.synchronize()
        engine.release(slot)
        if k >= 3:
            times.append(start.elapsed_time(stop))
    prefill_ms = statistics.median(times)
    pflops = prefill_flops(cfg, layers, PROMPT)

    # ---- long contexts on the same model: decode above the window (the windowed layers' ring is in use), a long prompt ----
    long_points = {}
    if not args.no_large:
        LONG = 6000
        for b in (1, 8):
            ms, _, mid = decode_run(engine, b, 20, 3, V, torch, rng, LONG)
            long_points[f"decode_b{b}_ctx{LONG}"] = round(b / (ms * 1e-3), 1)
            long_points[f"decode_b{b}_ctx{LONG}_hbm_frac"] = round((wbytes + cache_bytes_read(cfg, layers, mid)) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        long_prompt = [int(v) for v in rng.integers(0, V, size=CONTEXT)]
        times8k = []
        for k in range(3):
            slot = engine.new_sequence()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            engine.step([slot], [long_prompt], "last")
            stop.record()
            torch.cuda.synchronize()
            engine.release(slot)
            if k >= 1:
                times8k.append(start.elapsed_time(stop))
        ms8k = statistics.median(times8k)
        long_points[f"prefill_{CONTEXT}_tok_s"] = round(CONTEXT / (ms8k * 1e-3), 1)
        long_points[f"prefill_{CONTEXT}_frac"] = round(prefill_flops(cfg, layers, CONTEXT) / (ms8k * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)

    # ---- the larger shapes of the reference's list: 9B (8 unequal prompts, 256 new) and 27B (16 prompts, 128 new) ----
    large = {}
    if not args.no_large and args.layers is None:
        del engine, model
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for name, shape, lens, new in (("gemma2_9b", GEMMA2_9B, spread(64, 6000, 8), 256),
                                       ("gemma2_27b", GEMMA2_27B, spread(1024, 4096, 16), 128)):
            try:
                large[name] = workload(shape, lens, new, pk, torch, rng)
            except Exception as e:      # the headline above stands whatever becomes of the larger shapes
                large[name] = {"error": f"{type(e).__name__}: {e}"[:200]}
                gc.collect()
                torch.cuda.empty_cache()
    clock_info = clocks.stop()

    step_bytes = wbytes + cache_bytes_read(cfg, layers, mid8)
    achieved = step_bytes / (ms8 * 1e-3) / 1e9
    value = 8 / (ms8 * 1e-3)
    out = {
        "metric": "Gemma2-2B decode tok/s @ batch 8 (prefill tok/s @ 2,048 tokens and batch 1/64 alongside)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), seeded uniform-random token ids",
        "config": {
            "model": "Gemma 2 2B shape", "layers": layers, "layers_in_configuration": full_layers,
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": V,
            "sliding_window": cfg["sliding_window"], "global_batch": 8, "seq_len": CONTEXT, "prompt_len": PROMPT,
            "new_tokens": NEW_TOKENS, "parallelism": "single GPU", "cache": "paged, 64 positions a page, sized for 8192 a sequence",
            "l2": "inputs larger than L2: 5.2 GB of weights read per step",
            "points_long": "2B shape: decode at batch 1 and 8 from 6000-token prompts, one prompt of 8192 tokens",
            "points_9b": "42 layers, hidden 3584, 16/8 heads, head 256, intermediate 14336; 8 prompts 64..6000, 256 new",
            "points_27b": "46 layers, hidden 4608, 32/16 heads, head 128, intermediate 36864; 16 prompts 1024..4096, 128 new",
        },
        "clocks": clock_info,
        "e2e": {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8 * 4},
        "gpu_launches": launches,
        "prefill": {"value": round(PROMPT / (prefill_ms * 1e-3), 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(pflops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": {"decode_b1": round(1 / (ms1 * 1e-3), 1), "decode_b64": round(64 / (ms64 * 1e-3), 1),
                   "decode_b64_hbm_frac": round((wbytes + cache_bytes_read(cfg, layers, mid64)) / (ms64 * 1e-3) / 1e9
                                                / pk["hbm_gbs"], 4),
                   "decode_b1_hbm_frac": round((wbytes + cache_bytes_read(cfg, layers, [PROMPT + NEW_TOKENS // 2])) / (ms1 * 1e-3) / 1e9
                                               / pk["hbm_gbs"], 4)},
    }
    out["points"].update(long_points)
    for name, figures in large.items():
        for k, v in figures.items():
            out["points"][f"{name}_{k}"] = v
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
