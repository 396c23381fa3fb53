#!/usr/bin/env python3
"""Decode and prefill throughput of wick_b200 on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32
heads over 8 kv heads of 128, intermediate 12288, vocabulary 151936) with random
bfloat16 weights drawn on the device, a batch of 8 sequences with 512-token
random-id prompts, and a context of 4096 tokens per sequence.  A "step" is one
decode step of the whole batch.

``value``: decoded tokens per second, timed on the device with CUDA events over
exactly K steps (after W warm-up steps); ``e2e``: the same through the Python
entry point ``wick_b200.generate`` with token ids going in and coming out on the
host at every step.  ``prefill``: one 2,048-token prompt.  ``roofline``: the bytes
a decode step has to read (every weight it uses once, plus the cache of the
live requests) over its time, against the measured copy bandwidth.  ``points``:
decode at batch 1 and 64.  Every weight matrix is far larger than the L2 cache,
so consecutive steps never find their inputs there.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=12288, num_hidden_layers=36, vocab_size=151936,
                max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False)
CONTEXT = 4096
PROMPT = 512
PREFILL = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            j = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(j.get(k), (int, float)):
                out[k] = float(j[k])
        out["source"] = "measured"
        return out
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while it is open."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass
        return self

    def __exit__(self, *a):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                           "samples": len(sm)}


def reference_arm():
    # wick is a Rust program (Cargo.toml, no Python package): pip cannot build it
    # and this image has no cargo/rustc.
    print(json.dumps({"impl": "reference",
                      "unavailable": "pMag11-alt/wick is a Rust crate without a Python package; no cargo/rustc "
                                     "in this image, so it cannot be installed or run offline"}))
    return 0


def device_timed_decode(torch, wick, ops, eng, batch, steps, warmup, vocab, seed, prompt_len=PROMPT):
    """W + K decode steps of `batch` sequences after prompts of prompt_len tokens; returns
    (ms per step over the K timed steps, kernels launched in them, kv tokens read)."""
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in range(batch)]
    slots = [eng.open_seq() for _ in prompts]
    for s in slots:
        eng.cache.reserve(s, min(CONTEXT, prompt_len + warmup + steps + 1))
    # prompts in chunks of at most 8 sequences to bound activation memory
    tok = []
    for i in range(0, batch, 8):
        logits = eng.step(slots[i:i + 8], prompts[i:i + 8])
        tok += ops.argmax(logits).tolist()
    for _ in range(warmup):
        logits = eng.step(slots, [[t] for t in tok])
        tok = ops.argmax(logits).tolist()
    torch.cuda.synchronize()
    kv_tokens = sum(eng.seq_len(s) for s in slots) * steps + batch * steps * (steps + 1) // 2
    l0 = ops.launches[0]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        logits = eng.step(slots, [[t] for t in tok])
        tok = ops.argmax(logits).tolist()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = ops.launches[0] - l0
    for s in slots:
        eng.close_seq(s)
    return ms, launches, kv_tokens / steps


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of each prompt before the timed decode steps")
    ap.add_argument("--skip-points", action="store_true", help="no batch 1 / 64 runs")
    ap.add_argument("--skip-e2e", action="store_true", help="no run through the Python entry point")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-decode", action="store_true", help="prefill only (for profiling)")
    ap.add_argument("--eager", action="store_true", help="no CUDA graphs (every kernel is a launch of its own)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not built")
        return 2
    warmup = max(args.warmup, 3)
    steps = max(1, min(args.steps, CONTEXT - args.prompt_len - warmup - 2))

    import torch

    import wick_b200 as wick
    from wick_b200 import ops

    pk = peaks()
    cfg_json = dict(QWEN3_8B)
    full_layers = cfg_json["num_hidden_layers"]
    if args.layers:
        cfg_json["num_hidden_layers"] = args.layers
    cfg = wick.config_from_json(cfg_json)
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    per_seq = (args.prompt_len + 3 + steps + 64 + 63) // 64 * 64
    max_tokens = max(max_batch * per_seq, PREFILL + 64)
    t0 = time.time()
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens,
                                  use_graphs=False if args.eager else None)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    vocab = cfg.vocab_size
    weight_bytes = eng.model.weight_bytes_per_step()
    kv_bytes_per_token = eng.cache.bytes_per_token()

    # ---- decode, device-timed (the headline value) ----
    with Clocks() as clk:
        if args.skip_decode:
            ms, launches, kv_tokens = float("nan"), 0, 0
        else:
            ms, launches, kv_tokens = device_timed_decode(torch, wick, ops, eng, args.batch, steps, warmup, vocab, 1, args.prompt_len)
    value = args.batch * 1e3 / ms
    step_bytes = weight_bytes + kv_tokens * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # ---- decode through the Python entry point, host tokens in and out ----
    e2e_value = None
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist() for _ in range(args.batch)]
    opts = wick.GenOptions(max_tokens=steps + 1, sampler=wick.SamplerConfig.greedy(), context=CONTEXT,
                           max_batch=args.batch)
    if not args.skip_e2e and not args.skip_decode:
        wick.generate(eng, [p[:16] for p in prompts], wick.GenOptions(max_tokens=4, sampler=wick.SamplerConfig.greedy(),
                                                                      context=CONTEXT, max_batch=args.batch))
        res = wick.generate(eng, prompts, opts)
        gen_ms = max(r.gen_ms for r in res)
        e2e_value = sum(len(r.tokens) - 1 for r in res) / (gen_ms * 1e-3)
    from wick_b200.engine.batch import BatchLayout
    h2d = BatchLayout(args.batch, args.batch, 16, args.batch, args.batch).size * 4
    d2h = args.batch * 4

    # ---- prefill of one 2,048-token prompt ----
    g = torch.Generator().manual_seed(3)
    ptoks = torch.randint(0, vocab, (PREFILL,), generator=g).tolist()
    times = []
    for i in range(0 if args.skip_prefill else 2 + 3):
        s = eng.open_seq()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([s], [ptoks])
        e1.record()
        torch.cuda.synchronize()
        eng.close_seq(s)
        if i >= 2:
            times.append(e0.elapsed_time(e1))
    pms = statistics.median(times) if times else float("nan")
    c = cfg
    gemm_params = len(eng.spec.schedule) * (c.hidden_size * (2 * c.q_dim + 2 * c.kv_dim) + 3 * c.hidden_size * c.intermediate_size)
    flops = 2.0 * PREFILL * gemm_params + 2.0 * vocab * c.hidden_size            # head on one row
    flops += len(eng.spec.schedule) * 4.0 * c.num_attention_heads * c.head_dim * PREFILL * (PREFILL + 1) / 2
    prefill = {"value": PREFILL / (pms * 1e-3), "tokens": PREFILL, "ms": pms,
               "frac": flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
               "tflops": flops / (pms * 1e-3) / 1e12, "peak_tflops": pk["bf16_tflops_sustained"]}

    # ---- other batch sizes ----
    points = {}
    if not args.skip_points and not args.skip_decode:
        for b in (1, 64):
            pms_b, _, _ = device_timed_decode(torch, wick, ops, eng, b, min(steps, 64), warmup, vocab, 10 + b, args.prompt_len)
            points[f"decode_b{b}"] = b * 1e3 / pms_b

    line = {
        "metric": f"Qwen3-8B bf16 decode tok/s @ bs {args.batch} ({args.prompt_len}-token prompts, context {CONTEXT})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), seeded uniform random token ids",
        "config": {"model": "Qwen3-8B sizes", "layers": len(eng.spec.schedule), "layers_of_config": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": args.prompt_len, "parallelism": "none",
                   "l2": "inputs larger than L2 (weights per step far exceed 126 MB)",
                   "peaks": pk["source"]},
        "clocks": clk.result,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "load_s": load_s,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
