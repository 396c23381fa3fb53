#!/usr/bin/env python3
"""Decode and prefill throughput of wick_b200 on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--model 8b|14b|32b]

The default run has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32
heads over 8 kv heads of 128, intermediate 12288, vocabulary 151936) with random
bfloat16 weights drawn on the device, a batch of 8 sequences with 512-token
random-id prompts, and a context of 4096 tokens per sequence.  A "step" is one
decode step of the whole batch.

``value``: decoded tokens per second, timed on the device with CUDA events over
exactly K steps after W warm-up steps, as the median of three such regions
(``spread`` has the fastest and the slowest); ``e2e``: the same through the Python
entry point ``wick_b200.generate``, token ids going in and coming out on the host.
``prefill``: one 2,048-token prompt (median of 40 steps back to back, about a second).  ``roofline``: the bytes a
decode step has to read (every weight it uses once, plus the cache of the live
requests) over its time, against the measured copy bandwidth.  ``points``: decode
at batch 1 and 64, and the workloads at Qwen3-14B sizes (ragged batch of 16,
prompts of 64 to 2,048 tokens) and Qwen3-32B sizes (batch 8, 1,024-token prompts),
each with its fraction of the copy bandwidth.  Every weight matrix is far larger
than the L2 cache, so consecutive steps never find their inputs there.  The run
fails if any step it timed produced logits that are not finite.
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

def _qwen3(hidden, heads, kv_heads, intermediate, layers):
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=hidden, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=128, intermediate_size=intermediate, num_hidden_layers=layers,
                vocab_size=151936, max_position_embeddings=40960, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=False)


# The layer sizes of the three Qwen3 models measured here, and their workloads:
# 8b: batch 1 / 8 / 64, 512-token prompts (the headline is batch 8) and one 2,048-token prompt;
# 14b: a ragged batch of 16, prompt lengths uniform in [64, 2048] in one prompt step, 128 decode steps;
# 32b: a batch of 8 with 1,024-token prompts, 128 decode steps.
MODELS = {"8b": _qwen3(4096, 32, 8, 12288, 36), "14b": _qwen3(5120, 40, 8, 17408, 40),
          "32b": _qwen3(5120, 64, 8, 25600, 64)}
QWEN3_8B = MODELS["8b"]
CONTEXT = 4096
PROMPT = 512
PREFILL = 2048
REPEATS = 3
E2E_WARMUP = 24
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


def device_timed_decode(torch, wick, eng, prompts, steps, warmup, repeats=REPEATS):
    """The prompts in one step, W decode steps, then ``repeats`` timed regions of exactly
    ``steps`` decode steps each (CUDA events on the launching stream, a synchronize on both
    sides).  The batch is stepped the way ``wick_b200.generate`` steps it: the sampled token
    and the lengths stay on the device, the host launches a step ahead and reads every step's
    tokens from pinned memory one step behind.  Returns the regions' milliseconds per step, the
    kernels launched in one region, the cached tokens a step reads on average, the prompt
    step's milliseconds, and whether the last step's logits were finite."""
    from wick_b200 import ops
    batch = len(prompts)
    slots = [eng.open_seq() for _ in prompts]
    total = warmup + repeats * steps + 2
    for s, p in zip(slots, prompts):
        eng.cache.reserve(s, len(p) + total)
    run = eng.begin_run(wick.SamplerConfig.greedy(), ())
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run.start(slots, prompts, [1 << 30] * batch)
    e1.record()
    run.collect()
    prompt_ms = e0.elapsed_time(e1)
    for _ in range(warmup):
        run.launch(slots)
        run.collect()
    regions, launches, kv_tokens = [], 0, 0.0
    for _ in range(repeats):
        torch.cuda.synchronize()
        l0 = ops.launches[0]
        kv_tokens = sum(eng.seq_len(s) for s in slots) + batch * (steps + 1) / 2.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(steps):
            run.launch(slots)
            if k:
                run.collect()
        e1.record()
        run.collect()
        torch.cuda.synchronize()
        regions.append(e0.elapsed_time(e1) / steps)
        launches = ops.launches[0] - l0
    finite = run.last_logits is not None and bool(torch.isfinite(run.last_logits).all().item())
    eng.check_kernels()
    for s in slots:
        eng.close_seq(s)
    return regions, launches, kv_tokens, prompt_ms, finite


def decode_point(torch, wick, eng, pk, prompts, steps, warmup, repeats=REPEATS):
    """One decode workload as a dictionary: tokens a second (median region), spread, roofline."""
    regions, launches, kv_tokens, prompt_ms, finite = device_timed_decode(torch, wick, eng, prompts, steps, warmup, repeats)
    ms = statistics.median(regions)
    step_bytes = eng.model.weight_bytes_per_step() + eng.cache.read_bytes(int(kv_tokens), len(prompts))
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {"value": len(prompts) * 1e3 / ms, "ms_per_step": ms, "ms_min": min(regions), "ms_max": max(regions),
            "regions": len(regions), "gb_per_step": step_bytes / 1e9, "hbm_frac": achieved / pk["hbm_gbs"],
            "achieved_gbs": achieved, "launches": launches, "prompt_ms": prompt_ms, "finite": finite}


def random_prompts(torch, vocab, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in lens]


def other_model(torch, wick, pk, name, steps, warmup, layers=None):
    """The 14b / 32b workload on an engine of its own (built here, dropped afterwards)."""
    cfg_json = dict(MODELS[name])
    full = cfg_json["num_hidden_layers"]
    if layers:
        cfg_json["num_hidden_layers"] = min(layers, full)
    cfg = wick.config_from_json(cfg_json)
    if name == "14b":
        g = torch.Generator().manual_seed(14)
        lens = torch.randint(64, 2049, (16,), generator=g).tolist()
    else:
        lens = [1024] * 8
    need = sum((n + warmup + REPEATS * steps + 2 + 63) // 64 * 64 for n in lens)
    t0 = time.time()
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=need)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    out = decode_point(torch, wick, eng, pk, random_prompts(torch, cfg.vocab_size, lens, 15), steps, warmup)
    out.update({"layers": len(eng.spec.schedule), "layers_of_config": full, "batch": len(lens),
                "prompt_tokens": sum(lens), "load_s": load_s,
                "prompt_tok_s": sum(lens) / (out["prompt_ms"] * 1e-3)})
    del eng
    torch.cuda.empty_cache()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="8b", choices=sorted(MODELS), help="8b: the headline line with all its parts; "
                    "14b / 32b: only that model's workload, as a line of its own")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of each prompt before the timed decode steps")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL, help="tokens of the prefill step (the contract's is 2,048)")
    ap.add_argument("--repeats", type=int, default=REPEATS, help="timed regions of --steps decode steps each (median reported)")
    ap.add_argument("--skip-points", action="store_true", help="no batch 1 / 64 runs")
    ap.add_argument("--skip-models", action="store_true", help="no 14b / 32b workloads")
    ap.add_argument("--skip-e2e", action="store_true", help="no run through the Python entry point")
    ap.add_argument("--prefill-steps", type=int, default=0, help="timed prompt steps (default: about a second's worth, at most 40)")
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
    repeats = max(1, args.repeats)
    steps = max(1, min(args.steps, (CONTEXT - args.prompt_len - max(warmup, E2E_WARMUP) - 2) // repeats))

    import torch

    import wick_b200 as wick
    from wick_b200 import ops

    pk = peaks()
    if args.model != "8b":
        with Clocks() as clk:
            out = other_model(torch, wick, pk, args.model, steps, warmup, args.layers)
        out.update({"metric": f"Qwen3-{args.model.upper()} sizes bf16 decode tok/s", "unit": "tokens/s", "clocks": clk.result,
                    "peaks": pk["source"]})
        print(json.dumps(out))
        return 0
    cfg_json = dict(QWEN3_8B)
    full_layers = cfg_json["num_hidden_layers"]
    if args.layers:
        cfg_json["num_hidden_layers"] = args.layers
    cfg = wick.config_from_json(cfg_json)
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    per_seq = (args.prompt_len + warmup + repeats * steps + 2 + 64 + 63) // 64 * 64
    n_prefill = args.prefill_tokens
    max_tokens = max(max_batch * per_seq, n_prefill + 64)
    t0 = time.time()
    eng = wick.Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens,
                                  use_graphs=False if args.eager else None)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    vocab = cfg.vocab_size

    # ---- decode, device-timed (the headline value) ----
    with Clocks() as clk:
        if args.skip_decode:
            head = {"value": float("nan"), "ms_per_step": float("nan"), "launches": 0, "achieved_gbs": float("nan"),
                    "hbm_frac": float("nan"), "gb_per_step": float("nan"), "finite": True, "ms_min": None, "ms_max": None}
        else:
            head = decode_point(torch, wick, eng, pk, random_prompts(torch, vocab, [args.prompt_len] * args.batch, 1),
                                steps, warmup, repeats)
    ms = head["ms_per_step"]

    # ---- decode through the Python entry point, host tokens in and out ----
    # One generate() call per region: the prompts, E2E_WARMUP untimed decode steps (the steps
    # right after a prompt step run up to 15 % slower for some 20 steps while the clocks
    # recover from the prompt's power draw; the device-timed regions leave them out through
    # their warm-up steps too), then exactly K steps timed on the host's clock between the
    # loop's per-step callbacks.  Every step's ids reach the host before its callback runs.
    e2e_value, e2e_whole, h2d, d2h = None, None, None, None
    e2e_warmup = max(warmup, E2E_WARMUP)
    prompts = random_prompts(torch, vocab, [args.prompt_len] * args.batch, 2)
    opts = wick.GenOptions(max_tokens=1 + e2e_warmup + steps, sampler=wick.SamplerConfig.greedy(), context=CONTEXT,
                           max_batch=args.batch)
    if not args.skip_e2e and not args.skip_decode:
        wick.generate(eng, [p[:16] for p in prompts], wick.GenOptions(max_tokens=4, sampler=wick.SamplerConfig.greedy(),
                                                                      context=CONTEXT, max_batch=args.batch))
        runs = []
        begin = eng.begin_run
        eng.begin_run = lambda *a, **kw: runs.append(begin(*a, **kw)) or runs[-1]
        vals, whole = [], []
        for _ in range(repeats):
            stamps = []
            res = wick.generate(eng, prompts, opts, on_step=lambda n, live: stamps.append(time.perf_counter()))
            assert len(stamps) == 1 + e2e_warmup + steps and all(len(r.tokens) == 1 + e2e_warmup + steps for r in res)
            vals.append(args.batch * steps / (stamps[-1] - stamps[e2e_warmup]))
            whole.append(sum(len(r.tokens) - 1 for r in res) / (max(r.gen_ms for r in res) * 1e-3))
        del eng.begin_run
        e2e_value, e2e_whole = statistics.median(vals), statistics.median(whole)
        # what crosses the bus: the prompts' description once, a description of the decode batch
        # when its composition changes, and the sampled ids (with a status word) every step
        h2d = sum(r.h2d_bytes for r in runs) / (repeats * (1 + e2e_warmup + steps))
        d2h = (args.batch + 1) * 4

    # ---- prefill of one 2,048-token prompt ----
    ptoks = random_prompts(torch, vocab, [n_prefill], 3)[0]
    times = []
    # The fraction is of the peak SUSTAINED under the power cap (a seconds-long loop of products), so the prompt
    # step is timed in the same state: after 3 warm-up steps, a second or so of steps back to back (the first
    # steps of a product-heavy phase run at the part's full clock, the next ones while the power control settles).
    pf_warm = 3
    pf_timed = 0 if args.skip_prefill else (args.prefill_steps or max(5, min(40, int(40 * 2048 / max(n_prefill, 1)))))
    for i in range(0 if args.skip_prefill else pf_warm + pf_timed):
        s = eng.open_seq()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        plog = eng.step([s], [ptoks])
        e1.record()
        torch.cuda.synchronize()
        eng.close_seq(s)
        if i >= pf_warm:
            times.append(e0.elapsed_time(e1))
            head["finite"] = head["finite"] and bool(torch.isfinite(plog).all().item())
    pms = statistics.median(times) if times else float("nan")
    c = cfg
    gemm_params = len(eng.spec.schedule) * (c.hidden_size * (2 * c.q_dim + 2 * c.kv_dim) + 3 * c.hidden_size * c.intermediate_size)
    flops = 2.0 * n_prefill * gemm_params + 2.0 * vocab * c.hidden_size            # head on one row
    flops += len(eng.spec.schedule) * 4.0 * c.num_attention_heads * c.head_dim * n_prefill * (n_prefill + 1) / 2
    prefill = {"value": n_prefill / (pms * 1e-3), "tokens": n_prefill, "ms": pms,
               "frac": flops / (pms * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
               "tflops": flops / (pms * 1e-3) / 1e12, "peak_tflops": pk["bf16_tflops_sustained"],
               "ms_min": min(times) if times else None, "ms_max": max(times) if times else None, "timed_steps": len(times)}

    # ---- other batch sizes, other models ----
    points = {}
    if not args.skip_points and not args.skip_decode:
        for b in (1, 64):
            pt = decode_point(torch, wick, eng, pk, random_prompts(torch, vocab, [args.prompt_len] * b, 10 + b),
                              min(steps, 64), warmup, repeats)
            points[f"decode_b{b}"] = pt["value"]
            points[f"decode_b{b}_hbm_frac"] = pt["hbm_frac"]
            head["finite"] = head["finite"] and pt["finite"]
    n_layers = len(eng.spec.schedule)
    del eng
    torch.cuda.empty_cache()
    if not args.skip_models and not args.skip_decode and not args.layers:
        for name in ("14b", "32b"):
            pt = other_model(torch, wick, pk, name, min(steps, 128), warmup)
            points[f"qwen3_{name}_decode"] = pt["value"]
            points[f"qwen3_{name}_hbm_frac"] = pt["hbm_frac"]
            points[f"qwen3_{name}_ms_per_step"] = pt["ms_per_step"]
            points[f"qwen3_{name}_prompt_tok_s"] = pt["prompt_tok_s"]
            head["finite"] = head["finite"] and pt["finite"]
    if not head["finite"]:
        print("bench.py: a step produced logits that are not finite", file=sys.stderr)
        return 1

    line = {
        "metric": f"Qwen3-8B bf16 decode tok/s @ bs {args.batch} ({args.prompt_len}-token prompts, context {CONTEXT})",
        "value": head["value"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), seeded uniform random token ids",
        "config": {"model": "Qwen3-8B sizes", "layers": n_layers, "layers_of_config": full_layers,
                   "hidden": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": vocab,
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": args.prompt_len, "parallelism": "none",
                   "l2": "inputs larger than L2 (weights per step far exceed 126 MB)",
                   "peaks": pk["source"], "timed_regions": repeats,
                   "points_models": "qwen3_14b: 40 layers, ragged batch 16, prompts U[64,2048]; qwen3_32b: 64 layers, "
                                    "batch 8, 1024-token prompts; 128 decode steps each"},
        "spread": {"ms_min": head["ms_min"], "ms_max": head["ms_max"], "regions": repeats},
        "clocks": clk.result,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "warmup_steps": e2e_warmup, "from_first_token": e2e_whole,
                "note": "wick_b200.generate, host clock over the last K steps of each call; prompt ids and the batch "
                        "description go to the device when a batch starts or changes, every step's sampled ids "
                        "come back through pinned memory; from_first_token counts every decode step of the call"},
        "gpu_launches": head["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": head["achieved_gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": head["hbm_frac"], "bytes_per_step": head["gb_per_step"] * 1e9},
        "points": points,
        "load_s": load_s,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
