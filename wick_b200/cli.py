"""The ``wick`` command line, in the manner of wick's ``src/main.rs``.

Option names, defaults and exit codes are wick's where it has them
(``main.rs:12-40,60-120,319-343``): ``-n/--max-tokens`` 256, ``-t/--temperature``
0.7 (0 = greedy), ``--top-k`` 40, ``--top-p`` 0.9, ``--min-p`` 0, ``--repeat-penalty``
1.0, ``--seed``, ``-q/--quant`` (here ``bf16`` or ``f32``), ``-c/--context`` 4096,
``--prompt-len`` 128; usage errors exit with 2, other errors with 1; the banner
and the statistics go to stderr, results to stdout.  Prompts are token ids (the
tokenizer is not part of this library): ``--ids 1,2,3`` once per prompt, or
``--ids-file`` with a JSON list of lists.
"""
from __future__ import annotations

import json
import sys
import time
from typing import List, Optional

USAGE = """\
wick: run Qwen3 language models on one NVIDIA B200

usage:
  wick run    <model-dir> --ids 1,2,3 [--ids 4,5 ...]   generate continuations of token-id prompts
  wick bench  <model-dir>                               prompt and generation speed
  wick random <out-dir> --config <config.json>          write a model folder with random weights

options:
      --ids <a,b,c>        a prompt as token ids (repeat for a batch)
      --ids-file <path>    JSON list of prompts (lists of token ids)
  -n, --max-tokens <n>     tokens to generate (default 256)
  -t, --temperature <x>    sampling temperature, 0 = greedy (default 0.7)
      --top-k <n>          (default 40)     --top-p <x>   (default 0.9)
      --min-p <x>          (default 0)      --repeat-penalty <x> (default 1.0)
      --seed <n>           RNG seed
      --stop-id <id>       extra stop token (repeatable; the config's eos ids always stop)
  -q, --quant <fmt>        weights and activations: bf16 (default) or f32
  -c, --context <n>        context length per sequence (default 4096)
      --batch <n>          sequences that start together (default 64; bench: 1)
      --prompt-len <n>     bench: prompt tokens (default 128)
      --config <path>      random: the config.json to draw weights for
"""


class UsageError(Exception):
    pass


class Args:
    def __init__(self):
        from .sampling.sampler import SamplerConfig
        self.cmd = ""
        self.dir = ""
        self.prompts: List[List[int]] = []
        self.max_tokens = 256
        self.sampler = SamplerConfig()
        self.stop_ids: List[int] = []
        self.quant = "bf16"
        self.context = 4096
        self.batch: Optional[int] = None
        self.prompt_len = 128
        self.config: Optional[str] = None


def _ids(text: str) -> List[int]:
    try:
        return [int(x) for x in text.replace(" ", "").split(",") if x != ""]
    except ValueError:
        raise UsageError(f"bad value for --ids: {text}") from None


def parse_args(argv: List[str]) -> Args:
    if not argv or argv[0] in ("-h", "--help", "help"):
        raise UsageError(USAGE)
    a = Args()
    a.cmd = argv[0]
    it = iter(argv[1:])
    positional = []

    def num(kind, name):
        try:
            v = next(it)
        except StopIteration:
            raise UsageError(f"{name} needs a value") from None
        try:
            return kind(v, 0) if kind is int else kind(v)
        except ValueError:
            raise UsageError(f"bad value for {name}: {v}") from None

    for arg in it:
        if arg == "--ids":
            a.prompts.append(_ids(num(str, arg)))
        elif arg == "--ids-file":
            path = num(str, arg)
            try:
                data = json.load(open(path))
                a.prompts += [[int(t) for t in p] for p in data]
            except (OSError, ValueError, TypeError) as e:
                raise UsageError(f"{path}: {e}") from None
        elif arg in ("-n", "--max-tokens"):
            a.max_tokens = num(int, arg)
        elif arg in ("-t", "--temperature"):
            a.sampler.temperature = num(float, arg)
        elif arg == "--top-k":
            a.sampler.top_k = num(int, arg)
        elif arg == "--top-p":
            a.sampler.top_p = num(float, arg)
        elif arg == "--min-p":
            a.sampler.min_p = num(float, arg)
        elif arg == "--repeat-penalty":
            a.sampler.repetition_penalty = num(float, arg)
        elif arg == "--seed":
            a.sampler.seed = num(int, arg)
        elif arg == "--stop-id":
            a.stop_ids.append(num(int, arg))
        elif arg in ("-q", "--quant"):
            v = num(str, arg).lower()
            if v in ("q8", "q8_0", "q4", "q4_0"):
                raise UsageError(f"unsupported format {v}: quantized weights are not built (bf16, f32)")
            if v not in ("bf16", "f32"):
                raise UsageError(f"unknown format {v} (bf16, f32)")
            a.quant = v
        elif arg in ("-c", "--context"):
            a.context = num(int, arg)
        elif arg == "--batch":
            a.batch = num(int, arg)
        elif arg == "--prompt-len":
            a.prompt_len = num(int, arg)
        elif arg == "--config":
            a.config = num(str, arg)
        elif arg.startswith("-") and len(arg) > 1:
            raise UsageError(f"unknown option {arg}\n\n{USAGE}")
        else:
            positional.append(arg)
    if not positional:
        raise UsageError(f"missing <model-dir>\n\n{USAGE}")
    a.dir = positional[0]
    return a


def _load(a: Args, max_tokens: int):
    import os

    import wick_b200 as wick
    t0 = time.perf_counter()
    eng = wick.Engine.from_dir(a.dir, dtype=a.quant, max_tokens=max_tokens)
    cfg = eng.config
    name = os.path.basename(os.path.normpath(a.dir)) or "model"
    params = cfg.param_count(getattr(eng.model.head, "is_tied", None)) if hasattr(cfg, "param_count") else 0
    print(f"wick: {name} ({params / 1e6:.0f}M params, {len(eng.spec.schedule)} layers, "
          f"{eng.spec.architecture}) as {a.quant}, {eng.model.weight_bytes_per_step() / 2**30:.1f} GiB, "
          f"sm_100a kernels, cache of {eng.cache.max_tokens} tokens, loaded in "
          f"{(time.perf_counter() - t0) * 1e3:.0f} ms", file=sys.stderr)
    return eng


def cmd_run(a: Args) -> None:
    import wick_b200 as wick
    if not a.prompts:
        raise UsageError("run needs --ids <a,b,c> or --ids-file <path>")
    batch = a.batch or 64
    per_seq = [min(a.context, len(p) + a.max_tokens) for p in a.prompts]
    need = sum(sorted(((n + 63) // 64 * 64 for n in per_seq), reverse=True)[:batch])
    eng = _load(a, max(need, 64))
    # (the model's own end-of-sequence ids are added by the generation loop)
    opts = wick.GenOptions(max_tokens=a.max_tokens, sampler=a.sampler, stop_token_ids=a.stop_ids, context=a.context,
                           max_batch=batch)
    res = wick.generate(eng, a.prompts, opts)
    for r in res:
        print(json.dumps(r.tokens))
    for r in res:
        print(f"[{r.prompt_tokens} prompt tokens (0 cached) at {r.prompt_tps():.1f} tok/s, {len(r.tokens)} generated "
              f"at {r.gen_tps():.1f} tok/s, {r.finish.capitalize()}]", file=sys.stderr)


def cmd_bench(a: Args) -> None:
    """main.rs:223-259: a warm-up pass, a timed prompt, a timed greedy generation."""
    import torch

    import wick_b200 as wick
    from . import ops
    batch = a.batch or 1
    n, n_gen = a.prompt_len, min(a.max_tokens, 128)
    per_seq = (n + n_gen + 8 + 63) // 64 * 64
    eng = _load(a, per_seq * batch)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, eng.spec.vocab, (n,), generator=g).tolist() for _ in range(batch)]
    greedy = wick.GenOptions(max_tokens=2, sampler=wick.SamplerConfig.greedy(), context=n + n_gen + 8, max_batch=batch)
    wick.generate(eng, [p[:8] for p in prompts], greedy)                 # warm-up
    slots = [eng.open_seq() for _ in prompts]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    logits = eng.step(slots, prompts)
    tok = ops.argmax(logits).tolist()
    torch.cuda.synchronize()
    pp = time.perf_counter() - t0
    t1 = time.perf_counter()
    for _ in range(n_gen):
        logits = eng.step(slots, [[t] for t in tok])
        tok = ops.argmax(logits).tolist()
    torch.cuda.synchronize()
    tg = time.perf_counter() - t1
    for s in slots:
        eng.close_seq(s)
    print(f"{a.dir.rstrip('/').split('/')[-1]} {a.quant}: prompt {n * batch} tokens {n * batch / pp:.1f} tok/s | "
          f"generate {n_gen * batch} tokens {n_gen * batch / tg:.1f} tok/s ({tg * 1e3 / n_gen:.2f} ms/step, batch {batch})")


def cmd_random(a: Args) -> None:
    import wick_b200 as wick
    if not a.config:
        raise UsageError("random needs --config <config.json>")
    cfg = wick.config_from_json(json.load(open(a.config)))
    import torch
    wick.write_random_model(cfg, a.sampler.seed, a.dir,
                            dtype=torch.bfloat16 if a.quant == "bf16" else torch.float32)
    print(f"wick: wrote {a.dir} (seed {a.sampler.seed}, {a.quant})", file=sys.stderr)


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        a = parse_args(argv)
    except UsageError as e:
        print(e, file=sys.stderr)
        return 2
    cmds = {"run": cmd_run, "bench": cmd_bench, "random": cmd_random}
    try:
        if a.cmd not in cmds:
            raise UsageError(f"unknown command {a.cmd}\n\n{USAGE}")
        cmds[a.cmd](a)
        return 0
    except UsageError as e:
        print(e, file=sys.stderr)
        return 2
    except Exception as e:  # errors become one line and exit code 1, as in main.rs:336-342
        print(f"wick: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
