"""The generation loop above the step function.

Requests (token-id prompts) are served in batches of sequences that start
together: as many of the waiting requests as the batch limit and the cache's
free pages allow start with one step that runs all their prompts (unequal
lengths), then the batch decodes one token per sequence and step.  A sequence
ends on a stop token or at its length limit, leaves the batch at once and gives
its slot and pages back; when the batch is empty the next one starts, until no
request waits.

Per sequence the loop follows wick ``src/engine.rs:157-223``: the limit is
``min(max_tokens, context - prompt)`` (``:169-170``); a sampled stop token ends
the sequence and is neither returned nor fed (``:181-184``); no step runs after
the last token (``:204-206``); ``finish`` is ``stop`` or ``length`` (``:72-77``).
An empty prompt and a prompt longer than the context are errors (``:121-126``).

The decisions (who starts, who stops, what is fed next) are plain Python over an
object with ``open_seq/close_seq/step`` and a sampler, so that they can be tested
without a GPU.
"""
from __future__ import annotations

import collections
import dataclasses
import time
from typing import Callable, List, Optional, Sequence

from ..sampling.sampler import Sampler, SamplerConfig
from .run import StepRun

from ..layout import PAGE


@dataclasses.dataclass
class GenOptions:
    max_tokens: int = 256
    sampler: SamplerConfig = dataclasses.field(default_factory=SamplerConfig)
    stop_token_ids: Sequence[int] = ()
    context: int = 4096                 # tokens a sequence may hold (prompt + generated)
    max_batch: int = 64                 # sequences that start together


@dataclasses.dataclass
class GenResult:
    tokens: List[int]
    prompt_tokens: int
    finish: str                         # "stop" | "length"
    prompt_ms: float = 0.0
    gen_ms: float = 0.0

    def prompt_tps(self) -> float:
        return self.prompt_tokens / max(self.prompt_ms / 1e3, 1e-9)

    def gen_tps(self) -> float:
        return max(len(self.tokens) - 1, 0) / max(self.gen_ms / 1e3, 1e-9)


class _Live:
    __slots__ = ("req", "slot", "prompt", "out", "limit", "launched", "done", "t_prompt")

    def __init__(self, req, slot, prompt, limit):
        self.req, self.slot, self.prompt, self.limit = req, slot, prompt, limit
        self.out: List[int] = []
        self.launched = 0          # steps launched that sample a token for this sequence
        self.done = False
        self.t_prompt = 0.0


def _pages(n: int) -> int:
    return (n + PAGE - 1) // PAGE


def plan_batch(waiting: Sequence[int], prompt_lens: Sequence[int], limits: Sequence[int], *, free_pages: int,
               free_slots: int, max_batch: int) -> List[int]:
    """Which of the waiting requests (indices, in order) start together now:
    the longest prefix of the queue that fits the batch limit, the free slots
    and the pages each will need at its full length."""
    chosen: List[int] = []
    pages = 0
    for r in waiting:
        need = _pages(prompt_lens[r] + limits[r])
        if len(chosen) >= min(max_batch, free_slots) or pages + need > free_pages:
            break
        chosen.append(r)
        pages += need
    return chosen


def stop_set(engine, opts: GenOptions) -> set:
    """The tokens that end a sequence: the model's own (its configuration's end-of-sequence
    ids, as wick's engine collects them, engine.rs:41-51) and the caller's."""
    own = getattr(getattr(engine, "spec", None), "stop_token_ids", ()) or ()
    return set(int(t) for t in own) | set(int(t) for t in opts.stop_token_ids)


def generate(engine, prompts: Sequence[Sequence[int]], opts: Optional[GenOptions] = None,
             sampler_factory: Optional[Callable[[SamplerConfig, int], object]] = None,
             on_step: Optional[Callable[[int, List[int]], None]] = None,
             run_factory: Optional[Callable[[object, GenOptions, set, int], object]] = None) -> List[GenResult]:
    """Generate a continuation for every prompt; results in the prompts' order.

    engine: anything with ``open_seq()``, ``close_seq(slot)``, a ``cache`` that tells free
    pages and slots, and either ``begin_run(sampler_config, stop_ids)`` (a batch that is
    stepped on the device, see ``engine/run.py``) or ``step(slots, tokens, want) -> logits``
    (then, or when ``sampler_factory`` is given, one step at a time with a sampler on this
    side).  ``run_factory(engine, opts, stops, n)`` overrides the choice.

    A batch that is stepped on the device is one step ahead of what this loop has read: a
    sequence that samples a stop token rides along, frozen, in the step that was launched
    before the loop learned of it; that step changes nothing and its token is dropped."""
    opts = opts or GenOptions()
    stops = stop_set(engine, opts)
    n = len(prompts)
    context = min(opts.context, getattr(engine.cache, "max_position", None) or opts.context)
    limits: List[int] = []
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError("empty prompt")
        if len(p) > context:
            raise ValueError(f"prompt is {len(p)} tokens, context is {context}")
        limits.append(min(opts.max_tokens, context - len(p)))
    results: List[Optional[GenResult]] = [None] * n
    waiting = list(range(n))

    def make_run(k: int):
        if run_factory is not None:
            return run_factory(engine, opts, stops, k)
        if sampler_factory is None and hasattr(engine, "begin_run"):
            return engine.begin_run(opts.sampler, stops)
        make_sampler = sampler_factory or (lambda cfg, m: Sampler(cfg, m))
        return StepRun(engine, make_sampler(opts.sampler, k), opts.sampler.repetition_penalty != 1.0)

    while waiting:
        cache = engine.cache
        chosen = plan_batch(waiting, [len(p) for p in prompts], limits, free_pages=cache.pages.n_free,
                            free_slots=cache.slots.n_free, max_batch=opts.max_batch)
        if not chosen:
            r = waiting[0]
            raise RuntimeError(f"request {r} needs {_pages(len(prompts[r]) + limits[r])} cache pages of {PAGE} "
                               f"tokens; the cache has {cache.pages.capacity}")
        waiting = waiting[len(chosen):]
        live: List[_Live] = []
        for r in chosen:
            if limits[r] == 0:                         # nothing to generate: no slot, no step
                results[r] = GenResult([], len(prompts[r]), "length")
                continue
            slot = engine.open_seq()
            cache.reserve(slot, len(prompts[r]) + limits[r])
            live.append(_Live(r, slot, list(prompts[r]), limits[r]))
        if not live:
            continue
        run = make_run(len(live))
        t0 = time.perf_counter()
        run.start([s.slot for s in live], [s.prompt for s in live], [s.limit for s in live])
        for s in live:
            s.launched = 1
        pending = collections.deque([list(live)])      # the sequences of each step launched and not yet read
        t1 = t0
        step_no = 0
        while True:
            # Launch ahead: a step for every sequence that is not known to be finished and that
            # its limit allows another token.  (None of them: nothing runs after the last token.)
            while len(pending) < run.depth + 1:
                rows = [s for s in live if not s.done and s.launched < s.limit]
                if not rows:
                    break
                run.launch([s.slot for s in rows])
                for s in rows:
                    s.launched += 1
                pending.append(rows)
            if not pending:
                break
            rows = pending.popleft()
            toks = run.collect()
            now = time.perf_counter()
            if step_no == 0:
                for s in rows:
                    s.t_prompt = (now - t0) * 1e3
                t1 = now
            for s, tok in zip(rows, toks):
                if s.done:
                    continue                           # it rode along after its end
                tok = int(tok)
                finish = None
                if tok in stops:
                    finish = "stop"
                else:
                    s.out.append(tok)
                    if len(s.out) >= s.limit:
                        finish = "length"
                if finish:
                    s.done = True
                    results[s.req] = GenResult(s.out, len(s.prompt), finish, s.t_prompt, (now - t1) * 1e3)
                    engine.close_seq(s.slot)
            live = [s for s in live if not s.done]
            step_no += 1
            if on_step is not None:
                on_step(step_no, [s.req for s in live])
        check = getattr(engine, "check_kernels", None)
        if check is not None:
            check()                                    # a kernel that gave up a wait must not go unnoticed
    return results  # type: ignore[return-value]
