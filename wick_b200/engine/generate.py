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

import dataclasses
import time
from typing import Callable, List, Optional, Sequence

from ..sampling.sampler import Sampler, SamplerConfig

PAGE = 64


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
    __slots__ = ("req", "slot", "prompt", "out", "limit", "next_token", "t_start", "t_prompt")

    def __init__(self, req, slot, prompt, limit):
        self.req, self.slot, self.prompt, self.limit = req, slot, prompt, limit
        self.out: List[int] = []
        self.next_token = -1


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


def generate(engine, prompts: Sequence[Sequence[int]], opts: Optional[GenOptions] = None,
             sampler_factory: Optional[Callable[[SamplerConfig, int], object]] = None,
             on_step: Optional[Callable[[int, List[int]], None]] = None) -> List[GenResult]:
    """Generate a continuation for every prompt; results in the prompts' order.

    engine: anything with ``open_seq()``, ``close_seq(slot)``, ``step(slots,
    tokens, want) -> logits`` and a ``cache`` that tells free pages and slots."""
    opts = opts or GenOptions()
    stops = set(int(t) for t in opts.stop_token_ids)
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
    make_sampler = sampler_factory or (lambda cfg, k: Sampler(cfg, k))
    needs_history = opts.sampler.repetition_penalty != 1.0

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
            slot = engine.open_seq()
            cache.reserve(slot, len(prompts[r]) + limits[r])
            live.append(_Live(r, slot, list(prompts[r]), limits[r]))
        sampler = make_sampler(opts.sampler, len(live))
        index = {id(s): i for i, s in enumerate(live)}

        t0 = time.perf_counter()
        feed = [s.prompt for s in live]
        first = True
        step_no = 0
        while live:
            # Sequences with a zero limit need no logits at all.
            active = [s for s in live if s.limit > 0]
            for s in live:
                if s.limit == 0:
                    results[s.req] = GenResult([], len(s.prompt), "length")
                    engine.close_seq(s.slot)
            if not active:
                break
            if len(active) != len(live):
                feed = [f for f, s in zip(feed, live) if s.limit > 0]
                live = active
            logits = engine.step([s.slot for s in live], feed, [[len(f) - 1] for f in feed])
            hist = [s.prompt + s.out for s in live] if needs_history else None
            toks = sampler.sample(logits, [index[id(s)] for s in live], hist)
            now = time.perf_counter()
            if first:
                for s in live:
                    s.t_prompt = (now - t0) * 1e3
                t1 = now
                first = False
            nxt: List[_Live] = []
            for s, tok in zip(live, toks):
                tok = int(tok)
                done = None
                if tok in stops:
                    done = "stop"
                else:
                    s.out.append(tok)
                    if len(s.out) >= s.limit:
                        done = "length"
                if done:
                    results[s.req] = GenResult(s.out, len(s.prompt), done, s.t_prompt, (now - t1) * 1e3)
                    engine.close_seq(s.slot)
                else:
                    s.next_token = tok
                    nxt.append(s)
            live = nxt
            feed = [[s.next_token] for s in live]
            step_no += 1
            if on_step is not None:
                on_step(step_no, [s.req for s in live])
    return results  # type: ignore[return-value]
