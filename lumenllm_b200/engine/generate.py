"""The generation loop above the step function.

Per request the loop is the reference's (crates/aegisllm-base/src/executor/
generation.rs:16-94): prompt in, first token sampled from the prompt's last
position; then for each produced token, in this order: an EOS token ends the
request and is NOT kept (reason "eos_token"); a stop token is kept and ends it
("stop"); otherwise the token is kept and, unless it was the last allowed one,
one more step runs ("length" when the allowance is used up). No forward pass
runs after the last allowed token.

The reference serves one request at a time. Here requests run in batches: the
prompts of a batch, of unequal lengths, go through one step together; then
every live request adds one token per step; a request that ends leaves the
batch at once and its slot is given back; when the batch is empty the next one
starts, on the same slots.

The loop only decides; it needs a backend with
  alloc_slot() / free_slot(slot),
  run(entries: [(slot, tokens)], configs, uniforms) -> one token per entry
so that its decisions can be tested without a GPU.

A backend may also offer
  launch(entries, configs, uniforms, after=None, rows=None) -> handle
  collect(handle) -> one token per entry
Then the loop keeps one step in flight: while the host waits for the tokens of step n, the
device already runs step n + 1, fed on the device with step n's tokens (`after` is step n's
handle, `rows[k]` the place of entry k's sequence in it; such an entry brings no host token).
Step n + 1 is launched before step n's tokens are known, so it holds every sequence that
step n cannot end by length; for a sequence that step n then ends by EOS or a stop token,
the token of step n + 1 is dropped, and its slot is given back when the step that held it
has been collected. A sequence's tokens, its uniforms (numbered by its own steps) and
its finish reason are the same as without the run-ahead.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..cache.kv import PAGE
from ..sampling import SamplingConfig, fresh_seed, uniform


@dataclass
class GenerateRequest:
    """Fields as crates/aegisllm-base/src/generation.rs:3-20, with token ids in
    place of text (no tokenizer is part of this library)."""
    prompt_tokens: Sequence[int]
    max_tokens: int = 32
    sampling: SamplingConfig = field(default_factory=SamplingConfig)
    stop_token_ids: Sequence[int] = ()


@dataclass
class GenerateOutput:
    tokens: List[int]
    prompt_tokens: int
    completion_tokens: int
    finish_reason: str
    prefill_s: float = 0.0
    decode_s: float = 0.0


class GenerationError(ValueError):
    pass


def tokens_held(req: GenerateRequest, page: int = PAGE) -> int:
    """Most cache a request can come to hold: the last allowed token is never fed back."""
    n = len(req.prompt_tokens) + max(0, req.max_tokens - 1)
    return (n + page - 1) // page * page


def plan_batches(requests: Sequence[GenerateRequest], max_batch: int, token_budget: int,
                 page: int = PAGE) -> List[List[int]]:
    """Cuts the requests, in their order, into batches that fit the slots and the cache."""
    if max_batch <= 0:
        raise GenerationError("max_batch must be positive")
    batches, cur, used = [], [], 0
    for i, r in enumerate(requests):
        need = tokens_held(r, page)
        if need > token_budget:
            raise GenerationError(f"request {i} may hold {need} tokens; the cache holds {token_budget}")
        if cur and (len(cur) >= max_batch or used + need > token_budget):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def generate(backend, requests: Sequence[GenerateRequest], eos_token_ids: Sequence[int] = (),
             max_batch: int = 64, token_budget: int = 1 << 62,
             on_token: Optional[Callable[[int, int], None]] = None,
             clock: Callable[[], float] = time.perf_counter) -> List[GenerateOutput]:
    requests = list(requests)
    eos = set(int(t) for t in eos_token_ids)
    for i, r in enumerate(requests):
        if len(r.prompt_tokens) == 0:
            raise GenerationError(f"request {i}: prompt produced no tokens")
        if r.max_tokens < 0:
            raise GenerationError(f"request {i}: max_tokens must not be negative")
        r.sampling.validate()
    seeds = [r.sampling.seed if r.sampling.seed is not None else fresh_seed() for r in requests]
    outputs: List[Optional[GenerateOutput]] = [None] * len(requests)

    pipelined = hasattr(backend, "launch") and hasattr(backend, "collect")

    for batch in plan_batches(requests, max_batch, token_budget):
        live = []            # request indices still generating
        slot_of, produced, nsteps = {}, {}, {}
        t0 = clock()
        for i in batch:
            if requests[i].max_tokens == 0:
                outputs[i] = GenerateOutput([], len(requests[i].prompt_tokens), 0, "length")
                continue
            slot_of[i] = backend.alloc_slot()
            produced[i], nsteps[i] = [], 0
            live.append(i)
        if not live:
            continue
        try:
            t_prefill = [0.0]

            def decide(i, tok):
                """Books request i's next token; returns its finish reason or None."""
                tok = int(tok)
                r = requests[i]
                reason = None
                if tok in eos:
                    reason = "eos_token"
                elif tok in set(r.stop_token_ids):
                    produced[i].append(tok)
                    reason = "stop"
                else:
                    produced[i].append(tok)
                    if len(produced[i]) >= r.max_tokens:
                        reason = "length"
                if on_token is not None and reason != "eos_token":
                    on_token(i, tok)
                if reason is not None:
                    outputs[i] = GenerateOutput(produced[i], len(r.prompt_tokens), len(produced[i]),
                                                reason, t_prefill[0], clock() - t0 - t_prefill[0])
                return reason

            def step_inputs(members):
                cfgs = [requests[i].sampling for i in members]
                us = [uniform(seeds[i], 0, nsteps[i]) for i in members]
                for i in members:
                    nsteps[i] += 1
                return cfgs, us

            if not pipelined:
                feed = {i: list(requests[i].prompt_tokens) for i in live}
                first = True
                while live:
                    entries = [(slot_of[i], feed[i]) for i in live]
                    cfgs, us = step_inputs(live)
                    nxt = backend.run(entries, cfgs, us)
                    if first:
                        t_prefill[0] = clock() - t0
                        first = False
                    still = []
                    for i, tok in zip(live, nxt):
                        if decide(i, tok) is None:
                            feed[i] = [int(tok)]
                            still.append(i)
                        else:
                            backend.free_slot(slot_of.pop(i))
                    live = still
                continue

            # One step in flight ahead of the host.
            cfgs, us = step_inputs(live)
            handle = backend.launch([(slot_of[i], list(requests[i].prompt_tokens)) for i in live], cfgs, us)
            members = list(live)
            done = set()             # ended, slot still held by a step in flight
            first = True
            while members:
                # who goes on after this step whatever it samples, unless it is EOS or a stop token
                ahead = [i for i in members
                         if i not in done and len(produced[i]) + 1 < requests[i].max_tokens]
                nxt_handle = None
                if ahead:
                    cfgs, us = step_inputs(ahead)
                    rows = [members.index(i) for i in ahead]
                    nxt_handle = backend.launch([(slot_of[i], None) for i in ahead], cfgs, us,
                                                after=handle, rows=rows)
                toks = backend.collect(handle)
                if first:
                    t_prefill[0] = clock() - t0
                    first = False
                for i, tok in zip(members, toks):
                    if i in done:                    # ended a step ago; this token was run ahead
                        done.discard(i)
                        backend.free_slot(slot_of.pop(i))
                        continue
                    if decide(i, tok) is not None:
                        if i in ahead:
                            done.add(i)              # the step in flight still writes to its slot
                        else:
                            backend.free_slot(slot_of.pop(i))
                handle, members = nxt_handle, ahead
        except BaseException:
            # a step was refused (cache full, bad token) or the caller's callback raised: the
            # batch's slots go back before the error goes on, so the backend stays usable
            for i in list(slot_of):
                backend.free_slot(slot_of.pop(i))
            raise
    return outputs  # type: ignore[return-value]
