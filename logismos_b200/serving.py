"""Host-side continuous-batching scheduler for the decoder executors, and the synthetic serving load
of the hybrid-decoder sweep (lognormal prompt lengths, uniform output lengths, Poisson arrivals).

The reference has no scheduler (crates/sched/src/lib.rs:1-30 is an empty scaffold); the contract the
executors give it is "a packed step equals running every sequence alone", so scheduling decisions
change throughput only, never results. Policy: first come first served; every running sequence
decodes one token per step; waiting requests that have arrived are admitted while a state slot, the
KV blocks of their whole lifetime (prompt + max_new tokens, so nothing is ever preempted), a row of
the step and room in the step's token budget are available. With ``chunked_prefill`` a prompt is fed
in chunks: each step gives the prompts in flight (oldest first) what is left of its prefill budget,
a sequence starts decoding after the step that took the last token of its prompt, and no step has to
hold a whole prompt; without it a prompt is prefilled whole in one step.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

import numpy as np

BLOCK = 16


@dataclass
class Request:
    rid: int
    prompt: np.ndarray          # uint32 token ids
    max_new: int                # tokens to generate (>= 1)
    arrival: float = 0.0        # seconds since the start of the run
    output: List[int] = field(default_factory=list)
    first_token_at: Optional[float] = None
    finished_at: Optional[float] = None


@dataclass
class StepPlan:
    ids: np.ndarray             # uint32, packed in entry order
    cached: np.ndarray          # int32 [n]
    new: np.ndarray             # int32 [n]
    tables: np.ndarray          # int32 [n, max_blocks_per_seq]
    slots: np.ndarray           # int32 [n]
    rids: List[int]
    n_decode: int
    n_prefill_tokens: int
    emits: Optional[np.ndarray] = None   # bool [n]: the entry's next token is a generated token (None: all)


def synthetic_load(n_requests: int, seed: int, vocab: int, prompt_median: int = 1024, prompt_sigma: float = 1.0,
                   prompt_cap: int = 16384, out_lo: int = 64, out_hi: int = 1024, rate_per_s: float = 0.0) -> List[Request]:
    """Seeded requests with prompt lengths lognormal(median, sigma) clipped to [1, cap], output lengths
    uniform in [out_lo, out_hi], uniform token ids and exponential inter-arrival times of mean
    1 / rate_per_s (rate 0: everything has arrived at time 0)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    plen = np.clip(np.rint(np.exp(rng.normal(np.log(prompt_median), prompt_sigma, n_requests))), 1, prompt_cap).astype(np.int64)
    olen = rng.integers(out_lo, out_hi + 1, n_requests)
    t = np.cumsum(rng.exponential(1.0 / rate_per_s, n_requests)) if rate_per_s > 0 else np.zeros(n_requests)
    return [Request(i, rng.integers(0, vocab, int(plen[i]), dtype=np.uint32), int(olen[i]), float(t[i])) for i in range(n_requests)]


def shard_requests(requests: List[Request], world: int, rank: int) -> List[Request]:
    """Round-robin by arrival order: rank r serves requests r, r + world, ... (no data-path exchange)."""
    return [r for i, r in enumerate(requests) if i % world == rank]


class Scheduler:
    def __init__(self, n_pool_blocks: int, max_blocks_per_seq: int, n_state_slots: int, max_step_tokens: int, max_step_seqs: int,
                 prefill_token_budget: int = 0, chunked_prefill: bool = False):
        self.max_blocks, self.max_step_tokens, self.max_step_seqs = max_blocks_per_seq, max_step_tokens, max_step_seqs
        self.prefill_budget = prefill_token_budget or max_step_tokens
        self.chunked = chunked_prefill
        self.prefilling: Dict[int, Request] = {}   # admitted, prompt not yet fully fed (insertion order = age)
        self.free_blocks: List[int] = list(range(n_pool_blocks - 1, -1, -1))
        self.free_slots: List[int] = list(range(n_state_slots - 1, -1, -1))
        self.waiting: Deque[Request] = deque()
        self.running: Dict[int, Request] = {}
        self.tables: Dict[int, np.ndarray] = {}
        self.slot_of: Dict[int, int] = {}
        self.cached: Dict[int, int] = {}
        self.done: List[Request] = []
        self.generated = 0
        self.prefilled = 0

    def add(self, req: Request):
        need = -(-(len(req.prompt) + req.max_new) // BLOCK)
        if need > self.max_blocks or len(req.prompt) < 1 or req.max_new < 1 or (not self.chunked and len(req.prompt) > self.max_step_tokens):
            raise ValueError(f"request {req.rid} cannot be served: {len(req.prompt)} + {req.max_new} tokens")
        self.waiting.append(req)

    def idle(self) -> bool:
        return not self.waiting and not self.running

    def next_arrival(self) -> Optional[float]:
        return self.waiting[0].arrival if self.waiting else None

    def plan(self, now: float) -> Optional[StepPlan]:
        """The next step: one decode token for every running sequence whose prompt is in the cache (oldest
        first, up to the step's rows), then prefill: chunks of the prompts in flight, then admitted
        prompts (whole, or as much as the step's budget leaves when chunking). None when nothing can run
        at `now`."""
        rids, ids, cached, new, emits = [], [], [], [], []
        for rid, req in self.running.items():
            if len(rids) >= self.max_step_seqs or len(rids) >= self.max_step_tokens:
                break
            if rid in self.prefilling:
                continue
            rids.append(rid); ids.append(np.asarray([req.output[-1]], np.uint32)); cached.append(self.cached[rid]); new.append(1); emits.append(True)
        n_decode, tokens, pre_tokens = len(rids), len(rids), 0

        def room():
            return min(self.max_step_tokens - tokens, self.prefill_budget - pre_tokens)

        for rid, req in self.prefilling.items():  # chunked mode only: continue the prompts in flight
            if len(rids) >= self.max_step_seqs or room() <= 0:
                break
            done = self.cached[rid]
            n = min(len(req.prompt) - done, room())
            rids.append(rid); ids.append(req.prompt[done:done + n]); cached.append(done); new.append(n)
            emits.append(done + n == len(req.prompt))
            tokens += n; pre_tokens += n
        while self.waiting and self.waiting[0].arrival <= now and len(rids) < self.max_step_seqs:
            req = self.waiting[0]
            p = len(req.prompt)
            need = -(-(p + req.max_new) // BLOCK)
            if not self.free_slots or need > len(self.free_blocks):
                break
            if self.chunked:
                n = min(p, room())
                if n <= 0:
                    break
            else:
                n = p
                if tokens + p > self.max_step_tokens or (pre_tokens > 0 and pre_tokens + p > self.prefill_budget):
                    break
            self.waiting.popleft()
            row = np.full(self.max_blocks, -1, np.int32)
            row[:need] = [self.free_blocks.pop() for _ in range(need)]
            self.tables[req.rid], self.slot_of[req.rid], self.cached[req.rid] = row, self.free_slots.pop(), 0
            self.running[req.rid] = req
            if n < p:
                self.prefilling[req.rid] = req
            rids.append(req.rid); ids.append(req.prompt[:n]); cached.append(0); new.append(n); emits.append(n == p)
            tokens += n; pre_tokens += n
        if not rids:
            return None
        return StepPlan(np.concatenate(ids).astype(np.uint32), np.asarray(cached, np.int32), np.asarray(new, np.int32),
                        np.stack([self.tables[r] for r in rids]), np.asarray([self.slot_of[r] for r in rids], np.int32), rids,
                        n_decode, pre_tokens, np.asarray(emits, bool))

    def commit(self, plan: StepPlan, next_tokens, now: float):
        """Records the step's results: appends each sequence's new token (a chunk that does not end its
        prompt produces none), retires finished sequences and returns their blocks and slots."""
        for i, rid in enumerate(plan.rids):
            req = self.running[rid]
            self.cached[rid] += int(plan.new[i])
            if plan.emits is not None and not plan.emits[i]:
                continue
            self.prefilling.pop(rid, None)
            req.output.append(int(next_tokens[i]))
            self.generated += 1
            if req.first_token_at is None:
                req.first_token_at = now
            if len(req.output) >= req.max_new:
                req.finished_at = now
                row = self.tables.pop(rid)
                self.free_blocks.extend(int(b) for b in row[row >= 0][::-1])
                self.free_slots.append(self.slot_of.pop(rid))
                del self.cached[rid], self.running[rid]
                self.done.append(req)
        self.prefilled += plan.n_prefill_tokens


def serve(model_step, sched: Scheduler, requests: List[Request], clock, max_steps: int = 0, on_step=None) -> int:
    """Drives `sched` until every request is done (or max_steps steps ran). ``model_step(plan)`` returns
    the next token of every entry; ``clock()`` returns seconds since the start. Returns the step count."""
    for r in requests:
        sched.add(r)
    steps = 0
    while not sched.idle() and (max_steps <= 0 or steps < max_steps):
        now = clock()
        plan = sched.plan(now)
        if plan is None:
            nxt = sched.next_arrival()
            if nxt is None or nxt <= now:
                raise RuntimeError("scheduler stalled: a waiting request fits neither the pool nor the step")
            continue
        toks = model_step(plan)
        sched.commit(plan, toks, clock())
        steps += 1
        if on_step:
            on_step(plan)
    return steps
