"""Continuous batching over one attention handle: which request runs in which sequence slot, and when.

The reference serves one session at a time behind a mutex (server/src/main.rs:84); the batched and ragged workloads
need the opposite: requests join a running decode batch as soon as a sequence slot and enough KV pages are free, and
leave it when they are done, their pages going back to the pool (flint_attn_seq_release).  This class only keeps
the books -- slots, page reservations, the queue -- and tells the caller what to run each step; the caller owns the
model around attention and makes the prefill / decode calls.  `Router` spreads requests over the ranks of a
multi-GPU job by outstanding KV bytes (no data-path collective: a request lives on one rank).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

from .shard import kv_bytes_per_token_step

PAGE_KEYS = 64


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE_KEYS - 1) // PAGE_KEYS


@dataclass
class Running:
    req_id: int
    slot: int
    prompt_len: int
    max_new: int
    generated: int = 0
    pages_reserved: int = 0


@dataclass
class StepPlan:
    admit: List[Running] = field(default_factory=list)    # prefill these (their prompt), then they decode from the next step
    decode: List[Running] = field(default_factory=list)   # one new token for each of these, as one batch


class ContinuousBatcher:
    """FCFS admission with full reservation: a request is admitted only when a slot is free and the pool can hold
    its prompt plus everything it may generate, so a running request never hits an exhausted pool."""

    def __init__(self, max_seqs: int, kv_pages: int, n_ctx: int, max_batch: Optional[int] = None):
        self.free_slots: List[int] = list(range(max_seqs - 1, -1, -1))
        self.pages_total, self.pages_reserved = kv_pages, 0
        self.n_ctx = n_ctx
        self.max_batch = max_batch or max_seqs
        self.queue: Deque[tuple] = deque()
        self.running: Dict[int, Running] = {}
        self.finished: List[int] = []

    def submit(self, req_id: int, prompt_len: int, max_new: int) -> None:
        if prompt_len < 1 or max_new < 0 or prompt_len + max_new > self.n_ctx:
            raise ValueError("request does not fit the context")
        if pages_for(prompt_len + max_new) > self.pages_total:
            raise ValueError("request does not fit the page pool")
        self.queue.append((req_id, prompt_len, max_new))

    def next_step(self) -> StepPlan:
        """What to run now.  Requests admitted in this step are prefilled by the caller and decode from the next one."""
        plan = StepPlan(decode=[r for r in self.running.values() if r.generated < r.max_new])
        while self.queue and self.free_slots and len(self.running) < self.max_batch:
            req_id, prompt_len, max_new = self.queue[0]
            need = pages_for(prompt_len + max_new)
            if self.pages_reserved + need > self.pages_total:
                break  # FCFS: the head of the queue waits for pages; nothing overtakes it
            self.queue.popleft()
            r = Running(req_id, self.free_slots.pop(), prompt_len, max_new, pages_reserved=need)
            self.pages_reserved += need
            self.running[req_id] = r
            plan.admit.append(r)
        return plan

    def complete(self, plan: StepPlan) -> List[Running]:
        """Book one finished step; returns the requests to retire (the caller releases their slots' pages)."""
        for r in plan.decode:
            r.generated += 1
        done = [r for r in self.running.values() if r.generated >= r.max_new and r not in plan.admit] + \
               [r for r in plan.admit if r.max_new == 0]
        for r in done:
            del self.running[r.req_id]
            self.free_slots.append(r.slot)
            self.pages_reserved -= r.pages_reserved
            self.finished.append(r.req_id)
        return done

    @property
    def idle(self) -> bool:
        return not self.queue and not self.running


class Router:
    """Least-outstanding-KV-bytes placement of incoming requests on ranks (greedy, the online form of
    shard.balance_by_kv_bytes)."""

    def __init__(self, n_ranks: int, n_full_layers: int = 1, n_swa_layers: int = 0):
        self.load = [0] * n_ranks
        self.where: Dict[int, tuple] = {}
        self.n_full, self.n_swa = n_full_layers, n_swa_layers

    def place(self, req_id: int, prompt_len: int, max_new: int) -> int:
        cost = kv_bytes_per_token_step(prompt_len + max_new, self.n_full, self.n_swa)
        rank = min(range(len(self.load)), key=lambda k: (self.load[k], k))
        self.load[rank] += cost
        self.where[req_id] = (rank, cost)
        return rank

    def retire(self, req_id: int) -> None:
        rank, cost = self.where.pop(req_id)
        self.load[rank] -= cost
