"""Continuous batching with chunked prefill over a model that runs ragged-batch steps (`Engine.step_batch`).

What crane-serve's engine thread does for its sequences (crane-serve/src/engine/mod.rs:169-271 loop, :822-1062 batch decode,
scheduler.rs admission): requests wait in a queue, are admitted while a sequence slot and KV pages are free, have their prompts
fed in portions of at most `chunk` tokens beside the single decoded tokens of the requests that are already generating, and give
their slot and pages back when they finish.  One `step()` = one engine iteration = one batch over the weights.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field


@dataclass
class Request:
    rid: int
    prompt: list
    max_new_tokens: int
    sampling: dict = field(default_factory=dict)      # make_sampling keywords; empty = greedy
    eos: tuple = ()
    seq: int = -1
    fed: int = 0                                      # prompt tokens already in the cache
    output: list = field(default_factory=list)
    done: bool = False


class BatchScheduler:
    def __init__(self, model, chunk: int = 256, max_live: int = 4, token_budget: int = 1024, page: int = 64):
        self.m, self.chunk, self.max_live, self.budget, self.page = model, chunk, max_live, token_budget, page
        self.waiting, self.live, self.finished = deque(), [], {}
        self._next = 0
        self._slot0_free = True
        self.pool_tokens = int(model.config.get("engine", {}).get("max_tokens", 4096))

    def add(self, prompt, max_new_tokens: int, eos=(), **sampling) -> int:
        r = Request(self._next, [int(t) for t in prompt], int(max_new_tokens), dict(sampling), tuple(eos))
        if not r.prompt or r.max_new_tokens < 1:
            raise ValueError("a request needs a prompt and at least one new token")
        self._next += 1
        self.waiting.append(r)
        return r.rid

    def _pages(self, n_tokens: int) -> int:
        return (n_tokens + self.page - 1) // self.page

    def _reserved(self) -> int:
        return sum(self._pages(len(r.prompt) + r.max_new_tokens) for r in self.live)

    def _admit(self):
        while self.waiting and len(self.live) < self.max_live:
            r = self.waiting[0]
            need = self._pages(len(r.prompt) + r.max_new_tokens)
            if need > self._pages(self.pool_tokens):
                raise ValueError(f"request {r.rid} needs {need} pages, the pool has {self._pages(self.pool_tokens)}")
            if self._reserved() + need > self._pages(self.pool_tokens):
                break                                   # wait until a running request gives pages back
            self.waiting.popleft()
            if self._slot0_free:
                r.seq, self._slot0_free = 0, False
            else:
                r.seq = self.m.seq_create()
            self.live.append(r)

    def _retire(self, r: Request):
        r.done = True
        self.finished[r.rid] = r.output
        if r.seq == 0:
            self.m.seq_select(0)
            self.m.clear_kv_cache()
            self._slot0_free = True
        else:
            self.m.seq_free(r.seq)
        self.live.remove(r)

    def step(self) -> bool:
        """One engine iteration; False when nothing is left to do."""
        self._admit()
        if not self.live:
            return False
        entries, owners, budget = [], [], self.budget
        for r in self.live:                             # decoding requests first: one token each
            if r.fed == len(r.prompt):
                entries.append((r.seq, [r.output[-1]], [0])); owners.append(r); budget -= 1
        for r in self.live:                             # then prompt portions within the budget
            if r.fed < len(r.prompt) and budget > 0:
                n = min(self.chunk, len(r.prompt) - r.fed, budget)
                last = r.fed + n == len(r.prompt)
                entries.append((r.seq, r.prompt[r.fed:r.fed + n], [n - 1] if last else []))
                if last:
                    owners.append(r)
                r.fed += n
                budget -= n
        # the wanted rows come back in entry order; decoding entries were listed first, finished prompts after them
        self.m.step_batch(entries, copy=False)
        if owners:
            toks = self.m.sample_rows([o.sampling for o in owners])
            for o, t in zip(owners, toks):
                o.output.append(int(t))
                if len(o.output) >= o.max_new_tokens or int(t) in o.eos:
                    self._retire(o)
        return True

    def run(self) -> dict:
        while self.step():
            pass
        return dict(self.finished)
