"""Continuous-batching scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees, and decides what happens when pages run out.

Policy (AxiomOperator/rllm, crates/rllm-server/src/engine.rs):
* accept (583-625): an empty prompt or one that does not leave room in the context is refused;
  budget = min(max_tokens, ctx - prompt length); a budget of 0 finishes at once ("length").
* admission (676-698): strictly first-in first-out while fewer than `max_num_seqs` run; a
  request is admitted only if pages for its whole remaining prompt plus one spare page per
  running request are free, else it stays at the head of the queue.
* portions (735-757): every decoding request takes one token; requests still reading their
  prompt share `prefill_chunk` tokens in admission order; a request left with nothing sits the
  step out.  Logits are wanted only for an item that ends at the request's last token.
* pages run out (739-774): the newest-admitted running request is preempted: its pages are
  freed and it goes back to the head of the queue, to recompute its tokens (prompt and what
  it generated) later.  If nothing is left to run, or the head of the queue cannot be
  admitted into an empty engine, the request fails: it needs more cache than the pool has.
* finishing (1223-1241): a stop token ends with "stop", the budget with "length".

The scheduler does host bookkeeping only; it talks to the cache manager through
`pages_needed`, `can_append`, `n_free_pages` and `free`, so its decisions are tested without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Optional, Sequence

from ..sampling.params import SamplingParams


@dataclass
class Request:
    request_id: object
    prompt: Sequence[int]
    max_tokens: int = 256
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: frozenset = frozenset()


@dataclass
class Finished:
    request_id: object
    tokens: list                 # generated token ids
    reason: str                  # "stop" | "length" | "error"
    error: Optional[str] = None


class _Seq:
    def __init__(self, req: Request, budget: int, order: int):
        self.req = req
        self.tokens = list(req.prompt)       # prompt + generated
        self.n_prompt = len(req.prompt)
        self.cached = 0                      # tokens whose keys/values are in the cache
        self.budget = budget
        self.order = order                   # admission order (set when admitted)
        self.counts: dict = {}               # token -> times generated (for the penalties; survives preemption)

    @property
    def rid(self):
        return self.req.request_id

    @property
    def generated(self) -> list:
        return self.tokens[self.n_prompt:]

    def todo(self) -> int:
        return len(self.tokens) - self.cached

    def decoding(self) -> bool:
        return self.todo() == 1 and len(self.tokens) > self.n_prompt


@dataclass
class PlannedItem:
    seq: _Seq
    take: int
    want_last: bool
    ahead: int = 0          # tokens of the request that an uncommitted earlier step holds (plan_ahead)
    sampled: bool = False   # its one token is what that earlier step samples: still on the device

    @property
    def tokens(self) -> list:
        if self.sampled:
            return [0] * self.take       # not known on the host yet: the step takes them from the device
        first = self.seq.cached + self.ahead
        return self.seq.tokens[first:first + self.take]

    @property
    def counter(self) -> int:
        """The request's length when this item's last token is in: the sampler's counter."""
        return self.seq.cached + self.ahead + self.take


def _wants(plan, seq) -> bool:
    """Whether `plan` samples for `seq`."""
    return any(p.seq is seq and p.want_last for p in plan)


class Scheduler:
    def __init__(self, cache, ctx: int = 4096, max_num_seqs: int = 4, prefill_chunk: int = 512, row_quantum: int = 0):
        """row_quantum: the rows of a tile of the many-row kernels (0: none).  A step that holds prompt
        tokens beside decoding requests is then trimmed to a whole number of tiles where that costs
        at most an eighth of its prompt tokens: 512 prompt tokens beside 32 decoding requests are 544
        rows, five tiles of 128 of which the last is a quarter full; 480 beside 32 are four."""
        if max_num_seqs <= 0 or prefill_chunk <= 0 or ctx <= 0 or row_quantum < 0:
            raise ValueError("ctx, max_num_seqs and prefill_chunk must be positive")
        self.cache, self.ctx = cache, ctx
        self.max_num_seqs, self.prefill_chunk = max_num_seqs, prefill_chunk
        self.row_quantum = row_quantum
        self.waiting: deque = deque()
        self.running: list = []
        self._order = 0
        self.done: list = []                 # Finished records not yet collected
        self.stats = {"preemptions": 0, "admitted": 0, "steps": 0, "prompt_tokens": 0,
                      "generated_tokens": 0}

    # ------------------------------------------------------------------ accept
    def add(self, req: Request) -> None:
        n = len(req.prompt)
        if n == 0:
            raise ValueError(f"request {req.request_id!r}: empty prompt")
        if n >= self.ctx:
            raise ValueError(f"request {req.request_id!r}: prompt of {n} tokens does not fit the "
                             f"context of {self.ctx}")
        budget = min(req.max_tokens, self.ctx - n)
        if budget <= 0:
            self.done.append(Finished(req.request_id, [], "length"))
            return
        self.waiting.append(_Seq(req, budget, -1))

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def collect(self) -> list:
        out, self.done = self.done, []
        return out

    # ------------------------------------------------------------------ admission
    def _fits_admission(self, seq: _Seq) -> bool:
        need = self.cache.pages_needed(seq.rid, seq.todo())
        spare = len(self.running)
        return all(n + spare <= self.cache.n_free_pages(g) for g, n in enumerate(need)) \
            and self.cache.slots.n_free >= 1

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            if not self._fits_admission(seq):
                if not self.running:
                    # an empty engine cannot hold it: it never will
                    self.waiting.popleft()
                    self.done.append(Finished(seq.rid, seq.generated, "error",
                                              "request needs more KV cache than the pool has"))
                    continue
                break
            self.waiting.popleft()
            seq.order = self._order
            self._order += 1
            self.running.append(seq)
            self.stats["admitted"] += 1

    # ------------------------------------------------------------------ planning
    def _takes(self) -> list:
        decoders = [s for s in self.running if s.decoding()]
        prefilling = sorted((s for s in self.running if not s.decoding()), key=lambda s: s.order)
        plan = [PlannedItem(s, 1, True) for s in decoders]
        left = self.prefill_chunk
        for s in prefilling:
            take = min(s.todo(), left)
            if take <= 0:
                continue
            left -= take
            plan.append(PlannedItem(s, take, s.cached + take == len(s.tokens)))
        return self._trim(plan, len(decoders))

    def _trim(self, plan: list, n_decoders: int) -> list:
        """A step with prompt tokens, cut to a whole number of tiles (row_quantum) where that is cheap."""
        q = self.row_quantum
        if q and len(plan) > n_decoders:
            rows = sum(p.take for p in plan)
            prompt_rows = rows - n_decoders
            over = rows % q
            last = plan[-1]
            if rows > q and 0 < over <= prompt_rows // 8 and over < last.take:
                plan[-1] = PlannedItem(last.seq, last.take - over, False, ahead=last.ahead)
        return plan

    def _preempt_newest(self) -> Optional[_Seq]:
        if not self.running:
            return None
        victim = max(self.running, key=lambda s: s.order)
        self.running.remove(victim)
        if self.cache.has(victim.rid):
            self.cache.free(victim.rid)
        victim.cached = 0
        self.waiting.appendleft(victim)
        self.stats["preemptions"] += 1
        return victim

    def plan(self) -> list:
        """Returns the items of the next step (possibly empty when nothing can run)."""
        self._admit()
        while True:
            plan = self._takes()
            if not plan:
                return []
            if self.cache.can_append([(p.seq.rid, p.take) for p in plan]):
                self.stats["steps"] += 1
                return plan
            if len(self.running) == 1:
                # alone and still out of pages: it can never finish
                seq = self.running.pop()
                if self.cache.has(seq.rid):
                    self.cache.free(seq.rid)
                self.done.append(Finished(seq.rid, seq.generated, "error",
                                          "request needs more KV cache than the pool has"))
                self._admit()
                continue
            self._preempt_newest()

    def plan_ahead(self, plan: Sequence[PlannedItem]) -> Optional[list]:
        """The step after `plan`, planned before `plan`'s sampled tokens are known on the host, so
        that it can be launched while they are still on their way: every request for which `plan`
        samples decodes that token (it is taken from the device), every request that `plan` leaves in
        the middle of its prompt goes on with it, and waiting requests are admitted as in `plan()`.
        A request that reaches its budget with the token under way is left out (it ends when `plan`
        is committed; the place it leaves is filled one step later).  None when the step cannot be
        known yet: a decoding request is not in `plan`, one of them needs the host for its next token
        (penalties, bias), or the pages are short (the caller then commits `plan` first and plans as
        usual, which may preempt).  The decoding requests come first, in the order in which `plan`
        samples for them.  A request that `plan`'s token ends by a stop id has then run one token
        too far; its pages go back when `plan` is committed, and its row of the step planned here is
        dropped."""
        live = [p for p in plan if p.seq in self.running]       # the others ended with the step before `plan`
        in_plan = {id(p.seq) for p in live}
        # a running request that `plan` left out waits for its share of the prompt budget: it is as the
        # host knows it; one that decodes would have to be in `plan`
        if not live or any(id(s) not in in_plan and s.decoding() for s in self.running):
            return None
        nxt = []
        for p in live:
            s = p.seq
            if not p.want_last:
                continue
            if s.req.params.adjusts:
                return None
            if len(s.tokens) - s.n_prompt + 1 < s.budget:
                nxt.append(PlannedItem(s, 1, True, ahead=p.take, sampled=True))
        n_decoders = len(nxt)
        self._admit()
        held = {id(p.seq): p.take for p in live}                # tokens that `plan` holds, not yet committed
        left = self.prefill_chunk
        for s in sorted((s for s in self.running if id(s) not in held or not _wants(live, s)), key=lambda s: s.order):
            ahead = held.get(id(s), 0)
            take = min(s.todo() - ahead, left)                   # what is left of the prompt behind plan's portion
            if take <= 0:
                continue
            left -= take
            nxt.append(PlannedItem(s, take, s.cached + ahead + take == len(s.tokens), ahead=ahead))
        if not nxt:
            return None
        nxt = self._trim(nxt, n_decoders)
        if not self.cache.can_append([(p.seq.rid, p.take) for p in nxt]):
            return None
        self.stats["steps"] += 1
        return nxt

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: Sequence[PlannedItem], sampled: Sequence[int]) -> list:
        """`sampled`: one token id per planned item with want_last, in plan order.  Returns the
        requests that finished with this step (also kept for `collect`)."""
        it = iter(sampled)
        finished = []
        for p in plan:
            s = p.seq
            if p.ahead and s not in self.running:
                if p.want_last:
                    next(it)             # the request ended with the step before: this token was one too far
                continue
            if s.cached < s.n_prompt:
                self.stats["prompt_tokens"] += min(p.take, s.n_prompt - s.cached)
            s.cached += p.take
            if not p.want_last:
                continue
            tok = int(next(it))
            s.tokens.append(tok)
            if s.req.params.adjusts:
                s.counts[tok] = s.counts.get(tok, 0) + 1
            self.stats["generated_tokens"] += 1
            reason = None
            if tok in s.req.stop_ids:
                reason = "stop"
            elif len(s.tokens) - s.n_prompt >= s.budget:
                reason = "length"
            if reason:
                self.running.remove(s)
                if self.cache.has(s.rid):
                    self.cache.free(s.rid)
                finished.append(Finished(s.rid, s.generated, reason))
        self.done.extend(finished)
        return finished

    def fail_running(self, message: str) -> list:
        """A failed step fails every running request and frees what they hold; the queue goes on
        (crates/rllm-server/src/engine.rs:569-578)."""
        out = []
        for s in self.running:
            if self.cache.has(s.rid):
                self.cache.free(s.rid)
            out.append(Finished(s.rid, s.generated, "error", message))
        self.running = []
        self.done.extend(out)
        return out

    def release_all(self) -> None:
        """Frees what any request this scheduler knows still holds in the cache and forgets them
        all (the end of a generate call, however it ended)."""
        for s in list(self.running) + list(self.waiting):
            if self.cache.has(s.rid):
                self.cache.free(s.rid)
        self.running = []
        self.waiting.clear()
