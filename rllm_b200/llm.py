"""The Python entry point: ``LLM(...).generate(prompts, ...)`` and the one-call ``generate``.

Token ids in, token ids out (the engine has no tokenizer).  Options carry AxiomOperator/rllm's
names and meanings where it has them (crates/rllm-cli/src/main.rs:39-110, 195-237):
``ctx`` (context per request, default 4096), ``block_size`` (32 tokens per page; the reference defaults to 16, here a page is a TMA box and 32 halves the copies per key tile), ``prefill_chunk`` (512),
``parallel`` (requests running at once, 4), ``kv_tokens`` (tokens the cache holds, default
ctx * parallel), ``max_tokens`` (256), ``temperature`` (0 = greedy), ``top_k`` (0 = off),
``top_p`` (1.0 = off), ``seed`` (0), ``frequency_penalty`` / ``presence_penalty`` / ``logit_bias``
(the request parameters of the reference's server), ``host_sampling`` (sample on the host from copied logits
instead of on the device).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .engine.core import Engine
from .engine.batch import StepItem
from .engine.scheduler import Finished, Request, Scheduler
from .models.model import load_model
from .sampling.device import sample_rows
from .sampling.host import HostSampler
from .sampling.params import SamplingParams


class _SampledIds:
    """The ids a step's sampler left on the device, on their way to the host.  The copy runs on a
    stream of its own, as soon as the sampler is done: on the engine's stream it would queue behind
    the NEXT step, which has been launched by the time the ids are read (Scheduler.plan_ahead), and
    the host would see them a whole step late."""

    def __init__(self, ids: torch.Tensor, copy_stream):
        self.device_ids = ids
        self.host = torch.empty(ids.shape, dtype=ids.dtype, pin_memory=True)
        ready = torch.cuda.Event()
        ready.record()                                   # the sampler, on the engine's stream
        ids.record_stream(copy_stream)
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ready)
            self.host.copy_(ids, non_blocking=True)
            self.done = torch.cuda.Event()
            self.done.record(copy_stream)

    def tolist(self) -> list:
        self.done.synchronize()
        return self.host.tolist()


class LLM:
    def __init__(self, model, dtype="bfloat16", device="cuda:0", ctx: int = 4096, block_size: int = 32,
                 prefill_chunk: int = 512, parallel: int = 4, kv_tokens: Optional[int] = None,
                 host_sampling: bool = False):
        """`model`: a folder with config.json and model.safetensors, or a loaded DecoderModel."""
        if isinstance(model, (str, bytes)) or hasattr(model, "__fspath__"):
            self.config, self.model = load_model(model, dtype, device)
        else:
            self.config, self.model = None, model
        limit = int(getattr(self.model.spec, "max_position", 0) or 0)
        if limit and ctx > limit:
            from .config.base import ConfigError
            raise ConfigError(f"ctx {ctx} exceeds the model's max_position_embeddings ({limit}): positions beyond "
                              f"it are outside what the model was made for")
        kv_tokens = max(kv_tokens or ctx * parallel, ctx)
        self.engine = Engine(self.model, block_size=block_size, max_tokens=kv_tokens,
                             max_requests=max(parallel, 1), max_step_tokens=prefill_chunk)
        self.ctx, self.prefill_chunk, self.parallel = ctx, prefill_chunk, parallel
        # steps with prompt tokens are trimmed to whole 128-row tiles of the many-row kernels (Scheduler)
        self.row_quantum = 128 if self.engine.runtime.dtype == torch.bfloat16 else 0
        self.host_sampling = host_sampling
        self.last_stats = {}
        self.last_errors = {}
        self._copy_stream = None

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens=256, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0, stop_ids: Sequence[int] = (),
                 return_reasons: bool = False, frequency_penalty: float = 0.0, presence_penalty: float = 0.0,
                 logit_bias=()):
        """Generates for every prompt (continuous batching); returns the generated ids per prompt,
        in order.  A step that fails (an exception from the engine or the sampler, or a kernel that
        gave up a bounded wait) fails the requests running in it and frees their pages; the waiting
        ones still run.  Failed requests raise GenerationError at the end (its `results` hold
        what the others generated), or, with return_reasons, come back with the reason "error" and
        their message in `last_errors`.  max_tokens: one number, or one per prompt.  Request i samples with seed
        `seed + i`.  logit_bias: (token, delta) pairs or a
        {token: delta} mapping, added to the logits with the frequency and presence penalties over
        the tokens generated so far before the token is chosen."""
        if isinstance(logit_bias, dict):
            logit_bias = tuple(logit_bias.items())
        limits = [max_tokens] * len(prompts) if isinstance(max_tokens, int) else list(max_tokens)
        if len(limits) != len(prompts):
            raise ValueError(f"max_tokens: {len(limits)} numbers for {len(prompts)} prompts")
        sched = Scheduler(self.engine.cache, ctx=self.ctx, max_num_seqs=self.parallel,
                          prefill_chunk=self.prefill_chunk, row_quantum=getattr(self, "row_quantum", 0))
        for i, p in enumerate(prompts):
            sched.add(Request(i, list(p), int(limits[i]),
                              SamplingParams(temperature, top_k, top_p, seed + i, frequency_penalty,
                                             presence_penalty, tuple(logit_bias)), frozenset(stop_ids)))
        results = {}
        host_samplers = {}
        steps = 0
        # A step whose sampled ids are still on the device: (plan, ids).  While they travel to the host
        # the next step is planned and launched already where that is possible (Scheduler.plan_ahead),
        # taking its tokens from the device; the host's work for a step then hides behind the GPU's.
        pending = also = None
        try:
            while sched.has_work() or pending is not None:
                try:
                    if pending is None:
                        plan = sched.plan()
                        for f in sched.collect():
                            results[f.request_id] = f
                        if not plan:
                            continue
                        ids = self._run_step(plan, host_samplers)
                        if isinstance(ids, _SampledIds):
                            pending = (plan, ids)
                            continue
                    else:
                        plan, sampled = pending
                        ahead = sched.plan_ahead(plan)
                        ahead_ids = (self._run_step(ahead, host_samplers, device_tokens=self._ids_for(plan, ahead, sampled))
                                     if ahead else None)
                        ids = sampled.tolist()
                        pending = (ahead, ahead_ids) if isinstance(ahead_ids, _SampledIds) else None
                        if ahead and pending is None:
                            also = (ahead, ahead_ids)         # a step that samples nothing: committed right behind
                    sched.commit(plan, ids)
                    if also is not None:
                        sched.commit(*also)
                        also = None
                    for f in sched.collect():
                        results[f.request_id] = f
                    steps += 1
                    if steps % 64 == 0:
                        self.engine.check_device_errors()
                except Exception as e:
                    # a failed step fails the requests that were running and frees what they hold; the
                    # queue goes on (crates/rllm-server/src/engine.rs:569-578)
                    pending = also = None
                    sched.fail_running(f"step failed: {type(e).__name__}: {e}")
                    for f in sched.collect():
                        results[f.request_id] = f
            try:
                self.engine.check_device_errors()
            except Exception as e:
                # which step the kernel belonged to is not known: nothing generated in this call is to be used
                for i in range(len(prompts)):
                    f = results.get(i)
                    if f is None or f.reason != "error":
                        results[i] = Finished(i, f.tokens if f else [], "error", f"{type(e).__name__}: {e}")
        finally:
            # whatever ended the loop (an interrupt included), nothing of this call stays in the cache:
            # the next call numbers its requests from 0 again
            sched.release_all()
        self.last_stats = dict(sched.stats)
        out = [results[i] for i in range(len(prompts))]
        self.last_errors = {f.request_id: f.error for f in out if f.reason == "error"}
        if return_reasons:
            return [(f.tokens, f.reason) for f in out]
        if self.last_errors:
            raise GenerationError(out)
        return [f.tokens for f in out]

    @staticmethod
    def _ids_for(plan, ahead, sampled):
        """The ids that `plan`'s sampler left on the device, in the order of the items of `ahead` that
        take them (those of `plan`'s requests that go on; one that ends with its token is not among them)."""
        order = {id(p.seq): j for j, p in enumerate(q for q in plan if q.want_last)}
        src = [order[id(p.seq)] for p in ahead if p.sampled]
        ids = sampled.device_ids
        if src == list(range(len(src))):
            return ids
        return ids.index_select(0, torch.tensor(src, dtype=torch.int64, device=ids.device))

    def _run_step(self, plan, host_samplers, device_tokens=None):
        """One engine step for the planned items and one sampled id per item that wants its last row:
        a list (no row wanted, or sampled on the host) or the ids still on the device (_SampledIds)."""
        items = [StepItem(p.seq.rid, p.tokens, [p.take - 1] if p.want_last else []) for p in plan]
        logits = self.engine.step(items, device_tokens=device_tokens,
                                  n_device=sum(1 for p in plan if p.sampled) if device_tokens is not None else None)
        wanted = [p for p in plan if p.want_last]
        if not wanted:
            return []
        if self.host_sampling:
            ids = []
            rows = logits.float().cpu().numpy()
            for r, p in enumerate(wanted):
                hs = host_samplers.setdefault(p.seq.rid, HostSampler(p.seq.req.params))
                ids.append(hs.sample(rows[r], p.seq.counts))
            return ids
        ids = sample_rows(logits, [p.seq.req.params for p in wanted], [p.counter for p in wanted],
                          [p.seq.counts for p in wanted])
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=ids.device)
        return _SampledIds(ids, self._copy_stream)


class GenerationError(RuntimeError):
    """Some requests of a generate() call failed.  `results`: one scheduler record per prompt
    (`tokens`, `reason`, `error`), the successful ones with their tokens; `errors`: index -> message."""

    def __init__(self, results):
        self.results = list(results)
        self.errors = {f.request_id: f.error for f in self.results if f.reason == "error"}
        first = next(iter(self.errors.items()))
        more = f" (and {len(self.errors) - 1} more)" if len(self.errors) > 1 else ""
        super().__init__(f"request {first[0]}: {first[1]}{more}")


def generate(model, prompts, max_tokens: int = 256, temperature: float = 0.0, top_k: int = 0,
             top_p: float = 1.0, seed: int = 0, dtype="bfloat16", device="cuda:0", ctx: int = 4096,
             block_size: int = 32, prefill_chunk: int = 512, parallel: int = 4,
             kv_tokens: Optional[int] = None, stop_ids=(), host_sampling: bool = False,
             frequency_penalty: float = 0.0, presence_penalty: float = 0.0, logit_bias=()):
    """One call: load `model` (a folder), generate for `prompts` (lists of token ids)."""
    llm = LLM(model, dtype=dtype, device=device, ctx=ctx, block_size=block_size,
              prefill_chunk=prefill_chunk, parallel=parallel, kv_tokens=kv_tokens,
              host_sampling=host_sampling)
    return llm.generate(prompts, max_tokens=max_tokens, temperature=temperature, top_k=top_k,
                        top_p=top_p, seed=seed, stop_ids=stop_ids, frequency_penalty=frequency_penalty,
                        presence_penalty=presence_penalty, logit_bias=logit_bias)
