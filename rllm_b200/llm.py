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


class LLM:
    def __init__(self, model, dtype="bfloat16", device="cuda:0", ctx: int = 4096, block_size: int = 32,
                 prefill_chunk: int = 512, parallel: int = 4, kv_tokens: Optional[int] = None,
                 host_sampling: bool = False):
        """`model`: a folder with config.json and model.safetensors, or a loaded DecoderModel."""
        if isinstance(model, (str, bytes)) or hasattr(model, "__fspath__"):
            self.config, self.model = load_model(model, dtype, device)
        else:
            self.config, self.model = None, model
        kv_tokens = max(kv_tokens or ctx * parallel, ctx)
        self.engine = Engine(self.model, block_size=block_size, max_tokens=kv_tokens,
                             max_requests=max(parallel, 1))
        self.ctx, self.prefill_chunk, self.parallel = ctx, prefill_chunk, parallel
        self.host_sampling = host_sampling
        self.last_stats = {}

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens=256, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0, stop_ids: Sequence[int] = (),
                 return_reasons: bool = False, frequency_penalty: float = 0.0, presence_penalty: float = 0.0,
                 logit_bias=()):
        """Generates for every prompt (continuous batching); returns the generated ids per prompt,
        in order.  max_tokens: one number, or one per prompt.  Request i samples with seed
        `seed + i`.  logit_bias: (token, delta) pairs or a
        {token: delta} mapping, added to the logits with the frequency and presence penalties over
        the tokens generated so far before the token is chosen."""
        if isinstance(logit_bias, dict):
            logit_bias = tuple(logit_bias.items())
        limits = [max_tokens] * len(prompts) if isinstance(max_tokens, int) else list(max_tokens)
        if len(limits) != len(prompts):
            raise ValueError(f"max_tokens: {len(limits)} numbers for {len(prompts)} prompts")
        sched = Scheduler(self.engine.cache, ctx=self.ctx, max_num_seqs=self.parallel,
                          prefill_chunk=self.prefill_chunk)
        for i, p in enumerate(prompts):
            sched.add(Request(i, list(p), int(limits[i]),
                              SamplingParams(temperature, top_k, top_p, seed + i, frequency_penalty,
                                             presence_penalty, tuple(logit_bias)), frozenset(stop_ids)))
        results = {}
        host_samplers = {}
        steps = 0
        while sched.has_work():
            plan = sched.plan()
            for f in sched.collect():
                results[f.request_id] = f
            if not plan:
                continue
            items = [StepItem(p.seq.rid, p.tokens, [p.take - 1] if p.want_last else []) for p in plan]
            try:
                logits = self.engine.step(items)
            except Exception as e:           # a failed step fails the running requests, not the queue
                for f in sched.fail_running(f"step failed: {e}"):
                    results[f.request_id] = f
                sched.collect()
                raise
            wanted = [p for p in plan if p.want_last]
            ids = []
            if wanted:
                if self.host_sampling:
                    rows = logits.float().cpu().numpy()
                    for r, p in enumerate(wanted):
                        hs = host_samplers.setdefault(p.seq.rid, HostSampler(p.seq.req.params))
                        ids.append(hs.sample(rows[r], p.seq.counts))
                else:
                    counters = [p.seq.cached + p.take for p in wanted]
                    ids = sample_rows(logits, [p.seq.req.params for p in wanted], counters,
                                      [p.seq.counts for p in wanted]).tolist()
            sched.commit(plan, ids)
            for f in sched.collect():
                results[f.request_id] = f
            steps += 1
            if steps % 64 == 0:
                self.engine.check_device_errors()     # the ids were just read: the device is idle
        self.engine.check_device_errors()
        self.last_stats = dict(sched.stats)
        out = [results[i] for i in range(len(prompts))]
        for f in out:
            if f.reason == "error":
                raise RuntimeError(f"request {f.request_id}: {f.error}")
        if return_reasons:
            return [(f.tokens, f.reason) for f in out]
        return [f.tokens for f in out]


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
