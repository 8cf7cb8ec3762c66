"""Benchmark of the engine on one B200: decode tokens per second at the layer sizes of
Qwen3-8B (random bf16 weights, batch 8, 2,048-token prompts in a 4,096-token context), plus
prefill of 2,048 tokens, decode at batch 1 and 64, the same decode end to end through the
Python entry point, and the roofline fractions.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Timing: CUDA events on the launching stream,
synchronize on both sides, W >= 3 warm-up steps; every step streams all weights (16 GB at full
depth, far above the 126 MB L2), so no L2 flush is needed between steps.  `e2e` is the same decode
step through the call a user makes, `LLM.generate` (host token ids in and out every step, the
scheduler in the loop), timed by the wall clock as the difference between two generations.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960, use_sliding_window=False)
# the other Qwen3 shapes the reference's numbers are quoted on (not the default run)
QWEN3_06B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600)
SHAPES = {"8b": QWEN3_8B, "0.6b": QWEN3_06B, "32b": QWEN3_32B}
FULL_LAYERS = 36
CTX, PROMPT, PREFILL_TOKENS = 4096, 2048, 2048
METRIC = "decode tok/s at batch 8 (Qwen3-8B bf16, 2,048-token prompts, ctx 4,096)"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
        sm = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples if len(s) >= 6 for n, v in zip(names, s[2:6]) if v == "Active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def reference_arm():
    """AxiomOperator/rllm is a Rust workspace (Cargo.toml, no setup.py / pyproject.toml): pip has
    nothing to install, and neither cargo nor rustc exist in this image."""
    print(json.dumps({"impl": "reference",
                      "unavailable": "AxiomOperator/rllm is a Rust workspace: pip answers 'not installable, neither "
                                     "setup.py nor pyproject.toml found', and cargo/rustc are not in this image"}))
    return 0


def weight_bytes(model):
    """Bytes of every weight a decode step reads once: all layer matrices and norms, the final
    norm and the LM head (the embedding table only gives one row per token)."""
    seen, total = set(), 0
    parts = [p for b in model.blocks for p in b.parts()] + [model.final_norm, model.lm_head]
    for p in parts:
        for v in vars(p).values():
            if hasattr(v, "data_ptr") and hasattr(v, "numel") and v.is_cuda and v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                total += v.numel() * v.element_size()
    return total


def main():
    global PROMPT, CTX
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: Qwen3-8B (default), 0.6B or 32B")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--block-size", type=int, default=16, help="tokens per page of the KV cache (16: the reference's default)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of every prompt (the context the decode steps start from)")
    ap.add_argument("--ctx", type=int, default=None, help="tokens a request may hold (default: twice the prompt)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and prefill")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving"],
                    help="decode: the default line.  serving: --requests prompts of 16..2,048 tokens with 128..512 "
                         "generated tokens each through LLM.generate (continuous batching), one line of its own")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--parallel", type=int, default=32, help="serving: requests running at once")
    ap.add_argument("--prefill-chunk", type=int, default=512, help="serving: prompt tokens per step")
    ap.add_argument("--profile", choices=["decode", "prefill"],
                    help="run only that step between cudaProfilerStart/Stop (for ncu --profile-from-start off) "
                         "and print no benchmark line")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm()
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    PROMPT = a.prompt_len
    CTX = a.ctx if a.ctx is not None else 2 * PROMPT

    import torch
    from rllm_b200.config import config_from_dict
    from rllm_b200.csrc import ops
    from rllm_b200.engine import Engine, StepItem
    from rllm_b200.models.model import random_model
    from rllm_b200.sampling.device import sample_rows
    from rllm_b200.sampling.params import SamplingParams

    pk = peaks()
    full_layers = SHAPES[a.shape]["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    cfg_d = dict(SHAPES[a.shape], num_hidden_layers=a.layers)
    config = config_from_dict(cfg_d)
    torch.cuda.set_device(0)
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0", generate_on_device=True)
    V = config.vocab_size
    wbytes = weight_bytes(model)
    g = torch.Generator().manual_seed(1)
    greedy = SamplingParams()

    def decode_run(batch, steps, warmup):
        """Prefills `batch` prompts of PROMPT tokens, then times `steps` decode steps."""
        eng = Engine(model, block_size=a.block_size, max_tokens=batch * CTX, max_requests=batch)
        prompts = [torch.randint(0, V, (PROMPT,), generator=g).tolist() for _ in range(batch)]
        for b in range(batch):                       # prefill in portions of 512, one request at a time
            for c in range(0, PROMPT, 512):
                eng.step([StepItem(b, prompts[b][c:c + 512], [])])
        nxt = [torch.randint(0, V, (steps + warmup,), generator=g).tolist() for _ in range(batch)]
        cur = [int(n[0]) for n in nxt]
        launches0 = ops.launch_count()
        h2d = 0
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                launches0 = ops.launch_count()
                start.record()
            items = [StepItem(b, [cur[b]], [0]) for b in range(batch)]
            logits = eng.step(items)
            ids = sample_rows(logits, [greedy] * batch, [0] * batch)
            cur = [int(n[i + 1]) if i + 1 < len(n) else 0 for n in nxt]
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        kv_tokens = sum(eng.cache.length(b) for b in range(batch)) - batch * steps / 2.0
        kv_bytes = kv_tokens * eng.cache.bytes_per_token(2)
        launches = (ops.launch_count() - launches0)
        staging = eng.last_upload_bytes
        for b in range(batch):
            eng.finish(b)
        del eng
        gc.collect()                                 # the graphs of the engine hold memory pools
        torch.cuda.empty_cache()
        return {"ms": ms, "tok_s": batch * 1000.0 / ms, "bytes": wbytes + kv_bytes, "launches": launches,
                "h2d": staging, "d2h": 4 * batch}

    def generate_run(batch, steps, warmup):
        """The same decode steps through the entry point a user calls, LLM.generate: token ids in
        on the host, token ids out on the host, every step (the step's index arrays go up from
        pinned memory, the sampled ids come back and decide the next step's input).  The prompts
        are prefilled whole, 16 to a step at most (the activations of more would not fit beside
        the largest shape), so the requests start and end at most three steps apart; the time of
        a decode step is the difference between a run that generates warmup + 3 * steps tokens and
        one that generates warmup tokens, over 3 * steps: the steps the long run has more are steps
        in which all `batch` requests decode (wall clock, synchronized on both sides)."""
        from rllm_b200 import LLM
        llm = LLM(model, ctx=CTX, block_size=a.block_size, prefill_chunk=min(batch, 16) * PROMPT, parallel=batch,
                  kv_tokens=batch * CTX)
        prompts = [torch.randint(0, V, (PROMPT,), generator=g).tolist() for _ in range(batch)]

        def timed(n_tokens):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = llm.generate(prompts, max_tokens=n_tokens)
            torch.cuda.synchronize()
            assert all(len(o) == n_tokens for o in out)
            return time.perf_counter() - t0

        timed(warmup)                                   # kernels loaded, the graph of this shape captured
        # the prefill of the prompts is in both runs and varies by some milliseconds from run to run: the
        # long run has three times the steps asked for, so that this noise is small against the difference
        short = min(timed(warmup) for _ in range(3))
        long_ = min(timed(warmup + 3 * steps) for _ in range(2))
        ms = (long_ - short) * 1000.0 / (3 * steps)
        staging = llm.engine.last_upload_bytes
        del llm
        gc.collect()
        torch.cuda.empty_cache()
        return {"ms": ms, "tok_s": batch * 1000.0 / ms, "h2d": staging, "d2h": 4 * batch}

    def idle(seconds=2.0):
        torch.cuda.synchronize()
        time.sleep(seconds)

    def serving_run():
        """Continuous batching through the entry point: requests of mixed lengths wait, are admitted
        as others finish, prompts go in portions beside decoded tokens.  Wall clock around the
        second of two identical generations (the first loads kernels and captures graphs)."""
        from rllm_b200 import LLM
        lens = torch.randint(16, PROMPT + 1, (a.requests,), generator=g).tolist()
        outs = torch.randint(128, 513, (a.requests,), generator=g).tolist()
        prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]
        llm = LLM(model, ctx=CTX, block_size=a.block_size, prefill_chunk=a.prefill_chunk, parallel=a.parallel,
                  kv_tokens=a.parallel * (PROMPT + 512))
        llm.generate(prompts, max_tokens=outs)
        clocks = ClockSampler()
        clocks.start()
        launches0 = ops.launch_count()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = llm.generate(prompts, max_tokens=outs)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        clk = clocks.stop()
        st = llm.last_stats
        assert [len(r) for r in res] == outs
        gen = sum(outs)
        print(json.dumps({
            "metric": f"generated tok/s, continuous batching (Qwen3-{a.shape.upper()} bf16, {a.requests} requests, "
                      "prompts 16..2,048, 128..512 generated)",
            "value": round(gen / dt, 1), "unit": "tok/s", "n_gpus": 1, "steps": st["steps"], "warmup": 1,
            "ms_per_step": round(dt * 1000.0 / st["steps"], 4), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic: random weights N(0,0.02), uniform random token ids", "impl": "ours",
            "config": {"model": f"Qwen3-{a.shape.upper()}-shaped", "layers": a.layers, "layers_full_model": full_layers,
                       "requests": a.requests, "parallel": a.parallel, "prefill_chunk": a.prefill_chunk,
                       "kv_block": a.block_size, "prompt_tokens": sum(lens), "generated_tokens": gen},
            "prompt_tok_s": round(sum(lens) / dt, 1), "seconds": round(dt, 3), "preemptions": st["preemptions"],
            "clocks": clk, "gpu_launches": ops.launch_count() - launches0}))
        return 0

    if a.workload == "serving":
        return serving_run()

    if a.profile:
        eng = Engine(model, block_size=a.block_size, max_tokens=a.batch * CTX, max_requests=a.batch)
        prompts = [torch.randint(0, V, (PROMPT,), generator=g).tolist() for _ in range(a.batch)]
        if a.profile == "prefill":
            eng.step([StepItem(0, prompts[0], [PROMPT - 1])])          # warm-up
            eng.finish(0)
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            eng.step([StepItem(0, prompts[0], [PROMPT - 1])])
        else:
            for b in range(a.batch):
                for c in range(0, PROMPT, 512):
                    eng.step([StepItem(b, prompts[b][c:c + 512], [])])
            for i in range(3):                                         # eager, capture, replay
                eng.step([StepItem(b, [1 + i], [0]) for b in range(a.batch)])
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            logits = eng.step([StepItem(b, [7], [0]) for b in range(a.batch)])
            sample_rows(logits, [greedy] * a.batch, [0] * a.batch)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(f"profiled one {a.profile} step: layers {a.layers}, batch {a.batch}")
        return 0

    clocks = ClockSampler()
    clocks.start()
    main_run = decode_run(a.batch, a.steps, a.warmup)
    clk = clocks.stop()
    e2e_run = generate_run(a.batch, a.steps, a.warmup)

    out = {
        "metric": METRIC.replace("Qwen3-8B", f"Qwen3-{a.shape.upper()}").replace("batch 8", f"batch {a.batch}")
                        .replace("2,048-token", f"{PROMPT:,}-token").replace("ctx 4,096", f"ctx {CTX:,}"), "value": round(main_run["tok_s"], 2), "unit": "tok/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(main_run["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids", "impl": "ours",
        "config": {"model": f"Qwen3-{a.shape.upper()}-shaped", "layers": a.layers, "layers_full_model": full_layers,
                   "hidden": config.hidden_size, "heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size,
                   "vocab": V, "global_batch": a.batch, "seq_len": CTX, "prompt_len": PROMPT,
                   "kv_block": a.block_size, "parallelism": "single GPU",
                   "l2": "no flush: each step streams %.1f GB of weights (> 126 MB L2)" % (wbytes / 1e9),
                   "peaks": pk["source"]},
        "clocks": clk,
        "e2e": {"value": round(e2e_run["tok_s"], 2), "unit": "tok/s", "h2d_bytes_per_step": e2e_run["h2d"],
                "d2h_bytes_per_step": e2e_run["d2h"]},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(main_run["bytes"] / main_run["ms"] / 1e6, 1),
                     "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["bytes"] / main_run["ms"] / 1e6 / pk["hbm_gbs"], 4)},
    }
    if not a.skip_points:
        # Decode at batch 1 and 64, device-timed like the main run.  What ran before decides the clock a
        # measurement starts with (after seconds at the power cap it stays low for a while; a prefill
        # behind the batch-64 steps took 24.8 ms, behind two idle seconds 23.8), so each of the
        # measurements below starts from a device that has idled for two seconds, and warms up by itself.
        steps = a.steps
        points, fracs, e2es = {}, {}, {}
        for b in (1, 64):
            idle()
            r = decode_run(b, steps, a.warmup)
            points[f"decode_b{b}"] = round(r["tok_s"], 2)
            fracs[f"decode_b{b}"] = round(r["bytes"] / r["ms"] / 1e6 / pk["hbm_gbs"], 4)
        # prefill of 2,048 tokens in one step
        toks = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()

        def prefill_ms(block_size):
            eng = Engine(model, block_size=block_size, max_tokens=CTX, max_requests=1)
            times = []
            for rep in range(4):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                s.record()
                eng.step([StepItem("p", toks, [PREFILL_TOKENS - 1])])
                e.record()
                torch.cuda.synchronize()
                eng.finish("p")
                if rep:
                    times.append(s.elapsed_time(e))
            del eng
            torch.cuda.empty_cache()
            return min(times)
        idle()
        ms = prefill_ms(a.block_size)
        # The two page sizes against each other (16 is the reference's default): a prefill runs at the
        # power cap and the clock settles lower from run to run, so they are measured in turn, after the
        # runs above have warmed the device up; comparable with each other, not with the figure above.
        by_block = {16: float("inf"), 32: float("inf")}
        for _ in range(2):
            for b in by_block:
                by_block[b] = min(by_block[b], prefill_ms(b))
        c = config
        per_tok = 2 * a.layers * (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                                  + c.num_attention_heads * c.head_dim * c.hidden_size
                                  + 3 * c.hidden_size * c.intermediate_size)
        attn = a.layers * 4 * c.num_attention_heads * c.head_dim * PREFILL_TOKENS * PREFILL_TOKENS / 2
        flops = per_tok * PREFILL_TOKENS + attn + 2 * c.hidden_size * V
        out["prefill"] = {"value": round(PREFILL_TOKENS * 1000.0 / ms, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(ms, 3), "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                          "peak_tflops": pk["bf16_tflops_sustained"]}
        out["prefill_ms_warm"] = {f"block{b}": round(v, 3) for b, v in by_block.items()}
        for b in (1, 64):
            e2es[f"decode_b{b}"] = round(generate_run(b, max(8, steps // 2), a.warmup)["tok_s"], 2)
        out["points"] = points
        out["points_frac"] = fracs              # achieved share of the HBM roofline (weights once + live cache) / time
        out["points_e2e"] = e2es                # the same batches through LLM.generate
    ops.check_device_errors("cuda:0")          # a kernel that gave up a bounded wait: no number
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
