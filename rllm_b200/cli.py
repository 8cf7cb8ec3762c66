"""Command line in the manner of AxiomOperator/rllm's ``rllm`` (crates/rllm-cli/src/main.rs:24-237):

  rllm run MODEL PROMPT [-n/--max-tokens 256] [-t/--temperature 0] [--top-k 0] [--top-p 1.0]
                        [--seed 0] [--ctx 4096] [--block-size 32] [--prefill-chunk 512]
                        [--kv-type bf16|f32] [--show-ids]
  rllm bench MODEL [-p/--n-prompt 512] [-n/--n-gen 128] [-r/--reps 3] [--depth 0] [-b/--batch 1]
  rllm compare MODEL PROMPT [-n/--steps 32]      engine float32 against engine bfloat16, same tokens
  rllm compare-ref MODEL DUMP [--prefill-chunk 512]
                                                  engine against a reference's logits on the same tokens
  rllm perplexity MODEL TOKENS [--ctx 512] [--chunks N]
                                                  perplexity over a file of token ids, chunk by chunk
  rllm inspect MODEL                              configuration and tensor list
  rllm random-model OUT --config FILE [--seed 0] [--dtype bfloat16] [--shards 1]
  rllm replay ...                                 same as bin/trace_run

The engine has no tokenizer: PROMPT is token ids separated by commas or spaces, or @FILE holding
them.  MODEL is a folder with config.json and model.safetensors.  ``--kv-type`` chooses the
precision of the whole engine (bf16 serving path, f32 true 32-bit path).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def _ids(text: str) -> list:
    if text.startswith("@"):
        text = Path(text[1:]).read_text()
    return [int(t) for t in text.replace(",", " ").split()]


def _dtype(kv_type: str) -> str:
    return {"bf16": "bfloat16", "bfloat16": "bfloat16", "f32": "float32", "float32": "float32"}[kv_type]


def cmd_run(a) -> int:
    from .llm import LLM
    prompt = _ids(a.prompt)
    if len(prompt) + a.max_tokens > a.ctx:
        print(f"prompt ({len(prompt)}) + max tokens ({a.max_tokens}) exceed --ctx {a.ctx}", file=sys.stderr)
        return 2
    t0 = time.time()
    llm = LLM(a.model, dtype=_dtype(a.kv_type), device=a.device, ctx=a.ctx, block_size=a.block_size,
              prefill_chunk=a.prefill_chunk, parallel=1, host_sampling=a.host_sampling)
    print(f"[rllm] loaded in {time.time() - t0:.2f} s", file=sys.stderr)
    t0 = time.time()
    out = llm.generate([prompt], max_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k,
                       top_p=a.top_p, seed=a.seed, stop_ids=a.stop_id or ())[0]
    dt = time.time() - t0
    print(" ".join(map(str, out)))
    if a.show_ids:
        print(f"[rllm] prompt ids: {prompt}", file=sys.stderr)
    print(f"[rllm] {len(prompt)} prompt + {len(out)} generated tokens in {dt:.3f} s "
          f"({len(out) / dt:.1f} tok/s overall)", file=sys.stderr)
    return 0


def cmd_bench(a) -> int:
    import torch
    from .engine import Engine, StepItem
    from .models.model import load_model
    _, model = load_model(a.model, _dtype(a.kv_type), a.device)
    V = model.spec.vocab_size
    per_req = max(a.depth, 0) + a.n_prompt + a.n_gen
    eng = Engine(model, block_size=a.block_size, max_tokens=(per_req + 64) * a.batch, max_requests=a.batch)
    g = torch.Generator().manual_seed(1)
    res = {"pp": [], "tg": []}
    for rep in range(a.reps + 1):                     # first repetition is the warm-up
        ids = [torch.randint(0, V, (per_req,), generator=g).tolist() for _ in range(a.batch)]
        if a.depth > 0:
            eng.step([StepItem(b, ids[b][:a.depth], []) for b in range(a.batch)])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.step([StepItem(b, ids[b][a.depth:a.depth + a.n_prompt], [a.n_prompt - 1]) for b in range(a.batch)])
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        for i in range(a.n_gen):
            p = a.depth + a.n_prompt + i
            logits = eng.step([StepItem(b, [ids[b][p]], [0]) for b in range(a.batch)])
            logits.argmax(-1)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        for b in range(a.batch):
            eng.finish(b)
        if rep:
            res["pp"].append(a.batch * a.n_prompt / (t1 - t0))
            res["tg"].append(a.batch * a.n_gen / (t2 - t1) if a.n_gen else 0.0)
    mean = lambda v: sum(v) / len(v)
    print(json.dumps({"pp": a.n_prompt, "tg": a.n_gen, "batch": a.batch, "depth": a.depth,
                      "pp_tok_s": mean(res["pp"]), "tg_tok_s": mean(res["tg"])}))
    return 0


def cmd_compare(a) -> int:
    """Feeds the same tokens through the float32 and the bfloat16 engine; both continue from the
    float32 argmax so that errors do not compound (crates/rllm-cli/src/main.rs:465-508)."""
    import torch
    from .engine import Engine, StepItem
    from .models.model import load_model
    prompt = _ids(a.prompt)
    engines = []
    for dt in ("float32", "bfloat16"):
        _, m = load_model(a.model, dt, a.device)
        engines.append(Engine(m, block_size=a.block_size, max_tokens=len(prompt) + a.steps + 64, max_requests=1))
    feed, worst, mism = prompt, 0.0, 0
    for i in range(a.steps + 1):
        rows = []
        for e in engines:
            if len(feed) > 1:
                for c in range(0, len(feed) - 1, a.prefill_chunk):
                    e.step([StepItem(0, feed[c:min(c + a.prefill_chunk, len(feed) - 1)], [])])
            rows.append(e.step([StepItem(0, feed[-1:], [0])])[0].float().cpu())
        diff = float((rows[0] - rows[1]).abs().max())
        rel = diff / float(rows[0].abs().max())
        worst = max(worst, rel)
        mism += int(rows[0].argmax()) != int(rows[1].argmax())
        feed = [int(rows[0].argmax())]
    print(f"max relative logit diff {worst:.3e}; argmax mismatches {mism}/{a.steps + 1}")
    return 0


def read_ref_dump(path):
    """A reference dump: "RLLMREF1" | u32 n_vocab | u32 n_prompt | u32 n_total | u32 tokens[n_total] |
    f32 logits[n_total][n_vocab], little-endian; row i holds the logits after tokens[0..=i]
    (tools/llama-ref/llama_ref.cpp:6-9, crates/rllm-cli/src/main.rs:525-536)."""
    import numpy as np
    raw = Path(path).read_bytes()
    if len(raw) < 20 or raw[:8] != b"RLLMREF1":
        raise ValueError(f"{path} is not a reference dump (no RLLMREF1 header)")
    n_vocab, n_prompt, n_total = (int(x) for x in np.frombuffer(raw, "<u4", 3, 8))
    tok_end = 20 + 4 * n_total
    if len(raw) != tok_end + 4 * n_total * n_vocab:
        raise ValueError(f"{path}: truncated reference dump")
    tokens = np.frombuffer(raw, "<u4", n_total, 20).astype(np.int64).tolist()
    logits = np.frombuffer(raw, "<f4", n_total * n_vocab, tok_end).reshape(n_total, n_vocab)
    return n_vocab, n_prompt, tokens, logits


def write_ref_dump(path, n_prompt: int, tokens, logits) -> None:
    """Writes a dump in the format read_ref_dump reads (logits: [len(tokens), vocab] float32)."""
    import numpy as np
    logits = np.ascontiguousarray(logits, dtype="<f4")
    head = np.array([logits.shape[1], n_prompt, len(tokens)], dtype="<u4").tobytes()
    Path(path).write_bytes(b"RLLMREF1" + head + np.asarray(tokens, dtype="<u4").tobytes() + logits.tobytes())


def cmd_compare_ref(a) -> int:
    """Feeds the dump's token ids through the engine (prompt in portions of --prefill-chunk) and
    reports, per position, the largest logit difference, the relative difference, KL(reference ||
    ours) and the two top-1 tokens, then a summary (crates/rllm-cli/src/main.rs:538-606)."""
    import numpy as np
    from .engine import Engine, StepItem
    from .models.model import load_model
    n_vocab, n_prompt, tokens, ref = read_ref_dump(a.reference)
    _, model = load_model(a.model, _dtype(a.kv_type), a.device)
    if model.spec.vocab_size != n_vocab:
        print(f"vocab mismatch: model {model.spec.vocab_size} vs reference {n_vocab}", file=sys.stderr)
        return 2
    eng = Engine(model, block_size=a.block_size, max_tokens=len(tokens) + 64, max_requests=1)
    rows = []
    for c in range(0, len(tokens), a.prefill_chunk):
        part = tokens[c:c + a.prefill_chunk]
        rows.append(eng.step([StepItem(0, part, list(range(len(part))))]).float().cpu().numpy())
    ours = np.concatenate(rows)

    def log_softmax(x):
        x = x.astype(np.float64)
        m = x.max()
        return x - (m + np.log(np.exp(x - m).sum()))

    kl_sum = kl_max = worst_rel = 0.0
    agree = 0
    print(f"{'pos':>6} {'max|diff|':>10} {'rel':>10} {'KL':>10}  {'ref':>8} {'rllm':>8}  next token")
    for i in range(len(tokens)):
        diff = float(np.abs(ref[i] - ours[i]).max())
        rel = diff / max(float(np.abs(ref[i]).max()), 1e-30)
        lp, lq = log_softmax(ref[i]), log_softmax(ours[i])
        kl = max(float((np.exp(lp) * (lp - lq)).sum()), 0.0)
        ta, tb = int(np.nan_to_num(ref[i], nan=-np.inf).argmax()), int(np.nan_to_num(ours[i], nan=-np.inf).argmax())
        kl_sum, kl_max, worst_rel, agree = kl_sum + kl, max(kl_max, kl), max(worst_rel, rel), agree + (ta == tb)
        if i + 3 >= n_prompt or ta != tb:           # the last prompt rows and every generated row
            print(f"{i:>6} {diff:>10.4f} {rel:>10.2e} {kl:>10.2e}  {ta:>8} {tb:>8}" + ("  <-- top-1 differs" if ta != tb else ""))
    n = len(tokens)
    print(f"summary: {n} positions | top-1 agreement {agree}/{n} | KL mean {kl_sum / n:.2e} max {kl_max:.2e} | "
          f"worst relative logit diff {worst_rel:.2e}")
    return 0


def cmd_perplexity(a) -> int:
    """Perplexity over a file of token ids (the engine has no tokenizer: the reference scores a text
    file): chunks of --ctx tokens, each in a fresh cache, the positions ctx/2 .. ctx-2 of a chunk
    scored on the token that follows; log-sum-exp on the device in float64
    (crates/rllm-cli/src/main.rs:608-679)."""
    import math
    import torch
    from .engine import Engine, StepItem
    from .models.model import load_model
    tokens = _ids(a.tokens if a.tokens.startswith("@") else "@" + a.tokens)
    n_ctx = a.ctx
    if n_ctx < 4 or len(tokens) < 2 * n_ctx:
        print(f"need at least {2 * n_ctx} tokens for --ctx {n_ctx}", file=sys.stderr)
        return 2
    n_chunk = min(len(tokens) // n_ctx, a.chunks or 1 << 60)
    _, model = load_model(a.model, _dtype(a.kv_type), a.device)
    eng = Engine(model, block_size=a.block_size, max_tokens=n_ctx + 64, max_requests=1)
    first = n_ctx // 2
    rows = list(range(first, n_ctx - 1))
    nll = nll2 = 0.0
    count = 0
    t0 = time.time()
    for c in range(n_chunk):
        chunk = tokens[c * n_ctx:(c + 1) * n_ctx]
        logits = eng.step([StepItem(c, chunk, rows)]).double()
        eng.finish(c)
        target = torch.tensor(chunk[first + 1:], dtype=torch.long, device=logits.device)
        v = (torch.logsumexp(logits, dim=1) - logits.gather(1, target[:, None])[:, 0]).cpu()
        nll += float(v.sum())
        nll2 += float((v * v).sum())
        count += v.numel()
        print(f"[{c + 1}]{math.exp(nll / count):.4f} ", end="", file=sys.stderr, flush=True)
    print(file=sys.stderr)
    mean = nll / count
    ppl = math.exp(mean)
    err = ppl * math.sqrt(max(nll2 / count - mean * mean, 0.0) / max(count - 1, 1))
    print(f"Final estimate: PPL = {ppl:.4f} +/- {err:.5f}  ({n_chunk} chunks, {count} scored tokens, "
          f"{time.time() - t0:.1f} s)")
    return 0


def cmd_inspect(a) -> int:
    from .config import load_config
    from .weights import SafetensorsFile
    cfg = load_config(a.model)
    print(cfg)
    from .weights import weight_files
    for path in weight_files(a.model)[1]:
        with SafetensorsFile(path) as f:
            for n in sorted(f.names()):
                print(f"{n:60s} {str(f.dtype(n)):16s} {str(list(f.shape(n))):20s} {path.name}")
    return 0


def cmd_random_model(a) -> int:
    import torch
    from .config import config_from_dict
    from .weights import write_random_model
    cfg = config_from_dict(json.loads(Path(a.config).read_text()))
    write_random_model(cfg, a.out, seed=a.seed, shards=a.shards,
                       dtype={"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype])
    print(a.out)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="rllm", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("model")
        p.add_argument("-d", "--device", default="cuda:0")
        p.add_argument("--block-size", type=int, default=32)
        p.add_argument("--kv-type", default="bf16", choices=["bf16", "f32", "bfloat16", "float32"])

    p = sub.add_parser("run"); common(p)
    p.add_argument("prompt")
    p.add_argument("-n", "--max-tokens", type=int, default=256)
    p.add_argument("-t", "--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--ctx", type=int, default=4096)
    p.add_argument("--prefill-chunk", type=int, default=512)
    p.add_argument("--show-ids", action="store_true")
    p.add_argument("--host-sampling", action="store_true")
    p.add_argument("--stop-id", type=int, action="append")
    p.set_defaults(fn=cmd_run)

    p = sub.add_parser("bench"); common(p)
    p.add_argument("-p", "--n-prompt", type=int, default=512)
    p.add_argument("-n", "--n-gen", type=int, default=128)
    p.add_argument("-r", "--reps", type=int, default=3)
    p.add_argument("--depth", type=int, default=0)
    p.add_argument("-b", "--batch", type=int, default=1)
    p.set_defaults(fn=cmd_bench)

    p = sub.add_parser("compare"); common(p)
    p.add_argument("prompt")
    p.add_argument("-n", "--steps", type=int, default=32)
    p.add_argument("--prefill-chunk", type=int, default=512)
    p.set_defaults(fn=cmd_compare)

    p = sub.add_parser("compare-ref"); common(p)
    p.add_argument("reference")
    p.add_argument("--prefill-chunk", type=int, default=512)
    p.set_defaults(fn=cmd_compare_ref)

    p = sub.add_parser("perplexity"); common(p)
    p.add_argument("tokens", help="file of token ids")
    p.add_argument("--ctx", type=int, default=512)
    p.add_argument("--chunks", type=int, default=None)
    p.set_defaults(fn=cmd_perplexity)

    p = sub.add_parser("inspect"); p.add_argument("model"); p.set_defaults(fn=cmd_inspect)

    p = sub.add_parser("random-model")
    p.add_argument("out"); p.add_argument("--config", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--shards", type=int, default=1,
                   help="write this many model-0000i-of-0000N.safetensors files and a weight map")
    p.set_defaults(fn=cmd_random_model)

    p = sub.add_parser("replay", add_help=False)
    p.set_defaults(fn=None)
    argv = sys.argv[1:] if argv is None else argv
    if argv and argv[0] == "replay":
        from .replay import main as replay_main
        return replay_main(argv[1:])
    a = ap.parse_args(argv)
    rc = a.fn(a)
    if getattr(a, "device", "").startswith("cuda"):
        from .csrc import ops
        ops.check_device_errors(a.device)       # a kernel that gave up a bounded wait: the command fails
    return rc


if __name__ == "__main__":
    sys.exit(main())
