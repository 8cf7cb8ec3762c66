"""Trace replay driver behind ``bin/trace_run`` (see that file for the formats).

In the spirit of AxiomOperator/rllm's ``compare-ref`` (crates/rllm-cli/src/main.rs:518-606),
which re-feeds dumped token ids and compares logits position by position: this tool only
produces the logits, under whatever cutting of the work the trace prescribes.  It has no
forward pass, cache or loader of its own.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_TOKENS = 32      # the engine's page size; 64 is a multiple, so --max-tokens needs no rounding


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=PAGE_TOKENS)
    ap.add_argument("--max-requests", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; the engine has no CPU path", file=sys.stderr)
        return 3
    from .engine import Engine, StepItem
    from .models.model import load_model

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    _, model = load_model(args.model, args.dtype, args.device)
    engine = Engine(model, block_size=args.block_size, max_tokens=args.max_tokens,
                    max_requests=args.max_requests)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        items = [StepItem(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        if items:
            logits = engine.step(items)
            if logits is not None:
                rows = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4")
                engine.check_device_errors()          # a kernel that gave up a wait: no logits are written
                rows.tofile(out_dir / f"{step}.f32")
        for rid in rec.get("end", []):
            engine.finish(rid)
        print(f"done {step}", flush=True)
    return 0
