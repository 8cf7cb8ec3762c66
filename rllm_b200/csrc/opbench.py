"""Times one product kernel the way a decode step runs it: a CUDA graph of back-to-back launches
(programmatic dependent launch between them) over a rotation of weight matrices larger than L2.

    python -m rllm_b200.csrc.opbench --op skinny_gemm_tc --m 64 --n 4096 --k 4096 --epilogue accum [--splits 4]

Prints microseconds per launch (the best of five replays) and the weight bytes per second.
Ops: skinny_gemm, skinny_gemm_tc, gemv_stream, gemm_tc, gemm_lib.  Epilogues: store, accum, swiglu
(n is then the number of gate rows; the weight matrix has 2 n rows).
"""
from __future__ import annotations

import argparse

import torch

from . import ops

EPILOGUES = {"store": ops.EPI_STORE, "accum": ops.EPI_ACCUM, "swiglu": ops.EPI_SWIGLU}


def time_product(op: str, m: int, n: int, k: int, epilogue: str = "store", launches: int = 48, splits=None,
                 device: str = "cuda:0"):
    """(microseconds per launch, weight GB/s) of `op` on an [m, k] activation and an [n, k] weight."""
    epi = EPILOGUES[epilogue]
    rows = 2 * n if epi == ops.EPI_SWIGLU else n
    copies = max(2, -(-(3 * 126 * 2 ** 20) // (rows * k * 2)))           # the rotation covers three times L2
    copies = min(copies, launches)
    ws = [(torch.randn(rows, k, device=device) * 0.05).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(m, k, device=device).to(torch.bfloat16)
    out = torch.zeros(m, n, device=device, dtype=torch.bfloat16 if epi == ops.EPI_SWIGLU else torch.float32)
    up = n if epi == ops.EPI_SWIGLU else 0

    def call(w):
        if op == "gemm_lib":
            if epi == ops.EPI_SWIGLU:
                raise SystemExit("gemm_lib has no SwiGLU epilogue")
            return ops.gemm_lib(x, w, out, accumulate=epi == ops.EPI_ACCUM)
        if op == "skinny_gemm_tc":
            return ops.skinny_gemm_tc(x, w, out, epi, up, n_splits=splits)
        return getattr(ops, op)(x, w, out, epi, up)

    call(ws[0])
    torch.cuda.synchronize()
    ops.check_device_errors(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            call(ws[i % copies])
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(5):
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(stop) * 1000.0 / launches)
    ops.check_device_errors(device)
    return best, rows * k * 2 / best / 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--op", required=True, choices=["skinny_gemm", "skinny_gemm_tc", "gemv_stream", "gemm_tc", "gemm_tc2", "gemm_lib"])
    ap.add_argument("--m", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--epilogue", default="store", choices=sorted(EPILOGUES))
    ap.add_argument("--splits", type=int, default=None, help="skinny_gemm_tc: CTAs of a cluster along K")
    ap.add_argument("--launches", type=int, default=48)
    a = ap.parse_args(argv)
    us, gbs = time_product(a.op, a.m, a.n, a.k, a.epilogue, a.launches, a.splits)
    print(f"{a.op} m={a.m} n={a.n} k={a.k} {a.epilogue}" + (f" splits={a.splits}" if a.splits else "")
          + f": {us:.2f} us per launch, {gbs:.0f} GB/s of weights")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
