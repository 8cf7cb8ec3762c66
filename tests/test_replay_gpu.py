"""The engine against the plain implementation under every way of cutting the work:
whole prompts, most in one step then the last 32 tokens one by one, portions of changing size
down to two tokens, and up to four live requests mixed (portions of some beside decoded tokens
of others) in a pool so small that pages are used again.  float32 and bfloat16.

The standard follows AxiomOperator/rllm's "same logits however the work is cut" test
(crates/rllm-model/tests/common/gpu.rs:74-104) and its CPU-vs-GPU comparison
(crates/rllm-cli/src/main.rs:465-508).
"""
import pytest
import torch

import helpers
from helpers import TINY, rel_err

pytestmark = pytest.mark.gpu

# max |engine - plain| / max |plain| over a logits row
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
STD = 0.08


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for name, cfg in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        helpers.make_model_dir(d, cfg, seed=11 + len(out), dtype=torch.float32, std=STD)
        out[name] = d
    return out


def make_engine(model_dir, dtype, max_tokens, block_size=16, max_requests=8):
    from rllm_b200.engine import Engine
    from rllm_b200.models.model import load_model
    _, model = load_model(model_dir, dtype, "cuda:0")
    return Engine(model, block_size=block_size, max_tokens=max_tokens, max_requests=max_requests)


def reference(model_dir, dtype, tokens):
    """Plain float32 logits; for the bfloat16 engine the weights are rounded to bfloat16 first
    (that rounding is the engine's storage format, not an error of its kernels)."""
    import plain_impl
    cfg, w = plain_impl.load_model(model_dir, torch.float32)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
    return plain_impl.forward(cfg, w, tokens)


def check(out, refs, dtype, what):
    worst = 0.0
    for (rid, pos), row in out.items():
        ref = refs[rid][pos]
        e = rel_err(row, ref)
        worst = max(worst, e)
        assert e <= TOL[dtype], f"{what}: request {rid} position {pos}: rel err {e:.3e} > {TOL[dtype]}"
        if dtype == "float32":
            assert int(row.argmax()) == int(ref.argmax()), f"{what}: request {rid} position {pos}: argmax differs"
    return worst


REQ_LENS = {"a": 70, "b": 45, "c": 97, "d": 33}


def requests_for(cfg, seed):
    return {rid: helpers.random_tokens(n, cfg["vocab_size"], seed + i)
            for i, (rid, n) in enumerate(REQ_LENS.items())}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_whole(model_dirs, name, dtype):
    cfg = TINY[name]
    reqs = requests_for(cfg, 100)
    refs = {rid: reference(model_dirs[name], dtype, t) for rid, t in reqs.items()}
    eng = make_engine(model_dirs[name], dtype, max_tokens=128)
    for rid, toks in reqs.items():
        steps = [{"entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}]
        out = helpers.run_steps(eng, steps)
        assert len(out) == len(toks)
        check(out, refs, dtype, f"whole {name}")
    eng.cache.check_invariants()
    assert eng.cache.n_free_pages(0) == eng.cache.n_blocks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_tail_decoded_one_by_one(model_dirs, name, dtype):
    cfg = TINY[name]
    reqs = requests_for(cfg, 200)
    refs = {rid: reference(model_dirs[name], dtype, t) for rid, t in reqs.items()}
    eng = make_engine(model_dirs[name], dtype, max_tokens=128)
    for rid, toks in reqs.items():
        head = max(1, len(toks) - 32)
        steps = [{"entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}]}]
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}]})
        steps[-1]["end"] = [rid]
        out = helpers.run_steps(eng, steps)
        check(out, refs, dtype, f"tail {name}")
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_portions_of_changing_size(model_dirs, name, dtype):
    cfg = TINY[name]
    reqs = requests_for(cfg, 300)
    refs = {rid: reference(model_dirs[name], dtype, t) for rid, t in reqs.items()}
    eng = make_engine(model_dirs[name], dtype, max_tokens=128)
    sizes = [7, 2, 16, 3, 2, 17, 1, 5, 32, 2, 9]
    for rid, toks in reqs.items():
        steps, i, si = [], 0, 0
        while i < len(toks):
            k = min(sizes[si % len(sizes)], len(toks) - i)
            steps.append({"entries": [{"id": rid, "tokens": toks[i:i + k], "want": list(range(k))}]})
            i += k
            si += 1
        steps[-1]["end"] = [rid]
        out = helpers.run_steps(eng, steps)
        assert len(out) == len(toks)
        check(out, refs, dtype, f"portions {name}")
    eng.cache.check_invariants()


def mixed_schedule(reqs):
    """Up to four live requests; each alternates portions of its prompt (down to two tokens) and
    single tokens while others do the same; finished requests free pages that later ones reuse.
    Every request runs twice (second time under a new id) so that pages are certainly reused."""
    order = list(reqs)
    jobs = [(rid, reqs[rid]) for rid in order] + [(rid + "2", reqs[rid]) for rid in order]
    sizes = [5, 1, 2, 1, 1, 13, 1, 3, 1, 8, 2, 1, 1, 21]
    live, steps, nxt, tick = {}, [], 0, 0
    while nxt < len(jobs) or live:
        while nxt < len(jobs) and len(live) < 3 + (tick % 2):
            live[jobs[nxt][0]] = [jobs[nxt][1], 0]
            nxt += 1
        entries, end = [], []
        for j, (rid, st) in enumerate(list(live.items())):
            if (tick + j) % 5 == 4 and len(live) > 1:
                continue                                  # sits this step out
            toks, i = st
            k = min(sizes[(tick + 3 * j) % len(sizes)], len(toks) - i)
            want = list(range(k)) if k <= 2 else [0, k - 1]
            entries.append({"id": rid, "tokens": toks[i:i + k], "want": want})
            st[1] = i + k
            if st[1] == len(toks):
                end.append(rid)
                del live[rid]
        steps.append({"entries": entries, "end": end})
        tick += 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_mixed_with_page_reuse(model_dirs, name, dtype):
    cfg = TINY[name]
    reqs = requests_for(cfg, 400)
    refs = {}
    for rid, t in reqs.items():
        refs[rid] = reference(model_dirs[name], dtype, t)
        refs[rid + "2"] = refs[rid]
    # four live requests of at most 97 tokens, each rounded up to 64: 4 * 128 = 512 would always fit;
    # 256 forces pages to be handed out again while other requests are still live.
    eng = make_engine(model_dirs[name], dtype, max_tokens=256)
    steps = mixed_schedule(reqs)
    assert max(len(s["entries"]) for s in steps) >= 3
    out = helpers.run_steps(eng, steps)
    check(out, refs, dtype, f"mixed {name}")
    eng.cache.check_invariants()
    assert eng.cache.n_free_pages(0) == eng.cache.n_blocks
    assert not eng.cache.requests
