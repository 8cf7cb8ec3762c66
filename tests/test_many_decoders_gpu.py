"""Many live requests decoding together: 12, 20, 40, 64 and 70 requests with staggered prompts that
decode side by side for 40 steps and more, twice over in a pool that holds one round only (the
second round lands on the pages the first gave back), a two-token tail portion beside 30 decoding
requests, page sizes 16 and 32; every (request, position) against the plain implementation, in
float32 and in bfloat16, at the two tiny configurations and at the layer sizes of Qwen3-8B.

These are the batch sizes of serving: decode batches above 8 take other product kernels (9 to 16
rows, 17 to 64 rows), other CUDA-graph buckets (16, 32, 64 with padded rows) and, above 64
requests, the eager path.  A spy records which product kernel got how many rows and which graph
buckets were captured.  AxiomOperator/rllm tests the same property on a real model
(crates/rllm-model/tests/common/gpu.rs:42-104) and its server with a pool that forces reuse
(docs/server.md, "Testing").
"""
import pytest
import torch

import helpers
import plain_impl
from helpers import TINY, rel_err
from test_replay_gpu import BIG, STD, TOL, check, make_engine, reference

pytestmark = pytest.mark.gpu

N_SEQS = 70
DECODE_STEPS = 40


def sequences(vocab, seed):
    """70 token sequences: prompts of 2 to 23 tokens (staggered, no two neighbours alike) followed by
    the 41 tokens that the decode steps feed."""
    out = []
    for i in range(N_SEQS):
        prompt = 2 + (i * 7) % 22
        out.append(helpers.random_tokens(prompt + DECODE_STEPS + 1, vocab, seed + i))
    return out


def schedule(seqs, n, ids):
    """Prompts in steps of up to 8 requests (whole prompts side by side), then all n decode together,
    one token each per step; everything ends with the last step."""
    steps = []
    for lo in range(0, n, 8):
        steps.append({"entries": [{"id": ids[i], "tokens": seqs[i][:len(seqs[i]) - DECODE_STEPS - 1],
                                   "want": [len(seqs[i]) - DECODE_STEPS - 2]} for i in range(lo, min(lo + 8, n))]})
    for j in range(DECODE_STEPS + 1):
        steps.append({"entries": [{"id": ids[i], "tokens": [seqs[i][len(seqs[i]) - DECODE_STEPS - 1 + j]], "want": [0]}
                                  for i in range(n)]})
    steps[-1]["end"] = [ids[i] for i in range(n)]
    return steps


class Spy:
    """Records (kernel, rows) of every few-row product the engine launches."""

    def __init__(self):
        from rllm_b200.csrc import ops
        self.ops, self.seen = ops, set()
        self.real = {n: getattr(ops, n) for n in ("gemv_stream", "skinny_gemm_tc", "skinny_gemm", "gemm_lib", "gemm_tc")}

    def __enter__(self):
        for name, fn in self.real.items():
            def wrapped(a, w, out, *args, _fn=fn, _name=name, **kw):
                self.seen.add((_name, a.shape[0]))
                return _fn(a, w, out, *args, **kw)
            setattr(self.ops, name, wrapped)
        return self

    def __exit__(self, *exc):
        for name, fn in self.real.items():
            setattr(self.ops, name, fn)

    def rows(self, name):
        return {m for k, m in self.seen if k == name}


def run_rounds(eng, seqs, n, refs, dtype, what, checker=check):
    """Two rounds of the same n requests under new names, the second in reverse order, on the pages
    the first round gave back."""
    for rnd, order in enumerate((list(range(n)), list(range(n - 1, -1, -1)))):
        ids = {i: f"r{rnd}_{i}" for i in range(n)}
        picked = [seqs[i] for i in order]
        names = [ids[i] for i in order]
        out = helpers.run_steps(eng, schedule(picked, n, names))
        assert len(out) == n * (DECODE_STEPS + 2)
        round_refs = {names[j]: refs[order[j]] for j in range(n)}
        checker(out, round_refs, dtype, f"{what}, {n} decoding, round {rnd}")
        eng.cache.check_invariants()
        assert not eng.cache.requests and eng.cache.n_free_pages(0) == eng.cache.n_blocks


def pool_tokens(seqs, n, block_size):
    """Exactly what one round of n requests holds at its end, in whole pages."""
    return sum(-(-len(s) // block_size) * block_size for s in seqs[:n])


@pytest.fixture(scope="module")
def tiny_refs(tmp_path_factory):
    out = {}
    for i, name in enumerate(("A", "B")):
        for dtype in ("float32", "bfloat16"):
            d = tmp_path_factory.mktemp(f"many_{name}_{dtype}")
            helpers.make_model_dir(d, TINY[name], seed=31 + i, dtype=getattr(torch, dtype), std=STD)
            seqs = sequences(TINY[name]["vocab_size"], 900 + 100 * i)
            out[name, dtype] = (d, seqs, [reference(d, dtype, s) for s in seqs])
    return out


@pytest.mark.parametrize("block_size", [16, 32])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_many_decoders_tiny(tiny_refs, name, dtype, block_size):
    d, seqs, refs = tiny_refs[name, dtype]
    for n in (12, 20, 40, 64, 70):
        eng = make_engine(d, dtype, max_tokens=pool_tokens(seqs, n, block_size), block_size=block_size, max_requests=n)
        run_rounds(eng, seqs, n, refs, dtype, f"tiny {name} pages of {block_size}")
        buckets = {k[0] for k in eng._graphs if k[1] == 0}            # decode shapes (k[1]: a portion's length)
        assert buckets == ({{12: 16, 20: 32, 40: 64, 64: 64}[n]} if n <= 64 else set())
        if n <= 64:
            assert eng.stats["graph_replays"] >= 2 * (DECODE_STEPS - 2)
        else:
            assert eng.stats["graph_replays"] == 0           # above 64 requests the decode step runs eagerly


def tail_schedule(seqs):
    """30 requests decode while request 30 brings its prompt in portions, the later ones of two tokens.
    The two-token portions want their last row only: such steps (one-token items, then one portion) are
    run from the padded layout of a graph (and are captured when their shape has come a few times)."""
    steps = [{"entries": [{"id": i, "tokens": seqs[i][:len(seqs[i]) - DECODE_STEPS - 1], "want": []}
                          for i in range(lo, min(lo + 10, 30))]} for lo in range(0, 30, 10)]
    late = seqs[30]
    cuts = [0, len(late) - 12, len(late) - 10, len(late) - 8, len(late) - 6]      # portion, then 2-token tails
    for j in range(8):
        entries = [{"id": i, "tokens": [seqs[i][len(seqs[i]) - DECODE_STEPS - 1 + j]], "want": [0]} for i in range(30)]
        if j < len(cuts) - 1:
            part = late[cuts[j]:cuts[j + 1]]
            entries.append({"id": 30, "tokens": part, "want": [len(part) - 1]})
        else:
            entries.append({"id": 30, "tokens": [late[cuts[-1] + j - (len(cuts) - 1)]], "want": [0]})
        steps.append({"entries": entries})
    steps[-1]["end"] = list(range(31))
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_two_token_tail_beside_thirty_decoders(tiny_refs, name, dtype):
    d, seqs, refs = tiny_refs[name, dtype]
    eng = make_engine(d, dtype, max_tokens=31 * 96, block_size=16, max_requests=31)
    steps = tail_schedule(seqs)
    assert any(len(e["tokens"]) == 2 for st in steps for e in st["entries"])
    out = helpers.run_steps(eng, steps)
    check(out, {i: refs[i] for i in range(31)}, dtype, f"tiny {name}: 2-token tail beside 30 decoding")
    eng.cache.check_invariants()
    assert eng.cache.n_free_pages(0) == eng.cache.n_blocks
    assert any(k[:2] == (32, 2) for k in eng._graphs)


# ---------------------------------------------------------------- the layer sizes of Qwen3-8B

@pytest.fixture(scope="module")
def big_refs(tmp_path_factory):
    """One layer at the 8B sizes.  bfloat16: all 70 sequences against the plain implementation and its
    storage-rounding twin.  float32: 20 sequences against the plain implementation's float64 twin (sums
    over 12,288 terms: the float32 plain run is itself some 1e-6 away from it)."""
    cfg = BIG["8b"]
    out = {}
    for dtype, count in (("bfloat16", N_SEQS), ("float32", 20)):
        d = tmp_path_factory.mktemp(f"many_8b_{dtype}")
        helpers.make_model_dir(d, cfg, seed=41, dtype=getattr(torch, dtype), std=0.02)
        seqs = sequences(cfg["vocab_size"], 1500)[:count]
        if dtype == "bfloat16":
            pcfg, w = plain_impl.load_model(d, torch.float32)
            refs = [(plain_impl.forward(pcfg, w, s), plain_impl.forward(pcfg, w, s, storage=torch.bfloat16)) for s in seqs]
        else:
            pcfg, w = plain_impl.load_model(d, torch.float32)
            _, w64 = plain_impl.load_model(d, torch.float64)
            refs = [(plain_impl.forward(pcfg, w, s), plain_impl.forward(pcfg, w64, s)) for s in seqs]
        out[dtype] = (d, seqs, refs)
    return out


def check_f64(out, refs, dtype, what):
    floor = max(rel_err(refs[rid][0][pos].double(), refs[rid][1][pos]) for (rid, pos) in out)
    assert floor < 2e-5, f"{what}: the plain implementation itself is {floor:.2e} from its float64 twin"
    for (rid, pos), row in out.items():
        e = rel_err(row.double(), refs[rid][1][pos])
        assert e <= TOL["float32"] + 2 * floor, f"{what}: request {rid} position {pos}: rel err {e:.3e} (floor {floor:.1e})"
        assert int(row.argmax()) == int(refs[rid][1][pos].argmax()), f"{what}: request {rid} position {pos}: argmax differs"


@pytest.mark.parametrize("block_size", [16, 32])
def test_many_decoders_at_8b_layer_sizes_bfloat16(big_refs, block_size):
    d, seqs, refs = big_refs["bfloat16"]
    for n in (12, 20, 40, 64, 70):
        eng = make_engine(d, "bfloat16", max_tokens=pool_tokens(seqs, n, block_size), block_size=block_size, max_requests=n)
        with Spy() as spy:
            run_rounds(eng, seqs, n, refs, "bfloat16", f"8B sizes, pages of {block_size}")
        buckets = {k[0] for k in eng._graphs if k[1] == 0}
        if n == 12:
            # 9 to 16 rows: the streaming kernel for QKV, O and down, the swapped tcgen05 kernel for gate/up and the head
            assert 16 in spy.rows("gemv_stream") and 16 in spy.rows("skinny_gemm_tc") and buckets == {16}
        elif n <= 64:
            bucket = 32 if n == 20 else 64
            assert bucket in spy.rows("skinny_gemm_tc") and bucket not in spy.rows("gemv_stream") and buckets == {bucket}
        else:
            assert not buckets and eng.stats["graph_replays"] == 0
            assert 70 in (spy.rows("gemm_tc") | spy.rows("gemm_lib"))
        from rllm_b200.csrc import ops
        ops.check_device_errors()


def test_many_decoders_at_8b_layer_sizes_float32(big_refs):
    d, seqs, refs = big_refs["float32"]
    for n in (12, 20):
        eng = make_engine(d, "float32", max_tokens=pool_tokens(seqs, n, 32), block_size=32, max_requests=n)
        run_rounds(eng, seqs, n, refs, "float32", "8B sizes float32", checker=check_f64)


def test_two_token_tail_beside_thirty_decoders_at_8b_layer_sizes(big_refs):
    d, seqs, refs = big_refs["bfloat16"]
    for block_size in (16, 32):
        eng = make_engine(d, "bfloat16", max_tokens=31 * 96, block_size=block_size, max_requests=31)
        out = helpers.run_steps(eng, tail_schedule(seqs))
        check(out, {i: refs[i] for i in range(31)}, "bfloat16", f"8B sizes: 2-token tail beside 30 decoding, pages of {block_size}")
        eng.cache.check_invariants()


def portion_schedule(seqs, n_dec, k, late):
    """n_dec requests decode, one token each per step, while the requests `late` bring their prompts one
    after the other in portions of exactly k tokens (the rest in a last, shorter portion): the shape
    (decoders, portion of k) repeats, so that it is captured and replayed."""
    steps = [{"entries": [{"id": i, "tokens": seqs[i][:len(seqs[i]) - DECODE_STEPS - 1], "want": []}
                          for i in range(lo, min(lo + 8, n_dec))]} for lo in range(0, n_dec, 8)]
    j = 0
    for rid in late:
        toks, cut = seqs[rid], 0
        while cut < len(toks):
            part = toks[cut:cut + k]
            entries = [{"id": i, "tokens": [seqs[i][len(seqs[i]) - DECODE_STEPS - 1 + j]], "want": [0]} for i in range(n_dec)]
            entries.append({"id": rid, "tokens": part, "want": [len(part) - 1] if len(part) > 1 else [0]})
            steps.append({"entries": entries})
            cut += len(part)
            j += 1
            assert j <= DECODE_STEPS
    steps[-1]["end"] = list(range(n_dec)) + list(late)
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_beside_decoders_from_graphs(tiny_refs, name, dtype, monkeypatch):
    from rllm_b200.engine import core
    monkeypatch.setattr(core, "GRAPH_MAX_PORTION", 1024)      # the default keeps graphs to portions of up to 8 tokens
    d, seqs, refs = tiny_refs[name, dtype]
    for n_dec, k in ((5, 12), (0, 16), (11, 9), (20, 5)):
        late = [40, 41, 42]
        eng = make_engine(d, dtype, max_tokens=(n_dec + 3) * 96, block_size=16, max_requests=n_dec + 3)
        steps = portion_schedule(seqs, n_dec, k, late)
        out = helpers.run_steps(eng, steps)
        check(out, {i: refs[i] for i in list(range(n_dec)) + late}, dtype,
              f"tiny {name}: portions of {k} beside {n_dec} decoding")
        eng.cache.check_invariants()
        assert eng.cache.n_free_pages(0) == eng.cache.n_blocks
        hit = [key for key, g in eng._graphs.items() if key[1] == k and g.graph is not None]
        assert hit and eng.stats["graph_replays"] >= 3, (sorted(eng._graphs), eng.stats)


def test_portions_beside_decoders_from_graphs_at_8b_layer_sizes(big_refs, monkeypatch):
    from rllm_b200.engine import core
    monkeypatch.setattr(core, "GRAPH_MAX_PORTION", 1024)
    d, seqs, refs = big_refs["bfloat16"]
    for block_size, n_dec, k in ((16, 6, 20), (32, 0, 24)):
        late = [50, 51, 52]
        eng = make_engine(d, "bfloat16", max_tokens=(n_dec + 3) * 96, block_size=block_size, max_requests=n_dec + 3)
        out = helpers.run_steps(eng, portion_schedule(seqs, n_dec, k, late))
        check(out, {i: refs[i] for i in list(range(n_dec)) + late}, "bfloat16",
              f"8B sizes: portions of {k} beside {n_dec} decoding, pages of {block_size}")
        assert [key for key, g in eng._graphs.items() if key[1] == k and g.graph is not None]
        eng.cache.check_invariants()
