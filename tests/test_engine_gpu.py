"""The engine above the kernels: trace replay as a program, generation through the Python entry
point, long decoding, the first tokens of a sequence, preemption, sampling, each part alone, and a
toy architecture with a stateful mixer that is registered here, without touching the package.
"""
import json
import math
import os
import subprocess
import sys
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
import plain_impl
from helpers import TINY, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
STD = 0.08


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        for dtype in ("float32", "bfloat16"):
            d = tmp_path_factory.mktemp(f"m_{name}_{dtype}")
            helpers.make_model_dir(d, cfg, seed=21 + i, dtype=getattr(torch, dtype), std=STD)
            out[name, dtype] = d
    return out


def engine(model_dir, dtype, **kw):
    from rllm_b200.engine import Engine
    from rllm_b200.models.model import load_model
    _, model = load_model(model_dir, dtype, DEV)
    return Engine(model, **kw)


# ---------------------------------------------------------------- bin/trace_run

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dirs, tmp_path, dtype):
    name = "B"
    cfg, w = plain_impl.load_model(dirs[name, dtype])
    a = helpers.random_tokens(40, cfg["vocab_size"], 1)
    b = helpers.random_tokens(23, cfg["vocab_size"], 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[17:19], "want": []},
                                {"id": "b", "tokens": b[:20], "want": [19]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[20:21], "want": [0]}], "end": []},   # a sits out
        {"step": 3, "entries": [{"id": "a", "tokens": a[19:], "want": [20]},
                                {"id": "b", "tokens": b[21:], "want": [0, 1]}], "end": ["a", "b"]},
        {"step": 4, "entries": [{"id": "c", "tokens": a[:5], "want": [4]}], "end": ["c"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(dirs[name, dtype]),
                           "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    la, lb = plain_impl.forward(cfg, w, a), plain_impl.forward(cfg, w, b)
    want = {0: [la[0], la[16]], 1: [lb[19]], 2: [lb[20]], 3: [la[39], lb[21], lb[22]], 4: [la[4]]}
    tol = 5e-6 if dtype == "float32" else 3e-2
    for step, rows in want.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), cfg["vocab_size"])
        for g_, r in zip(got, rows):
            assert rel_err(torch.from_numpy(g_.copy()), r) <= tol


def test_trace_run_rejects_bad_model(tmp_path):
    d = helpers.make_model_dir(tmp_path / "m", TINY["A"], seed=1)
    cfgp = d / "config.json"
    c = json.loads(cfgp.read_text()); c["architectures"] = ["NopeForCausalLM"]; cfgp.write_text(json.dumps(c))
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(d), "--dtype", "float32",
                           "--out", str(tmp_path / "o"), "--max-tokens", "64"], input="", capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode != 0 and "unsupported architecture" in proc.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharded_folder_gives_the_same_logits(tmp_path, dtype):
    """Three shards and a weight map in place of model.safetensors: the same bits out of the engine,
    and a request cannot grow beyond max_position_embeddings."""
    from rllm_b200.cache import RequestTooLong
    from rllm_b200.config import config_from_dict
    from rllm_b200.engine import StepItem
    from rllm_b200.weights import write_random_model
    cfg = config_from_dict(dict(TINY["B"], max_position_embeddings=64))
    one = write_random_model(cfg, tmp_path / "one", seed=3, dtype=getattr(torch, dtype), std=STD)
    three = write_random_model(cfg, tmp_path / "three", seed=3, dtype=getattr(torch, dtype), std=STD, shards=3)
    assert not (three / "model.safetensors").exists()
    toks = helpers.random_tokens(60, TINY["B"]["vocab_size"], 8)
    rows = []
    for d in (one, three):
        eng = engine(d, dtype, max_tokens=128, max_requests=2)
        rows.append(eng.step([StepItem("a", toks, list(range(60)))]).float().cpu())
    assert torch.equal(rows[0], rows[1])
    pcfg, w = plain_impl.load_model(one)
    assert rel_err(rows[1], plain_impl.forward(pcfg, w, toks)) <= (5e-6 if dtype == "float32" else 3e-2)
    eng.step([StepItem("a", [1, 2, 3, 4], [])])                       # 64 tokens: the last position the model has
    for more in ([5], [5, 6, 7]):                                     # the decode path and the portion path
        with pytest.raises(RequestTooLong, match="max_position_embeddings"):
            eng.step([StepItem("a", more, [0])])
    assert eng.cache.length("a") == 64


# ---------------------------------------------------------------- generation through the entry point

@pytest.mark.parametrize("name", ["A", "B", "W", "F"])
def test_greedy_generation_matches_plain(dirs, name):
    from rllm_b200 import LLM
    cfg, w = plain_impl.load_model(dirs[name, "float32"])
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 50 + n) for n in (5, 11, 24, 1)]
    want = [plain_impl.greedy_generate(cfg, w, p, 8) for p in prompts]
    llm = LLM(dirs[name, "float32"], dtype="float32", device=DEV, ctx=128, parallel=3, prefill_chunk=8)
    assert llm.generate(prompts, max_tokens=8) == want
    assert llm.engine.cache.n_free_pages(0) == llm.engine.cache.n_blocks


def test_steps_with_prompt_portions_are_planned_ahead(dirs, monkeypatch):
    """Steps that hold the next portion of a prompt beside decoding requests are launched before the
    tokens of the step before are on the host (the decoding requests' ids come from the device, the
    portion's from the host): they happen, and the tokens are the plain implementation's."""
    from rllm_b200 import LLM
    from rllm_b200.engine import scheduler
    cfg, w = plain_impl.load_model(dirs["B", "float32"])
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 70 + n) for n in (5, 61, 47, 30, 52)]
    want = [plain_impl.greedy_generate(cfg, w, p, 12) for p in prompts]
    mixed = [0]
    real = scheduler.Scheduler.plan_ahead

    def counted(self, plan):
        nxt = real(self, plan)
        if nxt and any(not p.sampled for p in nxt) and any(p.sampled for p in nxt):
            mixed[0] += 1
        return nxt

    monkeypatch.setattr(scheduler.Scheduler, "plan_ahead", counted)
    llm = LLM(dirs["B", "float32"], dtype="float32", device=DEV, ctx=128, parallel=3, prefill_chunk=8)
    assert llm.generate(prompts, max_tokens=12) == want
    assert mixed[0] >= 5
    assert llm.engine.cache.n_free_pages(0) == llm.engine.cache.n_blocks


def test_bfloat16_generation_follows_plain_argmax(dirs):
    """bfloat16 greedy tokens agree with the plain implementation wherever its top two logits are
    further apart than the bfloat16 error bound."""
    from rllm_b200.engine import StepItem
    name = "F"
    cfg, w = plain_impl.load_model(dirs[name, "bfloat16"])
    toks = helpers.random_tokens(60, cfg["vocab_size"], 77)
    ref = plain_impl.forward(cfg, w, toks)
    eng = engine(dirs[name, "bfloat16"], "bfloat16", max_tokens=128)
    got = eng.step([StepItem(0, toks, list(range(60)))]).float().cpu()
    checked = 0
    for p in range(60):
        top = torch.topk(ref[p], 2).values
        if float(top[0] - top[1]) > 2 * 3e-2 * float(ref[p].abs().max()):
            assert int(got[p].argmax()) == int(ref[p].argmax())
            checked += 1
    assert checked >= 20


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "W", "F"])
def test_long_decoding_and_first_tokens(dirs, name, dtype):
    """A one-token prompt, then 330 tokens decoded one by one: crosses many page edges, the decode
    graphs' context paddings (256) and, for W, runs far past the window."""
    from rllm_b200.engine import StepItem
    cfg, w = plain_impl.load_model(dirs[name, dtype])
    toks = helpers.random_tokens(331, cfg["vocab_size"], 5)
    ref = plain_impl.forward(cfg, w, toks)
    eng = engine(dirs[name, dtype], dtype, max_tokens=384, max_requests=2)
    tol = 5e-6 if dtype == "float32" else 3e-2
    worst = 0.0
    for i, t in enumerate(toks):
        row = eng.step([StepItem("r", [t], [0])])[0].float().cpu()
        e = rel_err(row, ref[i])
        worst = max(worst, e)
        assert e <= tol, f"position {i}: {e:.3e}"
    assert eng.stats["graph_replays"] >= 300
    if name == "W":
        assert eng.cache.n_free_pages(1) > eng.cache.n_free_pages(0)     # the window gave pages back
    eng.finish("r")
    eng.cache.check_invariants()


def test_preemption_gives_the_same_tokens(dirs):
    from rllm_b200 import LLM
    cfg, _ = plain_impl.load_model(dirs["B", "float32"])
    prompts = [helpers.random_tokens(30, cfg["vocab_size"], 90 + i) for i in range(4)]
    roomy = LLM(dirs["B", "float32"], dtype="float32", device=DEV, ctx=256, parallel=4, kv_tokens=4096)
    want = roomy.generate(prompts, max_tokens=100)
    assert roomy.last_stats["preemptions"] == 0
    tight = LLM(dirs["B", "float32"], dtype="float32", device=DEV, ctx=256, parallel=4, kv_tokens=320)
    got = tight.generate(prompts, max_tokens=100)
    assert tight.last_stats["preemptions"] >= 1
    assert got == want
    # one limit per prompt: each request stops at its own, with the tokens it had under the common one
    limits = [3, 100, 1, 40]
    assert tight.generate(prompts, max_tokens=limits) == [w[:n] for w, n in zip(want, limits)]
    with pytest.raises(ValueError, match="max_tokens"):
        tight.generate(prompts, max_tokens=[3, 4])


def test_sampling_is_reproducible_whatever_the_batch(dirs):
    from rllm_b200 import LLM
    cfg, w = plain_impl.load_model(dirs["B", "float32"])
    prompts = [helpers.random_tokens(n, cfg["vocab_size"], 30 + n) for n in (1, 9, 40, 63)]
    kw = dict(max_tokens=12, temperature=0.8, top_p=0.95, top_k=50, seed=4)
    together = LLM(dirs["B", "float32"], dtype="float32", device=DEV, ctx=256, parallel=4, prefill_chunk=16,
                   block_size=8).generate(prompts, **kw)
    alone = LLM(dirs["B", "float32"], dtype="float32", device=DEV, ctx=256, parallel=1, block_size=8)
    for i, p in enumerate(prompts):
        assert alone.generate([p], **dict(kw, seed=4 + i))[0] == together[i]
    # and they are the plain sampler's draws from the plain implementation's logits
    seq = list(prompts[1])
    for _ in range(12):
        logits = plain_impl.forward(cfg, w, seq)[-1].numpy()
        seq.append(plain_impl.sample_row(logits, 0.8, 50, 0.95, 4 + 1, len(seq)))
    agree = next((j for j, (a, b) in enumerate(zip(seq[9:], together[1])) if a != b), 12)
    assert agree >= 8                # equal draws; only a rounding-level near tie could end the agreement
    host = LLM(dirs["B", "float32"], dtype="float32", device=DEV, ctx=256, parallel=2, host_sampling=True)
    h1 = host.generate(prompts[:2], **kw)
    assert h1 == host.generate(prompts[:2], **kw) and all(len(t) == 12 for t in h1)


def test_penalties_and_bias_through_generate(dirs):
    """frequency / presence penalties and logit bias reach the sampler through LLM.generate, on the
    device and on the host alike."""
    from rllm_b200 import LLM
    cfg, w = plain_impl.load_model(dirs["A", "float32"])
    prompt = helpers.random_tokens(12, cfg["vocab_size"], 77)
    llm = LLM(dirs["A", "float32"], dtype="float32", device=DEV, ctx=128, parallel=2)
    plain = llm.generate([prompt], max_tokens=24)[0]
    assert plain == plain_impl.greedy_generate(cfg, w, prompt, 24)
    assert len(set(plain)) < len(plain)                      # the tiny model repeats itself
    no_repeat = llm.generate([prompt], max_tokens=24, presence_penalty=1000.0)[0]
    assert len(set(no_repeat)) == len(no_repeat) and no_repeat[0] == plain[0]
    banned = llm.generate([prompt], max_tokens=6, logit_bias={plain[0]: -1000.0})[0]
    assert plain[0] not in banned
    # the plain implementation with the same rule, token by token
    seq, counts = list(prompt), {}
    for _ in range(10):
        row = plain_impl.forward(cfg, w, seq)[-1].numpy()
        adj = [(t, -(c * 0.7 + 0.3)) for t, c in counts.items()]
        tok = plain_impl.sample_row(row, 0, 0, 1.0, 0, 0, adjust=adj)
        counts[tok] = counts.get(tok, 0) + 1
        seq.append(tok)
    kw = dict(max_tokens=10, frequency_penalty=0.7, presence_penalty=0.3)
    assert llm.generate([prompt], **kw)[0] == seq[len(prompt):]
    host = LLM(dirs["A", "float32"], dtype="float32", device=DEV, ctx=128, parallel=2, host_sampling=True)
    assert host.generate([prompt], **kw)[0] == seq[len(prompt):]


def test_python_and_native_host_agree(dirs):
    """The C++ host runtime and the Python one drive the same kernels to the same logits."""
    from rllm_b200.engine import Engine
    from rllm_b200.models.model import load_model
    import test_replay_gpu as T
    _, model = load_model(dirs["W", "float32"], "float32", DEV)
    reqs = T.requests_for(TINY["W"], 500)
    steps = T.mixed_schedule(reqs)
    outs = []
    for native in (True, False):
        eng = Engine(model, block_size=16, max_tokens=256, max_requests=8, native_host=native)
        outs.append(helpers.run_steps(eng, steps))
        eng.cache.check_invariants()
        assert not eng.cache.requests
    assert set(outs[0]) == set(outs[1])
    for k in outs[0]:
        assert torch.equal(outs[0][k], outs[1][k])


def test_step_errors_change_nothing(dirs):
    from rllm_b200.cache import OutOfPages
    from rllm_b200.engine import StepError, StepItem
    eng = engine(dirs["A", "float32"], "float32", max_tokens=32, max_requests=2)
    eng.step([StepItem("a", [1, 2, 3], [2])])
    free = eng.cache.n_free_pages(0)
    for bad in ([StepItem("a", [], [])], [StepItem("a", [999], [0])], [StepItem("a", [1], [1])],
                [StepItem("a", [1], []), StepItem("a", [2], [])], []):
        with pytest.raises(StepError):
            eng.step(bad)
    with pytest.raises(OutOfPages):
        eng.step([StepItem("a", [1], [0]), StepItem("b", list(range(40)), [])])
    assert eng.cache.n_free_pages(0) == free and eng.cache.length("a") == 3 and not eng.cache.has("b")
    with pytest.raises(Exception, match="CUDA device only"):
        from rllm_b200.csrc import ops
        ops.silu_mul(torch.zeros(1, 4), torch.zeros(1, 2))


# ---------------------------------------------------------------- each part alone

def rt(dtype=torch.float32):
    from rllm_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype)


def test_part_norm_and_rotary_alone():
    from rllm_b200.config import PartSpec
    from rllm_b200.parts import build_part
    norm = build_part("norm", PartSpec("rms_norm", {"size": 200, "eps": 1e-5}, "n."), rt())
    w = 1 + 0.1 * torch.randn(200)
    norm.load({"n.weight": w})
    assert list(norm.expected_tensors()) == ["n.weight"]
    x, d = torch.randn(9, 200), torch.randn(9, 200)
    xd = x.to(DEV)
    out = norm.forward(xd, d.to(DEV))
    assert rel_err(out.cpu(), plain_impl.rms_norm(x + d, w, 1e-5)) < 1e-5 and torch.equal(xd.cpu(), x + d)
    rot = build_part("position", PartSpec("rotary_neox", {"head_dim": 48, "theta": 50000.0}), rt())
    inv = 1.0 / torch.pow(torch.tensor(50000.0), torch.arange(0, 48, 2).float() / 48)
    assert torch.equal(rot.table().cpu(), inv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_part_ffn_and_head_alone(dtype):
    from rllm_b200.config import PartSpec
    from rllm_b200.parts import build_part
    d, F, V = 96, 224, 311
    ffn = build_part("ffn", PartSpec("swiglu", {"hidden_size": d, "intermediate_size": F}, "m."), rt(dtype))
    g = torch.Generator().manual_seed(3)
    ws = {"m.gate_proj.weight": torch.randn(F, d, generator=g) * 0.1, "m.up_proj.weight": torch.randn(F, d, generator=g) * 0.1,
          "m.down_proj.weight": torch.randn(d, F, generator=g) * 0.1}
    ws = {k: v.to(dtype) for k, v in ws.items()}
    ffn.load(ws)
    for n in (3, 70):                                   # the few-rows kernel and the library product
        h = torch.randn(n, d, generator=g).to(dtype)
        ref = plain_impl.swiglu(h.float(), *(ws[f"m.{p}_proj.weight"].float() for p in ("gate", "up", "down")),
                                storage=None if dtype == torch.float32 else dtype)
        out = ffn.forward(h.to(DEV))
        assert out.dtype == torch.float32 and rel_err(out.cpu(), ref) < (2e-6 if dtype == torch.float32 else 5e-3)
        res = torch.ones(n, d, device=DEV)
        assert ffn.forward(h.to(DEV), residual=res) is None
        assert rel_err(res.cpu(), ref + 1) < (2e-6 if dtype == torch.float32 else 5e-3)
    emb = build_part("embedding", PartSpec("embedding", {"vocab_size": V, "hidden_size": d}, "e."), rt(dtype))
    table = (torch.randn(V, d, generator=g) * 0.1).to(dtype)
    emb.load({"e.weight": table})
    toks = torch.tensor([0, 310, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(toks).cpu(), table.float()[[0, 310, 17]])
    head = build_part("lm_head", PartSpec("lm_head", {"vocab_size": V, "hidden_size": d, "tied_to": "e.weight"}, "h."), rt(dtype))
    assert head.expected_tensors() == {}
    head.load({}, shared={"e.weight": emb.weight})
    h = torch.randn(4, d, generator=g).to(dtype)
    assert rel_err(head.forward(h.to(DEV)).cpu(), h.float() @ table.float().t()) < (2e-6 if dtype == torch.float32 else 1e-5)


@pytest.mark.parametrize("dtype,hd,H,K,window", [(torch.float32, 32, 6, 2, 0), (torch.bfloat16, 64, 4, 2, 0),
                                                  (torch.float32, 16, 4, 4, 9), (torch.bfloat16, 128, 4, 1, 21)])
def test_part_attention_alone(dtype, hd, H, K, window):
    """The attention part with its own cache pages, fed in two portions and one decoded token,
    against the plain attention block over the whole sequence."""
    from rllm_b200.cache import CacheManager, PagedKVView
    from rllm_b200.config import PartSpec
    from rllm_b200.engine.batch import StepContext
    from rllm_b200.parts import build_part
    d, eps, theta, bs, n = 80, 1e-5, 30000.0, 8, 45
    att = build_part("mixer", PartSpec("attention", {"hidden_size": d, "num_heads": H, "num_kv_heads": K,
                     "head_dim": hd, "qk_norm": True, "qk_norm_eps": eps, "window": window, "scale": hd ** -0.5}, "a."), rt(dtype))
    rot = build_part("position", PartSpec("rotary_neox", {"head_dim": hd, "theta": theta}), rt(dtype))
    g = torch.Generator().manual_seed(11)
    ws = {n_: ((torch.randn(s, generator=g) * 0.15) if r != "norm" else 1 + 0.1 * torch.randn(s, generator=g)).to(dtype)
          for n_, (s, r) in att.expected_tensors().items()}
    att.load(ws)
    h = torch.randn(n, d, generator=g).to(dtype)
    cfg = dict(num_attention_heads=H, num_key_value_heads=K, head_dim=hd, hidden_size=d, rms_norm_eps=eps, rope_theta=theta)
    pw = {"x.self_attn." + k[2:]: v.float() for k, v in ws.items()}
    ref = plain_impl.attention_block(h.float(), list(range(n)), pw, "x.", cfg, window,
                                     storage=None if dtype == torch.float32 else dtype)
    cm = CacheManager([att.cache_need()], [None], bs, 64, 1)
    cm.allocate_device(torch.device(DEV), dtype)
    outs, start = [], 0
    for k in (30, 14, 1):
        slots = cm.append("r", k)[0]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        ctx = StepContext(n_tokens=k, n_requests=1, tokens=i32([0] * k), positions=i32(list(range(start, start + k))),
                          seq_ids=i32([0] * k), cu_q=i32([0, k]), ctx_lens=i32([start + k]), logit_rows=None,
                          q_lens=[k], start_pos=[start], ctx_lens_host=[start + k], max_q_len=k, max_ctx_len=start + k)
        pool = cm.paged[0].pool
        view = PagedKVView(pool[0, 0], pool[0, 1], i32([cm.block_table("r", 0)]), i32(slots), bs)
        outs.append(att.forward(h[start:start + k].to(DEV), ctx, view, rot).cpu())
        cm.release_passed("r")
        start += k
    got = torch.cat(outs)
    assert rel_err(got, ref) < (5e-6 if dtype == torch.float32 else 1.5e-2)


# ---------------------------------------------------------------- a toy architecture, defined here

def test_toy_stateful_mixer_registers_and_steps(tmp_path):
    """A mixer with a fixed-size state of its own (a decaying running sum of a projection), a toy
    architecture using it in every other layer beside attention layers that share one cache, and
    a layer that runs twice: all registered from this test, built and stepped by the package
    without any change to its files; checked against a whole-sequence computation."""
    from rllm_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, load_config,
                                  register_architecture)
    from rllm_b200.engine import Engine, StepItem
    from rllm_b200.models.model import load_model
    from rllm_b200.parts import Mixer, StateNeed, register_part
    from rllm_b200.weights import write_safetensors

    @register_part("mixer", "toy_decay_sum")
    class ToyDecaySum(Mixer):
        """state_t = decay * state_{t-1} + W_in x_t;  y_t = W_out state_t   (plain torch: a toy)."""

        def __init__(self, params, prefix, runtime):
            super().__init__(params, prefix, runtime)
            self.d, self.s, self.decay = params["hidden_size"], params["state_size"], params["decay"]

        def cache_need(self):
            return StateNeed((self.s,), torch.float32)

        def expected_tensors(self):
            return {self.prefix + "in.weight": ((self.s, self.d), "matrix"),
                    self.prefix + "out.weight": ((self.d, self.s), "matrix")}

        def load(self, tensors):
            self.w_in = self._to_device(tensors[self.prefix + "in.weight"], torch.float32)
            self.w_out = self._to_device(tensors[self.prefix + "out.weight"], torch.float32)

        def forward(self, h, ctx, cache, position, residual=None):
            u = h.float() @ self.w_in.t()
            out = torch.empty(h.shape[0], self.d, device=h.device)
            for r in range(ctx.n_requests):
                slot = int(cache.slots[r])
                lo = sum(ctx.q_lens[:r])
                st = cache.state[slot].clone()
                for t in range(lo, lo + ctx.q_lens[r]):
                    st = self.decay * st + u[t]
                    out[t] = self.w_out @ st
                cache.state[slot] = st
            return out

    @register_part("mixer", "toy_decay_sum_on_device")
    class ToyDecaySumOnDevice(ToyDecaySum):
        """The same mixer written so that a step may be captured into a CUDA graph and replayed: device
        operations only, the state slots taken from the device array, from the host no more than the
        step's shape (the number of requests and of tokens of each)."""
        CAPTURE_SAFE = True

        def forward(self, h, ctx, cache, position, residual=None):
            u = h.float() @ self.w_in.t()
            out = torch.empty(h.shape[0], self.d, device=h.device)
            lo = 0
            for r in range(ctx.n_requests):
                slot = cache.slots[r:r + 1].long()                   # stays on the device
                st = cache.state.index_select(0, slot)[0]
                for t in range(lo, lo + ctx.q_lens[r]):
                    st = self.decay * st + u[t]
                    out[t] = self.w_out @ st
                cache.state.index_copy_(0, slot, st[None])
                lo += ctx.q_lens[r]
            return out

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden: int
        vocab: int
        state: int
        decay: float
        mixer_kind: str = "toy_decay_sum"
        architecture: str = "ToyForCausalLM"

        @classmethod
        def from_dict(cls, d):
            return cls(d["hidden"], d["vocab"], d["state"], d["decay"], d.get("mixer_kind", "toy_decay_sum"))

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden=self.hidden, vocab=self.vocab,
                        state=self.state, decay=self.decay, mixer_kind=self.mixer_kind)

        def model_spec(self):
            norm = lambda p: PartSpec("rms_norm", {"size": self.hidden, "eps": 1e-6}, p)
            ffn = lambda p: PartSpec("swiglu", {"hidden_size": self.hidden, "intermediate_size": 2 * self.hidden}, p)
            attn = lambda p: PartSpec("attention", {"hidden_size": self.hidden, "num_heads": 2, "num_kv_heads": 1,
                                                    "head_dim": 16, "qk_norm": False, "window": 0, "scale": 0.25}, p)
            toy = lambda p: PartSpec(self.mixer_kind, {"hidden_size": self.hidden, "state_size": self.state,
                                                       "decay": self.decay}, p)
            layers = []
            for i, mixer in enumerate([attn, toy, attn]):
                p = f"l.{i}."
                layers.append(LayerSpec("pre_norm", mixer(p + "mix."), ffn(p + "mlp."),
                                        {"mixer": norm(p + "n1."), "ffn": norm(p + "n2.")},
                                        PartSpec("rotary_neox", {"head_dim": 16, "theta": 1e4}) if mixer is attn else None))
            # layer 1 (the stateful one) runs twice; entry 3 (layer 2) reads the cache entry 0 wrote
            order = (RunEntry(0), RunEntry(1), RunEntry(1), RunEntry(2, cache_of=0))
            return ModelSpec(self.vocab, self.hidden, PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.hidden}, "emb."),
                             tuple(layers), order, norm("fn."),
                             PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.hidden, "tied_to": "emb.weight"}, "head."),
                             512)

    register_architecture("ToyForCausalLM", ToyConfig)
    cfg = ToyConfig(hidden=32, vocab=50, state=6, decay=0.9)
    d = tmp_path / "toy"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg.to_dict()))
    from rllm_b200.models.model import expected_tensors
    g = torch.Generator().manual_seed(2)
    tensors = {n: (1 + 0.1 * torch.randn(s, generator=g)) if r == "norm" else 0.2 * torch.randn(s, generator=g)
               for n, (s, r) in expected_tensors(cfg.model_spec()).items()}
    write_safetensors(d / "model.safetensors", tensors)
    assert isinstance(load_config(d), ToyConfig)

    _, model = load_model(d, "float32", DEV)
    needs, cache_of = model.cache_needs()
    assert cache_of == [None, None, None, 0] and isinstance(needs[1], StateNeed)
    toks = {"a": helpers.random_tokens(21, 50, 1), "b": helpers.random_tokens(9, 50, 2)}

    def run(schedule):
        eng = Engine(model, block_size=4, max_tokens=64, max_requests=2)
        assert len(eng.cache.paged) == 1 and len(eng.cache.paged[0].entries) == 1     # one shared plane
        assert eng.cache.stateful[0].state.shape == (2, 3, 6)                          # two entries, two slots and the one for padding rows
        return helpers.run_steps(eng, schedule)

    whole = run([{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]} for r, t in toks.items()])
    a, b = toks["a"], toks["b"]
    cut = run([
        {"entries": [{"id": "a", "tokens": a[:7], "want": list(range(7))}]},
        {"entries": [{"id": "a", "tokens": a[7:9], "want": [0, 1]}, {"id": "b", "tokens": b[:8], "want": list(range(8))}]},
        {"entries": [{"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]},
        {"entries": [{"id": "a", "tokens": a[9:20], "want": list(range(11))}]},
        {"entries": [{"id": "a", "tokens": a[20:], "want": [0]}], "end": ["a"]},
    ])
    assert set(whole) == set(cut)
    for key in whole:
        assert rel_err(cut[key], whole[key]) < 1e-5
    # and the state really matters: a request that starts in a used slot starts from zero
    eng = Engine(model, block_size=4, max_tokens=64, max_requests=1)
    first = helpers.run_steps(eng, [{"entries": [{"id": "x", "tokens": a, "want": [20]}], "end": ["x"]}])
    again = helpers.run_steps(eng, [{"entries": [{"id": "y", "tokens": a, "want": [20]}], "end": ["y"]}])
    assert rel_err(again["y", 20], first["x", 20]) < 1e-6
    assert not eng.use_graphs                       # the toy reads its slots back to the host: never captured

    # The same mixer written with device operations only declares itself safe to capture: the model's
    # decode steps are then replayed from CUDA graphs although it holds state (three requests padded to
    # four: the padding row reads and writes the state slot that belongs to nobody), with the results of
    # the eager toy.
    d2 = tmp_path / "toy_on_device"
    d2.mkdir()
    (d2 / "config.json").write_text(json.dumps(dict(cfg.to_dict(), mixer_kind="toy_decay_sum_on_device")))
    write_safetensors(d2 / "model.safetensors", tensors)
    _, model2 = load_model(d2, "float32", DEV)
    assert model2.capture_safe and not model.capture_safe
    toks["c"] = helpers.random_tokens(15, 50, 3)
    whole3 = helpers.run_steps(Engine(model, block_size=4, max_tokens=64, max_requests=3),
                               [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]}
                                for r, t in toks.items()])
    eng2 = Engine(model2, block_size=4, max_tokens=64, max_requests=3)
    steps = [{"entries": [{"id": r, "tokens": t[:3], "want": [0, 1, 2]} for r, t in toks.items()]}]
    for j in range(3, 9):
        steps.append({"entries": [{"id": r, "tokens": [t[j]], "want": [0]} for r, t in toks.items()]})
    steps[-1]["end"] = list(toks)
    got = helpers.run_steps(eng2, steps)
    assert eng2.use_graphs and eng2.stats["graph_replays"] >= 4
    for key, row in got.items():
        assert rel_err(row, whole3[key]) < 1e-5, key
    # and a request that then takes a slot starts from zero: nothing of the padding row's state leaks
    after = helpers.run_steps(eng2, [{"entries": [{"id": "z", "tokens": a, "want": [20]}], "end": ["z"]}])
    assert rel_err(after["z", 20], first["x", 20]) < 1e-5


def test_toy_routed_ffn_and_other_position_encoding(tmp_path):
    """A feed-forward that routes every token to one of several experts, and two position encodings
    other than the model family's (rotary with interpolated positions through the table interface,
    and a partial rotation that does its own step), all defined here:
    registered, chosen by a configuration layer by layer beside the framework's own parts, built,
    loaded from a model folder and stepped, with no change to the framework's files.  Never a
    model of anyone's: two layers of toys.  (Toys have no plain implementation under tests/: the engine
    cut into portions and mixed with another request is compared with the engine on whole prompts,
    and each toy part is shown to matter by replacing it.)"""
    from rllm_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, load_config,
                                  register_architecture)
    from rllm_b200.engine import Engine
    from rllm_b200.models.model import expected_tensors, load_model
    from rllm_b200.parts import FeedForward, Part, register_part
    from rllm_b200.weights import write_safetensors

    chosen = []

    @register_part("ffn", "toy_top1_experts")
    class ToyTop1Experts(FeedForward):
        """out_t = W2[e_t] relu(W1[e_t] x_t) with e_t = argmax(router x_t); router logits in float32."""

        def __init__(self, params, prefix, runtime):
            super().__init__(params, prefix, runtime)
            self.d, self.f, self.e = params["hidden_size"], params["expert_size"], params["num_experts"]

        def expected_tensors(self):
            return {self.prefix + "router.weight": ((self.e, self.d), "matrix"),
                    self.prefix + "w1": ((self.e, self.f, self.d), "matrix"),
                    self.prefix + "w2": ((self.e, self.d, self.f), "matrix")}

        def load(self, tensors):
            self.router = self._to_device(tensors[self.prefix + "router.weight"], torch.float32)
            self.w1 = self._to_device(tensors[self.prefix + "w1"], torch.float32)
            self.w2 = self._to_device(tensors[self.prefix + "w2"], torch.float32)

        def forward(self, h, ctx=None, residual=None):
            x = h.float()
            e = (x @ self.router.t()).argmax(-1)
            chosen.extend(e.tolist())
            hid = torch.relu(torch.einsum("tfd,td->tf", self.w1[e], x))
            out = torch.einsum("tdf,tf->td", self.w2[e], hid)
            if residual is not None:
                residual += out
                return None
            return out

    @register_part("position", "toy_rotary_interpolated")
    class ToyRotaryInterpolated(Part):
        """Rotate-half rotary with positions divided by `factor`: the same table interface as the
        family's own rotary part (a float32 inv_freq vector), so the attention kernel takes it as is."""

        def __init__(self, params, prefix, runtime):
            super().__init__(params, prefix, runtime)
            hd, theta, factor = params["head_dim"], params["theta"], params["factor"]
            i = torch.arange(0, hd, 2, dtype=torch.float32)
            self.inv_freq = (1.0 / torch.pow(torch.tensor(float(theta)), i / hd) / factor).to(runtime.device)

        def table(self):
            return self.inv_freq

    @register_part("position", "toy_partial_rotary")
    class ToyPartialRotary(Part):
        """Rotates only the first `rot` dims of a head, in pairs (i, i + rot/2), and leaves the rest: not
        a table the fused kernel could take, so the part does the whole step itself (`apply_and_store`):
        q/k norm and rotation with torch operations, then the package's kernel, without a table, to
        write the queries out and the keys and values into the pages."""

        def __init__(self, params, prefix, runtime):
            super().__init__(params, prefix, runtime)
            self.rot = params["rot"]
            i = torch.arange(0, self.rot, 2, dtype=torch.float32)
            self.inv_freq = (1.0 / torch.pow(torch.tensor(float(params["theta"])), i / self.rot)).to(runtime.device)

        def apply_and_store(self, qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim):
            from rllm_b200.csrc import ops
            positions = ctx.positions
            n, half = qkv.shape[0], self.rot // 2
            x = qkv.float().view(n, H + 2 * K, head_dim).clone()
            if q_norm_w is not None:
                for lo, hi, w in ((0, H, q_norm_w), (H, H + K, k_norm_w)):
                    t = x[:, lo:hi]
                    x[:, lo:hi] = t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w
            ang = positions.float()[:, None] * self.inv_freq[None, :]
            c, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
            a, b = x[:, :H + K, :half].clone(), x[:, :H + K, half:self.rot].clone()
            x[:, :H + K, :half] = a * c - b * sn
            x[:, :H + K, half:self.rot] = a * sn + b * c
            ops.qk_norm_rope_store(x.view(n, -1), None, None, None, positions, cache.slots, q_out, cache.k, cache.v,
                                   H, K, head_dim, cache.block_size, eps, write_kv=cache.write)

    @dataclass(frozen=True)
    class Toy2Config(ModelConfig):
        hidden: int
        vocab: int
        experts: int
        factor: float
        rot: int = 8
        architecture: str = "Toy2ForCausalLM"

        @classmethod
        def from_dict(cls, d):
            return cls(d["hidden"], d["vocab"], d["experts"], d["factor"], d.get("rot", 8))

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden=self.hidden, vocab=self.vocab,
                        experts=self.experts, factor=self.factor, rot=self.rot)

        def model_spec(self):
            norm = lambda p: PartSpec("rms_norm", {"size": self.hidden, "eps": 1e-5}, p)
            attn = lambda p: PartSpec("attention", {"hidden_size": self.hidden, "num_heads": 3, "num_kv_heads": 3,
                                                    "head_dim": 16, "qk_norm": True, "qk_norm_eps": 1e-5, "window": 0,
                                                    "scale": 0.25}, p)
            routed = lambda p: PartSpec("toy_top1_experts", {"hidden_size": self.hidden, "expert_size": 24,
                                                             "num_experts": self.experts}, p)
            dense = lambda p: PartSpec("swiglu", {"hidden_size": self.hidden, "intermediate_size": 40}, p)
            pos = [PartSpec("toy_rotary_interpolated", {"head_dim": 16, "theta": 1e4, "factor": self.factor}),
                   PartSpec("toy_partial_rotary", {"rot": self.rot, "theta": 1e4}) if self.rot < 16 else
                   PartSpec("rotary_neox", {"head_dim": 16, "theta": 1e4})]
            layers = tuple(LayerSpec("pre_norm", attn(f"l.{i}.mix."), (routed if i == 0 else dense)(f"l.{i}.mlp."),
                                     {"mixer": norm(f"l.{i}.n1."), "ffn": norm(f"l.{i}.n2.")}, pos[i]) for i in range(2))
            return ModelSpec(self.vocab, self.hidden,
                             PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.hidden}, "emb."),
                             layers, (RunEntry(0), RunEntry(1)), norm("fn."),
                             PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.hidden, "tied_to": None}, "head."),
                             256)

    register_architecture("Toy2ForCausalLM", Toy2Config)

    def build(factor, sub, rot=8):
        cfg = Toy2Config(hidden=48, vocab=61, experts=4, factor=factor, rot=rot)
        d = tmp_path / sub
        d.mkdir()
        (d / "config.json").write_text(json.dumps(cfg.to_dict()))
        g = torch.Generator().manual_seed(5)
        tensors = {n: (1 + 0.1 * torch.randn(s, generator=g)) if r == "norm" else 0.3 * torch.randn(s, generator=g)
                   for n, (s, r) in expected_tensors(cfg.model_spec()).items()}
        write_safetensors(d / "model.safetensors", tensors)
        assert isinstance(load_config(d), Toy2Config)
        return load_model(d, "float32", DEV)[1]

    model = build(4.0, "toy2")
    a, b = helpers.random_tokens(37, 61, 3), helpers.random_tokens(12, 61, 4)
    whole = helpers.run_steps(Engine(model, block_size=8, max_tokens=64, max_requests=2),
                              [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))}], "end": [r]}
                               for r, t in (("a", a), ("b", b))])
    assert len(set(chosen)) > 1                     # the router sends tokens to different experts
    cut = helpers.run_steps(Engine(model, block_size=8, max_tokens=64, max_requests=2), [
        {"entries": [{"id": "a", "tokens": a[:9], "want": list(range(9))}]},
        {"entries": [{"id": "a", "tokens": a[9:11], "want": [0, 1]}, {"id": "b", "tokens": b[:5], "want": list(range(5))}]},
        {"entries": [{"id": "a", "tokens": [a[11]], "want": [0]}, {"id": "b", "tokens": b[5:], "want": list(range(7))}], "end": ["b"]},
        {"entries": [{"id": "a", "tokens": a[12:], "want": list(range(25))}], "end": ["a"]},
    ])
    assert set(whole) == set(cut)
    for key in whole:
        assert rel_err(cut[key], whole[key]) < 1e-5
    # the position encoding is really the toy's: factor 1 gives other logits from the second token on
    # (at position 0 every rotation is the identity), the same weights otherwise
    plain_pos = helpers.run_steps(Engine(build(1.0, "toy2_f1"), block_size=8, max_tokens=64, max_requests=1),
                                  [{"entries": [{"id": "a", "tokens": a, "want": [0, 20, 36]}], "end": ["a"]}])
    assert rel_err(plain_pos["a", 0], whole["a", 0]) < 1e-6
    assert rel_err(plain_pos["a", 20], whole["a", 20]) > 1e-3 and rel_err(plain_pos["a", 36], whole["a", 36]) > 1e-3
    # and so is the second layer's (the part that does its own step): with all 16 dims rotated by the family's
    # part the logits differ again; rotating all 16 dims through the toy (rot = 16 is not offered) is not needed
    full_rot = helpers.run_steps(Engine(build(4.0, "toy2_rot16", rot=16), block_size=8, max_tokens=64, max_requests=1),
                                 [{"entries": [{"id": "a", "tokens": a, "want": [0, 20, 36]}], "end": ["a"]}])
    assert rel_err(full_rot["a", 0], whole["a", 0]) < 1e-6
    assert rel_err(full_rot["a", 20], whole["a", 20]) > 1e-3


# ---------------------------------------------------------------- the command line

def _cli(*args, timeout=600):
    return subprocess.run([sys.executable, str(ROOT / "bin" / "rllm"), *map(str, args)], capture_output=True, text=True,
                          timeout=timeout)


def test_command_line(dirs, tmp_path):
    cfg, w = plain_impl.load_model(dirs["A", "float32"])
    prompt = helpers.random_tokens(9, cfg["vocab_size"], 8)
    want = plain_impl.greedy_generate(cfg, w, prompt, 6)
    r = _cli("run", dirs["A", "float32"], ",".join(map(str, prompt)), "-n", 6, "--kv-type", "f32", "--ctx", 64, "--show-ids")
    assert r.returncode == 0, r.stderr[-1500:]
    assert [int(t) for t in r.stdout.split()] == want and "tok/s" in r.stderr
    ids = tmp_path / "ids.txt"
    ids.write_text(" ".join(map(str, prompt)))
    r = _cli("run", dirs["A", "float32"], f"@{ids}", "-n", 6, "--kv-type", "f32", "--ctx", 64, "-t", 0.7, "--top-p", 0.9,
             "--top-k", 20, "--seed", 3)
    assert r.returncode == 0 and len(r.stdout.split()) == 6
    r = _cli("run", dirs["A", "float32"], "1,2,3", "-n", 100, "--ctx", 64)
    assert r.returncode == 2 and "exceed --ctx" in r.stderr
    r = _cli("bench", dirs["B", "bfloat16"], "-p", 40, "-n", 8, "-r", 1, "-b", 2, "--depth", 16)
    assert r.returncode == 0, r.stderr[-1500:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["pp_tok_s"] > 0 and res["tg_tok_s"] > 0 and res["batch"] == 2
    r = _cli("compare", dirs["B", "bfloat16"], ",".join(map(str, prompt)), "-n", 4)
    assert r.returncode == 0 and "max relative logit diff" in r.stdout
    assert float(r.stdout.split("diff")[1].split(";")[0]) < 3e-2
    # compare-ref: a dump of the plain implementation's logits in the reference's format
    from rllm_b200.cli import write_ref_dump
    cfgB, wB = plain_impl.load_model(dirs["B", "float32"])
    toks = helpers.random_tokens(23, cfgB["vocab_size"], 12)
    dump = tmp_path / "ref.bin"
    write_ref_dump(dump, 15, toks, plain_impl.forward(cfgB, wB, toks).numpy())
    r = _cli("compare-ref", dirs["B", "float32"], dump, "--kv-type", "f32", "--prefill-chunk", 7)
    assert r.returncode == 0, r.stderr[-1500:]
    assert "top-1 agreement 23/23" in r.stdout and float(r.stdout.split("worst relative logit diff")[1]) < 5e-6
    (tmp_path / "bad.bin").write_bytes(b"RLLMREF1" + b"\0" * 11)
    assert _cli("compare-ref", dirs["B", "float32"], tmp_path / "bad.bin").returncode != 0
    # perplexity over token ids, against the plain implementation's own log-likelihoods
    stream = helpers.random_tokens(100, cfgB["vocab_size"], 13)
    (tmp_path / "stream.txt").write_text(" ".join(map(str, stream)))
    r = _cli("perplexity", dirs["B", "float32"], tmp_path / "stream.txt", "--ctx", 32, "--kv-type", "f32")
    assert r.returncode == 0, r.stderr[-1500:]
    nll = []
    for c in range(3):
        chunk = stream[32 * c:32 * c + 32]
        lp = torch.log_softmax(plain_impl.forward(cfgB, wB, chunk).double(), dim=1)
        nll += [-float(lp[i, chunk[i + 1]]) for i in range(16, 31)]
    want_ppl = math.exp(sum(nll) / len(nll))
    got_ppl = float(r.stdout.split("PPL =")[1].split("+/-")[0])
    assert abs(got_ppl - want_ppl) / want_ppl < 1e-4 and "45 scored tokens" in r.stdout
    r = _cli("inspect", dirs["B", "bfloat16"])
    assert r.returncode == 0 and "model.layers.2.mlp.down_proj.weight" in r.stdout and "Qwen3Config" in r.stdout
    cfgfile = tmp_path / "c.json"
    cfgfile.write_text(json.dumps(TINY["F"]))
    r = _cli("random-model", tmp_path / "rm", "--config", cfgfile, "--seed", 5)
    assert r.returncode == 0 and (tmp_path / "rm" / "model.safetensors").exists()


def test_profile_switch_times_every_launcher(dirs):
    """RLLM_B200_PROFILE=1: event pairs around the launchers, a table at exit, graphs off."""
    env = dict(os.environ, RLLM_B200_PROFILE="1")
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "rllm"), "run", str(dirs["B", "bfloat16"]), "1,2,3,4,5", "-n", "6",
                        "--ctx", "64", "--show-ids"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-1500:]
    lines = [l for l in r.stderr.splitlines() if l.startswith("[rllm_b200 profile]")]
    names = {l.split()[2] for l in lines[1:-1]}
    assert {"rllm_embed", "rllm_add_rms_norm", "rllm_qk_norm_rope_store", "rllm_sample_rows"} <= names, r.stderr[-1500:]
    assert "graphs off" in lines[-1]
    plain = _cli("run", dirs["B", "bfloat16"], "1,2,3,4,5", "-n", 6, "--ctx", 64, "--show-ids")
    assert plain.stdout.split() == r.stdout.split()          # the switch changes no token


def test_graph_cache_is_bounded(dirs, monkeypatch):
    """Captured decode shapes are kept up to a bound; the least recently used one goes, and a shape
    that comes back is captured again with the same results."""
    from rllm_b200.engine import StepItem
    from rllm_b200.engine import core
    monkeypatch.setattr(core, "GRAPH_CACHE_MAX", 2)
    monkeypatch.setattr(core, "GRAPH_CTX_QUANTUM", 16)
    cfg, w = plain_impl.load_model(dirs["A", "float32"])
    toks = helpers.random_tokens(70, cfg["vocab_size"], 21)
    ref = plain_impl.forward(cfg, w, toks)
    eng = engine(dirs["A", "float32"], "float32", max_tokens=128, max_requests=2)
    for i, t in enumerate(toks):                      # context buckets of 16: five shapes in turn
        row = eng.step([StepItem("r", [t], [0])])[0].float().cpu()
        assert rel_err(row, ref[i]) <= 5e-6
        assert len(eng._graphs) <= 2
    assert eng.stats["graphs_captured"] >= 4
    eng.finish("r")


def test_a_kernel_that_gave_up_a_wait_fails_the_generation(dirs):
    """The error word that kernels with bounded waits write is read by the entry point: a code in
    it (set here by hand; no kernel is made to wait) raises, and the word is cleared."""
    from rllm_b200 import LLM
    from rllm_b200.csrc import ops
    llm = LLM(dirs["A", "bfloat16"], dtype="bfloat16", device=DEV, ctx=64, parallel=1)
    assert len(llm.generate([[1, 2, 3]], max_tokens=3)[0]) == 3
    ops.error_word(DEV).fill_(2)
    from rllm_b200.llm import GenerationError
    with pytest.raises(GenerationError, match="bounded wait"):
        llm.generate([[1, 2, 3]], max_tokens=3)
    assert len(llm.generate([[1, 2, 3]], max_tokens=3)[0]) == 3          # cleared: the next call is clean
    # the word is also read every 64 steps: the requests running then fail, nothing stays in the cache,
    # and the next call (whose requests are numbered from 0 again) gives what a fresh engine gives
    llm = LLM(dirs["A", "bfloat16"], dtype="bfloat16", device=DEV, ctx=256, parallel=1)
    want = llm.generate([[4, 5, 6, 7]], max_tokens=100)[0]
    assert len(want) == 100
    ops.error_word(DEV).fill_(1)
    with pytest.raises(GenerationError, match="bounded wait") as ei:
        llm.generate([[9, 8, 7]], max_tokens=100)
    assert ei.value.errors.keys() == {0}
    assert not llm.engine.cache.requests
    assert llm.engine.cache.n_free_pages(0) == llm.engine.cache.n_blocks
    assert llm.generate([[4, 5, 6, 7]], max_tokens=100)[0] == want


@pytest.mark.parametrize("library", ["tc", "stream", "attn_tc"])
def test_a_bounded_wait_runs_out_and_the_kernel_returns(library):
    """A wait of the TMA kernels' own kind (mbar_wait, the library's limit) on a barrier at which
    nothing ever arrives: with the limit set to 100,000 cycles the thread gives up within a
    millisecond, writes its code to the error word and the kernel returns; the entry points' check
    raises and clears the word, and the device is as usable as before."""
    import time
    from rllm_b200.csrc import ops
    ops.check_device_errors(DEV)
    ops.set_wait_cycles(100_000, [library])
    try:
        torch.cuda.synchronize()
        t0 = time.time()
        ops.wait_probe(library, 2, DEV)
        torch.cuda.synchronize()
        assert time.time() - t0 < 0.5                  # far below the default limit of about a second
        with pytest.raises(ops.KernelError, match="bounded wait ran out .code 2"):
            ops.check_device_errors(DEV)
        ops.check_device_errors(DEV)                   # cleared
    finally:
        ops.set_wait_cycles(0, [library])
    # the library's product kernels still run, with the default limit back
    a = torch.randn(24, 1024, device=DEV).bfloat16()
    w = torch.randn(2048, 1024, device=DEV).bfloat16()
    out = torch.empty(24, 2048, device=DEV)
    if library == "tc":
        ops.skinny_gemm_tc(a, w, out)
    elif library == "stream":
        ops.gemv_stream(a[:8], w, out[:8])
        out, a = out[:8], a[:8]
    if library != "attn_tc":
        assert rel_err(out.cpu(), a.float().cpu() @ w.float().cpu().t()) < 1e-5
    ops.check_device_errors(DEV)
