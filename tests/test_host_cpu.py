"""Host-side tests that need no GPU: configuration, weight files and their errors, the cache
manager under random orders of requests, the scheduler's decisions, and the plain implementation
itself.  In the manner of AxiomOperator/rllm's host unit tests (crates/rllm-kv/src/lib.rs:454-719,
crates/rllm-model/src/sampler.rs:460-569, crates/rllm-core/src/sample.rs:111-161).
"""
import json
import random
import struct

import numpy as np
import pytest
import torch

import helpers
import plain_impl
from rllm_b200.cache import BlockAllocator, CacheManager, OutOfPages
from rllm_b200.cache.native import NativeCacheManager
from rllm_b200.config import ConfigError, Qwen3Config, config_from_dict, load_config, supported_architectures
from rllm_b200.engine.scheduler import Request, Scheduler
from rllm_b200.parts import PagedKVNeed, StateNeed
from rllm_b200.sampling import HostSampler, SamplingParams, SplitMix64
from rllm_b200.weights import (SafetensorsFile, WeightFileError, WeightMismatchError, load_checked,
                               write_random_model, write_safetensors)


# ---------------------------------------------------------------- configuration

def test_config_reads_every_key():
    for name, d in helpers.TINY.items():
        c = config_from_dict(d)
        assert isinstance(c, Qwen3Config)
        assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                c.intermediate_size, c.vocab_size) == tuple(d[k] for k in (
                    "num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size"))
        assert c.rms_norm_eps == d["rms_norm_eps"] and c.rope_theta == d["rope_theta"]
        assert c.tie_word_embeddings == d["tie_word_embeddings"]
        assert list(c.layer_windows) == plain_impl.layer_windows(d)
        # what it writes reads back to the same configuration
        assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c
    w = config_from_dict(helpers.TINY_W)
    assert w.layer_windows == (0, 24, 24)
    g = config_from_dict(helpers.TINY_G)
    assert g.layer_windows == (40, 0)


def test_config_defaults_and_rope_parameters():
    d = dict(helpers.TINY_A)
    del d["head_dim"], d["rope_theta"], d["rms_norm_eps"]
    d["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    c = config_from_dict(d)
    assert c.head_dim == 64 // 4 and c.rope_theta == 12345.0 and c.rms_norm_eps == 1e-6
    # a window that is configured but switched off is no window
    d2 = dict(helpers.TINY_A, sliding_window=32, use_sliding_window=False, max_window_layers=0)
    assert config_from_dict(d2).layer_windows == (0, 0)
    d3 = dict(helpers.TINY_G, use_sliding_window=False)
    assert config_from_dict(d3).layer_windows == (0, 0) == tuple(plain_impl.layer_windows(d3))


@pytest.mark.parametrize("change,needle", [
    ({"architectures": ["GPT2LMHeadModel"]}, "unsupported architecture"),
    ({"hidden_size": None}, "'hidden_size'"),
    ({"num_hidden_layers": "two"}, "'num_hidden_layers'"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 20}, "'head_dim'"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"attention_bias": True}, "'attention_bias'"),
    ({"hidden_act": "gelu"}, "'hidden_act'"),
    ({"layer_types": ["full_attention"]}, "'layer_types'"),
    ({"vocab_size": 0}, "'vocab_size'"),
])
def test_config_errors_name_the_key(change, needle):
    d = dict(helpers.TINY_A, **change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert needle in str(e.value)
    if "unsupported" in needle:
        assert "Qwen3ForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in supported_architectures()


def test_model_spec_is_data():
    spec = config_from_dict(helpers.TINY_W).model_spec()
    assert [e.layer for e in spec.run_order] == [0, 1, 2]
    assert [l.mixer.params["window"] for l in spec.layers] == [0, 24, 24]
    assert spec.layers[0].mixer.kind == "attention" and spec.layers[0].ffn.kind == "swiglu"
    assert spec.layers[1].mixer.params["scale"] == 48 ** -0.5
    assert spec.lm_head.params["tied_to"] is None
    assert config_from_dict(helpers.TINY_A).model_spec().lm_head.params["tied_to"] == "model.embed_tokens.weight"


# ---------------------------------------------------------------- weights

def test_random_model_roundtrip_and_seed(tmp_path):
    cfg = config_from_dict(helpers.TINY_B)
    a = write_random_model(cfg, tmp_path / "a", seed=3, dtype=torch.bfloat16)
    b = write_random_model(cfg, tmp_path / "b", seed=3, dtype=torch.bfloat16)
    c = write_random_model(cfg, tmp_path / "c", seed=4, dtype=torch.float32)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert load_config(a) == cfg
    fa, fc = SafetensorsFile(a / "model.safetensors"), SafetensorsFile(c / "model.safetensors")
    assert set(fa.names()) == set(fc.names())
    assert "lm_head.weight" in fa.names()                       # untied
    assert fa.dtype("model.embed_tokens.weight") == torch.bfloat16 and fc.dtype("model.norm.weight") == torch.float32
    assert fa.shape("model.layers.2.self_attn.q_proj.weight") == (6 * 32, 96)
    assert fa.shape("model.layers.0.self_attn.k_norm.weight") == (32,)
    assert not torch.equal(fa.tensor("model.norm.weight").float(), fc.tensor("model.norm.weight"))
    # the plain implementation's own reader sees the same values
    mine = plain_impl.read_safetensors(a / "model.safetensors")
    for n in fa.names():
        assert torch.equal(mine[n], fa.tensor(n))
    tied = write_random_model(config_from_dict(helpers.TINY_A), tmp_path / "t", seed=0)
    assert "lm_head.weight" not in SafetensorsFile(tied / "model.safetensors").names()


def test_loader_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from rllm_b200.models.model import expected_tensors
    cfg = config_from_dict(helpers.TINY_A)
    exp = {n: s for n, (s, _) in expected_tensors(cfg.model_spec()).items()}
    d = write_random_model(cfg, tmp_path / "m", seed=0, dtype=torch.float32)
    good = load_checked(d, exp)
    assert set(good) == set(exp) and good["model.norm.weight"].dtype == torch.float32
    tensors = dict(good)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    tensors["model.layers.7.extra.weight"] = torch.zeros(3)
    write_safetensors(d / "model.safetensors", tensors)
    with pytest.raises(WeightMismatchError) as e:
        load_checked(d, exp)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    msg = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "is [64, 63], expected [64, 64]"):
        assert needle in msg
    # a tied model may still carry an lm_head: tolerated, not read
    tensors = dict(good, **{"lm_head.weight": torch.zeros(256, 64)})
    write_safetensors(d / "model.safetensors", tensors)
    assert set(load_checked(d, exp, ignorable={"lm_head.weight"})) == set(exp)


def test_sharded_checkpoints(tmp_path):
    """A folder with model.safetensors.index.json and model-0000i-of-0000N.safetensors shards loads to
    the same tensors as the one-file folder; every way in which index and shards can disagree is an
    error that names the file (the reference asks for each tensor by name and names it when it is
    not there: crates/rllm-model/src/loader.rs:8-23)."""
    import shutil
    from rllm_b200.models.model import expected_tensors
    from rllm_b200.weights import weight_files, write_sharded
    cfg = config_from_dict(helpers.TINY_B)
    exp = {n: s for n, (s, _) in expected_tensors(cfg.model_spec()).items()}
    one = load_checked(write_random_model(cfg, tmp_path / "one", seed=5, dtype=torch.bfloat16), exp)
    d = write_random_model(cfg, tmp_path / "three", seed=5, dtype=torch.bfloat16, shards=3)
    files = sorted(p.name for p in d.glob("*.safetensors"))
    assert files == [f"model-0000{i}-of-00003.safetensors" for i in (1, 2, 3)]
    where, paths = weight_files(d)
    assert len(paths) == 3 and set(where) == set(exp) and len(set(where.values())) == 3
    got = load_checked(d, exp)
    assert set(got) == set(one) and all(torch.equal(got[n], one[n]) for n in one)
    index = json.loads((d / "model.safetensors.index.json").read_text())

    def variant(name):
        v = tmp_path / name
        shutil.copytree(d, v)
        return v

    v = variant("missing_shard")
    (v / files[1]).unlink()
    with pytest.raises(WeightFileError, match=files[1] + ".*shard is missing"):
        load_checked(v, exp)

    v = variant("moved_tensor")                      # the index names a shard that does not hold the tensor
    moved = next(n for n, f in index["weight_map"].items() if f == files[0])
    idx = json.loads(json.dumps(index))
    idx["weight_map"][moved] = files[2]
    (v / "model.safetensors.index.json").write_text(json.dumps(idx))
    with pytest.raises(WeightFileError, match=files[2] + ".*" + moved.replace(".", r"\.") + ".*does not hold it.*" + files[0]):
        load_checked(v, exp)

    v = variant("twice")                             # one tensor stored in two shards
    with SafetensorsFile(v / files[0]) as f0, SafetensorsFile(v / files[1]) as f1:
        t1 = {n: f1.tensor(n) for n in f1.names()}
        dup = f0.names()[0]
        t1[dup] = f0.tensor(dup)
    write_safetensors(v / files[1], t1)
    with pytest.raises(WeightFileError, match="stored here and in"):
        load_checked(v, exp)

    v = variant("lists")                             # missing, unexpected and wrong shapes across shards: one error
    with SafetensorsFile(v / files[2]) as f2:
        t2 = {n: f2.tensor(n) for n in f2.names()}
    gone = sorted(t2)[0]
    del t2[gone]
    t2["model.extra.weight"] = torch.zeros(2)
    write_safetensors(v / files[2], t2)
    idx = json.loads(json.dumps(index))
    del idx["weight_map"][gone]
    idx["weight_map"]["model.extra.weight"] = files[2]
    (v / "model.safetensors.index.json").write_text(json.dumps(idx))
    with pytest.raises(WeightMismatchError) as e:
        load_checked(v, exp)
    assert e.value.missing == [gone] and e.value.unexpected == ["model.extra.weight"]
    assert "model.safetensors.index.json" in str(e.value)

    v = variant("bad_index")
    (v / "model.safetensors.index.json").write_text("{\"weight_map\": 3}")
    with pytest.raises(WeightFileError, match="not a weight map"):
        load_checked(v, exp)
    idx = json.loads(json.dumps(index))
    idx["weight_map"][moved] = "../elsewhere.safetensors"
    (v / "model.safetensors.index.json").write_text(json.dumps(idx))
    with pytest.raises(WeightFileError, match="not a file name in this folder"):
        load_checked(v, exp)
    with pytest.raises(WeightFileError, match="neither model.safetensors nor"):
        load_checked(tmp_path / "nowhere", exp)
    # more shards than tensors: one tensor each, none empty
    many = {f"t{i}": torch.full((i + 1,), float(i)) for i in range(3)}
    assert len(write_sharded(tmp_path, many, 7)) == 3


def test_ctx_beyond_the_models_positions_is_refused(tmp_path):
    from rllm_b200.llm import LLM
    from rllm_b200.config import ConfigError

    class Spec:
        max_position = 512

    class Model:
        spec = Spec()
    with pytest.raises(ConfigError, match="max_position_embeddings"):
        LLM(Model(), ctx=513)


def test_loader_dtypes(tmp_path):
    t = {"a": torch.ones(2, 2, dtype=torch.float16), "b": torch.ones(2, dtype=torch.float32),
         "c": torch.arange(4, dtype=torch.int64), "d": torch.ones(3, dtype=torch.bfloat16)}
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", t)
    got = load_checked(tmp_path / "m", {k: tuple(v.shape) for k, v in t.items()})
    assert [got[k].dtype for k in "abcd"] == [torch.bfloat16, torch.float32, torch.int32, torch.bfloat16]


def test_malformed_weight_files(tmp_path):
    p = tmp_path / "x.safetensors"
    write_safetensors(p, {"w": torch.arange(6, dtype=torch.float32).reshape(2, 3)})
    raw = p.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])

    def rewrite(h, data=raw[8 + hlen:]):
        hj = json.dumps(h).encode()
        p.write_bytes(struct.pack("<Q", len(hj)) + hj + data)

    p.write_bytes(raw[:-4])
    with pytest.raises(WeightFileError, match="truncated"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + raw[8:])
    with pytest.raises(WeightFileError, match="header length"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 5) + b"{nope" + raw[8 + hlen:])
    with pytest.raises(WeightFileError, match="not valid JSON"):
        SafetensorsFile(p)
    bad = json.loads(json.dumps(header)); bad["w"]["data_offsets"] = [0, 20]
    rewrite(bad)
    with pytest.raises(WeightFileError, match="do not hold 24 bytes"):
        SafetensorsFile(p)
    bad = json.loads(json.dumps(header)); bad["w"]["dtype"] = "F8_E4M3"
    rewrite(bad)
    with pytest.raises(WeightFileError, match="not supported"):
        SafetensorsFile(p)
    bad = json.loads(json.dumps(header)); bad["v"] = {"dtype": "F32", "shape": [2], "data_offsets": [16, 24]}
    rewrite(bad)
    with pytest.raises(WeightFileError, match="overlap"):
        SafetensorsFile(p)
    with pytest.raises(WeightFileError, match="no such file"):
        SafetensorsFile(tmp_path / "absent.safetensors")


# ---------------------------------------------------------------- cache manager

def test_block_allocator_all_or_nothing_and_double_free():
    a = BlockAllocator(4)
    assert a.alloc(2) == [0, 1]                               # lowest ids first
    with pytest.raises(OutOfPages) as e:
        a.alloc(3)
    assert (e.value.need, e.value.free) == (3, 2) and a.n_free == 2
    a.release(0)
    with pytest.raises(ValueError):
        a.release(0)
    assert a.alloc(1) == [0]                                  # a freed page is handed out again
    a.share(1); a.release(1)
    assert a.refcount(1) == 1 and a.n_free == 2


def test_cache_manager_slots_and_tables():
    cm = CacheManager([PagedKVNeed(2, 16)], [None], block_size=4, max_tokens=32, max_requests=2)
    assert cm.append("a", 5)[0] == [0, 1, 2, 3, 4]
    assert cm.append("b", 3)[0] == [8, 9, 10]
    assert cm.append("a", 4)[0] == [5, 6, 7, 12]              # a's third page comes after b's first
    assert cm.block_table("a", 0) == [0, 1, 3] and cm.length("a") == 9
    with pytest.raises(OutOfPages):
        cm.append("c", 1)                                     # no state slot left
    before = (cm.n_free_pages(0), cm.length("b"))
    with pytest.raises(OutOfPages):
        cm.append("b", 100)
    assert (cm.n_free_pages(0), cm.length("b")) == before     # nothing taken
    cm.truncate("a", 4)
    assert cm.block_table("a", 0) == [0] and cm.length("a") == 4
    cm.free("a"); cm.free("b")
    assert cm.n_free_pages(0) == 8
    cm.check_invariants()


def test_cache_groups_window_and_shared_cache():
    full, win = PagedKVNeed(2, 16, 0), PagedKVNeed(2, 16, 40)
    for manager in (CacheManager, NativeCacheManager):
        cm = manager([full, win, win, win, StateNeed((3,)), None], [None, None, None, 1, None, None],
                     block_size=16, max_tokens=1024, max_requests=3)
        assert len(cm.paged) == 2 and len(cm.stateful) == 1
        assert cm.entry_place[3] == cm.entry_place[1]             # entry 3 reads entry 1's cache
        assert cm.entry_place[5] is None
        assert [len(g.entries) for g in cm.paged] == [1, 2]
        # Pages are given back in runs of 128 keys (the kernels' largest key tile: a tile that still holds a
        # key inside the window is loaded whole).  After 166 tokens the next query sits at position 166 and
        # reads keys from 127 on; one token later the window starts at 128 and keys 0..127 are out of reach.
        cm.append("r", 166)
        assert cm.release_passed("r") == 0
        cm.append("r", 1)
        assert cm.release_passed("r") == 8                        # keys 0..127: eight pages of 16
        assert cm.block_table("r", 0) == list(range(11))          # the group without a window keeps everything
        assert cm.block_table("r", 1)[:9] == [0] * 8 + [8]        # pages given back read as 0
        # a long portion needs pages for all of its tokens at once, and gives most back after the step
        free_before = cm.n_free_pages(1)
        cm.append("r", 300)                                       # 167 -> 467 tokens: 30 pages where 11 were
        assert cm.n_free_pages(1) == free_before - 19
        assert cm.release_passed("r") == 16                       # the window now starts at 428: keys below 384 go
        cm.check_invariants()
        cm.free("r")
        assert cm.n_free_pages(0) == cm.n_free_pages(1) == cm.n_blocks
    with pytest.raises(ValueError):
        CacheManager([full, win], [None, 0], 4, 64, 2)        # reading a cache of another kind


def test_windowed_groups_get_smaller_pools_when_the_step_size_is_promised():
    full, win = PagedKVNeed(2, 16, 0), PagedKVNeed(2, 16, 40)
    for manager in (CacheManager, NativeCacheManager):
        cm = manager([full, win], [None, None], block_size=16, max_tokens=4096, max_requests=2, max_step_tokens=64)
        assert cm.paged[0].n_blocks == 256
        assert cm.paged[1].n_blocks == 2 * (-(-(40 + 64 + 128) // 16) + 1) == 32      # window + step + release alignment
        for _ in range(20):                                   # 1,280 tokens in portions of 64: the small pool suffices
            cm.append("a", 64)
            cm.release_passed("a")
            cm.append("b", 64)
            cm.release_passed("b")
            cm.check_invariants()
        assert cm.n_free_pages(0) == 256 - 2 * 80 and cm.n_free_pages(1) >= 32 - 2 * 16
        with pytest.raises(OutOfPages):                       # a portion beyond the promise: refused, nothing taken
            cm.append("a", 600)
        cm.check_invariants()
        cm.free("a"); cm.free("b")
        assert cm.n_free_pages(0) == 256 and cm.n_free_pages(1) == 32


def test_a_request_cannot_outgrow_the_models_positions():
    from rllm_b200.cache import RequestTooLong
    for manager in (CacheManager, NativeCacheManager):
        cm = manager([PagedKVNeed(1, 16)], [None], 16, 1024, 4)
        cm.set_max_length(100)
        cm.append("a", 90)
        assert cm.can_append([("a", 10)]) and not cm.can_append([("a", 11)])
        with pytest.raises(RequestTooLong, match="max_position_embeddings") as e:
            cm.append("a", 11)
        assert (e.value.length, e.value.limit) == (101, 100)
        with pytest.raises(RequestTooLong):
            cm.check_append([("b", 5), ("c", 101)])
        assert cm.length("a") == 90 and not cm.has("c")           # nothing changed
        cm.append("a", 10)
        cm.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_cache_manager_random_orders(seed):
    rng = random.Random(seed)
    needs = [PagedKVNeed(1, 16, 0), PagedKVNeed(1, 16, 9), PagedKVNeed(1, 16, 0), StateNeed((2,))]
    cm = CacheManager(needs, [None] * 4, block_size=rng.choice([1, 4, 16]), max_tokens=200, max_requests=5)
    live, nxt = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            live[nxt] = 0
            nxt += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 30])
            state = (cm.n_free_pages(0), cm.n_free_pages(1), cm.slots.n_free)
            try:
                slots = cm.append(rid, n)
            except OutOfPages:
                assert state == (cm.n_free_pages(0), cm.n_free_pages(1), cm.slots.n_free)
                victim = rng.choice(list(live))
                if cm.has(victim):
                    cm.free(victim)
                del live[victim]
            else:
                assert all(len(s) == n for s in slots)
                # what the kernels' range checks hold the host to: every slot lies inside the pool
                # (rows = pages x page size), every table entry names a page of the pool
                assert all(0 <= x < cm.n_blocks * cm.block_size for s in slots for x in s)
                assert all(0 <= b < cm.n_blocks for g in range(len(cm.paged)) for b in cm.block_table(rid, g))
                live[rid] += n
                assert cm.length(rid) == live[rid]
                cm.release_passed(rid)
        elif live:
            rid = rng.choice(list(live))
            if cm.has(rid):
                cm.free(rid)
                with pytest.raises(KeyError):
                    cm.free(rid)
            del live[rid]
        cm.check_invariants()
    for rid in list(live):
        if cm.has(rid):
            cm.free(rid)
    cm.check_invariants()
    assert all(cm.n_free_pages(g) == cm.n_blocks for g in range(2)) and cm.slots.n_free == 5


# ---------------------------------------------------------------- scheduler

def drive(sched, cache, pick=lambda seq_tokens: 7, max_steps=10000):
    """Runs the scheduler against the host cache manager with a fake model."""
    log = []
    while sched.has_work() and max_steps:
        max_steps -= 1
        plan = sched.plan()
        if not plan:
            continue
        assert cache.can_append([(p.seq.rid, p.take) for p in plan])
        for p in plan:
            cache.append(p.seq.rid, p.take)
        log.append([(p.seq.rid, p.take, p.want_last) for p in plan])
        sched.commit(plan, [pick(p.seq.tokens) for p in plan if p.want_last])
        cache.check_invariants()
    return log


def test_scheduler_portions_budget_and_order():
    cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, 4096, 8)
    s = Scheduler(cache, ctx=512, max_num_seqs=4, prefill_chunk=32)
    for i, n in enumerate([50, 20, 5]):
        s.add(Request(i, list(range(n)), max_tokens=3))
    log = drive(s, cache)
    assert log[0] == [(0, 32, False)]                          # the first prompt takes the whole budget
    assert log[1] == [(0, 18, True), (1, 14, False)]           # the rest is shared in admission order
    assert log[2] == [(0, 1, True), (1, 6, True), (2, 5, True)]   # decoders first, one token each
    done = {f.request_id: f for f in s.collect()}
    assert all(f.reason == "length" and len(f.tokens) == 3 for f in done.values())
    assert not cache.requests and cache.n_free_pages(0) == cache.n_blocks
    assert s.stats["prompt_tokens"] == 75 and s.stats["generated_tokens"] == 9


def test_scheduler_accept_and_stop():
    cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, 4096, 8)
    s = Scheduler(cache, ctx=64, max_num_seqs=2, prefill_chunk=512)
    with pytest.raises(ValueError, match="empty prompt"):
        s.add(Request("e", []))
    with pytest.raises(ValueError, match="does not fit"):
        s.add(Request("l", list(range(64))))
    s.add(Request("z", list(range(5)), max_tokens=0))
    assert s.collect()[0].reason == "length"
    s.add(Request("a", list(range(60)), max_tokens=100))       # budget = ctx - prompt = 4
    s.add(Request("b", [1, 2, 3], max_tokens=100, stop_ids=frozenset([9])))
    toks = iter([1, 2, 3, 9, 5, 6, 7, 8])
    drive(s, cache, pick=lambda t: 9 if len(t) == 6 and t[:3] == [1, 2, 3] else 4)
    done = {f.request_id: f for f in s.collect()}
    assert done["a"].reason == "length" and len(done["a"].tokens) == 4
    assert done["b"].reason == "stop" and done["b"].tokens[-1] == 9 and len(done["b"].tokens) == 4


def test_scheduler_preempts_newest_and_results_do_not_change():
    def run(max_tokens_pool):
        cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, max_tokens_pool, 8)
        s = Scheduler(cache, ctx=400, max_num_seqs=4, prefill_chunk=64)
        for i in range(4):
            s.add(Request(i, [i] * 30, max_tokens=120))
        # the fake model's token depends on the request's whole history: a recomputed request must
        # continue exactly where it was
        drive(s, cache, pick=lambda t: (sum(t) * 31 + len(t)) % 1000)
        return {f.request_id: f.tokens for f in s.collect()}, s.stats["preemptions"]
    roomy, p0 = run(4096)
    tight, p1 = run(384)             # 4 x 150 tokens do not fit 384: somebody must wait
    assert p0 == 0 and p1 >= 1
    assert roomy == tight


def test_scheduler_never_fits():
    cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, 64, 4)
    s = Scheduler(cache, ctx=4096, max_num_seqs=2, prefill_chunk=512)
    s.add(Request("big", list(range(200)), max_tokens=4))      # the prompt alone exceeds the pool
    s.add(Request("grow", list(range(40)), max_tokens=100))    # fits at first, outgrows the pool alone
    s.add(Request("ok", list(range(10)), max_tokens=2))
    drive(s, cache)
    done = {f.request_id: f for f in s.collect()}
    assert done["big"].reason == "error" and "more KV cache than the pool" in done["big"].error
    assert done["grow"].reason == "error" and len(done["grow"].tokens) > 0
    assert done["ok"].reason == "length"
    assert not cache.requests and cache.n_free_pages(0) == cache.n_blocks


def test_scheduler_failed_step_frees_running():
    cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, 1024, 4)
    s = Scheduler(cache, ctx=256, max_num_seqs=2, prefill_chunk=512)
    for i in range(3):
        s.add(Request(i, [1] * 20, max_tokens=5))
    plan = s.plan()
    for p in plan:
        cache.append(p.seq.rid, p.take)
    failed = s.fail_running("device fault (injected on the host)")
    assert sorted(f.request_id for f in failed) == [0, 1] and all(f.reason == "error" for f in failed)
    assert not cache.requests
    drive(s, cache)                                            # the queue goes on
    assert [f.request_id for f in s.collect() if f.reason == "length"] == [2]


def drive_pipelined(sched, cache, pick, max_steps=10000):
    """As `drive`, but the way LLM.generate runs with the sampler on the device: a step's tokens are
    committed only after the next step has been planned (plan_ahead) and appended to the cache."""
    pending, n_ahead = None, 0
    while (sched.has_work() or pending is not None) and max_steps:
        max_steps -= 1
        if pending is None:
            plan = sched.plan()
            if not plan:
                continue
            for p in plan:
                cache.append(p.seq.rid, p.take)
            pending = plan
            continue
        plan = pending
        ahead = sched.plan_ahead(plan)
        if ahead:
            n_ahead += 1
            # the requests that `plan` samples for decode that token (a placeholder until it is known), first
            # and in `plan`'s order; the others go on with their prompts, whose tokens are known
            n_dec = sum(p.sampled for p in ahead)
            sampled_for = [p.seq for p in plan if p.want_last and p.seq in sched.running]
            assert [p.seq for p in ahead[:n_dec]] == [q for q in sampled_for if any(a.seq is q for a in ahead[:n_dec])]
            assert all(p.sampled and p.tokens == [0] for p in ahead[:n_dec])
            for p in ahead[n_dec:]:
                mine = next((q for q in plan if q.seq is p.seq), None)      # None: admitted with this step
                first = p.seq.cached + (mine.take if mine else 0)
                assert not p.sampled and (mine is None or not mine.want_last)
                assert p.tokens == p.seq.tokens[first:first + p.take]
            if len(ahead) > n_dec:
                drive_pipelined.mixed += 1
            for p in ahead:
                cache.append(p.seq.rid, p.take)
        # the tokens of `plan` arrive: each from the request's history before it (an item planned ahead
        # does not know its own input token yet, the history does once the step before is committed)
        ids = [pick(p.seq.tokens) for p in plan if p.want_last and p.seq in sched.running]
        it = iter(ids)
        ids = [next(it) if p.seq in sched.running else -1 for p in plan if p.want_last]
        sched.commit(plan, ids)
        cache.check_invariants()
        pending = ahead
    return n_ahead


drive_pipelined.mixed = 0


def test_planning_ahead_changes_no_result():
    def pick(t):
        return (sum(t) * 31 + len(t)) % 1000

    def run(pipelined, pool, stop=frozenset()):
        cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, pool, 8)
        s = Scheduler(cache, ctx=400, max_num_seqs=3, prefill_chunk=64)
        for i in range(5):
            s.add(Request(i, [i + 1] * (20 + 7 * i), max_tokens=60 + 9 * i, stop_ids=stop))
        n = drive_pipelined(s, cache, pick) if pipelined else (drive(s, cache, pick) and 0)
        assert not cache.requests and cache.n_free_pages(0) == cache.n_blocks
        return {f.request_id: (f.tokens, f.reason) for f in s.collect()}, n, s.stats["preemptions"]
    plain, _, _ = run(False, 4096)
    ahead, n, _ = run(True, 4096)
    assert ahead == plain and n > 50                       # most decode steps were planned ahead
    # stop ids end requests in the middle (the step planned ahead then ran one token too far for them)
    some = sorted({t for toks, _ in plain.values() for t in toks[10:40]})[:25]
    plain_stop, _, _ = run(False, 4096, frozenset(some))
    ahead_stop, n, _ = run(True, 4096, frozenset(some))
    assert ahead_stop == plain_stop and any(r == "stop" for _, r in plain_stop.values()) and n > 2
    # a pool so small that requests are preempted: planning ahead steps back when pages are short
    plain_tight, _, p0 = run(False, 208)
    ahead_tight, _, p1 = run(True, 208)
    assert ahead_tight == plain_tight == plain and p0 >= 1 and p1 >= 1

    # long prompts in portions beside decoding requests: those steps are planned ahead too
    def run_long(pipelined, quantum=0):
        cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, 8192, 8)
        s = Scheduler(cache, ctx=2048, max_num_seqs=3, prefill_chunk=64, row_quantum=quantum)
        for i in range(6):
            s.add(Request(i, [(i * 7 + j) % 50 + 1 for j in range(150 + 90 * i)], max_tokens=20 + 5 * i))
        drive_pipelined.mixed = 0
        if pipelined:
            drive_pipelined(s, cache, pick)
        else:
            drive(s, cache, pick)
        assert not cache.requests and cache.n_free_pages(0) == cache.n_blocks
        return {f.request_id: (f.tokens, f.reason) for f in s.collect()}, drive_pipelined.mixed
    plain_long, _ = run_long(False)
    ahead_long, mixed = run_long(True)
    assert ahead_long == plain_long and mixed > 10
    trimmed, mixed = run_long(True, quantum=32)
    assert trimmed == plain_long and mixed > 10


class _FakeEngine:
    """Stands in for the engine under LLM.generate: the host cache manager and a step that returns
    logits naming token (number of tokens the request holds) % 50, or raises on the steps listed."""

    def __init__(self, fail_steps=(), device_error_at=()):
        self.cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, 1024, 4)
        self.calls, self.fail_steps, self.device_error_at = 0, set(fail_steps), set(device_error_at)
        self.checks = 0

    def step(self, items, device_tokens=None, n_device=None):
        self.calls += 1
        if self.calls in self.fail_steps:
            raise RuntimeError(f"injected fault in step {self.calls}")
        rows = []
        for it in items:
            self.cache.append(it.request_id, len(it.tokens))
            for _ in it.want:
                row = torch.zeros(50)
                row[self.cache.length(it.request_id) % 50] = 1.0
                rows.append(row)
        return torch.stack(rows) if rows else None

    def check_device_errors(self):
        self.checks += 1
        if self.checks in self.device_error_at:
            raise RuntimeError("a kernel's bounded wait ran out (injected)")


def _fake_llm(engine, parallel=2):
    from rllm_b200.llm import LLM
    llm = object.__new__(LLM)
    llm.engine, llm.ctx, llm.prefill_chunk, llm.parallel = engine, 256, 512, parallel
    llm.host_sampling, llm.last_stats, llm.last_errors = True, {}, {}
    return llm


def test_generate_goes_on_after_a_failed_step():
    """A failed step fails the requests running in it and frees their pages; the waiting requests
    still run, and the errors are reported per request (crates/rllm-server/src/engine.rs:569-578)."""
    from rllm_b200.llm import GenerationError
    prompts = [[1] * 5, [2] * 7, [3] * 4, [4] * 9]
    good = _fake_llm(_FakeEngine()).generate(prompts, max_tokens=6)
    assert good[0] == [(5 + i) % 50 for i in range(6)]
    eng = _FakeEngine(fail_steps={3})                          # requests 0 and 1 run then, 2 and 3 wait
    llm = _fake_llm(eng)
    with pytest.raises(GenerationError, match="injected fault in step 3") as ei:
        llm.generate(prompts, max_tokens=6)
    err = ei.value
    assert sorted(err.errors) == [0, 1]
    assert [f.tokens for f in err.results[2:]] == good[2:] and all(f.reason == "length" for f in err.results[2:])
    assert len(err.results[0].tokens) == 2                     # what it had generated before the fault
    assert not eng.cache.requests and eng.cache.n_free_pages(0) == eng.cache.n_blocks
    # with return_reasons nothing is raised: the failed requests come back with the reason "error"
    eng = _FakeEngine(fail_steps={1})
    llm = _fake_llm(eng)
    out = llm.generate(prompts, max_tokens=6, return_reasons=True)
    assert [r for _, r in out] == ["error", "error", "length", "length"] and sorted(llm.last_errors) == [0, 1]
    assert [t for t, _ in out[2:]] == good[2:]
    # the same engine again: numbered from 0 again, on a clean cache, the same tokens as a fresh one
    assert llm.generate(prompts, max_tokens=6) == good


def test_generate_leaves_nothing_in_the_cache_however_it_ends():
    from rllm_b200.llm import GenerationError

    class Interrupting(_FakeEngine):
        def step(self, items, device_tokens=None, n_device=None):
            if self.calls == 2:
                raise KeyboardInterrupt
            return super().step(items, device_tokens)

    eng = Interrupting()
    llm = _fake_llm(eng)
    with pytest.raises(KeyboardInterrupt):
        llm.generate([[1] * 5, [2] * 7], max_tokens=6)
    assert not eng.cache.requests and eng.cache.n_free_pages(0) == eng.cache.n_blocks
    # the device's error word read in the middle (every 64 steps) fails the running requests only
    eng = _FakeEngine(device_error_at={1})
    llm = _fake_llm(eng, parallel=1)
    with pytest.raises(GenerationError, match="bounded wait") as ei:
        llm.generate([[1] * 5, [2] * 7], max_tokens=80)
    assert sorted(ei.value.errors) == [0] and len(ei.value.results[1].tokens) == 80
    assert not eng.cache.requests
    # read at the end, it fails everything the call generated
    eng = _FakeEngine(device_error_at={1})
    with pytest.raises(GenerationError) as ei:
        _fake_llm(eng).generate([[1] * 5, [2] * 7], max_tokens=6)
    assert sorted(ei.value.errors) == [0, 1]


# ---------------------------------------------------------------- samplers and the plain implementation

def test_host_sampler():
    logits = np.array([0.1, 3.0, 3.0, -1.0, np.nan], dtype=np.float32)
    assert HostSampler(SamplingParams()).sample(logits) == 1          # first index on ties, NaN never wins
    r = SplitMix64(1)
    assert [r.next_u64() for _ in range(2)] == [0x910A2DEC89025CC1, 0xBEEB8DA1658EEC67]
    s = HostSampler(SamplingParams(temperature=1.0, top_k=2, seed=3))
    assert {s.sample(logits) for _ in range(50)} <= {1, 2}
    ids, probs = HostSampler(SamplingParams(temperature=1.0, top_p=0.5)).candidates(
        np.array([2.0, 1.0, 0.0, -1.0], dtype=np.float32))
    assert list(ids) == [0]
    x = np.array([2.0, 1.0, 0.0, -1.0, 1.5], dtype=np.float32)
    s = HostSampler(SamplingParams(temperature=0.7, seed=11))
    n = 20000
    freq = np.bincount([s.sample(x) for _ in range(n)], minlength=5) / n
    p = np.exp(x / 0.7) / np.exp(x / 0.7).sum()
    assert np.abs(freq - p).max() < 0.012


def test_logit_bias_and_penalties():
    """The adjustments of crates/rllm-server/src/engine.rs:1113-1129: bias pairs, and for every
    token generated c times so far -(c * frequency_penalty + presence_penalty); equal tokens summed."""
    p = SamplingParams(frequency_penalty=0.5, presence_penalty=1.0, logit_bias=((3, 2.0), (7, -100.0), (3, 0.25)))
    assert p.adjusts and not SamplingParams().adjusts
    assert p.adjustments(None) == {3: 2.25, 7: -100.0}
    assert p.adjustments({3: 2, 5: 1}) == {3: 2.25 - 2.0, 7: -100.0, 5: -1.5}
    logits = np.array([0.0, 1.0, 0.5, 0.9, 0.2, 0.95, 0.1, 5.0], dtype=np.float32)
    assert HostSampler(SamplingParams()).sample(logits) == 7
    assert HostSampler(p).sample(logits) == 3                          # 7 is biased away, 3 biased up
    assert HostSampler(p).sample(logits, {3: 4}) == 1                  # 3 generated four times: 3.15 - 3.0 < 1.0
    assert logits[7] == 5.0                                            # the row itself is left alone
    assert plain_impl.sample_row(logits, 0, 0, 1.0, 0, 0, adjust=p.adjustments({3: 4}).items()) == 1
    # the scheduler counts what a request generated
    from rllm_b200.cache import CacheManager
    from rllm_b200.parts import PagedKVNeed
    cache = CacheManager([PagedKVNeed(1, 16, 0)], [None], 4, 64, 2)
    sched = Scheduler(cache, ctx=64, max_num_seqs=2, prefill_chunk=16)
    sched.add(Request("a", [1, 2, 3], 4, p, frozenset()))
    for tok in (5, 5, 9):
        plan = sched.plan()
        cache.append("a", plan[0].take)
        sched.commit(plan, [tok])
    assert sched.running[0].counts == {5: 2, 9: 1}


def test_plain_sampler_reference():
    x = np.array([2.0, 1.0, 0.0, -1.0, 1.5, -3.0], dtype=np.float32)
    assert plain_impl.sample_row(x, 0, 0, 1.0, 0, 0) == 0
    assert abs(float(plain_impl.threshold(x, 2, 1.0)) - 1.5) < 1e-5
    thr = plain_impl.threshold(x, 0, 0.6)
    assert int((x >= thr).sum()) == 2                       # 0.47 + 0.29 >= 0.6
    u = [float(plain_impl.uniform(5, c, 3)) for c in range(2000)]
    assert 0 < min(u) and max(u) < 1 and abs(sum(u) / len(u) - 0.5) < 0.02
    draws = [plain_impl.sample_row(x, 0.7, 0, 1.0, 5, c) for c in range(4000)]
    freq = np.bincount(draws, minlength=6) / 4000
    p = np.exp(x / 0.7) / np.exp(x / 0.7).sum()
    assert np.abs(freq - p).max() < 0.03


def test_plain_implementation_parts():
    torch.manual_seed(0)
    x = torch.randn(5, 8)
    w = torch.rand(8) + 0.5
    ref = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(plain_impl.rms_norm(x, w, 1e-5), ref, atol=1e-6)
    # rotary: position 0 is the identity, norms are kept, and q.k depends on the distance only
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    assert torch.allclose(plain_impl.rope_neox(q, [0], 1e4), q)
    d1 = (plain_impl.rope_neox(q, [7], 1e4) * plain_impl.rope_neox(k, [3], 1e4)).sum()
    d2 = (plain_impl.rope_neox(q, [104], 1e4) * plain_impl.rope_neox(k, [100], 1e4)).sum()
    assert abs(float(d1 - d2)) < 1e-4
    assert torch.allclose(plain_impl.rope_neox(q, [9], 1e4).norm(), q.norm(), atol=1e-5)
    # attention: the first token sees itself only; a window of 1 returns v; GQA maps heads h // g
    qq, kk, vv = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    a = plain_impl.attention(qq, kk, vv, 0.3)
    assert torch.allclose(a[0, 3], vv[0, 1], atol=1e-6)
    a1 = plain_impl.attention(qq, kk, vv, 0.3, window=1)
    assert torch.allclose(a1[:, 0], vv[:, 0], atol=1e-6) and torch.allclose(a1[:, 2], vv[:, 1], atol=1e-6)
    aw = plain_impl.attention(qq, kk, vv, 0.3, window=3)
    assert torch.allclose(aw[:3], a[:3], atol=1e-6) and not torch.allclose(aw[5], a[5], atol=1e-4)


def test_plain_forward_is_causal_and_windows_matter(tmp_path):
    d = helpers.make_model_dir(tmp_path / "w", helpers.TINY_W, seed=5, std=0.08)
    cfg, w = plain_impl.load_model(d)
    toks = helpers.random_tokens(40, cfg["vocab_size"], 1)
    full = plain_impl.forward(cfg, w, toks)
    assert torch.allclose(plain_impl.forward(cfg, w, toks[:17]), full[:17], atol=1e-5)
    nowin = dict(cfg, use_sliding_window=False)
    other = plain_impl.forward(nowin, w, toks)
    assert torch.allclose(other[:24], full[:24], atol=1e-5)            # within the window nothing changes
    assert not torch.allclose(other[30:], full[30:], atol=1e-3)
    assert plain_impl.greedy_generate(cfg, w, toks[:5], 3) == plain_impl.greedy_generate(cfg, w, toks[:5], 3)


# ---------------------------------------------------------------- the C++ host runtime against the Python one

def _needs():
    return [PagedKVNeed(1, 16, 0), PagedKVNeed(1, 16, 9), PagedKVNeed(1, 16, 0), StateNeed((2,)), None], [None, None, 0, None, None]


@pytest.mark.parametrize("seed", range(4))
def test_native_cache_manager_matches_python(seed):
    from rllm_b200.cache.native import NativeCacheManager
    rng = random.Random(100 + seed)
    needs, cache_of = _needs()
    bs = rng.choice([1, 4, 16])
    py = CacheManager(needs, cache_of, bs, 150, 4)
    nat = NativeCacheManager(needs, cache_of, bs, 150, 4)
    assert nat.entry_place == py.entry_place and len(nat.paged) == 2
    live = []
    for step in range(500):
        op = rng.random()
        if op < 0.6:
            rid = rng.choice(live) if live and rng.random() < 0.7 else f"r{step}"
            n = rng.choice([1, 1, 2, 7, 30, 64])
            assert py.pages_needed(rid, n) == nat.pages_needed(rid, n)
            assert py.can_append([(rid, n)]) == nat.can_append([(rid, n)])
            try:
                want = py.append(rid, n)
            except OutOfPages as e:
                with pytest.raises(OutOfPages) as e2:
                    nat.append(rid, n)
                assert (e.need, e.free, e.what) == (e2.value.need, e2.value.free, e2.value.what)
                assert nat.has(rid) == py.has(rid)
            else:
                assert nat.append(rid, n) == want
                if rid not in live:
                    live.append(rid)
                assert py.release_passed(rid) == nat.release_passed(rid)
        elif op < 0.75 and live:
            rid = rng.choice(live)
            keep = rng.randrange(0, py.length(rid) + 1)
            if all(None not in py.requests[rid].tables[g] for g in range(2)):
                py.truncate(rid, keep); nat.truncate(rid, keep)
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            py.free(rid); nat.free(rid)
            with pytest.raises(KeyError):
                nat.free(rid)
        for rid in live:
            assert py.length(rid) == nat.length(rid) and py.state_slot(rid) == nat.state_slot(rid)
            for g in range(2):
                assert py.block_table(rid, g) == nat.block_table(rid, g)
                assert py.requests[rid].tables[g] == nat.block_table(rid, g, raw=True)
        assert [py.n_free_pages(g) for g in range(2)] == [nat.n_free_pages(g) for g in range(2)]
        assert py.slots.n_free == nat.slots.n_free
        nat.check_invariants()
    for rid in live:
        nat.free(rid)
    nat.check_invariants()
    assert nat.n_free_pages(0) == nat.n_blocks and not nat.requests


def test_native_step_builder_arrays():
    from rllm_b200.cache.native import NativeCacheManager
    from rllm_b200.engine.batch import StepItem
    needs, cache_of = _needs()
    nat = NativeCacheManager(needs, cache_of, 4, 200, 8)
    buf = torch.zeros(4096, dtype=torch.int32)
    nat.append("a", 6)
    items = [StepItem("a", [5, 6, 7], [0, 2]), StepItem("b", [9], []), StepItem("c", [1, 2, 3, 4, 5], [4])]
    off, (n, R, m, width, total, longest), flags = nat.build_step(items, 100, buf)
    assert (n, R, m, width, longest) == (9, 3, 3, 3, 9) and flags == [0, 1, 1] and all(o % 4 == 0 for o in off)
    a = buf.numpy()
    assert a[off[0]:off[0] + n].tolist() == [5, 6, 7, 9, 1, 2, 3, 4, 5]
    assert a[off[1]:off[1] + n].tolist() == [6, 7, 8, 0, 0, 1, 2, 3, 4]
    assert a[off[2]:off[2] + n].tolist() == [0, 0, 0, 1, 2, 2, 2, 2, 2]
    assert a[off[3]:off[3] + R + 1].tolist() == [0, 3, 4, 9] and a[off[4]:off[4] + R].tolist() == [9, 1, 5]
    assert a[off[5]:off[5] + R].tolist() == [nat.state_slot(r) for r in "abc"]
    assert a[off[6]:off[6] + m].tolist() == [0, 2, 8]
    for g in range(2):
        tab = a[off[9 + g]:off[9 + g] + R * width].reshape(R, width)
        slots = a[off[7 + g]:off[7 + g] + n]
        for i, r in enumerate("abc"):
            t = nat.block_table(r, g)
            assert tab[i, :len(t)].tolist() == t
        pos = a[off[1]:off[1] + n]; seq = a[off[2]:off[2] + n]
        assert all(slots[t] == tab[seq[t], pos[t] // 4] * 4 + pos[t] % 4 for t in range(n))
    # errors change nothing
    before = (nat.n_free_pages(0), nat.length("a"), len(nat.requests))
    with pytest.raises(OutOfPages):
        nat.build_step([StepItem("a", [1], [0]), StepItem("z", list(range(99)) * 9, [])], 100, buf)
    with pytest.raises(ValueError):
        nat.build_step([StepItem("a", [1], [3])], 100, buf)
    with pytest.raises(ValueError):
        nat.build_step([StepItem("q", [100], [0])], 100, buf)
    assert before == (nat.n_free_pages(0), nat.length("a"), len(nat.requests))
    # a buffer that is too small reports the size and appends nothing
    small = torch.zeros(8, dtype=torch.int32)
    off2, meta2, _ = nat.build_step([StepItem("a", [1, 2], [1])], 100, small)
    assert off2 is None and meta2[4] > 8 and nat.length("a") == 9
    # padded decode step
    off, (n, R, m, width, total, longest), _ = nat.build_step([StepItem("a", [3], [0]), StepItem("b", [4], [0])],
                                                              100, buf, pad_requests=4, pad_width=16)
    a = buf.numpy()
    assert (n, R, m, width, longest) == (4, 4, 4, 16, 10)
    assert a[off[0]:off[0] + 4].tolist() == [3, 4, 0, 0] and a[off[1]:off[1] + 4].tolist() == [9, 1, 0, 0]
    assert a[off[7]:off[7] + 4].tolist()[2:] == [-1, -1] and a[off[6]:off[6] + 4].tolist() == [0, 1, 2, 3]
    # the builder pads the tables itself to the longest request rounded up to a quantum of tokens
    off, meta3, _ = nat.build_step([StepItem("a", [3], [0]), StepItem("b", [4], [])], 100, buf, pad_requests=2,
                                   pad_quantum=32)
    assert meta3[5] == 11 and meta3[3] == 32 // 4
    # padded step with a portion: [one-token items][padding][portion]; logit rows: the padded one-token rows
    # and the portion's last row
    la, lc = nat.length("a"), nat.length("c")
    off, (n, R, m, width, total, longest), _ = nat.build_step(
        [StepItem("a", [3], [0]), StepItem("b", [4], []), StepItem("c", [7, 8, 9], [2])], 100, buf, pad_requests=4,
        pad_quantum=16)
    a = buf.numpy()
    assert (n, R, m, longest) == (7, 5, 5, max(la + 1, lc + 3))
    assert a[off[0]:off[0] + n].tolist() == [3, 4, 0, 0, 7, 8, 9]
    assert a[off[1]:off[1] + n].tolist() == [la, nat.length("b") - 1, 0, 0, lc, lc + 1, lc + 2]
    assert a[off[2]:off[2] + n].tolist() == [0, 1, 2, 3, 4, 4, 4]
    assert a[off[3]:off[3] + R + 1].tolist() == [0, 1, 2, 3, 4, 7]
    assert a[off[4]:off[4] + R].tolist() == [la + 1, nat.length("b"), 1, 1, lc + 3]
    assert a[off[6]:off[6] + m].tolist() == [0, 1, 2, 3, 6]
    for g in range(2):
        slots = a[off[7 + g]:off[7 + g] + n]
        tab = a[off[9 + g]:off[9 + g] + R * width].reshape(R, width)
        assert slots[2] == slots[3] == -1 and (tab[2] == 0).all() and (tab[3] == 0).all()
        t = nat.block_table("c", g)
        assert tab[4, :len(t)].tolist() == t
        assert all(slots[4 + j] == tab[4, (lc + j) // 4] * 4 + (lc + j) % 4 for j in range(3))
    # a lone portion is padded with one one-token row
    off, (n, R, m, width, total, longest), _ = nat.build_step([StepItem("c", [1, 2], [])], 100, buf, pad_requests=1)
    a = buf.numpy()
    assert (n, R, m) == (3, 2, 2) and a[off[2]:off[2] + 3].tolist() == [0, 1, 1] and a[off[6]:off[6] + 2].tolist() == [0, 2]
    # a portion anywhere but last, or two of them, is no padded shape
    for bad in ([StepItem("c", [1, 2], []), StepItem("a", [3], [])], [StepItem("a", [1, 2], []), StepItem("c", [1, 2], [])]):
        with pytest.raises(ValueError):
            nat.build_step(bad, 100, buf, pad_requests=4)
    nat.check_invariants()


def test_launch_plans_of_the_few_row_products():
    """The rules that pick CTAs and K splits are plain functions of the shape (no device needed)."""
    from rllm_b200.csrc import ops
    # swapped tcgen05 product: a power of two, CTAs up to 1.6 per SM, at least 4 blocks of 64 along K each
    assert ops.tc_swap_splits(48, 4096) == 4            # QKV of the 8B sizes: 192 CTAs
    assert ops.tc_swap_splits(32, 4096) == 4 and ops.tc_swap_splits(32, 12288) == 4      # O, down
    assert ops.tc_swap_splits(40, 8192) == 4            # 160 CTAs
    assert ops.tc_swap_splits(8, 2048) == 8
    assert ops.tc_swap_splits(8, 512) == 2              # 8 blocks along K: 4 each
    assert ops.tc_swap_splits(400, 4096) == 1
    assert ops.tc_swap_splits(192, 4096, swiglu=True) == 1
    assert ops.tc_swap_splits(48, 1024, swiglu=True) == 2 and ops.tc_swap_splits(48, 4096, swiglu=True) == 2
    for tiles in range(1, 300, 7):
        for k in (64, 512, 4096, 12288):
            for sw in (False, True):
                s = ops.tc_swap_splits(tiles, k, sw)
                assert s in (1, 2, 4, 8) and (s == 1 or -(-k // 64) // s >= 4)
    # weight-streaming product: two or three CTAs per SM, three stages
    assert ops.stream_plan(4096, 4096) == (296, 3)
    assert ops.stream_plan(12288, 4096, swiglu=True) == (444, 3)
    assert ops.stream_plan(151936, 4096) == (444, 3)


def test_which_many_row_kernel_and_which_norms_are_deferred():
    """The two-SM product is taken where it needs fewer waves than the one-CTA kernel; a norm is
    deferred whenever both products around it can run on a few-row kernel.  Plain functions of
    shapes and types."""
    from rllm_b200.csrc import ops
    cols_8b = 12288 // 128
    want = {70: False, 128: False, 200: True, 256: True, 384: False, 544: True, 672: True, 896: False,
            1152: False, 2048: True, 4096: True}
    for m, two in want.items():
        assert ops._prefer_tc2(m, cols_8b) == two, m
    assert ops._prefer_tc2(2048, 3072 // 128) and ops._prefer_tc2(210, 25600 // 128)
    w_o = torch.empty(256, 128, dtype=torch.bfloat16)
    w_gu = torch.empty(512, 256, dtype=torch.bfloat16)
    for m, yes in ((0, False), (1, True), (8, True), (9, True), (16, True), (17, True), (64, True), (65, False)):
        assert ops.defers_norm(m, w_o, w_gu, True) == yes, m
    assert not ops.defers_norm(8, w_o.float(), w_gu)                                     # the 32-bit path
    assert not ops.defers_norm(8, w_o, torch.empty(64, 100, dtype=torch.bfloat16))       # rows of 100 elements


def test_scheduler_trims_mixed_steps_to_whole_tiles():
    """With a row quantum, a step of decoding requests and prompt tokens is cut to a whole number of
    tiles when that costs at most an eighth of its prompt tokens; the tokens come in the next step."""
    def run(quantum):
        cache = CacheManager([PagedKVNeed(1, 16)], [None], 16, 8192, 8)
        s = Scheduler(cache, ctx=2048, max_num_seqs=4, prefill_chunk=512, row_quantum=quantum)
        for i, n in enumerate((20, 30, 1000)):
            s.add(Request(i, list(range(1, n + 1)), max_tokens=50))
        return [[(rid, take) for rid, take, _ in step] for step in drive(s, cache)]

    seen = run(128)
    # step 0: 20 + 30 + 462 prompt tokens = 512 rows: nothing to trim
    assert seen[0] == [(0, 20), (1, 30), (2, 462)]
    # step 1: two decoding requests beside 512 prompt tokens are 514 rows: the portion gives up two
    assert seen[1] == [(0, 1), (1, 1), (2, 510)]
    # step 2: the rest of the prompt (28 tokens) beside two: 30 rows, under one tile: as it is
    assert seen[2] == [(0, 1), (1, 1), (2, 28)]
    assert all(take == 1 for step in seen[3:] for _, take in step)
    # without a quantum nothing is trimmed
    assert run(0)[1] == [(0, 1), (1, 1), (2, 512)]
