"""Tiny configurations, model folders and trace drivers shared by the tests."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_impl

# Two tiny Qwen3 configurations that differ in every size and option, and a third with a window.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=512, hidden_act="silu", attention_bias=False)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96,
              num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=224,
              vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=1024, hidden_act="silu", attention_bias=False)
# window of 24 keys on layers 1.. (layer 0 sees everything): two cache groups
TINY_W = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=80,
              num_attention_heads=5, num_key_value_heads=1, head_dim=48, intermediate_size=176,
              vocab_size=311, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
              max_position_embeddings=1024, hidden_act="silu", attention_bias=False,
              use_sliding_window=True, sliding_window=24, max_window_layers=1)
# head sizes 64 and 128: the tensor-core attention kernels (groups of 4 and 1, one with a window)
TINY_F = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=128,
              num_attention_heads=4, num_key_value_heads=1, head_dim=64, intermediate_size=192,
              vocab_size=500, rope_theta=20000.0, rms_norm_eps=2e-6, tie_word_embeddings=True,
              max_position_embeddings=1024, hidden_act="silu", attention_bias=False)
TINY_G = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=72,
              num_attention_heads=3, num_key_value_heads=3, head_dim=128, intermediate_size=136,
              vocab_size=277, rope_theta=300000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=1024, hidden_act="silu", attention_bias=False,
              use_sliding_window=True, sliding_window=40,
              layer_types=["sliding_attention", "full_attention"])
TINY = {"A": TINY_A, "B": TINY_B, "W": TINY_W, "F": TINY_F, "G": TINY_G}


def make_model_dir(path, cfg: dict, seed: int, dtype=torch.float32, std=0.02, norm_std=0.1):
    """Writes config.json and model.safetensors with the package's random-weights mode."""
    from rllm_b200.config import config_from_dict
    from rllm_b200.weights import write_random_model
    config = config_from_dict(cfg)
    return write_random_model(config, path, seed=seed, dtype=dtype, std=std, norm_std=norm_std)


def random_tokens(n, vocab, seed):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, n)]


def plain_logits(model_dir, tokens, dtype=torch.float32):
    cfg, w = plain_impl.load_model(model_dir, dtype)
    return plain_impl.forward(cfg, w, tokens).to(torch.float32)


def run_steps(engine, steps):
    """Drives Engine.step like bin/trace_run: `steps` is a list of dicts {entries, end}.
    Returns {(request id, position): logits row (CPU float32)}."""
    from rllm_b200.engine import StepItem
    pos = {}
    out = {}
    for st in steps:
        items = [StepItem(e["id"], e["tokens"], e.get("want", [])) for e in st["entries"]]
        logits = engine.step(items) if items else None
        r = 0
        for e in st["entries"]:
            start = pos.get(e["id"], 0)
            for w in e.get("want", []):
                out[(e["id"], start + w)] = logits[r].detach().float().cpu()
                r += 1
            pos[e["id"]] = start + len(e["tokens"])
        for rid in st.get("end", []):
            engine.finish(rid)
            pos.pop(rid, None)
    return out


def rel_err(a, b):
    """max |a - b| / max |b|: the measure AxiomOperator/rllm's parity tests use
    (crates/rllm-cuda/tests/common/parity.rs:121-128)."""
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
