"""Plain, slow implementation of the Qwen3 dense decoder used as the oracle in tests.

Whole sequences, no cache, one function per part, torch on the CPU only.  It
shares no code with ``rllm_b200``: it reads config.json and model.safetensors by
itself and computes every part from the formulas of AxiomOperator/rllm's CPU
backend (the float32 oracle of that project), cited per function as
``path:line`` within that project.

AxiomOperator/rllm is a Rust workspace; neither cargo nor rustc exist where
these tests run, so its model code cannot be imported or compiled here and this
file rests on the formulas alone (see tests/golden/README.md).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "F64": torch.float64, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path):
    """Minimal safetensors reader: 8-byte little-endian header length, JSON header, raw data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        buf = bytearray(raw[base + lo:base + hi])
        t = torch.frombuffer(buf, dtype=dt).reshape(info["shape"]).clone()
        out[name] = t
    return out


def load_model(model_dir, dtype=torch.float32):
    """Returns (config dict, weights dict cast to `dtype`)."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    w = {k: v.to(dtype) for k, v in read_safetensors(model_dir / "model.safetensors").items()}
    return cfg, w


# ---------------------------------------------------------------- storage rounding
# The engine's bfloat16 mode stores activations between kernels and the cache in bfloat16 while
# every sum, norm, softmax and the residual stream stay float32.  `storage` names that type; the
# functions below round at exactly those hand-over points (norm outputs, rotated queries and keys,
# values, attention output, the SwiGLU activation) and nowhere else.  None: no rounding.

def _store(x, storage):
    return x if storage is None else x.to(storage).to(torch.float32)


# ---------------------------------------------------------------- parts

def embed(table, tokens):
    """x[t,:] = table[tokens[t],:], no scaling.  crates/rllm-cpu/src/lib.rs:190-200"""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rms_norm(x, w, eps):
    """ms = sum(x^2)/d; out = x * (1/sqrt(ms+eps)) * w (weight multiplies directly).
    crates/rllm-cpu/src/lib.rs:241-254"""
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(ms + eps)) * w


def linear(x, w):
    """out = x . W^T with W [n_out, k_in], no bias.  crates/rllm-core/src/lib.rs:206,
    crates/rllm-cpu/src/lib.rs:202-239"""
    return x @ w.t()


def rope_neox(x, positions, theta):
    """NeoX / rotate-half rotary embedding over the full head dim.
    x [n, heads, hd]; inv_freq_i = 1/theta^(2i/hd); pairs (i, i+hd/2).
    crates/rllm-cpu/src/lib.rs:256-290"""
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), 2.0 * i / hd)
    ang = torch.as_tensor(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention(q, k, v, scale, window=0):
    """Causal GQA attention over one whole sequence.
    q [n, H, hd], k/v [n, K, hd]; head h reads kv head h // (H/K); token t sees
    keys p with max(0, t+1-window) <= p <= t (window 0: all); softmax in the
    working precision of q.  crates/rllm-cpu/src/lib.rs:389-425"""
    n, H, hd = q.shape
    K = k.shape[1]
    g = H // K
    out = torch.zeros_like(q)
    for h in range(H):
        kh, vh = k[:, h // g, :], v[:, h // g, :]
        s = (q[:, h, :] @ kh.t()) * scale                      # [n, n]
        t = torch.arange(n)[:, None]
        p = torch.arange(n)[None, :]
        visible = p <= t
        if window and window > 0:
            visible = visible & (p >= t + 1 - window)
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        out[:, h, :] = (e / e.sum(-1, keepdim=True)) @ vh
    return out


def swiglu(x, w_gate, w_up, w_down, storage=None):
    """act = gate/(1+exp(-gate)) * up; out = act . Wd^T.
    crates/rllm-core/src/lib.rs:247-262, crates/rllm-cpu/src/lib.rs:292-298"""
    gate = linear(x, w_gate)
    up = linear(x, w_up)
    act = _store(gate / (1.0 + torch.exp(-gate)) * up, storage)
    return linear(act, w_down)


def attention_block(h, positions, w, prefix, cfg, window, storage=None):
    """q/k/v projections, per-head q/k RMSNorm (weight of hd entries shared by all
    heads, same eps as the layer norms, before RoPE), RoPE on q and k, attention,
    output projection.  crates/rllm-model/src/qwen3.rs:195-201,
    crates/rllm-core/src/lib.rs:459-476"""
    n = h.shape[0]
    H, K = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps = cfg["rms_norm_eps"]
    theta = _rope_theta(cfg)
    q = linear(h, w[prefix + "self_attn.q_proj.weight"]).view(n, H, hd)
    k = linear(h, w[prefix + "self_attn.k_proj.weight"]).view(n, K, hd)
    v = linear(h, w[prefix + "self_attn.v_proj.weight"]).view(n, K, hd)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    q = _store(rope_neox(q, positions, theta), storage)
    k = _store(rope_neox(k, positions, theta), storage)
    v = _store(v, storage)
    a = _store(attention(q, k, v, 1.0 / math.sqrt(hd), window), storage)
    return linear(a.reshape(n, H * hd), w[prefix + "self_attn.o_proj.weight"])


def _rope_theta(cfg):
    if "rope_theta" in cfg and cfg["rope_theta"] is not None:
        return cfg["rope_theta"]
    rp = cfg.get("rope_parameters") or {}
    return rp.get("rope_theta", 1_000_000.0)


def layer_windows(cfg):
    """Window per layer (0 = all keys).  Windows exist only when `use_sliding_window` is
    true; then a layer attends through a window of `sliding_window` keys when
    `layer_types[i] == "sliding_attention"`, or, without that list, when
    i >= `max_window_layers`.
    The window rule itself (keys pos+1-window..pos) is crates/rllm-cpu/src/lib.rs:402."""
    L = cfg["num_hidden_layers"]
    sw = (cfg.get("sliding_window") or 0) if cfg.get("use_sliding_window") else 0
    types = cfg.get("layer_types")
    if types is not None:
        return [sw if t == "sliding_attention" else 0 for t in types]
    if sw:
        mwl = cfg.get("max_window_layers", L)
        return [sw if i >= mwl else 0 for i in range(L)]
    return [0] * L


def forward(cfg, w, tokens, storage=None):
    """Logits [n, vocab] for one whole sequence; pre-norm decoder:
    x += attn(norm1(x)); x += ffn(norm2(x)); logits = lm_head(final_norm(x)),
    lm_head tied to the embedding when the tensor is absent.
    crates/rllm-model/src/qwen3.rs:162-234"""
    n = len(tokens)
    positions = list(range(n))
    eps = cfg["rms_norm_eps"]
    windows = layer_windows(cfg)
    x = embed(w["model.embed_tokens.weight"], tokens)
    for li in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{li}."
        h = _store(rms_norm(x, w[p + "input_layernorm.weight"], eps), storage)
        x = x + attention_block(h, positions, w, p, cfg, windows[li], storage)
        h = _store(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), storage)
        x = x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"], storage)
    x = _store(rms_norm(x, w["model.norm.weight"], eps), storage)
    head = w.get("lm_head.weight")
    if head is None:
        head = w["model.embed_tokens.weight"]
    return linear(x, head)


def greedy_generate(cfg, w, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence each step; argmax takes
    the lowest index on ties.  crates/rllm-core/src/sample.rs:58-67"""
    toks = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, w, toks)[-1]
        toks.append(int(torch.argmax(logits)))
    return toks[len(prompt):]


# ---------------------------------------------------------------- sampling

_M64 = (1 << 64) - 1


def uniform(seed, counter, token):
    """Counter-hash uniform in (0,1).  crates/rllm-core/src/sample.rs:38-45"""
    z = (seed ^ (counter * 0x9E3779B97F4A7C15) ^ (token * 0xD1B54A32D192ED03)) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return np.float32((np.float32(z >> 40) + np.float32(0.5)) * np.float32(1.0 / (1 << 24)))


def threshold(x, top_k, top_p, steps=40):
    """Bisection thresholds for top-k then top-p.  crates/rllm-core/src/sample.rs:86-109"""
    x = np.asarray(x, dtype=np.float32)
    lo, hi = np.float32(x.min()), np.float32(x.max())
    mx = hi
    thr = np.float32(-np.inf)
    if top_k > 0 and top_k < len(x):
        a, b = lo, hi
        for _ in range(steps):
            mid = np.float32(0.5) * (a + b)
            if int((x >= mid).sum()) >= top_k:
                a = mid
            else:
                b = mid
        thr = a
        lo = a
    if top_p < 1.0:
        def mass(t):
            sel = x[x >= t]
            return np.float32(np.exp(sel - mx, dtype=np.float32).sum(dtype=np.float32))
        total = mass(thr)
        a, b = lo, hi
        for _ in range(steps):
            mid = np.float32(0.5) * (a + b)
            if mass(mid) >= np.float32(top_p) * total:
                a = mid
            else:
                b = mid
        thr = a
    return thr


def sample_row(logits, temperature, top_k, top_p, seed, counter, adjust=()):
    """Greedy for temperature <= 0, else Gumbel-max over the thresholded candidates; `adjust`
    ((token, delta) pairs: logit bias, penalties) is added to a copy of the row first.
    crates/rllm-core/src/sample.rs:53-83"""
    x = np.asarray(logits, dtype=np.float32).copy()
    for t, d in adjust:
        if 0 <= t < x.size:
            x[t] += np.float32(d)
    if temperature <= 0:
        return int(np.argmax(x))
    x = x * np.float32(1.0 / temperature)
    thr = threshold(x, top_k, top_p)
    best, best_i = -np.inf, 0
    for i in np.nonzero(x >= thr)[0]:
        u = uniform(seed, counter, int(i))
        key = x[i] + np.float32(-np.log(-np.log(u)))
        if key > best:
            best, best_i = key, int(i)
    return best_i
