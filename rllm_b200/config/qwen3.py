"""Qwen3 dense: typed configuration from config.json and the model it describes.

A pre-norm decoder: RMSNorm, grouped-query attention with a per-head RMSNorm on
queries and keys, rotate-half rotary embedding, SwiGLU feed-forward, optionally
tied embeddings, no biases (AxiomOperator/rllm: crates/rllm-model/src/qwen3.rs:1-8,
fields 17-33, defaults 36-76).  The reference reads the same quantities from GGUF
metadata; here they come from the keys a Qwen3 config.json carries.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .base import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, coerce,
                   optional, require)


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    layer_windows: tuple          # per layer: number of keys seen, 0 = all
    sliding_window: int = 0       # as given in config.json (0: none)
    use_sliding_window: bool = False
    max_window_layers: int = 0
    architecture: str = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        H = require(d, "num_attention_heads", int)
        hidden = require(d, "hidden_size", int)
        L = require(d, "num_hidden_layers", int)
        K = optional(d, "num_key_value_heads", int, H)
        hd = optional(d, "head_dim", int, None)
        if hd is None:
            if hidden % H:
                raise ConfigError(f"config.json: 'head_dim' is absent and hidden_size {hidden} is not "
                                  f"a multiple of num_attention_heads {H}")
            hd = hidden // H
        # rope_theta may sit at the top level or inside rope_parameters
        rp = d.get("rope_parameters") or {}
        theta = d.get("rope_theta")
        if theta is None:
            theta = rp.get("rope_theta", 1_000_000.0)
        theta = coerce(theta, "rope_theta", float)
        for key, src in (("rope_scaling", d), ("rope_parameters", d)):
            sc = src.get(key)
            if isinstance(sc, Mapping):
                typ = sc.get("rope_type", sc.get("type", "default"))
                if typ not in (None, "default", "none"):
                    raise ConfigError(f"config.json: '{key}' of type {typ!r} is not supported "
                                      f"(only unscaled rotary embedding)")
                if sc.get("factor") not in (None, 1, 1.0):
                    raise ConfigError(f"config.json: '{key}.factor' = {sc.get('factor')!r} is not supported")
        if optional(d, "attention_bias", bool, False):
            raise ConfigError("config.json: 'attention_bias' = true is not supported (Qwen3 has no biases)")
        act = optional(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' = {act!r} is not supported (silu only)")
        # A window applies only when `use_sliding_window` is true: checkpoints carry a
        # `sliding_window` number beside `use_sliding_window: false`, which means no window.
        use_sw = optional(d, "use_sliding_window", bool, False)
        sw = optional(d, "sliding_window", int, 0) if use_sw else 0
        mwl = optional(d, "max_window_layers", int, L)
        types = d.get("layer_types")
        if types is not None:
            if not isinstance(types, (list, tuple)) or len(types) != L:
                raise ConfigError(f"config.json: 'layer_types' must list {L} entries")
            windows = []
            for i, t in enumerate(types):
                if t == "full_attention":
                    windows.append(0)
                elif t == "sliding_attention":
                    windows.append(sw)          # 0 when windows are switched off
                else:
                    raise ConfigError(f"config.json: 'layer_types[{i}]' = {t!r} is not supported")
        elif sw > 0:
            windows = [sw if i >= mwl else 0 for i in range(L)]
        else:
            windows = [0] * L
        cfg = cls(
            vocab_size=require(d, "vocab_size", int), hidden_size=hidden,
            intermediate_size=require(d, "intermediate_size", int), num_hidden_layers=L,
            num_attention_heads=H, num_key_value_heads=K, head_dim=hd,
            rms_norm_eps=optional(d, "rms_norm_eps", float, 1e-6), rope_theta=theta,
            max_position_embeddings=optional(d, "max_position_embeddings", int, 32768),
            tie_word_embeddings=optional(d, "tie_word_embeddings", bool, False),
            layer_windows=tuple(windows), sliding_window=sw, use_sliding_window=use_sw,
            max_window_layers=mwl)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"config.json: '{key}' must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ConfigError(f"config.json: 'head_dim' {self.head_dim} must be a multiple of 16 and at most 256 "
                              f"(the kernels take head sizes from 16 to 256 in steps of 16)")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: 'rms_norm_eps' must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("config.json: 'rope_theta' must be positive")
        if len(self.layer_windows) != self.num_hidden_layers:
            raise ConfigError("layer_windows must have one entry per layer")

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture], "model_type": "qwen3",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "hidden_act": "silu", "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "rope_scaling": None, "attention_bias": False,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window if self.sliding_window else None,
            "max_window_layers": self.max_window_layers,
        }
        if any(self.layer_windows):
            d["layer_types"] = ["sliding_attention" if w else "full_attention" for w in self.layer_windows]
        return d

    # ------------------------------------------------------------------ the model as data
    def model_spec(self) -> ModelSpec:
        norm = lambda prefix: PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.rms_norm_eps}, prefix)
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            layers.append(LayerSpec(
                block="pre_norm",
                mixer=PartSpec("attention", {
                    "hidden_size": self.hidden_size, "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                    "qk_norm": True, "qk_norm_eps": self.rms_norm_eps,
                    "window": self.layer_windows[i],
                    "scale": self.head_dim ** -0.5}, p + "self_attn."),
                ffn=PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                        "intermediate_size": self.intermediate_size}, p + "mlp."),
                norms={"mixer": norm(p + "input_layernorm."), "ffn": norm(p + "post_attention_layernorm.")},
                position=PartSpec("rotary_neox", {"head_dim": self.head_dim, "theta": self.rope_theta}),
            ))
        return ModelSpec(
            vocab_size=self.vocab_size, hidden_size=self.hidden_size,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size},
                               "model.embed_tokens."),
            layers=tuple(layers),
            run_order=tuple(RunEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=norm("model.norm."),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                                         "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None},
                             "lm_head."),
            max_position=self.max_position_embeddings,
        )
