"""Typed configuration of the Llama dense decoder, read from its own config.json keys.

The reference parses twelve keys into ``HFConfig`` and then drops rope_theta and
rms_norm_eps on the way to the C struct (internal/model/hf_config.go:10-55,
internal/backend/cuda/model_bridge.go:44-56).  Here every size and constant of
the model comes from config.json; nothing is a literal in code.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a key of the wrong type, or is inconsistent."""


def _need(d: dict, key: str, typ=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if typ is int and (isinstance(v, bool) or not isinstance(v, int)):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if typ is int and v <= 0:
        raise ConfigError(f"config.json: '{key}' must be positive, got {v}")
    return v


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` object of config.json. ``rope_type`` (or the older key
    ``type``) is one of "llama3", "linear", "default"."""
    rope_type: str
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_position_embeddings: int = 0

    @staticmethod
    def from_dict(d: Optional[dict]) -> Optional["RopeScaling"]:
        if not d:
            return None
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind == "linear":
            if "factor" not in d:
                raise ConfigError("config.json: rope_scaling 'linear' needs 'factor'")
            return RopeScaling("linear", factor=float(d["factor"]))
        if kind == "llama3":
            keys = ("factor", "low_freq_factor", "high_freq_factor",
                    "original_max_position_embeddings")
            missing = [k for k in keys if k not in d]
            if missing:
                raise ConfigError(f"config.json: rope_scaling 'llama3' lacks {missing}")
            if float(d["high_freq_factor"]) == float(d["low_freq_factor"]):
                raise ConfigError("config.json: rope_scaling high_freq_factor == low_freq_factor")
            return RopeScaling("llama3", float(d["factor"]), float(d["low_freq_factor"]),
                               float(d["high_freq_factor"]),
                               int(d["original_max_position_embeddings"]))
        raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported "
                          f"(known: llama3, linear, default)")


@dataclass(frozen=True)
class LlamaConfig:
    """config.json of ``LlamaForCausalLM`` (key names are the file's own)."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    hidden_act: str
    rope_interleaved: bool                 # adjacent pairs, the reference's kernel; default half-split
    sliding_window: Optional[int]          # optional: window of the layers marked sliding
    layer_types: tuple                     # per layer "full_attention" | "sliding_attention"
    bos_token_id: Optional[int]
    eos_token_ids: tuple
    torch_dtype: str
    architectures: tuple = field(default=("LlamaForCausalLM",))

    @staticmethod
    def from_dict(d: dict) -> "LlamaConfig":
        H = _need(d, "hidden_size")
        nh = _need(d, "num_attention_heads")
        nkv = d.get("num_key_value_heads") or nh      # 0/absent => MHA (cmd/gollmgo/gpu.go:87-89)
        hd = d.get("head_dim")
        if hd is None:
            if H % nh:
                raise ConfigError(f"config.json: hidden_size {H} is not a multiple of "
                                  f"num_attention_heads {nh} and no head_dim is given")
            hd = H // nh
        if not isinstance(nkv, int) or nkv <= 0 or nh % nkv:
            raise ConfigError(f"config.json: num_attention_heads {nh} is not a multiple of "
                              f"num_key_value_heads {nkv}")
        if not isinstance(hd, int) or hd <= 0 or hd % 2:
            raise ConfigError(f"config.json: head_dim {hd} must be a positive even integer")
        for k in ("attention_bias", "mlp_bias"):
            if d.get(k):
                raise ConfigError(f"config.json: {k}=true is not supported by this engine")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (known: silu)")
        L = _need(d, "num_hidden_layers")
        win = d.get("sliding_window") or None
        types = d.get("layer_types")
        if types is None:
            types = ["sliding_attention" if win else "full_attention"] * L
        if len(types) != L:
            raise ConfigError(f"config.json: layer_types has {len(types)} entries for {L} layers")
        for t in types:
            if t not in ("full_attention", "sliding_attention"):
                raise ConfigError(f"config.json: layer type {t!r} is not known")
            if t == "sliding_attention" and not win:
                raise ConfigError("config.json: a sliding_attention layer needs 'sliding_window'")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        eps = d.get("rms_norm_eps", 1e-5)       # the reference's fallback: kernels/gollmgo_model.cu:322-324
        if not (isinstance(eps, float) or isinstance(eps, int)) or eps <= 0:
            raise ConfigError(f"config.json: rms_norm_eps {eps!r} must be a positive number")
        return LlamaConfig(
            vocab_size=_need(d, "vocab_size"), hidden_size=H,
            intermediate_size=_need(d, "intermediate_size"), num_hidden_layers=L,
            num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            rms_norm_eps=float(eps), rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=act, rope_interleaved=bool(d.get("rope_interleaved", False)),
            sliding_window=int(win) if win else None, layer_types=tuple(types),
            bos_token_id=d.get("bos_token_id"), eos_token_ids=eos_ids,
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            architectures=tuple(d.get("architectures") or ("LlamaForCausalLM",)))


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
    try:
        with open(path) as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
