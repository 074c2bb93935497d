"""Typed model configuration read from a model folder's config.json.

The reference keeps every size as a constexpr in its model file
(model/llm/tiny_llama.cpp:17-21); here the same quantities come from the
architecture's own config.json keys and nothing else.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, Dict, Optional, Type


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine builds."""


_MISSING = object()


def _take(d: Dict[str, Any], key: str, kind, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if kind is int and isinstance(v, bool):
        raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
    if not isinstance(v, kind):
        raise ConfigError(f"config.json: key '{key}' must be {kind.__name__}, got {v!r}")
    return v


@dataclass(frozen=True)
class LlamaConfig:
    """config.json of a LlamaForCausalLM folder (pre-norm, RMSNorm, GQA with
    rotate-half RoPE, SwiGLU; biases on the attention and feed-forward projections if
    attention_bias / mlp_bias say so, as the reference's modules take them,
    model/modules/Attention.h:16-19, MLP.h:9-13)."""

    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    sliding_window: Optional[int] = None
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
        hidden = _take(d, "hidden_size", int)
        heads = _take(d, "num_attention_heads", int)
        if heads <= 0 or hidden <= 0:
            raise ConfigError("config.json: hidden_size and num_attention_heads must be positive")
        kv_heads = _take(d, "num_key_value_heads", int, heads)
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _take(d, "head_dim", int)
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads "
                    f"{heads} and no head_dim is given")
            head_dim = hidden // heads
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = cls(
            architecture=archs[0],
            hidden_size=hidden,
            intermediate_size=_take(d, "intermediate_size", int),
            num_hidden_layers=_take(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_take(d, "vocab_size", int),
            rms_norm_eps=_take(d, "rms_norm_eps", float),
            rope_theta=_take(d, "rope_theta", float, 10000.0),
            max_position_embeddings=_take(d, "max_position_embeddings", int),
            tie_word_embeddings=_take(d, "tie_word_embeddings", bool, False),
            hidden_act=_take(d, "hidden_act", str, "silu"),
            attention_bias=_take(d, "attention_bias", bool, False),
            mlp_bias=_take(d, "mlp_bias", bool, False),
            sliding_window=_take(d, "sliding_window", int, None),
            bos_token_id=_take(d, "bos_token_id", int, None),
            eos_token_id=eos,
            torch_dtype=_take(d, "torch_dtype", str, d.get("dtype")),
        )
        if d.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling is not supported (must be null or absent)")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for f in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"config.json: {f} must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotate-half RoPE")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (silu only)")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError("config.json: sliding_window must be positive or null")

    def to_dict(self) -> Dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "architecture"}
        d = {k: v for k, v in d.items() if v is not None}
        d["architectures"] = [self.architecture]
        return d


@dataclass(frozen=True)
class TevudraConfig:
    """config.json of a Tevudra folder: a decoder whose layers are listed one by one.

    Top level: `architecture`, `width`, `vocab`, `norm.eps`, `layers`.  A layer gives `type` (its
    mixer), `mixer` (the mixer's sizes and constants) and `mlp` (its feed-forward, or null).
    latent_attention mixer: heads, dim, vdim, kv_rank, scale, and kv_from (the layer whose latents
    it reads) where it keeps none of its own.  mlp: {kind: dense, ff} or {kind: moe, expert: {ff},
    router: {experts, top}, shared: {ff} or absent}.  The design has no positions, so no length
    limit of its own: max_position (optional) bounds what the engine sizes its tables for."""

    architecture: str
    width: int
    vocab: int
    norm_eps: float
    layers: tuple                      # of dicts, validated
    max_position: int = 131072
    eos_token_id: Optional[int] = None

    MIXERS = ("latent_attention",)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TevudraConfig":
        norm = _take(d, "norm", dict)
        layers = _take(d, "layers", list)
        if not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = _take(layer, "type", str)
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design {cls.MIXERS}")
            m = _take(layer, "mixer", dict)
            mixer = {k: _take(m, k, int) for k in ("heads", "dim", "vdim", "kv_rank")}
            mixer["scale"] = _take(m, "scale", float)
            mixer["kv_from"] = _take(m, "kv_from", int, None)
            if min(mixer[k] for k in ("heads", "dim", "vdim", "kv_rank")) <= 0:
                raise ConfigError(f"config.json: {where}.mixer sizes must be positive")
            src = mixer["kv_from"]
            if src is not None:
                if not (0 <= src < i) or out[src]["mixer"]["kv_from"] is not None:
                    raise ConfigError(f"config.json: {where}.mixer.kv_from={src} must name an earlier layer that keeps its own latents")
                if out[src]["mixer"]["kv_rank"] != mixer["kv_rank"]:
                    raise ConfigError(f"config.json: {where}.mixer.kv_rank differs from that of layer {src}, whose latents it reads")
            ff = layer.get("mlp")
            mlp = None
            if ff is not None:
                if not isinstance(ff, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                fk = _take(ff, "kind", str)
                if fk == "dense":
                    mlp = {"kind": "dense", "ff": _take(ff, "ff", int)}
                elif fk == "moe":
                    router = _take(ff, "router", dict)
                    shared = ff.get("shared")
                    mlp = {"kind": "moe", "ff": _take(_take(ff, "expert", dict), "ff", int),
                           "experts": _take(router, "experts", int), "top": _take(router, "top", int),
                           "shared_ff": _take(shared, "ff", int) if isinstance(shared, dict) else 0}
                    if not (0 < mlp["top"] <= mlp["experts"]):
                        raise ConfigError(f"config.json: {where}.mlp.router: top {mlp['top']} of {mlp['experts']} experts")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind '{fk}' is not 'dense' or 'moe'")
                if mlp["ff"] <= 0:
                    raise ConfigError(f"config.json: {where}.mlp: ff must be positive")
            out.append({"type": kind, "mixer": mixer, "mlp": mlp})
        eos = d.get("eos_token_id")
        cfg = cls(architecture=_take(d, "architecture", str), width=_take(d, "width", int), vocab=_take(d, "vocab", int),
                  norm_eps=_take(norm, "eps", float), layers=tuple(out),
                  max_position=_take(d, "max_position", int, 131072), eos_token_id=eos if isinstance(eos, int) else None)
        if cfg.width <= 0 or cfg.vocab <= 0 or cfg.max_position <= 0:
            raise ConfigError("config.json: width, vocab and max_position must be positive")
        return cfg

    @property
    def max_position_embeddings(self) -> int:
        return self.max_position


def _moe_of(ff, where: str):
    """{kind: moe, expert: {ff}, router: {experts, top}} -> a flat dict, validated."""
    if not isinstance(ff, dict):
        raise ConfigError(f"config.json: {where}.mlp must be an object or null")
    if _take(ff, "kind", str) != "moe":
        raise ConfigError(f"config.json: {where}.mlp.kind '{ff['kind']}' is not 'moe'")
    router = _take(ff, "router", dict)
    mlp = {"kind": "moe", "ff": _take(_take(ff, "expert", dict), "ff", int),
           "experts": _take(router, "experts", int), "top": _take(router, "top", int)}
    if not (0 < mlp["top"] <= mlp["experts"]) or mlp["ff"] <= 0:
        raise ConfigError(f"config.json: {where}.mlp: top {mlp['top']} of {mlp['experts']} experts of size {mlp['ff']}")
    return mlp


@dataclass(frozen=True)
class FopivikConfig:
    """config.json of a Fopivik folder: a decoder whose layers are listed one by one, part of which may run
    several times in a row.

    Top level: `architecture`, `width`, `vocab`, `norm.eps`, `residual_mult`, `logit_softcap`, `layers`, `loop`
    ({start, stop, times}: layers start..stop-1 run `times` times with the same weights; absent or null: once).
    A layer gives `type` (its mixer: "attention" or "gla"), `mixer` and `mlp` (a mixture of experts
    {kind: moe, expert: {ff}, router: {experts, top}}, or null).  attention: heads, kv_heads, dim, vdim, scale,
    softcap, mask {size, keep_first}, rot {dims, base, scaling {factor, low, high, original} or absent}.
    gla: heads, dim, vdim, tau.  The design has no length limit of its own: max_position (optional) bounds
    what the engine sizes its tables for."""

    architecture: str
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    logit_softcap: float
    layers: tuple                      # of dicts, validated
    loop: Optional[tuple] = None       # (start, stop, times)
    max_position: int = 131072
    eos_token_id: Optional[int] = None

    MIXERS = ("attention", "gla")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FopivikConfig":
        norm = _take(d, "norm", dict)
        layers = _take(d, "layers", list)
        if not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = _take(layer, "type", str)
            m = _take(layer, "mixer", dict)
            if kind == "attention":
                mixer = {k: _take(m, k, int) for k in ("heads", "kv_heads", "dim", "vdim")}
                mixer["scale"] = _take(m, "scale", float)
                mixer["softcap"] = _take(m, "softcap", float)
                mask, rot = _take(m, "mask", dict), _take(m, "rot", dict)
                mixer["window"], mixer["keep_first"] = _take(mask, "size", int), _take(mask, "keep_first", int, 0)
                mixer["rot_dims"], mixer["rot_base"] = _take(rot, "dims", int), _take(rot, "base", float)
                sc = rot.get("scaling")
                mixer["rot_scaling"] = None if sc is None else {k: _take(sc, k, float) for k in ("factor", "low", "high", "original")}
                if min(mixer[k] for k in ("heads", "kv_heads", "dim", "vdim", "window")) <= 0 or mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"config.json: {where}.mixer: sizes must be positive and heads a multiple of kv_heads")
                if mixer["keep_first"] < 0 or mixer["softcap"] <= 0:
                    raise ConfigError(f"config.json: {where}.mixer: keep_first must not be negative and softcap must be positive")
                if mixer["rot_dims"] < 0 or mixer["rot_dims"] % 2 or mixer["rot_dims"] > mixer["dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most dim")
            elif kind == "gla":
                mixer = {k: _take(m, k, int) for k in ("heads", "dim", "vdim")}
                mixer["tau"] = _take(m, "tau", float)
                if min(mixer[k] for k in ("heads", "dim", "vdim")) <= 0 or not mixer["tau"] > 0:
                    raise ConfigError(f"config.json: {where}.mixer: sizes and tau must be positive")
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design {cls.MIXERS}")
            ff = layer.get("mlp")
            out.append({"type": kind, "mixer": mixer, "mlp": None if ff is None else _moe_of(ff, where)})
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object or null")
            loop = (_take(loop, "start", int), _take(loop, "stop", int), _take(loop, "times", int))
            if not (0 <= loop[0] < loop[1] <= len(out)) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {loop} does not name layers of this model, or runs them less than once")
        eos = d.get("eos_token_id")
        cfg = cls(architecture=_take(d, "architecture", str), width=_take(d, "width", int), vocab=_take(d, "vocab", int),
                  norm_eps=_take(norm, "eps", float), residual_mult=_take(d, "residual_mult", float),
                  logit_softcap=_take(d, "logit_softcap", float), layers=tuple(out), loop=loop,
                  max_position=_take(d, "max_position", int, 131072), eos_token_id=eos if isinstance(eos, int) else None)
        if cfg.width <= 0 or cfg.vocab <= 0 or cfg.max_position <= 0 or cfg.logit_softcap <= 0:
            raise ConfigError("config.json: width, vocab, max_position and logit_softcap must be positive")
        return cfg

    @property
    def max_position_embeddings(self) -> int:
        return self.max_position


def _rot_of(m, where: str, limit: int):
    rot = _take(m, "rot", dict)
    dims, base = _take(rot, "dims", int), _take(rot, "base", float)
    if dims < 0 or dims % 2 or dims > limit or not base > 0:
        raise ConfigError(f"config.json: {where}.rot: dims must be even and at most {limit}, base positive")
    return dims, base


@dataclass(frozen=True)
class NorusunConfig:
    """config.json of a Norusun folder: a decoder whose layers are listed one by one, on a residual stream that is
    kept as several copies (hyper-connections), every mixer reading its input through a short causal convolution.

    Top level: `architecture`, `width`, `vocab`, `norm.eps`, `streams`, `canon.taps`, `layers`.  A layer gives `type`
    (its mixer), `mixer` and `mlp` ({kind: dense, ff, limit} or null).
      wkv               heads, dim
      latent_attention  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask.size, rot {dims, base}
      parallel          left  {heads, kv_heads, dim, vdim, scale, mask.size, rot {dims, base}}
                        right {heads, vdim, state, groups, norm_groups, conv}
    The design has no length limit of its own: max_position (optional) bounds what the engine sizes its tables for."""

    architecture: str
    width: int
    vocab: int
    norm_eps: float
    streams: int
    canon_taps: int
    layers: tuple                      # of dicts, validated
    max_position: int = 131072
    eos_token_id: Optional[int] = None

    MIXERS = ("wkv", "latent_attention", "parallel")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "NorusunConfig":
        norm = _take(d, "norm", dict)
        layers = _take(d, "layers", list)
        if not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = _take(layer, "type", str)
            m = _take(layer, "mixer", dict)
            if kind == "wkv":
                mixer = {k: _take(m, k, int) for k in ("heads", "dim")}
                if min(mixer.values()) <= 0:
                    raise ConfigError(f"config.json: {where}.mixer: sizes must be positive")
            elif kind == "latent_attention":
                mixer = {k: _take(m, k, int) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
                mixer["scale"] = _take(m, "scale", float)
                mixer["window"] = _take(_take(m, "mask", dict), "size", int)
                if min(mixer[k] for k in ("heads", "dim", "vdim", "kv_rank", "q_rank", "window")) <= 0 or mixer["rot_dim"] < 0 \
                        or mixer["rot_dim"] % 2:
                    raise ConfigError(f"config.json: {where}.mixer: sizes must be positive and rot_dim even")
                mixer["rot_dims"], mixer["rot_base"] = _rot_of(m, where + ".mixer", mixer["rot_dim"])
            elif kind == "parallel":
                left, right = _take(m, "left", dict), _take(m, "right", dict)
                a = {k: _take(left, k, int) for k in ("heads", "kv_heads", "dim", "vdim")}
                a["scale"] = _take(left, "scale", float)
                a["chunk"] = _take(_take(left, "mask", dict), "size", int)
                if min(a[k] for k in ("heads", "kv_heads", "dim", "vdim", "chunk")) <= 0 or a["heads"] % a["kv_heads"]:
                    raise ConfigError(f"config.json: {where}.mixer.left: sizes must be positive and heads a multiple of kv_heads")
                a["rot_dims"], a["rot_base"] = _rot_of(left, where + ".mixer.left", a["dim"])
                b = {k: _take(right, k, int) for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv")}
                if min(b.values()) <= 0 or b["heads"] % b["groups"] or (b["heads"] * b["vdim"]) % b["norm_groups"]:
                    raise ConfigError(f"config.json: {where}.mixer.right: sizes must be positive, heads a multiple of groups "
                                      f"and heads * vdim a multiple of norm_groups")
                mixer = {"left": a, "right": b}
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design {cls.MIXERS}")
            ff = layer.get("mlp")
            mlp = None
            if ff is not None:
                if not isinstance(ff, dict):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                if _take(ff, "kind", str) != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{ff['kind']}' is not 'dense'")
                mlp = {"kind": "dense", "ff": _take(ff, "ff", int), "limit": _take(ff, "limit", float)}
                if mlp["ff"] <= 0 or not mlp["limit"] > 0:
                    raise ConfigError(f"config.json: {where}.mlp: ff and limit must be positive")
            out.append({"type": kind, "mixer": mixer, "mlp": mlp})
        eos = d.get("eos_token_id")
        cfg = cls(architecture=_take(d, "architecture", str), width=_take(d, "width", int), vocab=_take(d, "vocab", int),
                  norm_eps=_take(norm, "eps", float), streams=_take(d, "streams", int),
                  canon_taps=_take(_take(d, "canon", dict), "taps", int), layers=tuple(out),
                  max_position=_take(d, "max_position", int, 131072), eos_token_id=eos if isinstance(eos, int) else None)
        if cfg.width <= 0 or cfg.vocab <= 0 or cfg.max_position <= 0:
            raise ConfigError("config.json: width, vocab and max_position must be positive")
        if not (1 <= cfg.streams <= 8) or not (1 <= cfg.canon_taps <= 16):
            raise ConfigError("config.json: streams must be 1 to 8 and canon.taps 1 to 16")
        return cfg

    @property
    def max_position_embeddings(self) -> int:
        return self.max_position


@dataclass(frozen=True)
class PotipelConfig:
    """config.json of a Potipel folder: a pre-norm decoder (RMS norms with a weight) whose `layers` list gives every layer
    one by one, with a scaled embedding and a short causal convolution added to what every sublayer reads.  Keys:
    `architecture`, `width`, `vocab`, `norm.eps`, `embedding.scale`, `canon.taps`, and per layer `type`, `mixer`, `mlp`
    (`dense` with `ff`; `moe` with `expert.{ff, limit}` and `router.{experts, top, groups.{count, keep}}`; or null) and,
    optionally, `weights_of`: the index of another layer whose tensors this one uses, with a cache and state of its own.
    Mixers:
      attention  heads, kv_heads, dim, vdim, scale, diff                      (differential attention, two maps per head)
      hgrn2      heads, dim, vdim
      parallel   left  {heads, kv_heads, dim, vdim, scale, softcap, conv, mask.size}      (windowed attention with a sink)
                 right {heads, kv_heads, dim, vdim, conv}                                  (gated delta rule)
                 left_scale, right_scale
    The design has no length limit of its own: max_position (optional) bounds what the engine sizes its tables for."""

    architecture: str
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    canon_taps: int
    layers: tuple                      # of dicts, validated; "weights_of" is None or an index
    max_position: int = 131072
    eos_token_id: Optional[int] = None

    MIXERS = ("attention", "hgrn2", "parallel")

    @staticmethod
    def _ints(d, keys, where):
        out = {k: _take(d, k, int) for k in keys}
        if min(out.values()) <= 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        return out

    @classmethod
    def _mixer(cls, kind: str, m: dict, where: str) -> dict:
        if kind == "attention":
            mixer = cls._ints(m, ("heads", "kv_heads", "dim", "vdim"), where)
            mixer["scale"], mixer["diff"] = _take(m, "scale", float), _take(m, "diff", float)
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"config.json: {where}: heads must be a multiple of kv_heads")
            return mixer
        if kind == "hgrn2":
            return cls._ints(m, ("heads", "dim", "vdim"), where)
        if kind == "parallel":
            left, right = _take(m, "left", dict), _take(m, "right", dict)
            a = cls._ints(left, ("heads", "kv_heads", "dim", "vdim", "conv"), where + ".left")
            a["scale"], a["softcap"] = _take(left, "scale", float), _take(left, "softcap", float)
            a["window"] = _take(_take(left, "mask", dict), "size", int)
            b = cls._ints(right, ("heads", "kv_heads", "dim", "vdim", "conv"), where + ".right")
            if a["heads"] % a["kv_heads"] or b["heads"] % b["kv_heads"] or a["window"] <= 0 or not a["softcap"] > 0:
                raise ConfigError(f"config.json: {where}: heads must be a multiple of kv_heads, the window and the soft cap positive")
            if max(a["conv"], b["conv"]) > 16:
                raise ConfigError(f"config.json: {where}: a convolution has at most 16 taps")
            return {"left": a, "right": b, "left_scale": _take(m, "left_scale", float), "right_scale": _take(m, "right_scale", float)}
        raise ConfigError(f"config.json: {where[:-6]}.type '{kind}' is not a mixer of this design {cls.MIXERS}")

    @staticmethod
    def _mlp(ff, where: str):
        if ff is None:
            return None
        if not isinstance(ff, dict):
            raise ConfigError(f"config.json: {where} must be an object or null")
        kind = _take(ff, "kind", str)
        if kind == "dense":
            mlp = {"kind": "dense", "ff": _take(ff, "ff", int)}
            if mlp["ff"] <= 0:
                raise ConfigError(f"config.json: {where}.ff must be positive")
            return mlp
        if kind == "moe":
            expert, router = _take(ff, "expert", dict), _take(ff, "router", dict)
            groups = _take(router, "groups", dict)
            mlp = {"kind": "moe", "ff": _take(expert, "ff", int), "limit": _take(expert, "limit", float),
                   "experts": _take(router, "experts", int), "top": _take(router, "top", int),
                   "groups": _take(groups, "count", int), "keep": _take(groups, "keep", int)}
            if mlp["ff"] <= 0 or not mlp["limit"] > 0 or not (0 < mlp["top"] <= mlp["experts"] <= 256):
                raise ConfigError(f"config.json: {where}: ff and limit must be positive and 1 <= top <= experts <= 256")
            if mlp["groups"] <= 0 or mlp["experts"] % mlp["groups"] or not (0 < mlp["keep"] <= mlp["groups"]) \
                    or mlp["top"] > mlp["keep"] * (mlp["experts"] // mlp["groups"]):
                raise ConfigError(f"config.json: {where}.router: {mlp['experts']} experts must divide into groups.count groups, "
                                  f"1 <= keep <= count, and top fit into the kept groups")
            return mlp
        raise ConfigError(f"config.json: {where}.kind '{kind}' is not 'dense' or 'moe'")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PotipelConfig":
        norm = _take(d, "norm", dict)
        layers = _take(d, "layers", list)
        if not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = _take(layer, "type", str)
            entry = {"type": kind, "mixer": cls._mixer(kind, _take(layer, "mixer", dict), where + ".mixer"),
                     "mlp": cls._mlp(layer.get("mlp"), where + ".mlp"), "weights_of": None}
            src = layer.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not (0 <= src < len(layers)) or src == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer")
                entry["weights_of"] = src
            out.append(entry)
        for i, entry in enumerate(out):          # a layer may name one that names another: the tensors are the last one's
            src, seen = entry["weights_of"], {i}
            while src is not None and out[src]["weights_of"] is not None:
                if src in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
                seen.add(src)
                src = out[src]["weights_of"]
            if src is not None and src in seen:
                raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
            entry["weights_of"] = src
            if src is not None and {k: v for k, v in out[src].items() if k != "weights_of"} != \
                    {k: v for k, v in entry.items() if k != "weights_of"}:
                raise ConfigError(f"config.json: layers[{i}] uses the tensors of layer {src} but differs from it")
        eos = d.get("eos_token_id")
        cfg = cls(architecture=_take(d, "architecture", str), width=_take(d, "width", int), vocab=_take(d, "vocab", int),
                  norm_eps=_take(norm, "eps", float), embedding_scale=_take(_take(d, "embedding", dict), "scale", float),
                  canon_taps=_take(_take(d, "canon", dict), "taps", int), layers=tuple(out),
                  max_position=_take(d, "max_position", int, 131072), eos_token_id=eos if isinstance(eos, int) else None)
        if cfg.width <= 0 or cfg.vocab <= 0 or cfg.max_position <= 0:
            raise ConfigError("config.json: width, vocab and max_position must be positive")
        if not (1 <= cfg.canon_taps <= 16):
            raise ConfigError("config.json: canon.taps must be 1 to 16")
        return cfg

    @property
    def max_position_embeddings(self) -> int:
        return self.max_position


@dataclass(frozen=True)
class Architecture:
    """One registry entry: how to read the config and how to lay the model out."""

    name: str
    config_class: Type
    build_spec: Callable  # (config) -> llm_b200.models.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type, build_spec: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture '{name}'; registered: {known}")
    return _ARCHITECTURES[name]


def registered_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    # Importing the models package registers the built-in architectures.
    import llm_b200.models  # noqa: F401


def parse_config(d: Dict[str, Any]):
    """config.json contents -> (Architecture, typed config).  The architecture is the first name of
    the list `architectures`, or the string `architecture`."""
    archs = d.get("architectures")
    if archs is None and isinstance(d.get("architecture"), str):
        archs = [d["architecture"]]
    if not isinstance(archs, list) or not archs:
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names (or 'architecture' a name)")
    arch = get_architecture(archs[0])
    return arch, arch.config_class.from_dict(d)


def load_config(model_dir: str):
    """Read <model_dir>/config.json -> (Architecture, typed config)."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: invalid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return parse_config(d)
