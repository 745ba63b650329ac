"""Typed model configurations, read from an architecture's own ``config.json`` keys.

Every size and constant of a model comes from here; nothing in the parts or the kernels
stands in for a value that ``config.json`` gives.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A ``config.json`` that is incomplete, of the wrong type, or outside what the engine runs."""


_MISSING = object()


def _take(d: Dict[str, Any], key: str, kind, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key '{key}'")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
        return v
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {v!r}")
        return v
    return v


@dataclass(frozen=True)
class Qwen3Config:
    """``config.json`` of ``Qwen3ForCausalLM``.

    Same keys, defaults and refusals as the reference's ``Qwen3Config``
    (models/qwen3/src/config.rs:6-56): the first ten keys have no default; ``head_dim`` is
    explicit and may differ from ``hidden_size / num_attention_heads``; attention bias, a
    sliding window and activations other than silu are refused.
    """

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
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    sliding_window: Optional[int] = None
    use_sliding_window: bool = False
    hidden_act: str = "silu"
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        eos = d.get("eos_token_id")
        if isinstance(eos, bool):
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(x) for x in eos if isinstance(x, int) and not isinstance(x, bool))
        else:
            eos_ids = ()
        if d.get("rope_scaling") not in (None, {}):
            rs = d["rope_scaling"]
            kind = rs.get("rope_type", rs.get("type")) if isinstance(rs, dict) else rs
            if kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling {kind!r} is not supported")
        archs = d.get("architectures") or ["Qwen3ForCausalLM"]
        cfg = cls(
            vocab_size=_take(d, "vocab_size", int),
            hidden_size=_take(d, "hidden_size", int),
            intermediate_size=_take(d, "intermediate_size", int),
            num_hidden_layers=_take(d, "num_hidden_layers", int),
            num_attention_heads=_take(d, "num_attention_heads", int),
            num_key_value_heads=_take(d, "num_key_value_heads", int),
            head_dim=_take(d, "head_dim", int),
            rms_norm_eps=_take(d, "rms_norm_eps", float),
            rope_theta=_take(d, "rope_theta", float),
            max_position_embeddings=_take(d, "max_position_embeddings", int),
            tie_word_embeddings=_take(d, "tie_word_embeddings", bool, False),
            attention_bias=_take(d, "attention_bias", bool, False),
            sliding_window=_take(d, "sliding_window", int, None),
            use_sliding_window=_take(d, "use_sliding_window", bool, False),
            hidden_act=_take(d, "hidden_act", str, "silu"),
            eos_token_ids=eos_ids,
            architecture=str(archs[0]),
        )
        cfg.check()
        return cfg

    def check(self) -> None:
        for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "num_key_value_heads", "head_dim",
                  "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"config.json: '{f}' must be positive, got {getattr(self, f)}")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: unsupported hidden_act {self.hidden_act!r}")
        if self.attention_bias:
            raise ConfigError("config.json: attention_bias is not supported")
        if self.use_sliding_window:
            raise ConfigError("config.json: sliding window is not supported")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: heads {self.num_attention_heads} not divisible by kv heads "
                f"{self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even (rotary pairs)")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")

    # derived sizes (models/qwen3/src/config.rs:66-77)
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def to_dict(self) -> Dict[str, Any]:
        """The ``config.json`` dictionary that reads back as this configuration."""
        d: Dict[str, Any] = {"architectures": [self.architecture], "model_type": "qwen3"}
        for f in fields(self):
            if f.name in ("eos_token_ids", "architecture"):
                continue
            d[f.name] = getattr(self, f.name)
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    _merge_generation_eos(model_dir, d)
    return d


def _merge_generation_eos(model_dir: str, d: Dict[str, Any]) -> None:
    """End-of-sequence ids that only ``generation_config.json`` names join those of config.json
    (the reference takes its stop ids from the generation config too: crates/server/src/service.rs:407)."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return
    with open(path, "r", encoding="utf-8") as f:
        try:
            g = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    extra = g.get("eos_token_id") if isinstance(g, dict) else None
    if extra is None:
        return
    def as_list(v):
        return [] if v is None else (list(v) if isinstance(v, (list, tuple)) else [v])
    have = as_list(d.get("eos_token_id"))
    merged = have + [t for t in as_list(extra) if t not in have]
    if not all(isinstance(t, int) and not isinstance(t, bool) for t in merged):
        raise ConfigError(f"{path}: eos_token_id must be an integer or a list of integers")
    d["eos_token_id"] = merged if len(merged) != 1 else merged[0]


# ---------------------------------------------------------------- Dobedra

def _section(d: Dict[str, Any], key: str, where: str, optional: bool = False) -> Optional[Dict[str, Any]]:
    v = d.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"config.json: {where}missing section '{key}'")
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


@dataclass(frozen=True)
class LatentAttentionSizes:
    """One ``latent_attention`` mixer: ``heads`` heads of ``dim`` unrotated + ``rot_dim`` rotated query/key
    elements and ``vdim`` value elements over a key/value latent of ``kv_rank`` (queries through one of
    ``q_rank``); ``kv_from``: the layer whose latent cache this one reads instead of keeping one."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "LatentAttentionSizes":
        rot = _section(m, "rot", where)
        s = cls(heads=_take(m, "heads", int), dim=_take(m, "dim", int), rot_dim=_take(m, "rot_dim", int),
                vdim=_take(m, "vdim", int), kv_rank=_take(m, "kv_rank", int), q_rank=_take(m, "q_rank", int),
                scale=_take(m, "scale", float), rot_base=_take(rot, "base", float),
                rot_dims=_take(rot, "dims", int), kv_from=_take(m, "kv_from", int, None))
        for f in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
            if getattr(s, f) <= 0:
                raise ConfigError(f"config.json: {where}'{f}' must be positive, got {getattr(s, f)}")
        if s.rot_dims <= 0 or s.rot_dims % 2 or s.rot_dims > s.rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims {s.rot_dims} must be even and at most rot_dim {s.rot_dim}")
        if not s.rot_base > 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
        return s


@dataclass(frozen=True)
class FeedForwardSizes:
    """``kind`` "dense" (gated, ``ff`` wide) or "moe" (``experts`` experts ``ff`` wide of which a token uses
    ``top``; ``shared_ff`` > 0: a shared expert of that width runs for every token)."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "FeedForwardSizes":
        kind = _take(m, "kind", str)
        if kind == "dense":
            s = cls("dense", _take(m, "ff", int))
        elif kind == "moe":
            router = _section(m, "router", where)
            shared = _section(m, "shared", where, optional=True)
            s = cls("moe", _take(_section(m, "expert", where), "ff", int), experts=_take(router, "experts", int),
                    top=_take(router, "top", int), shared_ff=_take(shared, "ff", int) if shared else 0)
            if not (0 < s.top <= s.experts):
                raise ConfigError(f"config.json: {where}router.top {s.top} must be between 1 and experts {s.experts}")
            if s.shared_ff < 0:
                raise ConfigError(f"config.json: {where}shared.ff must not be negative")
        else:
            raise ConfigError(f"config.json: {where}unknown mlp.kind {kind!r} (dense, moe)")
        if s.ff <= 0:
            raise ConfigError(f"config.json: {where}ff must be positive, got {s.ff}")
        return s


@dataclass(frozen=True)
class DobedraLayer:
    type: str
    mixer: LatentAttentionSizes
    mlp: Optional[FeedForwardSizes]


@dataclass(frozen=True)
class DobedraConfig:
    """``config.json`` of a Dobedra model: ``vocab``, ``width``, ``norm.eps``, ``logit_softcap`` and the list
    ``layers``, each entry with its ``type`` (the mixer it has), the mixer's sizes and its feed-forward (or none).
    ``max_positions`` is optional: the design has no longest sequence of its own, the engine's ``max_model_len``
    sizes the angle tables."""
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float
    layers: Tuple[DobedraLayer, ...]
    max_positions: int = 1 << 20
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Dobedra"

    MIXER_TYPES = ("latent_attention",)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DobedraConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]: "
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: {where}must be an object")
            kind = _take(l, "type", str)
            if kind not in cls.MIXER_TYPES:
                raise ConfigError(f"config.json: {where}unknown type {kind!r} ({', '.join(cls.MIXER_TYPES)})")
            mixer = LatentAttentionSizes.from_dict(_section(l, "mixer", where), where)
            mlp = _section(l, "mlp", where, optional=True)
            layers.append(DobedraLayer(kind, mixer, FeedForwardSizes.from_dict(mlp, where) if mlp else None))
        eos = d.get("eos_token_id")
        eos_ids = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ()
        cfg = cls(vocab=_take(d, "vocab", int), width=_take(d, "width", int),
                  norm_eps=_take(_section(d, "norm", ""), "eps", float),
                  logit_softcap=_take(d, "logit_softcap", float, 0.0), layers=tuple(layers),
                  max_positions=_take(d, "max_positions", int, 1 << 20), eos_token_ids=eos_ids,
                  architecture=str(d.get("architecture") or (d.get("architectures") or ["Dobedra"])[0]))
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 1:
            raise ConfigError("config.json: vocab, width and max_positions must be positive")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {self.norm_eps}")
        if self.logit_softcap < 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        for i, l in enumerate(self.layers):
            j = l.mixer.kv_from
            if j is None:
                continue
            if not (0 <= j < i) or self.layers[j].mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}]: kv_from {j} must name an earlier layer that has a "
                                  f"key/value down projection of its own")
            a, b = l.mixer, self.layers[j].mixer
            if (a.kv_rank, a.rot_dim, a.rot_dims, a.rot_base) != (b.kv_rank, b.rot_dim, b.rot_dims, b.rot_base):
                raise ConfigError(f"config.json: layers[{i}]: kv_rank, rot_dim and rotation must equal those of "
                                  f"layer {j}, whose latents it reads")

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for l in self.layers:
            m = l.mixer
            mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                     "q_rank": m.q_rank, "scale": m.scale, "rot": {"base": m.rot_base, "dims": m.rot_dims}}
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            f = l.mlp
            if f is None:
                mlp = None
            elif f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "logit_softcap": self.logit_softcap, "layers": layers}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


# ---------------------------------------------------------------- Zasipel

@dataclass(frozen=True)
class WindowAttentionSizes:
    """Grouped-query attention over a sliding window with a sink: ``heads`` query heads and ``kv_heads`` key/value
    heads of ``dim`` (queries, keys) and ``vdim`` (values) elements; the first ``rot_dims`` elements of a head rotate
    (pairs 2i, 2i + 1; base ``rot_base``); a query sees itself and the ``window - 1`` tokens before it."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_base: float
    rot_dims: int

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "WindowAttentionSizes":
        rot, mask = _section(m, "rot", where), _section(m, "mask", where)
        s = cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                vdim=_take(m, "vdim", int), scale=_take(m, "scale", float), window=_take(mask, "size", int),
                rot_base=_take(rot, "base", float), rot_dims=_take(rot, "dims", int))
        for f in ("heads", "kv_heads", "dim", "vdim", "window"):
            if getattr(s, f) <= 0:
                raise ConfigError(f"config.json: {where}'{f}' must be positive, got {getattr(s, f)}")
        if s.heads % s.kv_heads:
            raise ConfigError(f"config.json: {where}heads {s.heads} must be a multiple of kv_heads {s.kv_heads}")
        if s.rot_dims <= 0 or s.rot_dims % 2 or s.rot_dims > s.dim:
            raise ConfigError(f"config.json: {where}rot.dims {s.rot_dims} must be even and at most dim {s.dim}")
        if not s.rot_base > 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
        return s

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "mask": {"size": self.window}, "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class DeltaRuleSizes:
    """A gated delta-rule mixer: ``heads`` value heads of ``vdim``, ``kv_heads`` query/key heads of ``dim``, short
    convolutions of ``conv`` taps.  ``decay_rank`` / ``gate_rank``: the thin middle of the per-channel form's decay and
    gate projections; the weight file decides them unless the configuration names them (optional keys, which the
    random-weights mode needs)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int = -1
    gate_rank: int = -1

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "DeltaRuleSizes":
        s = cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                vdim=_take(m, "vdim", int), conv=_take(m, "conv", int), decay_rank=_take(m, "decay_rank", int, -1),
                gate_rank=_take(m, "gate_rank", int, -1))
        for f in ("heads", "kv_heads", "dim", "vdim", "conv"):
            if getattr(s, f) <= 0:
                raise ConfigError(f"config.json: {where}'{f}' must be positive, got {getattr(s, f)}")
        if s.heads % s.kv_heads:
            raise ConfigError(f"config.json: {where}heads {s.heads} must be a multiple of kv_heads {s.kv_heads}")
        if s.decay_rank == 0 or s.gate_rank == 0 or s.decay_rank < -1 or s.gate_rank < -1:
            raise ConfigError(f"config.json: {where}decay_rank and gate_rank must be positive where given")
        return s

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank > 0:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank > 0:
            d["gate_rank"] = self.gate_rank
        return d


@dataclass(frozen=True)
class ZasipelLayer:
    """``type`` "parallel": ``left`` (window attention) and ``right`` (delta rule, one decay a head) side by side;
    "channel_delta": ``right`` alone in its per-channel form.  ``mlp``: a routed feed-forward or none."""
    type: str
    left: Optional[WindowAttentionSizes]
    right: DeltaRuleSizes
    mlp: Optional[FeedForwardSizes]


@dataclass(frozen=True)
class ZasipelConfig:
    """``config.json`` of a Zasipel model: ``vocab``, ``width``, ``norm.eps`` and the list ``layers``, each entry with
    its ``type`` (the mixer it has), the mixer's sizes and its feed-forward (``mlp``: a mixture of experts chosen
    by a table, or null).  ``max_positions`` is optional: the design has no longest sequence of its own."""
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZasipelLayer, ...]
    max_positions: int = 1 << 20
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Zasipel"

    MIXER_TYPES = ("parallel", "channel_delta")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ZasipelConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]: "
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: {where}must be an object")
            kind = _take(l, "type", str)
            if kind not in cls.MIXER_TYPES:
                raise ConfigError(f"config.json: {where}unknown type {kind!r} ({', '.join(cls.MIXER_TYPES)})")
            mixer = _section(l, "mixer", where)
            if kind == "parallel":
                left = WindowAttentionSizes.from_dict(_section(mixer, "left", where), where + "left: ")
                right = DeltaRuleSizes.from_dict(_section(mixer, "right", where), where + "right: ")
            else:
                left, right = None, DeltaRuleSizes.from_dict(mixer, where)
            mlp = _section(l, "mlp", where, optional=True)
            ff = FeedForwardSizes.from_dict(mlp, where) if mlp else None
            if ff is not None and ff.kind != "moe":
                raise ConfigError(f"config.json: {where}mlp.kind {ff.kind!r}: the design's feed-forward is a mixture of experts")
            layers.append(ZasipelLayer(kind, left, right, ff))
        eos = d.get("eos_token_id")
        eos_ids = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ()
        cfg = cls(vocab=_take(d, "vocab", int), width=_take(d, "width", int),
                  norm_eps=_take(_section(d, "norm", ""), "eps", float), layers=tuple(layers),
                  max_positions=_take(d, "max_positions", int, 1 << 20), eos_token_ids=eos_ids,
                  architecture=str(d.get("architecture") or (d.get("architectures") or ["Zasipel"])[0]))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 1:
            raise ConfigError("config.json: vocab, width and max_positions must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {cfg.norm_eps}")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for l in self.layers:
            mixer = {"left": l.left.to_dict(), "right": l.right.to_dict()} if l.type == "parallel" else l.right.to_dict()
            f = l.mlp
            mlp = None
            if f is not None:
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top}}
                if f.shared_ff:
                    mlp["shared"] = {"ff": f.shared_ff}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


# ---------------------------------------------------------------- Sobivik

@dataclass(frozen=True)
class RetentionSizes:
    """A retention mixer: ``heads`` heads of ``dim`` query/key and ``vdim`` value channels, one fixed ``decay`` a head."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "RetentionSizes":
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            raise ConfigError(f"config.json: {where}'decay' must be a list of numbers")
        s = cls(heads=_take(m, "heads", int), dim=_take(m, "dim", int), vdim=_take(m, "vdim", int),
                decay=tuple(float(d) for d in decay))
        for f in ("heads", "dim", "vdim"):
            if getattr(s, f) <= 0:
                raise ConfigError(f"config.json: {where}'{f}' must be positive, got {getattr(s, f)}")
        if len(s.decay) != s.heads or not all(0.0 <= d <= 1.0 for d in s.decay):
            raise ConfigError(f"config.json: {where}'decay' must hold one number between 0 and 1 for each of the {s.heads} heads")
        return s

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class RampScaling:
    """A rotation stretched to ``factor`` times the ``original`` length by a ramp over its frequencies: those that make
    more than ``fast`` turns over the original length stay, those that make fewer than ``slow`` are divided by the
    factor."""
    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "RampScaling":
        s = cls(*(_take(m, k, float) for k in ("factor", "original", "fast", "slow")))
        if not (s.factor > 0 and s.original > 0 and s.fast > 0 and s.slow > 0):
            raise ConfigError(f"config.json: {where}rot.scaling: factor, original, fast and slow must be positive")
        return s

    def to_dict(self) -> Dict[str, Any]:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class WindowLatentSizes:
    """Latent attention (``LatentAttentionSizes``) over a sliding window, with a learned sink per head, an output gate
    and a rotation in halves (element i with i + dims / 2), optionally stretched (``scaling``)."""
    latent: LatentAttentionSizes
    window: int
    scaling: Optional[RampScaling]

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "WindowLatentSizes":
        latent = LatentAttentionSizes.from_dict(m, where)
        if latent.kv_from is not None:
            raise ConfigError(f"config.json: {where}kv_from is not part of this design")
        sc = _section(_section(m, "rot", where), "scaling", where, optional=True)
        s = cls(latent, _take(_section(m, "mask", where), "size", int), RampScaling.from_dict(sc, where) if sc else None)
        if s.window <= 0:
            raise ConfigError(f"config.json: {where}mask.size must be positive, got {s.window}")
        return s

    def to_dict(self) -> Dict[str, Any]:
        m = self.latent
        rot = {"base": m.rot_base, "dims": m.rot_dims}
        if self.scaling:
            rot["scaling"] = self.scaling.to_dict()
        return {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                "q_rank": m.q_rank, "scale": m.scale, "rot": rot, "mask": {"size": self.window}}


@dataclass(frozen=True)
class DifferentialAttentionSizes:
    """Differential attention: ``heads`` query heads and ``kv_heads`` key/value heads, two score maps of ``dim``
    elements each per head, values of ``vdim``; a window of ``window`` tokens behind which the first ``keep_first``
    tokens stay visible; ``diff``: the constant of lambda and of the output factor."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int
    diff: float

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "DifferentialAttentionSizes":
        mask = _section(m, "mask", where)
        s = cls(heads=_take(m, "heads", int), kv_heads=_take(m, "kv_heads", int), dim=_take(m, "dim", int),
                vdim=_take(m, "vdim", int), scale=_take(m, "scale", float), window=_take(mask, "size", int),
                keep_first=_take(mask, "keep_first", int, 0), diff=_take(m, "diff", float))
        for f in ("heads", "kv_heads", "dim", "vdim", "window"):
            if getattr(s, f) <= 0:
                raise ConfigError(f"config.json: {where}'{f}' must be positive, got {getattr(s, f)}")
        if s.heads % s.kv_heads:
            raise ConfigError(f"config.json: {where}heads {s.heads} must be a multiple of kv_heads {s.kv_heads}")
        if s.keep_first < 0:
            raise ConfigError(f"config.json: {where}mask.keep_first must not be negative")
        return s

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                "diff": self.diff, "mask": {"size": self.window, "keep_first": self.keep_first}}


@dataclass(frozen=True)
class SobivikLayer:
    """``type``: "retention", "latent_attention" or "attention" (differential); ``mixer``: that mixer's sizes;
    ``mlp``: a dense gated feed-forward or none."""
    type: str
    mixer: Any
    mlp: Optional[FeedForwardSizes]


@dataclass(frozen=True)
class SobivikConfig:
    """``config.json`` of a Sobivik model: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_scale``,
    ``canon.taps`` (the short convolution on every mixer's input) and the list ``layers``, each entry with its
    ``type`` (the mixer it has), the mixer's sizes and its feed-forward (``mlp``, or null).  ``max_positions`` is
    optional: the design has no longest sequence of its own."""
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    conv_taps: int
    layers: Tuple[SobivikLayer, ...]
    max_positions: int = 1 << 20
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Sobivik"

    MIXER_TYPES = {"retention": RetentionSizes, "latent_attention": WindowLatentSizes, "attention": DifferentialAttentionSizes}

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SobivikConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]: "
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: {where}must be an object")
            kind = _take(l, "type", str)
            if kind not in cls.MIXER_TYPES:
                raise ConfigError(f"config.json: {where}unknown type {kind!r} ({', '.join(cls.MIXER_TYPES)})")
            mixer = cls.MIXER_TYPES[kind].from_dict(_section(l, "mixer", where), where)
            mlp = _section(l, "mlp", where, optional=True)
            ff = FeedForwardSizes.from_dict(mlp, where) if mlp else None
            if ff is not None and ff.kind != "dense":
                raise ConfigError(f"config.json: {where}mlp.kind {ff.kind!r}: the design's feed-forward is dense")
            layers.append(SobivikLayer(kind, mixer, ff))
        eos = d.get("eos_token_id")
        eos_ids = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ()
        cfg = cls(vocab=_take(d, "vocab", int), width=_take(d, "width", int),
                  norm_eps=_take(_section(d, "norm", ""), "eps", float),
                  embedding_scale=_take(_section(d, "embedding", ""), "scale", float),
                  logit_scale=_take(d, "logit_scale", float),
                  conv_taps=_take(_section(d, "canon", ""), "taps", int), layers=tuple(layers),
                  max_positions=_take(d, "max_positions", int, 1 << 20), eos_token_ids=eos_ids,
                  architecture=str(d.get("architecture") or (d.get("architectures") or ["Sobivik"])[0]))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 1:
            raise ConfigError("config.json: vocab, width and max_positions must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {cfg.norm_eps}")
        if not (1 <= cfg.conv_taps <= 16):
            raise ConfigError(f"config.json: canon.taps must be between 1 and 16, got {cfg.conv_taps}")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        layers = [{"type": l.type, "mixer": l.mixer.to_dict(),
                   "mlp": {"kind": "dense", "ff": l.mlp.ff} if l.mlp is not None else None} for l in self.layers]
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
             "canon": {"taps": self.conv_taps}, "layers": layers}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


# ---------------------------------------------------------------- Porovik

def _positive(s, fields, where: str) -> None:
    for f in fields:
        if getattr(s, f) <= 0:
            raise ConfigError(f"config.json: {where}'{f}' must be positive, got {getattr(s, f)}")


@dataclass(frozen=True)
class GateWriteSizes:
    """An ``hgrn2`` mixer: ``heads`` heads of ``dim`` query / forget-gate channels and ``vdim`` value channels."""
    heads: int
    dim: int
    vdim: int

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "GateWriteSizes":
        dim = _take(m, "dim", int)
        s = cls(heads=_take(m, "heads", int), dim=dim, vdim=_take(m, "vdim", int, dim))
        _positive(s, ("heads", "dim", "vdim"), where)
        return s

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}


@dataclass(frozen=True)
class GeneralDeltaSizes:
    """A ``general_delta`` mixer: ``heads`` heads of ``dim`` key channels (values as wide unless ``vdim`` says
    otherwise); the thin middle of the decay's projection is whatever the weight file holds (``decay_rank`` names it
    for weights that are drawn, not read)."""
    heads: int
    dim: int
    vdim: int
    decay_rank: int = -1

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "GeneralDeltaSizes":
        dim = _take(m, "dim", int)
        s = cls(heads=_take(m, "heads", int), dim=dim, vdim=_take(m, "vdim", int, dim),
                decay_rank=_take(m, "decay_rank", int, -1))
        _positive(s, ("heads", "dim", "vdim"), where)
        if s.decay_rank == 0 or s.decay_rank < -1:
            raise ConfigError(f"config.json: {where}'decay_rank' must be positive where it is given")
        return s

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim}
        if self.vdim != self.dim:
            d["vdim"] = self.vdim
        if self.decay_rank > 0:
            d["decay_rank"] = self.decay_rank
        return d


@dataclass(frozen=True)
class BiasedAttentionSizes:
    """An ``attention`` mixer of Porovik: grouped heads without a rotation, a query temperature that grows with the
    position (``q_temp.coef``, ``q_temp.every``; absent: none), a distance bias per head, values that may be mixed
    with an earlier layer's (``v_mix``) and a sigmoid gate on the heads."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float = 0.0
    temp_every: int = 1
    v_mix: bool = False

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "BiasedAttentionSizes":
        heads, dim = _take(m, "heads", int), _take(m, "dim", int)
        qt = _section(m, "q_temp", where, optional=True)
        s = cls(heads=heads, kv_heads=_take(m, "kv_heads", int, heads), dim=dim, vdim=_take(m, "vdim", int, dim),
                scale=_take(m, "scale", float), temp_coef=_take(qt, "coef", float) if qt else 0.0,
                temp_every=_take(qt, "every", int) if qt else 1, v_mix=_take(m, "v_mix", bool, False))
        _positive(s, ("heads", "kv_heads", "dim", "vdim", "temp_every"), where)
        if s.heads % s.kv_heads:
            raise ConfigError(f"config.json: {where}heads {s.heads} must be a multiple of kv_heads {s.kv_heads}")
        return s

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "v_mix": self.v_mix}
        if self.temp_coef != 0.0:
            d["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return d


@dataclass(frozen=True)
class BigramHash:
    """The hashed bigram table of the embedding: row ``(previous * mul_prev + current * mul_cur) mod buckets``, and row
    ``buckets`` for a sequence's first token."""
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class PorovikLayer:
    type: str
    mixer: Any
    mlp: Optional[FeedForwardSizes]      # None: the layer has no feed-forward


@dataclass(frozen=True)
class PorovikConfig:
    """``config.json`` of a Porovik model: ``vocab``, ``width``, ``max_positions`` (rows of the learned position
    table), ``norm.eps``, ``embedding.bigram.{buckets, mul_prev, mul_cur}`` and the list ``layers``, each entry with
    its ``type`` (``hgrn2``, ``general_delta`` or ``attention``), the mixer's sizes and its feed-forward (``mlp``:
    dense, a mixture of experts, or null)."""
    vocab: int
    width: int
    norm_eps: float
    max_positions: int
    bigram: Optional[BigramHash]
    layers: Tuple[PorovikLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Porovik"

    MIXER_TYPES = {"hgrn2": GateWriteSizes, "general_delta": GeneralDeltaSizes, "attention": BiasedAttentionSizes}

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PorovikConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]: "
            if not isinstance(l, dict):
                raise ConfigError(f"config.json: {where}must be an object")
            kind = _take(l, "type", str)
            if kind not in cls.MIXER_TYPES:
                raise ConfigError(f"config.json: {where}unknown type {kind!r} ({', '.join(cls.MIXER_TYPES)})")
            mixer = cls.MIXER_TYPES[kind].from_dict(_section(l, "mixer", where), where)
            mlp = _section(l, "mlp", where, optional=True)
            ff = FeedForwardSizes.from_dict(mlp, where) if mlp else None
            if ff is not None and ff.shared_ff:
                raise ConfigError(f"config.json: {where}the design's mixture of experts has no shared expert")
            layers.append(PorovikLayer(kind, mixer, ff))
        emb = _section(d, "embedding", "", optional=True) or {}
        bg = _section(emb, "bigram", "embedding: ", optional=True)
        bigram = BigramHash(_take(bg, "buckets", int), _take(bg, "mul_prev", int), _take(bg, "mul_cur", int)) if bg else None
        if bigram is not None and (bigram.buckets <= 0 or bigram.mul_prev < 0 or bigram.mul_cur < 0):
            raise ConfigError("config.json: embedding.bigram: buckets must be positive, the multipliers not negative")
        eos = d.get("eos_token_id")
        eos_ids = (eos,) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else ()
        cfg = cls(vocab=_take(d, "vocab", int), width=_take(d, "width", int),
                  norm_eps=_take(_section(d, "norm", ""), "eps", float), max_positions=_take(d, "max_positions", int),
                  bigram=bigram, layers=tuple(layers), eos_token_ids=eos_ids,
                  architecture=str(d.get("architecture") or (d.get("architectures") or ["Porovik"])[0]))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.max_positions <= 1:
            raise ConfigError("config.json: vocab and width must be positive, max_positions at least 2")
        mixed = {(l.mixer.kv_heads, l.mixer.vdim) for l in cfg.layers if l.type == "attention" and l.mixer.v_mix}
        if len(mixed) > 1:
            raise ConfigError(f"config.json: layers with v_mix share the first one's values, so their kv_heads and vdim "
                              f"must agree, got {sorted(mixed)}")
        if not cfg.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {cfg.norm_eps}")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        def mlp(f):
            if f is None:
                return None
            if f.kind == "dense":
                return {"kind": "dense", "ff": f.ff}
            return {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top}}
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "max_positions": self.max_positions,
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": mlp(l.mlp)} for l in self.layers]}
        if self.bigram is not None:
            d["embedding"] = {"bigram": {"buckets": self.bigram.buckets, "mul_prev": self.bigram.mul_prev,
                                         "mul_cur": self.bigram.mul_cur}}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
