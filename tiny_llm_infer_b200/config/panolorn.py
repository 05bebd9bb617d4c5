"""Typed configuration of the Panolorn design, read from its own config.json keys.

config.json carries ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps`` and ``layers``: a list with, per layer, ``type`` (which mixer), ``mixer`` (its sizes and
constants) and ``mlp`` (its feed-forward, or null for a layer without one).  Nothing else exists:
every size and constant the engine uses comes from these keys or from the shapes of the tensors.

Mixer ``attention``: ``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values), ``scale``,
``softcap`` (absent or null: no cap) and ``mask.size`` (the chunk; absent: plain causal).
Feed-forward ``dense``: ``ff``.  ``moe``: ``router.experts``, ``router.top``, ``expert.ff`` and, if the
layer has a shared expert, ``shared.ff``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, coerce, optional, require

ARCHITECTURE = "Panolorn"


def _section(raw: Dict[str, Any], key: str, where: str, needed: bool = True) -> Optional[Dict[str, Any]]:
    value = raw.get(key)
    if value is None:
        if needed:
            raise ConfigError(f"config.json: {where}{key!r} is missing")
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return value


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float] = None
    chunk: Optional[int] = None

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str) -> "AttentionMixerConfig":
        mask = _section(raw, "mask", where, needed=False)
        softcap = optional(raw, "softcap", None, float)
        heads = require(raw, "heads")
        return cls(heads=heads, kv_heads=optional(raw, "kv_heads", heads), dim=require(raw, "dim"),
                   vdim=optional(raw, "vdim", raw.get("dim")), scale=require(raw, "scale", float),
                   softcap=softcap if softcap else None,
                   chunk=None if mask is None else require(mask, "size"))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
                               "vdim": self.vdim, "scale": self.scale}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        return out

    def validate(self, where: str) -> None:
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {where}{name} must be positive")
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        if self.chunk is not None and self.chunk <= 0:
            raise ConfigError(f"config.json: {where}mask.size must be positive")
        if self.softcap is not None and not self.softcap > 0:
            raise ConfigError(f"config.json: {where}softcap must be positive")


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                         # "dense" or "moe"
    ff: int                           # width of the dense unit, or of one expert
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None   # width of the shared expert, None for none

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str) -> "FeedForwardConfig":
        kind = require(raw, "kind", str)
        if kind == "dense":
            return cls("dense", require(raw, "ff"))
        if kind == "moe":
            router = _section(raw, "router", where)
            expert = _section(raw, "expert", where)
            shared = _section(raw, "shared", where, needed=False)
            return cls("moe", require(expert, "ff"), experts=require(router, "experts"),
                       top=require(router, "top"), shared_ff=None if shared is None else require(shared, "ff"))
        raise ConfigError(f"config.json: {where}kind {kind!r} is neither 'dense' nor 'moe'")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                               "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out

    def validate(self, where: str) -> None:
        if self.ff <= 0:
            raise ConfigError(f"config.json: {where}ff must be positive")
        if self.kind == "moe":
            if not 0 < self.top <= self.experts:
                raise ConfigError(f"config.json: {where}router.top must lie in 1..experts")
            if self.shared_ff is not None and self.shared_ff <= 0:
                raise ConfigError(f"config.json: {where}shared.ff must be positive")


@dataclass(frozen=True)
class PanolornLayerConfig:
    type: str
    mixer: AttentionMixerConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class PanolornConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[PanolornLayerConfig, ...]
    # not part of config.json: positions have no table or rotation, so nothing bounds them but memory
    max_position_embeddings: int = 1 << 20
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    architecture: str = field(default=ARCHITECTURE)

    # the names the engine's tools use for every architecture
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PanolornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = require(entry, "type", str)
            if kind != "attention":
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design ('attention')")
            mixer = AttentionMixerConfig.from_dict(_section(entry, "mixer", where), where + "mixer.")
            mlp_raw = _section(entry, "mlp", where, needed=False)
            mlp = None if mlp_raw is None else FeedForwardConfig.from_dict(mlp_raw, where + "mlp.")
            layers.append(PanolornLayerConfig(kind, mixer, mlp))
        embedding = _section(raw, "embedding", "", needed=False) or {}
        norm = _section(raw, "norm", "")
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(coerce(x, "eos_token_id[]", int) for x in eos)
        else:
            eos_ids = (coerce(eos, "eos_token_id", int),)
        bos = raw.get("bos_token_id")
        return cls(vocab=require(raw, "vocab"), width=require(raw, "width"),
                   embedding_scale=optional(embedding, "scale", 1.0, float),
                   norm_eps=require(norm, "eps", float), layers=tuple(layers),
                   max_position_embeddings=optional(raw, "max_position_embeddings", 1 << 20),
                   eos_token_ids=eos_ids, bos_token_id=None if bos is None else coerce(bos, "bos_token_id", int))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(),
                        "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.max_position_embeddings != 1 << 20:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_position_embeddings <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            layer.mixer.validate(f"layers[{i}].mixer.")
            if layer.mlp is not None:
                layer.mlp.validate(f"layers[{i}].mlp.")
        for tok in self.eos_token_ids:
            if not 0 <= tok < self.vocab:
                raise ConfigError(f"config.json: eos_token_id {tok} is outside the vocabulary")
