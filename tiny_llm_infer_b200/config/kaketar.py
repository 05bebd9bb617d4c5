"""Typed configuration of the Kaketar design, read from its own config.json keys.

config.json carries ``architecture`` (the name), ``vocab``, ``width``, ``max_positions`` (rows of the
learned position table), ``embedding.scale``, ``norm.eps``, ``logit_softcap`` (absent or null: none),
``token_side.dim`` (absent: no per-layer token input) and ``layers``: per layer ``type`` (which mixer),
``mixer`` (its sizes and constants) and ``mlp`` (its feed-forward, or null for a layer without one).

Mixer ``channel_delta``: ``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values), ``conv``
(taps of the short convolution).  The ranks of its two low-rank projections are the shapes of the tensors.
Mixer ``latent_attention``: ``heads``, ``dim`` (unrotated part of a query or key), ``rot_dim`` (rotated
part), ``vdim``, ``q_rank``, ``kv_rank``, ``scale``, ``mask.size`` (the window; absent: plain causal) and
``rot``: ``base``, ``dims`` and, optionally, ``scaling`` with ``factor``, ``original``, ``fast``, ``slow``.
Feed-forward ``dense``: ``ff``.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Dict, Optional, Tuple, Union

from .base import ConfigError, ModelConfig, coerce, optional, require

ARCHITECTURE = "Kaketar"


def _section(raw: Dict[str, Any], key: str, where: str, needed: bool = True) -> Optional[Dict[str, Any]]:
    value = raw.get(key)
    if value is None:
        if needed:
            raise ConfigError(f"config.json: {where}{key!r} is missing")
        return None
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return value


def default_rank(width: int) -> int:
    """Rank of the delta rule's two low-rank projections where no checkpoint says it (random weights)."""
    return max(8, width // 32 * 2)


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    # not keys of config.json: the shapes of the checkpoint's tensors give them (``with_tensor_shapes``)
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str) -> "ChannelDeltaConfig":
        heads = require(raw, "heads")
        return cls(heads=heads, kv_heads=optional(raw, "kv_heads", heads), dim=require(raw, "dim"),
                   vdim=optional(raw, "vdim", raw.get("dim")), conv=require(raw, "conv"))

    def to_dict(self) -> Dict[str, Any]:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "vdim": self.vdim}

    def validate(self, where: str) -> None:
        for name in ("heads", "kv_heads", "dim", "vdim", "conv"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {where}{name} must be positive")
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")


@dataclass(frozen=True)
class RotationScaling:
    """Stretching of the slow frequencies of a rotation for contexts longer than ``original``."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    window: Optional[int] = None
    scaling: Optional[RotationScaling] = None

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str) -> "LatentAttentionConfig":
        rot = _section(raw, "rot", where)
        mask = _section(raw, "mask", where, needed=False)
        sc = _section(rot, "scaling", where + "rot.", needed=False)
        rot_dim = require(raw, "rot_dim")
        scaling = None
        if sc is not None:
            scaling = RotationScaling(require(sc, "factor", float), require(sc, "original", float),
                                      require(sc, "fast", float), require(sc, "slow", float))
        return cls(heads=require(raw, "heads"), dim=require(raw, "dim"), rot_dim=rot_dim,
                   vdim=optional(raw, "vdim", raw.get("dim")), q_rank=require(raw, "q_rank"),
                   kv_rank=require(raw, "kv_rank"), scale=require(raw, "scale", float),
                   rot_base=require(rot, "base", float), rot_dims=optional(rot, "dims", rot_dim),
                   window=None if mask is None else require(mask, "size"), scaling=scaling)

    def to_dict(self) -> Dict[str, Any]:
        rot: Dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.scaling is not None:
            s = self.scaling
            rot["scaling"] = {"factor": s.factor, "fast": s.fast, "original": s.original, "slow": s.slow}
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank,
                               "q_rank": self.q_rank, "rot": rot, "rot_dim": self.rot_dim,
                               "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out

    def validate(self, where: str) -> None:
        for name in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {where}{name} must be positive")
        if self.rot_dims <= 0 or self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most rot_dim")
        if not self.rot_base > 1.0:
            raise ConfigError(f"config.json: {where}rot.base must be larger than 1")
        if self.window is not None and self.window <= 0:
            raise ConfigError(f"config.json: {where}mask.size must be positive")
        if self.scaling is not None:
            s = self.scaling
            if not (s.factor >= 1.0 and s.original > 0 and s.fast > 0 and s.slow > 0):
                raise ConfigError(f"config.json: {where}rot.scaling needs factor >= 1 and positive original, fast, slow")


@dataclass(frozen=True)
class DenseConfig:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"ff": self.ff, "kind": "dense"}


MIXERS = {"channel_delta": ChannelDeltaConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class KaketarLayerConfig:
    type: str
    mixer: Union[ChannelDeltaConfig, LatentAttentionConfig]
    mlp: Optional[DenseConfig]


@dataclass(frozen=True)
class KaketarConfig(ModelConfig):
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[KaketarLayerConfig, ...]
    logit_softcap: Optional[float] = None
    side_dim: Optional[int] = None
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

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KaketarConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = require(entry, "type", str)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design {sorted(MIXERS)}")
            mixer = MIXERS[kind].from_dict(_section(entry, "mixer", where), where + "mixer.")
            mlp_raw = _section(entry, "mlp", where, needed=False)
            mlp = None
            if mlp_raw is not None:
                ff_kind = optional(mlp_raw, "kind", "dense", str)
                if ff_kind != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {ff_kind!r} is not 'dense'")
                mlp = DenseConfig(require(mlp_raw, "ff"))
            layers.append(KaketarLayerConfig(kind, mixer, mlp))
        embedding = _section(raw, "embedding", "", needed=False) or {}
        norm = _section(raw, "norm", "")
        side = _section(raw, "token_side", "", needed=False)
        cap = optional(raw, "logit_softcap", None, float)
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(coerce(x, "eos_token_id[]", int) for x in eos)
        else:
            eos_ids = (coerce(eos, "eos_token_id", int),)
        bos = raw.get("bos_token_id")
        return cls(vocab=require(raw, "vocab"), width=require(raw, "width"),
                   max_positions=require(raw, "max_positions"),
                   embedding_scale=optional(embedding, "scale", 1.0, float),
                   norm_eps=require(norm, "eps", float), layers=tuple(layers),
                   logit_softcap=cap if cap else None,
                   side_dim=None if side is None else require(side, "dim"),
                   eos_token_ids=eos_ids, bos_token_id=None if bos is None else coerce(bos, "bos_token_id", int))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(),
                        "type": l.type} for l in self.layers],
            "max_positions": self.max_positions,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "KaketarConfig":
        """The sizes that only the checkpoint gives: the ranks of the delta rule's low-rank projections
        (rows of ``l<i>.mix.a1`` and ``l<i>.mix.g1``)."""
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if isinstance(m, ChannelDeltaConfig):
                a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
                m = replace(m, decay_rank=int(a1[0]) if a1 else m.decay_rank, gate_rank=int(g1[0]) if g1 else m.gate_rank)
            layers.append(replace(layer, mixer=m))
        return replace(self, layers=tuple(layers))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0:
            raise ConfigError("config.json: vocab, width and max_positions must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        if self.side_dim is not None and self.side_dim <= 0:
            raise ConfigError("config.json: token_side.dim must be positive")
        for i, layer in enumerate(self.layers):
            layer.mixer.validate(f"layers[{i}].mixer.")
            if layer.mlp is not None and layer.mlp.ff <= 0:
                raise ConfigError(f"config.json: layers[{i}].mlp.ff must be positive")
        for tok in self.eos_token_ids:
            if not 0 <= tok < self.vocab:
                raise ConfigError(f"config.json: eos_token_id {tok} is outside the vocabulary")
