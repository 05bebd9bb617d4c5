"""Kaketar as data: which registered parts each layer is made of.

The stream starts as the norm of (scaled token embedding + learned position vector).  Every layer is a
``stream_*`` block: its sub-layers read the stream itself and only their outputs are normed before the sum
(the model's norm, whose stored weight is the gain minus one).  The mixer is

* ``channel_delta``: the delta rule with a decay per head and key channel, short convolutions on q, k, v, unit
  q and k, a normed and gated read-out; its memory is a float32 matrix per head and request, or
* ``latent_attention``: attention over one cached latent per token (plus one rotated key part for all heads)
  with interleaved rotation and stretched slow frequencies, a sliding window, a learned sink per head and an
  output gate;

then, where the layer has one, a plain feed-forward with the exact GELU, and, where the model has a token
side table, a small gated input looked up by the row's token (layer i reads columns [i dim, (i + 1) dim) of
the shared table), normed with a plain gain.  The head has its own matrix and a tanh cap on the logits.

Tensor names: ``embed``, ``pos``, ``embed.norm``, ``side.embed``, ``l<i>.norm1|norm2``,
``l<i>.mix.q|k|v`` (+ ``.conv``) ``|b|A_log|norm|a1|a2|dt_bias|g1|g2|o``,
``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|sink|g|o``, ``l<i>.mlp.up|down``,
``l<i>.side.gate|proj|norm``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.kaketar import ARCHITECTURE, ChannelDeltaConfig, KaketarConfig, default_rank
from ..parts.spec import ExecEntry, LayerSpec, ModelDescription, PartSpec

NORM_OFFSET = 1.0             # the model's norm stores its gain as the distance from one
UNIT_EPS = 1e-6               # under the root when q and k are made unit vectors
FF_ACTIVATION = "gelu_erf"
SIDE_ACTIVATION = "gelu_tanh"


def describe_kaketar(cfg: KaketarConfig) -> ModelDescription:
    layers = []

    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, name=name, offset=NORM_OFFSET), prefix)

    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if isinstance(m, ChannelDeltaConfig):
            mixer = PartSpec("channel_delta", dict(
                hidden_size=cfg.width, heads=m.heads, kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                conv_taps=m.conv, decay_rank=m.decay_rank or default_rank(cfg.width),
                gate_rank=m.gate_rank or default_rank(cfg.width), norm_eps=cfg.norm_eps, unit_eps=UNIT_EPS), p + "mix.")
        else:
            scaling = None
            if m.scaling is not None:
                s = m.scaling
                scaling = dict(factor=s.factor, original=s.original, fast=s.fast, slow=s.slow)
            mixer = PartSpec("latent_attention", dict(
                hidden_size=cfg.width, heads=m.heads, plain_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
                q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale, norm_eps=cfg.norm_eps, rot_base=m.rot_base,
                rot_dims=m.rot_dims, scaling=scaling, window=m.window, sink=True, output_gate=True), p + "mix.")
        parts = {"mixer": mixer, "norm1": norm(p, "norm1")}
        block = "stream_mixer"
        if layer.mlp is not None:
            parts["ffn"] = PartSpec("mlp", dict(hidden_size=cfg.width, intermediate_size=layer.mlp.ff,
                                                activation=FF_ACTIVATION), p + "mlp.")
            parts["norm2"] = norm(p, "norm2")
            block += "_ffn"
        if cfg.side_dim is not None:
            parts["side"] = PartSpec("token_side", dict(hidden_size=cfg.width, side_dim=cfg.side_dim,
                                                        first_column=i * cfg.side_dim, activation=SIDE_ACTIVATION),
                                     p + "side.")
            parts["norm3"] = PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, name="norm",
                                                      float32_gain=True), p + "side.")
            block += "_side"
        layers.append(LayerSpec(block, parts))
    side_columns = 0 if cfg.side_dim is None else cfg.side_dim * len(cfg.layers)
    return ModelDescription(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_position_embedding", dict(
            vocab_size=cfg.vocab, hidden_size=cfg.width, max_positions=cfg.max_positions, scale=cfg.embedding_scale,
            name="embed", pos_name="pos", norm_name="embed.norm", norm_eps=cfg.norm_eps, norm_offset=NORM_OFFSET,
            side_columns=side_columns, side_name="side.embed"), ""),
        layers=tuple(layers),
        order=tuple(ExecEntry(i) for i in range(len(cfg.layers))),
        final_norm=PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, name="norm", offset=NORM_OFFSET), "final."),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied=False, name="head",
                                      softcap=cfg.logit_softcap), ""),
    )


register_architecture(ARCHITECTURE, KaketarConfig, describe_kaketar, model_types=("kaketar",))
