"""Panolorn as data: which registered parts each layer is made of.

The stream starts as the scaled embedding.  Every layer is a ``sandwich`` block (a norm before and
after each sub-layer; ``sandwich_mixer`` where the layer has no feed-forward) around

* ``biased_attention``: grouped-query attention without rotation; queries and keys divided by their
  root mean square per head (the layer's eps), a tanh cap on the scores, a distance bias with slopes
  2^(-8 (h + 1) / heads), keys only from the query's own chunk, a sink in the softmax's denominator and
  a sigmoid output gate;
* ``swiglu`` with the tanh form of GELU for dense layers, or ``moe`` (sigmoid scores, the weight on the
  expert's input, SiLU experts, an optional shared expert).

The head is the embedding table itself.  Tensor names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.q|k|v|g|o``, ``l<i>.mlp.gate|up|down``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down``, ``final.norm``.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.panolorn import ARCHITECTURE, PanolornConfig
from ..parts.spec import ExecEntry, LayerSpec, ModelDescription, PartSpec

SLOPE_EXPONENT = 8.0          # slope of head h: 2^(-8 (h + 1) / heads)
GATED_NAMES = ("gate", "up", "down")


def describe_panolorn(cfg: PanolornConfig) -> ModelDescription:
    layers = []

    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, name=name), prefix)

    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        parts = {
            "norm1": norm(p, "norm1"),
            "mixer": PartSpec("biased_attention", dict(
                hidden_size=cfg.width, q_heads=m.heads, kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                scale=m.scale, unit_norm_eps=cfg.norm_eps, softcap=m.softcap, slope_exponent=SLOPE_EXPONENT,
                chunk=m.chunk, sink=True, output_gate=True), p + "mix."),
            "norm1b": norm(p, "norm1b"),
        }
        if layer.mlp is None:
            layers.append(LayerSpec("sandwich_mixer", parts))
            continue
        f = layer.mlp
        if f.kind == "dense":
            ffn = PartSpec("swiglu", dict(hidden_size=cfg.width, intermediate_size=f.ff, activation="gelu_tanh",
                                          names=GATED_NAMES), p + "mlp.")
        else:
            shared = None
            if f.shared_ff is not None:
                shared = PartSpec("swiglu", dict(hidden_size=cfg.width, intermediate_size=f.shared_ff,
                                                 activation="silu", names=GATED_NAMES), "shared.")
            ffn = PartSpec("moe", dict(hidden_size=cfg.width, experts=f.experts, top=f.top, expert_size=f.ff,
                                       activation="silu", router_scores="sigmoid", weight_on="input",
                                       shared=shared, names=GATED_NAMES), p + "mlp.")
        parts.update({"norm2": norm(p, "norm2"), "ffn": ffn, "norm2b": norm(p, "norm2b")})
        layers.append(LayerSpec("sandwich", parts))
    return ModelDescription(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=cfg.width,
                                                   scale=cfg.embedding_scale, name="embed"), ""),
        layers=tuple(layers),
        order=tuple(ExecEntry(i) for i in range(len(cfg.layers))),
        final_norm=PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, name="norm"), "final."),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, tied=True), "lm_head."),
    )


register_architecture(ARCHITECTURE, PanolornConfig, describe_panolorn, model_types=("panolorn",))
