"""Tiny Kaketar configurations for the tests.  They differ in every size and constant and take values that
hide nothing: fewer query/key heads than value heads, key and value widths that differ and that are no
multiples of four, two to four taps, low ranks that differ, a rotation of part of the rotated elements, with
and without stretched frequencies, windows smaller than a page and no multiple of one, a layer without a
window, more heads than a tile has rows, cached vectors wider than the tensor-core kernels take, layers with
and without a feed-forward in every order, a model without the token side input and without a cap on the
logits.  Half of the delta rule's decays are made slow (a bias far below zero), so that what was written
hundreds of tokens ago still shows in the read-out."""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tiny_llm_infer_b200.config.kaketar import (ChannelDeltaConfig, DenseConfig, KaketarConfig, KaketarLayerConfig,
                                                 LatentAttentionConfig, RotationScaling)
from tiny_llm_infer_b200.weights import write_random_model
from tiny_llm_infer_b200.weights.safetensors_io import SafetensorsFile, save_file


def delta(heads, kv, dim, vdim, conv, ranks, ff=None):
    return KaketarLayerConfig("channel_delta", ChannelDeltaConfig(heads, kv, dim, vdim, conv, ranks[0], ranks[1]),
                              None if ff is None else DenseConfig(ff))


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, rot_dims, window, scaling=None, ff=None):
    sc = None if scaling is None else RotationScaling(*scaling)
    return KaketarLayerConfig("latent_attention",
                              LatentAttentionConfig(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, rot_dims,
                                                    window, sc), None if ff is None else DenseConfig(ff))


# cached vectors of 80 (the tensor-core kernels' widths), window 40 over pages of 16, stretched frequencies
K1 = dict(cfg=KaketarConfig(vocab=320, width=128, max_positions=512, embedding_scale=2.5, norm_eps=1e-5, layers=(
    latent(4, 32, 16, 32, 48, 64, 0.21, 10000.0, 16, 40, (8.0, 64.0, 16.0, 2.0), ff=160),
    delta(4, 2, 32, 48, 4, (8, 16)),
    delta(2, 2, 64, 32, 2, (16, 8), ff=96),
    latent(8, 16, 8, 24, 32, 40, 0.3, 500.0, 8, 23, None),
), logit_softcap=12.0, side_dim=8), seed=21, std=0.08, norm_range=(0.7, 1.3), page_size=16,
    lengths=(70, 97, 130, 41, 66, 35))
# no side input, no cap, scale 1; key width 20 and 72 (rows dealt to 4 and 8 lanes), a window of 7 under pages of
# 8, a layer without a window with 20 heads (more than a tile's rows), a rotation of 4 of 8 rotated elements
K2 = dict(cfg=KaketarConfig(vocab=401, width=88, max_positions=300, embedding_scale=1.0, norm_eps=3e-6, layers=(
    delta(6, 3, 20, 24, 3, (8, 24)),
    latent(3, 24, 8, 40, 40, 56, 0.25, 250000.0, 4, 7, None, ff=100),
    latent(20, 8, 8, 8, 24, 24, 0.35, 1000.0, 8, None, (2.0, 32.0, 8.0, 1.0)),
    delta(1, 1, 72, 40, 2, (8, 8), ff=64),
)), seed=22, std=0.1, norm_range=(0.6, 1.4), page_size=8, lengths=(70, 97, 41, 35, 66))
# pages of 32; cached vectors of 160 (wider than the tensor-core kernels take); keys and values of 128
K3 = dict(cfg=KaketarConfig(vocab=512, width=160, max_positions=400, embedding_scale=4.0, norm_eps=1e-6, layers=(
    delta(2, 1, 128, 128, 2, (8, 16), ff=320),
    latent(2, 48, 16, 64, 72, 144, 0.1, 50000.0, 16, 100, (4.0, 128.0, 32.0, 1.0)),
    delta(5, 5, 16, 16, 5, (24, 8)),
), logit_softcap=30.0, side_dim=24), seed=23, std=0.07, norm_range=(0.8, 1.2), page_size=32,
    lengths=(70, 300, 130, 41, 210, 35))
# nothing a multiple of eight, little a multiple of four: width 100, key widths 10 and 6, value widths 6 and 10,
# six taps, a window of 3, a rotation of 2 of 6 rotated elements, five and three heads, a side input of 3
K4 = dict(cfg=KaketarConfig(vocab=333, width=100, max_positions=200, embedding_scale=0.5, norm_eps=2e-5, layers=(
    latent(5, 6, 6, 10, 12, 10, 0.4, 77.0, 2, 3, (3.0, 20.0, 6.0, 1.5), ff=50),
    delta(3, 1, 10, 6, 6, (8, 9)),
    delta(2, 2, 6, 10, 1, (11, 8), ff=30),
), logit_softcap=5.0, side_dim=3), seed=24, std=0.12, norm_range=(0.7, 1.3), page_size=16,
    lengths=(70, 97, 41, 35, 66))
KAKETARS = {"K1": K1, "K2": K2, "K3": K3, "K4": K4}


def make_folder(tiny, folder=None, dtype=torch.bfloat16) -> Path:
    """Random weights, then: the decays of every second head made slow, and the sinks spread out."""
    folder = Path(folder or tempfile.mkdtemp(prefix="tllm_kake_"))
    write_random_model(folder, tiny["cfg"], tiny["seed"], tiny["std"], tiny["norm_range"], dtype=dtype)
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: f.read(name).clone() for name in f.tensors}
    f.close()
    for i, layer in enumerate(tiny["cfg"].layers):
        m = layer.mixer
        if layer.type == "channel_delta":
            bias = tensors[f"l{i}.mix.dt_bias"].float().view(m.heads, m.dim)
            bias[::2] -= 6.0                                   # softplus near 0.003: a memory of hundreds of tokens
            tensors[f"l{i}.mix.dt_bias"] = bias.reshape(-1).to(dtype)
        else:
            tensors[f"l{i}.mix.sink"] = (tensors[f"l{i}.mix.sink"].float() * 3.0).to(dtype)
    save_file(tensors, folder / "model.safetensors")
    return folder


def prompt(seed: int, length: int, vocab: int):
    g = torch.Generator().manual_seed(3000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def requests_for(tiny):
    return {str(i): prompt(i, n, tiny["cfg"].vocab) for i, n in enumerate(tiny["lengths"])}
