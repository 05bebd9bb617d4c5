"""Tiny Panolorn configurations for the tests.  They differ in every size and constant, and take
values that hide nothing: key and value widths that differ, one key/value head per query head and one for
all, top 2 and top 3 of the experts, a layer without a shared expert, a layer without a feed-forward,
a layer without a cap, a layer without chunks, chunks that are no multiple of the page and smaller than it."""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tiny_llm_infer_b200.config.panolorn import (AttentionMixerConfig, FeedForwardConfig, PanolornConfig,
                                                  PanolornLayerConfig)
from tiny_llm_infer_b200.weights import write_random_model


def layer(heads, kv, dim, vdim, scale, softcap, chunk, mlp):
    return PanolornLayerConfig("attention", AttentionMixerConfig(heads, kv, dim, vdim, scale, softcap, chunk), mlp)


def dense(ff):
    return FeedForwardConfig("dense", ff)


def moe(ff, experts, top, shared):
    return FeedForwardConfig("moe", ff, experts=experts, top=top, shared_ff=shared)


# widths the tensor-core kernels take (64, 64), pages of 16, chunks of 50
P1 = dict(cfg=PanolornConfig(vocab=320, width=128, embedding_scale=7.5, norm_eps=1e-5, layers=(
    layer(4, 2, 64, 64, 0.25, 20.0, 50, dense(160)),
    layer(4, 2, 64, 64, 0.25, 20.0, 50, moe(48, 8, 2, 96)),
    layer(4, 2, 64, 64, 0.25, 20.0, 50, None),
)), seed=11, std=0.06, norm_range=(0.7, 1.3), page_size=16, lengths=(70, 97, 130, 41, 66, 35))
# key and value widths differ (32, 48), six heads on six key/value heads, chunk 24 beside a layer
# without chunks and one without a cap; top 3, no shared expert; widths that are no multiples of 16
P2 = dict(cfg=PanolornConfig(vocab=401, width=88, embedding_scale=1.0, norm_eps=3e-6, layers=(
    layer(6, 6, 32, 48, 0.4, 8.0, 24, moe(40, 5, 3, None)),
    layer(3, 1, 40, 24, 0.3, None, None, dense(100)),
    layer(6, 3, 32, 48, 0.4, 30.0, 7, moe(24, 12, 1, 56)),
)), seed=12, std=0.08, norm_range=(0.6, 1.4), page_size=8, lengths=(70, 97, 41, 35, 66))
# widths 80 (padded to 128 in the tensor-core kernel) and 128 / 64, eight query heads on one key/value head,
# chunks longer than some requests and pages of 32
P3 = dict(cfg=PanolornConfig(vocab=512, width=160, embedding_scale=11.0, norm_eps=1e-6, layers=(
    layer(8, 1, 80, 80, 0.17, 40.0, 200, dense(320)),
    layer(2, 2, 128, 64, 0.12, 15.0, 64, moe(56, 12, 2, 136)),
)), seed=13, std=0.05, norm_range=(0.8, 1.2), page_size=32, lengths=(70, 300, 130, 41, 210, 35))
PANOLORNS = {"P1": P1, "P2": P2, "P3": P3}


def make_folder(tiny, folder=None, dtype=torch.bfloat16) -> Path:
    folder = Path(folder or tempfile.mkdtemp(prefix="tllm_pano_"))
    return write_random_model(folder, tiny["cfg"], tiny["seed"], tiny["std"], tiny["norm_range"], dtype=dtype)


def prompt(seed: int, length: int, vocab: int):
    g = torch.Generator().manual_seed(2000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def requests_for(tiny):
    return {str(i): prompt(i, n, tiny["cfg"].vocab) for i, n in enumerate(tiny["lengths"])}
