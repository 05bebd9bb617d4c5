"""Panolorn without a GPU: its configuration, the description the model is assembled from, what its
mixer asks of the cache manager, and the plain implementation's own mechanisms on cases small enough
to check by hand."""
import json
import math

import pytest
import torch

import plain_panolorn as plain
from tiny_panolorn import PANOLORNS, make_folder

from tiny_llm_infer_b200.config import ConfigError, config_from_dict, load_config
from tiny_llm_infer_b200.config.base import describe_model
from tiny_llm_infer_b200.config.panolorn import PanolornConfig
from tiny_llm_infer_b200.models.model import Model, expected_tensors


@pytest.mark.parametrize("name", sorted(PANOLORNS))
def test_config_round_trip_and_tensor_names(name, tmp_path):
    tiny = PANOLORNS[name]
    folder = make_folder(tiny, tmp_path)
    raw = json.loads((folder / "config.json").read_text())
    assert raw["architecture"] == "Panolorn" and "architectures" not in raw
    cfg = load_config(folder)
    assert isinstance(cfg, PanolornConfig) and cfg == tiny["cfg"] and cfg.to_dict() == raw
    expected, _ = expected_tensors(describe_model(cfg))
    _, weights = plain.read_model(folder)
    assert set(expected) == set(weights)
    assert "embed" in expected and "final.norm" in expected and "l0.mix.g" in expected
    for i, layer in enumerate(cfg.layers):
        has_ffn = f"l{i}.norm2b" in expected
        assert has_ffn == (layer.mlp is not None)
        if layer.mlp is not None and layer.mlp.kind == "moe":
            assert (f"l{i}.mlp.shared.up" in expected) == (layer.mlp.shared_ff is not None)
            assert expected[f"l{i}.mlp.router"].shape == (layer.mlp.experts, cfg.width)
            assert f"l{i}.mlp.e{layer.mlp.experts - 1}.down" in expected


def test_config_errors():
    good = PANOLORNS["P1"]["cfg"].to_dict()
    for path, value in ((("layers", 0, "type"), "recurrent"), (("layers", 1, "mlp", "kind"), "sparse"),
                        (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 1, "mlp", "router", "top"), 9),
                        (("norm", "eps"), 0.0), (("layers", 0, "mixer", "mask", "size"), 0)):
        raw = json.loads(json.dumps(good))
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(raw)
    raw = json.loads(json.dumps(good))
    del raw["layers"][0]["mixer"]["scale"]
    with pytest.raises(ConfigError):
        config_from_dict(raw)


def test_the_cache_keeps_what_a_chunk_can_still_see():
    cfg = PANOLORNS["P2"]["cfg"]
    model = Model(describe_model(cfg), torch.float32, "cpu")
    needs = model.cache_needs()
    windows = [needs[i][0].window for i in sorted(needs)]
    assert windows == [24, None, 7]
    planes = [needs[i][0].planes for i in sorted(needs)]
    assert planes[0] == ((6, 32), (6, 48)) and planes[1] == ((1, 40), (1, 24))
    assert all(state is None for _, state in needs.values())


def test_plain_mask_sink_and_bias_by_hand():
    vis = plain.visible(7, 3)
    assert vis[2].tolist() == [True, True, True, False, False, False, False]
    assert vis[3].tolist() == [False, False, False, True, False, False, False]
    assert vis[5].tolist() == [False, False, False, True, True, True, False]
    assert plain.visible(4, None)[3].tolist() == [True] * 4
    # one visible key of score 0: the sink takes half
    p = plain.sink_softmax(torch.tensor([[0.0, float("-inf")]], dtype=torch.float64))
    assert p.tolist() == [[0.5, 0.0]]
    big = plain.sink_softmax(torch.tensor([[800.0, 799.0]], dtype=torch.float64))
    assert abs(float(big.sum()) - 1.0) < 1e-12
    assert plain.slopes(4).tolist() == [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8]
    q = torch.ones(3, 4, dtype=torch.float64)
    s = plain.attention_scores(q, q, 1, 4, 0.5, 1.0, None)
    assert abs(float(s[2, 0]) - (math.tanh(2.0) - 2 * 2.0 ** -4)) < 1e-12
    assert s[0, 1] == float("-inf")


def test_plain_router_weights_scale_the_input():
    torch.manual_seed(0)
    u = torch.randn(3, 6, dtype=torch.float64)
    w = {"m.router": torch.randn(4, 6, dtype=torch.float64)}
    for e in range(4):
        w[f"m.e{e}.gate"] = torch.randn(5, 6, dtype=torch.float64)
        w[f"m.e{e}.up"] = torch.randn(5, 6, dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.randn(6, 5, dtype=torch.float64)
    out = plain.moe(u, w, "m.", {"router": {"experts": 4, "top": 2}})
    idx, weights = plain.router(u, w["m.router"], 2)
    s = torch.sigmoid(u @ w["m.router"].t())
    assert (weights <= 1).all() and torch.equal(weights, torch.gather(s, 1, idx))
    t = 1
    want = sum(plain.gated_mlp((weights[t, k] * u[t])[None], w, f"m.e{int(idx[t, k])}.", plain.silu)[0] for k in range(2))
    assert torch.allclose(out[t], want, atol=1e-12)


def test_pages_behind_a_chunk_go_back_and_never_a_page_a_later_query_reads():
    """Two requests grow in uneven portions on a small pool: in the groups of chunked layers pages behind
    the reach are given back while the request lives and used again, and at every moment every key that a
    query at or after the computed length can still see (its own chunk from the chunk's first position) lies
    on a page the request holds."""
    import random
    from tiny_llm_infer_b200.cache import CacheManager
    cfg = PANOLORNS["P2"]["cfg"]                      # chunks of 24 and 7 beside a layer that keeps every key
    model = Model(describe_model(cfg), torch.float32, "cpu")
    page = 8
    cache = CacheManager(model.cache_needs(), page, {24: 14, None: 40, 7: 10}, max_slots=2, max_seq_len=160,
                         dtype=torch.float32, device=None)
    rng = random.Random(3)
    length = {"a": 0, "b": 0}
    cache.admit("a")
    cache.admit("b")
    seen_pages = {24: set(), 7: set()}
    reused = False
    while min(length.values()) < 150:
        name = rng.choice(["a", "b"])
        n = min(160 - length[name], rng.choice([1, 1, 2, 3, 5, 13]))
        if n <= 0:
            continue
        cache.reserve(name, length[name] + n)
        cache.commit(name, length[name] + n)
        length[name] += n
        cache.audit()
        for window, pages in cache.pages_of(name).items():
            if window is None:
                assert len(pages) == -(-length[name] // page)
                continue
            first_needed = (length[name] // window) * window if length[name] < 160 else length[name]
            table = cache.groups[window].table[cache.slot_of(name)]
            for key in range(first_needed, length[name]):
                assert table[key // page] >= 0, (window, name, key)
            assert len(pages) <= -(-window // page) + 2              # the reach, its ragged ends, the page ahead
            reused = reused or any(p in seen_pages[window] for p in pages)
            seen_pages[window].update(pages)
    assert reused
    cache.release("a")
    cache.release("b")
    cache.audit()
    assert cache.free_pages() == {24: 14, None: 40, 7: 10}
