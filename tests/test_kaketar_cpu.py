"""Kaketar without a GPU: its configuration (config.json keys, the sizes only the checkpoint gives), the
description the model is assembled from, what its mixers ask of the cache manager, and the plain
implementation's own mechanisms on cases small enough to check by other means."""
import json
import math

import pytest
import torch

import plain_kaketar as plain
from tiny_kaketar import KAKETARS, make_folder

from tiny_llm_infer_b200.config import ConfigError, config_from_dict, load_config
from tiny_llm_infer_b200.config.base import describe_model
from tiny_llm_infer_b200.config.kaketar import KaketarConfig
from tiny_llm_infer_b200.models.model import Model, expected_tensors
from tiny_llm_infer_b200.parts import delta_rule
from tiny_llm_infer_b200.weights.safetensors_io import tensor_shapes


@pytest.mark.parametrize("name", sorted(KAKETARS))
def test_config_round_trip_and_tensor_names(name, tmp_path):
    tiny = KAKETARS[name]
    folder = make_folder(tiny, tmp_path)
    raw = json.loads((folder / "config.json").read_text())
    assert raw["architecture"] == "Kaketar" and "decay_rank" not in json.dumps(raw)
    cfg = load_config(folder)
    assert isinstance(cfg, KaketarConfig) and cfg == tiny["cfg"] and cfg.to_dict() == raw
    bare = config_from_dict(raw)                       # without the checkpoint the low ranks are not known
    assert bare != cfg and bare.with_tensor_shapes(tensor_shapes(folder)) == cfg
    expected, _ = expected_tensors(describe_model(cfg))
    shapes = tensor_shapes(folder)
    assert {k: tuple(v.shape) for k, v in expected.items()} == shapes
    for i, layer in enumerate(cfg.layers):
        assert (f"l{i}.norm2" in expected) == (layer.mlp is not None)
        assert (f"l{i}.side.gate" in expected) == (cfg.side_dim is not None)
        assert (f"l{i}.mix.A_log" in expected) == (layer.type == "channel_delta")
        assert (f"l{i}.mix.sink" in expected) == (layer.type == "latent_attention")
    assert ("side.embed" in expected) == (cfg.side_dim is not None)
    if cfg.side_dim is not None:
        assert expected["side.embed"].shape == (cfg.vocab, cfg.side_dim * len(cfg.layers))


def test_config_errors():
    good = KAKETARS["K1"]["cfg"].to_dict()
    for path, value in ((("layers", 0, "type"), "attention"), (("layers", 0, "mlp", "kind"), "moe"),
                        (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 7),
                        (("layers", 0, "mixer", "rot", "dims"), 18), (("norm", "eps"), 0.0),
                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 1, "mixer", "conv"), 0),
                        (("logit_softcap",), -1.0), (("token_side", "dim"), 0), (("max_positions",), 0)):
        raw = json.loads(json.dumps(good))
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(raw)
    for path in (("layers", 0, "mixer", "scale"), ("layers", 0, "mixer", "rot"), ("layers", 1, "mixer", "conv"), ("max_positions",)):
        raw = json.loads(json.dumps(good))
        at = raw
        for key in path[:-1]:
            at = at[key]
        del at[path[-1]]
        with pytest.raises(ConfigError):
            config_from_dict(raw)


def test_what_the_mixers_ask_of_the_cache_manager():
    cfg = KAKETARS["K2"]["cfg"]
    model = Model(describe_model(cfg), torch.float32, "cpu")
    needs = model.cache_needs()
    assert len(needs) == len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        spec, state = needs[i]
        m = layer.mixer
        if layer.type == "channel_delta":
            assert spec is None and state.dtype == "float32"
            lanes = delta_rule.scan_lanes(m.dim)
            rows = -(-m.dim // lanes) * lanes                       # key rows, rounded up to whole lanes
            assert state.shape == (m.heads * rows * m.vdim + (m.conv - 1) * (2 * m.kv_heads * m.dim + m.heads * m.vdim),)
            assert rows >= m.dim and -(-m.dim // lanes) <= delta_rule.SCAN_MAX_ROWS
        else:
            assert state is None and spec.planes == ((1, m.kv_rank + m.rot_dim),) and spec.window == m.window
    from tiny_llm_infer_b200.cache import CacheManager
    cache = CacheManager(needs, 8, 12, max_slots=3, max_seq_len=96, dtype=torch.float32, device="cpu")
    assert set(cache.groups) == {7, None}                           # the window of 7 gives pages back, the other keeps all
    cache.admit("a")
    cache.reserve("a", 40)
    cache.commit("a", 40)
    assert cache.free_pages() == {7: 11, None: 7}
    cache.state[0][0].fill_(3.0)
    cache.release("a")
    cache.admit("b")                                                # the slot comes back with its state zeroed
    assert cache.slot_of("b") == 0 and float(cache.state[0][0].abs().max()) == 0.0


def test_plain_delta_rule_against_its_closed_form_for_two_tokens():
    """One head, no convolution memory (one tap), two tokens: S1 = k1 u1^T, then the second step by hand."""
    torch.manual_seed(0)
    dk, dv, D = 4, 3, 6
    m = dict(heads=1, kv_heads=1, dim=dk, vdim=dv, conv=1)
    w = {"m." + k: torch.randn(s, dtype=torch.float64) for k, s in dict(
        q=(dk, D), k=(dk, D), v=(dv, D), b=(1, D), A_log=(1,), norm=(dv,), a1=(2, D), a2=(dk, 2), dt_bias=(dk,),
        g1=(2, D), g2=(dv, 2), o=(D, dv)).items()}
    for n in ("q", "k", "v"):
        w[f"m.{n}.conv"] = torch.randn(w["m." + n].shape[0], 1, dtype=torch.float64)
    h = torch.randn(2, D, dtype=torch.float64)
    got = plain.channel_delta(h, w, "m.", m, 1e-5)

    def parts(x):
        q = plain.silu((w["m.q"] @ x) * w["m.q.conv"][:, 0])
        k = plain.silu((w["m.k"] @ x) * w["m.k.conv"][:, 0])
        v = plain.silu((w["m.v"] @ x) * w["m.v.conv"][:, 0])
        q = q / torch.sqrt(q @ q + 1e-6) / math.sqrt(dk)
        k = k / torch.sqrt(k @ k + 1e-6)
        beta = torch.sigmoid(w["m.b"] @ x)
        g = torch.exp(-torch.exp(w["m.A_log"]) * torch.log1p(torch.exp(w["m.a2"] @ (w["m.a1"] @ x) + w["m.dt_bias"])))
        gate = torch.sigmoid(w["m.g2"] @ (w["m.g1"] @ x))
        return q, k, v, beta, g, gate

    def read_out(o, gate):
        return w["m.o"] @ (o / torch.sqrt((o * o).mean() + 1e-5) * w["m.norm"] * gate)

    q1, k1, v1, b1, g1, gate1 = parts(h[0])
    S1 = torch.outer(k1, b1 * v1)
    q2, k2, v2, b2, g2, gate2 = parts(h[1])
    S1d = g2[:, None] * S1
    S2 = S1d + torch.outer(k2, b2 * (v2 - S1d.T @ k2))
    want = torch.stack([read_out(S1.T @ q1, gate1), read_out(S2.T @ q2, gate2)])
    assert torch.allclose(got, want, atol=1e-12)


def test_plain_rotation_and_window():
    rot = dict(base=100.0, dims=4, scaling=None)
    x = torch.arange(12, dtype=torch.float64).view(2, 6) + 1
    y = plain.rotate_pairs(x, torch.tensor([0, 3]), rot)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, 4:], x[:, 4:])       # position 0 and the unrotated rest
    a = 3 * 100.0 ** (-2 / 4)
    assert math.isclose(float(y[1, 2]), x[1, 2] * math.cos(a) - x[1, 3] * math.sin(a), rel_tol=1e-12)
    assert math.isclose(float(y[1, 3]), x[1, 3] * math.cos(a) + x[1, 2] * math.sin(a), rel_tol=1e-12)
    f, mag = plain.yarn_frequencies(dict(base=100.0, dims=8, scaling=dict(factor=4.0, original=16, fast=4.0, slow=1.0)))
    plain_f = 100.0 ** (-2 * torch.arange(4, dtype=torch.float64) / 8)
    assert float(f[0]) == 1.0 and math.isclose(float(f[-1]), float(plain_f[-1]) / 4.0) and mag == 0.1 * math.log(4.0) + 1.0
