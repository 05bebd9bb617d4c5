"""Kaketar on the GPU against the plain implementation (``plain_kaketar.py``).

Each mechanism alone, with sizes of its own: the embedding with learned positions and its norm; the residual
sum that norms a sub-layer's output and hands the stream on without a norm; the plain feed-forward and the
token side input; the paged attention kernels over cached latents (values inside the keys' rows, a learned
sink per head, a window) with inputs shaped so that one key stands out far back, just inside and just outside
the window, and so that the sink takes nearly all the weight; the delta rule (whole sequences, portions down
to one token, requests side by side, slots used again) with decays slow enough that the first tokens still
show at the end; the latent attention as a part.  Then whole models through ``bin/trace_run`` in every way of
cutting, the first tokens one by one, decoding while the window passes over decoded tokens, and greedy
generation through the engine's entry point under budgets and starved pools, with CUDA graphs.

Tolerances, as a row's root-mean-square difference (its mean taken off) over the row's own spread: float32
2e-4 against the plain implementation and between the ways of cutting; bfloat16 three times what a B200
shows per configuration."""
import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_kaketar as plain
import replay
from tiny_kaketar import KAKETARS, make_folder, prompt, requests_for

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F64 = torch.float64


def read_model(folder):
    from safetensors import safe_open
    cfg = json.loads((Path(folder) / "config.json").read_text())
    w = {}
    with safe_open(str(Path(folder) / "model.safetensors"), framework="pt") as fh:
        for name in fh.keys():
            w[name] = fh.get_tensor(name)
    return cfg, w


def make_ctx(rows, token_ids=None):
    """rows: (slot, first position, count) per portion -> the step's context, as the runner lays it out."""
    from tiny_llm_infer_b200.engine.batch import StepContext
    pos, slots, seg, tiles, dec, row = [], [], [], [], [], 0
    for s, (slot, p0, n) in enumerate(rows):
        pos += list(range(p0, p0 + n))
        slots += [slot] * n
        seg.append([slot, row, n, p0])
        if n == 1:
            dec.append(row)
        else:
            tiles += [[s, off] for off in range(0, n, 64)]
        row += n
    i32 = dict(dtype=torch.int32, device=DEV)
    return StepContext(tokens=row, token_ids=None if token_ids is None else torch.tensor(token_ids, **i32),
                       positions=torch.tensor(pos, **i32), token_slot=torch.tensor(slots, **i32), want_rows=None,
                       segments=[], seg_info=torch.tensor(seg, **i32),
                       dec_rows=torch.tensor(dec, **i32) if dec and len(dec) < row else None, n_dec=len(dec),
                       pf_tiles=torch.tensor(tiles, **i32).view(-1, 2), n_tiles=len(tiles),
                       decode_only=all(n == 1 for _, _, n in rows), max_context=max(p0 + n for _, p0, n in rows),
                       max_segment=max(n for _, _, n in rows))


# ----------------------------------------------------------------------------- small kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 200])
def test_embedding_with_positions_and_norm(dtype, width):
    from tiny_llm_infer_b200 import ops
    torch.manual_seed(width)
    table = torch.randn(50, width, device=DEV).to(dtype)
    pos_table = torch.randn(30, width, device=DEV).to(dtype)
    stored = (torch.rand(width, device=DEV) * 0.6 - 0.3).to(dtype)          # the gain minus one
    ids = torch.tensor([3, 49, -1, 0, 7], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 29, 5, 1, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, width, device=DEV)
    ops.embedding_norm(ids, table, out, 3.5, pos, pos_table, stored.float() + 1.0, 1e-5)
    x = table.double()[ids.clamp(min=0).long()] * 3.5 + pos_table.double()[pos.long()]
    want = plain.norm_around_one(x, stored.double(), 1e-5)
    want[2] = 0
    assert (out.double() - want).abs().max() < 1e-5
    ops.embedding_norm(ids, table, out, 1.0)                               # neither positions nor norm
    assert torch.equal(out[0], table[3].float()) and out[2].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [100, 520])
def test_sum_of_a_normed_output_without_a_norm_behind_it(dtype, width):
    from tiny_llm_infer_b200 import ops
    torch.manual_seed(width)
    h = torch.randn(9, width, device=DEV) * 3
    delta = (torch.randn(9, width, device=DEV) * 5).to(dtype)
    stored = (torch.rand(width, device=DEV) - 0.5).to(dtype)
    out = torch.empty(9, width, dtype=dtype, device=DEV)
    want = h.double() + plain.norm_around_one(delta.double(), stored.double(), 2e-6)
    ops.stream_add(h, delta, out, post_gain=stored.float() + 1.0, post_eps=2e-6)
    assert (h.double() - want).abs().max() < 2e-5                          # the stream itself stays float32
    assert (out.double() - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.1)
    before = h.clone()
    ops.stream_add(h, None, out)                                           # the first layer: nothing to add yet
    assert torch.equal(h, before) and torch.equal(out, h.to(dtype))
    ops.stream_add(h, delta, out)                                          # a plain delta
    assert (h.double() - (before.double() + delta.double())).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 6, 70, 300])
def test_plain_feed_forward_and_token_side_input(dtype, rows):
    from tiny_llm_infer_b200.engine.runner import strict_float32
    from tiny_llm_infer_b200.parts.registry import lookup
    strict_float32()
    torch.manual_seed(rows)
    hidden, inter, side, layers, vocab = 136, 200, 24, 3, 90
    w = {"l1.mlp.up": torch.randn(inter, hidden) * 0.2, "l1.mlp.down": torch.randn(hidden, inter) * 0.2,
         "l1.side.gate": torch.randn(side, hidden) * 0.3, "l1.side.proj": torch.randn(hidden, side) * 0.3,
         "l1.side.norm": torch.rand(hidden) + 0.5, "side.embed": torch.randn(vocab, layers * side)}
    w = {k: v.to(dtype).to(DEV) for k, v in w.items()}
    w64 = {k: v.double().cpu() for k, v in w.items()}
    x = (torch.randn(rows, hidden) * 1.5).to(dtype).to(DEV)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    ffn = lookup("feed_forward", "mlp")(hidden_size=hidden, intermediate_size=inter, dtype=dtype, device=DEV)
    ffn.load({"up": w["l1.mlp.up"], "down": w["l1.mlp.down"]})
    want = plain.dense_ff(x.double().cpu(), w64, "l1.mlp.")
    assert (ffn.forward(x, None).double().cpu() - want).abs().max() < tol * want.abs().max()
    part = lookup("feed_forward", "token_side")(hidden_size=hidden, side_dim=side, first_column=side, dtype=dtype, device=DEV)
    part.load({"gate": w["l1.side.gate"], "proj": w["l1.side.proj"]})
    tokens = torch.randint(0, vocab, (rows,)).tolist()
    ctx = make_ctx([(0, 0, rows)], tokens)
    ctx.memo["token_side_table"] = w["side.embed"]
    got = part.forward(x, ctx).double().cpu()
    got = plain.norm_plain(got, w64["l1.side.norm"], 1e-5)
    want = plain.token_side(x.double().cpu(), torch.tensor(tokens), w64, {"token_side": {"dim": side}, "norm": {"eps": 1e-5}}, 1)
    assert (got - want).abs().max() < tol * want.abs().max()


@pytest.mark.parametrize("act", ["gelu_erf", "gelu_tanh", "silu"])
@pytest.mark.parametrize("rows", [3, 1024, 40])
def test_products_with_a_plain_activation_in_their_epilogue(act, rows):
    """The weight-streaming product (few rows) and the tcgen05 product (many) with the activation on every
    output in the same kernel, against the float64 arithmetic of the same operands; in between the library's
    product followed by the activation kernel."""
    from tiny_llm_infer_b200 import ops
    torch.manual_seed(rows)
    k, n = 256, 8192
    x = torch.randn(rows, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    before = ops.launches
    got = ops.linear_act(x, w, act, torch.bfloat16)
    fused = rows <= ops.SKINNY_MAX_ROWS or ops.tcgen05_pays(rows, n, k, torch.bfloat16)
    assert fused == (rows != 40) and ops.launches - before == 1     # one kernel of this package either way: the fused
                                                                    # product, or the activation behind the library's product
    ops.check_error_word(x.device)
    f = {"gelu_erf": plain.gelu_erf, "gelu_tanh": plain.gelu_tanh, "silu": plain.silu}[act]
    want = f(x.double() @ w.double().t())
    assert (got.double() - want).abs().max() < 0.02 * want.abs().max()


# ----------------------------------------------------------------------------- attention over cached latents
def latent_reference(q, kv, heads, dv, scale, window, sink):
    """q [T, H, dk], kv [T, dk] float64 (one shared key per token whose first dv elements are its value)."""
    T = q.shape[0]
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    seen = (j <= i) & ((i - j < window) if window else True)
    outs = []
    for h in range(heads):
        s = (q[:, h] @ kv.T * scale).masked_fill(~seen, -math.inf)
        both = torch.cat([s, sink[h].expand(T, 1)], 1)
        outs.append(torch.softmax(both, 1)[:, :T] @ kv[:, :dv])
    return torch.cat(outs, 1)


LATENT_CASES = [dict(H=4, dk=80, dv=64, page=16, window=40), dict(H=8, dk=48, dv=40, page=8, window=23),
                dict(H=16, dk=112, dv=96, page=16, window=72), dict(H=3, dk=64, dv=56, page=8, window=7),
                dict(H=20, dk=32, dv=24, page=16, window=None), dict(H=2, dk=160, dv=144, page=32, window=100)]


@pytest.mark.parametrize("case", LATENT_CASES, ids=lambda c: f"h{c['H']}k{c['dk']}v{c['dv']}w{c['window']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_over_latents_with_learned_sinks(case, dtype):
    from tiny_llm_infer_b200 import ops
    H, dk, dv, page, window = case["H"], case["dk"], case["dv"], case["page"], case["window"]
    scale = 1.2 / math.sqrt(dk)
    lengths = (150, 75, 1, 260)
    g = torch.Generator().manual_seed(dk + dv)
    sink = torch.randn(H, generator=g, dtype=F64) * 2
    reqs = []
    for n, L in enumerate(lengths):
        q = torch.randn(L, H, dk, generator=g, dtype=F64)
        kv = torch.randn(L, dk, generator=g, dtype=F64)
        if n == 1:
            kv = -q[:, 0].clone() * 3
            q = q[:, :1].expand(L, H, dk).clone()                 # every score strongly negative: the sink takes the weight
        else:
            for pos in range(L - 1, 0, -max(3, L // 9)):
                edge = max(0, pos - window + 1) if window else pos // 3
                for key, gain in ((edge, 4.0), (edge - 1, 6.0)):   # just inside, and (louder) just outside
                    if 0 <= key < pos:
                        kv[key] = q[pos, pos % H] * gain
        reqs.append((q.to(dtype).double(), kv.to(dtype).double()))
    want = [latent_reference(q, kv, H, dv, scale, window, sink) for q, kv in reqs]
    max_pages = -(-max(lengths) // page)
    n_pages = sum(-(-L // page) for L in lengths) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lengths), max_pages), -1, dtype=torch.int32)
    plane = torch.zeros(n_pages, 1, page, dk, dtype=dtype, device=DEV)
    for slot, L in enumerate(lengths):
        for i in range(-(-L // page)):
            table[slot, i] = order.pop()
            chunk = reqs[slot][1][i * page:(i + 1) * page]
            plane[table[slot, i], 0, :chunk.shape[0]] = chunk.to(dtype).to(DEV)
    table_d, sink_d = table.to(DEV), sink.float().to(DEV)

    def run(rows, fast):
        qs = torch.cat([reqs[slot][0][p0:p0 + n].reshape(n, -1) for slot, p0, n in rows]).to(dtype).to(DEV).contiguous()
        ctx = make_ctx(rows)
        out = torch.empty(qs.shape[0], H * dv, dtype=dtype, device=DEV)
        ops.attention_biased(qs, plane, plane, ctx.positions, ctx.token_slot, table_d, page, H, 1, dk, dv, scale, out,
                             window=window or 0, sink=True, sink_logits=sink_d, ctx=ctx if fast else None,
                             values_in_keys=True)
        torch.cuda.synchronize()
        expect = torch.cat([want[slot][p0:p0 + n] for slot, p0, n in rows])
        return ((out.double().cpu() - expect).abs().max() / expect.abs().max()).item()   # values are as loud as the keys

    tol = 2e-5 if dtype == torch.float32 else 2e-2
    ways = (False, True) if dtype == torch.bfloat16 else (False,)
    whole = [(s, 0, L) for s, L in enumerate(lengths)]
    edges = [p for p in (window, page) if p]
    singles = sorted({p for e in edges for p in (e - 1, e, e + 1, 2 * e - 1, 2 * e) if 0 < p < 150} | {149, 1})
    mixed = [(0, p, 1) for p in singles[:3]] + [(3, 100, 2), (3, 131, 129)] + [(1, 40, 35)]
    for fast in ways:
        assert run(whole, fast) < tol
        assert run(mixed, fast) < tol
        for p in singles:
            assert run([(0, p, 1), (3, 259, 1), (2, 0, 1), (1, 74, 1)], fast) < tol, p


# ----------------------------------------------------------------------------- the delta rule as a part
DELTA_CASES = [dict(H=4, G=2, dk=32, dv=48, taps=4, ranks=(8, 16)), dict(H=6, G=3, dk=20, dv=24, taps=3, ranks=(8, 24)),
               dict(H=1, G=1, dk=72, dv=40, taps=2, ranks=(8, 8)), dict(H=2, G=1, dk=128, dv=128, taps=2, ranks=(8, 16)),
               dict(H=5, G=5, dk=16, dv=16, taps=5, ranks=(24, 8)), dict(H=3, G=3, dk=200, dv=8, taps=1, ranks=(8, 8))]


def delta_part(case, dtype, hidden=96, seed=0):
    from tiny_llm_infer_b200.parts.registry import lookup
    params = dict(hidden_size=hidden, heads=case["H"], kv_heads=case["G"], key_dim=case["dk"], value_dim=case["dv"],
                  conv_taps=case["taps"], decay_rank=case["ranks"][0], gate_rank=case["ranks"][1], norm_eps=1e-5)
    cls = lookup("mixer", "channel_delta")
    g = torch.Generator().manual_seed(seed + case["dk"])
    w = {}
    for name, spec in cls.param_specs(**params).items():
        std = 0.5 if spec.init == "unit" else (0.3 if name in ("q", "k", "v", "b", "o") else 0.5)
        w[name] = torch.randn(spec.shape, generator=g) * std
    w["norm"] = torch.rand(case["dv"], generator=g) + 0.5
    w["a2"] *= 0.05                                              # the decay's input-dependent part stays small, so that
    w["dt_bias"].view(case["H"], case["dk"])[::2] -= 6.0        # every second head forgets slowly
    w = {k: v.to(dtype) for k, v in w.items()}
    part = cls(dtype=dtype, device=DEV, **params)
    part.load({k: v.to(DEV) for k, v in w.items()})
    mixer = dict(heads=case["H"], kv_heads=case["G"], dim=case["dk"], vdim=case["dv"], conv=case["taps"])
    return part, {"m." + k: v.double() for k, v in w.items()}, mixer


@pytest.mark.parametrize("case", DELTA_CASES, ids=lambda c: f"h{c['H']}g{c['G']}k{c['dk']}v{c['dv']}t{c['taps']}")
def test_delta_rule_whole_in_portions_and_side_by_side(case):
    """float32: one sequence whole, then the same cut into portions of every size down to one token, beside
    a second request in the same steps, in slots that are then given to other requests."""
    from tiny_llm_infer_b200.cache.manager import LayerCacheView
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    dtype = torch.float32
    part, w64, mixer = delta_part(case, dtype)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(L, 96, generator=g).to(dtype) for L in (230, 61, 1)]
    want = [plain.channel_delta(x.double(), w64, "m.", mixer, 1e-5) for x in xs]
    state = torch.zeros(4, part.state_spec().shape[0], device=DEV)
    view = LayerCacheView(kv=None, block_table=None, page_size=16, writes=True, state=state)

    def step(rows):
        x = torch.cat([xs[r][p0:p0 + n] for r, _, p0, n in rows]).to(DEV)
        ctx = make_ctx([(slot, p0, n) for _, slot, p0, n in rows])
        got = part.forward(x, ctx, view).double().cpu()
        expect = torch.cat([want[r][p0:p0 + n] for r, _, p0, n in rows])
        return ((got - expect).abs().max() / expect.abs().max()).item()

    assert step([(0, 2, 0, 230), (1, 0, 0, 61), (2, 3, 0, 1)]) < 2e-5
    # the first tokens still show at the end: without the state carried over 200 tokens the answer differs
    short = plain.channel_delta(xs[0][30:].double(), w64, "m.", mixer, 1e-5)
    assert (short[-1] - want[0][-1]).abs().max() > 1e-3 * want[0].abs().max()
    # slots 2 and 0 are used again (zeroed, as the cache manager does at admission), by other requests
    state[2].zero_()
    state[0].zero_()
    sizes = [1, 1, 2, 1, 3, 2, 17, 2, 1, 16, 33, 1, 64, 5]
    at0 = at1 = worst = 0
    k = 0
    while at0 < 230:
        n0 = min(sizes[k % len(sizes)], 230 - at0)
        rows = [(0, 0, at0, n0)]
        if at1 < 61 and k % 3 != 1:                              # the second request sits some steps out
            n1 = min(sizes[(k + 5) % len(sizes)], 61 - at1)
            rows.append((1, 2, at1, n1))
            at1 += n1
        worst = max(worst, step(rows))
        at0 += n0
        k += 1
    assert at1 == 61 and worst < 2e-5, worst


@pytest.mark.parametrize("case", DELTA_CASES[:4], ids=lambda c: f"h{c['H']}g{c['G']}k{c['dk']}v{c['dv']}t{c['taps']}")
def test_delta_rule_in_bfloat16(case):
    from tiny_llm_infer_b200.cache.manager import LayerCacheView
    part, w64, mixer = delta_part(case, torch.bfloat16)
    x = torch.randn(150, 96, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    want = plain.channel_delta(x.double(), w64, "m.", mixer, 1e-5)
    state = torch.zeros(2, part.state_spec().shape[0], device=DEV)
    view = LayerCacheView(kv=None, block_table=None, page_size=16, writes=True, state=state)
    got = torch.cat([part.forward(x[a:b].to(DEV), make_ctx([(1, a, b - a)]), view) for a, b in ((0, 100), (100, 101), (101, 150))])
    err = (got.double().cpu() - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt()
    assert err < 0.03, err


# ----------------------------------------------------------------------------- the latent attention as a part
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [dict(H=4, dn=32, dr=16, dv=32, qr=48, kr=64, rd=16, window=40, page=16,
                                        scaling=dict(factor=8.0, original=64.0, fast=16.0, slow=2.0)),
                                   dict(H=3, dn=24, dr=8, dv=40, qr=40, kr=56, rd=4, window=7, page=8, scaling=None),
                                   dict(H=20, dn=8, dr=8, dv=8, qr=24, kr=24, rd=8, window=None, page=16,
                                        scaling=dict(factor=2.0, original=32.0, fast=8.0, slow=1.0))],
                         ids=["h4", "h3", "h20"])
def test_latent_attention_part(dtype, sizes):
    from tiny_llm_infer_b200.cache.manager import LayerCacheView
    from tiny_llm_infer_b200.engine.runner import strict_float32
    from tiny_llm_infer_b200.parts.registry import lookup
    strict_float32()
    s, hidden = sizes, 104
    params = dict(hidden_size=hidden, heads=s["H"], plain_dim=s["dn"], rot_dim=s["dr"], value_dim=s["dv"], q_rank=s["qr"],
                  kv_rank=s["kr"], scale=0.9 / math.sqrt(s["dn"] + s["dr"]), norm_eps=1e-5, rot_base=3000.0,
                  rot_dims=s["rd"], scaling=s["scaling"], window=s["window"], sink=True, output_gate=True)
    cls = lookup("mixer", "latent_attention")
    g = torch.Generator().manual_seed(s["H"])
    w = {}
    for name, spec in cls.param_specs(**params).items():
        w[name] = (torch.rand(spec.shape, generator=g) + 0.5) if spec.init == "norm" else torch.randn(spec.shape, generator=g) * 0.4
    w["sink"] = w["sink"] * 4
    w = {k: v.to(dtype) for k, v in w.items()}
    part = cls(dtype=dtype, device=DEV, **params)
    part.load({k: v.to(DEV) for k, v in w.items()})
    mixer = dict(heads=s["H"], dim=s["dn"], rot_dim=s["dr"], vdim=s["dv"], kv_rank=s["kr"], scale=params["scale"],
                 rot=dict(base=3000.0, dims=s["rd"], scaling=s["scaling"]))
    if s["window"]:
        mixer["mask"] = {"size": s["window"]}
    L, page = 170, s["page"]
    x = (torch.randn(L, hidden, generator=g) * 1.5).to(dtype)
    want = plain.latent_attention(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", mixer, 1e-5)
    n_pages = -(-L // page) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((2, n_pages), -1, dtype=torch.int32)
    table[1, :-(-L // page)] = torch.tensor(order[:-(-L // page)], dtype=torch.int32)
    plane = torch.zeros(n_pages, 1, page, s["kr"] + s["dr"], dtype=dtype, device=DEV)
    view = LayerCacheView(kv=None, block_table=table.to(DEV), page_size=page, writes=True, state=None,
                          window=s["window"], planes=(plane,))
    cuts = [0, 90, 91, 93, 120, 121, 122, 170]
    got = torch.cat([part.forward(x[a:b].to(DEV), make_ctx([(1, a, b - a)]), view) for a, b in zip(cuts, cuts[1:])])
    err = ((got.double().cpu() - want).abs().max() / want.abs().max()).item()
    assert err < (3e-5 if dtype == torch.float32 else 0.05), err


def test_rotation_frequencies_with_stretching():
    from tiny_llm_infer_b200.parts.latent_attention import rotation_frequencies
    for dims, base, sc in ((16, 250000.0, dict(factor=4.0, original=512, fast=32.0, slow=1.0)), (8, 1000.0, None),
                           (32, 10000.0, dict(factor=16.0, original=128, fast=8.0, slow=2.0))):
        got, mag = rotation_frequencies(dims, base, sc)
        want, want_mag = plain.yarn_frequencies(dict(dims=dims, base=base, scaling=sc))
        assert torch.equal(got, want.float()) and mag == want_mag


# ----------------------------------------------------------------------------- whole models, every way of cutting
BF16_RMS = {"K1": 0.25, "K2": 0.1, "K3": 0.1, "K4": 0.36}          # three times what a B200 shows (0.082, 0.033, 0.033, 0.119) as a row's
                                                       # root-mean-square difference over the row's spread


@pytest.fixture(scope="module", params=sorted(KAKETARS))
def case(request, tmp_path_factory):
    name = request.param
    tiny = KAKETARS[name]
    folder = make_folder(tiny, tmp_path_factory.mktemp(name))
    cfg, w = read_model(folder)
    reqs = requests_for(tiny)
    want = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    tb = replay.TraceBuilder()
    replay.whole(tb, reqs)
    replay.tail_one_by_one(tb, reqs)
    replay.portions(tb, reqs)
    replay.mixed(tb, reqs, seed=7)
    return name, tiny, folder, cfg, w, want, tb, reqs


def run_tool(folder, dtype, out, tb, page_size):
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(tb.max_tokens), "--page-size", str(page_size), "--max-requests", "4"]
    res = subprocess.run(cmd, input=tb.text(), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    done = [l for l in res.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(tb.steps))]


def relative_rows(out, tb, want, vocab):
    """Per way of cutting every row's root-mean-square difference from the plain implementation (the mean
    taken off) over the row's own spread, and the same between each way and the whole-request run."""
    errors, base, spread, rows_of = {}, {}, {}, {}
    for step, rows in tb.expect.items():
        got = replay.read_logits(out, step, vocab).astype(np.float64)
        assert np.isfinite(got).all()
        for r, (name, pos) in enumerate(rows):
            rows_of[(name, pos)] = got[r]
            ref = want[name[1:]][pos]
            d = got[r] - ref
            errors.setdefault(name[0], []).append(float(np.sqrt(np.mean((d - d.mean()) ** 2)) / ref.std()))
            if name[0] == "w":
                base[(name[1:], pos)] = got[r]
    for (name, pos), row in rows_of.items():
        if name[0] != "w" and (name[1:], pos) in base:
            ref = base[(name[1:], pos)]
            spread.setdefault(name[0], []).append(float(np.sqrt(np.mean((row - ref) ** 2)) / ref.std()))
    return {k: np.array(v) for k, v in errors.items()}, {k: np.array(v) for k, v in spread.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_ways_of_cutting(case, dtype, tmp_path):
    name, tiny, folder, cfg, w, want, tb, reqs = case
    out = tmp_path / "out"
    run_tool(folder, dtype, out, tb, tiny["page_size"])
    errors, spread = relative_rows(out, tb, want, cfg["vocab"])
    assert set(errors) == {"w", "t", "p", "m"}
    summary = {k: (round(float(np.percentile(v, 50)), 6), round(float(v.max()), 6)) for k, v in errors.items()}
    between = {k: (round(float(np.percentile(v, 50)), 6), round(float(v.max()), 6)) for k, v in spread.items()}
    print(f"\n[{name} {dtype}] against plain (median, max) {summary}; between the ways (median, max) {between}")
    limit = 2e-4 if dtype == "float32" else BF16_RMS[name]
    assert max(v.max() for v in errors.values()) < limit, summary
    assert max(v.max() for v in spread.values()) < limit, between


def test_first_tokens_one_by_one_and_a_window_passing_over_decoded_tokens(case, tmp_path):
    """One token at a time from an empty cache and an empty state, across page and window edges, beside a
    second request that decodes from the middle of a page; then the last 140 tokens of a long request one
    by one, more than any window of the configurations, so that decoded tokens leave it again."""
    name, tiny, folder, cfg, w, want, _, reqs = case
    a, b = reqs["0"], reqs["1"]
    tb = replay.TraceBuilder()
    tb.step([("f1", b[:29])])
    for i in range(len(a)):
        extra = [("f1", b[29 + i:30 + i])] if 29 + i < len(b) else []
        tb.step([("f0", a[i:i + 1])] + extra)
    tb.step([], end=["f0", "f1"])
    long_one = max(reqs, key=lambda r: len(reqs[r]))
    replay.tail_one_by_one(tb, {long_one: reqs[long_one]}, tail=min(140, len(reqs[long_one]) - 3), tag="f")
    out = tmp_path / "out"
    run_tool(folder, "float32", out, tb, tiny["page_size"])
    errors, _ = relative_rows(out, tb, want, cfg["vocab"])
    assert errors["f"].max() < 2e-4, errors["f"].max()


def test_a_missing_mechanism_would_show(case):
    """The weights of the tiny models make every mechanism matter: the plain implementation without the sink,
    with a window one token longer, without the first tokens' state, or without the side input moves the
    logits far beyond the tolerances above."""
    name, tiny, folder, cfg, w, want, _, reqs = case
    toks = max(reqs.values(), key=len)
    ref = plain.forward(cfg, w, toks).numpy()

    def moved(changed_cfg=None, changed_w=None):
        got = plain.forward(changed_cfg or cfg, changed_w or w, toks).numpy()
        d = got - ref
        return float((np.sqrt(((d - d.mean(1, keepdims=True)) ** 2).mean(1)) / ref.std(1)).max())

    no_sink = {k: (torch.full_like(v, -80.0) if k.endswith(".sink") else v) for k, v in w.items()}
    assert moved(changed_w=no_sink) > 0.01
    longer = json.loads(json.dumps(cfg))
    for layer in longer["layers"]:
        if layer["type"] == "latent_attention" and layer["mixer"].get("mask"):
            layer["mixer"]["mask"]["size"] += 1
    assert moved(changed_cfg=longer) > 0.003
    if cfg.get("token_side"):
        no_side = {k: (torch.zeros_like(v) if k == "side.embed" else v) for k, v in w.items()}
        assert moved(changed_w=no_side) > 0.01
    cut = plain.forward(cfg, w, toks[40:]).numpy()[-1] - ref[-1]     # the first forty tokens forgotten
    assert np.sqrt(((cut - cut.mean()) ** 2).mean()) / ref[-1].std() > 0.003


# ----------------------------------------------------------------------------- generation through the entry point
def plain_greedy(cfg, w, prompt_ids, n):
    ids = list(prompt_ids)
    for _ in range(n):
        ids.append(int(plain.forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt_ids):]


@pytest.mark.parametrize("name", ["K1", "K2"])
@pytest.mark.parametrize("budget,blocks", [(256, 64), (8, 64), (7, 9)])
def test_greedy_generation_equals_plain(name, budget, blocks, tmp_path):
    """Budgets down to seven tokens a step and a pool so small that requests are preempted and computed
    again (their state starts from zero again), with decode steps replayed as CUDA graphs."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = KAKETARS[name]
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((5, 27, 53, 1))]
    want = [plain_greedy(cfg, w, p, 12) for p in prompts]
    llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=blocks, block_size=tiny["page_size"],
              max_num_batched_tokens=budget, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.cache.audit()
    assert all(v == blocks for v in llm.cache.free_pages().values())


def test_a_model_of_delta_rule_layers_alone(tmp_path):
    """No layer with a cache: the cache manager has no group of pages at all and only the state slots."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    from tiny_kaketar import delta
    from tiny_llm_infer_b200.config.kaketar import KaketarConfig
    tiny = dict(cfg=KaketarConfig(vocab=150, width=64, max_positions=96, embedding_scale=1.5, norm_eps=1e-5, layers=(
        delta(2, 1, 24, 16, 3, (8, 8), ff=80), delta(4, 4, 8, 8, 2, (8, 8))), logit_softcap=None, side_dim=4),
        seed=31, std=0.1, norm_range=(0.7, 1.3))
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((19, 3, 40))]
    want = [plain_greedy(cfg, w, p, 10) for p in prompts]
    llm = LLM(str(folder), dtype="float32", max_model_len=96, num_kv_blocks=8, block_size=16,
              max_num_batched_tokens=16, max_num_seqs=2)
    assert not llm.cache.groups
    outs = llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.cache.audit()


def test_long_decoding_in_bfloat16_through_graphs(tmp_path):
    """Sixty tokens each for three requests, decode steps replayed as CUDA graphs, bfloat16 kernels: every token
    is the plain implementation's choice given the same beginning, or within a near-tie of it."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = KAKETARS["K3"]
    folder = make_folder(tiny, tmp_path)
    cfg, w = read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((60, 9, 190))]
    llm = LLM(str(folder), dtype="bfloat16", max_model_len=256, num_kv_blocks=24, block_size=32,
              max_num_batched_tokens=64, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=60, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p) + list(o.token_ids)
        logits = plain.forward(cfg, w, ids[:-1]).numpy()
        near = [logits[len(p) - 1 + i][tok] >= logits[len(p) - 1 + i].max() - 0.15 * logits[len(p) - 1 + i].std()
                for i, tok in enumerate(o.token_ids)]
        assert sum(near) >= 0.9 * len(near), near


def test_command_line_writes_and_runs_a_model(tmp_path):
    """``bin/model_main``: a random Kaketar model from its config.json, greedy tokens equal to the plain
    implementation's in float32, and seeded sampling that repeats itself."""
    tiny = KAKETARS["K2"]
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny["cfg"].to_dict()))
    folder = tmp_path / "model"
    tool = [sys.executable, str(ROOT / "bin" / "model_main")]
    res = subprocess.run(tool + ["--write-random-model", str(folder), "--config", str(cfg_path), "--random-weights", "21",
                                 "--weight-std", "0.07"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    cfg, w = read_model(folder)
    prompts = [prompt(40 + i, n, cfg["vocab"]) for i, n in enumerate((9, 31))]
    ids = [a for p in prompts for a in ("--prompt-ids", ",".join(map(str, p)))]
    common = tool + ["--infer", "--model", str(folder), "--max-seq-len", "128", "--max-new-tokens", "7"] + ids
    res = subprocess.run(common + ["--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    got = [[int(x) for x in line.split(",")] for line in res.stdout.strip().splitlines()[-2:]]
    assert got == [plain_greedy(cfg, w, p, 7) for p in prompts]
    draws = []
    for _ in range(2):
        res = subprocess.run(common + ["--dtype", "bfloat16", "--temperature", "0.8", "--top-p", "0.9", "--seed", "5"],
                             capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        draws.append(res.stdout.strip().splitlines()[-2:])
    assert draws[0] == draws[1]
