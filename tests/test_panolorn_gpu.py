"""Panolorn on the GPU against the plain implementation (``plain_panolorn.py``).

Each mechanism alone, with sizes of its own: the output norm fused with the residual sum and the next
norm; the score-modified attention kernels (general, tensor-core prompt tiles, one-token rows) over a
hand-made paged cache with scrambled pages, with inputs shaped so that one key stands out far back, just
inside and just outside a chunk or a window, and so that the sink takes nearly all the weight; the router
and the experts' products; the gated unit with the tanh GELU.  Then whole models through ``bin/trace_run``
in every way of cutting (whole, last tokens one by one, portions down to two tokens, mixed batches on a
pool so small that pages and slots are used again), decoding across many chunk edges, the first tokens one
by one, and greedy generation through the engine's entry point under budgets and starved pools.

Tolerances, as a row's root-mean-square difference (its mean taken off) over the row's own spread: float32
1e-4 against the plain implementation and between the ways of cutting; bfloat16 three times what a B200
shows per configuration, and half of that between the ways of cutting.  The prompts of the whole-model
comparisons are searched so that no router meets a near-tie on them (``plain.decisive_tokens``): in
bfloat16 such a choice falls either way and moves the row by a whole expert's output."""
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_panolorn as plain
import replay
from tiny_panolorn import PANOLORNS, make_folder, prompt, requests_for

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F64 = torch.float64


# ----------------------------------------------------------------------------- norms
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [100, 200, 4096 + 8])
def test_output_norm_fused_with_sum_and_next_norm(dtype, width):
    from tiny_llm_infer_b200 import ops
    torch.manual_seed(width)
    rows = 37
    h = torch.randn(rows, width, device=DEV) * 3
    delta = (torch.randn(rows, width, device=DEV) * 5).to(dtype)
    post = (torch.rand(width, device=DEV) + 0.5).to(dtype)
    gain = (torch.rand(width, device=DEV) + 0.5).to(dtype)
    d64 = delta.double().cpu()
    v = h.double().cpu() + plain.rms_norm(d64, post.double().cpu(), 1e-5)
    want = plain.rms_norm(v, gain.double().cpu(), 2e-6)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    # only some rows, the stream untouched (the model's last norm)
    pick = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(4, width, dtype=dtype, device=DEV)
    before = h.clone()
    ops.add_rmsnorm(h, delta, gain, 2e-6, out, pick, post_gain=post, post_eps=1e-5)
    assert torch.equal(h, before)
    assert (out.double().cpu() - want[pick.long().cpu()]).abs().max() < tol
    # every row, the sum written back in float32
    out = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.add_rmsnorm(h, delta, gain, 2e-6, out, post_gain=post, post_eps=1e-5)
    assert (h.double().cpu() - v).abs().max() < 1e-5
    assert (out.double().cpu() - want).abs().max() < tol


def test_embedding_scale():
    from tiny_llm_infer_b200 import ops
    table = torch.randn(50, 72, device=DEV).to(torch.bfloat16)
    ids = torch.tensor([3, 49, -1, 0], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 72, device=DEV)
    ops.embedding(ids, table, out, 13.25)
    want = table.float()[ids.clamp(min=0).long()] * 13.25
    want[2] = 0
    assert torch.equal(out, want)


# ----------------------------------------------------------------------------- attention kernels
def reference_attention(q, k, v, heads, kv_heads, scale, softcap, chunk, window, sink, slopes, gate):
    """[T, heads * dv] float64 for one whole sequence; q [T, H, dk], k [T, G, dk], v [T, G, dv] float64."""
    T = q.shape[0]
    outs = []
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = plain.attention_scores(q[:, h], k[:, g], h, heads, scale, softcap, chunk)
        if slopes is None:                      # take the bias off again
            s = s + plain.slopes(heads)[h] * (i - j).to(F64)
        if window:
            s = s.masked_fill(j < i - window + 1, float("-inf"))
        p = plain.sink_softmax(s) if sink else torch.softmax(s, -1)
        outs.append(p @ v[:, g])
    o = torch.cat(outs, -1)
    return o * torch.sigmoid(gate) if gate is not None else o


ATTENTION_CASES = [
    # heads, kv, dk, dv, page, chunk, window, softcap, sink, bias, gate
    dict(H=4, G=2, dk=64, dv=64, page=16, chunk=50, window=None, softcap=20.0, sink=True, bias=True, gate=True),
    dict(H=8, G=1, dk=80, dv=80, page=32, chunk=110, window=None, softcap=45.0, sink=True, bias=True, gate=True),
    dict(H=6, G=6, dk=32, dv=48, page=8, chunk=24, window=None, softcap=8.0, sink=True, bias=True, gate=True),
    dict(H=3, G=1, dk=40, dv=24, page=16, chunk=None, window=None, softcap=None, sink=True, bias=True, gate=False),
    dict(H=2, G=2, dk=128, dv=64, page=16, chunk=64, window=None, softcap=15.0, sink=True, bias=True, gate=True),
    dict(H=4, G=4, dk=64, dv=128, page=16, chunk=None, window=33, softcap=None, sink=False, bias=False, gate=False),
    dict(H=4, G=2, dk=16, dv=16, page=4, chunk=7, window=5, softcap=3.0, sink=False, bias=True, gate=True),
    dict(H=16, G=1, dk=64, dv=64, page=16, chunk=90, window=None, softcap=None, sink=True, bias=True, gate=False),
    dict(H=2, G=1, dk=136, dv=136, page=16, chunk=100, window=None, softcap=30.0, sink=True, bias=True, gate=True),
]


def _shape_inputs(case, lengths, seed):
    """Projections per request with single keys made to stand out: for some queries the key at the start
    of their chunk or window (just inside) and the one before it (just outside) point along the query,
    scaled up; one request's keys all point away from its queries, so that the sink takes the weight."""
    g = torch.Generator().manual_seed(seed)
    H, G, dk, dv = case["H"], case["G"], case["dk"], case["dv"]
    reqs = []
    for n, L in enumerate(lengths):
        q = torch.randn(L, H, dk, generator=g, dtype=F64)
        k = torch.randn(L, G, dk, generator=g, dtype=F64)
        v = torch.randn(L, G, dv, generator=g, dtype=F64)
        gate = torch.randn(L, H * dv, generator=g, dtype=F64) * 2
        if n == 1:
            k = -q[:, ::H // G].clone() * 3                      # every score strongly negative
        else:
            for pos in range(L - 1, 0, -max(3, L // 9)):
                if case["chunk"]:
                    edge = (pos // case["chunk"]) * case["chunk"]
                    if case["window"]:
                        edge = max(edge, pos - case["window"] + 1)
                elif case["window"]:
                    edge = max(0, pos - case["window"] + 1)
                else:
                    edge = pos // 3                                # just a key far back
                head = pos % H
                for key, gainf in ((edge, 4.0), (edge - 1, 6.0)):
                    if 0 <= key < pos:
                        k[key, head // (H // G)] = q[pos, head] * gainf
        reqs.append((q, k, v, gate))
    return reqs


@pytest.mark.parametrize("case", ATTENTION_CASES, ids=lambda c: f"h{c['H']}g{c['G']}k{c['dk']}v{c['dv']}c{c['chunk']}w{c['window']}")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_kernels_over_scrambled_pages(case, dtype):
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.engine.batch import StepContext
    H, G, dk, dv, page = case["H"], case["G"], case["dk"], case["dv"], case["page"]
    eps, scale = 1e-5, 1.3 / math.sqrt(dk)
    lengths = (150, 75, 1, 260)
    reqs = _shape_inputs(case, lengths, seed=dk + dv)
    max_pages = -(-max(lengths) // page)
    n_pages = sum(-(-L // page) for L in lengths) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5)).tolist()
    table = torch.full((len(lengths), max_pages), -1, dtype=torch.int32)
    for slot, L in enumerate(lengths):
        for i in range(-(-L // page)):
            table[slot, i] = order.pop()
    flat = torch.zeros(n_pages, page * G * (dk + dv), dtype=dtype, device=DEV)
    k_plane = flat[:, :G * page * dk].unflatten(1, (G, page, dk))
    v_plane = flat[:, G * page * dk:].unflatten(1, (G, page, dv))
    slopes = torch.tensor(plain.slopes(H).tolist(), dtype=torch.float32, device=DEV) if case["bias"] else None
    table_d = table.to(DEV)

    # the rounded projections are what both sides start from
    rounded = []
    for q, k, v, gate in reqs:
        rounded.append(tuple(t.to(dtype).double() for t in (q, k, v, gate)))
    want = []
    for q, k, v, gate in rounded:
        qn, kn = plain.rms_norm(q, None, eps), plain.rms_norm(k, None, eps)
        if dtype == torch.bfloat16:                       # the cache and the queries are stored rounded
            qn, kn = qn.to(dtype).double(), kn.to(dtype).double()
        want.append(reference_attention(qn, kn, v, H, G, scale, case["softcap"], case["chunk"], case["window"],
                                        case["sink"], slopes, gate if case["gate"] else None))

    def run(rows, fast):
        """rows: list of (slot, first position, count); all of them one step."""
        proj, pos, slot_of = [], [], []
        for slot, p0, n in rows:
            q, k, v, gate = rounded[slot]
            proj.append(torch.cat([q[p0:p0 + n].reshape(n, -1), k[p0:p0 + n].reshape(n, -1),
                                   v[p0:p0 + n].reshape(n, -1), gate[p0:p0 + n]], 1))
            pos += list(range(p0, p0 + n))
            slot_of += [slot] * n
        proj = torch.cat(proj).to(dtype).to(DEV).contiguous()
        T = proj.shape[0]
        positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
        slots = torch.tensor(slot_of, dtype=torch.int32, device=DEV)
        q_out = torch.empty(T, H * dk, dtype=dtype, device=DEV)
        ops.qkv_unit_store(proj, q_out, positions, slots, table_d, k_plane, v_plane, page, H, G, dk, dv, eps)
        at = (H + G) * dk + G * dv
        gate = proj[:, at:] if case["gate"] else None
        out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
        ctx = None
        if fast:
            seg, tiles, dec, row = [], [], [], 0
            for s, (slot, p0, n) in enumerate(rows):
                seg.append([slot, row, n, p0])
                if n == 1:
                    dec.append(row)
                else:
                    tiles += [[s, off] for off in range(0, n, 64)]
                row += n
            ctx = StepContext(tokens=T, token_ids=None, positions=positions, token_slot=slots, want_rows=None,
                              segments=[], seg_info=torch.tensor(seg, dtype=torch.int32, device=DEV),
                              dec_rows=torch.tensor(dec, dtype=torch.int32, device=DEV) if dec else None,
                              n_dec=len(dec), pf_tiles=torch.tensor(tiles, dtype=torch.int32, device=DEV).view(-1, 2),
                              n_tiles=len(tiles))
        ops.attention_biased(q_out, k_plane, v_plane, positions, slots, table_d, page, H, G, dk, dv, scale, out,
                             softcap=case["softcap"] or 0.0, chunk=case["chunk"] or 0, window=case["window"] or 0,
                             sink=case["sink"], slopes=slopes, gate=gate, ctx=ctx)
        torch.cuda.synchronize()
        expect = torch.cat([want[slot][p0:p0 + n] for slot, p0, n in rows])
        return (out.double().cpu() - expect).abs().max().item()

    tol = 2e-5 if dtype == torch.float32 else 4e-2
    # whole prompts in one step
    whole = [(s, 0, L) for s, L in enumerate(lengths)]
    assert run(whole, fast=False) < tol
    if dtype == torch.bfloat16:
        before = ops.launches
        assert run(whole, fast=True) < tol
        fast_ok = bool(ops.lib().tllm_attention_biased_fast_ok(H, G, dk, dv))
        reach = min(v for v in (case["chunk"], case["window"], 1 << 30) if v)
        runs = ops.biased_decode_splits(1, G, reach)                  # the one-token request of the step
        # store + (one-token kernel, the sum of its runs of keys if it has several, prompt kernel | general)
        assert ops.launches - before == ((3 if runs == 1 else 4) if fast_ok else 2)
    # the cache is filled: portions that start anywhere, beside single rows at every kind of place
    edges = [p for p in (case["chunk"], case["window"], page) if p]
    singles = sorted({p for e in edges for p in (e - 1, e, e + 1, 2 * e - 1, 2 * e) if 0 < p < 150} | {149, 1})
    mixed = [(0, p, 1) for p in singles[:3]] + [(3, 100, 2), (3, 131, 129)] + [(1, 40, 35)]
    assert run(mixed, fast=False) < tol
    if dtype == torch.bfloat16:
        assert run(mixed, fast=True) < tol
    for p in singles:
        rows = [(0, p, 1), (3, 259, 1), (2, 0, 1), (1, 74, 1)]
        assert run(rows, fast=False) < tol, p
        if dtype == torch.bfloat16:
            assert run(rows, fast=True) < tol, p


# ----------------------------------------------------------------------------- feed-forwards
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 5, 40, 300])
def test_gated_unit_with_tanh_gelu(dtype, rows):
    from tiny_llm_infer_b200.parts.registry import lookup
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    torch.manual_seed(rows)
    hidden, inter = 136, 264
    part = lookup("feed_forward", "swiglu")(hidden_size=hidden, intermediate_size=inter, dtype=dtype, device=DEV,
                                            activation="gelu_tanh", names=("gate", "up", "down"))
    w = {n: (torch.randn(s, device=DEV) * 0.2).to(dtype) for n, s in
         (("gate", (inter, hidden)), ("up", (inter, hidden)), ("down", (hidden, inter)))}
    part.load(dict(w))
    x = (torch.randn(rows, hidden, device=DEV) * 1.5).to(dtype)
    got = part.forward(x, None).double().cpu()
    want = plain.gated_mlp(x.double().cpu(), {k: v.double().cpu() for k, v in w.items()}, "", plain.gelu_tanh)
    tol = (1e-5 if dtype == torch.float32 else 0.02) * want.abs().max().item()
    assert (got - want).abs().max() < tol


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("rows", [3, 512])
def test_products_with_the_activation_in_their_epilogue(act, rows):
    """The weight-streaming product (few rows) and the tcgen05 product (many) with act(gate) * up fused,
    against the float32 arithmetic of the same operands."""
    from tiny_llm_infer_b200 import ops
    torch.manual_seed(rows)
    k, inter = 256, 8192
    x = torch.randn(rows, k, device=DEV).to(torch.bfloat16)
    gate = (torch.randn(inter, k, device=DEV) * 0.1).to(torch.bfloat16)
    up = (torch.randn(inter, k, device=DEV) * 0.1).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate, up).contiguous()
    assert rows <= ops.SKINNY_MAX_ROWS or ops.tcgen05_pays(rows, inter, k, torch.bfloat16, col_tile=128)
    before = ops.launches
    got = ops.linear_swiglu(x, w, torch.bfloat16, interleaved=True, act=act)
    assert ops.launches - before == 1                      # one kernel: product and activation
    ops.check_error_word(x.device)
    f = plain.gelu_tanh if act == "gelu_tanh" else plain.silu
    want = f(x.double() @ gate.double().t()) * (x.double() @ up.double().t())
    assert (got.double() - want).abs().max() < 0.02 * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,shared,inter,hidden", [(16, 1, 112, 72, 176), (5, 3, None, 40, 88),
                                                             (8, 2, 96, 48, 128), (33, 4, 24, 72, 100),
                                                             (6, 2, 20, 36, 64)])
def test_mixture_of_experts_alone(dtype, experts, top, shared, inter, hidden):
    from tiny_llm_infer_b200.parts.registry import lookup
    from tiny_llm_infer_b200.parts.spec import PartSpec
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    g = torch.Generator().manual_seed(experts * 7 + top)
    names = ("gate", "up", "down")
    shared_spec = None if shared is None else PartSpec("swiglu", dict(hidden_size=hidden, intermediate_size=shared,
                                                                     names=names), "shared.")
    params = dict(hidden_size=hidden, experts=experts, top=top, expert_size=inter, shared=shared_spec, names=names)
    cls = lookup("feed_forward", "moe")
    part = cls(dtype=dtype, device=DEV, **params)
    w = {}
    for name, spec in cls.param_specs(**params).items():
        std = 0.15 if name == "router" else 0.25          # logits of a few units: no sigmoid at 1 to the last bit
        w[name] = (torch.randn(spec.shape, generator=g) * std).to(dtype).to(DEV)
    part.load(dict(w))
    w64 = {"m." + k: v.double().cpu() for k, v in w.items()}
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    from tiny_llm_infer_b200 import ops
    for rows in (1, 7, 150, 1100):                       # 1100: the grouped tcgen05 product where the sizes allow
        x = torch.randn(rows, hidden, generator=g).to(dtype).to(DEV)
        before = ops.tcgen05_calls
        got = part.forward(x, None).double().cpu()
        want = plain.moe(x.double().cpu(), w64, "m.", mlp)
        tol = (1e-5 if dtype == torch.float32 else 0.03) * want.abs().max().item()
        bad = (got - want).abs().amax(1) > tol
        # bfloat16: the weight times the row is rounded before the product; a row may differ by that much, none by an expert
        assert not bad.any(), (rows, (got - want).abs().max().item(), tol)
        on_tensor_memory = part.interleaved and ops.moe_tcgen05_pays(rows * top, experts, inter, hidden, dtype)
        assert (ops.tcgen05_calls - before >= 2) == on_tensor_memory
        ops.check_error_word(x.device)


def test_router_takes_the_largest_and_the_lowest_index_on_ties():
    from tiny_llm_infer_b200 import ops
    z = torch.tensor([[0.0, 2.0, 2.0, -1.0, 5.0], [1.0, 1.0, 1.0, 1.0, 1.0], [-9.0, -8.0, -7.0, -6.0, 30.0]],
                     device=DEV)
    ids, weights = ops.moe_route(z, 3)
    assert ids.tolist() == [[4, 1, 2], [0, 1, 2], [4, 3, 2]]
    want = torch.sigmoid(torch.gather(z, 1, ids.long()))
    assert torch.allclose(weights, want, atol=1e-6)
    wide = torch.randn(9, 700, device=DEV)
    ids, _ = ops.moe_route(wide, 6)
    assert torch.equal(ids.long(), torch.topk(wide, 6, dim=1).indices)


# ----------------------------------------------------------------------------- whole models, every way of cutting
BF16_RMS = {"P1": 0.08, "P2": 0.11, "P3": 0.06}        # three times what a B200 shows (0.027, 0.038, 0.019)        # a row's root-mean-square difference over the row's spread


@pytest.fixture(scope="module", params=sorted(PANOLORNS))
def case(request, tmp_path_factory):
    name = request.param
    tiny = PANOLORNS[name]
    folder = make_folder(tiny, tmp_path_factory.mktemp(name))
    cfg, w = plain.read_model(folder)
    # prompts on which no router meets a near-tie: bfloat16 would let it fall either way
    reqs = {rid: plain.decisive_tokens(cfg, w, toks, seed=int(rid)) for rid, toks in requests_for(tiny).items()}
    want = {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    tb = replay.TraceBuilder()
    replay.whole(tb, reqs)
    replay.tail_one_by_one(tb, reqs)
    replay.portions(tb, reqs)
    replay.mixed(tb, reqs, seed=7)
    return name, tiny, folder, cfg, want, tb, reqs


def run_tool(folder, dtype, out, tb, page_size):
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(tb.max_tokens), "--page-size", str(page_size), "--max-requests", "4"]
    res = subprocess.run(cmd, input=tb.text(), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    done = [l for l in res.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(tb.steps))]


def relative_rows(out, tb, want, vocab):
    """Per way of cutting, every row's root-mean-square difference from the plain implementation (the
    mean taken off) over the row's own spread; and the same between each way and the whole-request run."""
    errors, base, spread = {}, {}, {}
    rows_of = {}
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
        if name[0] != "w":
            ref = base[(name[1:], pos)]
            spread.setdefault(name[0], []).append(float(np.sqrt(np.mean((row - ref) ** 2)) / ref.std()))
    return {k: np.array(v) for k, v in errors.items()}, {k: np.array(v) for k, v in spread.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_ways_of_cutting(case, dtype, tmp_path):
    name, tiny, folder, cfg, want, tb, reqs = case
    out = tmp_path / "out"
    run_tool(folder, dtype, out, tb, tiny["page_size"])
    errors, spread = relative_rows(out, tb, want, cfg["vocab"])
    assert set(errors) == {"w", "t", "p", "m"}
    summary = {k: (round(float(np.percentile(v, 50)), 5), round(float(v.max()), 5)) for k, v in errors.items()}
    between = {k: (round(float(np.percentile(v, 50)), 5), round(float(v.max()), 5)) for k, v in spread.items()}
    print(f"\n[{name} {dtype}] against plain (median, max) {summary}; between the ways (median, max) {between}")
    limit = 1e-4 if dtype == "float32" else BF16_RMS[name]
    assert max(v.max() for v in errors.values()) < limit, summary
    assert max(v.max() for v in spread.values()) < (limit if dtype == "float32" else limit / 2), between


def test_first_tokens_and_decoding_across_chunk_edges(case, tmp_path):
    """One token at a time from an empty cache, across page and chunk edges, beside a second request that
    decodes from the middle of a chunk; then the last 90 tokens of a long request one by one."""
    name, tiny, folder, cfg, want, _, reqs = case
    a, b = reqs["0"], reqs["1"]
    tb = replay.TraceBuilder()
    tb.step([("f1", b[:29])])
    for i in range(len(a)):
        extra = [("f1", b[29 + i:30 + i])] if 29 + i < len(b) else []
        tb.step([("f0", a[i:i + 1])] + extra)
    tb.step([], end=["f0", "f1"])
    replay.tail_one_by_one(tb, {"2": reqs["2"]}, tail=90, tag="f")
    out = tmp_path / "out"
    run_tool(folder, "float32", out, tb, tiny["page_size"])
    worst, _ = relative_rows_no_base(out, tb, want, cfg["vocab"])
    assert worst < 1e-4, worst


def relative_rows_no_base(out, tb, want, vocab):
    worst, where = 0.0, None
    for step, rows in tb.expect.items():
        got = replay.read_logits(out, step, vocab).astype(np.float64)
        for r, (name, pos) in enumerate(rows):
            ref = want[name[1:]][pos]
            d = got[r] - ref
            e = float(np.sqrt(np.mean((d - d.mean()) ** 2)) / ref.std())
            if e > worst:
                worst, where = e, (step, name, pos)
    return worst, where


def test_experts_on_tcgen05_agree_with_the_mma_tiles_inside_a_model(tmp_path, monkeypatch):
    """The same prompts through the model with the experts' products on the grouped tcgen05 kernel (its
    threshold lowered for this) and on the mma.sync tiles: the logits agree as two bfloat16 paths do."""
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.engine import ModelRunner, StepEntry, load_model
    tiny = PANOLORNS["P1"]
    folder = make_folder(tiny, tmp_path)
    cfg, w = plain.read_model(folder)
    model, _ = load_model(folder, torch.bfloat16, DEV)
    toks = plain.decisive_tokens(cfg, w, prompt(3, 200, cfg["vocab"]), seed=3)
    want = plain.forward(cfg, w, toks).numpy()
    got = {}
    for rows in (64, 1 << 30):
        monkeypatch.setattr(ops, "MOE_TCGEN05_ROWS", rows)
        cache = CacheManager(model.cache_needs(), 16, 32, max_slots=2, max_seq_len=512, dtype=torch.bfloat16, device=DEV)
        runner = ModelRunner(model, cache, max_batch_tokens=512)
        before = ops.tcgen05_calls
        got[rows] = runner.step([StepEntry("a", toks, list(range(len(toks))))]).double().cpu().numpy()
        assert (ops.tcgen05_calls > before) == (rows == 64)
        runner.check_kernels()
    for a in got.values():
        d = a - want
        err = np.sqrt(((d - d.mean(1, keepdims=True)) ** 2).mean(1)) / want.std(1)
        assert err.max() < BF16_RMS["P1"], err.max()
    d = got[64] - got[1 << 30]
    assert (np.sqrt((d ** 2).mean(1)) / want.std(1)).max() < BF16_RMS["P1"] / 2


# ----------------------------------------------------------------------------- generation through the entry point
def plain_greedy(cfg, w, prompt_ids, n):
    ids = list(prompt_ids)
    for _ in range(n):
        ids.append(int(plain.forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt_ids):]


@pytest.mark.parametrize("name", ["P1", "P2"])
@pytest.mark.parametrize("budget,blocks", [(256, 64), (8, 64), (7, 14)])
def test_greedy_generation_equals_plain(name, budget, blocks, tmp_path):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = PANOLORNS[name]
    folder = make_folder(tiny, tmp_path)
    cfg, w = plain.read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((5, 27, 53, 1))]
    want = [plain_greedy(cfg, w, p, 12) for p in prompts]
    llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=blocks, block_size=tiny["page_size"],
              max_num_batched_tokens=budget, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.cache.audit()
    assert all(v == blocks for v in llm.cache.free_pages().values())


def test_long_decoding_in_bfloat16_through_graphs(tmp_path):
    """Forty tokens each for three requests, decode steps replayed as CUDA graphs, bfloat16 kernels: every
    token is the plain implementation's choice given the same beginning, or within a near-tie of it."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = PANOLORNS["P3"]
    folder = make_folder(tiny, tmp_path)
    cfg, w = plain.read_model(folder)
    prompts = [prompt(i, n, cfg["vocab"]) for i, n in enumerate((60, 9, 190))]
    llm = LLM(str(folder), dtype="bfloat16", max_model_len=256, num_kv_blocks=24, block_size=32,
              max_num_batched_tokens=64, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p) + list(o.token_ids)
        logits = plain.forward(cfg, w, ids[:-1]).numpy()
        near = [logits[len(p) - 1 + i][tok] >= logits[len(p) - 1 + i].max() - 0.15 * logits[len(p) - 1 + i].std()
                for i, tok in enumerate(o.token_ids)]
        # a router's near-tie may fall the other way in bfloat16 and move a row by an expert's output
        assert sum(near) >= 0.9 * len(near), near


def test_command_line_writes_and_runs_a_model(tmp_path):
    """``bin/model_main``: a random Panolorn model from its config.json, greedy tokens equal to the plain
    implementation's in float32, and seeded temperature / top-p sampling that repeats itself."""
    import json
    tiny = PANOLORNS["P2"]
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny["cfg"].to_dict()))
    folder = tmp_path / "model"
    tool = [sys.executable, str(ROOT / "bin" / "model_main")]
    res = subprocess.run(tool + ["--write-random-model", str(folder), "--config", str(cfg_path), "--random-weights", "21",
                                 "--weight-std", "0.07"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    cfg, w = plain.read_model(folder)
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
    assert all(len(line.split(",")) == 7 and all(0 <= int(x) < cfg["vocab"] for x in line.split(",")) for line in draws[0])
