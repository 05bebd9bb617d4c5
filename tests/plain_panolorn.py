"""Plain, slow implementation of the Panolorn design: whole sequences, no cache, no batching,
one function per mechanism, float64 arithmetic on the CPU.  It shares no code with the
package: config.json is read as a dict, the weights through the ``safetensors`` library.

The design, in this file's notation (T tokens, width D, positions p = 0 .. T-1):

  x0 = E[token] * c_emb
  per layer:  x <- x + N_1b(mixer(N_1(x)));  if the layer has a feed-forward:  x <- x + N_2b(ff(N_2(x)))
  N(v) = v / sqrt(mean(v^2) + eps) * gain
  logits = E . N_final(x)          (the table itself, without c_emb)

Mixer: grouped-query attention without rotation.  Per head q and k are divided by their own
root mean square (no gain).  s_ij = (q_i . k_j) * c_scale, then s <- cap * tanh(s / cap), then
s <- s - m_h * (i - j) with m_h = 2^(-8 (h + 1) / H).  Key j is visible to query i when j <= i and
both lie in the same chunk of ``mask.size`` positions counted from 0.  The weights are
exp(s_ij) / (1 + sum_j exp(s_ij)): a sink of score 0 that carries no value.  The concatenated
heads are multiplied by sigmoid(W_g u), u the mixer's input, and projected by W_o.

Feed-forward, dense: W_down (gelu_tanh(W_gate u) * (W_up u)).  Mixture of experts: z = W_r u,
s = sigmoid(z), the ``top`` largest s choose the experts, each expert (silu-gated, same form) is
applied to s_e * u (the weight scales the input, not the output; no renormalisation), their
outputs are summed and a shared expert applied to u itself is added.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors import safe_open

F = torch.float64


def read_model(folder):
    """(config dict, {name: float64 tensor}) of a model folder."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = {}
    for f in sorted(folder.glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as fh:
            for name in fh.keys():
                weights[name] = fh.get_tensor(name).to(F)
    return cfg, weights


def rms_norm(x, gain, eps):
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def slopes(heads):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F)


def visible(T, chunk):
    """[T, T] bool: key j visible to query i."""
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    ok = j <= i
    if chunk:
        ok = ok & ((i // chunk) == (j // chunk))
    return ok


def attention_scores(q, k, head, heads, scale, softcap, chunk):
    """[T, T] scores of one head after cap and distance bias; hidden keys are -inf."""
    T = q.shape[0]
    s = (q @ k.t()) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    i = torch.arange(T, dtype=F).view(T, 1)
    j = torch.arange(T, dtype=F).view(1, T)
    s = s - slopes(heads)[head] * (i - j)
    return s.masked_fill(~visible(T, chunk), float("-inf"))


def sink_softmax(s):
    """exp(s) / (1 + sum exp(s)) along the last axis, computed with the maximum (or 0) taken off."""
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def attention_mixer(u, w, prefix, mix, eps):
    """u [T, D] -> [T, D].  ``mix`` is the layer's 'mixer' dict."""
    T = u.shape[0]
    H, G, dk, dv = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    chunk = (mix.get("mask") or {}).get("size")
    q = (u @ w[prefix + "q"].t()).view(T, H, dk)
    k = (u @ w[prefix + "k"].t()).view(T, G, dk)
    v = (u @ w[prefix + "v"].t()).view(T, G, dv)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    outs = []
    for h in range(H):
        g = h // (H // G)
        s = attention_scores(q[:, h], k[:, g], h, H, mix["scale"], mix.get("softcap"), chunk)
        outs.append(sink_softmax(s) @ v[:, g])
    o = torch.cat(outs, dim=-1)
    o = o * torch.sigmoid(u @ w[prefix + "g"].t())
    return o @ w[prefix + "o"].t()


def gated_mlp(u, w, prefix, act):
    return (act(u @ w[prefix + "gate"].t()) * (u @ w[prefix + "up"].t())) @ w[prefix + "down"].t()


def router(u, w_router, top):
    """(indices [T, top], weights [T, top]): the experts with the largest sigmoid scores."""
    s = torch.sigmoid(u @ w_router.t())
    weights, idx = torch.topk(s, top, dim=-1)
    return idx, weights


def router_gaps(u, w_router, top):
    """Per token, how far the last chosen expert's logit lies above the best one left out, in units of
    the logits' spread (infinite when every expert is chosen)."""
    z = u @ w_router.t()
    if top >= z.shape[-1]:
        return torch.full((u.shape[0],), float("inf"), dtype=F)
    ordered = torch.sort(z, dim=-1, descending=True).values
    return (ordered[:, top - 1] - ordered[:, top]) / z.std()


def moe(u, w, prefix, mlp, gaps_out=None):
    idx, weights = router(u, w[prefix + "router"], mlp["router"]["top"])
    if gaps_out is not None:
        gaps_out.append(router_gaps(u, w[prefix + "router"], mlp["router"]["top"]))
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for e, s in zip(idx[t].tolist(), weights[t]):
            out[t] += gated_mlp((s * u[t]).unsqueeze(0), w, f"{prefix}e{e}.", silu)[0]
    if mlp.get("shared"):
        out = out + gated_mlp(u, w, prefix + "shared.", silu)
    return out


def feed_forward(u, w, prefix, mlp, gaps_out=None):
    if mlp["kind"] == "dense":
        return gated_mlp(u, w, prefix, gelu_tanh)
    if mlp["kind"] == "moe":
        return moe(u, w, prefix, mlp, gaps_out)
    raise ValueError(mlp["kind"])


def forward(cfg, w, tokens, layers_out=None, gaps_out=None):
    """Logits [T, vocab] float64 of one whole sequence; ``layers_out`` (a list) receives the
    residual stream after every layer, ``gaps_out`` (a list) every router's ``router_gaps``."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens))] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        a = attention_mixer(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + rms_norm(a, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            m = feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"], gaps_out)
            x = x + rms_norm(m, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].t()


def decisive_tokens(cfg, w, tokens, seed, threshold=0.08, tries=400):
    """``tokens`` with some of them drawn again until no router of the model meets a near-tie anywhere
    in the sequence (every gap of ``router_gaps`` above ``threshold``).  In 16-bit arithmetic a near-tie
    falls either way, and the row then differs by a whole expert; a comparison of logits wants prompts
    on which the design's answer does not hang on the last bit.  Tokens before the first near-tie stay
    as they are (the model is causal), so the search moves from left to right."""
    g = torch.Generator().manual_seed(seed)
    tokens = list(tokens)
    for _ in range(tries):
        gaps = []
        forward(cfg, w, tokens, gaps_out=gaps)
        if not gaps:
            return tokens
        close = (torch.stack(gaps).min(0).values < threshold).nonzero().flatten()
        if close.numel() == 0:
            return tokens
        tokens[int(close[0])] = int(torch.randint(0, cfg["vocab"], (1,), generator=g))
    raise RuntimeError("no sequence without near-ties found")
