"""Kaketar, plainly: whole sequences, no cache, no batching, float64 unless told otherwise; one
function per mechanism.  It shares no code with the engine and is what the engine is compared with.

``weights`` maps tensor names to torch tensors (any float type), ``cfg`` is the dictionary of
config.json.  Notation: T tokens, D the model width, rows are tokens.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_one(x, w, eps):
    """The model's norm: the stored weight is the gain minus one."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]; y[t, c] = sum_j taps[c, K-1-j] x[t-j, c], zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        if j < T:
            y[j:] += x[:T - j] * taps[:, K - 1 - j]
    return y


def channel_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                  trace: Optional[dict] = None) -> torch.Tensor:
    """Delta rule with one decay per head and key channel.  h [T, D]."""
    heads, kv_heads, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, kv_heads, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, kv_heads, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, heads, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                        # [T, heads]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    decay = torch.exp(-torch.exp(w[p + "A_log"]).view(1, heads, 1)
                      * torch.nn.functional.softplus(a.view(T, heads, dk)))       # [T, heads, dk]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, heads, dv)
    rep = heads // kv_heads
    out = torch.zeros(T, heads, dv, dtype=h.dtype)
    for hd in range(heads):
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            kt, qt = k[t, hd // rep], q[t, hd // rep]
            S = decay[t, hd].unsqueeze(1) * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kt)
            S = S + torch.outer(kt, u)
            out[t, hd] = S.T @ qt
        if trace is not None:
            trace.setdefault("state", []).append(S)
    out = rms_unit(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, heads * dv) @ w[p + "o"].T


def yarn_frequencies(rot: dict) -> (torch.Tensor, float):
    """Angular frequency of every pair of the rotated part, and the factor on cos and sin."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, ..., R]: the first rot['dims'] elements rotate, neighbours (2i, 2i+1) forming a pair."""
    dims = rot["dims"]
    f, mag = yarn_frequencies(rot)
    ang = positions.to(torch.float64).unsqueeze(-1) * f                             # [T, dims/2]
    cos, sin = (torch.cos(ang) * mag).to(x.dtype), (torch.sin(ang) * mag).to(x.dtype)
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    y = x.clone()
    y[..., 0:dims:2] = a * cos - b * sin
    y[..., 1:dims:2] = b * cos + a * sin
    return y


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are made from one small vector per token.  h [T, D]."""
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    cq = norm_plain(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, dn + dr)
    q_n, q_r = q[..., :dn], rotate_pairs(q[..., dn:], pos, m["rot"])
    kv = h @ w[p + "dkv"].T
    c = norm_plain(kv[:, :rank], w[p + "dkv.norm"], eps)
    k_r = rotate_pairs(kv[:, rank:], pos, m["rot"])                                  # [T, dr], one for all heads
    k_n = (c @ w[p + "uk"].T).view(T, H, dn)
    val = (c @ w[p + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_n, k_n) + torch.einsum("ihd,jd->hij", q_r, k_r)) * m["scale"]
    i, j = pos.view(-1, 1), pos.view(1, -1)
    seen = (j <= i)
    if m.get("mask"):
        seen = seen & (i - j < m["mask"]["size"])
    s = s.masked_fill(~seen, -math.inf)
    sink = w[p + "sink"].to(h.dtype).view(H, 1, 1).expand(H, T, 1)
    both = torch.cat([s, sink], dim=-1)
    weights = torch.softmax(both, dim=-1)[..., :T]                                   # the sink takes its share and gives nothing
    o = torch.einsum("hij,jhd->ihd", weights, val).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def dense_ff(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def token_side(x, tokens, w, cfg, layer: int):
    dim, eps = cfg["token_side"]["dim"], cfg["norm"]["eps"]
    p = f"l{layer}.side."
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return norm_plain(y, w[p + "norm"], eps)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its start."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.tensor(tokens, dtype=torch.long)
    T = len(tokens)
    x = w["embed"][tok] * cfg.get("embedding", {}).get("scale", 1.0) + w["pos"][:T]
    x = norm_around_one(x, w["embed.norm"], eps)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "channel_delta":
            a = channel_delta(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            a = latent_attention(x, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm_around_one(a, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + norm_around_one(dense_ff(x, w, p + "mlp."), w[p + "norm2"], eps)
        if cfg.get("token_side"):
            x = x + token_side(x, tok, w, cfg, i)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = norm_around_one(x, w["final.norm"], eps)
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
