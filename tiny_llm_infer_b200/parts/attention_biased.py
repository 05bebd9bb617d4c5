"""Grouped-query attention without rotation, whose score is changed between the dot product and the
softmax, with an output gate.  Every step is a parameter, so other designs can pick their own mix:

  q, k        per head divided by their root mean square over the head (``unit_norm_eps``; None: not)
  score       s = (q . k) * scale;  ``softcap`` c: s <- c tanh(s / c);  ``bias_slopes`` m_h: s <- s - m_h (i - j)
              (``slope_exponent`` e instead of explicit slopes: m_h = 2^(-e (h + 1) / heads))
  visible     j <= i, within the query's own chunk of ``chunk`` positions counted from 0 (None: no
              chunks), and within ``window`` keys back (None: no window)
  softmax     ``sink``: one is added to the denominator (a key of score 0 that carries no value)
  gate        ``output_gate``: the concatenated heads are multiplied by sigmoid(Wg x), x the mixer's input

Keys have width ``key_dim`` and values ``value_dim``; they are two planes of the paged cache.  With a
chunk or a window the cache keeps only the keys a later query can still see (a chunk never reaches
further back than a window of the same size).  The projections q | k | v | gate are one product with
the row-wise concatenation of their weights; the norm of q and k and the write of k and v are one
kernel; the gate is applied where the attention kernel writes its result.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import ops
from .registry import register
from .spec import CacheSpec, ParamSpec, StateSpec


def slopes_from_exponent(heads: int, exponent: float):
    return [2.0 ** (-exponent * (h + 1) / heads) for h in range(heads)]


@register("mixer", "biased_attention")
class BiasedAttention:
    graph_safe = True
    NAMES = ("q", "k", "v", "o", "g")

    def __init__(self, hidden_size: int, q_heads: int, kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, dtype: torch.dtype, device, unit_norm_eps: Optional[float] = None,
                 softcap: Optional[float] = None, slope_exponent: Optional[float] = None,
                 bias_slopes: Optional[Sequence[float]] = None, chunk: Optional[int] = None,
                 window: Optional[int] = None, sink: bool = False, output_gate: bool = False,
                 names: Sequence[str] = NAMES):
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads cannot share {kv_heads} key/value heads")
        if unit_norm_eps is not None and not unit_norm_eps > 0.0:
            raise ValueError(f"unit_norm_eps must be positive (or None for no head norm), got {unit_norm_eps}")
        for what, v in (("chunk", chunk), ("window", window)):
            if v is not None and v <= 0:
                raise ValueError(f"{what} must be positive (or None), got {v}")
        if softcap is not None and not softcap > 0.0:
            raise ValueError(f"softcap must be positive (or None), got {softcap}")
        self.hidden, self.q_heads, self.kv_heads = hidden_size, q_heads, kv_heads
        self.dk, self.dv = key_dim, value_dim
        self.scale, self.softcap = float(scale), softcap
        self.unit_norm_eps, self.chunk, self.window = unit_norm_eps, chunk, window
        self.sink, self.output_gate = bool(sink), bool(output_gate)
        self.dtype, self.device, self.names = dtype, device, tuple(names)
        if bias_slopes is None and slope_exponent is not None:
            bias_slopes = slopes_from_exponent(q_heads, slope_exponent)
        self.slopes = None
        if bias_slopes is not None:
            if len(bias_slopes) != q_heads:
                raise ValueError(f"{len(bias_slopes)} slopes for {q_heads} heads")
            self.slopes = torch.tensor(list(bias_slopes), dtype=torch.float64).to(torch.float32).to(device)
        self.w_in = self.w_o = None

    # ---- weights
    @classmethod
    def param_specs(cls, hidden_size, q_heads, kv_heads, key_dim, value_dim, output_gate=False,
                    names=NAMES, **_) -> Dict[str, ParamSpec]:
        q, k, v, o, g = names
        specs = {
            q: ParamSpec((q_heads * key_dim, hidden_size)),
            k: ParamSpec((kv_heads * key_dim, hidden_size)),
            v: ParamSpec((kv_heads * value_dim, hidden_size)),
            o: ParamSpec((hidden_size, q_heads * value_dim)),
        }
        if output_gate:
            specs[g] = ParamSpec((q_heads * value_dim, hidden_size))
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        q, k, v, o, g = self.names
        parts = [t[q], t[k], t[v]] + ([t[g]] if self.output_gate else [])
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_in = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_o = t[o].contiguous()

    # ---- what the cache manager has to provide
    def reach(self) -> Optional[int]:
        """Keys back from a query (itself included) that the mask can let through, None for all."""
        limits = [v for v in (self.chunk, self.window) if v is not None]
        return min(limits) if limits else None

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(((self.kv_heads, self.dk), (self.kv_heads, self.dv)), self.reach())

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def workspace_floats(self, tokens: int) -> int:
        width_in = (self.q_heads + self.kv_heads) * self.dk + (self.kv_heads + 2 * self.q_heads) * self.dv
        return tokens * (width_in + self.q_heads * self.dk)

    # ---- one step
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        tokens = x.shape[0]
        proj = ops.linear(x, self.w_in, out_dtype=self.dtype)
        q = torch.empty((tokens, self.q_heads * self.dk), dtype=self.dtype, device=x.device)
        k_plane, v_plane = cache.planes
        ops.qkv_unit_store(proj, q, ctx.positions, ctx.token_slot, cache.block_table, k_plane, v_plane,
                           cache.page_size, self.q_heads, self.kv_heads, self.dk, self.dv,
                           self.unit_norm_eps, store=cache.writes)
        gate = None
        if self.output_gate:
            at = (self.q_heads + self.kv_heads) * self.dk + self.kv_heads * self.dv
            gate = proj[:, at:at + self.q_heads * self.dv]
        out = torch.empty((tokens, self.q_heads * self.dv), dtype=self.dtype, device=x.device)
        ops.attention_biased(q, k_plane, v_plane, ctx.positions, ctx.token_slot, cache.block_table,
                             cache.page_size, self.q_heads, self.kv_heads, self.dk, self.dv, self.scale, out,
                             softcap=self.softcap or 0.0, chunk=self.chunk or 0, window=self.window or 0,
                             sink=self.sink, slopes=self.slopes, gate=gate, ctx=ctx)
        return ops.linear(out, self.w_o, out_dtype=self.dtype)
