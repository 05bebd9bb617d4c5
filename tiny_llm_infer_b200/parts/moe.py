"""Mixture of experts as a feed-forward part: a router chooses ``top`` of ``experts`` small gated
feed-forward units per token, an optional shared unit runs for every token, and the results are summed.

  z = Wr x in float32; score s = sigmoid(z) (``router_scores='sigmoid'``) or the softmax of the chosen
  experts' logits (``'softmax'``); the experts with the largest z are chosen, lowest index on ties
  expert e: Wd_e (act(Wg_e u) * (Wu_e u)); with ``weight_on='input'`` u = s_e x and the outputs are
  summed as they are, with ``'output'`` u = x and the outputs are weighted by s_e
  out = sum over the chosen experts + shared(x)

The step's rows are sorted by expert on the device (``ops.MoePlan``); the experts' gate|up product
gathers its rows from the tokens and applies the activation in its epilogue, the down product leaves
rows that one kernel sums per token, in float32, with the shared unit's output.  Steps with many rows run
both products on the grouped tcgen05 kernel (row tiles of 128 per expert), steps with few on mma.sync
tiles of 64 rows that read the chosen experts' weights once.  Nothing is read by the host,
so steps with this part are captured as CUDA graphs like the others.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .registry import lookup, register
from .spec import ParamSpec, PartSpec


@register("feed_forward", "moe")
class MixtureOfExperts:
    graph_safe = True

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, dtype: torch.dtype, device,
                 activation: str = "silu", router_scores: str = "sigmoid", weight_on: str = "input",
                 shared: Optional[PartSpec] = None, router_name: str = "router", expert_prefix: str = "e",
                 names=("gate", "up", "down")):
        if not 0 < top <= experts:
            raise ValueError(f"top {top} of {experts} experts")
        if router_scores not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError(f"router_scores {router_scores!r} / weight_on {weight_on!r}")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ACTIVATIONS)}")
        self.hidden, self.experts, self.top, self.inter = hidden_size, experts, top, expert_size
        self.dtype, self.device, self.activation = dtype, device, activation
        self.router_scores, self.weight_on = router_scores, weight_on
        self.router_name, self.expert_prefix, self.names = router_name, expert_prefix, tuple(names)
        self.shared_spec = shared
        self.shared = None
        if shared is not None:
            self.shared = lookup("feed_forward", shared.kind)(dtype=dtype, device=device, **shared.params)
        self.w_router = self.w_gate_up = self.w_down = None

    @classmethod
    def param_specs(cls, hidden_size, experts, top, expert_size, shared: Optional[PartSpec] = None,
                    router_name: str = "router", expert_prefix: str = "e", names=("gate", "up", "down"),
                    **_) -> Dict[str, ParamSpec]:
        gate, up, down = names
        specs = {router_name: ParamSpec((experts, hidden_size))}
        for e in range(experts):
            p = f"{expert_prefix}{e}."
            specs[p + gate] = ParamSpec((expert_size, hidden_size))
            specs[p + up] = ParamSpec((expert_size, hidden_size))
            specs[p + down] = ParamSpec((hidden_size, expert_size))
        if shared is not None:
            for k, v in lookup("feed_forward", shared.kind).param_specs(**shared.params).items():
                specs[shared.prefix + k] = v
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        gate, up, down = self.names
        self.w_router = t[self.router_name].contiguous()
        # gate and up of an expert as one matrix, their rows interleaved by eight where the width allows
        # (the layout whose products apply the activation in their epilogue), else stacked
        self.interleaved = self.inter % 8 == 0
        stacks = []
        for e in range(self.experts):
            p = f"{self.expert_prefix}{e}."
            if self.interleaved:
                stacks.append(ops.interleave_gate_up(t[p + gate], t[p + up]))
            else:
                stacks.append(torch.cat([t[p + gate], t[p + up]], dim=0))
        self.w_gate_up = torch.stack(stacks).contiguous()                       # [E, 2 I, H]
        self.w_down = torch.stack([t[f"{self.expert_prefix}{e}.{down}"] for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            n = len(self.shared_spec.prefix)
            self.shared.load({k[n:]: v for k, v in t.items() if k.startswith(self.shared_spec.prefix)})

    def workspace_floats(self, tokens: int) -> int:
        own = tokens * self.top * (self.inter + self.hidden) + tokens * self.experts
        shared = int(self.shared.workspace_floats(tokens)) if hasattr(self.shared, "workspace_floats") else 0
        return own + shared

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        z = ops.linear(x, self.w_router, out_dtype=torch.float32)
        ids, weights = ops.moe_route(z, self.top, softmax_weights=self.router_scores == "softmax")
        rows = ids.numel()
        tensor_cores = self.interleaved and x.dtype == self.w_gate_up.dtype \
            and ops.moe_tcgen05_pays(rows, self.experts, self.inter, self.hidden, x.dtype)
        plan = ops.MoePlan(ids, self.experts, ops.MOE_TCGEN05_TILE if tensor_cores else None)
        on_input = self.weight_on == "input"
        act = ops.moe_grouped(x, self.w_gate_up, plan, self.top, gated=True, gather=True,
                              weights=weights if on_input else None, act=self.activation,
                              interleaved=self.interleaved)
        y = ops.moe_grouped(act, self.w_down, plan, self.top, gated=False, gather=False)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        return ops.moe_combine(y, plan, self.top, shared, self.dtype, weights=None if on_input else weights)
