"""Dense gated feed-forward: d = (act(x Wg^T) * (x Wu^T)) Wd^T, no biases, act in float32:
silu(g) = g / (1 + exp(-g)) (SwiGLU; reference: model/src/qwen3_paged_batch.cpp:281-295,
kernels/src/swiglu_kernel_cpu.cpp:20-24) or, by the ``activation`` parameter, the tanh form of GELU.
``names`` are the checkpoint's names of the gate, up and down matrices behind the part's prefix.  Gate and up projections are one product with
one weight of 2 I rows, fused at load time: eight rows of Wg, the eight rows of Wu that belong
to them, and so on (``ops.interleave_gate_up``), so that a gate and its up meet in one
accumulator of the products' kernels; [Wg; Wu] if I is no multiple of eight.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .registry import register
from .spec import ParamSpec


@register("feed_forward", "swiglu")
class SwiGLUFeedForward:
    NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    def __init__(self, hidden_size: int, intermediate_size: int, dtype: torch.dtype, device,
                 activation: str = "silu", names=NAMES):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ACTIVATIONS)}")
        self.hidden, self.inter, self.dtype, self.device = hidden_size, intermediate_size, dtype, device
        self.activation, self.names = activation, tuple(names)
        self.w_gate_up = self.w_down = None

    @classmethod
    def param_specs(cls, hidden_size, intermediate_size, activation: str = "silu", names=NAMES) -> Dict[str, ParamSpec]:
        gate, up, down = names
        return {
            gate: ParamSpec((intermediate_size, hidden_size)),
            up: ParamSpec((intermediate_size, hidden_size)),
            down: ParamSpec((hidden_size, intermediate_size)),
        }

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        parts = [t[self.names[0]], t[self.names[1]]]
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.interleaved = self.inter % 8 == 0
        if self.interleaved:
            self.w_gate_up = ops.interleave_gate_up(*[p.to(common) for p in parts]).contiguous()
        else:
            self.w_gate_up = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_down = t[self.names[2]].contiguous()

    def workspace_floats(self, tokens: int) -> int:
        return 3 * tokens * self.inter          # the product of gate and up, and the activation

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        act = ops.linear_swiglu(x, self.w_gate_up, out_dtype=self.dtype, interleaved=self.interleaved,
                                act=self.activation)
        return ops.linear(act, self.w_down, out_dtype=self.dtype)
