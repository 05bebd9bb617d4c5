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


@register("feed_forward", "mlp")
class PlainFeedForward:
    """d = act(x Wu^T) Wd^T, no gate and no biases; ``activation`` is ``gelu_erf`` (the exact GELU,
    0.5 z (1 + erf(z / sqrt 2))), ``gelu_tanh`` or ``silu``, computed in float32."""
    NAMES = ("up", "down")

    def __init__(self, hidden_size: int, intermediate_size: int, dtype: torch.dtype, device,
                 activation: str = "gelu_erf", names=NAMES):
        if activation not in ops.ELEMENTWISE_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ELEMENTWISE_ACTIVATIONS)}")
        self.hidden, self.inter, self.dtype, self.device = hidden_size, intermediate_size, dtype, device
        self.activation, self.names = activation, tuple(names)
        self.w_up = self.w_down = None

    @classmethod
    def param_specs(cls, hidden_size, intermediate_size, activation: str = "gelu_erf", names=NAMES) -> Dict[str, ParamSpec]:
        up, down = names
        return {up: ParamSpec((intermediate_size, hidden_size)), down: ParamSpec((hidden_size, intermediate_size))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = t[self.names[0]].contiguous(), t[self.names[1]].contiguous()

    def workspace_floats(self, tokens: int) -> int:
        return 2 * tokens * self.inter

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return ops.linear(ops.linear_act(x, self.w_up, self.activation, self.dtype), self.w_down, out_dtype=self.dtype)


@register("feed_forward", "token_side")
class TokenSideInput:
    """A small input per layer that depends on the row's token: e = table[token, first_column : first_column +
    side_dim]; d = (act(x Wg^T) * e) Wp^T.  The table belongs to the embedding, which publishes it in the
    step's memo under ``memo_key`` (all layers share it and read their own columns); the look-up, the
    activation and the product with e are one kernel."""
    NAMES = ("gate", "proj")

    def __init__(self, hidden_size: int, side_dim: int, first_column: int, dtype: torch.dtype, device,
                 activation: str = "gelu_tanh", memo_key: str = "token_side_table", names=NAMES):
        if activation not in ops.ELEMENTWISE_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ELEMENTWISE_ACTIVATIONS)}")
        self.hidden, self.side_dim, self.first_column = hidden_size, int(side_dim), int(first_column)
        self.dtype, self.device, self.activation, self.memo_key, self.names = dtype, device, activation, memo_key, tuple(names)
        self.w_gate = self.w_proj = None

    @classmethod
    def param_specs(cls, hidden_size, side_dim, first_column=0, activation: str = "gelu_tanh",
                    memo_key: str = "token_side_table", names=NAMES) -> Dict[str, ParamSpec]:
        gate, proj = names
        return {gate: ParamSpec((side_dim, hidden_size)), proj: ParamSpec((hidden_size, side_dim))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_gate, self.w_proj = t[self.names[0]].contiguous(), t[self.names[1]].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        table = ctx.memo.get(self.memo_key)
        if table is None:
            raise ValueError(f"no table under {self.memo_key!r} in the step's memo: the embedding has to publish it")
        z = ops.linear(x, self.w_gate, out_dtype=self.dtype)
        g = ops.activation(z, self.activation, ids=ctx.token_ids, table=table, col0=self.first_column)
        return ops.linear(g, self.w_proj, out_dtype=self.dtype)
