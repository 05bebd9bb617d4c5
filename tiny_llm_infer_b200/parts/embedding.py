"""Token embedding and the output head.

h0[t] = E[token[t]] * scale, scale 1 unless the model gives one (reference, which has none:
kernels/src/embed_kernel_cuda.cu:6-28); the
logits of the wanted rows are hN[row] . W^T in float32.  The reference always uses the
embedding matrix as W (model/src/qwen3_layers.cpp:246-265); here ``tied`` decides, and an
untied head reads ``lm_head.weight``.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .registry import register
from .spec import ParamSpec


@register("embedding", "token_embedding")
class TokenEmbedding:
    def __init__(self, vocab_size: int, hidden_size: int, dtype: torch.dtype, device, scale: float = 1.0,
                 name: str = "weight"):
        self.vocab, self.hidden, self.dtype, self.device = vocab_size, hidden_size, dtype, device
        self.scale, self.name = float(scale), name
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, vocab_size, hidden_size, scale: float = 1.0, name: str = "weight") -> Dict[str, ParamSpec]:
        return {name: ParamSpec((vocab_size, hidden_size))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.weight = t[self.name].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        h = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        if self.scale != 1.0:
            return ops.embedding(token_ids, self.weight, h, self.scale)
        return ops.embedding(token_ids, self.weight, h)


@register("embedding", "token_position_embedding")
class TokenPositionEmbedding:
    """h0[t] = norm(E[token[t]] * scale + P[position[t]]): a learned vector per position (``max_positions``
    rows, not scaled) and, if ``norm_eps`` is given, an RMS norm of the sum with the gain ``norm_offset`` +
    stored weight, all in float32 in one kernel.  The engine bounds a request's length by the model's
    ``max_positions`` (the cache manager refuses to reserve beyond it), so no row comes with a position past the table.

    ``side_columns`` > 0 adds a second table [vocab, side_columns] (``side_name``) that this part owns and
    layers look rows up in by the step's token ids (a per-layer input that depends on the token alone); it is
    published in the step's memo under ``TOKEN_SIDE`` so that the parts that use it need no copy of it."""
    TOKEN_SIDE = "token_side_table"
    takes_context = True

    def __init__(self, vocab_size: int, hidden_size: int, max_positions: int, dtype: torch.dtype, device,
                 scale: float = 1.0, name: str = "weight", pos_name: str = "pos", norm_name: Optional[str] = None,
                 norm_eps: Optional[float] = None, norm_offset: float = 0.0, side_columns: int = 0,
                 side_name: str = "side"):
        self.vocab, self.hidden, self.max_positions = vocab_size, hidden_size, int(max_positions)
        self.dtype, self.device, self.scale = dtype, device, float(scale)
        self.name, self.pos_name, self.norm_name, self.side_name = name, pos_name, norm_name, side_name
        self.norm_eps, self.norm_offset, self.side_columns = norm_eps, float(norm_offset), int(side_columns)
        self.weight = self.pos = self.gain = self.side = None

    @classmethod
    def param_specs(cls, vocab_size, hidden_size, max_positions, scale: float = 1.0, name: str = "weight",
                    pos_name: str = "pos", norm_name: Optional[str] = None, norm_eps: Optional[float] = None,
                    norm_offset: float = 0.0, side_columns: int = 0, side_name: str = "side") -> Dict[str, ParamSpec]:
        specs = {name: ParamSpec((vocab_size, hidden_size)), pos_name: ParamSpec((max_positions, hidden_size))}
        if norm_name is not None:
            specs[norm_name] = ParamSpec((hidden_size,), "norm_zero" if norm_offset else "norm")
        if side_columns:
            specs[side_name] = ParamSpec((vocab_size, side_columns))
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.weight = t[self.name].contiguous()
        self.pos = t[self.pos_name].to(self.weight.dtype).contiguous()
        if self.norm_name is not None:
            self.gain = (t[self.norm_name].to(torch.float32) + self.norm_offset).contiguous()
        if self.side_columns:
            self.side = t[self.side_name].contiguous()

    def forward(self, token_ids: torch.Tensor, ctx=None) -> torch.Tensor:
        if ctx is None:
            raise ValueError("an embedding with positions needs the step's context")
        if self.side is not None:
            ctx.memo[self.TOKEN_SIDE] = self.side
        h = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        return ops.embedding_norm(token_ids, self.weight, h, self.scale, ctx.positions, self.pos, self.gain,
                                  self.norm_eps or 0.0)


@register("head", "lm_head")
class LMHead:
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, dtype: torch.dtype, device,
                 name: str = "weight", softcap: Optional[float] = None):
        """``softcap`` c: logits <- c tanh(logits / c), in float32."""
        self.vocab, self.hidden, self.tied, self.dtype, self.device = vocab_size, hidden_size, tied, dtype, device
        self.name, self.softcap = name, softcap
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, vocab_size, hidden_size, tied, name: str = "weight", softcap=None) -> Dict[str, ParamSpec]:
        return {} if tied else {name: ParamSpec((vocab_size, hidden_size))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = t[self.name].contiguous()

    def tie(self, embedding: TokenEmbedding) -> None:
        if self.tied:
            self.weight = embedding.weight

    def workspace_floats(self, rows: int) -> int:
        return rows * self.vocab                 # the logits

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(x, self.weight, out_dtype=torch.float32)
        if self.softcap:
            return ops.softcap(logits, self.softcap)
        return logits
