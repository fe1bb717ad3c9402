"""Token shift: what a mixer reads is mixed with what it would have read one token earlier.

  h'_t = h_t + (h_{t-1} - h_t) * mix        (element by element; mix is a learned vector of the stream's width)

h_{t-1} is the row of the token before in the same request as it was BEFORE this replacement, and zeros for the request's
first token.  Between steps it is state of the request (float32 [width] per state slot): a portion's first token reads the
slot, the portion's last row is left there.  One kernel (csrc/stream_norm.cu, `token_shift`), float32 inside.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import Shift, StateSpec, StepContext, WeightSpec, register_part


@register_part("shift", "token_shift")
class TokenShift(Shift):
    graph_safe = True

    def __init__(self, hidden_size: int):
        self.hidden_size = int(hidden_size)
        self.mix: Optional[torch.Tensor] = None
        self._mix32: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"mix": WeightSpec([(self.hidden_size,)], keep_fp32=True)}

    def state_spec(self) -> StateSpec:
        return StateSpec((self.hidden_size,), torch.float32)

    def prepare(self, dtype, device) -> None:
        self._mix32 = self.mix.float().contiguous()

    def forward(self, ctx: StepContext, h: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(h)
        kernels.token_shift(out, h, self._mix32, state, ctx.positions, ctx.token_seq, ctx.cu_q, ctx.state_slot)
        return out
