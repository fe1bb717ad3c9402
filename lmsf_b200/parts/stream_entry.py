"""What a span of layers that runs several times with the same weights does to the residual stream at the start of each
pass: the embedding's output is added again (every pass but the first), or the stream and the embedding's output pass
through one projection together (every pass), and a learned vector per pass is added."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import StepContext, StreamEntry, WeightSpec, register_part
from .linear import matmul_tn


@register_part("stream_entry", "loop_entry")
class LoopEntry(StreamEntry):
    """res += first (passes 1, 2, ... when `readd_first`) ; res += step[n_pass].  float32, one kernel.
    `mix_first`: instead of the sum, every pass (the first too) starts with res <- W [res | first] (weight `mix`
    [width, 2 width], the stream's columns first), a product in the activation type whose float32 result is the new
    stream; step[n_pass] is added to it."""
    graph_safe = True

    def __init__(self, hidden_size: int, times: int, readd_first: bool = True, step_vector: bool = True,
                 mix_first: bool = False):
        self.hidden_size, self.times = int(hidden_size), int(times)
        self.mix_first = bool(mix_first)
        self.readd_first, self.step_vector = bool(readd_first) and not self.mix_first, bool(step_vector)
        self.needs_first = self.mix_first or (self.readd_first and self.times > 1)
        self.step: Optional[torch.Tensor] = None
        self.mix: Optional[torch.Tensor] = None
        self._step32: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"step": WeightSpec([(self.times, self.hidden_size)], keep_fp32=True)} if self.step_vector else {}
        if self.mix_first:
            specs["mix"] = WeightSpec([(self.hidden_size, 2 * self.hidden_size)])
        return specs

    def prepare(self, dtype, device) -> None:
        self._step32 = self.step.float().contiguous() if self.step_vector else None

    def forward(self, ctx: StepContext, res: torch.Tensor, first: Optional[torch.Tensor], n_pass: int) -> Optional[torch.Tensor]:
        if not (0 <= n_pass < self.times):
            raise ValueError(f"pass {n_pass} of a span that runs {self.times} times")
        if self.mix_first:
            if first is None:
                raise ValueError("the embedding's output was not kept for the span's entry")
            both = torch.empty((res.shape[0], 2 * self.hidden_size), dtype=self.mix.dtype, device=res.device)
            kernels.stream_concat(both, res, first)
            new = matmul_tn(both, self.mix, out_dtype=torch.float32)
            if self.step_vector:
                kernels.stream_norm(new, vec=self._step32[n_pass])
            return new
        add_first = first if (self.readd_first and n_pass > 0) else None
        if self.readd_first and n_pass > 0 and first is None:
            raise ValueError("the embedding's output was not kept for the later passes")
        kernels.stream_norm(res, first=add_first, vec=self._step32[n_pass] if self.step_vector else None)
