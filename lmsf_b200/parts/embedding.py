"""Token embedding: x[t] = E[id_t] (core/src/model_executor/layers/vocab_parallel_embedding.rs:5-38)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import Part, StepContext, WeightSpec, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, as_stream: bool = False):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale = float(scale)      # every embedding is multiplied by it (1 for Llama; sqrt(width) elsewhere)
        # as_stream: the embedding's output is handed over as the float32 residual stream (with a second copy for layers
        # that read it again), for models whose first block or stream entry wants a complete stream
        self.emits_stream = bool(as_stream)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec([(self.vocab_size, self.hidden_size)])}

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = torch.empty((ctx.n_tokens, self.hidden_size), dtype=self.weight.dtype, device=self.weight.device)
        kernels.embedding(x, self.weight, ctx.token_ids, ctx.error_flag, scale=self.scale)
        return x

    def forward_stream(self, ctx: StepContext, keep: bool = False):
        """(stream, copy of it or None), both float32 [n_tokens, hidden]."""
        x = self.forward(ctx)
        if x.dtype == torch.float32:
            res = x
        else:
            res = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            kernels.stream_begin(res, x)
        first = None
        if keep:
            first = torch.empty_like(res)
            kernels.stream_begin(first, x)
        return res, first


@register_part("embedding", "normed_token_embedding")
class NormedTokenEmbedding(Part):
    """x[t] = norm(E[id_t] * scale) * w: an embedding that passes through an RMS norm before it enters the residual
    stream.  The norm is float32 and its output IS the float32 stream (`emits_stream`): nothing is rounded in between.
    One kernel gathers, norms and, when asked, leaves a second copy of the result for layers that add it again."""
    graph_safe = True
    emits_stream = True

    def __init__(self, vocab_size: int, hidden_size: int, eps: float, scale: float = 1.0):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.eps, self.scale = float(eps), float(scale)
        self.weight: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None
        self._norm32: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec([(self.vocab_size, self.hidden_size)]),
                "norm": WeightSpec([(self.hidden_size,)], keep_fp32=True)}

    def prepare(self, dtype, device) -> None:
        self._norm32 = self.norm.float().contiguous()

    def forward_stream(self, ctx: StepContext, keep: bool = False):
        """(stream, copy of it or None), both float32 [n_tokens, hidden]."""
        res = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=self.weight.device)
        first = torch.empty_like(res) if keep else None
        kernels.embed_norm(res, first, self.weight, ctx.token_ids, self._norm32, self.eps, self.scale, ctx.error_flag)
        return res, first
