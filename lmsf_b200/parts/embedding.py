"""Token embedding: x[t] = E[id_t] (core/src/model_executor/layers/vocab_parallel_embedding.rs:5-38)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import Part, StateSpec, StepContext, WeightSpec, register_part


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


@register_part("embedding", "pair_token_embedding")
class PairTokenEmbedding(Part):
    """x[t] = E[id_t] * scale + P[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets]: beside the token's own row a row of a
    second table that is chosen by the token and the one before it (a hashed pair); a request's first token takes that table's
    last row, number `buckets`.  The sum is float32 and IS the float32 residual stream (`emits_stream`).  The token before a
    portion's first token is state of the request: one int32 per state slot, kept on the device (`state_spec`), so that a
    token sampled on the device is the next step's token before without the host having seen it."""
    graph_safe = True
    emits_stream = True

    def __init__(self, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError(f"a pair table of {buckets} buckets with the multipliers {mul_prev}, {mul_cur}")
        self.scale = float(scale)
        self.weight: Optional[torch.Tensor] = None
        self.pairs: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec([(self.vocab_size, self.hidden_size)]),
                "pairs": WeightSpec([(self.buckets + 1, self.hidden_size)])}

    def state_spec(self) -> StateSpec:
        return StateSpec((1,), torch.int32)

    def forward_stream(self, ctx: StepContext, keep: bool = False):
        """(stream, copy of it or None), both float32 [n_tokens, hidden]."""
        if ctx.embedding_state is None:
            raise ValueError("the pair embedding needs its state slots (the step's context has none)")
        res = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=self.weight.device)
        kernels.embedding_pairs(res, self.weight, self.pairs, ctx.token_ids, ctx.positions, ctx.token_seq, ctx.cu_q,
                                ctx.state_slot, ctx.embedding_state, self.buckets, self.mul_prev, self.mul_cur, self.scale,
                                ctx.error_flag)
        return res, (res.clone() if keep else None)
