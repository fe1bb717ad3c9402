"""Attention whose keys and values are expanded from one low-rank vector per token, which is all that is cached.

  q = h Wq^T [heads x dk];  c = norm(h Wd^T) * w [rank];  k = c Wuk^T, v = c Wuv^T per head
  out = (sigmoid(h Wg^T)_head * softmax(scale q k^T over the window) v) Wo^T        (no position encoding)

Keys and values are linear in c, so the attention runs on c itself: the key expansion moves into the query
(q' = q Wuk per head, rank values), every head attends over the same cached c as key AND value (one kv head, one
plane of the paged cache: `KVCacheSpec(planes=1)`), and the value expansion is applied to the attention's output.
A step costs two small batched products per token instead of expanding every cached token again, and a page holds
`rank` values per token instead of heads x (dk + dv).  The rank is padded with zeros to what the attention kernels
take (a multiple of 16).  The norm of c is fused with the cache write (csrc/latent_cache.cu); the gate is applied by
the attention kernel to its output (it commutes with the linear value expansion).

With `rope_dim` > 0 every head has, beside its `head_dim` plain query values, `rope_dim` values that meet ONE key part
shared by all heads, a further `rope_dim` rows of the down projection that are not normed; both are rotated by their
positions (halves paired, the first `rope_dims` values) and the score is scale * (q_plain . k_plain + q_rot . k_rot).
The cached row is then [c | k_rot | zeros] and the query [Wuk^T q_plain | q_rot | zeros]: one dot product gives the
whole score, and the row still serves as the value because the value expansion reads its first `rank` values only.
`sink`: a learned number per head whose exponential joins the softmax's denominator without a key or a value.
"""
from __future__ import annotations

import warnings
from typing import Dict, Optional

import torch

from .. import kernels
from .base import KVCacheSpec, LayerCache, Mixer, StepContext, WeightSpec, register_part
from .attention import paged_attend
from .linear import batched_matmul_tn, matmul_tn

USE_FAST_KERNELS = True     # bfloat16: the tensor-core attention kernels on the one-plane cache


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, kv_rank: int, eps: float,
                 scale: Optional[float] = None, window: Optional[int] = None, gate: bool = True, rope_dim: int = 0,
                 rope_dims: Optional[int] = None, rope_base: float = 10000.0, sink: bool = False):
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.kv_rank = int(kv_rank)
        self.rope_dim = int(rope_dim or 0)
        self.rope_dims = int(rope_dims) if rope_dims is not None else self.rope_dim      # how many of them are rotated
        if self.rope_dims % 2 or not (0 <= self.rope_dims <= self.rope_dim):
            raise ValueError(f"{self.rope_dims} rotated values of {self.rope_dim}: an even number, at most all of them")
        self.rope_base = float(rope_base)
        self.has_sink = bool(sink)
        self.padded_rank = (self.kv_rank + self.rope_dim + 15) // 16 * 16
        if self.padded_rank > kernels.GENERIC_MAX_HEAD_DIM:
            raise ValueError(f"kv_rank {kv_rank} (+ {self.rope_dim}) is beyond the attention kernels (up to {kernels.GENERIC_MAX_HEAD_DIM})")
        self.eps = float(eps)
        self.scale = float(scale) if scale is not None else (self.head_dim + self.rope_dim) ** -0.5
        self.window = int(window) if window else None
        self.has_gate = bool(gate)
        self.q_size, self.v_size = self.num_heads * (self.head_dim + self.rope_dim), self.num_heads * self.value_dim
        self.sink: Optional[torch.Tensor] = None
        self._sink32: Optional[torch.Tensor] = None
        self._inv_freq: Optional[torch.Tensor] = None
        self.qcg: Optional[torch.Tensor] = None
        self.c_norm: Optional[torch.Tensor] = None
        self.uk: Optional[torch.Tensor] = None
        self.uv: Optional[torch.Tensor] = None
        self.o: Optional[torch.Tensor] = None
        self._uk_t: Optional[torch.Tensor] = None
        self._uv3: Optional[torch.Tensor] = None
        self._norm32: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, R = self.hidden_size, self.kv_rank
        merged = [(self.q_size, D), (R + self.rope_dim, D)] + ([(self.num_heads, D)] if self.has_gate else [])
        specs = {"qcg": WeightSpec(merged), "c_norm": WeightSpec([(R,)], keep_fp32=True),
                 "uk": WeightSpec([(self.num_heads * self.head_dim, R)]), "uv": WeightSpec([(self.v_size, R)]),
                 "o": WeightSpec([(D, self.v_size)])}
        if self.has_sink:
            specs["sink"] = WeightSpec([(self.num_heads,)], keep_fp32=True)
        return specs

    def cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(1, self.padded_rank, self.window, planes=1)

    def activation_width(self) -> int:
        return self.q_size + self.kv_rank + self.rope_dim + self.num_heads + 2 * self.num_heads * self.padded_rank + self.v_size

    def prepare(self, dtype, device) -> None:
        if dtype == torch.bfloat16 and not kernels.mma_attention_supported(dtype, self.padded_rank):
            warnings.warn(f"kv_rank {self.kv_rank} is beyond the tensor-core attention kernels (up to "
                          f"{kernels.MMA_MAX_HEAD_DIM}); bfloat16 attention runs on the plain kernel", RuntimeWarning, stacklevel=2)
        H, dk, dv, R, Rp = self.num_heads, self.head_dim, self.value_dim, self.kv_rank, self.padded_rank
        # the key expansion as the query sees it: per head [rank, dk]; without a rotated part the product also writes the
        # padding (zero rows), with one the rotation kernel writes everything behind the rank
        rows = R if self.rope_dim else Rp
        uk_t = torch.zeros((H, rows, dk), dtype=self.uk.dtype, device=self.uk.device)
        uk_t[:, :R, :] = self.uk.view(H, dk, R).transpose(1, 2)
        self._uk_t = uk_t
        self._uv3 = self.uv.view(H, dv, R)
        self._norm32 = self.c_norm.float().contiguous()
        self._sink32 = self.sink.float().contiguous() if self.has_sink else None
        if self.rope_dims:
            n = self.rope_dims
            self._inv_freq = torch.tensor([self.rope_base ** (-2.0 * i / n) for i in range(n // 2)],
                                          dtype=torch.float64).to(torch.float32).to(device)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        H, dk, dv, R, Rp = self.num_heads, self.head_dim, self.value_dim, self.kv_rank, self.padded_rank
        n = ctx.n_tokens
        group = ctx.groups[cache.group]
        dr = self.rope_dim
        p = matmul_tn(h, self.qcg)
        q, c_raw = p[:, :self.q_size], p[:, self.q_size:self.q_size + R + dr]
        g = p[:, self.q_size + R + dr:] if self.has_gate else None
        qa = torch.empty((n, H * Rp), dtype=p.dtype, device=p.device)
        if dr:
            if cache.owner:
                kernels.latent_norm_rope_cache_write(c_raw, self._norm32, self.eps, cache.kv, ctx.positions, ctx.token_seq,
                                                     group.block_table, group.block_size, R, dr, self.rope_dims,
                                                     self._inv_freq, ctx.error_flag)
            batched_matmul_tn(qa.view(n, H, Rp)[:, :, :R], q.view(n, H, dk + dr)[:, :, :dk], self._uk_t)
            kernels.latent_query_rope(qa, q, ctx.positions, H, dk, dr, self.rope_dims, self._inv_freq, R, Rp)
        else:
            if cache.owner:
                kernels.latent_norm_cache_write(c_raw, self._norm32, self.eps, cache.kv, ctx.positions, ctx.token_seq,
                                                group.block_table, group.block_size, R, ctx.error_flag)
            batched_matmul_tn(qa.view(n, H, Rp), q.view(n, H, dk), self._uk_t)
        oa = torch.empty_like(qa)
        self.attend(ctx, oa, qa, cache.kv, group, g)
        out = torch.empty((n, self.v_size), dtype=p.dtype, device=p.device)
        batched_matmul_tn(out.view(n, H, dv), oa.view(n, H, Rp)[:, :, :R], self._uv3)
        return matmul_tn(out, self.o)

    def attend(self, ctx: StepContext, out: torch.Tensor, q: torch.Tensor, kv: torch.Tensor, group, gate) -> None:
        """bfloat16 with a padded rank up to 256: the engine's tensor-core attention kernels (split-key decode, tcgen05
        or mma.sync prefill) with one kv head of `padded_rank` values whose cached vector is key and value at once,
        sinks included; the gate is a small kernel after them.  float32 and larger ranks: the plain kernel, gate included."""
        if USE_FAST_KERNELS and kernels.mma_attention_supported(q.dtype, self.padded_rank) and \
                not ctx.extras.get("force_generic_attention"):
            paged_attend(ctx, out, q, kv, group, num_heads=self.num_heads, num_kv_heads=1, head_dim=self.padded_rank,
                         scale=self.scale, window=self.window, kv_planes=1, sinks=self._sink32)
            if gate is not None:
                kernels.head_gate_(out, gate, self.num_heads, self.padded_rank)
            return
        kernels.attention_shared_kv(out, q, kv, group.block_table, group.block_size, ctx.token_seq, ctx.positions,
                                    self.scale, self.window or 0, self.num_heads, self.padded_rank, gate=gate,
                                    sinks=self._sink32)
