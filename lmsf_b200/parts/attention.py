"""Grouped-query attention over the paged cache.

The reference's CausalSelfAttention (core/src/model_executor/models/llama/llama.rs:45-221) projects
q, k, v with one merged matrix, rotates q and k, scatters k and v into pages
(core/src/model_executor/layers/attention.rs:185-207) and then runs a dense prompt attention on
the fresh k, v or a paged decode kernel (attention.rs:209-294).  Here one step may hold prompt
portions and decoded tokens together: k and v always go to pages first and every query reads all
its keys from pages, so a portion that starts in the middle of a prompt needs nothing special.
"""
from __future__ import annotations

import math
import os
import warnings
from typing import Dict, Optional

import torch

from .. import kernels
from .base import (KVCacheSpec, LayerCache, Mixer, NormAfter, PositionEncoding, Prenormed, StepContext, WeightSpec,
                   register_part)
from . import linear
from .linear import matmul_tn, matmul_tn_residual


SPLITS_PER_REQUEST = os.environ.get("LMSF_DECODE_ITEMS", "1") != "0"   # decode batches of very different lengths: splits per request
USE_TC_PREFILL = True     # head sizes 64 and 128: prompt portions run on the tcgen05 kernel (csrc/attention_tc.cu)
FUSE_QKV_ROPE = True      # up to 16 single tokens: rotary encoding and cache write in the q/k/v product's epilogue


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    graph_safe = True      # launch geometry depends on the batch's size only: a decode step can be replayed
    takes_prenormed = True
    fuses_norm = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: Optional[PositionEncoding] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, bias: bool = False, softcap: Optional[float] = None,
                 value_dim: Optional[int] = None, qk_norm: bool = False, qk_norm_eps: float = 1e-6,
                 qk_norm_weights: bool = True, value_norm: bool = False, chunk: Optional[int] = None,
                 head_gate: bool = False, keep_first: int = 0, score_weights: str = "softmax", head_bias: bool = False,
                 value_gate: bool = False, own_kv: bool = True, cache_window="own",
                 cache_keep_first: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot be grouped over {num_kv_heads} kv heads")
        # head_dim is the stored size of a query or key head, value_dim that of a value head (default: the same).  The
        # cache and the kernels work on ONE width per head, a multiple of 16; where the stored sizes differ from it the
        # weights are padded with zero rows and columns when they are set (zeros change neither scores nor outputs)
        self.qk_dim, self.value_dim = int(head_dim), int(value_dim or head_dim)
        padded = value_dim is not None or qk_norm
        width = (max(self.qk_dim, self.value_dim) + 15) // 16 * 16 if padded else head_dim
        if width % 16 or not (16 <= width <= 256):
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take multiples of 16 "
                             f"from 16 to 256")
        scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
        head_dim = width
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        # RMS norm of every query and key head before the rotation (weights q_norm, k_norm [qk_dim], shared by the heads)
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        # qk_norm_weights False: the norm has no weight (a division by the root mean square alone).  value_norm: every value
        # head is divided by its root mean square over value_dim on its way into the cache (no weight either)
        self.qk_norm_weights, self.value_norm = bool(qk_norm_weights), bool(value_norm)
        if self.value_norm and not self.qk_norm:
            raise ValueError("a norm of the values goes with a norm of queries and keys")
        # chunk c: a query at position p sees the keys of its own chunk of positions, p - p % c .. p, counted from the
        # request's first token.  Pages of earlier chunks are kept (a request may be cut anywhere)
        self.chunk = int(chunk) if chunk else None
        # head_gate: head h's output is multiplied by sigmoid(w_h . x), one number per token and head, before the output
        # projection; the rows w_h are stored behind q, k and v in the merged matrix
        self.head_gate = bool(head_gate)
        if self.head_gate and bias:
            raise ValueError("a gate per head with projection biases is not built")
        # keep_first n (with a window): the request's first n keys stay visible when the window has passed them, at their
        # true positions.  score_weights "sigmoid": a visible key's weight is sigmoid(score) and the weights are not
        # normalised over the keys (no softmax).  head_bias: a learned number per query head (weight `head_bias`) added to
        # every scaled score.  value_gate: the concatenated value heads are multiplied element by element by sigmoid(Wg x)
        # before the output projection; Wg's rows ride behind q, k, v in the merged matrix.
        self.keep_first = int(keep_first or 0) if window else 0
        if score_weights not in ("softmax", "sigmoid"):
            raise ValueError(f"score weights {score_weights!r} are not supported (known: softmax, sigmoid)")
        self.sigmoid_weights = score_weights == "sigmoid"
        self.has_head_bias, self.value_gate = bool(head_bias), bool(value_gate)
        # own_kv False: the part has no key and value projections; every call of it reads the cache that another call owns
        self.own_kv = bool(own_kv)
        if (self.value_gate or not self.own_kv) and (bias or self.head_gate or qk_norm):
            raise ValueError("a gate per element, or a part without keys and values of its own, is not built with projection "
                             "biases, a gate per head or a norm of queries and keys")
        # what the cache keeps may be more than this part sees: other calls that read this call's cache can have wider masks
        # ("own": what this part's mask needs; None: every key; a number: a window of that size)
        self.cache_window = (int(window) if window else None) if cache_window == "own" else (int(cache_window) if cache_window else None)
        self.cache_keep_first = int(cache_keep_first) if cache_keep_first is not None else self.keep_first
        self.head_bias: Optional[torch.Tensor] = None
        self._hb32: Optional[torch.Tensor] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None
        self._qn32: Optional[torch.Tensor] = None
        self._kn32: Optional[torch.Tensor] = None
        self.position_encoding = position_encoding
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        # scores capped smoothly, softcap * tanh(score / softcap), before the softmax (not a Llama constant).  Only the
        # generic kernel takes it: a part built with a cap runs on that kernel in bfloat16 too, which is right and slow
        self.softcap = float(softcap) if softcap else 0.0
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.has_bias = bool(bias)
        self.qkv: Optional[torch.Tensor] = None
        self.o: Optional[torch.Tensor] = None
        self.qkv_bias: Optional[torch.Tensor] = None
        self.o_bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        H, G, dk, dv, D = self.num_heads, self.num_kv_heads, self.qk_dim, self.value_dim, self.hidden_size
        merged = [(H * dk, D)] + ([(G * dk, D), (G * dv, D)] if self.own_kv else [])
        merged += ([(H, D)] if self.head_gate else []) + ([(H * dv, D)] if self.value_gate else [])
        specs = {"qkv": WeightSpec(merged), "o": WeightSpec([(D, H * dv)])}
        if self.has_head_bias:
            specs["head_bias"] = WeightSpec([(H,)], keep_fp32=True)
        if self.has_bias:
            specs["qkv_bias"] = WeightSpec([(H * dk,), (G * dk,), (G * dv,)])
            specs["o_bias"] = WeightSpec([(D,)])
        if self.qk_norm and self.qk_norm_weights:
            specs["q_norm"] = WeightSpec([(dk,)], keep_fp32=True)
            specs["k_norm"] = WeightSpec([(dk,)], keep_fp32=True)
        return specs

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        H, G, dk, dv, hd = self.num_heads, self.num_kv_heads, self.qk_dim, self.value_dim, self.head_dim
        if dk != hd or dv != hd:
            tensors = dict(tensors)

            def pad_heads(t, heads, size):           # rows [heads * size, ...] -> [heads * hd, ...], zeros after `size`
                t = t.reshape(heads, size, *t.shape[1:])
                out = t.new_zeros((heads, hd, *t.shape[2:]))
                out[:, :size] = t
                return out.reshape(heads * hd, *t.shape[2:])

            for name in ("qkv", "qkv_bias"):
                if name in tensors and not self.own_kv:
                    t = tensors[name]
                    tensors[name] = torch.cat([pad_heads(t[:H * dk], H, dk), t[H * dk:]], 0).contiguous()
                elif name in tensors:
                    t = tensors[name]
                    q, k, v = t[:H * dk], t[H * dk:(H + G) * dk], t[(H + G) * dk:(H + G) * dk + G * dv]
                    rest = t[(H + G) * dk + G * dv:]            # the rows of a gate, if any
                    tensors[name] = torch.cat([pad_heads(q, H, dk), pad_heads(k, G, dk), pad_heads(v, G, dv), rest], 0).contiguous()
            if "o" in tensors:
                o = tensors["o"].reshape(-1, H, dv)
                po = o.new_zeros((o.shape[0], H, hd))
                po[:, :, :dv] = o
                tensors["o"] = po.reshape(o.shape[0], H * hd).contiguous()
        if (self.head_gate or self.value_gate) and "qkv" in tensors and tensors["qkv"].shape[0] % 8:
            # the gate's rows end the merged matrix: zero rows after them keep the product's row stride a multiple of 16
            # bytes, which the attention kernels ask of the queries they read in place
            tensors = dict(tensors)
            t = tensors["qkv"]
            tensors["qkv"] = torch.cat([t, t.new_zeros((8 - t.shape[0] % 8, t.shape[1]))], 0).contiguous()
        super().set_weights(tensors)

    def cache_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.cache_window,
                           keep_first=self.cache_keep_first if self.cache_window else 0)

    def activation_width(self) -> int:
        # q, k, v and the attention's output; the logits of a gate per element ride in the merged product
        return 2 * self.q_size + 2 * self.kv_size + (self.num_heads * self.value_dim if self.value_gate else 0)

    def prepare(self, dtype, device) -> None:
        if self.position_encoding is not None:
            self.position_encoding.prepare(dtype, device)
        if self.qk_norm and self.qk_norm_weights:
            self._qn32, self._kn32 = self.q_norm.float().contiguous(), self.k_norm.float().contiguous()
        if self.has_head_bias:
            self._hb32 = self.head_bias.float().contiguous()
        if dtype == torch.bfloat16 and not kernels.mma_attention_supported(dtype, self.head_dim):
            # right but slow: said once, so that nobody wonders where the time goes
            warnings.warn(f"head_dim {self.head_dim} is beyond the tensor-core attention kernels "
                          f"(up to {kernels.MMA_MAX_HEAD_DIM}); bfloat16 attention runs on the generic kernel",
                          RuntimeWarning, stacklevel=2)
        elif dtype == torch.bfloat16 and (self.softcap or self._slopes() is not None):
            warnings.warn("a cap on the attention scores, or a bias that is linear in the distance, is taken by the generic "
                          "kernel only; bfloat16 attention runs on it", RuntimeWarning, stacklevel=2)
        slopes = self._slopes()
        if slopes is not None and slopes.numel() != self.num_heads:
            raise ValueError(f"{slopes.numel()} slopes for {self.num_heads} query heads")

    def _slopes(self) -> Optional[torch.Tensor]:
        return self.position_encoding.score_slopes() if self.position_encoding is not None else None

    def _log_bias(self):
        f = getattr(self.position_encoding, "score_log_bias", None)
        return f() if f is not None else None

    def forward(self, ctx: StepContext, h, cache: LayerCache, then: Optional[NormAfter] = None):
        group = ctx.groups[cache.group]
        fused = self.position_encoding.fused_rotary() if self.position_encoding is not None else None
        hx = h.x if isinstance(h, Prenormed) else h
        if not cache.owner and self.own_kv is False and cache.kv is None:
            raise ValueError("a part without keys and values of its own was given no cache to read")
        if cache.owner and not self.own_kv:
            raise ValueError("a part without key and value projections cannot own a cache: its call must name the call whose cache it reads")
        if (FUSE_QKV_ROPE and cache.owner and not self.value_gate and linear.USE_SKINNY and self.qkv_bias is None and not self.qk_norm and (fused is not None or self.position_encoding is None)
                and kernels.gemm_skinny_qkv_rope_supported(hx, self.qkv, self.head_dim, fused[1] if fused else 0,
                                                           fused[2] if fused else True)):
            # a few single tokens (a decode step): projection, rotation and cache write in one kernel
            inv_freq, rot_dim, is_neox = fused if fused is not None else (None, 0, True)
            q = torch.empty((ctx.n_tokens, self.q_size), dtype=hx.dtype, device=hx.device)
            kernels.gemm_skinny_qkv_rope(q, hx, self.qkv, ctx.positions, ctx.token_seq, group.block_table, group.block_size,
                                         cache.kv, inv_freq, rot_dim, is_neox, self.num_heads, self.num_kv_heads,
                                         self.head_dim, ctx.error_flag,
                                         prenorm=(h.sumsq, h.eps, h.width) if isinstance(h, Prenormed) else None)
            out = torch.empty((ctx.n_tokens, self.q_size), dtype=hx.dtype, device=hx.device)
            self.attend(ctx, out, q, cache.kv, group)
            return self._project_out(out, then)
        gate = vgate = None
        n_vg = self.num_heads * self.value_dim
        if cache.owner:
            qkv = matmul_tn(h, self.qkv, bias=self.qkv_bias)
            q = qkv[:, :self.q_size]
            k = qkv[:, self.q_size:self.q_size + self.kv_size]
            v = qkv[:, self.q_size + self.kv_size:self.q_size + 2 * self.kv_size]
            if self.head_gate:
                gate = qkv[:, self.q_size + 2 * self.kv_size:self.q_size + 2 * self.kv_size + self.num_heads]
            if self.value_gate:
                vgate = qkv[:, self.q_size + 2 * self.kv_size:self.q_size + 2 * self.kv_size + n_vg]
        elif not self.own_kv:   # queries (and the gate) in one product: the matrix holds nothing else
            qg = matmul_tn(h, self.qkv)
            q, k, v = qg[:, :self.q_size], None, None
            if self.value_gate:
                vgate = qg[:, self.q_size:self.q_size + n_vg]
        elif self.value_gate:   # the keys and values are another call's although this part has projections for them
            q = matmul_tn(h, self.qkv[:self.q_size])
            k = v = None
            vgate = matmul_tn(h, self.qkv[self.q_size + 2 * self.kv_size:])[:, :n_vg]
        else:  # keys and values are another call's: only the queries are needed
            q = matmul_tn(h, self.qkv[:self.q_size], bias=None if self.qkv_bias is None else self.qkv_bias[:self.q_size])
            k = v = None
            if self.head_gate:
                gate = matmul_tn(h, self.qkv[self.q_size + 2 * self.kv_size:])[:, :self.num_heads]
        if self.position_encoding is not None and fused is None and self._slopes() is None and self._log_bias() is None:
            if self.qk_norm:
                raise ValueError("a norm of queries and keys goes with a rotary encoding, a bias on the scores or none")
            self.position_encoding.apply(ctx, q, k, self.num_heads, self.num_kv_heads, self.head_dim)
        inv_freq, rot_dim, is_neox = fused if fused is not None else (None, 0, True)
        if self.qk_norm:
            # norm, rotation and cache write in one kernel; the value is rounded once
            kernels.qk_norm_rope_cache_write(q, k, v, ctx.positions, ctx.token_seq, group.block_table, group.block_size,
                                             cache.kv if cache.owner else None, inv_freq, rot_dim, is_neox, self.num_heads,
                                             self.num_kv_heads, self.head_dim, self.qk_dim, self._qn32, self._kn32,
                                             self.qk_norm_eps, ctx.error_flag, weightless=not self.qk_norm_weights,
                                             v_norm_dim=self.value_dim if self.value_norm else 0)
        elif fused is not None or cache.owner:
            kernels.rope_cache_write(q, k, v, ctx.positions, ctx.token_seq, group.block_table, group.block_size,
                                     cache.kv if cache.owner else None, inv_freq, rot_dim, is_neox, self.num_heads,
                                     self.num_kv_heads, self.head_dim, ctx.error_flag)
        out = torch.empty((ctx.n_tokens, self.q_size), dtype=q.dtype, device=q.device)
        self.attend(ctx, out, q, cache.kv, group, gate)
        if vgate is not None:
            kernels.value_gate_(out, vgate, self.num_heads, self.head_dim, self.value_dim)
        return self._project_out(out, then)

    def _project_out(self, out: torch.Tensor, then: Optional[NormAfter]):
        if then is not None and self.o_bias is None:
            p = matmul_tn_residual(out, self.o, then)
            if p is not None:
                return p
        return matmul_tn(out, self.o, bias=self.o_bias)

    def attend(self, ctx: StepContext, out: torch.Tensor, q: torch.Tensor, kv: torch.Tensor, group, gate=None) -> None:
        paged_attend(ctx, out, q, kv, group, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                     scale=self.scale, window=self.window, softcap=self.softcap, slopes=self._slopes(), chunk=self.chunk,
                     log_bias=self._log_bias(), gate=gate, keep_first=self.keep_first, sigmoid=self.sigmoid_weights,
                     head_bias=self._hb32)


def paged_attend(ctx: StepContext, out: torch.Tensor, q: torch.Tensor, kv: torch.Tensor, group, *, num_heads: int,
                 num_kv_heads: int, head_dim: int, scale: float, window: Optional[int] = None, softcap: float = 0.0,
                 slopes: Optional[torch.Tensor] = None, kv_planes: int = 2, chunk: Optional[int] = None,
                 log_bias=None, gate: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                 keep_first: int = 0, sigmoid: bool = False, head_bias: Optional[torch.Tensor] = None) -> None:
    """Attention over pages for any mix of tokens.  bfloat16 with a head size up to 256: single tokens go to the
    split-key decode kernel, longer portions to a tiled prefill kernel (tcgen05 with accumulators in tensor memory for
    head sizes 64 and 128, mma.sync otherwise).  Everything else, float32 included, runs on the generic kernel, which is
    also their plain twin.  kv_planes 1: one cached vector per token and kv head is key and value at once (the fast
    kernels only; the caller keeps its own plain kernel for that layout).  chunk: a query sees the keys of its own chunk of
    positions only; log_bias (r1, r2): r1 * log(1 + r2 * distance) is taken off the scores; sinks [heads]: exp(sink) joins
    the softmax's denominator (all three: every kernel); gate [n, heads]: the output of head h is multiplied by
    sigmoid(gate[:, h]) (the generic kernel itself, a small kernel after the fast ones).  keep_first: with a window, the
    request's first keys stay visible behind it; sigmoid: a key's weight is sigmoid(score), not normalised; head_bias [heads]:
    added to the scaled scores."""
    if kernels.mma_attention_supported(q.dtype, head_dim) and not softcap and slopes is None and \
            not ctx.extras.get("force_generic_attention"):
        extras = dict(chunk=chunk or 0, log_bias=log_bias, sinks=sinks, keep_first=keep_first if window else 0,
                      sigmoid=sigmoid, head_bias=head_bias)
        if ctx.n_decode_seqs:
            max_ctx = ctx.extras.get("decode_max_ctx")
            if max_ctx is None:
                max_ctx = ctx.extras["decode_max_ctx"] = max(c for c, n in zip(ctx.ctx_lens, ctx.q_lens) if n == 1)
            visible = min(max_ctx, window + (keep_first or 0)) if window else max_ctx
            if chunk:
                visible = min(visible, chunk)
            # the mean matters to the plan only where it is far below the longest context (a graph names its class)
            mean_ctx = ctx.extras.get("decode_mean_ctx")
            if mean_ctx is None:
                lens = [c for c, n in zip(ctx.ctx_lens, ctx.q_lens) if n == 1]
                mean_ctx = ctx.extras["decode_mean_ctx"] = sum(lens) / len(lens)
            mean_visible = min(mean_ctx, visible)
            group_size = num_heads // num_kv_heads
            all_decode = ctx.n_decode_seqs == ctx.n_seqs
            if SPLITS_PER_REQUEST and ctx.n_decode_seqs >= 2 and mean_visible * 4 <= visible:
                # Requests that differ much in length (a mean of a quarter of the longest and less): splits per
                # request, from a list of work items that a kernel makes from the step's context lengths (once a
                # step, for all layers of this geometry).  Measured, 8 layers of the 8B shape: one request at
                # 30,000 tokens beside 63 at 500: 1.64 ms a step against 2.11 ms with one number of splits for all;
                # one at 2,300 beside 63 at 1,200: 1.54 against 1.50 (the list's launch starts after the kernel
                # before it and adds up through global memory), hence the threshold.
                widths = kernels.decode_widths(head_dim, group_size)
                pairs = ctx.n_decode_seqs * num_kv_heads * ((group_size + 15) // 16)
                warps, slots = widths[0][0], widths[0][2][0]
                if len(widths) > 1 and pairs > slots:
                    warps, slots = widths[1][0], widths[1][2][0]
                key = ("decode_items", num_kv_heads, group_size, slots, window or 0, chunk or 0)
                items = ctx.extras.get(key)
                if items is None:
                    capacity = kernels.decode_items_capacity(ctx.n_decode_seqs, num_kv_heads, group_size, slots)
                    items = ctx.extras[key] = torch.empty((capacity, 4), dtype=torch.int32, device=q.device)
                    kernels.decode_build_items(items, ctx.ctx_len, None if all_decode else ctx.decode_seq_ids,
                                               ctx.n_decode_seqs, window or 0, num_heads, num_kv_heads,
                                               head_dim, slots, chunk=chunk or 0)
                need = kernels.attention_decode_items_scratch_floats(items.shape[0], num_heads, head_dim)
                scratch = ctx.extras.get("decode_items_scratch")
                if scratch is None or scratch.numel() < need:
                    scratch = ctx.extras["decode_items_scratch"] = torch.zeros(need, dtype=torch.float32, device=q.device)
                kernels.attention_decode_items(out, q, kv, group.block_table, group.block_size, items, ctx.cu_q,
                                               ctx.ctx_len, scale, window or 0, num_heads,
                                               num_kv_heads, head_dim, warps, scratch, kv_planes=kv_planes, **extras)
                splits = None
            else:
                splits, warps = kernels.decode_plan(ctx.n_decode_seqs, num_kv_heads, group_size, visible,
                                                    head_dim, kernels.decode_widths(head_dim, group_size),
                                                    mean_ctx=mean_visible if mean_visible * 4 <= visible * 3 else None)
            if splits is not None:
                need = kernels.attention_decode_scratch_floats(ctx.n_seqs, num_heads, splits, head_dim)
                scratch = ctx.extras.get("decode_scratch")
                if need and (scratch is None or scratch.numel() < need):
                    scratch = ctx.extras["decode_scratch"] = torch.zeros(need, dtype=torch.float32, device=q.device)
                kernels.attention_decode(out, q, kv, group.block_table, group.block_size,
                                         None if all_decode else ctx.decode_seq_ids, ctx.n_decode_seqs, ctx.cu_q,
                                         ctx.ctx_len, scale, window or 0, num_heads,
                                         num_kv_heads, head_dim, splits, scratch if need else None, warps,
                                         kv_planes=kv_planes, **extras)
        if ctx.n_q_tiles and USE_TC_PREFILL and kernels.tc_attention_supported(q.dtype, head_dim):
            kernels.attention_prefill_tc(out, q, kv, group.block_table, group.block_size, ctx.q_tile128_seq,
                                         ctx.q_tile128_q0, ctx.n_q_tiles128, ctx.cu_q, ctx.ctx_len, scale,
                                         window or 0, num_heads, num_kv_heads, head_dim,
                                         ctx.error_flag, kv_planes=kv_planes, **extras)
        elif ctx.n_q_tiles:
            kernels.attention_prefill(out, q, kv, group.block_table, group.block_size, ctx.q_tile_seq,
                                      ctx.q_tile_q0, ctx.n_q_tiles, ctx.cu_q, ctx.ctx_len, scale,
                                      window or 0, num_heads, num_kv_heads, head_dim, kv_planes=kv_planes, **extras)
        if gate is not None:
            kernels.head_gate_(out, gate, num_heads, head_dim)
        return
    if kv_planes != 2:
        raise ValueError("the plain attention kernel of keys and values takes a cache of two planes")
    kernels.attention_generic(out, q, kv, group.block_table, group.block_size, ctx.token_seq, ctx.positions,
                              scale, window or 0, num_heads, num_kv_heads, head_dim,
                              softcap=softcap, slopes=slopes, chunk=chunk or 0, log_bias=log_bias, gate=gate, sinks=sinks,
                              keep_first=keep_first if window else 0, sigmoid=sigmoid, head_bias=head_bias)
