"""Arrangements of parts inside one layer.

`pre_norm` is the reference's Block (core/src/model_executor/models/llama/llama.rs:276-385): norm,
mixer, norm, feed-forward, where each residual add is deferred into the following norm
(llama.rs:295-317, :333) and the layer hands (branch output, residual) to the next one.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from .. import kernels
from .base import Block, LayerCache, Norm, NormAfter, Normed, Part, StepContext, register_part

# A step of a few tokens in bfloat16: a norm between two weight-streaming products is done by those products
# (the one before adds to the residual stream and leaves sums of squares, the one after divides).  LMSF_FUSE_NORMS=0:
# every norm is a kernel of its own.
FUSE_NORMS = os.environ.get("LMSF_FUSE_NORMS", "1") != "0"


def norm_after(ctx: StepContext, producer: Part, norm: Norm, consumer: Part, res: Optional[torch.Tensor]) -> Optional[NormAfter]:
    """The offer to `producer` to take `norm` into its last product, if everybody involved is able to on this step."""
    if (FUSE_NORMS and res is not None and getattr(producer, "fuses_norm", False)
            and getattr(consumer, "takes_prenormed", False) and getattr(norm, "splittable", False)
            and ctx.dtype == torch.bfloat16 and ctx.n_tokens <= kernels.SKINNY_MAX_M):
        return NormAfter(norm, res)
    return None


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: Dict[str, Part]):
        super().__init__(parts)
        self.mixer_norm, self._mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.feed_forward = parts["ffn_norm"], parts["feed_forward"]

    fuses_next_norm = True

    def entry(self) -> Optional[Tuple[Norm, Part]]:
        return self.mixer_norm, self._mixer

    def forward(self, ctx: StepContext, x, res: Optional[torch.Tensor], cache: LayerCache,
                next_entry: Optional[Tuple[Norm, Part]] = None):
        h, res = self.mixer_norm.forward_residual(x, res)
        then = norm_after(ctx, self._mixer, self.ffn_norm, self.feed_forward, res)
        a = self._mixer.forward(ctx, h, cache, then=then) if then is not None else self._mixer.forward(ctx, h, cache)
        h, res = self.ffn_norm.forward_residual(a, res)
        then = norm_after(ctx, self.feed_forward, next_entry[0], next_entry[1], res) if next_entry is not None else None
        out = self.feed_forward.forward(ctx, h, then=then) if then is not None else self.feed_forward.forward(ctx, h)
        return out, res


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before AND after each branch:  x <- x + post(mixer(pre(x))),  x <- x + post(ff(pre(x))), where a post norm
    may carry a layer scale (a learned vector that multiplies its output).  The residual stream is float32 and every
    sum into it is made in float32 from the float32 normed branch (the branch is never rounded before it is added).
    One kernel does what lies between two branches: the post norm of the branch before, the add, and the pre norm of
    the branch after (`kernels.stream_norm`); with `next_entry` it also applies the next block's first norm and
    hands it over as a `Normed`.  A layer may have no feed-forward.  With a `mixer_shift` the mixer reads the first norm's
    output mixed with the row of the token before (a `Shift` part, whose state per request the block declares)."""
    ROLES = {"mixer_norm": "norm", "mixer_shift": "shift", "mixer": "mixer", "mixer_post_norm": "norm",
             "ffn_norm": "norm", "feed_forward": "feed_forward", "ffn_post_norm": "norm"}
    OPTIONAL_ROLES = ("mixer_shift", "ffn_norm", "feed_forward", "ffn_post_norm")
    fuses_next_norm = True

    def __init__(self, parts: Dict[str, Part]):
        super().__init__(parts)
        self.mixer_norm, self._mixer, self.mixer_post = parts["mixer_norm"], parts["mixer"], parts["mixer_post_norm"]
        self.mixer_shift = parts.get("mixer_shift")
        self.feed_forward = parts.get("feed_forward")
        self.ffn_norm, self.ffn_post = parts.get("ffn_norm"), parts.get("ffn_post_norm")
        if self.feed_forward is not None and (self.ffn_norm is None or self.ffn_post is None):
            raise ValueError("a feed-forward needs the norms before and after it")
        for n in (self.mixer_norm, self.mixer_post, self.ffn_norm, self.ffn_post):
            if n is not None and not hasattr(n, "weight_f32"):
                raise ValueError("the sandwich block takes norms that are a factor per row times a weight (rmsnorm)")

    def entry(self) -> Optional[Tuple[Norm, Part]]:
        return self.mixer_norm, self._mixer

    def state_specs(self):
        return {"mixer_shift": self.mixer_shift.state_spec()} if self.mixer_shift is not None else {}

    @staticmethod
    def _between(res: torch.Tensor, branch: torch.Tensor, post, nxt: Optional[Norm]):
        """res += post(branch); returns nxt(res) in the branch's type (None without nxt)."""
        h = torch.empty_like(branch) if nxt is not None else None
        kernels.stream_norm(res, y=branch, w_post=post.weight_f32(), layer_scale=post.scale_f32(), eps_post=post.eps,
                            h=h, w_next=nxt.weight_f32() if nxt is not None else None,
                            eps_next=nxt.eps if nxt is not None else 0.0)
        return h

    def forward(self, ctx: StepContext, x, res: Optional[torch.Tensor], cache: LayerCache,
                next_entry: Optional[Tuple[Norm, Part]] = None):
        h, res = self.mixer_norm.forward_residual(x, res)      # x: None (complete stream), a Normed, or a pending branch
        if self.mixer_shift is not None:
            h = self.mixer_shift.forward(ctx, h, cache.extra["mixer_shift"])
        a = self._mixer.forward(ctx, h, cache)
        nxt = next_entry[0] if next_entry is not None and hasattr(next_entry[0], "weight_f32") and \
            not getattr(next_entry[0], "has_layer_scale", False) else None
        if self.feed_forward is None:
            h = self._between(res, a, self.mixer_post, nxt)
            return (Normed(h, nxt, res) if nxt is not None else None), res
        h = self._between(res, a, self.mixer_post, self.ffn_norm)
        f = self.feed_forward.forward(ctx, h)
        h = self._between(res, f, self.ffn_post, nxt)
        return (Normed(h, nxt, res) if nxt is not None else None), res


@register_part("block", "branch_norm")
class BranchNormBlock(Block):
    """Norms on the branches' outputs only:  x <- x + m * norm(mixer(x)),  x <- x + m * norm(ff(x)), and, where the layer
    has one, a third branch after the feed-forward, x <- x + m * norm(side(x)).  The branches read the stream itself (in
    the activation type); m is one factor for the whole model.  The residual stream is float32 and every sum into it is
    made in float32 from the float32 normed branch.  One kernel does what lies between two branches: the norm of the
    branch before, the scaled add, and the stream in the activation type for the branch after (`kernels.stream_norm`
    without a next norm); with `next_entry` of a block of this kind the last of them also serves the next block."""
    ROLES = {"mixer": "mixer", "mixer_post_norm": "norm", "feed_forward": "feed_forward", "ffn_post_norm": "norm",
             "side": "feed_forward", "side_post_norm": "norm"}
    OPTIONAL_ROLES = ("feed_forward", "ffn_post_norm", "side", "side_post_norm")
    fuses_next_norm = True

    def __init__(self, parts: Dict[str, Part], residual_mult: float = 1.0):
        super().__init__(parts)
        self.residual_mult = float(residual_mult)
        self._mixer = parts["mixer"]
        self.branches = [(parts["mixer"], parts["mixer_post_norm"])]
        for role, norm in (("feed_forward", "ffn_post_norm"), ("side", "side_post_norm")):
            if role in parts:
                if norm not in parts:
                    raise ValueError(f"the branch {role!r} needs its norm {norm!r}")
                self.branches.append((parts[role], parts[norm]))
        for _, n in self.branches:
            if not hasattr(n, "weight_f32") or getattr(n, "has_layer_scale", False):
                raise ValueError("the branch-norm block takes norms that are a factor per row times a weight (rmsnorm)")

    def entry(self) -> Optional[Tuple[Norm, Part]]:
        return None, self._mixer          # no norm before the first branch: it wants the stream itself

    def forward(self, ctx: StepContext, x, res: Optional[torch.Tensor], cache: LayerCache,
                next_entry: Optional[Tuple[Norm, Part]] = None):
        if isinstance(x, Normed):             # the block before left the stream in the activation type
            if x.norm is not None or x.res is not res:
                raise ValueError("a prepared activation was made for another norm or residual stream")
            h = x.h
        elif x is None:                       # a complete float32 stream
            h = self._as_activation(ctx, res)
        elif res is None:                     # the embedding's output starts the stream
            h = x
            if x.dtype == torch.float32:
                res = x
            else:
                res = torch.empty(x.shape, dtype=torch.float32, device=x.device)
                kernels.stream_begin(res, x)
        else:
            raise ValueError("the branch-norm block takes a complete stream, not a pending branch")
        wants_stream = next_entry is not None and next_entry[0] is None
        for i, (part, norm) in enumerate(self.branches):
            y = part.forward(ctx, h, cache) if i == 0 else part.forward(ctx, h)
            last = i == len(self.branches) - 1
            need_h = (not last) or wants_stream
            h = torch.empty_like(y) if (need_h and ctx.dtype != torch.float32) else None
            kernels.stream_norm(res, y=y, w_post=norm.weight_f32(), eps_post=norm.eps, h=h,
                                branch_scale=self.residual_mult)
            if need_h and h is None:
                h = res                       # float32 activations: the stream itself (no part writes its input)
        return (Normed(h, None, res) if wants_stream else None), res

    @staticmethod
    def _as_activation(ctx: StepContext, res: torch.Tensor) -> torch.Tensor:
        if ctx.dtype == torch.float32:
            return res
        h = torch.empty(res.shape, dtype=ctx.dtype, device=res.device)
        kernels.stream_norm(res, h=h)
        return h


@register_part("block", "parallel_gated")
class ParallelGatedBlock(Block):
    """One norm, two branches side by side, each behind a gate of its own:
         h = norm(x);  x <- x + sigmoid(W1 h + b1) * mixer(h) + sigmoid(W2 h + b2) * ff(h)
    The gates are vectors of the stream's width, multiplied element by element; their logits come from ONE product
    (`gates`: a `gate_logits` part whose matrix stacks W1 and W2) in float32.  One kernel ends the layer: both sigmoids,
    both products, the float32 sum into the stream and, when the next block starts with a norm of the same kind, that
    norm too (`kernels.gated_branches`).  A layer may have no feed-forward (and then no second gate)."""
    ROLES = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward", "gates": "linear"}
    OPTIONAL_ROLES = ("feed_forward",)
    fuses_next_norm = True

    def __init__(self, parts: Dict[str, Part]):
        super().__init__(parts)
        self.norm, self._mixer, self.gates = parts["norm"], parts["mixer"], parts["gates"]
        self.feed_forward = parts.get("feed_forward")
        if not hasattr(self.norm, "weight_f32") or getattr(self.norm, "has_layer_scale", False):
            raise ValueError("the parallel block takes a norm that is a factor per row times a weight (rmsnorm)")
        branches = 2 if self.feed_forward is not None else 1
        if not hasattr(self.gates, "logits") or self.gates.out_features != branches * self.norm.hidden_size:
            raise ValueError(f"the parallel block needs gate logits of {branches} x the stream's width")

    def entry(self) -> Optional[Tuple[Norm, Part]]:
        return self.norm, self._mixer

    def forward(self, ctx: StepContext, x, res: Optional[torch.Tensor], cache: LayerCache,
                next_entry: Optional[Tuple[Norm, Part]] = None):
        if x is not None and not isinstance(x, Normed) and res is None:      # the embedding's output starts the stream
            if x.dtype == torch.float32:
                res = x
            else:
                res = torch.empty(x.shape, dtype=torch.float32, device=x.device)
                kernels.stream_begin(res, x)
            x = None
        h, res = self.norm.forward_residual(x, res)       # x: None (a complete stream), a Normed, or a pending branch
        z = self.gates.logits(h)
        a = self._mixer.forward(ctx, h, cache)
        f = self.feed_forward.forward(ctx, h) if self.feed_forward is not None else None
        nxt = next_entry[0] if next_entry is not None and hasattr(next_entry[0], "weight_f32") and \
            not getattr(next_entry[0], "has_layer_scale", False) else None
        h_next = torch.empty_like(a) if nxt is not None else None
        kernels.gated_branches(res, z, self.gates.bias_f32(), a, f, h=h_next,
                               w_next=nxt.weight_f32() if nxt is not None else None,
                               eps_next=nxt.eps if nxt is not None else 0.0)
        return (Normed(h_next, nxt, res) if nxt is not None else None), res
