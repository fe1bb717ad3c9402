"""Routed experts: `experts` small feed-forward layers of which every token uses `top`, plus an optional shared expert.

  z = h Wr^T + b (float32);  the `top` largest z are chosen, their weights are the softmax over the chosen z alone
  out = sum_j weight_j * expert_(e_j)(h)  +  sigmoid(h ws^T) * shared(h)
  expert(h) = act(h Wup^T) Wdown^T,  act = the square of relu (no gate matrix, no biases)

A second form of both halves, by parameters: `routing="sigmoid_groups"` scores the experts by s = sigmoid(z), chooses by
s + correction among the experts of the `group_keep` best of `groups` groups of neighbours (a group's score: the sum of its
two largest s + correction) and weighs by the chosen s themselves; `activation="clamped_swiglu"` gives every expert a gate
and an up matrix: g = min(gate h, limit), u = clamp(up h, -limit, limit), expert(h) = (g sigmoid(alpha g) (u + 1)) Wdown^T.

`routing="sigmoid_top"` is the same scoring without groups or correction.  `activation="silu"` or `"gelu_tanh"` gives gated
experts without the clamp, expert(h) = (act(gate h) * (up h)) Wdown^T; with `weight_on_input` the routing weight multiplies
what the expert reads, out = sum_j expert_(e_j)(w_j h): gate and up are linear in h, so the weight is applied, in float32, to
their products inside the activation kernel, and the combine adds the experts' outputs unweighted.

`routing="softmax_all"` scores by a softmax over ALL router outputs, chooses by score + correction and weighs by the chosen
scores themselves times `route_scale`, not renormalised.  With `identity_experts` = n the router has n outputs more than there
are experts; a token that chooses one of them gets its own input back, times the weight (the combine adds it; such a choice
costs no product).  A shared expert beside gated experts is gated like them (`shared_up` stacks its gate and up matrices).

All experts' matrices are stacked ([experts, ff, width], [experts, width, ff]).  The routing is sorted on the device
(csrc/moe.cu): no value comes back to the host, and a step's launches have the same shape whatever the routing is, so
decode steps can be replayed from CUDA graphs.  The router and the shared expert's gate are rows of one float32 product.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import FeedForward, StepContext, WeightSpec, register_part
from .linear import matmul_tn


USE_TC = True      # bfloat16: the experts' products on tcgen05 (csrc/moe_tc.cu)


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, expert_size: int, shared_size: int = 0,
                 activation: str = "relu2", router_bias: bool = True, shared_gate: bool = True,
                 routing: str = "softmax_top", groups: int = 1, group_keep: int = 1, limit: Optional[float] = None,
                 alpha: float = 1.702, weight_on_input: bool = False, route_scale: float = 1.0, identity_experts: int = 0):
        if not (0 < top_k <= num_experts + int(identity_experts or 0)):
            raise ValueError(f"{top_k} choices of {num_experts} experts")
        if activation not in kernels.MOE_ACTS and activation != "clamped_swiglu" and activation not in kernels.GLU_ACTS:
            raise ValueError(f"activation {activation!r} is not supported (known: relu2, clamped_swiglu, silu, gelu_tanh, none)")
        if routing not in ("softmax_top", "sigmoid_groups", "sigmoid_top", "softmax_all"):
            raise ValueError(f"routing {routing!r} is not supported (known: softmax_top, sigmoid_groups, sigmoid_top, softmax_all)")
        self.route_scale, self.identity_experts = float(route_scale), int(identity_experts or 0)
        if self.identity_experts < 0 or (self.identity_experts and routing != "softmax_all"):
            raise ValueError("experts that return their input are built for the routing softmax_all")
        if routing == "softmax_all" and (weight_on_input or top_k > num_experts + self.identity_experts):
            raise ValueError(f"softmax_all: {top_k} choices of {num_experts + self.identity_experts} outputs, weights on the output")
        if routing == "sigmoid_top":
            routing, groups, group_keep = "sigmoid_groups", 1, 1
        self.routing, self.groups, self.group_keep = routing, int(groups), int(group_keep)
        if routing == "sigmoid_groups" and (self.groups < 1 or num_experts % self.groups or not (1 <= self.group_keep <= self.groups)
                                            or self.group_keep * (num_experts // self.groups) < top_k):
            raise ValueError(f"{num_experts} experts in {groups} groups of which {group_keep} are kept cannot give {top_k} choices")
        self.clamped = activation == "clamped_swiglu"
        self.gated = self.clamped or activation in kernels.GLU_ACTS        # experts with a gate and an up matrix
        self.weight_on_input = bool(weight_on_input)
        if self.weight_on_input and (self.clamped or not self.gated):
            raise ValueError("the routing weight on the expert's input is built for silu and gelu_tanh gated experts")
        if self.clamped and not (limit is not None and limit > 0):
            raise ValueError("the clamped activation needs a positive limit")
        if self.clamped and shared_size:
            raise ValueError("a shared expert beside clamped experts is not built")
        self.limit, self.alpha = (float(limit) if limit is not None else None), float(alpha)
        self.hidden_size, self.num_experts, self.top_k = int(hidden_size), int(num_experts), int(top_k)
        self.expert_size, self.shared_size = int(expert_size), int(shared_size or 0)
        self.activation = activation
        self.has_router_bias = bool(router_bias)
        self.has_shared_gate = bool(shared_gate) and self.shared_size > 0
        self.up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None
        self.router: Optional[torch.Tensor] = None
        self.router_bias: Optional[torch.Tensor] = None
        self.shared_up: Optional[torch.Tensor] = None
        self.shared_down: Optional[torch.Tensor] = None
        self._bias32: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, E, F = self.hidden_size, self.num_experts, self.expert_size
        # gated experts: "up" lists, expert by expert, the gate matrix and then the up matrix
        R = E + self.identity_experts                     # router outputs
        specs = {"up": WeightSpec([(F, D)] * (2 * E if self.gated else E)), "down": WeightSpec([(D, F)] * E),
                 "router": WeightSpec([(R, D)] + ([(1, D)] if self.has_shared_gate else []))}
        if self.has_router_bias:
            specs["router_bias"] = WeightSpec([(R,)], keep_fp32=True)
        if self.shared_size:
            # beside gated experts the shared expert is gated too: its gate matrix, then its up matrix
            specs["shared_up"] = WeightSpec([(self.shared_size, D)] * (2 if self.gated else 1))
            specs["shared_down"] = WeightSpec([(D, self.shared_size)])
        return specs

    def activation_width(self) -> int:
        return self.top_k * ((3 if self.gated else 1) * self.expert_size + 2 * self.hidden_size) + self.shared_size + self.hidden_size

    def prepare(self, dtype, device) -> None:
        self._bias32 = self.router_bias.float().contiguous() if self.has_router_bias else None

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        n, D, E, K, F = h.shape[0], self.hidden_size, self.num_experts, self.top_k, self.expert_size
        dev = h.device
        z = matmul_tn(h, self.router, out_dtype=torch.float32)           # [n, experts (+ 1: the shared expert's gate)]
        ids = torch.empty((n, K), dtype=torch.int32, device=dev)
        wts = torch.empty((n, K), dtype=torch.float32, device=dev)
        R = E + self.identity_experts
        if self.routing == "sigmoid_groups":
            kernels.moe_topk_sigmoid(ids, wts, z, self._bias32, E, self.groups, self.group_keep)
        elif self.routing == "softmax_all":
            kernels.moe_topk_softmax_all(ids, wts, z, self._bias32, R, self.route_scale)
        else:
            kernels.moe_topk(ids, wts, z, self._bias32, E)
        pairs = n * K
        FU = 2 * F if self.gated else F                     # rows of an expert's first matrix
        act = None if self.gated else self.activation
        up3, down3 = self.up.view(E, FU, D), self.down.view(E, D, F)
        # bfloat16: the experts' products run on the tensor cores (tiles of 128 rows); float32, or sizes that the
        # 16-byte copies cannot take: the FFMA kernel (tiles of 64 rows)
        use_tc = USE_TC and F % 8 == 0 and kernels.moe_grouped_tc_supported(h, up3) and down3.data_ptr() % 16 == 0
        tile_rows = kernels.MOE_TC_TILE_ROWS if use_tc else kernels.moe_tile_rows()
        max_tiles = kernels.moe_max_tiles(pairs, E, tile_rows)
        book = torch.empty(E + 1 + 2 * pairs + 4 * max_tiles + 4, dtype=torch.int32, device=dev)
        offsets, pair_row = book[:E + 1], book[E + 1:E + 1 + pairs].view(n, K)
        row_token = book[E + 1 + pairs:E + 1 + 2 * pairs]
        tiles = book[E + 1 + 2 * pairs:E + 1 + 2 * pairs + 4 * max_tiles].view(max_tiles, 4)
        meta = book[E + 1 + 2 * pairs + 4 * max_tiles:]
        kernels.moe_align(ids, E, tile_rows, offsets, pair_row, row_token, tiles, meta)
        y = torch.empty((pairs, FU), dtype=h.dtype, device=dev)
        d = torch.empty((pairs, D), dtype=torch.float32, device=dev)
        flag = ctx.error_flag if ctx is not None else None
        if use_tc:
            kernels.moe_grouped_tc(y, h, up3, row_token, tiles, meta, act=act, error_flag=flag)
        else:
            kernels.moe_grouped(y, h, up3, row_token, tiles, meta, act=act)
        if self.gated:                                      # [pairs, gate | up] -> [pairs, F]
            y2 = torch.empty((pairs, F), dtype=h.dtype, device=dev)
            if self.clamped:
                kernels.clamped_glu(y2, y, self.limit, self.alpha)
            else:
                kernels.moe_weighted_glu(y2, y, pair_row, wts if self.weight_on_input else None, self.activation)
            y = y2
        if use_tc:
            kernels.moe_grouped_tc(d, y, down3, None, tiles, meta, error_flag=flag)
        else:
            kernels.moe_grouped(d, y, down3, None, tiles, meta)
        shared = None
        if self.shared_size:
            s = matmul_tn(h, self.shared_up)
            if self.gated:
                s2 = torch.empty((n, self.shared_size), dtype=h.dtype, device=dev)
                kernels.gated_act(s2, s, self.activation)
                s = s2
            elif self.activation == "relu2":
                kernels.relu2_(s)
            shared = matmul_tn(s, self.shared_down)
        out = torch.empty((n, D), dtype=h.dtype, device=dev)
        # weight_on_input: the weights are inside the experts already
        kernels.moe_combine(out, d, pair_row, None if self.weight_on_input else wts, shared, z[:, R] if self.has_shared_gate else None,
                            identity=(ids, E, h) if self.identity_experts else None)
        return out
