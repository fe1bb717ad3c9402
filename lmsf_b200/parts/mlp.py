"""Gated feed-forward: (act(h Wg^T) * (h Wu^T)) Wd^T, gate and up merged into one matrix.

Reference: Mlp in core/src/model_executor/models/llama/llama.rs:223-274 with silu_and_mul_kernel
(vllm/kernels/activation_kernels.cu:26-41).  The activation is a parameter here (the reference
fixes SiLU in code although it parses `hidden_act`).

A second form, `clamped_swiglu`, clamps both factors first: g = min(gate, limit), u = clamp(up, -limit, limit),
product g * sigmoid(alpha * g) * (u + 1); `limit` and `alpha` are parameters.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import FeedForward, NormAfter, Prenormed, StepContext, WeightSpec, register_part
from . import linear
from .linear import matmul_tn, matmul_tn_residual


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True
    takes_prenormed = True
    fuses_norm = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False,
                 limit: Optional[float] = None, alpha: float = 1.702):
        if activation not in kernels.ACT_CODES and activation != "clamped_swiglu":
            raise ValueError(f"activation {activation!r} is not supported (known: clamped_swiglu, "
                             f"{', '.join(sorted(kernels.ACT_CODES))})")
        if activation == "clamped_swiglu" and not (limit is not None and limit > 0):
            raise ValueError("the clamped activation needs a positive limit")
        self.hidden_size, self.intermediate_size, self.activation = int(hidden_size), int(intermediate_size), activation
        self.limit, self.alpha = (float(limit) if limit is not None else None), float(alpha)
        self.has_bias = bool(bias)
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None
        self.gate_up_bias: Optional[torch.Tensor] = None
        self.down_bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {"gate_up": WeightSpec([(self.intermediate_size, self.hidden_size)] * 2),
                 "down": WeightSpec([(self.hidden_size, self.intermediate_size)])}
        if self.has_bias:
            specs["gate_up_bias"] = WeightSpec([(self.intermediate_size,)] * 2)
            specs["down_bias"] = WeightSpec([(self.hidden_size,)])
        return specs

    def activation_width(self) -> int:
        return 3 * self.intermediate_size                    # gate, up and their product

    def forward(self, ctx: StepContext, h, then: Optional[NormAfter] = None):
        hx = h.x if isinstance(h, Prenormed) else h
        if linear.USE_SKINNY and self.gate_up_bias is None and self.activation in kernels.ACT_CODES and \
                kernels.gemm_skinny_supported(hx, self.gate_up):
            # a decode step: gate, up and the activation in one pass over the weights
            m = torch.empty((hx.shape[0], self.intermediate_size), dtype=hx.dtype, device=hx.device)
            kernels.gemm_skinny(m, hx, self.gate_up, fuse_act=self.activation,
                                prenorm=(h.sumsq, h.eps, h.width) if isinstance(h, Prenormed) else None)
            return self._down(m, then)
        gu = matmul_tn(h, self.gate_up, bias=self.gate_up_bias)
        m = torch.empty((gu.shape[0], self.intermediate_size), dtype=gu.dtype, device=gu.device)
        if self.activation == "clamped_swiglu":
            kernels.clamped_glu(m, gu, self.limit, self.alpha)
        else:
            kernels.gated_act(m, gu, self.activation)
        return self._down(m, then)

    def _down(self, m: torch.Tensor, then: Optional[NormAfter]):
        if then is not None and self.down_bias is None:
            p = matmul_tn_residual(m, self.down, then)
            if p is not None:
                return p
        return matmul_tn(m, self.down, bias=self.down_bias)


@register_part("feed_forward", "plain_mlp")
class PlainMLP(FeedForward):
    """A feed-forward without a gate: act(h Wu^T) Wd^T.  The one activation so far, `poly_norm`, is a polynomial whose powers
    are each divided by their root mean square over the row of `intermediate_size` values:
        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,   N(x) = x / sqrt(mean(x^2) + eps)
    with the four numbers (a, b, c, e) a weight of the part (`act`).  The sums and factors are float32 (csrc/activation.cu)."""
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, activation: str = "poly_norm"):
        if activation != "poly_norm":
            raise ValueError(f"activation {activation!r} is not supported by the plain feed-forward (known: poly_norm)")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.eps, self.activation = float(eps), activation
        self.up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None
        self.act: Optional[torch.Tensor] = None
        self._coef: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"up": WeightSpec([(self.intermediate_size, self.hidden_size)]),
                "down": WeightSpec([(self.hidden_size, self.intermediate_size)]),
                "act": WeightSpec([(4,)], keep_fp32=True)}

    def prepare(self, dtype, device) -> None:
        self._coef = self.act.float().contiguous()

    def activation_width(self) -> int:
        return 2 * self.intermediate_size

    def forward(self, ctx: StepContext, h):
        z = matmul_tn(h, self.up)
        m = torch.empty_like(z)
        kernels.poly_norm(m, z, self._coef, self.eps)
        return matmul_tn(m, self.down)
