"""Dense gated feed-forward (SwiGLU): residual += W_down (silu(W_gate x) * W_up x).

Reference: src/core/engine.cpp:1010-1024 and src/kernels/swiglu.cu:15-37
(silu(g) = g / (1 + exp(-g))); no biases.  Gate and up are one matrix made at
load, so the input is read once.  On the bfloat16 tensor-core path their rows are
interleaved in blocks of 16 and the activation is computed in the epilogue of
that matrix product, so gate and up never travel through memory; otherwise (the
32-bit path, or sizes the tensor-core kernel refuses) the rows are gate then up
and a separate kernel applies the activation.

The spec may ask for another gated activation ("clamped_swish": g sigmoid(alpha g) (u + 1) on a gate clamped
from above and an up projection clamped on both sides) and other tensor names: on the tensor-core path it runs in the same epilogue; elsewhere the gate/up product has
float32 results and one kernel applies the activation in float32.  :class:`DenseMLP` is the feed-forward
without a gate, down(act(up x)), with act = max(z, 0)^2.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import BuildContext, FeedForward, ParamSpec, register_ffn
from .linear import Linear


class SwiGLU(FeedForward):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.intermediate_size = int(spec.intermediate_size)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.fused = False
        self.gate_up: Linear = None
        self.down: Linear = None
        activation = getattr(spec, "activation", "silu")
        if activation not in ops.GATED_ACTIVATIONS:
            raise ValueError(f"unknown gated activation {activation!r}; known: {sorted(ops.GATED_ACTIVATIONS)}")
        self.act = ops.GATED_ACTIVATIONS[activation]
        self.limit, self.alpha = float(getattr(spec, "act_limit", 0.0)), float(getattr(spec, "act_alpha", 1.0))
        self.gate_name, self.up_name, self.down_name = getattr(spec, "names", None) or (
            "gate_proj.weight", "up_proj.weight", "down_proj.weight")
        self.bias_names = getattr(spec, "bias_names", None)

    def param_specs(self) -> List[ParamSpec]:
        I, H = self.intermediate_size, self.hidden_size
        specs = [ParamSpec(self.gate_name, (I, H)), ParamSpec(self.up_name, (I, H)), ParamSpec(self.down_name, (H, I))]
        if self.bias_names is not None:
            specs += [ParamSpec(n, (size,), role="bias", init="bias_normal") for n, size in zip(self.bias_names, (I, I, H))]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors[self.gate_name], tensors[self.up_name]
        bias = down_bias = None
        if self.bias_names is not None:
            bg, bu, down_bias = (tensors[n] for n in self.bias_names)
            dt = bg.dtype if bg.dtype == bu.dtype else torch.float32
            bias = (bg.to(dt), bu.to(dt))
        self.fused = (g.dtype == torch.bfloat16 and g.is_cuda and self.act in ops.GEMM_TC_GATED_ACTIVATIONS
                      and (bias is None or ops.GEMM_TC_GATED_BIAS) and self.intermediate_size % ops.SWIGLU_BLOCK == 0 and self.hidden_size % 8 == 0)
        if self.fused:
            # the bias of the interleaved rows is interleaved the same way
            b = None if bias is None else ops.interleave_gate_up(bias[0].view(-1, 1), bias[1].view(-1, 1)).view(-1)
            self.gate_up = Linear(ops.interleave_gate_up(g, u), b)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0), None if bias is None else torch.cat(bias))
        self.down = Linear(tensors[self.down_name], down_bias)

    def forward(self, x, residual, batch, accumulate: bool = True) -> None:
        if self.fused:
            a = ops.gemm_tc(x, self.gate_up.weight, self.gate_up.bias, swiglu=True, act=self.act, limit=self.limit,
                            alpha=self.alpha)
        elif self.act == ops.ACT_SILU and self.gate_up.bias is None:
            a = ops.swiglu(self.gate_up(x))
        else:
            a = ops.glu(self.gate_up(x, out_dtype=torch.float32), self.act, self.limit, self.alpha, out_dtype=x.dtype)
        if accumulate:
            self.down.add_to(a, residual)
        elif accumulate is None:
            self.down.write_to(a, residual)
        else:
            self.down(a, out=residual)


class DenseMLP(FeedForward):
    """``down(act(up x))`` without a gate; the activation runs in float32 on the up product's float32 result."""

    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.intermediate_size = int(spec.intermediate_size)
        self.hidden_size = hidden_size
        self.ctx = ctx
        if spec.activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r}; known: {sorted(ops.UNARY_ACTIVATIONS)}")
        self.act = ops.UNARY_ACTIVATIONS[spec.activation]
        self.up_name, self.down_name = spec.names
        self.up: Linear = None
        self.down: Linear = None

    def param_specs(self) -> List[ParamSpec]:
        I, H = self.intermediate_size, self.hidden_size
        return [ParamSpec(self.up_name, (I, H)), ParamSpec(self.down_name, (H, I))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.up = Linear(tensors[self.up_name])
        self.down = Linear(tensors[self.down_name])

    def forward(self, x, residual, batch, accumulate: bool = True) -> None:
        w = self.up.weight
        if w.dtype == torch.bfloat16 and ops.gemm_tc_supports(x, w):   # the activation in the product's epilogue
            a = ops.gemm_tc(x, w, act=self.act)
        else:
            a = ops.unary_act(self.up(x, out_dtype=torch.float32), self.act, out_dtype=x.dtype)
        if accumulate:
            self.down.add_to(a, residual)
        elif accumulate is None:
            self.down.write_to(a, residual)
        else:
            self.down(a, out=residual)


register_ffn("swiglu", SwiGLU)
register_ffn("dense_mlp", DenseMLP)
