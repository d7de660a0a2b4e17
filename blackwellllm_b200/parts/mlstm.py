"""Matrix memory with exponential gates (mLSTM): a recurrent mixer whose memory is a [key_dim, value_dim] matrix per head.

    q = W_q x / sqrt(key_dim)     k = W_k x     v = W_v x
    i = cap tanh((w_i x + b_i) / cap)                   log input gate, one number per head
    f = log_sigmoid(cap tanh((w_f x + b_f) / cap))      log forget gate, one number per head
    m' = max(f + m, i)                                  running maximum, m starts at 0
    S <- exp(f + m - m') S + exp(i - m') k v^T          n <- exp(f + m - m') n + exp(i - m') k
    o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
    y = W_o (concat_heads(o / rms(o)) * gain * sigmoid(W_g x))          gain: one entry per channel of all heads

The state (S and n as one [key_dim, value_dim + 1] matrix per head whose last column is n, its rows padded to a multiple
of four floats, and m) is float32, lives in the
request's slots of the cache manager's fixed-size state (zeroed when the slot is handed out, which is where S, n and m
start) and is carried from step to step.  q, k, v, the output gate and the two gates' projections are one matrix made at
load; their results are float32.  Three kernels follow: the gates (``ops.mlstm_gates``: cap, logarithm, the chain of
maxima, the three exponentials), the recurrence (``ops.gla_scan`` with one decay per head, the keys times exp(i - m') as
they are read, and a value column of ones, which makes n a column of S and n . q a column of the output), and the output
(``ops.mlstm_out``: the division, the head norm, gain and gate).  Everything but the projections is float32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import BuildContext, FixedStateRequest, Mixer, ParamSpec, register_mixer
from .linear import Linear

_DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                  "o": "o_proj.weight", "norm": "norm.weight", "i": "igate.weight", "i_bias": "igate.bias",
                  "f": "fgate.weight", "f_bias": "fgate.bias"}

DENOMINATOR_EPS = 1e-6   # added to max(|n . q|, exp(-m)) before the division


class MatrixLSTM(Mixer):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.heads, self.dk, self.dv = int(spec.num_heads), int(spec.key_dim), int(spec.value_dim)
        self.cap, self.eps = float(spec.gate_cap), float(spec.norm_eps)
        if not self.cap > 0:
            raise ValueError(f"gate_cap must be > 0, got {self.cap}")
        if self.dk > ops.GLA_MAX_KEY_DIM:
            raise ops.KernelError(f"matrix memory: key size {self.dk} exceeds the scan's {ops.GLA_MAX_KEY_DIM}")
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(dict(getattr(spec, "names", ()) or ()))
        self.proj: Linear = None
        self.o: Linear = None
        self.gain = self.bias_i = self.bias_f = None

    def cache_request(self):
        # [S | n] per head (rows padded to a multiple of four floats: the scan moves them in 16-byte pieces), and the
        # running maximum m per head
        return (FixedStateRequest((self.heads, self.dk, -(-(self.dv + 1) // 4) * 4), torch.float32),
                FixedStateRequest((self.heads,), torch.float32))

    def param_specs(self) -> List[ParamSpec]:
        H, K, V, n = self.hidden_size, self.heads * self.dk, self.heads * self.dv, self.names
        return [ParamSpec(n["q"], (K, H)), ParamSpec(n["k"], (K, H)), ParamSpec(n["v"], (V, H)),
                ParamSpec(n["g"], (V, H)), ParamSpec(n["o"], (H, V)),
                ParamSpec(n["norm"], (V,), role="gain", init="ones"),
                ParamSpec(n["i"], (self.heads, H)), ParamSpec(n["i_bias"], (self.heads,), role="bias", init="bias_normal"),
                ParamSpec(n["f"], (self.heads, H)), ParamSpec(n["f_bias"], (self.heads,), role="bias", init="bias_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.proj = Linear(torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]],
                                      tensors[n["i"]], tensors[n["f"]]], dim=0))
        self.o = Linear(tensors[n["o"]])
        self.gain = tensors[n["norm"]].float().contiguous()
        self.bias_i = tensors[n["i_bias"]].float().contiguous()
        self.bias_f = tensors[n["f_bias"]].float().contiguous()

    def forward(self, x, residual, batch, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        if not owns_cache:
            raise ops.KernelError("matrix memory: a run cannot read another run's state")
        memory, maxima = cache
        K, V = self.heads * self.dk, self.heads * self.dv
        proj = self.proj(x, out_dtype=torch.float32)          # [T, q | k | v | g | i | f]
        i_off = 2 * K + 2 * V
        a, b, e = ops.mlstm_gates(proj, i_off, i_off + self.heads, self.bias_i, self.bias_f, self.cap, batch, maxima.state,
                                  self.heads)
        o = ops.gla_scan(proj, 0, K, 2 * K, a, batch, memory.state, self.heads, self.dk, self.dv + 1, self.dk ** -0.5,
                         k_scale=b, scalar_decay=True, ones_col=True)
        y = ops.mlstm_out(o, e, proj, 2 * K + V, self.gain, self.heads, self.dv, self.eps, self.ctx.dtype, DENOMINATOR_EPS)
        if accumulate:
            self.o.add_to(y, residual)
        elif accumulate is None:
            self.o.write_to(y, residual)
        else:
            self.o(y, out=residual)


register_mixer("matrix_lstm", MatrixLSTM)
