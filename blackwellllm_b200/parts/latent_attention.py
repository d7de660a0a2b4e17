"""Latent attention: the keys and values of all heads are made from one small vector per token.

    q_h = W_q,h x                      laid out per head as [head_dim plain channels, rot_dim rotated channels]
    [c_raw, k_rot] = W_dkv x           kv_rank + rot_dim rows;  c = c_raw / rms(c_raw) * gain  (the latent)
    k_h = [W_uk,h c, rot(k_rot)]       v_h = W_uv,h c
    score_h(i, j) = (q_plain,h(i) . W_uk,h c(j) + rot(q_rot,h(i)) . rot(k_rot(j))) * scale
    y = W_o concat_h(sum_j p_h(i, j) v_h(j))          p: softmax over the window, with an optional sink per head

Only c and the rotated k_rot are cached: one row of kv_rank + rot_dim channels per token, shared by all heads.  The
heads' matrices are moved to the other side of the two sums ("absorbed"):

    q_plain,h . (W_uk,h c) = (W_uk,h^T q_plain,h) . c            sum_j p v_h(j) = W_uv,h (sum_j p c(j))

so the attention proper is a grouped-query attention with ONE key/value head whose key row is [c, k_rot] and whose
value row is c, a part of the same row: the framework's paged attention kernels run it as they are (sink, window), on a
cache with a single plane (``PagedKVRequest.single_plane``).  Around them: one product for q and the latent's
projection (float32 results); ``ops.latent_prep`` (norm of the latent, rotation of the shared key part and the queries'
rotated parts, append); ``ops.headwise_linear`` with W_uk,h^T on the queries' plain parts and with W_uv,h on the
attention's output; the output projection into the stream.  The rotation is the rotary encoding part's own table
(YaRN frequencies and magnitude included); the norm, the angles, the scores and the softmax are float32.

Options of the spec: ``q_rank`` (the queries come through a latent of their own: the first product also makes
``W_dq x``, an RMS norm with a gain follows, then ``W_uq`` makes the queries); ``output_gate`` (the concatenated heads'
outputs times ``sigmoid(W_g x)``, W_g's rows riding in the first product; the gate is applied in the per-head value
product's epilogue); a rotary encoding that pairs channel 2j with channel 2j + 1.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import BuildContext, Mixer, PagedKVRequest, ParamSpec, build_position, register_mixer
from .linear import Linear

_DEFAULT_NAMES = {"q": "q_proj.weight", "dkv": "kv_a_proj.weight", "dkv_norm": "kv_a_norm.weight", "uk": "k_b_proj.weight",
                  "uv": "v_b_proj.weight", "o": "o_proj.weight", "sink": "sinks", "dq": "q_a_proj.weight",
                  "dq_norm": "q_a_norm.weight", "uq": "q_b_proj.weight", "g": "g_proj.weight"}


class LatentAttention(Mixer):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.H, self.d, self.dr = int(spec.num_heads), int(spec.head_dim), int(spec.rot_dim)
        self.dv, self.rank = int(spec.v_head_dim), int(spec.kv_rank)
        self.eps = float(spec.norm_eps)
        self.scale = float(spec.softmax_scale)
        self.window = spec.window
        self.has_sink = bool(spec.sink)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(dict(getattr(spec, "names", ()) or ()))
        if self.dr <= 0 or self.dr % 2:
            raise ValueError(f"rot_dim {self.dr} must be even and positive")
        step = 16 if ctx.dtype == torch.bfloat16 else 1
        self.dpad = -(-(self.rank + self.dr) // step) * step      # the cached row, in steps the attention kernels take
        ops.check_attention_supported(ctx.dtype, self.dpad)   # (all heads share the one key/value head: beyond what a
                                                               # tile of the tensor-core kernels stacks, the CUDA-core kernel runs)
        # heads per attention call: all of them, or in bfloat16 the largest divisor of their number that the tensor-core
        # kernels stack on one key/value head (a number of heads without such a divisor of at least 4 runs in one call
        # on the CUDA-core kernel)
        self.heads_per_call = self.H
        if ctx.dtype == torch.bfloat16 and self.H > ops.MAX_GROUP_BF16 and self.dpad <= 256:
            n = max(k for k in range(1, ops.MAX_GROUP_BF16 + 1) if self.H % k == 0)
            if n >= 4:
                self.heads_per_call = n
        self.position = build_position(spec.position, self.dr, ctx)
        if getattr(self.position, "rotary_dim", None) != self.dr:
            raise ValueError("latent attention turns all rot_dim channels")
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        qr = getattr(spec, "q_rank", None)
        self.q_rank = int(qr) if qr else None
        self.gated = bool(getattr(spec, "output_gate", False))
        self.uq: Linear = None
        self.q_gain = None
        self.proj: Linear = None
        self.uk_t = self.uv = self.c_gain = self.sink = None
        self.o: Linear = None

    def cache_request(self):
        return PagedKVRequest(1, self.dpad, self.window, 0, single_plane=True)

    def param_specs(self) -> List[ParamSpec]:
        W, n = self.hidden_size, self.names
        if self.q_rank is None:
            specs = [ParamSpec(n["q"], (self.H * (self.d + self.dr), W))]
        else:
            specs = [ParamSpec(n["dq"], (self.q_rank, W)), ParamSpec(n["dq_norm"], (self.q_rank,), role="gain", init="ones"),
                     ParamSpec(n["uq"], (self.H * (self.d + self.dr), self.q_rank))]
        if self.gated:
            specs.append(ParamSpec(n["g"], (self.H * self.dv, W)))
        specs += [ParamSpec(n["dkv"], (self.rank + self.dr, W)),
                 ParamSpec(n["dkv_norm"], (self.rank,), role="gain", init="ones"),
                 ParamSpec(n["uk"], (self.H * self.d, self.rank)), ParamSpec(n["uv"], (self.H * self.dv, self.rank)),
                 ParamSpec(n["o"], (W, self.H * self.dv))]
        if self.has_sink:
            specs.append(ParamSpec(n["sink"], (self.H,), role="bias", init="bias_normal"))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        # one product reads the input: [queries or their latent | the keys' and values' latent and rotated part | gate]
        first = tensors[n["q"]] if self.q_rank is None else tensors[n["dq"]]
        self.q_cols = first.shape[0]
        self.proj = Linear(torch.cat([first, tensors[n["dkv"]]] + ([tensors[n["g"]]] if self.gated else []), dim=0))
        if self.q_rank is not None:
            self.q_gain = tensors[n["dq_norm"]].contiguous()
            self.uq = Linear(tensors[n["uq"]])
        self.c_gain = tensors[n["dkv_norm"]].float().contiguous()
        # per head [outputs, inputs]: W_uk,h^T takes head_dim inputs to kv_rank outputs, W_uv,h kv_rank inputs to v_head_dim
        self.uk_t = tensors[n["uk"]].view(self.H, self.d, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors[n["uv"]].view(self.H, self.dv, self.rank).contiguous()
        self.o = Linear(tensors[n["o"]])
        self.sink = tensors[n["sink"]].float().contiguous() if self.has_sink else None

    def forward(self, x, residual, batch, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        H, d, dr, rank = self.H, self.d, self.dr, self.rank
        proj = self.proj(x, out_dtype=torch.float32)       # [T, H * (d + dr) or q_rank | rank + dr | gate]
        kv_off = self.q_cols
        if self.q_rank is None:
            qs = proj
        else:   # the queries' latent, normed in float32, then the queries themselves (float32 results)
            cq = ops.rmsnorm(proj[:, :self.q_rank], self.q_gain, self.eps, self.ctx.dtype)
            qs = self.uq(cq, out_dtype=torch.float32)
        y = torch.empty((x.shape[0], H * self.dv), dtype=x.dtype, device=x.device)
        table, bt = self.position.table(batch), batch.block_tables[cache.group]
        # all heads share the one cached row; the tensor-core kernels stack up to ops.MAX_GROUP_BF16 query heads on a
        # key/value head, so more heads than that run as several groups of heads over the same rows
        n = self.heads_per_call
        for h0 in range(0, H, n):
            q = ops.latent_prep(proj, h0 * (d + dr), kv_off, batch, bt, table, self.c_gain, self.eps, cache.k_pages,
                                n, d, dr, rank, append=owns_cache and h0 == 0, q_src=qs, interleaved=self.interleaved)
            ops.headwise_linear(qs, h0 * (d + dr), d + dr, self.uk_t[h0:h0 + n], q, 0, self.dpad)
            o = ops.paged_attention(q, cache.k_pages, cache.v_pages, batch, bt, n, self.window, self.scale, None,
                                    None if self.sink is None else self.sink[h0:h0 + n], None)
            gate = None
            if self.gated:      # the gate's sigmoid multiplies the per-head value product's result as it is written
                g_off = kv_off + rank + dr + h0 * self.dv
                gate = proj[:, g_off:g_off + n * self.dv]
            ops.headwise_linear(o, 0, self.dpad, self.uv[h0:h0 + n], y, h0 * self.dv, self.dv, gate=gate)
        if accumulate:
            self.o.add_to(y, residual)
        elif accumulate is None:
            self.o.write_to(y, residual)
        else:
            self.o(y, out=residual)


register_mixer("latent_attention", LatentAttention)
