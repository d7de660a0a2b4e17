"""Grouped-query softmax attention over paged keys and values.

In the reference's order (src/core/engine.cpp:968-990): q, k, v = W x (+ bias, added
once after the dot product and before the rotation, bf16_linear_bias.cu:44-50);
rotation of q and k; append of k and v to the cache; causal attention with
scale head_dim**-0.5 applied to the scores (paged_flash_attention.cu:142-144,446);
output projection added to the residual stream (bf16_linear_residual.cu:42-46).

Here the three projections are one matrix (rows q, k, v) made at load, its result
stays float32 until the rotation, and the residual sum is float32.

Options of the spec beyond that: ``chunk`` (a query sees no key before the start of its own block of
positions), ``v_head_dim`` (value size of a head other than its key size: the cache and the attention
kernels run at the larger of the two, rounded up to what the kernels take, the rest zeros; the output
projection's weight gets zero columns there), ``qk_norm_eps`` (an RMS norm over the whole query and the
whole key projection before the rotation), an explicit ``softmax_scale``, and ``names`` for checkpoints
that call the tensors otherwise.  With any of the first three, or an encoding that has no fused
projection, the route is: projection (float32 out) -> one kernel that norms, rotates and appends
(``PositionEncoding.norm_rotate_append``) -> attention -> output projection.

Further options, each of which takes that route too: ``qk_norm = "head"`` (every query and key head normed by
itself, one gain vector of the head's size shared by the heads), ``q_temperature`` (the queries of position p
times 1 + coef log(1 + n), n the whole periods of ``every`` positions in p + 1), ``sink`` (one learned number per query head whose exponential
joins the softmax's denominator: the kernels add it when they normalise a row), ``output_gate`` (the heads'
outputs times sigmoid(W_g x) before the output projection; W_g's rows ride in the q/k/v product and the
attention kernels apply the sigmoid as they write a row), and
``shares_kv`` (no key and value tensors: the run reads the cache of the schedule entry it names, which the
other layer filled earlier in the same step, with its own queries).

And: ``gate_per_head`` (the output gate has one number per head), ``v_norm_eps`` (every value head divided by its
root mean square, without a gain, before it is cached: done by the kernel that appends), ``distance_bias`` (two
learned numbers per query head, r1 and r2: r1 ln(1 + r2 (i - j)) is taken off the score of query i and key j inside
the attention kernels) and ``keep_first`` (with a window, the first so many keys of a sequence stay visible, and
their pages stay with the request).

And: ``score_softcap`` (the scaled score s becomes cap tanh(s / cap)), ``distance_table_far`` (a learned bias per
distance and query head, tensor "rel" [rows, heads], added to the capped score; the rows' distances are
``ops.distance_bucket_table``; at load the table is spread out to one float32 entry per distance and head, which is
what the kernels read), ``fixed_sink`` (a sink whose score is a constant of the design: the same term in the
denominator as a learned sink) and ``value_mix`` (the values of every layer that has it, but the first such layer of
the model, are cached as (1 - lam) v + lam v_first, v_first the first such layer's values of the same token: that
layer leaves its values of the step in ``batch.extras``, the others read them in the kernel that appends).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import (BuildContext, Mixer, PagedKVRequest, ParamSpec, build_position, register_mixer)
from .linear import Linear


_DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                  "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
                  "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sinks", "g": "g_proj.weight",
                  "r1": "r1", "r2": "r2", "rel": "rel", "vmix": "vmix"}


class GQAAttention(Mixer):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.nh, self.nkv, self.hd = int(spec.num_heads), int(spec.num_kv_heads), int(spec.head_dim)
        if self.nh % self.nkv:
            raise ValueError(f"num_heads {self.nh} is not a multiple of num_kv_heads {self.nkv}")
        self.hidden_size = hidden_size
        self.qkv_bias = bool(spec.qkv_bias)
        self.window = spec.window
        self.chunk = getattr(spec, "chunk", None)
        self.dv = int(getattr(spec, "v_head_dim", None) or self.hd)
        self.qk_norm_eps = getattr(spec, "qk_norm_eps", None)
        self.norm_per_head = getattr(spec, "qk_norm", "whole") == "head"
        if getattr(spec, "qk_norm", "whole") not in ("whole", "head"):
            raise ValueError(f"qk_norm must be 'whole' or 'head', got {spec.qk_norm!r}")
        qt = getattr(spec, "q_temperature", None)
        self.q_temp = (float(qt[0]), float(qt[1])) if qt is not None and float(qt[0]) != 0.0 else None
        if self.q_temp is not None and not self.q_temp[1] > 0:
            raise ValueError("q_temperature needs every > 0")
        self.has_sink = bool(getattr(spec, "sink", False))
        self.gated = bool(getattr(spec, "output_gate", False))
        self.shares_kv = bool(getattr(spec, "shares_kv", False))
        self.gate_per_head = bool(getattr(spec, "gate_per_head", False))
        self.v_eps = getattr(spec, "v_norm_eps", None)
        self.has_dist = bool(getattr(spec, "distance_bias", False))
        self.keep_first = int(getattr(spec, "keep_first", 0) or 0)
        if self.keep_first < 0:
            raise ValueError("keep_first must not be negative")
        if self.gate_per_head and not self.gated:
            raise ValueError("gate_per_head goes with output_gate")
        if self.v_eps is not None and self.shares_kv:
            raise ValueError("a mixer that shares another run's keys and values norms no values")
        self.dist = None
        cap = getattr(spec, "score_softcap", None)
        self.softcap = float(cap) if cap else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError("score_softcap must be > 0")
        far = getattr(spec, "distance_table_far", None)
        self.rel_far = float(far) if far is not None else None
        self.rel_rows = getattr(spec, "distance_table_rows", None)
        self.rel = None
        fs = getattr(spec, "fixed_sink", None)
        self.fixed_sink = float(fs) if fs is not None else None
        if self.fixed_sink is not None and self.has_sink:
            raise ValueError("a mixer has a learned sink or a fixed one, not both")
        self.value_mix = getattr(spec, "value_mix", None)
        self.lam = None
        if (self.softcap is not None or self.rel_far is not None) and self.has_dist:
            raise ValueError("a soft cap or a table of biases by distance does not go with the logarithmic distance bias")
        if self.value_mix is not None and self.shares_kv:
            raise ValueError("a mixer that shares another run's keys and values mixes no values")
        self.names = dict(_DEFAULT_NAMES)
        self._given_names = dict(getattr(spec, "names", ()) or ())
        self.names.update(self._given_names)
        # head size of the cache and the attention kernels: both sizes fit, in steps the kernels take
        step = 16 if ctx.dtype == torch.bfloat16 else 1
        self.dpad = -(-max(self.hd, self.dv) // step) * step
        self.general = (self.qk_norm_eps is not None or self.dv != self.hd or self.dpad != self.hd or self.norm_per_head
                        or self.q_temp is not None or self.gated or self.shares_kv or self.v_eps is not None
                        or self.value_mix is not None)
        # the kernel that norms per head also takes rows with a gate's columns behind q, k, v, or without k and v,
        # and norms the values
        self.per_head_route = (self.norm_per_head or self.q_temp is not None or self.shares_kv
                               or self.v_eps is not None or self.gate_per_head or self.value_mix is not None)
        if self.shares_kv and self.qkv_bias:
            raise ValueError("a mixer that shares another run's keys and values has no key and value biases")
        if self.per_head_route and self.qk_norm_eps is not None and not self.norm_per_head:
            raise ValueError("a query temperature or shared keys and values go with the per-head norm (or none)")
        self.q_gain = self.k_gain = self.sink = None
        self.gate: Linear = None
        self.g_off = 0
        self.scale = float(spec.softmax_scale) if spec.softmax_scale is not None else self.hd ** -0.5
        self.ctx = ctx
        self.position = build_position(spec.position, self.hd, ctx)
        # (the general route hands ops.paged_attention finished queries: beyond the query heads per kv head that the
        # tensor-core kernels stack, it takes the CUDA-core kernel; the fused route goes to the tensor-core kernels only)
        ops.check_attention_supported(ctx.dtype, self.dpad, 1 if self.general else self.nh // self.nkv)
        self.qkv: Linear = None
        self.project = None
        self.o: Linear = None

    def cache_request(self):
        # (a run with ``shares_kv`` is never asked: its schedule entry names the run whose cache it reads)
        return PagedKVRequest(self.nkv, self.dpad, self.window, self.keep_first if self.window else 0)

    def param_specs(self) -> List[ParamSpec]:
        H, q, k, v = self.hidden_size, self.nh * self.hd, self.nkv * self.hd, self.nkv * self.dv
        n = self.names
        specs = [ParamSpec(n["q"], (q, H))]
        if not self.shares_kv:
            specs += [ParamSpec(n["k"], (k, H)), ParamSpec(n["v"], (v, H))]
        specs.append(ParamSpec(n["o"], (H, self.nh * self.dv)))
        if self.qkv_bias:
            specs += [ParamSpec(n["q_bias"], (q,), role="bias", init="bias_normal"),
                      ParamSpec(n["k_bias"], (k,), role="bias", init="bias_normal"),
                      ParamSpec(n["v_bias"], (v,), role="bias", init="bias_normal")]
        if self.qk_norm_eps is not None:
            specs.append(ParamSpec(n["q_norm"], (self.hd if self.norm_per_head else q,), role="gain", init="ones"))
            if not self.shares_kv:
                specs.append(ParamSpec(n["k_norm"], (self.hd if self.norm_per_head else k,), role="gain", init="ones"))
        if self.has_sink:
            specs.append(ParamSpec(n["sink"], (self.nh,), role="bias", init="bias_normal"))
        if self.gated:
            specs.append(ParamSpec(n["g"], (self.nh if self.gate_per_head else self.nh * self.dv, H)))
        if self.has_dist:
            specs += [ParamSpec(n["r1"], (self.nh,), role="bias", init="bias_normal"),
                      ParamSpec(n["r2"], (self.nh,), role="bias", init="ones")]
        if self.rel_far is not None:
            specs.append(ParamSpec(n["rel"], (-1 if self.rel_rows is None else int(self.rel_rows), self.nh), role="bias",
                                   init="bias_normal"))
        if self.value_mix is not None:
            specs.append(ParamSpec(n["vmix"], (), role="bias", init="bias_normal"))
        elif "vmix" in self._given_names:
            # a design that has the mixing number may store it in layers that do not mix: taken and not used
            specs.append(ParamSpec(n["vmix"], (), role="bias", init="bias_normal", optional=True))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        parts = [tensors[n["q"]]] + ([] if self.shares_kv else [tensors[n["k"]], tensors[n["v"]]])
        if self.has_sink:
            self.sink = tensors[n["sink"]].float().contiguous()
        elif self.fixed_sink is not None:
            self.sink = torch.full((self.nh,), self.fixed_sink, dtype=torch.float32, device=tensors[n["q"]].device)
        if self.has_dist:
            self.dist = torch.stack([tensors[n["r1"]].float(), tensors[n["r2"]].float()]).contiguous()
        if self.rel_far is not None:
            # one entry per (head, distance) up to the first distance that takes the table's last row
            table = tensors[n["rel"]].float()
            rows_of = ops.distance_bucket_table(int(table.shape[0]), self.rel_far).to(table.device)
            self.rel = table[rows_of].t().contiguous()
        if self.value_mix is not None:
            self.lam = tensors[n["vmix"]].float().reshape(1).contiguous()
        if self.gated:
            if self.per_head_route or self.qk_norm_eps is None:
                # the gate's rows ride in the q/k/v product; the kernel that follows leaves its columns alone
                self.g_off = sum(p.shape[0] for p in parts)
                parts.append(tensors[n["g"]])
            else:
                self.gate = Linear(tensors[n["g"]])
        w = torch.cat(parts, dim=0)
        b = None
        if self.qkv_bias:
            bs = [tensors[n["q_bias"]], tensors[n["k_bias"]], tensors[n["v_bias"]]]
            dt = bs[0].dtype if all(t.dtype == bs[0].dtype for t in bs) else torch.float32
            b = torch.cat([t.to(dt) for t in bs], dim=0)
            if w.shape[0] > b.numel():    # the gate's rows ride behind q, k, v and have no bias
                b = torch.cat([b, torch.zeros(w.shape[0] - b.numel(), dtype=dt, device=b.device)])
        wo = tensors[n["o"]]
        if self.qk_norm_eps is not None:
            self.q_gain = tensors[n["q_norm"]].float().contiguous()
            self.k_gain = None if self.shares_kv else tensors[n["k_norm"]].float().contiguous()
        if self.general:
            if self.dpad != self.dv:   # the attention's output has dpad channels a head; those beyond dv are zeros
                wo = torch.nn.functional.pad(wo.view(wo.shape[0], self.nh, self.dv), (0, self.dpad - self.dv)) \
                    .reshape(wo.shape[0], self.nh * self.dpad)
            self.project = None
        else:
            # an encoding that runs inside the projection takes the weight over; else project, then encode
            self.project = self.position.fuse_projection(w, b, self.nh, self.nkv, self.hd)
        self.qkv = Linear(w, b) if self.project is None else None
        self.o = Linear(wo)

    def forward(self, x, residual, batch, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        if self.project is not None:
            q = self.project(x, batch, cache, owns_cache)
        else:
            qkv = self.qkv(x, out_dtype=torch.float32)
            if self.per_head_route or (self.gated and self.gate is None):
                v_mix = None
                if self.value_mix is not None:
                    # this step's values of the model's first layer that mixes values: it leaves them, the others read them
                    v_off = (self.nh + self.nkv) * self.hd
                    mine = qkv[:, v_off:v_off + self.nkv * self.dv]
                    first = batch.extras.get("value_mix_first")
                    if first is None:
                        batch.extras["value_mix_first"] = mine
                    elif first.shape != mine.shape:
                        raise ops.KernelError("value mixing: the layers' values differ in size")
                    else:
                        v_mix = (first, self.lam)
                q = self.position.norm_rotate_append(qkv, batch, cache, self.nh, self.nkv, self.hd, self.dv, self.q_gain,
                                                     self.k_gain, float(self.qk_norm_eps or 0.0), append=owns_cache,
                                                     per_head=True, q_temp=self.q_temp, has_kv=not self.shares_kv,
                                                     v_eps=float(self.v_eps or 0.0), v_mix=v_mix)
            elif self.general:
                q = self.position.norm_rotate_append(qkv, batch, cache, self.nh, self.nkv, self.hd, self.dv, self.q_gain,
                                                     self.k_gain, float(self.qk_norm_eps or 0.0), append=owns_cache)
            else:
                q = self.position.rotate_append(qkv, batch, cache, self.nh, self.nkv, self.hd, append=owns_cache)
        gate = None
        if self.gated:   # the attention kernels multiply by the gate's sigmoid as they write a row
            if self.gate_per_head:
                gate = (qkv[:, self.g_off:self.g_off + self.nh], self.dv, "head")
            else:
                g = self.gate(x, out_dtype=torch.float32) if self.gate is not None \
                    else qkv[:, self.g_off:self.g_off + self.nh * self.dv]
                gate = (g, self.dv)
        o = ops.paged_attention(q, cache.k_pages, cache.v_pages, batch, batch.block_tables[cache.group],
                                self.nh, self.window, self.scale, self.chunk, self.sink, gate, self.dist,
                                self.keep_first if self.window else 0, self.softcap, self.rel)
        if accumulate:
            self.o.add_to(o, residual)
        elif accumulate is None:
            self.o.write_to(o, residual)
        else:
            self.o(o, out=residual)


register_mixer("gqa_attention", GQAAttention)
