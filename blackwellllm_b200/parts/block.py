"""Arrangements of norms, mixer and feed-forward in a layer.

``prenorm`` (src/core/engine.cpp:946-1024): the norm stands before each sublayer
and reads the residual stream without changing it; each sublayer adds its output
to the residual stream, which stays float32.  A sublayer's last product may leave its sum to the
next reader of the stream (``Linear.add_to``): the next norm, which adds it while it normalises.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import (Block, BuildContext, ParamSpec, build_ffn, build_mixer, build_norm,
                   register_block)


class PreNormBlock(Block):
    def __init__(self, layer_spec, hidden_size: int, ctx: BuildContext):
        self.spec = layer_spec
        self.mixer_norm = build_norm(layer_spec.mixer_norm, hidden_size, ctx)
        self.mixer = build_mixer(layer_spec.mixer, hidden_size, ctx)
        self.ffn = None
        self.ffn_norm = None
        if layer_spec.ffn is not None:
            self.ffn_norm = build_norm(layer_spec.ffn_norm, hidden_size, ctx)
            self.ffn = build_ffn(layer_spec.ffn, hidden_size, ctx)

    def _children(self):
        s = self.spec
        kids = [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer)]
        if self.ffn is not None:
            kids += [(s.ffn_norm_prefix, self.ffn_norm), (s.ffn_prefix, self.ffn)]
        return kids

    def param_specs(self) -> List[ParamSpec]:
        out = []
        for prefix, part in self._children():
            for p in part.param_specs():
                out.append(ParamSpec(prefix + p.name, p.shape, p.role, p.init, p.optional))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._children():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    takes_pending = True

    @staticmethod
    def _normed(norm, residual):
        # a sublayer may have left the sum of its last product to the stream's next reader: a norm
        # that adds it while it normalises, or else a kernel of its own here
        if not norm.adds_pending:
            ops.resolve_pending()
        return norm.forward(residual)

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        x = self._normed(self.mixer_norm, residual)
        self.mixer.forward(x, residual, batch, cache, owns_cache)
        if self.ffn is not None:
            x = self._normed(self.ffn_norm, residual)
            self.ffn.forward(x, residual, batch)


class SandwichBlock(PreNormBlock):
    """A norm before AND after each sublayer: ``x += post(mixer(pre(x)))``, ``x += post(ffn(pre(x)))``.  The
    sublayer writes its output to a float32 buffer of its own (``accumulate=False``); the second norm reads
    it and adds the result to the stream in one kernel.  A feed-forward with ``forward_post`` does the
    second norm inside its own last kernel."""
    takes_pending = False

    def __init__(self, layer_spec, hidden_size: int, ctx: BuildContext):
        super().__init__(layer_spec, hidden_size, ctx)
        if layer_spec.mixer_post_norm is None or (layer_spec.ffn is not None and layer_spec.ffn_post_norm is None):
            raise ValueError("the sandwich arrangement needs a norm after each sublayer")
        self.mixer_post = build_norm(layer_spec.mixer_post_norm, hidden_size, ctx)
        self.ffn_post = build_norm(layer_spec.ffn_post_norm, hidden_size, ctx) if self.ffn is not None else None
        for norm in (self.mixer_post, self.ffn_post):
            if norm is not None and not hasattr(norm, "add_to"):
                raise ValueError(f"{type(norm).__name__} cannot follow a sublayer (it has no add_to)")

    def _children(self):
        s = self.spec
        kids = super()._children() + [(s.mixer_post_norm_prefix, self.mixer_post)]
        if self.ffn is not None:
            kids.append((s.ffn_post_norm_prefix, self.ffn_post))
        return kids

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        x = self._normed(self.mixer_norm, residual)
        branch = torch.empty_like(residual)
        self.mixer.forward(x, branch, batch, cache, owns_cache, accumulate=False)
        if self.ffn is None:
            self.mixer_post.add_to(branch, residual)
        else:
            # the norm after the mixer and the norm before the feed-forward read the same row: one kernel if they can
            if hasattr(self.mixer_post, "add_to_then"):
                x = self.mixer_post.add_to_then(branch, residual, self.ffn_norm)
            else:
                self.mixer_post.add_to(branch, residual)
                x = self.ffn_norm.forward(residual)
            if hasattr(self.ffn, "forward_post"):
                self.ffn.forward_post(x, residual, batch, self.ffn_post)
            else:
                self.ffn.forward(x, branch, batch, accumulate=False)
                self.ffn_post.add_to(branch, residual)


register_block("prenorm", PreNormBlock)
register_block("sandwich", SandwichBlock)


class HyperBlock(PreNormBlock):
    """Pre-norm sublayers over a stream that is kept as several copies (hyper-connections): sublayer q reads
    ``u = sum_s in_q[s] x_s`` through its norm and writes ``x_t <- sum_s mix_q[s, t] x_s + out_q[t] y`` (all
    copies at once from the old ones).  ``residual`` is float32 [T, streams * hidden].  The write of one
    sublayer and the read and norm of the next are one kernel (``ops.hc_step``); the write of the block's
    last sublayer is left to whoever reads the stream next (the next block, the model's last norm):
    ``batch.extras["hc_write"]`` holds (y, mix, out) until then, and :func:`flush_hyper_write` makes it."""

    def __init__(self, layer_spec, hidden_size: int, ctx: BuildContext):
        super().__init__(layer_spec, hidden_size, ctx)
        hc = layer_spec.hyper
        if hc is None:
            raise ValueError("the hyper arrangement needs the layer's hyper-connection description")
        self.S = int(hc.streams)
        if not 1 <= self.S <= ops.HC_MAX_STREAMS:
            raise ValueError(f"{self.S} copies of the stream are not supported (1..{ops.HC_MAX_STREAMS})")
        self.hc_prefixes = (hc.mixer_prefix, hc.ffn_prefix)
        self.hc_optional = bool(hc.optional_tensors)
        self.hidden_size = hidden_size
        self.ctx = ctx
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "gain_f32"):
                raise ValueError(f"{type(norm).__name__} cannot stand before a sublayer of a hyper block (it has no gain_f32)")
        self.hc = []   # per sublayer: (in [S], out [S], mix [S, S]) float32

    def param_specs(self) -> List[ParamSpec]:
        out = super().param_specs()
        S = self.S
        for prefix in self.hc_prefixes[:1 if self.ffn is None else 2]:
            out += [ParamSpec(prefix + "in", (S,), role="bias", init="ones", optional=self.hc_optional),
                    ParamSpec(prefix + "out", (S,), role="bias", init="ones", optional=self.hc_optional),
                    ParamSpec(prefix + "mix", (S, S), role="bias", init="bias_normal", optional=self.hc_optional)]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().bind(tensors)
        S, dev = self.S, self.ctx.device
        self.hc = []
        for prefix in self.hc_prefixes[:1 if self.ffn is None else 2]:
            def get(name, default):
                t = tensors.get(prefix + name)
                return (default.to(dev) if t is None else t.float()).contiguous()
            self.hc.append((get("in", torch.ones(S)), get("out", torch.ones(S)), get("mix", torch.eye(S))))

    takes_pending = False

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        S = self.S
        T = residual.shape[0]
        write = batch.extras.pop("hc_write", None)     # the block before left its last write to this read
        y_prev, mix_prev, out_prev = write if write is not None else (None, None, None)
        w_in, w_out, w_mix = self.hc[0]
        x = ops.hc_step(residual, S, y_prev, mix_prev, out_prev, in_w=w_in, gain=self.mixer_norm.gain_f32(),
                        eps=self.mixer_norm.eps, out_dtype=self.ctx.dtype)
        y = torch.empty((T, self.hidden_size), dtype=torch.float32, device=residual.device)
        self.mixer.forward(x, y, batch, cache, owns_cache, accumulate=None)   # written; its sum may stay open for hc_step
        if self.ffn is not None:
            f_in, f_out, f_mix = self.hc[1]
            x = ops.hc_step(residual, S, y, w_mix, w_out, in_w=f_in, gain=self.ffn_norm.gain_f32(), eps=self.ffn_norm.eps,
                            out_dtype=self.ctx.dtype)
            y = torch.empty((T, self.hidden_size), dtype=torch.float32, device=residual.device)
            self.ffn.forward(x, y, batch, accumulate=None)
            w_out, w_mix = f_out, f_mix
        batch.extras["hc_write"] = (y, w_mix, w_out)


def flush_hyper_write(residual, batch, streams: int) -> None:
    """Makes the write that the last hyper block left open, so that ``residual`` holds the copies as they are."""
    write = batch.extras.pop("hc_write", None)
    if write is not None:
        ops.hc_step(residual, streams, write[0], write[1], write[2])


register_block("hyper", HyperBlock)


class ParallelBlock(PreNormBlock):
    """ONE norm whose output both sublayers read: ``h = norm(x)``, ``x += mixer(h') + ffn(h)``.  With the layer's
    ``token_shift`` (a vector s), the mixer reads ``h'_t = h_t + (h_{t-1} - h_t) * s`` (zeros before a sequence's first
    token) and the feed-forward h_t as it is; norm and shift are one kernel, and h of a request's last token is kept in a
    state slot of the block's own between steps (every run of the block has its own).  The two sublayers' sums into the
    stream may stay open together (``ops.gemm_tc_deferred`` chains them); the next block's norm adds them.

    With the layer's ``ffn_norm`` the feed-forward reads a second norm of the same stream: ``x += mixer(norm1(x)) +
    ffn(norm2(x))`` (no token shift then).  With the layer's ``layer_scale`` (two vectors s1, s2) the sublayers' outputs
    are multiplied channel by channel before they are added: ``x += s1 * mixer(..) + s2 * ffn(..)``; both sublayers then
    write to float32 buffers of their own, and the sum is left to whoever reads the stream next
    (``batch.extras["scaled_sum"]`` holds the buffers and vectors until then): the next such block makes it inside the
    kernel that norms the new rows (``ops.scale_add_norm2``: the sum and both norms in one pass over the stream); anyone
    else calls :func:`flush_scaled_sum` first (the decoder does, before a block of another kind, before the model's last
    norm and before it hands the stream out)."""
    takes_pending = True
    takes_scaled_sum = True

    def __init__(self, layer_spec, hidden_size: int, ctx: BuildContext):
        self.spec = layer_spec
        self.mixer_norm = build_norm(layer_spec.mixer_norm, hidden_size, ctx)
        self.mixer = build_mixer(layer_spec.mixer, hidden_size, ctx)
        self.ffn = build_ffn(layer_spec.ffn, hidden_size, ctx) if layer_spec.ffn is not None else None
        self.ffn_norm = None                   # one norm, unless the layer names a second one for the feed-forward
        self.shift_name = getattr(layer_spec, "token_shift", None)
        if layer_spec.ffn_norm is not None:
            if self.shift_name is not None:
                raise ValueError("the parallel arrangement with a token shift has one norm (mixer_norm); ffn_norm must be None")
            if self.ffn is not None:
                self.ffn_norm = build_norm(layer_spec.ffn_norm, hidden_size, ctx)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.shift = None
        self.scale_names = getattr(layer_spec, "layer_scale", None)
        self.scales = None
        # both norms plain RMS norms (a gain, no offset, nothing else): one kernel makes them, and the block before's sum
        from .norm import RMSNorm
        self._fused_norms = (self.shift_name is None and type(self.mixer_norm) is RMSNorm and self.mixer_norm.offset == 0.0
                             and (self.ffn_norm is None or (type(self.ffn_norm) is RMSNorm and self.ffn_norm.offset == 0.0))
                             and (self.scale_names is not None or self.ffn_norm is not None))
        if self.shift_name is not None and not hasattr(self.mixer_norm, "gain_f32"):
            raise ValueError(f"{type(self.mixer_norm).__name__} cannot stand before a token shift (it has no gain_f32)")

    def _children(self):
        s = self.spec
        kids = [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer)]
        if self.ffn_norm is not None:
            kids.append((s.ffn_norm_prefix, self.ffn_norm))
        if self.ffn is not None:
            kids.append((s.ffn_prefix, self.ffn))
        return kids

    def param_specs(self) -> List[ParamSpec]:
        out = super().param_specs()
        if self.shift_name is not None:
            out.append(ParamSpec(self.shift_name, (self.hidden_size,), role="bias", init="bias_normal"))
        if self.scale_names is not None:
            for k, name in enumerate(self.scale_names[:2]):
                # (a layer without a feed-forward may still store the second vector: taken and not used)
                out.append(ParamSpec(name, (self.hidden_size,), role="gain", init="ones", optional=k == 1 and self.ffn is None))
        if self.ffn is None and self.spec.ffn_norm is not None:     # likewise its second norm's gain
            out.append(ParamSpec(self.spec.ffn_norm_prefix + getattr(self.spec.ffn_norm, "param", "weight"), (self.hidden_size,),
                                 role="gain", init="ones", optional=True))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        super().bind(tensors)
        if self.shift_name is not None:
            self.shift = tensors[self.shift_name].float().contiguous()
        if self.scale_names is not None:
            self.scales = [tensors[name].float().contiguous() for name in self.scale_names[:2 if self.ffn is not None else 1]]
        if self._fused_norms and self.ffn_norm is not None and self.ffn_norm.weight.dtype != self.mixer_norm.weight.dtype:
            self._fused_norms = False     # gains stored in different types: each norm runs by itself

    def cache_request(self):
        rq = self.mixer.cache_request()
        if self.shift_name is None:
            return rq
        # the mixer's need first (None stays in its place), then the previous token's normed row
        from .base import FixedStateRequest
        return (rq, FixedStateRequest((self.hidden_size,), torch.float32)) if rq is not None \
            else (FixedStateRequest((self.hidden_size,), torch.float32),)

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        if self.shift_name is not None:
            if not owns_cache:
                raise ops.KernelError("a block with a token shift owns its state: it cannot run on another run's cache")
            flush_scaled_sum(residual, batch)
            mixer_cache, state = (cache[0], cache[1]) if len(cache) == 2 else (None, cache[0])
            h, hs = ops.rmsnorm_shift(residual, self.mixer_norm.gain_f32(), self.shift, state.state, batch,
                                      self.mixer_norm.eps, self.ctx.dtype, want_h=self.ffn is not None)
        elif self._fused_norms:
            # the sum that the block before left, and both norms of the new rows, in one pass over the stream
            mixer_cache = cache
            ops.resolve_pending()
            n1, n2 = self.mixer_norm, self.ffn_norm
            hs, h = ops.scale_add_norm2(residual, batch.extras.pop("scaled_sum", None), n1.weight, n1.eps,
                                        None if n2 is None else n2.weight, 0.0 if n2 is None else n2.eps, self.ctx.dtype)
        else:
            mixer_cache = cache
            flush_scaled_sum(residual, batch)
            h = hs = self._normed(self.mixer_norm, residual)
            if self.ffn_norm is not None:      # (the first norm has made any open sum of the stream)
                h = self.ffn_norm.forward(residual)
        if self.scales is None:
            self.mixer.forward(hs, residual, batch, mixer_cache, owns_cache)
            if self.ffn is not None:
                self.ffn.forward(h, residual, batch)
            return
        # each sublayer writes to a buffer of its own; x += s1 * mixer + s2 * ffn is one kernel
        ym = torch.empty_like(residual)
        self.mixer.forward(hs, ym, batch, mixer_cache, owns_cache, accumulate=False)
        yf = None
        if self.ffn is not None:
            yf = torch.empty_like(residual)
            self.ffn.forward(h, yf, batch, accumulate=False)
        batch.extras["scaled_sum"] = (ym, self.scales[0], yf, None if yf is None else self.scales[1])


def flush_scaled_sum(residual, batch) -> None:
    """Makes the sum that a block with a layer scale left open, so that ``residual`` holds the stream as it is."""
    pend = batch.extras.pop("scaled_sum", None)
    if pend is not None:
        ops.scale_add(residual, *pend)


register_block("parallel", ParallelBlock)
