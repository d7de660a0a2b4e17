"""The decoder that every registered architecture is run by: an embedding, blocks
built from the configuration's layer specs, a schedule that says in which order
they run and whose cache each run uses, a final norm and the output head; around
them the configuration's optional constants (embedding multiplier, logit scale,
logit soft cap), an optional vector of the position added to the embedding, and an
optional stream that is kept as several copies (``ModelConfig.streams``: every block
is then a "hyper" block, the stream is [T, streams * hidden], and the model's last
norm reads the sum of the copies), an optional second embedding table addressed by a hash
of the previous token and the token (``ModelConfig.bigram_embedding``; the previous token
of a request is kept in a state slot of the model's own), and an optional mixing of the
stream with the embedding's output before every pass over a repeated stretch of layers
(``ModelConfig.pass_input``).

It is driven by :class:`ModelConfig` alone and knows no architecture by name.
Reference for the sequence of operations: src/core/engine.cpp:921-1041.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.specs import ModelConfig
from ..kernels import ops
from ..parts import BuildContext, FixedStateRequest, ParamSpec, build_block, build_norm
from ..parts.block import flush_hyper_write, flush_scaled_sum
from ..parts.linear import Linear


def sinusoid_frequencies(width: int, base: float) -> torch.Tensor:
    """float32 [ceil(width / 2)]: base^(-2i / width), computed in float64 and rounded once."""
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / width).to(torch.float32)


class DecoderModel:
    def __init__(self, config: ModelConfig, ctx: BuildContext):
        self.config = config
        self.ctx = ctx
        H = config.hidden_size
        self.blocks = [build_block(ls, H, ctx) for ls in config.layers]
        self.final_norm = build_norm(config.final_norm, H, ctx)
        for e in config.schedule:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.blocks)}")
        for pos, e in enumerate(config.schedule):
            if e.cache_of is not None:
                if not 0 <= e.cache_of < pos or config.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {pos}: cache_of must name an earlier entry that owns its cache")
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None
        self.bigram = config.bigram_embedding
        self.bigram_table: Optional[torch.Tensor] = None
        self.pass_input = config.pass_input
        self.pass_in: List[Linear] = []        # one per pass: the same weight, the pass's own step vector as bias
        opens = [e.pass_input for e in config.schedule if e.pass_input is not None]
        if opens and self.pass_input is None:
            raise ValueError("a schedule entry opens a pass but the model has no pass_input")
        if self.pass_input is not None and any(not 0 <= t < self.pass_input.times for t in opens):
            raise ValueError(f"a schedule entry opens a pass outside 0 .. {self.pass_input.times - 1}")
        self._keeps_embedding = any(e.add_embedding for e in config.schedule) or bool(opens)
        self.streams = config.streams          # None: one plain stream
        if self.streams is not None:
            if any(ls.block != "hyper" for ls in config.layers) or self._keeps_embedding or self.bigram is not None:
                raise ValueError("a stream kept as several copies needs 'hyper' blocks throughout and no repeated stretch")
            if not hasattr(self.final_norm, "gain_f32"):
                raise ValueError(f"{type(self.final_norm).__name__} cannot close a stream of several copies (it has no gain_f32)")
            self._ones = torch.ones(self.streams, dtype=torch.float32, device=ctx.device)
        elif any(ls.block == "hyper" for ls in config.layers):
            raise ValueError("'hyper' blocks need ModelConfig.streams")
        from ..parts.norm import RMSNorm
        self._plain_final_norm = type(self.final_norm) is RMSNorm and self.final_norm.offset == 0.0
        self._pos_freq = None
        pe = config.position_embedding
        if pe is not None:
            if getattr(pe, "kind", None) != "sinusoidal":
                raise ValueError(f"unknown position embedding {pe!r}")
            self._pos_freq = sinusoid_frequencies(H, pe.base).to(ctx.device)
        # called as stream_hook(schedule position, stream [T, H] float32) after every run of a layer, if set:
        # for looking at the stream layer by layer (the engine then runs uncaptured; see Engine.step)
        self.stream_hook = None

    # ------------------------------------------------------------ parameters
    def param_specs(self) -> Dict[str, ParamSpec]:
        c = self.config
        specs: Dict[str, ParamSpec] = {}
        specs[c.embed_name] = ParamSpec(c.embed_name, (c.vocab_size, c.hidden_size))
        if self.bigram is not None:
            specs[self.bigram.name] = ParamSpec(self.bigram.name, (self.bigram.buckets + 1, c.hidden_size))
        if self.pass_input is not None:
            pi = self.pass_input
            specs[pi.weight] = ParamSpec(pi.weight, (c.hidden_size, 2 * c.hidden_size))
            specs[pi.step] = ParamSpec(pi.step, (pi.times, c.hidden_size), role="bias", init="bias_normal")
        for i, blk in enumerate(self.blocks):
            prefix = c.layer_prefix.format(i=i)
            for p in blk.param_specs():
                specs[prefix + p.name] = ParamSpec(prefix + p.name, p.shape, p.role, p.init, p.optional)
        for p in self.final_norm.param_specs():
            name = c.final_norm_prefix + p.name
            specs[name] = ParamSpec(name, p.shape, p.role, p.init, p.optional)
        # a tied head reuses the embedding table; a stored lm_head is then tolerated and ignored
        specs[c.head_name] = ParamSpec(c.head_name, (c.vocab_size, c.hidden_size),
                                       optional=c.tie_word_embeddings)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        c = self.config
        self.embed = tensors[c.embed_name].contiguous()
        if self.bigram is not None:
            self.bigram_table = tensors[self.bigram.name].to(self.embed.dtype).contiguous()
        if self.pass_input is not None:
            w, step = tensors[self.pass_input.weight], tensors[self.pass_input.step].float()
            self.pass_in = [Linear(w, step[t].contiguous()) for t in range(self.pass_input.times)]
        for i, blk in enumerate(self.blocks):
            prefix = c.layer_prefix.format(i=i)
            blk.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})
        stem = c.final_norm_prefix
        self.final_norm.bind({k[len(stem):]: v for k, v in tensors.items() if k.startswith(stem)})
        self.head = Linear(self.embed if c.tie_word_embeddings else tensors[c.head_name])

    # ------------------------------------------------------------ caches
    def cache_requests(self) -> List[object]:
        """Per schedule entry: what cache that run owns (None if it owns none; a tuple if the block keeps something
        beside its mixer's).  A model that keeps something per request itself (the previous token, for the hashed second
        embedding table) asks for it in one more entry behind the schedule's."""
        out = []
        for e in self.config.schedule:
            out.append(None if e.cache_of is not None else self.blocks[e.layer].cache_request())
        if self.bigram is not None:
            out.append(FixedStateRequest((1,), torch.int32))
        return out

    # ------------------------------------------------------------ forward
    def forward(self, batch, caches: List[object]) -> torch.Tensor:
        """Runs the batch's tokens through the schedule; returns float32 logits
        [len(batch.logit_rows), vocab] for the rows that were asked for."""
        c = self.config
        ops.discard_pending()   # nothing of an earlier (failed) pass is added into this one's tensors
        S = self.streams
        if S is not None or self._pos_freq is not None:
            h = ops.embed_positions(self.embed, batch.token_ids, batch.positions, self._pos_freq, copies=S or 1,
                                    scale=c.embedding_multiplier)
        elif self.bigram is not None:
            b = self.bigram
            h = ops.embed_bigram(self.embed, self.bigram_table, batch, caches[len(c.schedule)].state, b.buckets, b.mul_prev,
                                 b.mul_cur, scale=c.embedding_multiplier)
        else:
            h = ops.embed_gather(self.embed, batch.token_ids, scale=c.embedding_multiplier)
        h0 = h.clone() if self._keeps_embedding else None   # the embedding's output, for repeated passes
        for pos, e in enumerate(self.config.schedule):
            cache = caches[e.cache_of if e.cache_of is not None else pos]
            blk = self.blocks[e.layer]
            if not blk.takes_pending or e.add_embedding or e.pass_input is not None:
                ops.resolve_pending()   # the block before may have left its last sum to the next reader
            if not getattr(blk, "takes_scaled_sum", False) or e.add_embedding or e.pass_input is not None:
                flush_scaled_sum(h, batch)   # sublayer outputs that a block left to the stream's next reader
            if e.add_embedding:
                ops.add_into(h, h0)
            if e.pass_input is not None:
                # the stream becomes W [x; x0] + step[t]: both streams side by side in the compute type, one product
                self.pass_in[e.pass_input](ops.concat2_cast(h, h0, self.ctx.dtype), out=h)
            blk.forward(h, batch, cache, owns_cache=e.cache_of is None)
            if self.stream_hook is not None:
                ops.resolve_pending()
                flush_scaled_sum(h, batch)
                if S is not None:   # the hook sees the sum of the copies
                    flush_hyper_write(h, batch, S)
                    self.stream_hook(pos, ops.hc_step(h, S, in_w=self._ones))
                else:
                    self.stream_hook(pos, h)
        n = batch.logit_rows.numel()
        if n == 0:
            ops.discard_pending(h)
            batch.extras.pop("hc_write", None)
            batch.extras.pop("scaled_sum", None)
            return torch.empty((0, self.config.vocab_size), dtype=torch.float32, device=h.device)
        if S is not None:
            # the last block's write, the sum of the copies and the model's norm, on the wanted rows only
            y, mix, out_w = batch.extras.pop("hc_write", None) or (None, None, None)
            x = ops.hc_step(h, S, y, mix, out_w, in_w=self._ones, gain=self.final_norm.gain_f32(), eps=self.final_norm.eps,
                            rows=batch.logit_rows, out_dtype=self.ctx.dtype)
        elif "scaled_sum" in batch.extras and self._plain_final_norm:
            # the last block's open layer-scale sum and the model's norm, on the wanted rows only (the stream ends here)
            ops.resolve_pending()
            x, _ = ops.scale_add_norm2(h, batch.extras.pop("scaled_sum"), self.final_norm.weight, self.final_norm.eps, None, 0.0,
                                       self.ctx.dtype, rows=batch.logit_rows)
        else:
            if "scaled_sum" in batch.extras:
                ops.resolve_pending()
                flush_scaled_sum(h, batch)
            if not self.final_norm.adds_pending:
                ops.resolve_pending()
            x = self.final_norm.forward(h, rows=batch.logit_rows)
        ops.discard_pending(h)          # the stream ends here: only the chosen rows were summed
        logits = self.head(x, out_dtype=torch.float32)
        if c.logit_scale != 1.0 or c.logit_softcap is not None:
            ops.logit_transform(logits, c.logit_scale, c.logit_softcap)
        return logits
