"""Zigipel: config.json -> :class:`ModelConfig`.

A decoder whose layers are listed one by one (config ``layers``: each with ``type``, the mixer; ``mixer``, its sizes;
``mlp``, its feed-forward or null).  What sets the design apart:

* the embedding's output is the token's row plus a row of a second table (``bigram``) chosen by a hash of the previous
  token and the token (``embedding.bigram``: buckets, mul_prev, mul_cur; the table's last row for a sequence's first
  token);
* ``loop`` {start, stop, times}: layers start .. stop-1 run ``times`` times in a row with the same weights, each pass
  with caches and states of its own; before every pass (the first too) the stream becomes ``W_in [x; x0] + step[t]``
  with x0 the embedding's output (tensors ``loop.in`` [width, 2 width], ``loop.step`` [times, width]);
* a layer is parallel: ``h = norm1(x)``, ``x += mixer(h') + ffn(h)``, where the mixer's input is shifted toward the
  previous token, ``h'_t = h_t + (h_{t-1} - h_t) * shift`` (tensor ``l<i>.shift``; zeros before the first token);
* mixer ``attention``: grouped-query softmax attention without rotation; every value head divided by its root mean
  square; the score scale ``scale``; ``r1_h ln(1 + r2_h (i - j))`` taken off the score of query i and key j; a window
  of ``mask.size`` keys plus the first ``mask.keep_first`` keys of the sequence; a learned sink per head in the
  softmax's denominator; every head's output times one gate number ``sigmoid(W_g h')_h``;
* mixer ``latent_attention``: keys and values from a latent vector of ``kv_rank`` channels per token (normed with a
  gain) and one rotated key part of ``rot_dim`` channels shared by the heads; rotary encoding (channel i with channel
  i + dims / 2) with YaRN frequencies and magnitude on the rotated parts; a window of ``mask.size`` keys; a sink;
* feed-forward ``dense``: ``down(gelu_tanh(gate h) * (up h))``, every projection with a bias;
* logits = head(norm(x)) * ``logit_scale``.

Tensors: ``embed``, ``bigram``, ``loop.in``, ``loop.step``, ``l<i>.norm1``, ``l<i>.shift``,
``l<i>.mix.q|k|v|g|o|r1|r2|sink`` or ``l<i>.mix.q|dkv|dkv.norm|uk|uv|o|sink``, ``l<i>.mlp.gate|up|down`` (+ ``.b``),
``final.norm``, ``head``.

This module only describes the model.  It builds nothing and owns no tensor.
"""
from __future__ import annotations

from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, BigramEmbeddingSpec, LatentAttentionSpec, LayerSpec, ModelConfig, NoPositionSpec,
                            PassInputSpec, RMSNormSpec, RopeSpec, ScheduleEntry, SwiGLUSpec, YarnRopeScaling)

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("g", "g"), ("sink", "sink"), ("r1", "r1"), ("r2", "r2"))
_LATENT_NAMES = (("q", "q"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"), ("uk", "uk"), ("uv", "uv"), ("o", "o"), ("sink", "sink"))


def _get(d: Mapping[str, Any], key: str, where: str, kind=None):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    v = d[key]
    if kind is int and (isinstance(v, bool) or not isinstance(v, int) or v <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
        v = float(v)
    return v


def _window(m: Mapping[str, Any], where: str, with_kept: bool):
    """(window, keep_first) of ``mask``: a query sees itself and the ``size`` - 1 keys before it, and with
    ``keep_first`` the first so many keys of the sequence too.  No ``mask``: every earlier key."""
    mask = m.get("mask")
    if mask is None:
        return None, 0
    size = _get(mask, "size", where + ".mask", int)
    keep = mask.get("keep_first", 0) or 0
    if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
        raise ConfigError(f"config.json: {where}.mask.keep_first must be a non-negative integer, got {keep!r}")
    if keep and not with_kept:
        raise ConfigError(f"config.json: {where}.mask.keep_first: this mixer keeps no first keys")
    return size, keep


def _attention(m: Mapping[str, Any], w: str, eps: float) -> AttentionSpec:
    heads, kv = _get(m, "heads", w, int), _get(m, "kv_heads", w, int)
    if heads % kv:
        raise ConfigError(f"config.json: {w}: heads ({heads}) is not a multiple of kv_heads ({kv})")
    dim, vdim = _get(m, "dim", w, int), _get(m, "vdim", w, int)
    window, keep = _window(m, w, True)
    return AttentionSpec(num_heads=heads, num_kv_heads=kv, head_dim=dim, qkv_bias=False, position=NoPositionSpec(),
                         window=window, softmax_scale=_get(m, "scale", w, float), v_head_dim=vdim if vdim != dim else None,
                         names=_ATTENTION_NAMES, sink=True, output_gate=True, gate_per_head=True, v_norm_eps=eps,
                         distance_bias=True, keep_first=keep)


def _rotary(rot: Mapping[str, Any], w: str, rot_dim: int) -> RopeSpec:
    dims = _get(rot, "dims", w, int)
    if dims != rot_dim or dims % 2:
        raise ConfigError(f"config.json: {w}.dims ({dims}) must be the even rot_dim ({rot_dim})")
    scaling = None
    sc = rot.get("scaling")
    if sc is not None:
        ws = w + ".scaling"
        scaling = YarnRopeScaling(factor=_get(sc, "factor", ws, float), original=_get(sc, "original", ws, int),
                                  fast=_get(sc, "fast", ws, float), slow=_get(sc, "slow", ws, float))
        if not scaling.factor > 0 or not scaling.fast > 0 or not scaling.slow > 0:
            raise ConfigError(f"config.json: {ws}: factor, fast and slow must be > 0")
    base = _get(rot, "base", w, float)
    if not base > 1:
        raise ConfigError(f"config.json: {w}.base must be > 1, got {base!r}")
    return RopeSpec(theta=base, rotary_dim=dims, scaling=scaling, interleaved=False)


def _latent(m: Mapping[str, Any], w: str, eps: float) -> LatentAttentionSpec:
    rot_dim = _get(m, "rot_dim", w, int)
    window, _ = _window(m, w, False)
    return LatentAttentionSpec(num_heads=_get(m, "heads", w, int), head_dim=_get(m, "dim", w, int), rot_dim=rot_dim,
                               v_head_dim=_get(m, "vdim", w, int), kv_rank=_get(m, "kv_rank", w, int), norm_eps=eps,
                               position=_rotary(_get(m, "rot", w), w + ".rot", rot_dim),
                               softmax_scale=_get(m, "scale", w, float), window=window, sink=True, names=_LATENT_NAMES)


def _mixer(layer: Mapping[str, Any], where: str, eps: float):
    kind = _get(layer, "type", where)
    m = _get(layer, "mixer", where)
    if kind == "attention":
        return _attention(m, where + ".mixer", eps)
    if kind == "latent_attention":
        return _latent(m, where + ".mixer", eps)
    raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ('attention', 'latent_attention')")


def _ffn(layer: Mapping[str, Any], where: str):
    f = layer.get("mlp")
    if f is None:
        return None
    w = where + ".mlp"
    kind = _get(f, "kind", w)
    if kind != "dense":
        raise ConfigError(f"config.json: {w}.kind {kind!r} is not a feed-forward of this design ('dense')")
    return SwiGLUSpec(intermediate_size=_get(f, "ff", w, int), activation="gelu_tanh", names=("gate", "up", "down"),
                      bias_names=("gate.b", "up.b", "down.b"))


def parse_zigipel(raw: Mapping[str, Any]) -> ModelConfig:
    width, vocab = _get(raw, "width", "the top level", int), _get(raw, "vocab", "the top level", int)
    eps = _get(_get(raw, "norm", "the top level"), "eps", "norm", float)
    if not eps > 0:
        raise ConfigError(f"config.json: norm.eps must be > 0, got {eps!r}")
    raw_layers = _get(raw, "layers", "the top level")
    if not isinstance(raw_layers, list) or not raw_layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    layers = []
    for i, layer in enumerate(raw_layers):
        where = f"layers[{i}]"
        layers.append(LayerSpec(
            mixer=_mixer(layer, where, eps), ffn=_ffn(layer, where), block="parallel", token_shift="shift",
            mixer_norm=RMSNormSpec(eps=eps, param="norm1"), ffn_norm=None,
            mixer_prefix="mix.", ffn_prefix="mlp.", mixer_norm_prefix="", ffn_norm_prefix=""))
    n = len(layers)
    loop = raw.get("loop")
    pass_input = None
    if loop is None:
        schedule = [ScheduleEntry(layer=i) for i in range(n)]
    else:
        start, stop, times = (loop.get(k) for k in ("start", "stop", "times"))
        if not all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop, times)) \
                or not (0 <= start < stop <= n) or times < 1:
            raise ConfigError(f"config.json: loop needs integers 0 <= start < stop <= {n} and times >= 1, got {loop!r}")
        schedule = [ScheduleEntry(layer=i) for i in range(start)]
        for t in range(times):
            schedule += [ScheduleEntry(layer=i, pass_input=t if i == start else None) for i in range(start, stop)]
        schedule += [ScheduleEntry(layer=i) for i in range(stop, n)]
        pass_input = PassInputSpec(times=times, weight="loop.in", step="loop.step")
    bigram = None
    b = (raw.get("embedding") or {}).get("bigram")
    if b is not None:
        we = "embedding.bigram"
        bigram = BigramEmbeddingSpec(buckets=_get(b, "buckets", we, int), mul_prev=int(_get(b, "mul_prev", we)),
                                     mul_cur=int(_get(b, "mul_cur", we)), name="bigram")
    logit_scale = raw.get("logit_scale", 1.0)
    if isinstance(logit_scale, bool) or not isinstance(logit_scale, (int, float)):
        raise ConfigError(f"config.json: logit_scale must be a number, got {logit_scale!r}")
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
    return ModelConfig(
        architecture="Zigipel", hidden_size=width, vocab_size=vocab, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=RMSNormSpec(eps=eps, param="norm"), tie_word_embeddings=False, max_position_embeddings=0,
        weight_prefix="", layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head",
        logit_scale=float(logit_scale), bigram_embedding=bigram, pass_input=pass_input,
        eos_token_ids=eos_ids, stored_dtype=str(raw.get("torch_dtype", "bfloat16")), raw=dict(raw))


register_architecture("Zigipel", parse_zigipel, model_type="zigipel")
