"""Vubotar: config.json -> :class:`ModelConfig`.

A decoder whose layers are listed one by one (config ``layers``: each with ``type``, the mixer; ``mixer``, its sizes;
``mlp``, its feed-forward or null).  What sets the design apart:

* the embedding's rows are multiplied by ``embedding.scale``;
* a layer is parallel with two norms and a scale per channel on each sublayer's output:
  ``x += ls1 * mixer(norm1(x)) + ls2 * ffn(norm2(x))`` (tensors ``l<i>.norm1``, ``norm2``, ``ls1``, ``ls2``);
* mixer ``attention``: grouped-query softmax attention without rotation; queries and keys normed per head (one gain
  vector shared by the heads); the score scale ``scale``; a soft cap ``softcap * tanh(score / softcap)``; then a learned
  bias per (distance, head) added (tensor ``rel`` [rows, heads]: distances below rows / 2 have a row each, the larger
  ones share rows on a logarithmic scale that reaches the last row at ``bias_max``); a window of ``mask.size`` keys plus
  the first ``mask.keep_first`` keys of the sequence; one added to the softmax's denominator; with ``v_mix`` the values
  of every such layer but the model's first become ``(1 - vmix) v + vmix v_first``, v_first the first such layer's
  values of the same token;
* mixer ``latent_attention``: queries through a latent (``dq``, ``dq.norm``, ``uq``); keys and values from a latent of
  ``kv_rank`` channels per token (normed with a gain) and one rotated key part of ``rot_dim`` channels shared by the
  heads; rotary encoding of channel pairs (2i, 2i + 1) with frequencies ``rot.base^(-2i / rot.dims)``; plain causal
  softmax; the concatenated heads times ``sigmoid(W_g h)``;
* mixer ``mlstm``: a matrix memory per head with exponential gates capped at ``gate_cap`` (``parts/mlstm.py``);
* feed-forward ``moe``: ``router.experts`` gated silu experts of size ``expert.ff``, of which a token uses ``router.top``:
  sigmoid scores, the choice by score + ``correction``, the weights the chosen scores over their sum + 1e-20;
* logits = head(norm(x)) * ``logit_scale``, then ``logit_softcap * tanh(logits / logit_softcap)``.

Tensors: ``embed``, ``l<i>.norm1|norm2|ls1|ls2``, ``l<i>.mix.q|k|v|q.norm|k.norm|rel|vmix|o`` or
``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o`` or ``l<i>.mix.q|k|v|g|o|norm|i|i.b|f|f.b``,
``l<i>.mlp.router|correction|e<j>.gate|up|down``, ``final.norm``, ``head``.

A key the design does not have but this parser takes: ``mixer.bias_rows``, the rows of ``rel``, for writing a model with
random weights; a stored model gives them by the tensor's shape.

This module only describes the model.  It builds nothing and owns no tensor.
"""
from __future__ import annotations

from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, LatentAttentionSpec, LayerSpec, MatrixLSTMSpec, ModelConfig, NoPositionSpec,
                            RMSNormSpec, RopeSpec, RoutedFFNSpec, ScheduleEntry)

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"), ("k_norm", "k.norm"),
                    ("rel", "rel"), ("vmix", "vmix"))
_LATENT_NAMES = (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"), ("uk", "uk"),
                 ("uv", "uv"), ("g", "g"), ("o", "o"))
_MLSTM_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"), ("i", "i"), ("i_bias", "i.b"),
                ("f", "f"), ("f_bias", "f.b"))

RENORM_EPS = 1e-20   # added to the sum of the chosen experts' scores


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


def _positive(d, key, where) -> float:
    v = _get(d, key, where, float)
    if not v > 0:
        raise ConfigError(f"config.json: {where}.{key} must be > 0, got {v!r}")
    return v


def _window(m: Mapping[str, Any], where: str):
    mask = m.get("mask")
    if mask is None:
        return None, 0
    size = _get(mask, "size", where + ".mask", int)
    keep = mask.get("keep_first", 0) or 0
    if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
        raise ConfigError(f"config.json: {where}.mask.keep_first must be a non-negative integer, got {keep!r}")
    return size, keep


def _attention(m: Mapping[str, Any], w: str, eps: float) -> AttentionSpec:
    heads, kv = _get(m, "heads", w, int), _get(m, "kv_heads", w, int)
    if heads % kv:
        raise ConfigError(f"config.json: {w}: heads ({heads}) is not a multiple of kv_heads ({kv})")
    dim, vdim = _get(m, "dim", w, int), _get(m, "vdim", w, int)
    window, keep = _window(m, w)
    cap = m.get("softcap")
    if cap is not None:
        cap = _positive(m, "softcap", w)
    rows = m.get("bias_rows")
    if rows is not None:
        rows = _get(m, "bias_rows", w, int)
    return AttentionSpec(num_heads=heads, num_kv_heads=kv, head_dim=dim, qkv_bias=False, position=NoPositionSpec(),
                         window=window, softmax_scale=_get(m, "scale", w, float), v_head_dim=vdim if vdim != dim else None,
                         qk_norm_eps=eps, qk_norm="head", names=_ATTENTION_NAMES, keep_first=keep, score_softcap=cap,
                         distance_table_far=_positive(m, "bias_max", w), distance_table_rows=rows, fixed_sink=0.0,
                         value_mix="vmix" if m.get("v_mix") else None)


def _latent(m: Mapping[str, Any], w: str, eps: float) -> LatentAttentionSpec:
    rot_dim = _get(m, "rot_dim", w, int)
    rot = _get(m, "rot", w)
    dims = _get(rot, "dims", w + ".rot", int)
    if dims != rot_dim or dims % 2:
        raise ConfigError(f"config.json: {w}.rot.dims ({dims}) must be the even rot_dim ({rot_dim})")
    base = _get(rot, "base", w + ".rot", float)
    if not base > 1:
        raise ConfigError(f"config.json: {w}.rot.base must be > 1, got {base!r}")
    window, keep = _window(m, w)      # (the design's latent mixer sees every earlier key; a window is taken if one is given)
    if keep:
        raise ConfigError(f"config.json: {w}.mask.keep_first: this mixer keeps no first keys")
    return LatentAttentionSpec(num_heads=_get(m, "heads", w, int), head_dim=_get(m, "dim", w, int), rot_dim=rot_dim,
                               v_head_dim=_get(m, "vdim", w, int), kv_rank=_get(m, "kv_rank", w, int), norm_eps=eps,
                               position=RopeSpec(theta=base, rotary_dim=dims, scaling=None, interleaved=True),
                               softmax_scale=_get(m, "scale", w, float), window=window, sink=False, names=_LATENT_NAMES,
                               q_rank=_get(m, "q_rank", w, int), output_gate=True)


def _mlstm(m: Mapping[str, Any], w: str, eps: float) -> MatrixLSTMSpec:
    return MatrixLSTMSpec(num_heads=_get(m, "heads", w, int), key_dim=_get(m, "dim", w, int), value_dim=_get(m, "vdim", w, int),
                          gate_cap=_positive(m, "gate_cap", w), norm_eps=eps, names=_MLSTM_NAMES)


_MIXERS = {"attention": _attention, "latent_attention": _latent, "mlstm": _mlstm}


def _mixer(layer: Mapping[str, Any], where: str, eps: float):
    kind = _get(layer, "type", where)
    if kind not in _MIXERS:
        raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ({sorted(_MIXERS)})")
    return _MIXERS[kind](_get(layer, "mixer", where), where + ".mixer", eps)


def _ffn(layer: Mapping[str, Any], where: str):
    f = layer.get("mlp")
    if f is None:
        return None
    w = where + ".mlp"
    kind = _get(f, "kind", w)
    if kind != "moe":
        raise ConfigError(f"config.json: {w}.kind {kind!r} is not a feed-forward of this design ('moe')")
    router = _get(f, "router", w)
    experts, top = _get(router, "experts", w + ".router", int), _get(router, "top", w + ".router", int)
    if top > experts:
        raise ConfigError(f"config.json: {w}.router.top ({top}) exceeds the experts ({experts})")
    return RoutedFFNSpec(num_experts=experts, top_k=top, expert_size=_get(_get(f, "expert", w), "ff", w + ".expert", int),
                         score="sigmoid", renormalize=True, scale_input=False, router_name="router",
                         expert_names=("e{e}.", "gate", "up", "down"), choice_bias="correction", renorm_eps=RENORM_EPS,
                         activation="silu")


def parse_vubotar(raw: Mapping[str, Any]) -> ModelConfig:
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
        ffn = _ffn(layer, where)
        layers.append(LayerSpec(
            mixer=_mixer(layer, where, eps), ffn=ffn, block="parallel",
            mixer_norm=RMSNormSpec(eps=eps, param="norm1"), ffn_norm=RMSNormSpec(eps=eps, param="norm2"),
            mixer_prefix="mix.", ffn_prefix="mlp.", mixer_norm_prefix="", ffn_norm_prefix="", layer_scale=("ls1", "ls2")))
    # the layers that mix values share the first one's values: they must have the same number and size of value heads
    mixing = [(i, ls.mixer) for i, ls in enumerate(layers) if getattr(ls.mixer, "value_mix", None)]
    for i, m in mixing[1:]:
        first = mixing[0][1]
        if (m.num_kv_heads, m.v_head_dim or m.head_dim) != (first.num_kv_heads, first.v_head_dim or first.head_dim):
            raise ConfigError(f"config.json: layers[{i}] mixes its values with those of layers[{mixing[0][0]}], "
                              f"which has other kv_heads or vdim")
    scale = _get(_get(raw, "embedding", "the top level"), "scale", "embedding", float)
    logit_scale = raw.get("logit_scale", 1.0)
    if isinstance(logit_scale, bool) or not isinstance(logit_scale, (int, float)):
        raise ConfigError(f"config.json: logit_scale must be a number, got {logit_scale!r}")
    cap = raw.get("logit_softcap")
    if cap is not None:
        cap = _positive(raw, "logit_softcap", "the top level")
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
    return ModelConfig(
        architecture="Vubotar", hidden_size=width, vocab_size=vocab, layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
        final_norm=RMSNormSpec(eps=eps, param="norm"), tie_word_embeddings=False, max_position_embeddings=0,
        weight_prefix="", layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head",
        embedding_multiplier=scale, logit_scale=float(logit_scale), logit_softcap=cap,
        eos_token_ids=eos_ids, stored_dtype=str(raw.get("torch_dtype", "bfloat16")), raw=dict(raw))


register_architecture("Vubotar", parse_vubotar, model_type="vubotar")
