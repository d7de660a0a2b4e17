"""Typed descriptions of the parts a decoder is assembled from.

A model is data: a tuple of :class:`LayerSpec` (what each layer is made of) and a
tuple of :class:`ScheduleEntry` (the order in which layers run, and whose cache
each run reads).  Every size and constant lives in a spec; no part reads a
config.json key itself and no part knows which model it belongs to.

Each spec carries a ``kind`` string.  The part registries
(``blackwellllm_b200.parts.registry``) map ``kind`` to the class that builds the
part, so a new mixer, feed-forward, norm or position encoding is a new spec
dataclass plus one ``register_*`` call.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class Llama3RopeScaling:
    """Wavelength-band rescaling of rotary frequencies.

    Reference: src/kernels/rope.cuh:24-38 (apply_rope_scaling) and the keys read
    at src/core/config.cpp:263-273.
    """
    factor: float = 8.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192
    kind: str = "llama3"


@dataclass(frozen=True)
class YarnRopeScaling:
    """Rescaling of rotary frequencies by how often a pair turns within the original context.

    With ``pair(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(pair(fast)), 0)``
    and ``hi = min(ceil(pair(slow)), rotary_dim - 1)``, pair i gets ``ramp_i = clamp((i - lo) / max(hi - lo,
    0.001), 0, 1)`` and the frequency ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``; cosines and sines are
    multiplied by ``0.1 ln(factor) + 1``.
    """
    factor: float
    original: int
    fast: float
    slow: float
    kind: str = "yarn"


@dataclass(frozen=True)
class RopeSpec:
    """Rotary position encoding over the first ``rotary_dim`` channels of a head.  Channel i turns with
    channel i + rotary_dim / 2 (rotate_half), or with ``interleaved`` channel 2i with 2i + 1."""
    theta: float
    rotary_dim: int
    scaling: Optional[Any] = None   # Llama3RopeScaling | YarnRopeScaling
    interleaved: bool = False
    kind: str = "rope"


@dataclass(frozen=True)
class NoPositionSpec:
    """A mixer that encodes no position (keys and queries are used as projected)."""
    kind: str = "none"


@dataclass(frozen=True)
class SinusoidalEmbeddingSpec:
    """A vector of the token's position added to its embedding: entry 2i is sin(p * base^(-2i/width)), entry
    2i + 1 the cosine of the same angle (positions count from 0 in each sequence)."""
    base: float = 10000.0
    kind: str = "sinusoidal"


@dataclass(frozen=True)
class RMSNormSpec:
    eps: float
    kind: str = "rmsnorm"
    param: str = "weight"   # the gain's name below the norm's prefix
    offset: float = 0.0     # the gain is offset + the stored tensor (1: a weight that is stored around zero)


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a paged key/value cache.

    ``window`` is the number of most recent keys (the query's own position
    included) a query may see; ``None`` means all of them.
    """
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qkv_bias: bool
    position: Any  # RopeSpec | NoPositionSpec | any registered position spec
    window: Optional[int] = None
    softmax_scale: Optional[float] = None  # None -> head_dim ** -0.5
    kind: str = "gqa_attention"
    # ``chunk``: a query sees no key before the start of its own block of ``chunk`` positions (blocks are
    # counted from position 0 of the sequence).  ``v_head_dim``: the value size of a head where it differs
    # from the query/key size ``head_dim``.  ``qk_norm_eps``: RMS norm with a gain per channel over the
    # WHOLE query projection of a token (all heads at once), and over the whole key projection, before the
    # rotation.  ``names``: the tensors' names below the mixer's prefix, as (role, name) pairs for
    # q, k, v, o, q_bias, k_bias, v_bias, q_norm, k_norm (default: q_proj.weight, q_proj.bias, ...).
    chunk: Optional[int] = None
    v_head_dim: Optional[int] = None
    qk_norm_eps: Optional[float] = None
    names: Tuple[Tuple[str, str], ...] = ()
    # ``qk_norm``: "whole" (above) or "head": every query head and every key head is normed by itself over its
    # ``head_dim`` channels, with one gain vector of that size shared by the heads.  ``q_temperature`` =
    # (coef, every): the queries of position p are multiplied by 1 + coef * log(1 + n), n = whole periods of `every` positions that p + 1 holds.
    # ``sink``: a learned number per query head (tensor "sink") whose exponential joins the softmax's
    # denominator; it has no key and no value and is not scaled.  ``output_gate``: the heads' outputs are
    # multiplied element by element by sigmoid(W_g x) (tensor "g", [heads * value size, hidden]) before the
    # output projection; x is the mixer's input.  ``shares_kv``: the mixer has no key and value tensors (no
    # projections, no key norm) and reads the cache of another run of the schedule with its own queries.
    qk_norm: str = "whole"
    q_temperature: Optional[Tuple[float, float]] = None
    sink: bool = False
    output_gate: bool = False
    shares_kv: bool = False
    # ``gate_per_head``: the output gate has ONE number per query head (tensor "g" is [heads, hidden]) instead of one
    # per channel.  ``v_norm_eps``: every value head is divided by sqrt(mean(v^2) + eps) before it is cached (no
    # gain).  ``distance_bias``: r1_h ln(1 + r2_h (i - j)) is taken off the score of query i and key j, with two
    # learned numbers per query head (tensors "r1", "r2").  ``keep_first``: with a window, the first so many keys of
    # a sequence stay visible to every later query.
    gate_per_head: bool = False
    v_norm_eps: Optional[float] = None
    distance_bias: bool = False
    keep_first: int = 0
    # ``score_softcap``: the scaled score s becomes cap * tanh(s / cap) before any bias is added.  ``distance_table_far``:
    # a learned bias per (distance, query head) is added to the score (after the cap; the score scale does not multiply
    # it): tensor "rel" [rows, heads]; distances below rows / 2 have a row each, larger ones share rows on a logarithmic
    # scale that reaches the last row at this distance (``kernels.ops.distance_bucket_table``).  ``distance_table_rows``:
    # the table's rows where the configuration states them (None: whatever the stored tensor has).  ``fixed_sink``: the
    # softmax's denominator has one more term exp(fixed_sink) that is a constant of the design, not a tensor (0.0: one is
    # added to the denominator).  ``value_mix``: the name of a number lam (a tensor without axes): in every layer of the
    # model that has it but the first such layer, the values become (1 - lam) v + lam v_first before they are cached,
    # v_first being the first such layer's values of the same token (the first layer's own number is not used).
    score_softcap: Optional[float] = None
    distance_table_far: Optional[float] = None
    distance_table_rows: Optional[int] = None
    fixed_sink: Optional[float] = None
    value_mix: Optional[str] = None


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Softmax attention whose keys and values of all heads are made from one latent vector per token:
    ``[c_raw, k_rot] = W_dkv x`` (``kv_rank`` + ``rot_dim`` rows), ``c = rms_norm(c_raw) * gain``; head h has the key
    ``[W_uk,h c, rotated k_rot]`` and the value ``W_uv,h c``; its query ``W_q,h x`` is laid out as ``head_dim`` plain
    channels, then ``rot_dim`` rotated ones.  Only c and the rotated k_rot are cached.  ``position``: the rotary
    encoding of the rotated parts (its ``rotary_dim`` = ``rot_dim``).  ``window``, ``sink``, ``softmax_scale`` as in
    :class:`AttentionSpec`.  ``names``: (role, name) pairs for q, dkv, dkv_norm, uk, uv, o, sink (and dq, dq_norm, uq, g).
    ``q_rank``: the queries come through a latent of their own, ``q = W_uq rms_norm(W_dq x) * gain`` (tensors dq
    [q_rank, hidden], dq_norm [q_rank], uq [heads * (head_dim + rot_dim), q_rank]) instead of one tensor q.
    ``output_gate``: the concatenated heads' outputs are multiplied element by element by sigmoid(W_g x) (tensor g
    [heads * v_head_dim, hidden]) before the output projection."""
    num_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    kv_rank: int
    norm_eps: float
    position: Any
    softmax_scale: float
    window: Optional[int] = None
    sink: bool = False
    kind: str = "latent_attention"
    names: Tuple[Tuple[str, str], ...] = ()
    q_rank: Optional[int] = None
    output_gate: bool = False


@dataclass(frozen=True)
class MatrixLSTMSpec:
    """A recurrent mixer with a [key_dim, value_dim] matrix memory per head and exponential gates (mLSTM):
    ``q = W_q x / sqrt(key_dim)``, ``k = W_k x``, ``v = W_v x``; per head a log input gate ``i = cap tanh((w_i x + b_i) /
    cap)`` and a log forget gate ``f = log_sigmoid(cap tanh((w_f x + b_f) / cap))``; with a running maximum m (from 0):
    ``m' = max(f + m, i)``, ``S <- exp(f + m - m') S + exp(i - m') k v^T``, n likewise with k alone,
    ``o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)``; each head's o is divided by its root mean square, the heads side by
    side are multiplied by a gain of all heads' size and by ``sigmoid(W_g x)``, then projected.  ``names``: (role, name)
    pairs for q, k, v, g, o, norm, i, i_bias, f, f_bias."""
    num_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    norm_eps: float
    kind: str = "matrix_lstm"
    names: Tuple[Tuple[str, str], ...] = ()


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """A recurrent mixer with a [key_dim, value_dim] state per head and a decay per key channel:
    ``S <- diag(a) S + k v^T``, ``o = S^T q / sqrt(key_dim)``, ``a = sigmoid(W2 (W1 x) + b) ** (1 / tau)``;
    each head's output is RMS-normed over value_dim (one gain shared by the heads), multiplied by
    ``silu(W_g x)`` and projected.  ``decay_rank``: the inner size of the decay's two projections
    (None: whatever the stored tensors have)."""
    num_heads: int
    key_dim: int
    value_dim: int
    tau: float
    norm_eps: float
    decay_rank: Optional[int] = None
    kind: str = "gated_linear_attention"
    names: Tuple[Tuple[str, str], ...] = ()


@dataclass(frozen=True)
class RoutedFFNSpec:
    """Mixture of experts: ``num_experts`` gated feed-forwards ``down(silu(gate u) * (up u))`` without biases,
    of which each token uses the ``top_k`` with the largest router scores.  ``score``: "sigmoid" or
    "softmax" of the float32 router logits; ``renormalize``: the chosen scores are divided by their sum;
    ``scale_input``: the score multiplies what the expert reads (u = s x) instead of what it returns."""
    num_experts: int
    top_k: int
    expert_size: int
    score: str = "sigmoid"
    renormalize: bool = False
    scale_input: bool = False
    kind: str = "routed_ffn"
    router_name: str = "router"
    expert_names: Tuple[str, str, str, str] = ("e{e}.", "gate", "up", "down")
    # ``identity_experts``: the router has this many outputs more than there are experts; the last ones stand
    # for experts without tensors that return their input.  ``choice_bias``: the name of a vector with one entry
    # per router output that is added to the scores for the CHOICE only (the weights stay the scores), or None.
    # ``renorm_eps``: added to the sum that ``renormalize`` divides by.  ``activation``: the experts' gated
    # activation, "silu" (silu(g) u) or "clamped_swish" (g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit),
    # u' = clamp(u, -limit, limit)).  ``shared``: a dense gated feed-forward (a :class:`SwiGLUSpec`) that runs
    # for every token and is added; its tensors lie below ``shared_prefix``.
    identity_experts: int = 0
    choice_bias: Optional[str] = None
    renorm_eps: float = 0.0
    activation: str = "silu"
    act_limit: float = 0.0
    act_alpha: float = 1.0
    shared: Any = None
    shared_prefix: str = "shared."


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(silu(gate(x)) * up(x)); with ``activation`` "clamped_swish":
    down(g sigmoid(alpha g) (u + 1)), g = min(gate(x), limit), u = clamp(up(x), -limit, limit).
    ``names``: the three tensors (gate, up, down) below the part's prefix."""
    intermediate_size: int
    kind: str = "swiglu"
    activation: str = "silu"
    act_limit: float = 0.0
    act_alpha: float = 1.0
    names: Tuple[str, str, str] = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
    # ``activation`` "gelu_tanh": 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * u.  ``bias_names``: the three
    # projections' bias vectors (gate, up, down), or None for projections without biases.
    bias_names: Optional[Tuple[str, str, str]] = None


@dataclass(frozen=True)
class DenseMLPSpec:
    """Dense feed-forward without a gate: down(act(up(x))); ``activation`` "relu2": max(z, 0)^2."""
    intermediate_size: int
    activation: str = "relu2"
    kind: str = "dense_mlp"
    names: Tuple[str, str] = ("up", "down")


@dataclass(frozen=True)
class HyperConnectionSpec:
    """The stream as ``streams`` copies x_1 .. x_s.  Sublayer q of a layer reads u = sum_s in[s] x_s (through its
    norm) and writes x_t <- sum_s mix[s, t] x_s + out[t] * y, all copies at once from the old ones.  The
    tensors "in" [s], "out" [s], "mix" [s, s] lie below ``mixer_prefix`` / ``ffn_prefix`` of the layer."""
    streams: int
    mixer_prefix: str = "hc1."
    ffn_prefix: str = "hc2."
    optional_tensors: bool = False   # True: a missing tensor stands for in = out = 1, mix = identity (one copy only)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which mixer, which feed-forward, which norms, arranged how.

    ``block`` names the arrangement (``"prenorm"``: x += mixer(norm(x));
    x += ffn(norm(x)); ``"sandwich"``: the same with a second norm on each sublayer's output; ``"hyper"``:
    pre-norm sublayers over several copies of the stream, see ``hyper``; ``"parallel"``: one norm whose output both
    sublayers read, see ``token_shift``).  ``ffn`` may be ``None`` for a mixer-only layer.
    """
    mixer: Any
    ffn: Any
    mixer_norm: Any
    ffn_norm: Any
    block: str = "prenorm"
    # where each part's tensors sit below the layer's prefix in the checkpoint
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    ffn_norm_prefix: str = "post_attention_layernorm."
    # the "sandwich" arrangement norms each sublayer's OUTPUT too before it is added to the stream:
    # x += post(mixer(pre(x))); x += post(ffn(pre(x)))
    mixer_post_norm: Any = None
    ffn_post_norm: Any = None
    mixer_post_norm_prefix: str = ""
    ffn_post_norm_prefix: str = ""
    # the "hyper" arrangement keeps several copies of the stream (a :class:`HyperConnectionSpec`)
    hyper: Any = None
    # the "parallel" arrangement: ONE norm, both sublayers read its output, x += mixer(h) + ffn(h).  ``token_shift``:
    # the name of a vector s [hidden]; the mixer then reads h_t + (h_{t-1} - h_t) * s (zeros before a sequence's first
    # token; the feed-forward reads h_t as it is), and the block keeps h of a request's last token between steps.
    token_shift: Optional[str] = None
    # the "parallel" arrangement: the names of two vectors [hidden] ("layer scale"); the mixer's output is multiplied
    # channel by channel by the first and the feed-forward's by the second before they are added to the stream
    layer_scale: Optional[Tuple[str, str]] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_of`` is the schedule position whose cache this
    run reads instead of owning one (``None``: it owns its cache and appends to it).
    A layer index may appear in several entries (weights shared, caches separate).
    """
    layer: int
    cache_of: Optional[int] = None
    # the embedding's output (the stream as it was before the first run) is added to the stream right
    # before this run: the start of a repeated pass over a stretch of layers
    add_embedding: bool = False
    # the number t of the pass that this run opens (None: it opens none): right before it the stream becomes
    # W [x; x0] + step[t], x0 the embedding's output (:class:`PassInputSpec` of the model)
    pass_input: Optional[int] = None


@dataclass(frozen=True)
class BigramEmbeddingSpec:
    """A second table added to the embedding's output: row ``(previous token * mul_prev + token * mul_cur) mod
    buckets`` of a tensor [buckets + 1, hidden]; a sequence's first token takes the last row.  The engine keeps a
    request's last token between steps."""
    buckets: int
    mul_prev: int
    mul_cur: int
    name: str = "bigram"


@dataclass(frozen=True)
class PassInputSpec:
    """What happens to the stream before every pass over a repeated stretch of layers (the first pass too):
    ``x <- W [x; x0] + step[t]``, W [hidden, 2 hidden] with the columns for x first, x0 the embedding's output,
    step [times, hidden], t the number of the pass."""
    times: int
    weight: str = "loop.in"
    step: str = "loop.step"


@dataclass(frozen=True)
class ModelConfig:
    """Everything the engine needs to know about one checkpoint's architecture."""
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_word_embeddings: bool
    max_position_embeddings: int  # 0 = not stated
    weight_prefix: str = "model."
    layer_prefix: str = "model.layers.{i}."
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    # what a decoder may do besides its blocks (all off by default): the embedding rows times a
    # constant, the logits times a constant, and a soft cap  cap * tanh(logits / cap)
    embedding_multiplier: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    # a vector of the position added to the embedding's output (a :class:`SinusoidalEmbeddingSpec`), and the
    # number of copies the stream is kept in (None: one plain stream; a number: every layer is a "hyper" block)
    position_embedding: Any = None
    streams: Optional[int] = None
    # a hashed table of token pairs added to the embedding (:class:`BigramEmbeddingSpec`), and the mixing of the stream
    # with the embedding's output before every pass of a repeated stretch (:class:`PassInputSpec`)
    bigram_embedding: Any = None
    pass_input: Any = None
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    stored_dtype: str = "bfloat16"
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @property
    def num_layers(self) -> int:
        return len(self.layers)
