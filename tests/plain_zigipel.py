"""Plain implementation of the Zigipel decoder: whole sequences, float64, one function per mechanism, written from the
design's equations.  It shares no code with the package and is the oracle of the Zigipel tests.

Notation: T tokens, width W.  ``tensors`` maps the checkpoint's names to float64 tensors (integer tables stay integers).
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return rms_unit(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous token, token); the extra last row for the first."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets)
    return rows


def embedding(tokens, embed, bigram, cfg):
    x = embed[torch.tensor(tokens)]
    b = (cfg.get("embedding") or {}).get("bigram")
    if b is not None:
        x = x + bigram[torch.tensor(bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"]))]
    return x


def token_shift(h, shift):
    """h_t + (h_{t-1} - h_t) * shift, zeros standing before the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (prev - h) * shift


def sink_softmax(scores, visible, sink):
    """scores [H, T, T], visible [T, T] bool, sink [H]: weights whose denominator also holds exp(sink)."""
    s = scores.masked_fill(~visible, -math.inf)
    m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink.view(-1, 1, 1))
    e = torch.exp(s - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink.view(-1, 1, 1) - m))


def window_mask(T, size, keep_first=0):
    i = torch.arange(T).view(-1, 1)
    j = torch.arange(T).view(1, -1)
    return (j <= i) & ((i - j < size) | (j < keep_first))


def attention(h, t, m, eps):
    """The 'attention' mixer.  t: this mixer's tensors by their short names."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t["q"].T).view(T, H, d)
    k = (h @ t["k"].T).view(T, G, d)
    v = rms_unit((h @ t["v"].T).view(T, G, dv), eps)
    rep = H // G
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    dist = (torch.arange(T).view(-1, 1) - torch.arange(T).view(1, -1)).clamp(min=0).to(F64)
    scores = scores - t["r1"].view(H, 1, 1) * torch.log(1.0 + t["r2"].view(H, 1, 1) * dist)
    mask = m.get("mask") or {}
    w = sink_softmax(scores, window_mask(T, mask.get("size", T), mask.get("keep_first", 0)), t["sink"])
    o = torch.einsum("hij,jhd->ihd", w, v)
    o = o * torch.sigmoid(h @ t["g"].T).view(T, H, 1)
    return o.reshape(T, H * dv) @ t["o"].T


def yarn_frequencies(rot):
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    mag = 1.0
    if sc:
        def dim_of(turns):
            return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(dim_of(sc["fast"])), 0)
        hi = min(math.ceil(dim_of(sc["slow"])), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    return f, mag


def rotate_half(x, positions, rot):
    """x [T, heads, n]: the first rot.dims channels turn, channel i with channel i + dims / 2."""
    dims = rot["dims"]
    f, mag = yarn_frequencies(rot)
    a = positions.to(F64).view(-1, 1, 1) * f.view(1, 1, -1)
    c, s = torch.cos(a) * mag, torch.sin(a) * mag
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def latent_attention(h, t, m, eps):
    """The 'latent_attention' mixer: keys and values are made from a small latent vector per token."""
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ t["q"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_half(q[..., d:], pos, m["rot"])
    dkv = h @ t["dkv"].T
    c = rms_norm(dkv[:, :rank], t["dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, rank:].view(T, 1, dr), pos, m["rot"])
    k_plain = (c @ t["uk"].T).view(T, H, d)
    v = (c @ t["uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    mask = m.get("mask") or {}
    w = sink_softmax(scores, window_mask(T, mask.get("size", T)), t["sink"])
    o = torch.einsum("hij,jhd->ihd", w, v)
    return o.reshape(T, H * dv) @ t["o"].T


def dense_mlp(h, t):
    g = h @ t["gate"].T + t["gate.b"]
    u = h @ t["up"].T + t["up.b"]
    return (gelu_tanh(g) * u) @ t["down"].T + t["down.b"]


def layer_order(cfg):
    """The runs of layers as (layer, number of the pass it opens or None)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for p in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, p if i == loop["start"] else None))
    return order + [(i, None) for i in range(loop["stop"], n)]


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence; ``streams``: a list that receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = embedding(tokens, tensors["embed"], tensors.get("bigram"), cfg)
    x0 = x
    for i, opens in layer_order(cfg):
        if opens is not None:
            x = torch.cat([x, x0], dim=1) @ tensors["loop.in"].T + tensors["loop.step"][opens]
        layer = cfg["layers"][i]
        t = sub(tensors, f"l{i}.")
        h = rms_norm(x, t["norm1"], eps)
        hs = token_shift(h, t["shift"])
        mix = {"attention": attention, "latent_attention": latent_attention}[layer["type"]]
        y = mix(hs, sub(t, "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + dense_mlp(h, sub(t, "mlp."))
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, tensors["final.norm"], eps)
    return (x @ tensors["head"].T) * cfg.get("logit_scale", 1.0)
