"""Plain implementation of the Vubotar decoder: whole sequences, float64, one function per mechanism, written from the
design's equations.  It shares no code with the package and is the oracle of the Vubotar tests.

Notation: T tokens, width W.  ``tensors`` maps the checkpoint's names to float64 tensors.
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return rms_unit(x, eps) * gain


def soft_cap(x, cap):
    return cap * torch.tanh(x / cap)


def distance_bucket(n, rows, far):
    """The row of a distance table for the distance n >= 0: the first rows / 2 distances have a row each, the rest share
    rows on a logarithmic scale that reaches the last row at distance ``far``."""
    half = rows // 2
    if n < half:
        return n
    if half == 0:
        return 0
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(T, table, far):
    """[heads, T, T]: entry (h, i, j) = table[bucket(i - j), h] for j <= i, 0 elsewhere."""
    rows, heads = table.shape
    out = torch.zeros(heads, T, T, dtype=F64)
    for d in range(T):
        row = table[distance_bucket(d, rows, far)]
        for i in range(d, T):
            out[:, i, i - d] = row
    return out


def window_mask(T, size=None, keep_first=0):
    i = torch.arange(T).view(-1, 1)
    j = torch.arange(T).view(1, -1)
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def softmax_plus_one(scores, visible):
    """Weights exp(s_j) / (1 + sum exp(s_j)) over the visible keys: a sink of score 0 that has no value."""
    s = scores.masked_fill(~visible, -math.inf)
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(-m))


def plain_softmax(scores, visible):
    return torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)


def rotate_pairs(x, base, dims):
    """x [T, ..., D]: channels (2i, 2i + 1), i < dims / 2, of the token at position p are turned by p * base^(-2i/dims);
    channels from ``dims`` on pass."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.arange(T, dtype=F64).view(-1, 1) * base ** (-2.0 * i / dims)          # [T, dims / 2]
    shape = (T,) + (1,) * (x.dim() - 2) + (dims // 2,)
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def attention(h, w, m, eps, v_first):
    """The 'attention' mixer.  w: its tensors by short name; m: its config entry.  Returns (output, this layer's values
    before any mixing [T, G, vdim])."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = (h @ w["v"].T).view(T, G, dv)
    raw_v = v
    q = rms_norm(q, w["q.norm"], eps)
    k = rms_norm(k, w["k.norm"], eps)
    if m.get("v_mix") and v_first is not None:
        lam = w["vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    if m.get("softcap"):
        s = soft_cap(s, m["softcap"])
    s = s + distance_bias(T, w["rel"], m["bias_max"])
    mask = m.get("mask") or {}
    vis = window_mask(T, mask.get("size"), mask.get("keep_first", 0))
    p = softmax_plus_one(s, vis)
    o = torch.einsum("hij,jhd->ihd", p, vv).reshape(T, H * dv)
    return o @ w["o"].T, raw_v


def latent_attention(h, w, m, eps):
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, d + dr)
    kv = h @ w["dkv"].T
    c = rms_norm(kv[:, :rank], w["dkv.norm"], eps)
    k_rot = kv[:, rank:]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rotate_pairs(q[..., d:], base, dims)
    k_rot = rotate_pairs(k_rot, base, dims)
    k_plain = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    p = plain_softmax(s, window_mask(T))
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def log_sigmoid(z):
    return torch.minimum(z, torch.zeros_like(z)) - torch.log1p(torch.exp(-z.abs()))


def mlstm(h, w, m, eps):
    """Matrix memory with exponential gates, token by token from a zero state."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                  # [T, H] log input gate
    gf = log_sigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))    # [T, H] log forget gate
    S = torch.zeros(H, d, dv, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    mm = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mm, gi[t])
        a = torch.exp(gf[t] + mm - m_new)
        b = torch.exp(gi[t] - m_new)
        S = a.view(H, 1, 1) * S + b.view(H, 1, 1) * k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        n = a.view(H, 1) * n + b.view(H, 1) * k[t]
        mm = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mm)) + 1e-6
        out[t] = num / den.view(H, 1)
    o = rms_unit(out, eps).reshape(T, H * dv) * w["norm"]
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def routed_ffn(h, w, f):
    """Mixture of experts: sigmoid scores, the choice by score + correction, weights the chosen scores over their sum."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ w["router"].T)
    choice = s + w["correction"]
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(choice[t, e]), e))[:top]
        total = sum(s[t, e] for e in order) + 1e-20
        for e in order:
            g = h[t] @ w[f"e{e}.gate"].T
            u = h[t] @ w[f"e{e}.up"].T
            out[t] += (s[t, e] / total) * ((g * torch.sigmoid(g) * u) @ w[f"e{e}.down"].T)
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence.  ``streams``: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = tensors["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h1 = rms_norm(x, tensors[p + "norm1"], eps)
        w, m = sub(tensors, p + "mix."), layer["mixer"]
        if layer["type"] == "attention":
            y, raw_v = attention(h1, w, m, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = raw_v
        elif layer["type"] == "latent_attention":
            y = latent_attention(h1, w, m, eps)
        elif layer["type"] == "mlstm":
            y = mlstm(h1, w, m, eps)
        else:
            raise ValueError(layer["type"])
        y = y * tensors[p + "ls1"]
        if layer.get("mlp") is not None:
            h2 = rms_norm(x, tensors[p + "norm2"], eps)
            y = y + routed_ffn(h2, sub(tensors, p + "mlp."), layer["mlp"]) * tensors[p + "ls2"]
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, tensors["final.norm"], eps)
    logits = x @ tensors["head"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return soft_cap(logits, cap) if cap else logits
