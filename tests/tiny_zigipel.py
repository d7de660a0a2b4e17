"""Tiny Zigipel configurations for the tests, and their random weights.

They differ from one another in every size and option: where the repeated stretch starts and ends (the whole model,
the middle, none at all) and how often it runs (once, twice, three times); the order of the two mixers; layers
without a feed-forward; query heads per kv head (1, 2, 3, 4); key and value sizes that are equal or differ either
way; plain and rotated query sizes that are equal or differ either way; latent sizes whose cached row is and is not
a multiple of 16; windows shorter and longer than a page, windows that differ between layers, no window; kept first
keys (none, fewer than a page, more than a page, more than the window); YaRN constants (none, ramps that cover all
or part of the pairs); score scales, logit scales, eps; hash constants of the second embedding table (also one
bucket, and no table at all).  Sinks, distance constants, shifts and step vectors are not small, so that one that is
left out or read from the wrong place shows.
"""
import json
import os

import torch

from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
from blackwellllm_b200.weights.safetensors_io import write_file


def _attn(heads, kv, dim, vdim, scale, size=None, keep=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    return {"type": "attention", "mixer": m, "mlp": None if mlp is None else {"kind": "dense", "ff": mlp}}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base, size=None, scaling=None, mlp=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}
    if size is not None:
        m["mask"] = {"size": size}
    return {"type": "latent_attention", "mixer": m, "mlp": None if mlp is None else {"kind": "dense", "ff": mlp}}


# the middle two of four layers run three times; latent first; a layer without feed-forward; windows 24 and 9 with
# pages of 8; 20 kept keys (more than two pages, more than the window of 9 would be: here beside a window of 24)
MIDDLE = {
    "architecture": "Zigipel", "vocab": 210, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
    "embedding": {"bigram": {"buckets": 97, "mul_prev": 13, "mul_cur": 5}},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _latent(2, 16, 8, 24, 40, 0.2, 10000.0, size=9, scaling=(4.0, 64, 8.0, 2.0), mlp=96),
        _attn(4, 2, 32, 16, 0.15, size=24, keep=20, mlp=None),
        _latent(3, 8, 16, 8, 24, 0.3, 500.0, size=30, scaling=None, mlp=48),
        _attn(3, 1, 16, 16, 0.25, size=5, keep=0, mlp=80),
    ],
}
# the whole model runs twice; head sizes the tcgen05 prompt kernel takes (a cached row of 128, heads of 64); four
# query heads per kv head; 3 kept keys; windows longer than a page; one bucket
WHOLE = {
    "architecture": "Zigipel", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
    "embedding": {"bigram": {"buckets": 1, "mul_prev": 3, "mul_cur": 1}},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        _attn(4, 1, 64, 64, 0.125, size=50, keep=3, mlp=80),
        _latent(2, 48, 64, 40, 64, 0.11, 50000.0, size=33, scaling=(2.0, 128, 16.0, 1.0), mlp=64),
    ],
}
# no repeated stretch, no second table, no windows: every key stays visible; value size above key size; sizes that no
# fast kernel takes (a width that is no multiple of 8, a feed-forward size that is no multiple of 16, a cached row of 36)
OPEN = {
    "architecture": "Zigipel", "vocab": 77, "width": 50, "norm": {"eps": 3e-5}, "logit_scale": 2.0,
    "layers": [
        _attn(3, 3, 24, 40, 0.21, mlp=30),
        _latent(5, 12, 12, 20, 24, 0.17, 1000.0, scaling=(8.0, 32, 4.0, 0.5), mlp=None),
        _attn(2, 1, 8, 8, 0.35, size=16, keep=16, mlp=44),
    ],
}
# one layer of each, the stretch (the last layer alone) once; head size 128; a window of one page exactly
BROAD = {
    "architecture": "Zigipel", "vocab": 400, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
    "embedding": {"bigram": {"buckets": 1000, "mul_prev": 1, "mul_cur": 1000003}},
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        _attn(2, 1, 128, 128, 0.09, size=64, keep=70, mlp=256),
        _latent(2, 64, 64, 128, 192, 0.08, 10000.0, size=64, scaling=(3.0, 40, 6.0, 3.0), mlp=128),
    ],
}

# name -> (config, page size)
CONFIGS = {"middle": (MIDDLE, 8), "whole": (WHOLE, 16), "open": (OPEN, 32), "broad": (BROAD, 64)}


def make_tensors(raw, seed, std=0.08, bias_std=0.3, dtype=torch.bfloat16):
    """Random weights by their checkpoint names, rounded to ``dtype``.  Gains 1 + noise; sinks around the scores'
    size; r1 in [0, 2], r2 in (0, 0.5]; shifts in [0, 1]; step vectors and biases N(0, 0.3)."""
    specs = model_param_specs(raw)
    tensors = random_tensors(specs, seed, std, bias_std, dtype=torch.float32, skip_optional=False)
    g = torch.Generator().manual_seed(seed + 99)
    for name, spec in specs.items():
        if spec.role == "gain" and spec.init == "ones":
            tensors[name] = 1.0 + 0.4 * torch.randn(spec.shape, generator=g)
        if name.endswith(".mix.r1"):
            tensors[name] = 2.0 * torch.rand(spec.shape, generator=g)
        if name.endswith(".mix.r2"):
            tensors[name] = 0.02 + 0.48 * torch.rand(spec.shape, generator=g)
        if name.endswith(".shift"):
            tensors[name] = torch.rand(spec.shape, generator=g)
        if name.endswith(".mix.sink"):
            tensors[name] = torch.randn(spec.shape, generator=g)
        if name in ("embed", "bigram"):
            tensors[name] = 0.5 * torch.randn(spec.shape, generator=g)
        if name.endswith(".mix.q") or name.endswith(".mix.k"):
            tensors[name] = tensors[name] * 4.0        # scores that are not all alike
    return {k: v.to(dtype) for k, v in tensors.items()}


def make_folder(name, dtype, root, seed=5):
    raw, _ = CONFIGS[name]
    d = os.path.join(root, f"zigipel-{name}-{dtype}")
    if not os.path.isdir(d):
        os.makedirs(d)
        tensors = make_tensors(raw, seed, dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(raw, f)
        write_file(os.path.join(d, "model.safetensors"), tensors, metadata={"format": "pt"})
    return d


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
