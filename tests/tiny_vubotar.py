"""Tiny Vubotar configurations for the tests, and their random weights.

They differ from one another in every size and option: the order of the three mixers (each of them first somewhere);
layers without a feed-forward; query heads per kv head (1, 2, 3, 4); key and value sizes that are equal or differ either
way, multiples of 16 and not; windows shorter and longer than a page, windows that differ between layers, no window;
kept first keys (none, fewer than a page, more than a page, more than the window); soft caps small enough to bend every
score and none; distance tables of 2 to 32 rows with a farthest distance inside and far outside the prompts; value
mixing in the first attention layer only, in several, in none, and beginning in a later layer; plain and rotated query
sizes that are equal or differ either way; latents whose cached row is and is not a multiple of 16; matrix memories with
key sizes up to 160 (both register layouts of the scan) and value sizes that leave the last block of columns ragged;
gate caps; experts 2 to 9 with 1 to 4 chosen; embedding and logit scales; logit caps and none.  Table entries,
corrections, layer scales and gate biases are not small, so that one that is left out or read from the wrong place shows.
"""
import json
import os

import torch

from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
from blackwellllm_b200.weights.safetensors_io import write_file


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _attn(heads, kv, dim, vdim, scale, rows, far, cap=None, size=None, keep=None, v_mix=False, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far, "bias_rows": rows}
    if cap is not None:
        m["softcap"] = cap
    if v_mix:
        m["v_mix"] = True
    if size is not None:
        m["mask"] = {"size": size}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _latent(heads, dim, rot_dim, vdim, rank, q_rank, scale, base, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _mlstm(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


# memory first; two attention layers that mix values, windows 24 and 9 with pages of 8, 20 kept keys beside the window of
# 24; a layer without feed-forward; head sizes 32/16 and 16; three and two query heads per kv head
MIXED = {
    "architecture": "Vubotar", "vocab": 210, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "logit_scale": 0.7, "logit_softcap": 8.0,
    "layers": [
        _mlstm(2, 16, 24, 6.0, mlp=_moe(4, 2, 32)),
        _attn(6, 2, 32, 16, 0.15, 8, 30, cap=3.0, size=24, keep=20, v_mix=True, mlp=None),
        _latent(2, 16, 8, 24, 40, 24, 0.2, 10000.0, mlp=_moe(5, 1, 48)),
        _attn(4, 2, 16, 16, 0.25, 32, 600, cap=20.0, size=9, keep=0, v_mix=True, mlp=_moe(3, 3, 16)),
    ],
}
# head sizes the tcgen05 prompt kernel takes (heads of 64, a cached latent row of 128); four query heads per kv head;
# 3 kept keys; a window longer than a page; three attention layers of which the last two mix values (the first does not
# take part); a memory with a key size above 128
TENSOR = {
    "architecture": "Vubotar", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "logit_scale": 1.0,
    "layers": [
        _attn(4, 1, 64, 64, 0.125, 16, 100, cap=None, size=50, keep=3, mlp=_moe(2, 1, 80)),
        _attn(4, 2, 64, 64, 0.1, 6, 40, cap=5.0, v_mix=True, mlp=_moe(8, 4, 32)),
        _latent(2, 48, 64, 40, 64, 32, 0.11, 30000.0, mlp=_moe(4, 2, 64)),
        _mlstm(1, 160, 40, 15.0, mlp=None),
        _attn(2, 2, 64, 64, 0.2, 2, 5, cap=50.0, size=17, keep=40, v_mix=True, mlp=None),
    ],
}
# latent first; sizes that no fast kernel takes (a width that is no multiple of 8, an expert size that is no multiple of
# 16, head sizes 24/40 and 8, a cached row of 36, a memory of 12 x 33); no windows; no value mixing; no caps
OPEN = {
    "architecture": "Vubotar", "vocab": 77, "width": 50, "norm": {"eps": 3e-5}, "embedding": {"scale": 0.5},
    "logit_scale": 2.0,
    "layers": [
        _latent(5, 12, 12, 20, 24, 10, 0.17, 1000.0, mlp=_moe(9, 2, 30)),
        _attn(3, 3, 24, 40, 0.21, 5, 7, mlp=_moe(2, 2, 44)),
        _mlstm(3, 12, 33, 4.0, mlp=_moe(3, 1, 20)),
        _attn(2, 1, 8, 8, 0.35, 12, 1000, size=16, keep=16, mlp=None),
    ],
}
# one layer of each; head size 128; a window of one page exactly with more kept keys than that; a memory of 128 x 64
BROAD = {
    "architecture": "Vubotar", "vocab": 400, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
    "logit_scale": 0.5, "logit_softcap": 25.0,
    "layers": [
        _attn(2, 1, 128, 128, 0.09, 24, 200, cap=10.0, size=64, keep=70, v_mix=True, mlp=_moe(4, 2, 128)),
        _mlstm(2, 128, 64, 9.0, mlp=_moe(4, 3, 64)),
        _latent(2, 64, 64, 128, 192, 96, 0.08, 10000.0, mlp=_moe(6, 2, 96)),
    ],
}

# name -> (config, page size)
CONFIGS = {"mixed": (MIXED, 8), "tensor": (TENSOR, 16), "open": (OPEN, 32), "broad": (BROAD, 64)}


def make_tensors(raw, seed, std=0.08, bias_std=0.3, dtype=torch.bfloat16):
    """Random weights by their checkpoint names, rounded to ``dtype``.  Gains and layer scales 1 + noise; table entries
    N(0, 1); mixing numbers in [0.2, 0.8]; corrections N(0, 0.3); gate biases N(0, 1) and N(2, 1)."""
    specs = model_param_specs(raw)
    tensors = random_tensors(specs, seed, std, bias_std, dtype=torch.float32, skip_optional=False)
    g = torch.Generator().manual_seed(seed + 99)
    for name, spec in specs.items():
        if spec.role == "gain" and spec.init == "ones":
            tensors[name] = 1.0 + 0.4 * torch.randn(spec.shape, generator=g)
        if name.endswith(".mix.rel"):
            tensors[name] = torch.randn(spec.shape, generator=g)
        if name.endswith(".mix.vmix"):
            tensors[name] = 0.2 + 0.6 * torch.rand(spec.shape, generator=g)
        if name.endswith(".mix.i.b"):
            tensors[name] = torch.randn(spec.shape, generator=g)
        if name.endswith(".mix.f.b"):
            tensors[name] = 2.0 + torch.randn(spec.shape, generator=g)
        if name.endswith(".mix.i") or name.endswith(".mix.f"):
            tensors[name] = tensors[name] * 6.0        # gates that move with the token
        if name == "embed":
            tensors[name] = 0.5 * torch.randn(spec.shape, generator=g)
        if name.endswith(".mix.q") or name.endswith(".mix.k") or name.endswith(".mix.uq") or name.endswith(".mix.uk"):
            tensors[name] = tensors[name] * 4.0        # scores that are not all alike
        if name.endswith(".router"):
            tensors[name] = tensors[name] * 4.0        # scores apart from one another
    return {k: v.to(dtype) for k, v in tensors.items()}


def make_folder(name, dtype, root, seed=5):
    raw, _ = CONFIGS[name]
    d = os.path.join(root, f"vubotar-{name}-{dtype}")
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
