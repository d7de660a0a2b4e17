"""The Zigipel design without a GPU: what a configuration turns into (layer descriptions, the order of layer runs with
every form of the repeated stretch, what each run asks of the cache manager, names and shapes of the tensors),
refusals, the cache manager's handling of kept first keys, and properties of the plain implementation itself."""
import copy
import math

import pytest
import torch

import plain_zigipel as plain
import tiny_zigipel as tz
from blackwellllm_b200.config.registry import ConfigError, parse_config
from blackwellllm_b200.weights.random_init import model_param_specs


def test_registered_under_its_name_and_model_type():
    cfg = parse_config(tz.MIDDLE)
    assert cfg.architecture == "Zigipel" and not cfg.tie_word_embeddings and cfg.logit_scale == 0.7
    raw = {k: v for k, v in tz.MIDDLE.items() if k != "architecture"}
    raw["model_type"] = "zigipel"
    assert parse_config(raw).architecture == "Zigipel"


@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_layers(name):
    raw, _ = tz.CONFIGS[name]
    cfg = parse_config(raw)
    assert len(cfg.layers) == len(raw["layers"])
    for layer, spec in zip(raw["layers"], cfg.layers):
        m, a = layer["mixer"], spec.mixer
        assert spec.block == "parallel" and spec.token_shift == "shift" and spec.ffn_norm is None
        assert spec.mixer_norm.eps == raw["norm"]["eps"] and spec.mixer_norm.param == "norm1"
        mask = m.get("mask") or {}
        assert a.window == mask.get("size") and a.softmax_scale == m["scale"] and a.sink
        if layer["type"] == "attention":
            assert (a.num_heads, a.num_kv_heads, a.head_dim) == (m["heads"], m["kv_heads"], m["dim"])
            assert (a.v_head_dim or a.head_dim) == m["vdim"]
            assert a.output_gate and a.gate_per_head and a.distance_bias and not a.qkv_bias
            assert a.v_norm_eps == raw["norm"]["eps"] and a.keep_first == mask.get("keep_first", 0)
        else:
            assert a.kind == "latent_attention"
            assert (a.num_heads, a.head_dim, a.rot_dim, a.v_head_dim, a.kv_rank) == (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"])
            assert a.norm_eps == raw["norm"]["eps"]
            assert a.position.theta == m["rot"]["base"] and a.position.rotary_dim == m["rot_dim"] and not a.position.interleaved
            sc = m["rot"].get("scaling")
            assert (a.position.scaling is None) == (sc is None)
            if sc:
                s = a.position.scaling
                assert (s.factor, s.original, s.fast, s.slow) == (sc["factor"], sc["original"], sc["fast"], sc["slow"])
        f = layer["mlp"]
        if f is None:
            assert spec.ffn is None
        else:
            assert spec.ffn.intermediate_size == f["ff"] and spec.ffn.activation == "gelu_tanh"
            assert spec.ffn.bias_names == ("gate.b", "up.b", "down.b")
    b = (raw.get("embedding") or {}).get("bigram")
    assert (cfg.bigram_embedding is None) == (b is None)
    if b:
        e = cfg.bigram_embedding
        assert (e.buckets, e.mul_prev, e.mul_cur) == (b["buckets"], b["mul_prev"], b["mul_cur"])


@pytest.mark.parametrize("n,loop,want", [
    (4, {"start": 1, "stop": 3, "times": 3}, [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]),
    (2, {"start": 0, "stop": 2, "times": 2}, [(0, 0), (1, None), (0, 1), (1, None)]),
    (3, {"start": 2, "stop": 3, "times": 1}, [(0, None), (1, None), (2, 0)]),
    (3, {"start": 0, "stop": 1, "times": 2}, [(0, 0), (0, 1), (1, None), (2, None)]),
    (2, None, [(0, None), (1, None)]),
])
def test_order_of_layer_runs(n, loop, want):
    raw = copy.deepcopy(tz.MIDDLE)
    raw["layers"] = raw["layers"][:n]
    if loop is None:
        del raw["loop"]
    else:
        raw["loop"] = loop
    cfg = parse_config(raw)
    assert [(e.layer, e.pass_input) for e in cfg.schedule] == want
    assert all(e.cache_of is None and not e.add_embedding for e in cfg.schedule)      # every run owns its cache
    assert (cfg.pass_input is None) == (loop is None)
    if loop:
        assert cfg.pass_input.times == loop["times"]
    assert plain.layer_order(raw) == want


def test_names_and_shapes():
    specs = model_param_specs(tz.MIDDLE)
    shapes = {k: tuple(v.shape) for k, v in specs.items()}
    assert all(not v.optional for v in specs.values())
    assert shapes["embed"] == (210, 64) and shapes["bigram"] == (98, 64) and shapes["head"] == (210, 64)
    assert shapes["loop.in"] == (64, 128) and shapes["loop.step"] == (3, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.norm1"] == (64,) and shapes["l0.shift"] == (64,)
    assert shapes["l0.mix.q"] == (2 * (16 + 8), 64) and shapes["l0.mix.dkv"] == (40 + 8, 64) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (2 * 16, 40) and shapes["l0.mix.uv"] == (2 * 24, 40) and shapes["l0.mix.o"] == (64, 48)
    assert shapes["l0.mix.sink"] == (2,)
    assert shapes["l1.mix.q"] == (128, 64) and shapes["l1.mix.k"] == (64, 64) and shapes["l1.mix.v"] == (32, 64)
    assert shapes["l1.mix.g"] == (4, 64) and shapes["l1.mix.o"] == (64, 64)
    assert shapes["l1.mix.r1"] == shapes["l1.mix.r2"] == shapes["l1.mix.sink"] == (4,)
    assert "l1.mlp.gate" not in shapes and "l1.norm2" not in shapes
    assert shapes["l0.mlp.gate"] == (96, 64) and shapes["l0.mlp.gate.b"] == (96,) and shapes["l0.mlp.down.b"] == (64,)
    assert len(shapes) == 4 + 2 + (2 + 7 + 6) + (2 + 8) + (2 + 7 + 6) + (2 + 8 + 6)
    bare = model_param_specs(tz.OPEN)
    assert "bigram" not in bare and "loop.in" not in bare and "loop.step" not in bare


def test_what_each_run_asks_of_the_cache_manager():
    from blackwellllm_b200.models.decoder import DecoderModel
    from blackwellllm_b200.parts import BuildContext, FixedStateRequest, PagedKVRequest
    model = DecoderModel(parse_config(tz.MIDDLE), BuildContext(torch.device("cpu"), torch.float32))
    rq = model.cache_requests()
    assert len(rq) == 8 + 1 and rq[-1] == FixedStateRequest((1,), torch.int32)          # the previous token
    for pos, e in enumerate(model.config.schedule):
        pages, state = rq[pos]
        assert state == FixedStateRequest((64,), torch.float32)                         # the previous token's normed row
        m = tz.MIDDLE["layers"][e.layer]["mixer"]
        if tz.MIDDLE["layers"][e.layer]["type"] == "attention":
            assert pages == PagedKVRequest(m["kv_heads"], max(m["dim"], m["vdim"]), m["mask"]["size"], m["mask"].get("keep_first", 0))
        else:
            assert pages == PagedKVRequest(1, m["kv_rank"] + m["rot_dim"], m["mask"]["size"], 0, single_plane=True)
    # no second table: no state of the model's own
    assert len(DecoderModel(parse_config(tz.OPEN), BuildContext(torch.device("cpu"), torch.float32)).cache_requests()) == 3


def test_kept_first_pages_stay_with_the_request():
    """A window gives back the pages it has passed, but never the pages that hold kept first keys; a state per run
    and one of the model's own are handed out with the slot."""
    from blackwellllm_b200.cache.manager import CacheManager
    from blackwellllm_b200.parts import FixedStateRequest, PagedKVRequest
    page = 8
    rqs = [(PagedKVRequest(2, 16, 24, 20), FixedStateRequest((4,))), (PagedKVRequest(1, 48, 9, 0, single_plane=True), FixedStateRequest((4,))),
           FixedStateRequest((1,), torch.int32)]
    cm = CacheManager(rqs, page, 40, 2, dtype=torch.float32, device=None)
    assert len(cm.groups) == 2 and isinstance(cm.views[0], tuple) and len(cm.views[0]) == 2
    cm.add_request("a")
    cm.append("a", 100)
    cm.release_passed("a")
    kept, plain_window = cm.block_table("a", 0), cm.block_table("a", 1)
    # the next query sits at position 100: a window of 24 needs keys from 77 on (block 9); 20 kept keys are blocks 0..2
    assert [p >= 0 for p in kept] == [True] * 3 + [False] * 6 + [True] * 4
    assert [p >= 0 for p in plain_window] == [False] * 11 + [True] * 2                   # keys from 92 on: block 11
    cm.check_invariants()
    cm.append("a", 60)
    cm.release_passed("a")
    assert [p >= 0 for p in cm.block_table("a", 0)][:3] == [True] * 3
    free_before = cm.free_pages()
    cm.free_request("a")
    assert cm.free_pages() == [40, 40] and free_before != [40, 40]
    cm.check_invariants()


@pytest.mark.parametrize("change,needle", [
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][0]["mlp"].update(kind="moe"), "not a feed-forward"),
    (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=6), "rot_dim"),
    (lambda r: r["layers"][0]["mixer"].update(mask={"size": 9, "keep_first": 2}), "keeps no first keys"),
    (lambda r: r["layers"][1]["mixer"]["mask"].update(keep_first=-1), "non-negative"),
    (lambda r: r["loop"].update(stop=5), "loop"),
    (lambda r: r["loop"].update(times=0), "loop"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].update(eps=0), "eps"),
    (lambda r: r["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
])
def test_refusals(change, needle):
    raw = copy.deepcopy(tz.MIDDLE)
    change(raw)
    with pytest.raises(ConfigError, match=needle):
        parse_config(raw)


# ------------------------------------------------------------------ the plain implementation itself

def test_plain_hash_rows():
    assert plain.bigram_rows([5, 7, 7, 0], 97, 13, 5) == [97, (5 * 13 + 7 * 5) % 97, (7 * 13 + 7 * 5) % 97, (7 * 13) % 97]
    assert plain.bigram_rows([3, 4], 1, 9, 9) == [1, 0]


def test_plain_window_and_kept_keys():
    m = plain.window_mask(12, 4, 2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert m[3].tolist() == [True] * 4 + [False] * 8 and m[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert plain.window_mask(6, 2)[5].tolist() == [False] * 4 + [True] * 2
    assert plain.window_mask(5, 5).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()


def test_plain_sink_takes_weight_from_every_row():
    s = torch.zeros(1, 2, 2, dtype=torch.float64)
    vis = torch.tril(torch.ones(2, 2)).bool()
    w = plain.sink_softmax(s, vis, torch.tensor([0.0], dtype=torch.float64))
    assert torch.allclose(w[0, 0], torch.tensor([0.5, 0.0], dtype=torch.float64))
    assert torch.allclose(w[0, 1], torch.tensor([1 / 3, 1 / 3], dtype=torch.float64))
    w = plain.sink_softmax(s, vis, torch.tensor([-80.0], dtype=torch.float64))
    assert torch.allclose(w[0].sum(-1), torch.ones(2, dtype=torch.float64))


def test_plain_token_shift():
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, 5.0]], dtype=torch.float64)
    got = plain.token_shift(h, torch.tensor([0.0, 1.0], dtype=torch.float64))
    assert got.tolist() == [[1.0, 0.0], [3.0, 2.0], [5.0, 6.0]]


def test_plain_yarn_frequencies():
    rot = {"base": 10000.0, "dims": 8}
    f, mag = plain.yarn_frequencies(rot)
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=torch.float64))
    rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}
    f2, mag = plain.yarn_frequencies(rot)
    assert math.isclose(mag, 0.1 * math.log(4.0) + 1.0)
    # dim(8) = 8 ln(64 / 16 pi) / (2 ln 1e4) = 0.10: lo = 0; dim(2) = 0.71: hi = 1; pair 0 keeps its frequency, the rest is divided
    assert math.isclose(float(f2[0]), 1.0) and torch.allclose(f2[1:], f[1:] / 4.0)


def test_plain_rotation_keeps_lengths_and_relative_angles():
    rot = {"base": 100.0, "dims": 4}
    x = torch.randn(1, 1, 6, dtype=torch.float64, generator=torch.Generator().manual_seed(0)).expand(5, 1, 6)
    y = plain.rotate_half(x, torch.arange(5), rot)
    assert torch.allclose(y[..., 4:], x[..., 4:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[..., :4].norm(dim=-1), x[..., :4].norm(dim=-1))
    # q at position 3 against k at position 1 equals q at 4 against k at 2
    assert torch.allclose((y[3] * y[1]).sum(), (y[4] * y[2]).sum())


def test_plain_latent_scores_equal_the_absorbed_form():
    """(q_plain . W_uk c) equals (W_uk^T q_plain) . c: the form the engine caches."""
    g = torch.Generator().manual_seed(1)
    q, c, w = (torch.randn(*s, dtype=torch.float64, generator=g) for s in ((3, 5), (4, 7), (5, 7)))
    assert torch.allclose(q @ (c @ w.T).T, (q @ w) @ c.T)


def test_plain_model_looks_back_no_further_than_it_may():
    """With windows everywhere and no kept keys, a token far back changes nothing; with kept first keys it does."""
    raw = copy.deepcopy(tz.MIDDLE)
    raw["layers"][1]["mixer"]["mask"]["keep_first"] = 0
    W = {k: v.double() for k, v in tz.make_tensors(raw, 3, dtype=torch.float32).items()}
    ids = tz.prompt(260, raw["vocab"], 1)
    other = list(ids)
    other[2] = (other[2] + 1) % raw["vocab"]
    a, b = plain.forward(raw, W, ids), plain.forward(raw, W, other)
    # a run reaches back its window (the shift's one token included): 9 + 3 * (24 + 30) + 5 = 176 tokens, and one for the hash
    assert float((a[-1] - b[-1]).abs().max()) < 1e-12 and float((a[3] - b[3]).abs().max()) > 1e-6
    a, b = plain.forward(tz.MIDDLE, W, ids), plain.forward(tz.MIDDLE, W, other)
    assert float((a[-1] - b[-1]).abs().max()) > 1e-9
