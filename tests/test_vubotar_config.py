"""The Vubotar design without a GPU: what a configuration turns into (layer descriptions, what each layer asks of the
cache manager, names and shapes of the tensors), refusals, the table of rows per distance, and properties of the plain
implementation itself."""
import copy
import math

import pytest
import torch

import plain_vubotar as plain
import tiny_vubotar as tv
from blackwellllm_b200.config.registry import ConfigError, parse_config
from blackwellllm_b200.weights.random_init import model_param_specs

F64 = torch.float64


def test_registered_under_its_name_and_model_type():
    cfg = parse_config(tv.MIXED)
    assert cfg.architecture == "Vubotar" and not cfg.tie_word_embeddings
    assert (cfg.embedding_multiplier, cfg.logit_scale, cfg.logit_softcap) == (2.0, 0.7, 8.0)
    assert parse_config(tv.TENSOR).logit_softcap is None
    raw = {k: v for k, v in tv.MIXED.items() if k != "architecture"}
    raw["model_type"] = "vubotar"
    assert parse_config(raw).architecture == "Vubotar"


@pytest.mark.parametrize("name", list(tv.CONFIGS))
def test_layers(name):
    raw, _ = tv.CONFIGS[name]
    cfg = parse_config(raw)
    assert len(cfg.layers) == len(raw["layers"]) == len(cfg.schedule)
    for layer, spec in zip(raw["layers"], cfg.layers):
        m, a = layer["mixer"], spec.mixer
        assert spec.block == "parallel" and spec.token_shift is None and spec.layer_scale == ("ls1", "ls2")
        assert spec.mixer_norm.param == "norm1" and spec.ffn_norm.param == "norm2" and spec.mixer_norm.eps == raw["norm"]["eps"]
        if layer["type"] == "attention":
            mask = m.get("mask") or {}
            assert (a.num_heads, a.num_kv_heads, a.head_dim, a.v_head_dim or a.head_dim) == (m["heads"], m["kv_heads"], m["dim"], m["vdim"])
            assert a.window == mask.get("size") and a.keep_first == mask.get("keep_first", 0) and a.softmax_scale == m["scale"]
            assert a.qk_norm == "head" and a.qk_norm_eps == raw["norm"]["eps"] and not a.sink and a.fixed_sink == 0.0
            assert a.score_softcap == m.get("softcap") and a.distance_table_far == m["bias_max"] and a.distance_table_rows == m["bias_rows"]
            assert (a.value_mix == "vmix") == bool(m.get("v_mix")) and not a.output_gate and a.position.kind == "none"
        elif layer["type"] == "latent_attention":
            assert (a.num_heads, a.head_dim, a.rot_dim, a.v_head_dim, a.kv_rank, a.q_rank) == \
                (m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"])
            assert a.position.interleaved and a.position.scaling is None and a.position.theta == m["rot"]["base"]
            assert a.output_gate and not a.sink and a.window is None
        else:
            assert a.kind == "matrix_lstm"
            assert (a.num_heads, a.key_dim, a.value_dim, a.gate_cap, a.norm_eps) == (m["heads"], m["dim"], m["vdim"], m["gate_cap"], raw["norm"]["eps"])
        f = layer["mlp"]
        if f is None:
            assert spec.ffn is None
        else:
            r = spec.ffn
            assert (r.num_experts, r.top_k, r.expert_size) == (f["router"]["experts"], f["router"]["top"], f["expert"]["ff"])
            assert r.score == "sigmoid" and r.renormalize and not r.scale_input and r.choice_bias == "correction" and r.renorm_eps == 1e-20


def test_tensor_names_and_shapes():
    specs = model_param_specs(tv.MIXED)
    W = 64
    want = {"embed": (210, W), "head": (210, W), "final.norm": (W,),
            "l0.norm1": (W,), "l0.norm2": (W,), "l0.ls1": (W,), "l0.ls2": (W,),
            "l0.mix.q": (32, W), "l0.mix.k": (32, W), "l0.mix.v": (48, W), "l0.mix.g": (48, W), "l0.mix.o": (W, 48), "l0.mix.norm": (48,),
            "l0.mix.i": (2, W), "l0.mix.i.b": (2,), "l0.mix.f": (2, W), "l0.mix.f.b": (2,),
            "l0.mlp.router": (4, W), "l0.mlp.correction": (4,), "l0.mlp.e3.gate": (32, W), "l0.mlp.e3.down": (W, 32),
            "l1.mix.q": (192, W), "l1.mix.k": (64, W), "l1.mix.v": (32, W), "l1.mix.o": (W, 96), "l1.mix.q.norm": (32,), "l1.mix.k.norm": (32,),
            "l1.mix.rel": (8, 6), "l1.mix.vmix": (), "l1.ls1": (W,),
            "l2.mix.dq": (24, W), "l2.mix.dq.norm": (24,), "l2.mix.uq": (48, 24), "l2.mix.dkv": (48, W), "l2.mix.dkv.norm": (40,),
            "l2.mix.uk": (32, 40), "l2.mix.uv": (48, 40), "l2.mix.g": (48, W), "l2.mix.o": (W, 48),
            "l3.mix.rel": (32, 4), "l3.mix.vmix": ()}
    for name, shape in want.items():
        assert name in specs and tuple(specs[name].shape) == shape, (name, specs.get(name))
    # a layer without a feed-forward has no expert tensors; its second norm and second scale are taken if stored
    assert not any(k.startswith("l1.mlp.") for k in specs)
    assert specs["l1.norm2"].optional and specs["l1.ls2"].optional and not specs["l1.ls1"].optional
    assert "l2.mix.q" not in specs      # the latent mixer's queries come through dq and uq
    # without the rows stated, the table's first size is left to the stored tensor
    raw = copy.deepcopy(tv.MIXED)
    del raw["layers"][1]["mixer"]["bias_rows"]
    assert tuple(model_param_specs(raw)["l1.mix.rel"].shape) == (-1, 6)


def test_what_the_layers_ask_of_the_cache():
    from blackwellllm_b200.models.decoder import DecoderModel
    from blackwellllm_b200.parts import BuildContext, FixedStateRequest, PagedKVRequest
    model = DecoderModel(parse_config(tv.MIXED), BuildContext(torch.device("cpu"), torch.float32))
    rq = model.cache_requests()
    assert rq[0] == (FixedStateRequest((2, 16, 28), torch.float32), FixedStateRequest((2,), torch.float32))
    assert rq[1] == PagedKVRequest(2, 32, 24, 20) and rq[3] == PagedKVRequest(2, 16, 9, 0)
    assert rq[2] == PagedKVRequest(1, 48, None, 0, single_plane=True)
    model16 = DecoderModel(parse_config(tv.OPEN), BuildContext(torch.device("cpu"), torch.bfloat16))
    # bfloat16 pads head sizes to what the kernels take: 24/40 -> 48, the latent's row of 36 -> 48
    assert model16.cache_requests()[1] == PagedKVRequest(3, 48, None, 0)
    assert model16.cache_requests()[0] == PagedKVRequest(1, 48, None, 0, single_plane=True)


@pytest.mark.parametrize("edit,text", [
    (lambda r: r["layers"][0].__setitem__("type", "conv"), "not a mixer"),
    (lambda r: r["layers"][0]["mlp"].__setitem__("kind", "dense"), "not a feed-forward"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("kv_heads", 4), "multiple"),
    (lambda r: r["layers"][2]["mixer"]["rot"].__setitem__("dims", 6), "rot_dim"),
    (lambda r: r["layers"][2]["mixer"].__setitem__("mask", {"size": 4, "keep_first": 2}), "keeps no first keys"),
    (lambda r: r["layers"][3]["mixer"].__setitem__("vdim", 8), "other kv_heads or vdim"),
    (lambda r: r["layers"][0]["mixer"].__setitem__("gate_cap", 0.0), "> 0"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("softcap", -1.0), "> 0"),
    (lambda r: r["layers"][0]["mlp"]["router"].__setitem__("top", 9), "exceeds"),
    (lambda r: r.pop("embedding"), "embedding"),
    (lambda r: r["norm"].__setitem__("eps", 0), "eps"),
    (lambda r: r.__setitem__("layers", []), "non-empty"),
])
def test_refusals(edit, text):
    raw = copy.deepcopy(tv.MIXED)
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


@pytest.mark.parametrize("rows,far", [(32, 200), (2, 5), (5, 7), (16, 64), (9, 1000), (32, 256), (1, 3), (3, 2), (64, 4096)])
def test_rows_per_distance(rows, far):
    from blackwellllm_b200.kernels import ops
    tab = ops.distance_bucket_table(rows, far).tolist()
    assert tab == [plain.distance_bucket(n, rows, far) for n in range(len(tab))]
    assert tab[-1] == rows - 1 and all(b < rows - 1 for b in tab[:-1]) and tab == sorted(tab)
    assert tab[:rows // 2] == list(range(rows // 2))
    assert all(plain.distance_bucket(n, rows, far) == rows - 1 for n in (len(tab), 2 * len(tab) + 7, 10 ** 6))
    with pytest.raises(Exception):
        ops.distance_bucket_table(8, 4)


# ------------------------------------------------------------------ the plain implementation itself

def test_plain_memory_equals_its_unstabilised_sum():
    """The running maximum only rescales: the output equals the direct sums over all earlier tokens wherever the
    normaliser is above exp(-m)."""
    T, H, dk, dv, cap = 12, 2, 4, 3, 3.0
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, 8, generator=g, dtype=F64)
    w = {n: 0.5 * torch.randn(s, 8, generator=g, dtype=F64) for n, s in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("g", H * dv), ("i", H), ("f", H))}
    w.update({"i.b": torch.zeros(H, dtype=F64), "f.b": torch.ones(H, dtype=F64), "norm": torch.ones(H * dv, dtype=F64), "o": torch.eye(H * dv, dtype=F64)})
    got = plain.mlstm(x, w, {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}, 1e-6)
    q = (x @ w["q"].T).view(T, H, dk) * dk ** -0.5
    k, v = (x @ w["k"].T).view(T, H, dk), (x @ w["v"].T).view(T, H, dv)
    gi = cap * torch.tanh((x @ w["i"].T) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((x @ w["f"].T + 1.0) / cap))
    want = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for h in range(H):
            m, num, den = 0.0, torch.zeros(dv, dtype=F64), 0.0
            mm = [0.0]
            for s in range(t + 1):
                mm.append(max(float(gf[s, h]) + mm[-1], float(gi[s, h])))
            for s in range(t + 1):
                wgt = math.exp(float(gi[s, h]) + float(gf[s + 1:t + 1, h].sum()) - mm[t + 1])
                num += wgt * float(k[s, h] @ q[t, h]) * v[s, h]
                den += wgt * float(k[s, h] @ q[t, h])
            want[t, h] = num / (max(abs(den), math.exp(-mm[t + 1])) + 1e-6)
    want = plain.rms_unit(want, 1e-6).reshape(T, H * dv) * torch.sigmoid(x @ w["g"].T)
    assert float((got - want).abs().max()) < 1e-9


def test_plain_softmax_plus_one_and_window():
    s = torch.tensor([[[0.3, -1.0, 2.0], [0.0, 0.0, 0.0], [5.0, 1.0, -2.0]]], dtype=F64)
    vis = plain.window_mask(3, 2, 1)
    assert vis.tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    assert plain.window_mask(5, 2, 1)[4].tolist() == [True, False, False, True, True]
    p = plain.softmax_plus_one(s, vis)
    assert abs(float(p[0, 0, 0]) - math.exp(0.3) / (1 + math.exp(0.3))) < 1e-12
    assert abs(float(p[0, 1].sum()) - 2 / 3) < 1e-12 and float(p[0, 0, 1]) == 0.0


def test_plain_rotation_is_relative():
    g = torch.Generator().manual_seed(2)
    q, k = torch.randn(9, 6, generator=g, dtype=F64), torch.randn(9, 6, generator=g, dtype=F64)
    q[:] = q[0]
    k[:] = k[0]
    rq, rk = plain.rotate_pairs(q, 100.0, 4), plain.rotate_pairs(k, 100.0, 4)
    s = rq @ rk.T
    assert abs(float(s[5, 3] - s[8, 6])) < 1e-12 and abs(float(s[2, 2] - q[0] @ k[0])) < 1e-12
    assert torch.equal(rq[:, 4:], q[:, 4:])


def test_plain_value_mixing_starts_in_the_second_such_layer():
    raw = tv.MIXED
    tensors = {k: v.double() for k, v in tv.make_tensors(raw, seed=3, dtype=torch.float32).items()}
    ids = tv.prompt(12, raw["vocab"], 1)
    base = plain.forward(raw, tensors, ids)
    moved = dict(tensors)
    moved["l1.mix.vmix"] = tensors["l1.mix.vmix"] + 0.3      # the first such layer's number is not used
    assert torch.equal(plain.forward(raw, moved, ids), base)
    moved = dict(tensors)
    moved["l3.mix.vmix"] = tensors["l3.mix.vmix"] + 0.3
    assert float((plain.forward(raw, moved, ids) - base).abs().max()) > 1e-6
