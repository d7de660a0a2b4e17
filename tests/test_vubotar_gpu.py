"""The Vubotar design on the GPU against its plain implementation (tests/plain_vubotar.py): each mechanism's kernels
alone, then whole models through Engine.step in every way of cutting and batching, through the scheduler's
generate(), the command line and bin/trace_run."""
import math

import pytest
import torch

import plain_vubotar as plain
import replay
import tiny_vubotar as tv

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
# of the largest logit of the compared request.  The sharp comparison is the float32 one; every bfloat16 kernel has
# its own tight test below.
TOL = {"float32": 1e-4, "bfloat16": 5e-2}
F64 = torch.float64


@pytest.fixture(scope="module")
def ops():
    from blackwellllm_b200.kernels import ops as o
    return o


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def d(t):
    return t.to(DEV).contiguous()


class Rows:
    """A step's batch as the row kernels see it: requests' portions, their positions and state slots."""

    def __init__(self, q_lens, starts, slots):
        from test_kernels_gpu import FakeBatch
        fb = FakeBatch(q_lens, [s + q for s, q in zip(starts, q_lens)])
        self.__dict__.update(fb.__dict__)
        self.state_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)


# =============================================================================== mechanisms alone

@pytest.mark.parametrize("T,H", [(1, 64), (7, 50), (300, 2048)])
def test_layer_scale_sum(ops, T, H):
    x, a, b = rnd(T, H, seed=1), rnd(T, H, seed=2), rnd(T, H, seed=3)
    ga, gb = rnd(H, seed=4), rnd(H, seed=5)
    got = ops.scale_add(d(x.clone()), d(a), d(ga), d(b), d(gb)).cpu()
    assert float((got.double() - (x.double() + (a.double() * ga.double() + b.double() * gb.double()))).abs().max()) < 1e-5
    got = ops.scale_add(d(x.clone()), d(a), d(ga)).cpu()
    assert float((got.double() - (x.double() + a.double() * ga.double())).abs().max()) < 1e-5


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H", [(1, 64), (7, 50), (130, 2048), (3, 4100)])
def test_layer_scale_sum_and_both_norms_in_one_pass(ops, out_dtype, T, H):
    x, a, b = rnd(T, H, seed=1), rnd(T, H, seed=2), rnd(T, H, seed=3)
    ga, gb, w1, w2 = rnd(H, seed=4), rnd(H, seed=5), 1.0 + 0.3 * rnd(H, seed=6), 1.0 + 0.3 * rnd(H, seed=7)
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    for pending, two in ((True, True), (True, False), (False, True), ("one", True)):
        xs = d(x.clone())
        want_x = x.double()
        pend = None
        if pending == "one":
            pend, want_x = (d(a), d(ga), None, None), want_x + a.double() * ga.double()
        elif pending:
            pend, want_x = (d(a), d(ga), d(b), d(gb)), want_x + (a.double() * ga.double() + b.double() * gb.double())
        h1, h2 = ops.scale_add_norm2(xs, pend, d(w1), 1e-5, d(w2) if two else None, 1e-3, out_dtype)
        assert float((xs.double().cpu() - want_x).abs().max()) < 1e-5
        assert float((h1.double().cpu() - plain.rms_norm(want_x, w1.double(), 1e-5)).abs().max()) < tol * 4
        assert (h2 is None) == (not two)
        if two:
            assert float((h2.double().cpu() - plain.rms_norm(want_x, w2.double(), 1e-3)).abs().max()) < tol * 4
        if pending is True and T > 1:       # chosen rows: the stream stays, the rows' norms are those of the new rows
            xs, pick = d(x.clone()), torch.tensor([T - 1, 0], dtype=torch.int32)
            h1, _ = ops.scale_add_norm2(xs, pend, d(w1), 1e-5, None, 0.0, out_dtype, rows=d(pick))
            assert torch.equal(xs.cpu(), x) and h1.shape == (2, H)
            assert float((h1.double().cpu() - plain.rms_norm(want_x[[T - 1, 0]], w1.double(), 1e-5)).abs().max()) < tol * 4


@pytest.mark.parametrize("T,H,ld", [(5, 24, 100), (40, 128, 131), (3, 64, 64)])
def test_norm_of_a_range_of_columns(ops, T, H, ld):
    wide = rnd(T, ld, seed=7)
    gain = 1.0 + 0.3 * rnd(H, seed=8)
    got = ops.rmsnorm(d(wide)[:, :H], d(gain), 1e-5, torch.float32).cpu()
    want = plain.rms_norm(wide[:, :H].double(), gain.double(), 1e-5)
    assert float((got.double() - want).abs().max()) < 1e-5


@pytest.mark.parametrize("rows,far", [(32, 200), (2, 5), (5, 7), (16, 64), (9, 1000), (32, 256), (1, 3), (3, 2)])
def test_distance_rows(ops, rows, far):
    """The table of rows per distance equals the bucket function, ends at the first distance that takes the last row,
    and every larger distance takes the last row too."""
    tab = ops.distance_bucket_table(rows, far).tolist()
    for n, b in enumerate(tab):
        assert b == plain.distance_bucket(n, rows, far), (n, b)
    assert tab[-1] == rows - 1 and (len(tab) == 1 or tab[-2] < rows - 1)
    for n in (len(tab), len(tab) + 1, 10 * len(tab) + 1000):
        assert plain.distance_bucket(n, rows, far) == rows - 1


def _capped_attention(q, k, v, scale, cap, table, far, window, keep, sink=True):
    """q [L, nh, hd], k / v [L, nkv, hd] float64 -> [L, nh, hd]: the plain implementation's pieces."""
    L, nh, _ = q.shape
    rep = nh // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if cap:
        s = plain.soft_cap(s, cap)
    if table is not None:
        s = s + plain.distance_bias(L, table, far)
    vis = plain.window_mask(L, window, keep)
    w = plain.softmax_plus_one(s, vis) if sink else plain.plain_softmax(s, vis)
    return torch.einsum("hij,jhd->ihd", w, vv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page,window,keep,rows,far,cap",
                         [(4, 2, 80, 8, 44, 7, 24, 300, 40.0), (2, 2, 64, 16, 100, 70, 8, 30, 2.0), (8, 2, 128, 16, 33, 1, 6, 1000, None),
                          (6, 3, 96, 16, 64, 64, 2, 5, 1.0), (3, 1, 16, 32, 7, 20, 32, 600, 5.0), (4, 1, 32, 16, None, 0, 16, 100, 3.0),
                          (4, 4, 64, 64, 130, 0, 5, 7, 0.5), (20, 1, 32, 16, 40, 5, 12, 50, 4.0), (4, 1, 256, 16, 70, 130, 32, 64, 10.0),
                          (16, 4, 128, 16, 128, 64, 10, 900, 8.0), (6, 2, 48, 16, 52, 3, 20, 150, 25.0)])
def test_attention_with_soft_cap_distance_table_and_unit_sink(ops, dtype, nh, nkv, hd, page, window, keep, rows, far, cap):
    """Prompt portions from position 0 and continued, decode tokens with few and many keys, a two-token portion; the
    window's and the kept keys' edges fall inside tiles and pages; distances inside and far beyond the table."""
    from test_kernels_gpu import ATT_TOL, FakeBatch, paged_case
    q_lens = [150, 1, 1, 2, 77, 1, 1]
    kv_lens = [150, 900, 17, 130, 400, 1, (window or 50) + (keep or 3)]
    q, kp, vp, table, refs = paged_case(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=hd + nh)
    rel = rnd(rows, nh, seed=11, scale=1.5)
    spread = rel[ops.distance_bucket_table(rows, far)].t().contiguous()
    sink = torch.zeros(nh)
    scale = 0.2
    args = dict(sink=d(sink), keep_first=keep, softcap=cap, rel=d(spread))
    out = ops.paged_attention(q, kp, vp, FakeBatch(q_lens, kv_lens), table, nh, window, scale, **args)
    ref = []
    for (qq, kk, vv, start), n in zip(refs, q_lens):
        ref.append(_capped_attention(qq.double(), kk.double(), vv.double(), scale, cap, rel.double(), far, window, keep)[start:]
                   .reshape(-1, nh * hd))
    ref = torch.cat(ref)
    assert not torch.isnan(out).any()
    assert float((out.double().cpu() - ref).abs().max()) <= ATT_TOL[dtype] * float(ref.abs().max())
    # every option shows: leaving one out changes the result
    for kw in (dict(rel=None), dict(keep_first=0) if (window and keep) else None, dict(sink=None),
               dict(softcap=None) if cap and cap <= 2 else None):
        if kw is None:
            continue
        other = dict(args)
        other.update(kw)
        o2 = ops.paged_attention(q, kp, vp, FakeBatch(q_lens, kv_lens), table, nh, window, scale, **other)
        assert float((o2.double().cpu() - ref).abs().max()) > 5 * ATT_TOL[dtype] * float(ref.abs().max()), kw


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [48, 64])
@pytest.mark.parametrize("q_len", [1, 2, 50])
def test_one_loud_key_at_the_edges_of_window_and_kept_keys(ops, dtype, hd, q_len):
    """All scores of the last query are 0 but one key's (the cap leaves it loud).  Just inside the window or among the
    kept first keys the row returns that key's value; just outside either it returns the others' mean share (the unit
    sink takes one part in window + kept + 1); hundreds of positions back."""
    from test_kernels_gpu import FakeBatch, paged_case
    nh, nkv, page, window, keep = 4, 2, 16, 36, 5
    L = 700
    last = L - 1
    for loud, seen in [(last - window + 1, True), (last - window, False), (keep - 1, True), (keep, False), (0, True),
                       (last, True), (last - 1, True), (63, False), (64, False), (last - 63, False)]:
        def spike(r, q, k, v):
            k[:] = 0
            k[loud, :, 0] = 8.0
            q[-1] = 0
            q[-1, :, 0] = 5.0          # score 40 against 0 everywhere else; capped at 30: 28.9
            v[:] = 1.0
            v[loud] = 5.0
        q, kp, vp, table, _ = paged_case([q_len], [L], nh, nkv, hd, page, dtype, seed=2, spike=spike)
        out = ops.paged_attention(q, kp, vp, FakeBatch([q_len], [L]), table, nh, window, 1.0, sink=d(torch.zeros(nh)),
                                  keep_first=keep, softcap=30.0, rel=d(torch.zeros(nh, 9)))
        row = out[-1].float().cpu().view(nh, hd)
        want = 5.0 if seen else (window + keep) / (window + keep + 1.0)
        assert float((row - want).abs().max()) < 0.05, (loud, seen, float(row.mean()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_distance_table_picks_one_distance(ops, dtype):
    """Equal scores everywhere, values that rise with the position: a table that is large at one distance only returns
    the value at that distance, per head; a table whose LAST entry is large returns the mean of everything from there
    on back."""
    from test_kernels_gpu import FakeBatch, paged_case
    nh, nkv, hd, page, L = 2, 1, 32, 16, 300

    def flat(r, q, k, v):
        k[:] = 0
        q[:] = 0
        v[:] = torch.arange(L, dtype=torch.float32).view(L, 1, 1) / 64
    for q_len in (1, 40):
        q, kp, vp, table, _ = paged_case([q_len], [L], nh, nkv, hd, page, dtype, seed=1, spike=flat)
        rel = torch.zeros(nh, 120)
        rel[0, 17] = 40.0
        rel[1, 119] = 40.0
        out = ops.paged_attention(q, kp, vp, FakeBatch([q_len], [L]), table, nh, None, 1.0, rel=d(rel))[-1].float().cpu().view(nh, hd)
        assert float((out[0] - (L - 1 - 17) / 64).abs().max()) < 0.03
        assert float((out[1] - (L - 1 - 119) / 2 / 64).abs().max()) < 0.03


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dq,dv", [(4, 2, 32, 16), (3, 1, 24, 40), (2, 2, 64, 64)])
def test_values_mixed_with_another_layers_on_their_way_into_the_cache(ops, out_dtype, nh, nkv, dq, dv):
    from test_kernels_gpu import FakeBatch
    page, T = 8, 19
    cols = nh * dq + nkv * (dq + dv)
    qkv = rnd(T, cols + 3, seed=dq)
    first = rnd(T, nkv * dv + 4, seed=dv + 1)
    lam = torch.tensor([0.3])
    dpad = -(-max(dq, dv) // 16) * 16
    kp = torch.zeros(4, nkv, page, dpad, dtype=out_dtype, device=DEV)
    vp = torch.zeros_like(kp)
    table = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=DEV)
    gain = 1.0 + 0.2 * rnd(dq, seed=3)
    ops.head_norm_rope_append(d(qkv), FakeBatch([T], [T]), table, None, 0, False, d(gain), d(gain), 1e-5, kp, vp, nh, nkv, dq, dv,
                              v_mix=(d(first)[:, 2:2 + nkv * dv], d(lam)))
    v = qkv[:, nh * dq + nkv * dq:cols].double()
    want = (0.7 * v + 0.3 * first[:, 2:2 + nkv * dv].double()).view(T, nkv, dv)
    pages = [2, 0, 3, 1]
    tol = 1e-6 if out_dtype == torch.float32 else 1e-2
    for t in range(T):
        got = vp[pages[t // page], :, t % page, :dv].double().cpu()
        assert float((got - want[t]).abs().max()) <= tol * float(want.abs().max()), t
    assert float(vp[..., dv:].abs().max()) == 0.0 if dpad > dv else True


def _memory_reference(q, k, v, gi_raw, gf_raw, bi, bf, cap, eps, gain, g):
    """[T, heads * dv] float64 through the plain implementation's mixer with identity projections."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    eye = lambda n: torch.eye(n, dtype=F64)
    h = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gi_raw, gf_raw, g], dim=1)
    n_q, n_v = H * dk, H * dv
    sel = lambda a, n: torch.cat([torch.zeros(n, a, dtype=F64), eye(n), torch.zeros(n, h.shape[1] - a - n, dtype=F64)], dim=1)
    w = {"q": sel(0, n_q), "k": sel(n_q, n_q), "v": sel(2 * n_q, n_v), "i": sel(2 * n_q + n_v, H), "f": sel(2 * n_q + n_v + H, H),
         "g": sel(2 * n_q + n_v + 2 * H, n_v), "i.b": bi, "f.b": bf, "norm": gain, "o": eye(n_v)}
    return plain.mlstm(h, w, {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}, eps)


@pytest.mark.parametrize("heads,dk,dv,cap", [(2, 16, 24, 6.0), (1, 160, 40, 15.0), (3, 12, 33, 4.0), (2, 128, 64, 9.0), (4, 40, 72, 10.0)])
def test_matrix_memory_across_steps_and_slots(ops, heads, dk, dv, cap):
    """Three requests in slots out of order, cut into steps of unequal portions (down to single tokens, beside one
    another); the state travels through the slots; gates large enough that the running maximum moves both ways."""
    lens = [70, 9, 131]
    slots = [2, 0, 3]
    cuts = [[33, 2, 1, 1, 20, 13], [9], [1, 1, 64, 33, 2, 30]]
    K, V = heads * dk, heads * dv
    cols = 2 * K + 2 * V + 2 * heads
    data, want = [], []
    bi, bf = rnd(heads, seed=1), 1.0 + rnd(heads, seed=2)
    gain = 1.0 + 0.3 * rnd(V, seed=3)
    for r, L in enumerate(lens):
        x = rnd(L, cols, seed=10 + r)
        x[:, 2 * K + 2 * V:] *= 8.0          # the gates' projections
        data.append(x)
        xd = x.double()
        want.append(_memory_reference(xd[:, :K].view(L, heads, dk), xd[:, K:2 * K].view(L, heads, dk),
                                      xd[:, 2 * K:2 * K + V].view(L, heads, dv), xd[:, 2 * K + 2 * V:2 * K + 2 * V + heads],
                                      xd[:, 2 * K + 2 * V + heads:], bi.double(), bf.double(), cap, 1e-5, gain.double(),
                                      xd[:, 2 * K + V:2 * K + 2 * V]))
    memory = torch.zeros(4, heads, dk, -(-(dv + 1) // 4) * 4, device=DEV)     # rows padded as the mixer asks for them
    maxima = torch.zeros(4, heads, device=DEV)
    memory[1] = float("nan")            # a slot nobody owns
    at = [0, 0, 0]
    step = 0
    got = [torch.zeros(L, V, dtype=F64) for L in lens]
    while any(at[r] < lens[r] for r in range(3)):
        part = [(r, cuts[r][step]) for r in range(3) if step < len(cuts[r])]
        step += 1
        rows = Rows([n for _, n in part], [at[r] for r, _ in part], [slots[r] for r, _ in part])
        proj = d(torch.cat([data[r][at[r]:at[r] + n] for r, n in part]))
        a, b, e = ops.mlstm_gates(proj, 2 * K + 2 * V, 2 * K + 2 * V + heads, d(bi), d(bf), cap, rows, maxima, heads)
        o = ops.gla_scan(proj, 0, K, 2 * K, a, rows, memory, heads, dk, dv + 1, dk ** -0.5, k_scale=b, scalar_decay=True, ones_col=True)
        y = ops.mlstm_out(o, e, proj, 2 * K + V, d(gain), heads, dv, 1e-5, torch.float32).double().cpu()
        row = 0
        for r, n in part:
            got[r][at[r]:at[r] + n] = y[row:row + n]
            row += n
            at[r] += n
    for r in range(3):
        assert float((got[r] - want[r]).abs().max()) <= 2e-4 * float(want[r].abs().max()), r


def test_matrix_memory_keeps_a_far_token(ops):
    """A forget gate that is open (f = 0 after the logarithm: large positive projection) and one loud key 400 tokens back:
    the query that matches it reads that token's value; with the forget gate closed in between it reads nothing of it."""
    heads, dk, dv, cap, L = 1, 16, 8, 20.0, 420
    K, V = dk, dv
    cols = 2 * K + 2 * V + 2
    for closed in (False, True):
        x = torch.zeros(L, cols)
        x[:, 2 * K:2 * K + V] = 1.0                       # values 1 everywhere
        x[:, K] = 0.0001                                  # faint keys along the query's channel
        x[10, K] = 6.0                                    # the loud key, value 5
        x[10, 2 * K:2 * K + V] = 5.0
        x[:, 2 * K + 2 * V] = 0.0                         # input gates: i = 0
        x[:, 2 * K + 2 * V + 1] = 19.0                    # forget gates open
        if closed:
            x[200, 2 * K + 2 * V + 1] = -19.0             # once closed: everything before is scaled by exp(-19)
        x[-1, 0] = 4.0 * dk ** 0.5                        # the last query matches the loud key
        rows = Rows([L], [0], [0])
        memory, maxima = torch.zeros(1, heads, dk, dv + 1, device=DEV), torch.zeros(1, heads, device=DEV)
        proj = d(x)
        a, b, e = ops.mlstm_gates(proj, 2 * K + 2 * V, 2 * K + 2 * V + 1, d(torch.zeros(1)), d(torch.zeros(1)), cap, rows, maxima, heads)
        o = ops.gla_scan(proj, 0, K, 2 * K, a, rows, memory, heads, dk, dv + 1, dk ** -0.5, k_scale=b, scalar_decay=True, ones_col=True)
        last = o[-1].cpu()
        ratio = float(last[0] / last[dv])                 # S^T q over n . q: the value the query reads
        assert abs(ratio - (1.0 if closed else 5.0)) < 0.2, (closed, ratio)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d_,dr,dv,rank,qr,page", [(2, 16, 8, 24, 40, 24, 8), (3, 8, 16, 8, 24, 10, 16), (4, 32, 32, 48, 96, 64, 16),
                                                     (20, 12, 12, 20, 24, 16, 32), (2, 16, 16, 24, 272, 40, 16), (17, 8, 8, 8, 24, 8, 8)])
def test_latent_attention_with_latent_queries_paired_rotation_and_gate(ops, dtype, H, d_, dr, dv, rank, qr, page):
    """The mixer alone against the plain function: a prompt in two portions and then single tokens, next to another
    request; the cache holds one row of rank + rot_dim channels per token; 20 heads share it (two groups on the tensor
    cores) or 17 (one call); a latent row wider than the tensor-core kernels' head sizes."""
    from blackwellllm_b200.config.specs import LatentAttentionSpec, RopeSpec
    from blackwellllm_b200.parts import BuildContext, build_mixer
    from test_kernels_gpu import FakeBatch
    W, eps, L = 64, 1e-5, 75
    names = (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"), ("uk", "uk"), ("uv", "uv"),
             ("g", "g"), ("o", "o"))
    spec = LatentAttentionSpec(num_heads=H, head_dim=d_, rot_dim=dr, v_head_dim=dv, kv_rank=rank, norm_eps=eps,
                               position=RopeSpec(theta=700.0, rotary_dim=dr, scaling=None, interleaved=True),
                               softmax_scale=0.2, window=None, sink=False, names=names, q_rank=qr, output_gate=True)
    mixer = build_mixer(spec, W, BuildContext(DEV, dtype))
    t = {p.name: rnd(*p.shape, seed=i + 1, scale=0.3 if len(p.shape) > 1 else 1.0).to(dtype) for i, p in enumerate(mixer.param_specs())}
    for n in ("dkv.norm", "dq.norm"):
        t[n] = (1.0 + 0.3 * t[n].float()).to(dtype)
    t["uq"] = (t["uq"].float() * 2.0).to(dtype)
    mixer.bind({k: d(v if len(v.shape) > 1 else v.float()) for k, v in t.items()})
    rq = mixer.cache_request()
    assert rq.single_plane and rq.num_kv_heads == 1 and rq.head_dim >= rank + dr
    xs = {0: rnd(L, W, seed=50).to(dtype), 1: rnd(30, W, seed=51).to(dtype)}
    m = {"heads": H, "dim": d_, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "q_rank": qr, "scale": 0.2, "rot": {"base": 700.0, "dims": dr}}
    want = {r: plain.latent_attention(x.double(), {k: v.double() for k, v in t.items()}, m, eps) for r, x in xs.items()}
    n_pages = -(-L // page) + -(-30 // page)
    pool = torch.full((1, n_pages, 1, page, rq.head_dim), float("nan"), dtype=dtype, device=DEV)

    class View:
        group, k_pages, v_pages, page_size = 0, pool[0], pool[0], page
    table = torch.full((2, -(-L // page)), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(9)).tolist()
    for r, n in ((0, L), (1, 30)):
        for b in range(-(-n // page)):
            table[r, b] = perm.pop()
    got = {0: [], 1: []}
    at = {0: 0, 1: 0}
    steps = [[(0, 33), (1, 2)], [(1, 1), (0, 30)]] + [[(0, 1), (1, 1)] for _ in range(12)]
    for step in steps:
        batch = FakeBatch([n for _, n in step], [at[r] + n for r, n in step])
        batch.block_tables = {0: d(table[[r for r, _ in step]])}
        x = torch.cat([xs[r][at[r]:at[r] + n] for r, n in step])
        res = torch.zeros(x.shape[0], W, device=DEV)
        mixer.forward(d(x), res, batch, View)
        ops.resolve_pending()
        o = 0
        for r, n in step:
            got[r].append(res[o:o + n].cpu().double())
            o += n
            at[r] += n
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    for r in (0, 1):
        g = torch.cat(got[r])
        assert float((g - want[r][:g.shape[0]]).abs().max()) <= tol * float(want[r].abs().max()), r


@pytest.mark.parametrize("E,top,F,H", [(8, 3, 32, 64), (2, 2, 44, 50), (5, 1, 48, 64), (16, 4, 64, 128)])
def test_routed_feed_forward_chooses_by_score_plus_correction(ops, E, top, F, H):
    """float32: every row equals the plain function's; a correction large enough to overturn the scores' order decides
    the choice while the weights stay the uncorrected scores over their sum."""
    from blackwellllm_b200.config.specs import RoutedFFNSpec
    from blackwellllm_b200.parts import BuildContext, build_ffn
    from test_kernels_gpu import FakeBatch
    spec = RoutedFFNSpec(num_experts=E, top_k=top, expert_size=F, score="sigmoid", renormalize=True, scale_input=False,
                         router_name="router", expert_names=("e{e}.", "gate", "up", "down"), choice_bias="correction", renorm_eps=1e-20)
    ffn = build_ffn(spec, H, BuildContext(DEV, torch.float32))
    t = {p.name: rnd(*p.shape, seed=i + 3, scale=0.3) for i, p in enumerate(ffn.param_specs())}
    t["correction"] = rnd(E, seed=77, scale=2.0)
    ffn.bind({k: d(v) for k, v in t.items()})
    f = {"router": {"experts": E, "top": top}, "expert": {"ff": F}}
    for T in (1, 7, 200):
        x = rnd(T, H, seed=T)
        want = plain.routed_ffn(x.double(), {k: v.double() for k, v in t.items()}, f)
        out = torch.zeros(T, H, device=DEV)
        ffn.forward(d(x), out, FakeBatch([T], [T]), accumulate=False)
        assert float((out.double().cpu() - want).abs().max()) <= 2e-5 * float(want.abs().max()), T
        without = plain.routed_ffn(x.double(), dict({k: v.double() for k, v in t.items()}, correction=torch.zeros(E, dtype=F64)), f)
        if top < E and T == 200:
            assert float((without - want).abs().max()) > 1e-3 * float(want.abs().max())


# =============================================================================== whole models through the engine

_models = {}
_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def plain_logits(raw, tensors, ids, streams=None):
    return plain.forward(raw, {k: v.double() for k, v in tensors.items()}, ids, streams)


def model(name, dtype):
    key = (name, dtype)
    if key not in _models:
        raw, page = tv.CONFIGS[name]
        tensors = tv.make_tensors(raw, seed=7, dtype=_DT[dtype])
        reqs = {f"r{i}": tv.prompt(n, raw["vocab"], 50 + i) for i, n in enumerate([70, 33, 131, 2, 90])}
        ref = {rid: plain_logits(raw, tensors, ids) for rid, ids in reqs.items()}
        _models[key] = (raw, page, tensors, reqs, ref)
    return _models[key]


def engine_for(name, dtype, **kw):
    from blackwellllm_b200.engine.engine import Engine
    raw, page, tensors, _, _ = model(name, dtype)
    opts = dict(dtype=dtype, page_size=page, num_pages=64, max_requests=4, max_batch_tokens=1 << 16)
    opts.update(kw)
    return Engine.from_tensors(raw, tensors, **opts)


def check_rows(rows, ref, dtype, what):
    """rows {(rid, pos): logits}.  float32: every row within the bound.  bfloat16: a router score that is a near-tie in
    the plain implementation goes the other way now and then, which changes that row altogether; there the rows are
    judged together: all finite, the median within 0.6 of the bound, 4 of 5 within 1.2 of it.  (A wrong key, page,
    state or edge moves every row it touches by far more; the float32 runs of the same schedules have no exception.)"""
    errs = []
    for (rid, p), row in rows.items():
        err = float((row.double().cpu() - ref[rid][p]).abs().max()) / float(ref[rid].abs().max())
        assert err == err and err != float("inf"), (what, rid, p)
        errs.append((err, rid, p))
    errs.sort()
    if dtype == "float32":
        assert errs[-1][0] <= TOL[dtype], (what, errs[-1])
    else:
        assert errs[len(errs) // 2][0] <= 0.6 * TOL[dtype], (what, "median", errs[len(errs) // 2])
        assert errs[(4 * len(errs)) // 5][0] <= 1.2 * TOL[dtype], (what, "4 of 5", errs[(4 * len(errs)) // 5])


def run_steps(eng, steps):
    """steps: [[(rid, tokens, start)]]: every position's logits by (rid, position)."""
    from blackwellllm_b200.engine.engine import StepEntry
    rows = {}
    for step in steps:
        out = eng.step([StepEntry(rid, toks, list(range(len(toks)))) for rid, toks, _ in step]).cpu()
        at = 0
        for rid, toks, start in step:
            for i in range(len(toks)):
                rows[(rid, start + i)] = out[at + i].clone()
            at += len(toks)
    return rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tv.CONFIGS))
def test_whole_prompts_and_the_stream_after_every_layer(name, dtype):
    raw, _, tensors, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    streams, want_streams = [], []
    plain_logits(raw, tensors, reqs["r0"], want_streams)
    eng.model.stream_hook = lambda pos, h: streams.append(h.double().cpu().clone())
    rows = run_steps(eng, [[("r0", reqs["r0"], 0)]])
    eng.model.stream_hook = None
    assert len(streams) == len(want_streams) == len(raw["layers"])
    if dtype == "float32":
        for i, (got, want) in enumerate(zip(streams, want_streams)):
            assert float((got - want).abs().max()) <= 2e-5 * float(want.abs().max()), f"layer {i}"
    eng.end_request("r0")
    for rid in ("r1", "r2", "r3", "r4"):
        rows.update(run_steps(eng, [[(rid, reqs[rid], 0)]]))
        eng.end_request(rid)
    check_rows(rows, ref, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tv.CONFIGS))
def test_token_by_token_from_the_first_token(name, dtype):
    """Decoding from position 0 (the first tokens of a sequence, every page border, the window's and the kept keys'
    edges passing over decoded tokens, the memory from its zero state), long enough that the decode steps are replayed
    from a CUDA graph."""
    _, _, _, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    ids = reqs["r2"]
    rows = run_steps(eng, [[("r2", [t], i)] for i, t in enumerate(ids)])
    check_rows(rows, ref, dtype, "token by token")
    assert eng.graph_kernel_count(1) > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tv.CONFIGS))
@pytest.mark.parametrize("sizes", [(2,), (7, 2, 13, 3, 5, 2, 16, 17, 4, 31, 2), (64, 1, 1, 1, 40, 1)])
def test_portions(name, dtype, sizes):
    _, _, _, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    rows = {}
    for rid in ("r0", "r2", "r4"):
        ids, at, k, steps = reqs[rid], 0, 0, []
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            steps.append([(rid, ids[at:at + n], at)])
            at, k = at + n, k + 1
        rows.update(run_steps(eng, steps))
        eng.end_request(rid)
    check_rows(rows, ref, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tv.CONFIGS))
def test_unequal_requests_together_and_pages_used_again(name, dtype):
    """A pool that holds two requests: five pass through, portions of one beside single tokens of another; every
    later request gets a slot (with the memories of its layers in it) and pages that an earlier one gave back."""
    raw, page, _, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype, num_pages=-(-(131 + 90) // page) + 2, max_requests=2)
    waiting = list(reqs.items())
    live, rows = {}, {}
    g = torch.Generator().manual_seed(3)
    while waiting or live:
        while waiting and len(live) < 2:
            rid, ids = waiting.pop(0)
            live[rid] = 0
        step = []
        for rid in list(live):
            ids, at = reqs[rid], live[rid]
            if at >= len(ids) - 6:
                n = 1
            else:
                n = min(int(torch.randint(2, 30, (1,), generator=g)), len(ids) - 6 - at)
            step.append((rid, ids[at:at + n], at))
            live[rid] = at + n
        rows.update(run_steps(eng, [step]))
        for rid in list(live):
            if live[rid] == len(reqs[rid]):
                eng.end_request(rid)
                del live[rid]
    check_rows(rows, ref, dtype, "mixed")
    eng.cache.check_invariants()
    assert eng.cache.slots.num_free == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "tensor"])
def test_a_long_request_in_portions_then_decoded(name, dtype):
    """700 tokens: the windows have passed dozens of pages (given back meanwhile), the kept first keys are hundreds of
    positions away, the distances lie far beyond the tables, the memory has run 700 steps; prompt portions that start
    and end inside pages, then 40 tokens one by one."""
    raw, page, tensors, _, _ = model(name, dtype)
    ids = tv.prompt(700, raw["vocab"], 999)
    ref = {"long": plain_logits(raw, tensors, ids)}
    eng = engine_for(name, dtype, num_pages=-(-700 // page) + 1, max_requests=1)
    steps, at = [], 0
    for n in (333, 2, 190, 135):
        steps.append([("long", ids[at:at + n], at)])
        at += n
    steps += [[("long", [ids[i]], i)] for i in range(at, 700)]
    check_rows(run_steps(eng, steps), ref, dtype, "long")
    # the windows gave pages back on the way: the groups with a window hold far fewer than 700 tokens' worth now
    held = [sum(1 for p in eng.cache.block_table("long", g) if p >= 0) for g in range(len(eng.cache.groups))]
    assert all(h * page < 300 for h, grp in zip(held, eng.cache.groups) if grp.request.window), held


@pytest.mark.parametrize("name", list(tv.CONFIGS))
def test_a_batch_changes_no_bit_of_a_request(name):
    """float32: a request's logits beside other requests equal its logits alone, bit for bit."""
    _, _, _, reqs, _ = model(name, "float32")
    alone = engine_for(name, "float32")
    a = run_steps(alone, [[("r1", reqs["r1"][:20], 0)], [("r1", reqs["r1"][20:21], 20)]])
    both = engine_for(name, "float32")
    b = run_steps(both, [[("r4", reqs["r4"][:9], 0), ("r1", reqs["r1"][:20], 0), ("r0", reqs["r0"][:3], 0)],
                         [("r0", reqs["r0"][3:4], 3), ("r1", reqs["r1"][20:21], 20), ("r4", reqs["r4"][9:40], 9)]])
    for key, row in a.items():
        assert torch.equal(row, b[key]), key


def test_a_request_left_out_of_steps_goes_on_where_it_was():
    """A request that sits out some steps finds its memory and its keys as it left them, while another request in the
    neighbouring slot runs on."""
    _, _, _, reqs, ref = model("mixed", "float32")
    eng = engine_for("mixed", "float32")
    a, b = reqs["r0"], reqs["r4"]
    steps = [[("r0", a[:10], 0), ("r4", b[:3], 0)], [("r4", b[3:50], 3)], [("r4", b[50:51], 50)],
             [("r0", a[10:11], 10), ("r4", b[51:52], 51)], [("r0", a[11:70], 11)], [("r4", b[52:90], 52)]]
    check_rows(run_steps(eng, steps), ref, "float32", "left out")


@pytest.mark.parametrize("name", list(tv.CONFIGS))
def test_greedy_generation_through_the_entry_point(name, tmp_path):
    """generate() (scheduler, sampling, continuous batching) gives the plain implementation's greedy tokens."""
    import os
    from safetensors.torch import load_file
    from blackwellllm_b200 import BlackwellEngine, InferenceConfig, SamplingParams
    raw, page = tv.CONFIGS[name]
    folder = tv.make_folder(name, "float32", str(tmp_path))
    W = load_file(os.path.join(folder, "model.safetensors"))
    prompts = [tv.prompt(n, raw["vocab"], 80 + n) for n in (5, 40, 1)]
    steps = 12
    llm = BlackwellEngine(folder, InferenceConfig(max_context_length=128, max_batch_size=3), dtype="float32")
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=steps))
    for p, g in zip(prompts, got):
        ids = list(p)
        for _ in range(steps):
            ids.append(int(torch.argmax(plain_logits(raw, W, ids)[-1])))
        assert list(g.token_ids) == ids[len(p):]


def test_command_line_and_position_addressed_calls(tmp_path, capsys):
    import os
    from safetensors.torch import load_file
    from blackwellllm_b200 import BlackwellEngine, InferenceConfig, cli
    name = "mixed"
    raw, _ = tv.CONFIGS[name]
    folder = tv.make_folder(name, "float32", str(tmp_path))
    W = load_file(os.path.join(folder, "model.safetensors"))
    prompt = tv.prompt(9, raw["vocab"], 4)
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(torch.argmax(plain_logits(raw, W, ids)[-1])))
    want = ids[len(prompt):]
    rc = cli.main(["-m", folder, "--dtype", "float32", "--ctx", "128", "--temperature", "0", "--max-new-tokens", "6",
                   "--prompt-ids", ",".join(map(str, prompt))])
    out = capsys.readouterr().out
    assert rc == 0 and [int(t) for t in out.strip().splitlines()[0].split()] == want
    llm = BlackwellEngine(folder, InferenceConfig(max_context_length=128, max_batch_size=2), dtype="float32")
    nxt = llm.prefill(prompt, start_pos=0, temperature=0.0, seq_id=0)
    got = [nxt]
    for i in range(5):
        nxt = llm.forward(nxt, pos=len(prompt) + i, temperature=0.0, seq_id=0)
        got.append(nxt)
    assert got == want


# =============================================================================== bin/trace_run

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["tail", "portions", "mixed"])
def test_replay(tmp_path_factory, dtype, family):
    import os
    from safetensors.torch import load_file
    name = "mixed"
    raw, page = tv.CONFIGS[name]
    folder = tv.make_folder(name, dtype, str(tmp_path_factory.mktemp("vubotar")))
    W = load_file(os.path.join(folder, "model.safetensors"))
    reqs = {f"q{i}": tv.prompt(n, raw["vocab"], 200 + i) for i, n in enumerate([40, 97, 50, 70, 130, 65])}
    ref = {rid: plain_logits(raw, W, ids) for rid, ids in reqs.items()}
    if family == "tail":
        steps, max_tokens = replay.trace_tail(reqs)
    elif family == "portions":
        steps, max_tokens = replay.trace_portions(reqs)
    else:
        max_tokens = 384
        steps = replay.trace_mixed(reqs, max_tokens, seed=3)
    rows = replay.run_trace(folder, dtype, steps, max_tokens, raw["vocab"], page_size=page)
    check_rows(rows, ref, dtype, f"replay {family}")


# =============================================================================== random configurations

def _random_configuration(rng):
    def pick(*xs):
        return xs[int(torch.randint(0, len(xs), (1,), generator=rng))]
    width = pick(40, 48, 72)
    layers = []
    kv_mix, vdim_mix = pick(1, 2), pick(8, 12, 20)
    for _ in range(pick(1, 2, 3, 4)):
        mlp = pick(None, tv._moe(pick(1, 2, 5), 1, pick(24, 40)), tv._moe(4, pick(2, 3, 4), 16))
        kind = pick(0, 0, 1, 2)
        if kind == 0:
            mix = pick(False, True, True)
            kv = kv_mix if mix else pick(1, 2)
            size = pick(None, 3, 11, 40)
            layers.append(tv._attn(kv * pick(1, 2, 3), kv, pick(8, 12, 20), vdim_mix if mix else pick(8, 12, 20), pick(0.1, 0.3),
                                   pick(2, 3, 8, 32), pick(40, 64, 500), cap=pick(None, 1.0, 50.0), size=size,
                                   keep=pick(None, 0, 1, 9, 50) if size else None, v_mix=mix, mlp=mlp))
        elif kind == 1:
            layers.append(tv._latent(pick(1, 2, 5), pick(4, 8, 12), pick(2, 6, 8), pick(4, 8, 12), pick(8, 20, 30), pick(4, 16, 24),
                                     pick(0.1, 0.3), pick(100.0, 20000.0), mlp=mlp))
        else:
            layers.append(tv._mlstm(pick(1, 2, 3), pick(4, 8, 20), pick(4, 31, 32, 40), pick(2.0, 12.0), mlp=mlp))
    raw = {"architecture": "Vubotar", "vocab": pick(60, 130), "width": width, "norm": {"eps": pick(1e-5, 1e-3)},
           "embedding": {"scale": pick(0.5, 1.0, 4.0)}, "logit_scale": pick(0.25, 1.0, 3.0), "layers": layers}
    if pick(0, 1):
        raw["logit_softcap"] = pick(8.0, 30.0)
    return raw, pick(8, 16)


@pytest.mark.parametrize("seed", range(10))
def test_random_configurations_float32(seed):
    from blackwellllm_b200.engine.engine import Engine
    rng = torch.Generator().manual_seed(2000 + seed)
    raw, page = _random_configuration(rng)
    tensors = tv.make_tensors(raw, seed=seed, dtype=torch.float32)
    ids = tv.prompt(90, raw["vocab"], seed)
    ref = {"a": plain_logits(raw, tensors, ids)}
    eng = Engine.from_tensors(raw, tensors, dtype="float32", page_size=page, num_pages=24, max_requests=2)
    check_rows(run_steps(eng, [[("a", ids, 0)]]), ref, "float32", f"whole {raw}")
    eng.end_request("a")
    steps, at = [], 0
    for n in (5, 2, 30, 1, 1, 17, 2, 32):
        steps.append([("a", ids[at:at + n], at)])
        at += n
    check_rows(run_steps(eng, steps), ref, "float32", f"portions {raw}")
