"""The Zigipel design on the GPU against its plain implementation (tests/plain_zigipel.py): each mechanism's kernels
alone, then whole models through Engine.step in every way of cutting and batching, through the scheduler's
generate(), the command line and bin/trace_run."""
import math

import pytest
import torch

import plain_zigipel as plain
import replay
import tiny_zigipel as tz

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

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,buckets,mp,mc", [(64, 97, 13, 5), (50, 1, 3, 1), (200, 1000, 1, 1000003)])
def test_hashed_second_table_across_steps(ops, dtype, H, buckets, mp, mc):
    """Three requests in slots out of order; portions of 1, 2 and many tokens; the previous token of a portion's first
    token comes from the step before; a slot used again by another request starts with the extra row."""
    V = 300
    table, second = rnd(V, H, seed=1).to(dtype), rnd(buckets + 1, H, seed=2).to(dtype)
    seqs = {0: tz.prompt(9, V, 3), 1: tz.prompt(5, V, 4), 2: tz.prompt(12, V, 5)}
    want = {r: table[torch.tensor(s)].double() + second[torch.tensor(plain.bigram_rows(s, buckets, mp, mc))].double()
            for r, s in seqs.items()}
    prev = torch.full((4,), 123456, dtype=torch.int32, device=DEV)        # garbage: a first token must not read it
    slots = {0: 3, 1: 0, 2: 1}
    at = {r: 0 for r in seqs}
    got = {r: [] for r in seqs}
    for step in ([(0, 4), (1, 1)], [(1, 2), (0, 1), (2, 7)], [(2, 1), (0, 4), (1, 2)], [(2, 4)]):
        b = Rows([n for _, n in step], [at[r] for r, _ in step], [slots[r] for r, _ in step])
        b.token_ids = torch.tensor([t for r, n in step for t in seqs[r][at[r]:at[r] + n]], dtype=torch.int32, device=DEV)
        out = ops.embed_bigram(d(table), d(second), b, prev, buckets, mp, mc).cpu().double()
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n])
            o += n
            at[r] += n
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    for r in seqs:
        assert float((torch.cat(got[r]) - want[r]).abs().max()) <= tol * float(want[r].abs().max()), r
    assert prev.cpu().tolist()[3] == seqs[0][-1] and prev.cpu().tolist()[0] == seqs[1][-1]


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [64, 50, 328, 2052, 4096])
def test_norm_and_token_shift_across_steps(ops, out_dtype, H):
    eps = 1e-5
    gain, shift = 1.0 + rnd(H, seed=1, scale=0.3), torch.rand(H, generator=torch.Generator().manual_seed(2))
    xs = {0: rnd(9, H, seed=3, scale=3.0), 1: rnd(5, H, seed=4), 2: rnd(12, H, seed=5, scale=0.2)}
    want_h = {r: plain.rms_norm(x.double(), gain.double(), eps) for r, x in xs.items()}
    want_s = {r: plain.token_shift(h, shift.double()) for r, h in want_h.items()}
    state = torch.full((4, H), 77.0, device=DEV)                            # garbage: a first token must not read it
    slots = {0: 2, 1: 3, 2: 0}
    at = {r: 0 for r in xs}
    got_h, got_s = {r: [] for r in xs}, {r: [] for r in xs}
    for step in ([(0, 4), (1, 1)], [(1, 2), (0, 1), (2, 7)], [(2, 1), (0, 4), (1, 2)], [(2, 4)]):
        b = Rows([n for _, n in step], [at[r] for r, _ in step], [slots[r] for r, _ in step])
        x = torch.cat([xs[r][at[r]:at[r] + n] for r, n in step])
        h, hs = ops.rmsnorm_shift(d(x), d(gain), d(shift), state, b, eps, out_dtype)
        only = ops.rmsnorm_shift(d(x), d(gain), d(shift), state.clone(), b, eps, out_dtype, want_h=False)
        assert only[0] is None
        o = 0
        for r, n in step:
            got_h[r].append(h[o:o + n].cpu().double())
            got_s[r].append(hs[o:o + n].cpu().double())
            o += n
            at[r] += n
    tol = 2e-6 if out_dtype == torch.float32 else 1e-2
    for r in xs:
        assert float((torch.cat(got_h[r]) - want_h[r]).abs().max()) <= tol * float(want_h[r].abs().max())
        assert float((torch.cat(got_s[r]) - want_s[r]).abs().max()) <= tol * float(want_h[r].abs().max())
    # float32: the shifted row of a portion's first token is the same bits as inside a longer portion
    if out_dtype == torch.float32:
        st = torch.zeros((1, H), device=DEV)
        whole = ops.rmsnorm_shift(d(xs[2]), d(gain), d(shift), st, Rows([12], [0], [0]), eps, out_dtype)[1].cpu()
        assert torch.equal(whole, torch.cat(got_s[2]).float())


@pytest.mark.parametrize("T,n_req", [(3, 3), (1, 1), (6, 2), (40, 40)])
def test_two_open_sums_into_the_stream_are_added_by_the_next_norm(ops, T, n_req):
    """Two products of a few tokens into the same float32 stream stay open together; the norm-and-shift kernel adds them
    in a step of single tokens (and leaves the stream summed), a kernel of its own does otherwise; either way the stream
    and both outputs are those of the sums made one after the other."""
    from blackwellllm_b200.parts.linear import Linear
    H, K1, K2, eps = 256, 512, 1024, 1e-5
    gain, shift = 1.0 + rnd(H, seed=1, scale=0.3), torch.rand(H, generator=torch.Generator().manual_seed(2))
    x = rnd(T, H, seed=3)
    a1, a2 = rnd(T, K1, seed=4).bfloat16(), rnd(T, K2, seed=5).bfloat16()
    w1, w2 = rnd(H, K1, seed=6, scale=0.05).bfloat16(), rnd(H, K2, seed=7, scale=0.05).bfloat16()
    b2 = rnd(H, seed=8).bfloat16()
    per = T // n_req
    batch = Rows([per] * n_req, [5 * (r + 1) for r in range(n_req)], list(range(n_req)))
    state0 = rnd(n_req, H, seed=9)
    stream, state = d(x), d(state0)
    ops.discard_pending()
    Linear(d(w1)).add_to(d(a1), stream)
    Linear(d(w2), d(b2)).add_to(d(a2), stream)
    assert ops.pending_target() is stream
    h, hs = ops.rmsnorm_shift(stream, d(gain), d(shift), state, batch, eps, torch.float32)
    assert ops.pending_target() is None
    total = x.double() + a1.double() @ w1.double().T + a2.double() @ w2.double().T + b2.double()
    assert float((stream.cpu().double() - total).abs().max()) <= 2e-5 * float(total.abs().max())
    want_h = plain.rms_norm(total, gain.double(), eps)
    assert float((h.cpu().double() - want_h).abs().max()) <= 1e-4 * float(want_h.abs().max())
    for r in range(n_req):
        rows = slice(r * per, (r + 1) * per)
        before = torch.cat([state0[r:r + 1].double(), want_h[rows][:-1]])
        want_s = want_h[rows] + (before - want_h[rows]) * shift.double()
        assert float((hs[rows].cpu().double() - want_s).abs().max()) <= 1e-4 * float(want_h.abs().max())
        assert float((state[r].cpu().double() - want_h[rows][-1]).abs().max()) <= 1e-4 * float(want_h.abs().max())
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_streams_side_by_side_and_gated_gelu(ops, dtype):
    a, b = rnd(7, 50, seed=1), rnd(7, 50, seed=2)
    out = ops.concat2_cast(d(a), d(b), dtype).cpu()
    assert torch.equal(out, torch.cat([a, b], dim=1).to(dtype))
    a, b = rnd(5, 2052, seed=1), rnd(5, 2052, seed=2)
    assert torch.equal(ops.concat2_cast(d(a), d(b), dtype).cpu(), torch.cat([a, b], dim=1).to(dtype))
    gu = rnd(9, 2 * 40, seed=3, scale=2.0)
    got = ops.glu(d(gu), ops.ACT_GELU_TANH, out_dtype=dtype).cpu().double()
    want = plain.gelu_tanh(gu[:, :40].double()) * gu[:, 40:].double()
    assert float((got - want).abs().max()) <= (1e-6 if dtype == torch.float32 else 1e-2) * float(want.abs().max())


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("T", [1, 8, 16, 17, 100, 300, 600, 1100])
@pytest.mark.parametrize("H,F", [(64, 96), (256, 1024), (2048, 512)])
def test_dense_feed_forward_with_biases_bfloat16(ops, act, T, H, F):
    """The gated feed-forward part on the tensor cores: the gate/up product adds the biases and applies the activation
    in its epilogue, in every form of that product (few tokens with the K splits summed in the kernel, split K with a
    second kernel, whole tiles, CTA pairs)."""
    from blackwellllm_b200.config.specs import SwiGLUSpec
    from blackwellllm_b200.parts import BuildContext, build_ffn
    spec = SwiGLUSpec(intermediate_size=F, activation=act, names=("gate", "up", "down"), bias_names=("gate.b", "up.b", "down.b"))
    ffn = build_ffn(spec, H, BuildContext(DEV, torch.bfloat16))
    t = {"gate": rnd(F, H, seed=1, scale=H ** -0.5), "up": rnd(F, H, seed=2, scale=H ** -0.5), "down": rnd(H, F, seed=3, scale=F ** -0.5),
         "gate.b": rnd(F, seed=4), "up.b": rnd(F, seed=5), "down.b": rnd(H, seed=6)}
    t = {k: v.to(torch.bfloat16) for k, v in t.items()}
    ffn.bind({k: d(v) for k, v in t.items()})
    assert ffn.fused
    x = rnd(T, H, seed=7).to(torch.bfloat16)
    res = torch.zeros(T, H, device=DEV)
    ffn.forward(d(x), res, None)
    ops.resolve_pending()
    w = {k: v.double() for k, v in t.items()}
    g, u = x.double() @ w["gate"].T + w["gate.b"], x.double() @ w["up"].T + w["up.b"]
    a = plain.gelu_tanh(g) * u if act == "gelu_tanh" else g * torch.sigmoid(g) * u
    want = a @ w["down"].T + w["down.b"]
    assert float((res.cpu().double() - want).abs().max()) <= 1.5e-2 * float(want.abs().max())
    assert ops.gemm_tc_status() == 0


def _biased_attention(q, k, v, sink, scale, r1, r2, window, keep, gate=None):
    """q [L, nh, hd], k / v [L, nkv, hd] float64 -> [L, nh, hd]: the plain implementation's pieces."""
    L, nh, _ = q.shape
    rep = nh // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if r1 is not None:
        dist = (torch.arange(L).view(-1, 1) - torch.arange(L).view(1, -1)).clamp(min=0).to(F64)
        s = s - r1.view(nh, 1, 1) * torch.log(1.0 + r2.view(nh, 1, 1) * dist)
    w = plain.sink_softmax(s, plain.window_mask(L, window or L, keep), sink)
    o = torch.einsum("hij,jhd->ihd", w, vv)
    return o if gate is None else o * torch.sigmoid(gate).view(L, nh, 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page,window,keep", [(4, 2, 80, 8, 44, 7), (2, 2, 64, 16, 100, 70), (8, 2, 128, 16, 33, 1),
                                                        (6, 3, 96, 16, 64, 64), (3, 1, 16, 32, 7, 20), (4, 1, 32, 16, None, 0),
                                                        (4, 4, 64, 64, 130, 0), (20, 1, 32, 16, 40, 5), (4, 1, 256, 16, 70, 130),
                                                        (16, 4, 128, 16, 128, 64)])
def test_attention_with_distance_bias_kept_keys_and_head_gate(ops, dtype, nh, nkv, hd, page, window, keep):
    """Prompt portions from position 0 and continued, decode tokens with few and many keys, a two-token portion; the
    window's and the kept keys' edges fall inside tiles and pages."""
    from test_kernels_gpu import ATT_TOL, FakeBatch, paged_case
    q_lens = [150, 1, 1, 2, 77, 1, 1]
    kv_lens = [150, 900, 17, 130, 400, 1, (window or 50) + (keep or 3)]
    q, kp, vp, table, refs = paged_case(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=hd + nh)
    g = torch.Generator().manual_seed(7)
    sink = torch.linspace(-3.0, 3.0, nh)
    r1, r2 = 2.0 * torch.rand(nh, generator=g), 0.02 + 0.48 * torch.rand(nh, generator=g)
    gate = torch.randn(sum(q_lens), nh + 5, generator=g)
    batch = FakeBatch(q_lens, kv_lens)
    out = ops.paged_attention(q, kp, vp, batch, table, nh, window, 0.2, sink=d(sink), gate=(d(gate)[:, 5:], hd, "head"),
                              dist=d(torch.stack([r1, r2])), keep_first=keep)
    ref, at = [], 0
    for (qq, kk, vv, start), n in zip(refs, q_lens):
        gfull = torch.zeros(qq.shape[0], nh, dtype=F64)
        gfull[start:] = gate[at:at + n, 5:].double()
        at += n
        ref.append(_biased_attention(qq.double(), kk.double(), vv.double(), sink.double(), 0.2, r1.double(), r2.double(),
                                     window, keep, gfull)[start:].reshape(-1, nh * hd))
    ref = torch.cat(ref)
    assert not torch.isnan(out).any()
    assert float((out.double().cpu() - ref).abs().max()) <= ATT_TOL[dtype] * float(ref.abs().max())
    # every option shows: leaving one out changes the result
    for kw in (dict(dist=None), dict(keep_first=0) if (window and keep) else None, dict(gate=None)):
        if kw is None:
            continue
        args = dict(sink=d(sink), gate=(d(gate)[:, 5:], hd, "head"), dist=d(torch.stack([r1, r2])), keep_first=keep)
        args.update(kw)
        other = ops.paged_attention(q, kp, vp, FakeBatch(q_lens, kv_lens), table, nh, window, 0.2, **args)
        assert float((other.double().cpu() - ref).abs().max()) > 5 * ATT_TOL[dtype] * float(ref.abs().max()), kw


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [80, 64])
@pytest.mark.parametrize("q_len", [1, 2, 50])
def test_one_loud_key_at_the_edges_of_window_and_kept_keys(ops, dtype, hd, q_len):
    """All scores of the last query are 0 but one key's.  Just inside the window or among the kept first keys the row
    returns that key's value; just outside either it returns the mean of the others; hundreds of positions back."""
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
            q[-1, :, 0] = 5.0          # score 40 against 0 everywhere else
            v[:] = 1.0
            v[loud] = 5.0
        q, kp, vp, table, _ = paged_case([q_len], [L], nh, nkv, hd, page, dtype, seed=2, spike=spike)
        sink = torch.full((nh,), -30.0)
        out = ops.paged_attention(q, kp, vp, FakeBatch([q_len], [L]), table, nh, window, 1.0, sink=d(sink), keep_first=keep,
                                  dist=d(torch.zeros(2, nh)))
        row = out[-1].float().cpu().view(nh, hd)
        want = 5.0 if seen else 1.0
        assert float((row - want).abs().max()) < 0.05, (loud, seen, float(row.mean()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_distance_bias_silences_far_keys(ops, dtype):
    """Equal scores everywhere, values that rise with the position: with r1 = 0 the row is the mean of the values, with
    a large r1 it is the last value (distance 0 has no bias), per head."""
    from test_kernels_gpu import FakeBatch, paged_case
    nh, nkv, hd, page, L = 2, 1, 32, 16, 300

    def flat(r, q, k, v):
        k[:] = 0
        q[:] = 0
        v[:] = torch.arange(L, dtype=torch.float32).view(L, 1, 1) / 64
    for q_len in (1, 40):
        q, kp, vp, table, _ = paged_case([q_len], [L], nh, nkv, hd, page, dtype, seed=1, spike=flat)
        dist = torch.tensor([[0.0, 60.0], [0.3, 0.3]])
        out = ops.paged_attention(q, kp, vp, FakeBatch([q_len], [L]), table, nh, None, 1.0, sink=d(torch.full((nh,), -50.0)),
                                  dist=d(dist))[-1].float().cpu().view(nh, hd)
        assert float((out[0] - (L - 1) / 128).abs().max()) < 0.03 and float((out[1] - (L - 1) / 64).abs().max()) < 0.03


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dq,dv", [(4, 2, 32, 16), (3, 1, 24, 40), (2, 2, 64, 64)])
def test_values_are_cached_with_unit_root_mean_square(ops, out_dtype, nh, nkv, dq, dv):
    from test_kernels_gpu import FakeBatch
    page, eps = 8, 1e-3
    step = 16 if out_dtype == torch.bfloat16 else 1
    dpad = -(-max(dq, dv) // step) * step
    q_lens, kv_lens = [5, 1, 2], [5, 64, 130]
    batch = FakeBatch(q_lens, kv_lens)
    T = sum(q_lens)
    qkv = rnd(T, nh * dq + nkv * (dq + dv) + nh, seed=dq + dv, scale=3.0)
    blocks = [-(-k // page) for k in kv_lens]
    table = torch.full((3, max(blocks)), -1, dtype=torch.int32)
    perm = torch.randperm(sum(blocks) + 2, generator=torch.Generator().manual_seed(3)).tolist()
    for r, b in enumerate(blocks):
        table[r, :b] = torch.tensor([perm.pop() for _ in range(b)], dtype=torch.int32)
    kp = torch.full((sum(blocks) + 2, nkv, page, dpad), 7.0, dtype=out_dtype, device=DEV)
    vp = torch.full((sum(blocks) + 2, nkv, page, dpad), 7.0, dtype=out_dtype, device=DEV)
    q = ops.head_norm_rope_append(d(qkv), batch, d(table), None, 0, False, None, None, 0.0, kp, vp, nh, nkv, dq, dv,
                                  v_eps=eps).cpu().double().view(T, nh, dpad)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert float((q[..., :dq] - qkv[:, :nh * dq].double().view(T, nh, dq)).abs().max()) <= tol * 12       # queries as they are
    want_k = qkv[:, nh * dq:nh * dq + nkv * dq].double().view(T, nkv, dq)
    want_v = plain.rms_unit(qkv[:, (nh + nkv) * dq:(nh + nkv) * dq + nkv * dv].double().view(T, nkv, dv), eps)
    pos, req = batch.positions.cpu(), batch.req_of_token.cpu()
    for t in range(T):
        p = int(pos[t])
        pg = int(table[int(req[t]), p // page])
        k_row, v_row = kp[pg, :, p % page].cpu().double(), vp[pg, :, p % page].cpu().double()
        assert float((k_row[:, :dq] - want_k[t]).abs().max()) <= tol * 12
        assert float((v_row[:, :dv] - want_v[t]).abs().max()) <= tol * float(want_v.abs().max())
        assert float(k_row[:, dq:].abs().sum()) == 0.0 and float(v_row[:, dv:].abs().sum()) == 0.0


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,n_in,n_out", [(1, 3, 40, 24), (70, 2, 64, 64), (130, 4, 128, 192), (65, 2, 192, 128), (9, 1, 256, 72),
                                            (100, 2, 320, 40), (33, 1, 520, 130), (64, 3, 24, 200)])
def test_a_product_per_head_on_the_tensor_cores(ops, x_dtype, T, H, n_in, n_out):
    """y[t, h] = W_h x[t, h] with bfloat16 weights: inner sizes below, at and above what one round of staging takes, rows
    with other columns around the heads' inputs and outputs."""
    x_hs, y_hs = n_in + 8, n_out + 16
    x = rnd(T, 16 + H * x_hs, seed=1).to(x_dtype)
    w = rnd(H, n_out, n_in, seed=2, scale=n_in ** -0.5).bfloat16()
    y = torch.full((T, 8 + H * y_hs), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.headwise_linear(d(x), 16, x_hs, d(w), y, 8, y_hs)
    xin = x[:, 16:].view(T, H, x_hs)[:, :, :n_in].bfloat16().double()      # float32 inputs are rounded on the way
    want = torch.einsum("thi,hoi->tho", xin, w.double())
    got = y.cpu().double()[:, 8:].view(T, H, y_hs)
    assert float((got[:, :, :n_out] - want).abs().max()) <= 1e-2 * float(want.abs().max())
    assert torch.all(got[:, :, n_out:] == 7.0) and torch.all(y.cpu()[:, :8] == 7.0)      # nothing beside the outputs is touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d_,dr,dv,rank,page,window", [(2, 16, 8, 24, 40, 8, 9), (3, 8, 16, 8, 24, 16, 30), (4, 32, 32, 48, 96, 16, None),
                                                         (20, 12, 12, 20, 24, 32, 50), (2, 16, 16, 24, 272, 16, 40), (17, 8, 8, 8, 24, 8, 20)])
def test_latent_attention_mixer_alone(ops, dtype, H, d_, dr, dv, rank, page, window):
    """The mixer part against the plain function: a prompt in two portions and then single tokens, next to another
    request; the cache holds one row of rank + rot_dim channels per token (one plane); 20 heads share it (two groups of 10 on the tensor cores) or 17 (one call); a latent
    row wider than the tensor-core kernels' head sizes."""
    _latent_mixer_case(ops, dtype, H, d_, dr, dv, rank, page, window)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d_,dr,dv,rank,page,window", [(2, 16, 16, 24, 40, 8, 9), (3, 8, 32, 8, 24, 16, 30), (4, 64, 64, 32, 64, 16, 17)])
def test_latent_attention_loud_keys_at_the_windows_edge(ops, dtype, H, d_, dr, dv, rank, page, window):
    """Three tokens whose rotated key part is many times the others': each lies just inside the window of one query (the
    last of a prompt portion, one in its middle, a decoded one) and just outside the next query's.  Their sign is chosen so
    that the plain result of the query that still sees them changes greatly when the window is one key shorter; the mixer
    must then agree with the plain result at the true window.  (bfloat16: keys three times the others' instead of eight
    times, and a wider bound: the rounding of a score grows with the score.)"""
    factor = 8.0 if dtype == torch.float32 else 3.0

    def loud(xs, t, m, eps):
        x = xs[0]
        for i in (62, 50, 74):          # the queries: last of the second portion, inside it, the last decoded token
            j = i - window + 1
            best = None
            for sign in (factor, -factor):
                y = x.clone()
                y[j] = x[j] * sign
                tt = {k: v.double() for k, v in t.items()}
                full = plain.latent_attention(y.double(), tt, m, eps)[i]
                short = plain.latent_attention(y.double(), tt, dict(m, mask={"size": window - 1}), eps)[i]
                gap = float((full - short).abs().max()) / float(full.abs().max())
                if best is None or gap > best[0]:
                    best = (gap, y)
            assert best[0] > 0.2, (i, best[0])      # the edge key decides the row
            x = best[1]
        xs[0] = x
    _latent_mixer_case(ops, dtype, H, d_, dr, dv, rank, page, window, edit=loud, bf16_tol=5e-2)


def _latent_mixer_case(ops, dtype, H, d_, dr, dv, rank, page, window, edit=None, bf16_tol=3e-2):
    from blackwellllm_b200.config.specs import LatentAttentionSpec, RopeSpec, YarnRopeScaling
    from blackwellllm_b200.parts import BuildContext, build_mixer
    from test_kernels_gpu import FakeBatch
    W, eps, L = 64, 1e-5, 75
    rot = {"base": 5000.0, "dims": dr, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}
    spec = LatentAttentionSpec(num_heads=H, head_dim=d_, rot_dim=dr, v_head_dim=dv, kv_rank=rank, norm_eps=eps,
                               position=RopeSpec(theta=5000.0, rotary_dim=dr, scaling=YarnRopeScaling(4.0, 32, 8.0, 1.0), interleaved=False),
                               softmax_scale=0.2, window=window, sink=True,
                               names=(("q", "q"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"), ("uk", "uk"), ("uv", "uv"), ("o", "o"), ("sink", "sink")))
    mixer = build_mixer(spec, W, BuildContext(DEV, dtype))
    t = {p.name: rnd(*p.shape, seed=i + 1, scale=0.3 if len(p.shape) > 1 else 1.0).to(dtype) for i, p in enumerate(mixer.param_specs())}
    t["dkv.norm"] = (1.0 + 0.3 * t["dkv.norm"].float()).to(dtype)
    mixer.bind({k: d(v if len(v.shape) > 1 else v.float()) for k, v in t.items()})
    rq = mixer.cache_request()
    assert rq.single_plane and rq.num_kv_heads == 1 and rq.head_dim >= rank + dr
    xs = {0: rnd(L, W, seed=50).to(dtype), 1: rnd(30, W, seed=51).to(dtype)}
    m = {"heads": H, "dim": d_, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "scale": 0.2, "rot": rot}
    if window:
        m["mask"] = {"size": window}
    if edit is not None:
        edit(xs, t, m, eps)
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
    tol = 2e-5 if dtype == torch.float32 else bf16_tol
    for r in (0, 1):
        g = torch.cat(got[r])
        assert float((g - want[r][:g.shape[0]]).abs().max()) <= tol * float(want[r].abs().max()), r


# =============================================================================== whole models through the engine

_models = {}
_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def plain_logits(raw, tensors, ids, streams=None):
    return plain.forward(raw, {k: v.double() for k, v in tensors.items()}, ids, streams)


def model(name, dtype):
    key = (name, dtype)
    if key not in _models:
        raw, page = tz.CONFIGS[name]
        tensors = tz.make_tensors(raw, seed=7, dtype=_DT[dtype])
        reqs = {f"r{i}": tz.prompt(n, raw["vocab"], 50 + i) for i, n in enumerate([70, 33, 131, 2, 90])}
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
    worst = (0.0, None, None)
    for (rid, p), row in rows.items():
        err = float((row.double().cpu() - ref[rid][p]).abs().max()) / float(ref[rid].abs().max())
        assert err == err and err != float("inf"), (what, rid, p)
        worst = max(worst, (err, rid, p))
    assert worst[0] <= TOL[dtype], (what, worst)


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
@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_whole_prompts_and_the_stream_after_every_layer(name, dtype):
    raw, _, tensors, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    streams, want_streams = [], []
    plain_logits(raw, tensors, reqs["r0"], want_streams)
    eng.model.stream_hook = lambda pos, h: streams.append(h.double().cpu().clone())
    rows = run_steps(eng, [[("r0", reqs["r0"], 0)]])
    eng.model.stream_hook = None
    assert len(streams) == len(want_streams) == len(plain.layer_order(raw))
    if dtype == "float32":
        for i, (got, want) in enumerate(zip(streams, want_streams)):
            assert float((got - want).abs().max()) <= 2e-5 * float(want.abs().max()), f"layer run {i}"
    eng.end_request("r0")
    for rid in ("r1", "r2", "r3", "r4"):
        rows.update(run_steps(eng, [[(rid, reqs[rid], 0)]]))
        eng.end_request(rid)
    check_rows(rows, ref, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_token_by_token_from_the_first_token(name, dtype):
    """Decoding from position 0 (the first tokens of a sequence, every page border, the window's and the kept keys'
    edges passing over decoded tokens), long enough that the decode steps are replayed from a CUDA graph."""
    _, _, _, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    ids = reqs["r2"]
    rows = run_steps(eng, [[("r2", [t], i)] for i, t in enumerate(ids)])
    check_rows(rows, ref, dtype, "token by token")
    assert eng.graph_kernel_count(1) > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tz.CONFIGS))
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
@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_unequal_requests_together_and_pages_used_again(name, dtype):
    """A pool that holds two requests: five pass through, portions of one beside single tokens of another; every
    later request gets a slot (with the states of every layer run and the previous token in it) and pages that an
    earlier one gave back."""
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
@pytest.mark.parametrize("name", ["middle", "whole"])
def test_a_long_request_in_portions_then_decoded(name, dtype):
    """700 tokens: the windows have passed dozens of pages (given back meanwhile), the kept first keys are hundreds of
    positions away; prompt portions that start and end inside pages, then 40 tokens one by one."""
    raw, page, tensors, _, _ = model(name, dtype)
    ids = tz.prompt(700, raw["vocab"], 999)
    ref = {"long": plain_logits(raw, tensors, ids)}
    eng = engine_for(name, dtype, num_pages=-(-700 // page) + 1, max_requests=1)
    steps, at = [], 0
    for n in (333, 2, 190, 135):
        steps.append([("long", ids[at:at + n], at)])
        at += n
    steps += [[("long", [ids[i]], i)] for i in range(at, 700)]
    check_rows(run_steps(eng, steps), ref, dtype, "long")
    # the windows gave pages back on the way: the groups hold far fewer than 700 tokens' worth now
    held = [sum(1 for p in eng.cache.block_table("long", g) if p >= 0) for g in range(len(eng.cache.groups))]
    assert all(h * page < 300 for h, grp in zip(held, eng.cache.groups) if grp.request.window), held


@pytest.mark.parametrize("name", list(tz.CONFIGS))
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
    """A request that sits out some steps finds its previous token, its normed rows and its keys as it left them,
    while another request in the neighbouring slot runs on."""
    _, _, _, reqs, ref = model("middle", "float32")
    eng = engine_for("middle", "float32")
    a, b = reqs["r0"], reqs["r4"]
    steps = [[("r0", a[:10], 0), ("r4", b[:3], 0)], [("r4", b[3:50], 3)], [("r4", b[50:51], 50)],
             [("r0", a[10:11], 10), ("r4", b[51:52], 51)], [("r0", a[11:70], 11)], [("r4", b[52:90], 52)]]
    check_rows(run_steps(eng, steps), ref, "float32", "left out")


@pytest.mark.parametrize("name", list(tz.CONFIGS))
def test_greedy_generation_through_the_entry_point(name, tmp_path):
    """generate() (scheduler, sampling, continuous batching) gives the plain implementation's greedy tokens."""
    import os
    from safetensors.torch import load_file
    from blackwellllm_b200 import BlackwellEngine, InferenceConfig, SamplingParams
    raw, page = tz.CONFIGS[name]
    folder = tz.make_folder(name, "float32", str(tmp_path))
    W = load_file(os.path.join(folder, "model.safetensors"))
    prompts = [tz.prompt(n, raw["vocab"], 80 + n) for n in (5, 40, 1)]
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
    name = "middle"
    raw, _ = tz.CONFIGS[name]
    folder = tz.make_folder(name, "float32", str(tmp_path))
    W = load_file(os.path.join(folder, "model.safetensors"))
    prompt = tz.prompt(9, raw["vocab"], 4)
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
    name = "middle"
    raw, page = tz.CONFIGS[name]
    folder = tz.make_folder(name, dtype, str(tmp_path_factory.mktemp("zigipel")))
    W = load_file(os.path.join(folder, "model.safetensors"))
    reqs = {f"q{i}": tz.prompt(n, raw["vocab"], 200 + i) for i, n in enumerate([40, 97, 50, 70, 130, 65])}
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
    for _ in range(pick(1, 2, 3)):
        mlp = pick(None, 24, 40)
        if pick(0, 1):
            kv = pick(1, 2)
            size = pick(None, 3, 11, 40)
            layers.append(tz._attn(kv * pick(1, 2, 3), kv, pick(8, 12, 20), pick(8, 12, 20), pick(0.1, 0.3), size=size,
                                   keep=pick(None, 0, 1, 9, 50) if size else None, mlp=mlp))
        else:
            layers.append(tz._latent(pick(1, 2, 5), pick(4, 8, 12), pick(2, 6, 8), pick(4, 8, 12), pick(8, 20, 30), pick(0.1, 0.3),
                                     pick(100.0, 20000.0), size=pick(None, 2, 17, 64),
                                     scaling=pick(None, (2.0, 16, 4.0, 1.0), (16.0, 1000, 32.0, 0.25)), mlp=mlp))
    raw = {"architecture": "Zigipel", "vocab": pick(60, 130), "width": width, "norm": {"eps": pick(1e-5, 1e-3)},
           "logit_scale": pick(0.25, 1.0, 3.0), "layers": layers}
    if pick(0, 1):
        raw["embedding"] = {"bigram": {"buckets": pick(1, 7, 300), "mul_prev": pick(1, 31), "mul_cur": pick(1, 7)}}
    if pick(0, 1, 1):
        start = pick(*range(len(layers)))
        raw["loop"] = {"start": start, "stop": pick(*range(start + 1, len(layers) + 1)), "times": pick(1, 2, 3)}
    return raw, pick(8, 16)


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_float32(seed):
    from blackwellllm_b200.engine.engine import Engine
    rng = torch.Generator().manual_seed(1000 + seed)
    raw, page = _random_configuration(rng)
    tensors = tz.make_tensors(raw, seed=seed, dtype=torch.float32)
    ids = tz.prompt(90, raw["vocab"], seed)
    ref = {"a": plain_logits(raw, tensors, ids)}
    eng = Engine.from_tensors(raw, tensors, dtype="float32", page_size=page, num_pages=24, max_requests=2)
    check_rows(run_steps(eng, [[("a", ids, 0)]]), ref, "float32", f"whole {raw}")
    eng.end_request("a")
    steps, at = [], 0
    for n in (5, 2, 30, 1, 1, 17, 2, 32):
        steps.append([("a", ids[at:at + n], at)])
        at += n
    check_rows(run_steps(eng, steps), ref, "float32", f"portions {raw}")
