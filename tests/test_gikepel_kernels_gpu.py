"""The kernels behind the Gikepel decoder one at a time, against the plain statements in `plain_gikepel.py` and
`plain_ops.py` (64-bit): the hashed bigram embedding with its carried token, one row normed twice with scaled
branches, the squared-ReLU product, the YaRN rotary table, latent attention's prepare / per-head products / attention
on the latent, the short convolution with its carried inputs, the two recurrences with their carried state, and the
gated group norm.  Sizes are odd on purpose (heads that do not fill a warp, states that do not fill a row group)."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.ops.types import PagedKV
from gpt_fast_b200.parts.rope import Rope
import plain_gikepel as pg
from test_kernels_gpu import DEV, DTYPES, REF, make_batch, rnd, tol

pytestmark = pytest.mark.gpu


def d64(t):
    return t.detach().double().cpu()


def cpu_batch(batch):
    """The same batch for the plain operations on the CPU."""
    import dataclasses
    return dataclasses.replace(batch, **{f: getattr(batch, f).cpu() for f in ("cu_seqlens", "tok_seq", "slots", "lengths", "status")})


# ---- embedding ----------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_hashed_whole_and_in_portions(dtype):
    V, D, buckets, mp, mc = 300, 56, 37, 3_000_000_019, 7        # a multiplier beyond 32 bits
    table, extra = rnd(V, D, dtype=dtype, seed=1), rnd(buckets + 1, D, dtype=dtype, seed=2)
    toks = torch.randint(0, V, (23,), generator=torch.Generator().manual_seed(3)).tolist()
    want = pg.embedding(toks, d64(table), d64(extra), buckets, mp, mc)
    for cuts in ([23], [1, 1, 21], [5, 2, 16], [22, 1]):
        prev = torch.full((4,), -7, dtype=torch.int32, device=DEV)          # garbage of an earlier user of the slot
        got, at = [], 0
        for n in cuts:
            batch, _, _ = make_batch([n], [at], 4, 64, 2, seed=9)
            tk = torch.tensor(toks[at:at + n], dtype=torch.int32, device=DEV)
            out = torch.empty(n, D, device=DEV)
            ops.embed_hashed(tk, table, extra, out, batch, prev, buckets, mp, mc)
            ops.check_status(batch.status)
            got.append(out)
            at += n
        torch.testing.assert_close(d64(torch.cat(got)), want, rtol=1e-6, atol=1e-6)


def test_embed_hashed_batch_keeps_sequences_apart():
    V, D, buckets = 50, 16, 11
    table, extra = rnd(V, D, seed=1), rnd(buckets + 1, D, seed=2)
    seqs = [[3, 9, 4], [7], [1, 1, 1, 2]]
    batch, _, _ = make_batch([3, 1, 4], [0, 0, 0], 5, 64, 2, seed=4)
    prev = torch.zeros(5, dtype=torch.int32, device=DEV)
    out = torch.empty(8, D, device=DEV)
    ops.embed_hashed(torch.tensor(sum(seqs, []), dtype=torch.int32, device=DEV), table, extra, out, batch, prev, buckets, 5, 3)
    want = torch.cat([pg.embedding(s, d64(table), d64(extra), buckets, 5, 3) for s in seqs])
    torch.testing.assert_close(d64(out), want, rtol=1e-6, atol=1e-6)
    assert [int(prev[int(s)]) for s in batch.slots] == [4, 7, 2]


# ---- one row, two norms, scaled branches ------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,D", [(5, 50), (3, 1000), (130, 96)])
def test_layernorm_multi(dtype, T, D):
    x = rnd(T, D, seed=1) * 3 + 20.0                                      # a large mean: the variance must come from deviations
    w1, w2 = rnd(D, dtype=dtype, seed=2) + 1, rnd(D, dtype=dtype, seed=3) + 1
    s1, s2 = rnd(D, dtype=dtype, seed=4), rnd(D, dtype=dtype, seed=5)
    y1, y2 = rnd(T, D, seed=6), rnd(T, D, seed=7) * 2
    parts = torch.stack([y2 * 0.5, y2 * 0.25, y2 * 0.25]).contiguous()
    o1, o2 = torch.empty(T, D, dtype=dtype, device=DEV), torch.empty(T, D, dtype=dtype, device=DEV)
    x2 = x.clone()
    ops.layernorm_multi(x2, [(y1, s1), (parts, s2)], [(w1, 1e-5, o1), (w2, 1e-3, o2)])
    want_x = d64(x) + d64(s1) * d64(y1) + d64(s2) * d64(y2)
    torch.testing.assert_close(d64(x2), want_x, rtol=2e-6, atol=2e-5)
    torch.testing.assert_close(d64(o1), pg.layer_norm(want_x, d64(w1), 1e-5), **tol(dtype))
    torch.testing.assert_close(d64(o2), pg.layer_norm(want_x, d64(w2), 1e-3), **tol(dtype))
    x3 = x.clone()
    ops.layernorm_multi(x3, [(y1, s1), (y2, None)])                                   # the sums alone, one without a factor
    torch.testing.assert_close(d64(x3), d64(x) + d64(s1) * d64(y1) + d64(y2), rtol=2e-6, atol=2e-5)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    picked = torch.empty(2, D, dtype=dtype, device=DEV)
    ops.layernorm_multi(x, (), [(w1, 1e-5, picked)], rows)
    torch.testing.assert_close(d64(picked), pg.layer_norm(d64(x)[[T - 1, 0]], d64(w1), 1e-5), **tol(dtype))
    ops.layernorm(x, w1, None, 1e-5, picked, rows)                                    # the one-norm kernel without a bias
    torch.testing.assert_close(d64(picked), pg.layer_norm(d64(x)[[T - 1, 0]], d64(w1), 1e-5), **tol(dtype))


# ---- the squared ReLU in a product's epilogue ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(5, 72, 40), (1, 256, 128), (150, 384, 256), (700, 512, 256), (33, 100, 50), (8, 256, 2048), (130, 1024, 512)])
def test_linear_relu2(dtype, M, N, K):
    a, w = rnd(M, K, dtype=dtype, seed=1), rnd(N, K, dtype=dtype, scale=0.2, seed=2)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    ops.linear(a, w, out, mode="relu2")
    want = torch.relu(d64(a) @ d64(w).T) ** 2
    t = tol(dtype)
    torch.testing.assert_close(d64(out), want, rtol=t["rtol"], atol=t["atol"] * max(1.0, float(want.max()) ** 0.5))
    x = rnd(7, 33, dtype=dtype, seed=3)
    ops.activation(x, "relu2", out=(y := torch.empty_like(x)))
    torch.testing.assert_close(d64(y), torch.relu(d64(x)) ** 2, **t)


# ---- YaRN ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dims,base,sc", [(16, 10000.0, dict(factor=4.0, original=64, fast=8.0, slow=2.0)),
                                          (24, 300.0, dict(factor=1.0, original=4096, fast=32.0, slow=1.0)),
                                          (8, 50000.0, dict(factor=16.0, original=32, fast=4.0, slow=0.5))])
def test_yarn_table(dims, base, sc):
    rope = Rope(dims, base, dict(sc, type="yarn"), pairing="interleaved", freq_dtype="float64")
    rope.prepare(300, DEV)
    f, amp = pg.yarn_frequencies(dims, base, sc)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f.float().double()[None, :]
    torch.testing.assert_close(d64(rope.table[..., 0]), torch.cos(ang) * amp, rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(d64(rope.table[..., 1]), torch.sin(ang) * amp, rtol=1e-5, atol=2e-5)
    assert len(set(f.tolist())) == dims // 2 and (sc["factor"] == 1.0 or float(f[-1]) < base ** (-(dims - 2) / dims))


# ---- latent attention -----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,r,R,pairing", [(3, 12, 8, 20, "interleaved"), (1, 40, 2, 9, "half"), (5, 8, 16, 130, "interleaved")])
def test_latent_prepare_and_headwise(dtype, H, d, r, R, pairing):
    q_lens, starts = [3, 1, 70], [62, 130, 0]
    batch, table, n_pages = make_batch(q_lens, starts, 5, 64, 4, seed=2)
    T = batch.n_tokens
    q_off, kv_off = 8, 8 + H * (d + r) + 3
    W = kv_off + R + r + 5
    src = rnd(T, W, dtype=dtype, seed=3)
    nw = rnd(R, dtype=dtype, seed=4) + 1
    rope = Rope(r, 100.0, None, pairing=pairing)
    rope.prepare(256, DEV)
    kv = PagedKV(torch.zeros(n_pages, 1, 64, R + r, dtype=dtype, device=DEV), torch.zeros(n_pages, 1, 64, 0, dtype=dtype, device=DEV), table, 64)
    q = torch.zeros(T, H, R + r, dtype=dtype, device=DEV)
    ops.latent_prepare(src, q_off, kv_off, q, kv, batch, H, d, r, R, nw, 1e-5, rope.table, pairing)
    ops.check_status(batch.status)
    wuk = rnd(H, d, R, dtype=dtype, scale=0.3, seed=5)
    ops.headwise_linear(src, wuk, q.view(T, -1), H, d, R, a_off=q_off, a_stride=d + r, out_stride=R + r)
    kv2 = PagedKV(torch.zeros_like(kv.k_pool).cpu(), kv.v_pool.cpu(), table.cpu(), 64)
    q2 = torch.zeros(T, H, R + r, dtype=dtype)
    REF.latent_prepare(src.cpu(), q_off, kv_off, q2, kv2, cpu_batch(batch), H, d, r, R, nw.cpu(), 1e-5, rope.table.cpu(), pairing)
    REF.headwise_linear(src.cpu(), wuk.cpu(), q2.view(T, -1), H, d, R, a_off=q_off, a_stride=d + r, out_stride=R + r)
    t = tol(dtype)
    torch.testing.assert_close(d64(q), d64(q2), **t)
    torch.testing.assert_close(d64(kv.k_pool), d64(kv2.k_pool), **t)
    # many inputs per head, few outputs, with a sigmoid gate
    o = rnd(T, H * R, dtype=dtype, seed=6)
    wuv = rnd(H, R, 7, dtype=dtype, scale=0.3, seed=7)
    gate = rnd(T, H * 7 + 4, dtype=dtype, seed=8)
    y, y2 = torch.empty(T, H * 7, dtype=dtype, device=DEV), torch.empty(T, H * 7, dtype=dtype)
    ops.headwise_linear(o, wuv, y, H, R, 7, gate=gate, gate_off=4)
    REF.headwise_linear(o.cpu(), wuv.cpu(), y2, H, R, 7, gate=gate.cpu(), gate_off=4)
    torch.testing.assert_close(d64(y), d64(y2), **t)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_on_the_latent_finds_a_far_key(dtype):
    """One key row far back (and one at a page's last position) is made to stand out; values are the rows' leading part."""
    H, R, r = 3, 24, 8
    q_lens, starts = [1, 5], [700, 60]
    batch, table, n_pages = make_batch(q_lens, starts, 4, 64, 12, seed=5)
    kv = PagedKV(rnd(n_pages, 1, 64, R + r, dtype=dtype, scale=0.3, seed=1), torch.zeros(n_pages, 1, 64, 0, dtype=dtype, device=DEV), table, 64)
    q = rnd(batch.n_tokens, H, R + r, dtype=dtype, scale=0.3, seed=2)
    marked = ((0, 3, 0), (1, 63, 4))            # (sequence, key position, which of its queries looks for it)
    for s, far, which in marked:
        slot = int(batch.slots[s])
        page = int(table[slot, far // 64])
        kv.k_pool[page, 0, far % 64] = (q[int(batch.cu_seqlens[s]) + which, 1] * 40).to(dtype)     # head 1 of that query
    out = torch.empty(batch.n_tokens, H * R, dtype=dtype, device=DEV)
    ops.attention(q, kv, batch, out, H, 1, R + r, 0.5, v_head_dim=R, values_in_keys=True)
    ops.check_status(batch.status)
    out2 = torch.empty(batch.n_tokens, H * R, dtype=dtype)
    REF.attention(q.cpu(), PagedKV(kv.k_pool.cpu(), kv.v_pool.cpu(), table.cpu(), 64), cpu_batch(batch), out2, H, 1, R + r, 0.5,
                  v_head_dim=R, values_in_keys=True)
    torch.testing.assert_close(d64(out), d64(out2), **tol(dtype))
    for s, far, which in marked:
        slot, t0 = int(batch.slots[s]), int(batch.cu_seqlens[s])
        row = kv.k_pool[int(table[slot, far // 64]), 0, far % 64, :R]
        torch.testing.assert_close(d64(out[t0 + which, R:2 * R]), d64(row), rtol=0.05, atol=0.05)    # all weight on that key


# ---- short convolution ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,bias", [(4, True), (3, False), (2, True), (1, False), (7, True)])
def test_short_conv_in_portions(dtype, taps, bias):
    C, off, n = 150, 5, 31
    src = rnd(n, C + 9, dtype=dtype, seed=1)
    w = rnd(C, taps, dtype=dtype, scale=0.5, seed=2)
    b = rnd(C, dtype=dtype, seed=3) if bias else None
    want = pg.silu(pg.causal_conv(d64(src)[:, off:off + C], d64(w), None if b is None else d64(b)))
    for cuts in ([n], [1] * 6 + [n - 6], [2, 3, 1, n - 6], [n - 1, 1]):
        state = torch.zeros(3, 11 + (taps - 1) * C, device=DEV)
        got, at = [], 0
        for q in cuts:
            batch, _, _ = make_batch([q], [at], 3, 64, 2, seed=7)
            out = torch.empty(q, C, device=DEV)
            ops.short_conv(src[at:at + q].contiguous(), off, C, w, b, state, 11, out, batch)
            got.append(out)
            at += q
        torch.testing.assert_close(d64(torch.cat(got)), want, rtol=2e-5, atol=2e-5)
        assert float(state[:, :11].abs().max()) == 0.0                       # what lies ahead of the state's offset is not touched


# ---- the two recurrences --------------------------------------------------------------------------------------------------

def _state_batches(cuts, n_slots=3, seed=7):
    at = 0
    for q in cuts:
        yield at, q, make_batch([q], [at], n_slots, 64, 2, seed=seed)[0]
        at += q


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,P,N,G", [(6, 8, 12, 2), (2, 40, 70, 1), (3, 5, 16, 3), (1, 64, 128, 1)])
def test_ssd_scan_in_portions(dtype, H, P, N, G):
    n, inner = 29, H * P
    x = rnd(n, inner + 2 * G * N, seed=1) * 0.7
    dt_src = rnd(n, H + 3, dtype=dtype, seed=2)
    dt_bias, a_log, skip = rnd(H, dtype=dtype, seed=3), rnd(H, dtype=dtype, scale=0.5, seed=4), rnd(H, dtype=dtype, seed=5)
    S = n_floats = H * N * P
    want = torch.empty(n, H, P)
    state_ref = torch.zeros(3, S + 4)
    REF.ssd_scan(x.cpu(), inner, inner + G * N, dt_src.cpu(), 3, dt_bias.cpu(), a_log.cpu(), skip.cpu(), state_ref, 4, want,
                 cpu_batch(make_batch([n], [0], 3, 64, 2, seed=7)[0]), H, P, N, G)
    outs = []
    for cuts in ([n], [1] * 5 + [n - 5], [9, 2, n - 11]):
        state = torch.zeros(3, S + 4, device=DEV)
        got = []
        for at, q, batch in _state_batches(cuts):
            out = torch.empty(q, H, P, device=DEV)
            ops.ssd_scan(x[at:at + q].contiguous(), inner, inner + G * N, dt_src[at:at + q].contiguous(), 3, dt_bias, a_log, skip,
                         state, 4, out, batch, H, P, N, G)
            got.append(out)
        outs.append(torch.cat(got))
        torch.testing.assert_close(d64(outs[-1]), d64(want), rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(d64(state), d64(state_ref), rtol=2e-5, atol=2e-5)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])      # the same bits however the sequence is cut


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,J,d,dv", [(2, 2, 24, 12), (4, 2, 16, 40), (3, 1, 70, 9), (1, 1, 128, 128)])
def test_delta_rule_in_portions(dtype, H, J, d, dv):
    n = 27
    qkv = rnd(n, 2 * J * d + H * dv + 2, seed=1)
    offs = (2, 2 + J * d, 2 + 2 * J * d)
    beta_src = rnd(n, H + 1, dtype=dtype, seed=2)
    a_src = rnd(n, H * d + 6, seed=3)
    dt_bias, a_log = rnd(H * d, dtype=dtype, seed=4), rnd(H, dtype=dtype, scale=0.5, seed=5)
    S = H * d * dv
    want, state_ref = torch.empty(n, H, dv), torch.zeros(3, S)
    REF.delta_rule(qkv.cpu(), offs, beta_src.cpu(), 1, a_src.cpu(), 6, dt_bias.cpu(), a_log.cpu(), state_ref, 0, want,
                   cpu_batch(make_batch([n], [0], 3, 64, 2, seed=7)[0]), H, J, d, dv, d ** -0.5)
    outs = []
    for cuts in ([n], [1] * 4 + [n - 4], [8, 2, 1, n - 11]):
        state = torch.zeros(3, S, device=DEV)
        got = []
        for at, q, batch in _state_batches(cuts):
            out = torch.empty(q, H, dv, device=DEV)
            ops.delta_rule(qkv[at:at + q].clone(), offs, beta_src[at:at + q].contiguous(), 1, a_src[at:at + q].clone(), 6,      # scratch: overwritten
                           dt_bias, a_log, state, 0, out, batch, H, J, d, dv, d ** -0.5)
            got.append(out)
        outs.append(torch.cat(got))
        torch.testing.assert_close(d64(outs[-1]), d64(want), rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(d64(state), d64(state_ref), rtol=2e-5, atol=2e-5)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_delta_rule_reads_its_own_write_and_forgets_by_channel():
    """One head, beta = 1, no decay: after writing (k, v) the read-out with q = k returns v exactly (the current
    token's write is seen); with a strong decay on one key channel only that channel's memory fades."""
    d, dv = 4, 3
    k = torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0], [1.0, 0, 0, 0], [0, 1.0, 0, 0]])
    v = torch.tensor([[1.0, 2, 3], [4.0, 5, 6], [0.0, 0, 0], [0.0, 0, 0]])
    qkv = torch.cat([k * 5, k * 5, v], dim=1).to(DEV).contiguous()              # q = k (made unit vectors by the kernel)
    beta = torch.tensor([[30.0], [30.0], [-30.0], [-30.0]], device=DEV)         # sigmoid: 1, 1, 0, 0 (the last two only read)
    a = torch.full((4, d), -40.0, device=DEV)                                   # softplus -> 0: no decay ...
    a[2:, 1] = 3.0                                                              # ... but channel 1 fades in the last two tokens
    state = torch.zeros(1, d * dv, device=DEV)
    out = torch.empty(4, 1, dv, device=DEV)
    batch, _, _ = make_batch([4], [0], 1, 64, 2)
    ops.delta_rule(qkv, (0, d, 2 * d), beta, 0, a, 0, torch.zeros(d, device=DEV), torch.zeros(1, device=DEV), state, 0, out, batch,
                   1, 1, d, dv, 1.0)
    g = math.exp(-math.log1p(math.exp(3.0)))
    want = torch.tensor([[1.0, 2, 3], [4.0, 5, 6], [1.0, 2, 3], [4 * g * g, 5 * g * g, 6 * g * g]])
    torch.testing.assert_close(out[:, 0].cpu(), want, rtol=1e-5, atol=1e-5)


# ---- gated group norm ------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("groups,gs,shared,act,first", [(2, 96, False, "silu", True), (5, 9, True, "sigmoid", False), (1, 300, False, "silu", True),
                                                        (7, 64, True, "sigmoid", False)])
def test_gated_norm(dtype, groups, gs, shared, act, first):
    T, C = 6, groups * gs
    y = rnd(T, C, seed=1) * 2
    gate = rnd(T, C + 5, dtype=dtype, seed=2)
    w = rnd(gs if shared else C, dtype=dtype, seed=3) + 1
    out, out2 = torch.empty(T, C, dtype=dtype, device=DEV), torch.empty(T, C, dtype=dtype)
    ops.gated_norm(y, gate, 5, w, out, gs, 1e-5, act=act, gate_first=first)
    REF.gated_norm(y.cpu(), gate.cpu(), 5, w.cpu(), out2, gs, 1e-5, act=act, gate_first=first)
    torch.testing.assert_close(d64(out), d64(out2), **tol(dtype))
    z = d64(gate)[:, 5:]
    a = torch.sigmoid(z) if act == "sigmoid" else pg.silu(z)
    v = d64(y) * a if first else d64(y)
    n = pg.rms(v.view(T, groups, gs), 1e-5).reshape(T, C) * d64(w).repeat(C // w.numel())
    torch.testing.assert_close(d64(out), n if first else n * a, **tol(dtype))


# ---- attention on the latent with many queries: the tensor-core kernel -----------------------------------------------------

@pytest.mark.parametrize("H,R,r", [(16, 64, 16), (3, 48, 16), (5, 512, 64), (1, 16, 16), (8, 128, 32)])
def test_latent_attention_many_queries(H, R, r):
    """Portions that start at 0, in the middle of a tile of 32 keys, at a page's edge and far into a sequence; heads
    that do not fill the 16 rows of an MMA; every row masked by its own position."""
    dtype = torch.bfloat16
    q_lens, starts = [70, 33, 2, 5], [0, 61, 31, 640]
    _latent_attention_case(H, R, r, q_lens, starts)


@pytest.mark.parametrize("H,R,r", [(16, 64, 16), (3, 48, 16), (40, 32, 16)])
def test_latent_attention_decode_step(H, R, r):
    """One query per sequence: a sequence's heads are the rows of the MMA (40 heads: three row tiles, the last part-filled)."""
    _latent_attention_case(H, R, r, [1, 1, 1, 1], [0, 31, 64, 644], marked=((0, 7), (0, 643)))


def _latent_attention_case(H, R, r, q_lens, starts, marked=((1, 7), (4, 643))):
    dtype = torch.bfloat16
    batch, table, n_pages = make_batch(q_lens, starts, 6, 64, 12, seed=3)
    kv = PagedKV(rnd(n_pages, 1, 64, R + r, dtype=dtype, scale=0.5, seed=1), torch.zeros(n_pages, 1, 64, 0, dtype=dtype, device=DEV), table, 64)
    q = rnd(batch.n_tokens, H, R + r, dtype=dtype, scale=0.5, seed=2)
    # the last sequence's second query looks for a key far back, its last query for the key just before it
    slot, t0 = int(batch.slots[3]), int(batch.cu_seqlens[3])
    for which, key in marked[-1:] if marked[0][0] == marked[1][0] else marked:
        kv.k_pool[int(table[slot, key // 64]), 0, key % 64] = (q[t0 + which, H - 1] * 30).to(dtype)
    out = torch.empty(batch.n_tokens, H * R, dtype=dtype, device=DEV)
    with ops.trace() as rec:
        ops.attention(q, kv, batch, out, H, 1, R + r, 0.3, v_head_dim=R, values_in_keys=True)
    assert [label for label, _, _ in rec] == ["gfb_latent_attention"]
    ops.check_status(batch.status)
    out2 = torch.empty(batch.n_tokens, H * R, dtype=dtype)
    REF.attention(q.cpu(), PagedKV(kv.k_pool.cpu(), kv.v_pool.cpu(), table.cpu(), 64), cpu_batch(batch), out2, H, 1, R + r, 0.3,
                  v_head_dim=R, values_in_keys=True)
    torch.testing.assert_close(d64(out), d64(out2), rtol=3e-2, atol=3e-2)
    for which, key in marked[-1:] if marked[0][0] == marked[1][0] else marked:
        row = kv.k_pool[int(table[slot, key // 64]), 0, key % 64, :R]
        torch.testing.assert_close(d64(out[t0 + which, (H - 1) * R:]), d64(row), rtol=0.05, atol=0.05)
