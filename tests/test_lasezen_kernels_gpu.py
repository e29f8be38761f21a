"""The mechanisms of the Lasezen decoder one at a time, each kernel against the plain statement in
`plain_lasezen.py` (64-bit): layer norm with a normed branch, the dense GELU feed-forward's product, q/k
norm and partial rotation on the way into the cache, attention with a block mask, a sink and a value head
size of its own, and retention with its carried state.  Where random inputs would hide a fault (a key far
back among hundreds, the keys on both sides of a block's edge, the sink) the inputs are made so that it shows."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.ops.types import PagedKV
import plain_lasezen as pl
from test_kernels_gpu import DEV, DTYPES, make_batch, rnd, tol

pytestmark = pytest.mark.gpu


def d64(t):
    return t.detach().double().cpu()


# ---- layer norm ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,D", [(5, 50), (3, 1000), (2, 4100), (130, 96)])
def test_layernorm_and_branch(dtype, T, D):
    x = rnd(T, D, seed=1) * 3 + 0.5
    w, b = rnd(D, dtype=dtype, seed=2) + 1, rnd(D, dtype=dtype, seed=3)
    pw, pb = rnd(D, dtype=dtype, seed=4) + 1, rnd(D, dtype=dtype, seed=5)
    out = torch.empty(T, D, dtype=dtype, device=DEV)
    ops.layernorm(x, w, b, 1e-5, out)
    torch.testing.assert_close(d64(out), pl.layer_norm(d64(x), d64(w), d64(b), 1e-5), **tol(dtype))
    # a branch, whole and as three partial sums, added with a factor and the sum normed in the same launch
    y = rnd(T, D, seed=6) * 2 - 1
    parts = torch.stack([y * 0.5, y * 0.25, y * 0.25]).contiguous()
    want_x = d64(x) + 0.6 * pl.layer_norm(d64(y), d64(pw), d64(pb), 1e-3)
    for branch in (y, parts):
        x2 = x.clone()
        ops.layernorm(x2, w, b, 1e-5, out, branch=(branch, pw, pb, 1e-3, 0.6))
        torch.testing.assert_close(d64(x2), want_x, rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(d64(out), pl.layer_norm(want_x, d64(w), d64(b), 1e-5), **tol(dtype))
        x3 = x.clone()
        ops.layernorm(x3, None, None, 0.0, None, branch=(branch, pw, pb, 1e-3, 0.6))     # the sum alone
        assert torch.equal(x3, x2)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    picked = torch.empty(2, D, dtype=dtype, device=DEV)
    ops.layernorm(x, w, b, 1e-5, picked, rows)
    torch.testing.assert_close(d64(picked), pl.layer_norm(d64(x)[[T - 1, 0]], d64(w), d64(b), 1e-5), **tol(dtype))


def test_layernorm_uses_deviations_not_raw_squares():
    """A row with a large mean: the variance must come from the deviations."""
    x = (rnd(2, 64, seed=1) * 0.01 + 30.0).contiguous()
    w, b = torch.ones(64, device=DEV), torch.zeros(64, device=DEV)
    out = torch.empty(2, 64, device=DEV)
    ops.layernorm(x, w, b, 1e-6, out)
    torch.testing.assert_close(d64(out), pl.layer_norm(d64(x), d64(w), d64(b), 1e-6), rtol=1e-3, atol=1e-3)


# ---- products with a unary activation ----------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["gelu", "gelu_tanh", "silu"])
@pytest.mark.parametrize("M,N,K", [(5, 72, 40), (1, 256, 128), (150, 384, 256), (700, 512, 256), (33, 100, 50), (8, 256, 2048),
                                   (64, 512, 1024), (130, 1024, 512)])
def test_linear_with_activation(dtype, kind, M, N, K):
    a, w = rnd(M, K, dtype=dtype, seed=1), rnd(N, K, dtype=dtype, scale=0.2, seed=2)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    ops.linear(a, w, out, mode=kind)
    z = d64(a) @ d64(w).T
    want = {"gelu": pl.gelu_erf, "gelu_tanh": pl.gelu_tanh, "silu": pl.silu}[kind](z)
    torch.testing.assert_close(d64(out), want, **tol(dtype))
    if kind != "gelu":
        assert (want - pl.gelu_erf(z)).abs().max() > 1e-4          # the three are told apart at these inputs


# ---- q/k norm, partial rotation, append ------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,rot,pairing,norm", [(6, 2, 16, 24, 0, "half", True), (3, 3, 24, 8, 16, "half", False),
                                                      (2, 1, 40, 40, 40, "half", True), (4, 2, 32, 16, 8, "interleaved", True)])
def test_qkv_prepare(dtype, H, G, d, dv, rot, pairing, norm):
    q_lens, starts = [3, 1, 70], [62, 130, 0]
    batch, table, n_pages = make_batch(q_lens, starts, 5, 64, 4, seed=2)
    T = batch.n_tokens
    W = H * d + G * d + G * dv + 8
    offs = (8, 8 + H * d, 8 + H * d + G * d)
    src = rnd(T, W, dtype=dtype, seed=3)
    qn, kn = (rnd(d, dtype=dtype, seed=4) + 1, rnd(d, dtype=dtype, seed=5) + 1) if norm else (None, None)
    kv = PagedKV(torch.zeros(n_pages, G, 64, d, dtype=dtype, device=DEV), torch.zeros(n_pages, G, 64, dv, dtype=dtype, device=DEV), table, 64)
    rt = None
    if rot:
        inv = (100.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float().to(DEV)
        rt = torch.empty(256, rot // 2, 2, device=DEV)
        ops.rope_table(inv, rt)
    q = torch.empty(T, H, d, dtype=dtype, device=DEV)
    parts = torch.stack([src.float() * 0.5, src.float() * 0.5]).contiguous()
    for source, partials in ((src, None), (None, parts)):
        kv.k_pool.zero_()
        ops.qkv_prepare(source, partials, offs, q, kv, batch, H, G, d, dv, table=rt, rot_dims=rot, pairing=pairing, q_norm=qn,
                        k_norm=kn, norm_eps=1e-5, k_scale=0.5)
        ops.check_status(batch.status)
        x = d64(src)
        at = 0
        for s, (n, p0) in enumerate(zip(q_lens, starts)):
            slot = int(batch.slots[s])
            xq = x[at:at + n, offs[0]:offs[0] + H * d].reshape(n, H, d)
            xk = x[at:at + n, offs[1]:offs[1] + G * d].reshape(n, G, d)
            xv = x[at:at + n, offs[2]:offs[2] + G * dv].reshape(n, G, dv)
            if norm:
                xq, xk = pl.unit_rms(xq, 1e-5) * d64(qn), pl.unit_rms(xk, 1e-5) * d64(kn)
            if rot and pairing == "half":
                # the plain rotation counts positions from 0: rotate a sequence of p0 + n places and keep the last n
                pad = torch.zeros(p0, H, d, dtype=torch.float64)
                xq = pl.rotate_front(torch.cat([pad, xq]), rot, 100.0)[p0:]
                xk = pl.rotate_front(torch.cat([pad[:, :G], xk]), rot, 100.0)[p0:]
            for i in range(n):
                p = p0 + i
                page = int(table[slot, p // 64])
                if not (rot and pairing == "interleaved"):
                    torch.testing.assert_close(d64(q[at + i]), xq[i], **tol(dtype))
                    torch.testing.assert_close(d64(kv.k_pool[page, :, p % 64]), xk[i] * 0.5, **tol(dtype))
                torch.testing.assert_close(d64(kv.v_pool[page, :, p % 64]), xv[i], **tol(dtype))
            at += n
    if rot and pairing == "interleaved":                    # same numbers as the half-split rotation, reordered within the rotated part
        perm = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2), torch.arange(rot, d)]).to(DEV)
        srcp = src.clone()
        for off, heads in ((offs[0], H), (offs[1], G)):
            blk = src[:, off:off + heads * d].reshape(T, heads, d)[:, :, perm]
            srcp[:, off:off + heads * d] = blk.reshape(T, heads * d)
        q2 = torch.empty_like(q)
        ops.qkv_prepare(srcp, None, offs, q2, kv, batch, H, G, d, dv, table=rt, rot_dims=rot, pairing="half",
                        q_norm=None if qn is None else qn[perm].contiguous(), k_norm=None if kn is None else kn[perm].contiguous(),
                        norm_eps=1e-5, k_scale=0.5)
        torch.testing.assert_close(q2.float(), q[:, :, perm].float(), **tol(dtype))


# ---- attention with a block mask, a sink and its own value head size ------------------------------------------------------

def run_attention(dtype, q_lens, starts, H, G, d, dv, chunk, sink, scale, k_all, v_all, q_all, force=None):
    """Put every sequence's keys and values (positions 0 .. start + q_len - 1) into pages and attend with the last
    q_len queries.  k_all / v_all / q_all: per sequence [len, G, d], [len, G, dv], [len, H, d] (float)."""
    batch, table, n_pages = make_batch(q_lens, starts, len(q_lens) + 2, 64, max(-(-(s + q) // 64) for s, q in zip(starts, q_lens)), seed=4)
    kp = torch.zeros(n_pages, G, 64, d, dtype=dtype, device=DEV)
    vp = torch.zeros(n_pages, G, 64, dv, dtype=dtype, device=DEV)
    qs = []
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        slot = int(batch.slots[s])
        for p in range(p0 + n):
            page = int(table[slot, p // 64])
            kp[page, :, p % 64] = k_all[s][p].to(dtype)
            vp[page, :, p % 64] = v_all[s][p].to(dtype)
        qs.append(q_all[s][p0:p0 + n])
    q = torch.cat(qs).to(dtype).to(DEV).contiguous()
    out = torch.empty(batch.n_tokens, H * dv, dtype=dtype, device=DEV)
    if force is None:
        ops.attention(q, PagedKV(kp, vp, table, 64), batch, out, H, G, d, scale, None, chunk, sink, dv)
    else:                                                    # one of the tensor-core kernels, named
        ops.kernels()._attention_bf16(q, PagedKV(kp, vp, table, 64), batch, out, H, G, d, scale, None, chunk=chunk, sink=sink, **force)
    ops.check_status(batch.status)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,chunk", [(6, 2, 16, 24, 5), (4, 4, 24, 16, 70), (8, 1, 64, 64, 64), (2, 1, 40, 40, 128), (3, 1, 32, 48, None)])
def test_attention_block_mask_and_sink(dtype, H, G, d, dv, chunk):
    q_lens, starts = [150, 1, 1, 3, 1], [0, 63, 64, 126, 139]           # a prompt, and decoding at and around the edges
    g = torch.Generator().manual_seed(5)
    L = [s + n for s, n in zip(starts, q_lens)]
    R = lambda *shape: torch.randn(*shape, generator=g).to(dtype).double()      # the oracle sees what the cache stores
    k_all, v_all, q_all = [R(n, G, d) for n in L], [R(n, G, dv) for n in L], [R(n, H, d) for n in L]
    sink = torch.randn(H, generator=g).to(DEV)
    out = run_attention(dtype, q_lens, starts, H, G, d, dv, chunk, sink, 0.3, k_all, v_all, q_all)
    at = 0
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        want = pl.sink_softmax_attention(q_all[s], k_all[s], v_all[s], d64(sink), 0.3, chunk)[p0:].reshape(n, H * dv)
        torch.testing.assert_close(d64(out[at:at + n]), want, **tol(dtype))
        at += n


@pytest.mark.parametrize("force", [dict(prefill=True, tiles=1), dict(prefill=True, tiles=2), dict(splits=1), dict(splits=3)],
                         ids=["prefill-one-tile", "prefill-two-tiles", "decode", "decode-three-slices"])
@pytest.mark.parametrize("H,G,d,chunk", [(8, 1, 64, 64), (4, 4, 128, 48), (6, 2, 128, 200), (8, 2, 64, 5), (2, 1, 128, 4096), (5, 1, 64, None)])
def test_tensor_core_attention_with_block_mask_and_sink(force, H, G, d, chunk):
    """The bfloat16 tensor-core kernels (prefill on tcgen05, one or two query tiles; decode, one slice or several)
    with the block mask and the sink, where blocks end inside pages, inside query tiles and between sequences."""
    if force.get("tiles") == 2 and d != 128:
        pytest.skip("the two-tile kernel is built for heads of 128")
    dtype = torch.bfloat16
    decode = "splits" in force
    q_lens, starts = ([1, 1, 1, 1, 1], [0, 63, 64, 300, 511]) if decode else ([300, 1, 70, 3, 129], [0, 63, 130, 126, 383])
    g = torch.Generator().manual_seed(9)
    L = [s + n for s, n in zip(starts, q_lens)]
    R = lambda *shape: torch.randn(*shape, generator=g).to(dtype).double()
    k_all, v_all, q_all = [R(n, G, d) for n in L], [R(n, G, d) for n in L], [R(n, H, d) for n in L]
    sink = torch.randn(H, generator=g).to(DEV) * 2
    out = run_attention(dtype, q_lens, starts, H, G, d, d, chunk, sink, 0.2, k_all, v_all, q_all, force)
    at = 0
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        want = pl.sink_softmax_attention(q_all[s], k_all[s], v_all[s], d64(sink), 0.2, chunk)[p0:].reshape(n, H * d)
        torch.testing.assert_close(d64(out[at:at + n]), want, rtol=3e-2, atol=3e-2)
        at += n
    if chunk and chunk < 300:                               # the mask matters at these sizes: plain causal attention differs
        causal = pl.sink_softmax_attention(q_all[-1], k_all[-1], v_all[-1], d64(sink), 0.2, None)[starts[-1]:].reshape(q_lens[-1], H * d)
        assert (causal - d64(out[at - q_lens[-1]:at])).abs().max() > 0.1


@pytest.mark.parametrize("force", [None, dict(prefill=True, tiles=1), dict(prefill=True, tiles=2), dict(splits=1), dict(splits=2)],
                         ids=["dispatch", "prefill-one-tile", "prefill-two-tiles", "decode", "decode-two-slices"])
def test_tensor_core_attention_block_edges_and_sink_share(force):
    """As the test below, for the tensor-core kernels: the key at the first position of the query's block is found,
    the one before it is not seen; and a sink equal to the only visible score takes half of the weight."""
    dtype, H, G, d, chunk = torch.bfloat16, 2, 1, 128, 48
    p = 48 * 6 + 40
    decode = force is not None and "splits" in force
    g = torch.Generator().manual_seed(10)
    for key_at, seen in ((288, True), (287, False), (p, True), (3, False)):
        k = torch.randn(p + 1, G, d, generator=g) * 0.1
        v = torch.randn(p + 1, G, d, generator=g)
        q = torch.randn(p + 1, H, d, generator=g) * 0.1
        q[p, :, 0] = 40.0
        k[key_at, :, 0] = 40.0
        sink = torch.full((H,), -30.0, device=DEV)
        q_lens, starts = ([1], [p]) if decode else ([p + 1], [0])
        out = run_attention(dtype, q_lens, starts, H, G, d, d, chunk, sink, 1.0, [k], [v], [q], force)[-1].float().cpu().view(H, d)
        target = v[key_at, 0].to(dtype).float()
        if seen:
            torch.testing.assert_close(out, target.expand(H, d), rtol=2e-2, atol=2e-2)
        else:
            assert (out - target).abs().max() > 0.3, f"the key at {key_at} lies outside the block of {p} and was seen"
    # position 96 starts a block: its own key is all it sees
    k, v, q = torch.zeros(97, G, d), torch.ones(97, G, d) * 2.0, torch.zeros(97, H, d)
    k[:, 0, 0], q[:, :, 0] = 2.0, 3.0                       # every score is 6 * scale = 1.5
    q_lens, starts = ([1], [96]) if decode else ([97], [0])
    for sink_value, share in ((1.5, 0.5), (60.0, 0.0), (-60.0, 1.0)):
        sink = torch.full((H,), sink_value, device=DEV)
        out = run_attention(dtype, q_lens, starts, H, G, d, d, chunk, sink, 0.25, [k], [v], [q], force)[-1:].float().cpu()
        torch.testing.assert_close(out, torch.full((1, H * d), 2.0 * share), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_attention_sees_the_block_start_and_nothing_before(dtype, decode):
    """One key is made to dominate.  At the first position of the query's block it must be found (the output is
    its value), one position earlier it must not be seen at all, however strong: in a prompt and in decoding."""
    H, G, d, dv, chunk = 2, 1, 32, 16, 48
    p = 48 * 6 + 40                                          # the query's position; its block starts at 288, on no page edge
    g = torch.Generator().manual_seed(6)
    for key_at, seen in ((288, True), (287, False), (p, True), (3, False)):
        k = torch.randn(p + 1, G, d, generator=g) * 0.1
        v = torch.randn(p + 1, G, dv, generator=g)
        q = torch.randn(p + 1, H, d, generator=g) * 0.1
        q[p, :, 0] = 40.0
        k[key_at, :, 0] = 40.0
        sink = torch.full((H,), -30.0, device=DEV)
        q_lens, starts = ([1], [p]) if decode else ([p + 1], [0])
        out = run_attention(dtype, q_lens, starts, H, G, d, dv, chunk, sink, 1.0, [k], [v], [q])[-1].float().cpu().view(H, dv)
        target = v[key_at, 0].to(dtype).float()
        if seen:
            torch.testing.assert_close(out, target.expand(H, dv), rtol=2e-2, atol=2e-2)
        else:
            assert (out - target).abs().max() > 0.3, f"the key at {key_at} lies outside the block of {p} and was seen"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_in_a_large_block(dtype):
    H, G, d, dv, chunk, p = 4, 2, 32, 48, 4096, 900
    g = torch.Generator().manual_seed(7)
    k, v, q = torch.randn(p + 1, G, d, generator=g) * 0.1, torch.randn(p + 1, G, dv, generator=g), torch.randn(p + 1, H, d, generator=g) * 0.1
    q[p, :, 1] = 40.0
    k[7, :, 1] = 40.0
    out = run_attention(dtype, [1], [p], H, G, d, dv, chunk, torch.zeros(H, device=DEV), 1.0, [k], [v], [q])[0].float().cpu().view(H, dv)
    torch.testing.assert_close(out, v[7].to(dtype).float().repeat_interleave(H // G, dim=0), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_sink_takes_its_share(dtype):
    """With one key whose score equals the sink the output is half its value; a huge sink leaves nothing, a very
    negative one changes nothing; the sink is not multiplied by the score scale."""
    H, G, d, dv = 2, 1, 16, 16
    k, v, q = torch.zeros(1, G, d), torch.ones(1, G, dv) * 2.0, torch.zeros(1, H, d)
    k[0, 0, 0], q[0, :, 0] = 2.0, 3.0                       # score = 6 * scale
    for sink_value, share in ((6.0 * 0.25, 0.5), (60.0, 0.0), (-60.0, 1.0)):
        sink = torch.full((H,), sink_value, device=DEV)
        out = run_attention(dtype, [1], [0], H, G, d, dv, 8, sink, 0.25, [k], [v], [q]).float().cpu()
        torch.testing.assert_close(out, torch.full((1, H * dv), 2.0 * share), rtol=1e-2, atol=1e-2)


# ---- retention ------------------------------------------------------------------------------------------------------------

def run_retention(dtype, q, k, v, decay, rot, base, cuts, k_scale, n_slots=3, slot=1, state=None):
    """Feed one sequence's projections [S, H, *] through the kernel in pieces; returns (o [S, H, dv], state)."""
    S, H, d = q.shape
    dv = v.shape[-1]
    src = torch.cat([q.reshape(S, -1), k.reshape(S, -1), v.reshape(S, -1)], dim=1).to(dtype).to(DEV).contiguous()
    offs = (0, H * d, 2 * H * d)
    rt = None
    if rot:
        inv = (float(base) ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float().to(DEV)
        rt = torch.empty(S + 8, rot // 2, 2, device=DEV)
        ops.rope_table(inv, rt)
    if state is None:
        state = torch.zeros(n_slots, H, d, dv, device=DEV)
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    outs, at = [], 0
    for c in list(cuts) + [S]:
        if c <= at:
            continue
        n = c - at
        batch, _, _ = make_batch([n], [at], n_slots, 64, 1)
        batch.slots[0] = slot
        batch.lengths.zero_()
        batch.lengths[slot] = at
        o = torch.empty(n, H, dv, device=DEV)
        ops.retention(src[at:c].contiguous(), offs, state, o, batch, H, d, dv, dec, table=rt, rot_dims=rot, pairing="half", k_scale=k_scale)
        ops.check_status(batch.status)
        outs.append(o)
        at = c
    return torch.cat(outs), state


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv,rot", [(3, 24, 40, 16), (2, 16, 72, 16), (1, 8, 8, 4), (4, 32, 64, 32), (2, 128, 130, 64), (5, 12, 20, 0)])
@pytest.mark.parametrize("cuts", [pytest.param([], id="whole"), pytest.param([2, 4, 70, 72, 73, 200], id="portions"),
                                  pytest.param(list(range(180, 230)), id="prefill-then-decode")])
def test_retention_against_the_recurrence(dtype, H, d, dv, rot, cuts):
    S = 230
    g = torch.Generator().manual_seed(8)
    R = lambda *shape: torch.randn(*shape, generator=g).to(dtype).double()
    q, k, v = R(S, H, d), R(S, H, d), R(S, H, dv)
    decay = [1.0 - 2.0 ** (-2 - 2 * h) for h in range(H)]
    got, state = run_retention(dtype, q, k, v, decay, rot, 500.0, cuts, d ** -0.5)
    qr = pl.rotate_front(q, rot, 500.0) if rot else q
    kr = (pl.rotate_front(k, rot, 500.0) if rot else k) * d ** -0.5
    want = pl.retention_scan(qr, kr, v, torch.tensor(decay, dtype=torch.float64))
    torch.testing.assert_close(d64(got), want, rtol=5e-4, atol=5e-4)            # 32-bit behind the projections in both types
    assert state[0].abs().sum() == 0 and state[2].abs().sum() == 0              # other sequences' state is not touched


def test_retention_remembers_the_first_token_through_a_long_decode():
    """decay close to 1: the first token's value, hundreds of steps back, is what the last query reads."""
    H, d, dv, S = 1, 16, 32, 600
    q, k, v = torch.zeros(S, H, d).double(), torch.zeros(S, H, d).double(), torch.zeros(S, H, dv).double()
    k[0, 0, 3], q[S - 1, 0, 3] = 1.0, 1.0
    v[0, 0] = torch.arange(dv).double()
    k[1:, 0, 5] = 1.0                                         # later keys are orthogonal to the last query
    v[1:] = 7.0
    decay = [0.999]
    got, _ = run_retention(torch.float32, q, k, v, decay, 0, 1.0, [64] + list(range(65, S)), 1.0)
    torch.testing.assert_close(d64(got[S - 1, 0]), 0.999 ** (S - 1) * v[0, 0], rtol=1e-4, atol=1e-5)


def test_retention_gate_divides_by_the_root_mean_square():
    T, H, dv = 5, 3, 40
    o = rnd(T, H, dv, seed=1) * 0.01
    src = rnd(T, 16 + H * dv, seed=2)
    out = torch.empty(T, H * dv, device=DEV)
    ops.retention_gate(o, src, 16, out, H, dv, 1e-5)
    want = pl.unit_rms(d64(o), 1e-5).reshape(T, -1) * pl.silu(d64(src)[:, 16:])
    torch.testing.assert_close(d64(out), want, rtol=2e-5, atol=2e-5)
    assert (want - (d64(o) / d64(o).pow(2).mean(-1, keepdim=True).sqrt()).reshape(T, -1) * pl.silu(d64(src)[:, 16:])).abs().max() > 1e-3   # eps matters here
