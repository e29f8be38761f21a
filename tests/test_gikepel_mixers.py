"""Each mixer of the Gikepel design alone, as a part with a cache entry of its own, against the plain statement of its
mechanism in `plain_gikepel.py`: the normed input goes in whole, in portions and as a batch of two sequences, and what the
mixer adds to an empty stream is compared.  Three back ends as in `test_gikepel.py`."""
import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.cache import Cache
from gpt_fast_b200.config.spec import PartSpec
from gpt_fast_b200.ops.types import BatchMeta
from gpt_fast_b200.parts import MIXERS, POSITIONS, build_part
from gpt_fast_b200.parts.residual import Branch
import plain_gikepel as pg
import plain_ops

BACKENDS = [
    pytest.param(("cpu", torch.float32), id="cpu-standin-f32"),
    pytest.param(("cuda", torch.float32), id="cuda-f32", marks=pytest.mark.gpu),
    pytest.param(("cuda", torch.bfloat16), id="cuda-bf16", marks=pytest.mark.gpu),
]
D, EPS = 40, 1e-5


@pytest.fixture(params=BACKENDS)
def backend(request):
    device, dtype = request.param
    prev = ops.use_kernels(plain_ops.PlainOps()) if device == "cpu" else None
    yield device, dtype
    if device == "cpu":
        ops.use_kernels(prev)


def rand(shape, seed, scale=1.0, shift=0.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale + shift).to(torch.bfloat16)


def run(mixer, h, seqs, cuts, device, dtype):
    """Feed the sequences (lists of row ranges of h) through the mixer as one batch, each cut at `cuts`; returns what it
    added, in h's row order."""
    cache = Cache({0: mixer.cache_needs()}, dtype, device, max_tokens=1024, max_seqs=4)
    if getattr(mixer, "position", None) is not None:
        mixer.position.prepare(cache.max_pages * cache.page_size, device)
    slots = cache.begin(len(seqs))
    out = torch.zeros(h.shape[0], D)
    bounds = [0] + list(cuts) + [max(len(s) for s in seqs)]
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        live = [(slot, s[lo:hi]) for slot, s in zip(slots, seqs) if len(s[lo:hi])]
        if not live:
            continue
        rows = [r for _, part in live for r in part]
        q_lens = [len(part) for _, part in live]
        for slot, part in live:
            cache.reserve(slot, cache.lengths_host[slot] + len(part))
        cache.sync_tables()
        cu = [0]
        for q in q_lens:
            cu.append(cu[-1] + q)
        batch = BatchMeta(torch.tensor(cu, dtype=torch.int32).to(device),
                          torch.tensor([i for i, q in enumerate(q_lens) for _ in range(q)], dtype=torch.int32).to(device),
                          torch.tensor([s for s, _ in live], dtype=torch.int32).to(device), cache.lengths, len(live), len(rows),
                          max(q_lens), max(cache.lengths_host[s] + q for (s, _), q in zip(live, q_lens)), ops.new_status(device))
        y = Branch(len(rows), D, device)
        mixer.forward(h[rows].to(dtype).to(device).contiguous(), batch, cache.view(0), residual=y, append=True)
        out[rows] = y.tensor().float().cpu()
        ops.advance_lengths(batch)
        cache.note_advance([s for s, _ in live], q_lens)
        ops.check_status(batch.status)
    return out


def judge(got, want, dtype, where):
    if dtype == torch.float32:
        torch.testing.assert_close(got, want.float(), rtol=3e-4, atol=3e-4, msg=lambda m: f"{where}\n{m}")
    else:
        scale = float(want.pow(2).mean().sqrt())
        assert float((got - want.float()).pow(2).mean().sqrt()) <= 0.03 * scale, where


def check(mixer, weights, names, plain_fn, m, backend, seed):
    device, dtype = backend
    mixer.load({k: weights[v].to(dtype if weights[v].dim() > 1 else torch.float32).to(device) for k, v in names.items()})
    h = rand((75, D), seed).float()
    a, b = list(range(0, 70)), list(range(70, 75))
    W = {"p." + k: v.double() for k, v in weights.items()}
    want = torch.cat([plain_fn(h[a].double(), W, m, EPS, "p."), plain_fn(h[b].double(), W, m, EPS, "p.")])
    for seqs, cuts, where in (([a], [], "whole"), ([a], [1, 3, 64, 66], "portions"), ([a, b], [2, 4], "a batch of two, cut")):
        got = run(mixer, h, seqs, cuts, device, dtype)
        rows = [r for s in seqs for r in s]
        judge(got[rows], want[rows], dtype, f"{type(mixer).__name__}: {where}")


def test_latent_attention_alone(backend):
    m = dict(heads=3, dim=16, rot_dim=16, vdim=8, kv_rank=32, scale=0.35,
             rot=dict(dims=16, base=300.0, scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0)))
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    w = {"q": rand((H * (d + r), D), 1, 0.3), "dkv": rand((R + r, D), 2, 0.3), "dkv.norm": rand((R,), 3, 0.2, 1.0),
         "uk": rand((H * d, R), 4, 0.3), "uv": rand((H * dv, R), 5, 0.3), "g": rand((H * dv, D), 6, 0.3), "o": rand((D, H * dv), 7, 0.3)}
    pos = build_part(POSITIONS, PartSpec("rope", dict(head_dim=r, base=300.0, scaling=dict(m["rot"]["scaling"], type="yarn"),
                                                      pairing="interleaved", freq_dtype="float64")))
    mixer = build_part(MIXERS, PartSpec("latent_attention", dict(dim=D, n_head=H, head_dim=d, rot_dim=r, v_head_dim=dv, rank=R,
                                                                 scale=m["scale"], eps=EPS)), dtype=backend[1], position=pos)
    names = dict(wq="q", wdkv="dkv", latent_norm="dkv.norm", wuk="uk", wuv="uv", wg="g", wo="o")
    check(mixer, w, names, pg.latent_attention, m, backend, seed=11)


def test_state_space_alone(backend):
    m = dict(heads=4, vdim=8, state=24, groups=2, norm_groups=4, conv=4)
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, C = H * P, H * P + 2 * G * N
    w = {"in": rand((2 * inner + 2 * G * N + H, D), 1, 0.3), "conv": rand((C, 4), 2, 0.5), "conv.b": rand((C,), 3, 0.2),
         "dt_bias": rand((H,), 4, 0.5), "A_log": rand((H,), 5, 0.5), "D": rand((H,), 6, 0.5, 1.0), "norm": rand((inner,), 7, 0.2, 1.0),
         "o": rand((D, inner), 8, 0.3)}
    mixer = build_part(MIXERS, PartSpec("state_space", dict(dim=D, n_head=H, head_dim=P, n_state=N, n_groups=G, norm_groups=4, taps=4,
                                                            eps=EPS)), dtype=backend[1], position=None)
    names = dict(w_in="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", skip="D", norm="norm", wo="o")
    check(mixer, w, names, pg.mamba2, m, backend, seed=12)


def test_delta_rule_alone(backend):
    m = dict(heads=4, kv_heads=2, dim=24, vdim=8, conv=3)
    H, J, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"q": rand((J * d, D), 1, 0.3), "k": rand((J * d, D), 2, 0.3), "v": rand((H * dv, D), 3, 0.3), "b": rand((H, D), 4, 0.3),
         "q.conv": rand((J * d, 3), 5, 0.5), "k.conv": rand((J * d, 3), 6, 0.5), "v.conv": rand((H * dv, 3), 7, 0.5),
         "a1": rand((6, D), 8, 0.3), "a2": rand((H * d, 6), 9, 0.3), "dt_bias": rand((H * d,), 10, 0.5), "A_log": rand((H,), 11, 0.5),
         "g1": rand((5, D), 12, 0.3), "g2": rand((H * dv, 5), 13, 0.3), "norm": rand((dv,), 14, 0.2, 1.0), "o": rand((D, H * dv), 15, 0.3)}
    mixer = build_part(MIXERS, PartSpec("delta_rule", dict(dim=D, n_head=H, n_qk=J, head_dim=d, v_head_dim=dv, taps=3, decay_rank=6,
                                                           gate_rank=5, eps=EPS)), dtype=backend[1], position=None)
    names = dict(wq="q", wk="k", wv="v", wb="b", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", wa1="a1", wa2="a2",
                 dt_bias="dt_bias", a_log="A_log", wg1="g1", wg2="g2", norm="norm", wo="o")
    check(mixer, w, names, pg.channel_delta, m, backend, seed=13)
