"""The Lasezen decoder through the whole engine, against the plain statement in `plain_lasezen.py`:
two small configurations that differ in every size and option (grouped and ungrouped heads, value heads
larger and smaller than key heads, a mask block of 5 and of 70 positions, rotation of a whole head and of
a part of it, one head, a looped span, layers with and without a feed-forward), random weights.

Every test runs three ways: the host logic on the CPU against the plain statement of the kernels, and the
kernels themselves in 32-bit and in bfloat16 on a GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gpt_fast_b200 as gf
from gpt_fast_b200 import ops
from gpt_fast_b200.engine.step import Stepper
import plain_lasezen as pl
import plain_ops
import traces
from conftest import assert_within_bf16_noise

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ["lasezen-tiny-a", "lasezen-tiny-b"]
BACKENDS = [
    pytest.param(("cpu", "float32"), id="cpu-standin-f32"),
    pytest.param(("cuda", "float32"), id="cuda-f32", marks=pytest.mark.gpu),
    pytest.param(("cuda", "bfloat16"), id="cuda-bf16", marks=pytest.mark.gpu),
]


@pytest.fixture(params=BACKENDS)
def backend(request):
    device, dtype = request.param
    prev = ops.use_kernels(plain_ops.PlainOps()) if device == "cpu" else None
    yield device, dtype
    if device == "cpu":
        ops.use_kernels(prev)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, name in enumerate(NAMES):
        d = str(tmp_path_factory.mktemp(name.replace("-", "_")))
        gf.write_model_folder(d, name, seed=31 + i, std=0.11, jitter=0.2, vector_dtype="float32" if i else "bfloat16")
        out[name] = d
    return out


_plain_cache = {}


def plain(folder, tokens):
    """(64-bit logits, logits with activations rounded to bfloat16) of the plain statement, remembered.  The
    library rounds the feed-forward's first product before the activation in one of its product kernels and not in
    the other, and the first tokens of a sequence are sensitive to it; of the two emulations the one further from
    the 64-bit logits is the measure of the format's noise."""
    key = (folder, tuple(tokens))
    if key not in _plain_cache:
        P, cfg = pl.load_folder(folder)
        want = pl.forward(tokens, P, cfg).float()
        emus = [pl.forward(tokens, P, cfg, act=torch.bfloat16, round_before_gelu=r).float() for r in (True, False)]
        _plain_cache[key] = (want, max(emus, key=lambda e: float((e - want).pow(2).mean())))
    return _plain_cache[key]


def judge(got, folder, tokens, rows, dtype, where):
    want, emu = plain(folder, tokens)
    got = got.float().cpu()
    if dtype == "float32":
        torch.testing.assert_close(got, want[rows], rtol=2e-4, atol=2e-4, msg=lambda m: f"{where}\n{m}")
    else:
        assert_within_bf16_noise(got, want[rows], emu[rows], where, rms_factor=2.0, max_factor=3.0)


def tokens_of(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def stepped(stepper, slot, toks, cuts):
    """Feed toks in pieces that end at `cuts`; logits of every position."""
    outs, at = [], 0
    for c in list(cuts) + [len(toks)]:
        if c > at:
            outs.append(stepper.step([slot], [toks[at:c]], "all"))
            at = c
    stepper.check()
    return torch.cat(outs)


def make(folder, backend, max_tokens=2048, max_seqs=8):
    device, dtype = backend
    model = gf.load(folder, dtype=dtype, device=device)
    cache = model.new_cache(max_tokens=max_tokens, max_seqs=max_seqs)
    return model, cache, Stepper(model, cache)


# ---- whole prompts, and the first tokens of a sequence ------------------------------------------------

@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(folders, backend, name):
    model, cache, st = make(folders[name], backend)
    for n in (1, 2, 6, 64, 71, 150):
        toks = tokens_of(model.vocab_size, n, seed=n)
        (slot,) = cache.begin(1)
        got = st.step([slot], [toks], "all")
        st.check()
        cache.end([slot])
        judge(got, folders[name], toks, slice(None), backend[1], f"{name}: prompt of {n}")


# ---- prefill against token-by-token decoding, portions down to two tokens, long decoding ----------------

@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("cuts", [
    pytest.param(lambda n: range(1, n), id="token-by-token"),
    pytest.param(lambda n: [40] + list(range(41, n)), id="prefill-then-long-decode"),
    pytest.param(lambda n: [2, 4, 5, 9, 10, 64, 66, 69, 70, 72, 128, 130, 139, 141], id="portions"),
    pytest.param(lambda n: [63, 65, 140], id="page-and-block-edges"),
])
def test_cuts_agree_with_the_whole(folders, backend, name, cuts):
    model, cache, st = make(folders[name], backend)
    toks = tokens_of(model.vocab_size, 143, seed=5)
    (slot,) = cache.begin(1)
    got = stepped(st, slot, toks, cuts(len(toks)))
    cache.end([slot])
    judge(got, folders[name], toks, slice(None), backend[1], f"{name}: cut prompt")
    if backend[1] == "float32":
        (slot,) = cache.begin(1)
        whole = st.step([slot], [toks], "all")
        cache.end([slot])
        torch.testing.assert_close(got, whole, rtol=1e-4, atol=1e-4)


# ---- batches of unequal requests against each alone; slots, pages and state used again ------------------

@pytest.mark.parametrize("name", NAMES)
def test_batches_and_reuse(folders, backend, name):
    model, cache, st = make(folders[name], backend, max_tokens=1024, max_seqs=4)
    V = model.vocab_size
    for round_ in range(3):                                  # the later rounds get slots and pages that were used before
        lens = [[70, 3, 131], [1, 66, 9, 20], [129, 2]][round_]
        reqs = [tokens_of(V, n + 6, seed=100 * round_ + n) for n in lens]
        slots = cache.begin(len(reqs))
        rows = {i: [] for i in range(len(reqs))}
        out = st.step(slots, [r[:n] for r, n in zip(reqs, lens)], "all")       # packed prefill
        at = 0
        for i, n in enumerate(lens):
            rows[i].append(out[at:at + n])
            at += n
        live = list(range(len(reqs)))
        for k in range(6):                                   # decode together; the shorter ones (by index) leave early
            live = [i for i in live if not (k >= 2 + 2 * i and i < len(reqs) - 1)]
            out = st.step([slots[i] for i in live], [[reqs[i][lens[i] + k]] for i in live], "all")
            for j, i in enumerate(live):
                rows[i].append(out[j:j + 1])
        st.check()
        cache.end(slots)
        for i, r in enumerate(reqs):
            got = torch.cat(rows[i])
            judge(got, folders[name], r, slice(0, got.shape[0]), backend[1], f"{name}: round {round_}, request {i}")
    assert cache.slots.n_free == cache.n_slots and all(g.pages.n_free == cache.n_pages for g in cache.kv_groups)


# ---- greedy generation through the library's entry point and scheduler -----------------------------------

@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation(folders, backend, name):
    device, dtype = backend
    model = gf.load(folders[name], dtype=dtype, device=device)
    P, cfg = pl.load_folder(folders[name])
    prompts = [tokens_of(model.vocab_size, n, seed=7 * n) for n in (5, 1, 68, 12)]
    seqs, stats = gf.generate(model, prompts, 9, temperature=0.0, batch_size=3)
    assert stats.batches == 2 and [len(s) for s in seqs] == [len(p) + 9 for p in prompts]
    for p, s in zip(prompts, seqs):
        assert s[:len(p)] == p
        logits = pl.forward(s[:-1], P, cfg).float()
        for j in range(len(p) - 1, len(s) - 1):
            margin = 1e-3 if dtype == "float32" else 0.35
            assert logits[j, s[j + 1]] >= logits[j].max() - margin, f"{name}: token {j + 1} is not the plain argmax"


# ---- a looped span has a cache entry per run; the same layer's runs must not share state --------------------

def test_loop_runs_have_their_own_cache(folders, backend):
    model, cache, st = make(folders["lasezen-tiny-a"], backend)
    sched = model.spec.schedule
    assert [e.layer for e in sched] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert len({e.cache for e in sched}) == len(sched) and all(e.owns_cache for e in sched)
    needs = model.cache_needs()
    assert sum(n.state is not None for n in needs.values()) == 4 and sum(n.kv is not None for n in needs.values()) == 4


# ---- configuration and weights ------------------------------------------------------------------------------

def test_config_errors_name_the_key():
    cfg = gf.config_from_name("lasezen-tiny-a")
    for path, value, word in [(("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "decay"), [0.5], "decay"),
                              (("layers", 0, "mixer", "kv_heads"), 4, "kv_heads"), (("loop", "stop"), 9, "loop"),
                              (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mlp", "kind"), "moe", "mlp")]:
        bad = json.loads(json.dumps(cfg))
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(gf.ConfigError, match=word):
            gf.load(bad, device="cpu", random_weights=True)


def test_weights_round_trip_and_one_error(folders, tmp_path):
    from safetensors.torch import load_file, save_file
    model = gf.load(folders["lasezen-tiny-a"], dtype="bfloat16", device="cpu")
    gf.save_folder(model, str(tmp_path / "again"))
    a, b = load_file(os.path.join(folders["lasezen-tiny-a"], "model.safetensors")), load_file(str(tmp_path / "again" / "model.safetensors"))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    broken = dict(a)
    del broken["l1.mix.g"]
    broken["l0.mix.sink"] = torch.zeros(5)
    broken["l9.extra"] = torch.zeros(1)
    os.makedirs(tmp_path / "broken")
    save_file(broken, str(tmp_path / "broken" / "model.safetensors"))
    with open(tmp_path / "broken" / "config.json", "w") as f:
        json.dump(gf.config_from_name("lasezen-tiny-a"), f)
    with pytest.raises(gf.WeightError) as e:
        gf.load(str(tmp_path / "broken"), device="cpu")
    assert e.value.missing == ["l1.mix.g"] and e.value.unexpected == ["l9.extra"] and e.value.wrong_shape[0][0] == "l0.mix.sink"


def test_replay_has_room_for_many_short_requests(folders, backend):
    """The replay's --max-tokens counts tokens, not pages: seven live requests of three tokens need seven pages."""
    from gpt_fast_b200.engine.replay import Replayer
    device, dtype = backend
    folder = folders["lasezen-tiny-b"]
    model = gf.load(folder, dtype=dtype, device=device)
    reqs = {f"r{i}": tokens_of(model.vocab_size, 3, seed=40 + i) for i in range(7)}
    rp = Replayer(model, 21, None)
    rp.run_step({"step": 0, "entries": [{"id": k, "tokens": v[:2], "want": []} for k, v in reqs.items()], "end": []})
    out = rp.run_step({"step": 1, "entries": [{"id": k, "tokens": v[2:], "want": [0]} for k, v in reqs.items()], "end": list(reqs)})
    for i, v in enumerate(reqs.values()):
        judge(torch.from_numpy(out[i:i + 1].copy()), folder, v, slice(2, 3), dtype, f"request {i}")
    assert rp.cache.slots.n_free == rp.cache.n_slots


# ---- the trace program as a user runs it ----------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(folders, tmp_path, dtype):
    folder = folders["lasezen-tiny-a"]
    V = gf.config_from_name("lasezen-tiny-a")["vocab"]
    reqs = traces.make_requests(V, [40, 3, 77, 65], seed=3)
    for cut, steps in (("whole", traces.whole(reqs)), ("stepped", traces.stepped(reqs)), ("batched", traces.batched(reqs, 3))):
        out_dir = str(tmp_path / cut)
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
               "--max-tokens", str(traces.peak_tokens(steps))]
        proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        try:
            for s in steps:
                proc.stdin.write(json.dumps(s) + "\n")
                proc.stdin.flush()
                assert proc.stdout.readline().strip() == f"done {s['step']}"
            proc.stdin.close()
            assert proc.wait(timeout=120) == 0
        finally:
            if proc.poll() is None:
                proc.kill()
        outputs = {}
        for s in steps:
            wanted = sum(len(e["want"]) for e in s["entries"])
            if wanted:
                outputs[s["step"]] = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(wanted, V)
        for (rid, j), row in traces.collect(steps, outputs, V).items():
            judge(torch.from_numpy(row.copy())[None], folder, reqs[rid], slice(j, j + 1), dtype, f"{cut}: {rid}[{j}]")
