"""The Gikepel decoder through the whole engine, against the plain statement in `plain_gikepel.py`: two small
configurations that differ in every size and option (one and several heads, grouped and ungrouped query/key heads,
value heads larger and smaller than key heads, rotated parts of other sizes than the unrotated, with and without the
YaRN rule and the logit cap, state sizes that fill one or several row groups of the kernels, convolutions of 2 to 5
taps, layers with and without a feed-forward, every order of the three mixers), random weights.

Every test runs three ways: the host logic on the CPU against the plain statement of the kernels, and the kernels
themselves in 32-bit and in bfloat16 on a GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
from safetensors.torch import load_file

import gpt_fast_b200 as gf
from gpt_fast_b200 import ops
from gpt_fast_b200.engine.step import Stepper
import plain_gikepel as pg
import plain_ops
import traces

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ["gikepel-tiny-a", "gikepel-tiny-b"]
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
        gf.write_model_folder(d, name, seed=41 + i, std=0.11, jitter=0.2, vector_dtype="float32" if i else "bfloat16")
        out[name] = d
    return out


_plain_cache = {}


def plain(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain_cache:
        with open(os.path.join(folder, "config.json")) as f:
            cfg = json.load(f)
        _plain_cache[key] = pg.forward(cfg, load_file(os.path.join(folder, "model.safetensors")), tokens).float()
    return _plain_cache[key]


def judge(got, folder, tokens, rows, dtype, where):
    """32-bit: equal to rounding.  bfloat16: within a few per cent of the logits' own scale in the mean and a sixth of it
    at the worst element; a wrong token, key, page or state moves logits by about their scale."""
    want = plain(folder, tokens)[rows]
    got = got.float().cpu()
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=3e-4, atol=3e-4, msg=lambda m: f"{where}\n{m}")
    else:
        scale = float(want.pow(2).mean().sqrt())
        err = got - want
        assert float(err.pow(2).mean().sqrt()) <= 0.04 * scale, f"{where}: rms error {float(err.pow(2).mean().sqrt()):.4f} of scale {scale:.4f}"
        assert float(err.abs().max()) <= 0.17 * scale + 0.02, f"{where}: max error {float(err.abs().max()):.4f} of scale {scale:.4f}"


def tokens_of(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def stepped(stepper, slot, toks, cuts):
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
    for n in (1, 2, 3, 6, 64, 71, 150):
        toks = tokens_of(model.vocab_size, n, seed=n)
        (slot,) = cache.begin(1)
        got = st.step([slot], [toks], "all")
        st.check()
        cache.end([slot])
        judge(got, folders[name], toks, slice(None), backend[1], f"{name}: prompt of {n}")


def test_a_repeated_token_and_the_first_token(folders, backend):
    """The hashed table's row depends on the token before: the same token gives other logits at the start of a
    sequence, behind itself and behind another token."""
    name = NAMES[0]
    model, cache, st = make(folders[name], backend)
    for toks in ([7, 7, 7, 9, 7], [9], [9, 9]):
        (slot,) = cache.begin(1)
        got = stepped(st, slot, toks, range(1, len(toks)))
        cache.end([slot])
        judge(got, folders[name], toks, slice(None), backend[1], f"{name}: {toks}")


# ---- prefill against token-by-token decoding, portions down to two tokens, long decoding ----------------

@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("cuts", [
    pytest.param(lambda n: range(1, n), id="token-by-token"),
    pytest.param(lambda n: [20] + list(range(21, n)), id="prefill-then-long-decode"),
    pytest.param(lambda n: [2, 4, 5, 9, 10, 64, 66, 69, 70, 72, 128, 130, 139, 141], id="portions"),
    pytest.param(lambda n: [63, 65, 140], id="page-edges"),
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
    for round_ in range(3):                                  # the later rounds get slots, pages and state that were used before
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
    prompts = [tokens_of(model.vocab_size, n, seed=7 * n) for n in (5, 1, 68, 12)]
    seqs, stats = gf.generate(model, prompts, 9, temperature=0.0, batch_size=3)
    assert stats.batches == 2 and [len(s) for s in seqs] == [len(p) + 9 for p in prompts]
    for p, s in zip(prompts, seqs):
        assert s[:len(p)] == p
        logits = plain(folders[name], s[:-1])
        for j in range(len(p) - 1, len(s) - 1):
            margin = 1e-3 if dtype == "float32" else 0.05 * float(logits[j].pow(2).mean().sqrt()) + 0.05
            assert logits[j, s[j + 1]] >= logits[j].max() - margin, f"{name}: token {j + 1} is not the plain argmax"


# ---- what the model asks of the cache -----------------------------------------------------------------------

def test_cache_entries(folders, backend):
    model, cache, st = make(folders[NAMES[1]], backend)
    needs = model.cache_needs()
    assert needs[-1].state.dtype == torch.int32                                   # the embedding's carried token
    kinds = [("kv" if needs[i].kv is not None else "state") for i in range(4)]
    assert kinds == ["kv", "state", "state", "kv"]
    assert all(not g.need.values and g.v_pool.numel() == 0 and g.need.n_kv == 1 for g in cache.kv_groups)   # only the latent is kept
    assert {g.need.head_dim for g in cache.kv_groups} == {12 + 8, 24 + 4}
    d, dv, taps = 20, 32, 5
    assert needs[1].state.shape == (2 * d * dv + (taps - 1) * (2 * d + 2 * dv),)


# ---- configuration and weights ------------------------------------------------------------------------------

def test_config_errors_name_the_key():
    cfg = gf.config_from_name("gikepel-tiny-a")
    for path, value, word in [(("layers", 0, "type"), "attention", "type"), (("layers", 0, "mixer", "groups"), 3, "groups"),
                              (("layers", 1, "mixer", "rot", "dims"), 4, "rot.dims"), (("layers", 2, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 0, "mlp", "kind"), "moe", "mlp"), (("embedding", "bigram", "buckets"), 0, "buckets"),
                              (("logit_softcap",), -1.0, "logit_softcap"), (("layers", 0, "mixer", "norm_groups"), 5, "norm_groups")]:
        bad = json.loads(json.dumps(cfg))
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(gf.ConfigError, match=word):
            gf.load(bad, device="cpu", random_weights=True)


def test_weights_round_trip_and_one_error(folders, tmp_path):
    from safetensors.torch import save_file
    name = NAMES[0]
    model = gf.load(folders[name], dtype="bfloat16", device="cpu")
    gf.save_folder(model, str(tmp_path / "again"))
    a, b = load_file(os.path.join(folders[name], "model.safetensors")), load_file(str(tmp_path / "again" / "model.safetensors"))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    broken = dict(a)
    del broken["l1.mix.uk"]
    broken["l0.mix.conv"] = torch.zeros(5, 3)
    broken["l9.extra"] = torch.zeros(1)
    os.makedirs(tmp_path / "broken")
    save_file(broken, str(tmp_path / "broken" / "model.safetensors"))
    with open(tmp_path / "broken" / "config.json", "w") as f:
        json.dump(gf.config_from_name(name), f)
    with pytest.raises(gf.WeightError) as e:
        gf.load(str(tmp_path / "broken"), device="cpu")
    assert e.value.missing == ["l1.mix.uk"] and e.value.unexpected == ["l9.extra"] and e.value.wrong_shape[0][0] == "l0.mix.conv"


def test_low_ranks_come_from_the_tensor_shapes(folders, tmp_path, plain_kernels):
    """config.json does not name the ranks of the delta rule's decay and gate projections: the checkpoint's shapes do."""
    from safetensors.torch import save_file
    name = NAMES[0]
    w = load_file(os.path.join(folders[name], "model.safetensors"))
    g = torch.Generator().manual_seed(1)
    w["l2.mix.a1"] = (torch.randn(5, 48, generator=g) * 0.1).to(torch.bfloat16)
    w["l2.mix.a2"] = (torch.randn(48, 5, generator=g) * 0.1).to(torch.bfloat16)
    w["l2.mix.g1"] = (torch.randn(11, 48, generator=g) * 0.1).to(torch.bfloat16)
    w["l2.mix.g2"] = (torch.randn(20, 11, generator=g) * 0.1).to(torch.bfloat16)
    os.makedirs(tmp_path / "m")
    save_file(w, str(tmp_path / "m" / "model.safetensors"))
    cfg = gf.config_from_name(name)
    del cfg["layers"][2]["mixer"]["low_rank"]
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    model = gf.load(str(tmp_path / "m"), dtype="float32", device="cpu")
    toks = tokens_of(cfg["vocab"], 9, seed=2)
    cache = model.new_cache(max_tokens=64, max_seqs=1)
    got = Stepper(model, cache).step(cache.begin(1), [toks], "all")
    torch.testing.assert_close(got, pg.forward(cfg, w, toks).float(), rtol=3e-4, atol=3e-4)


# ---- the trace program as a user runs it ----------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(folders, tmp_path, dtype):
    name = NAMES[1]
    folder = folders[name]
    V = gf.config_from_name(name)["vocab"]
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


# ---- long decoding: the states carry over hundreds of steps ------------------------------------------------------

def test_long_decoding(folders, backend):
    name = NAMES[0]
    model, cache, st = make(folders[name], backend)
    toks = tokens_of(model.vocab_size, 330, seed=9)
    (slot,) = cache.begin(1)
    got = stepped(st, slot, toks, [5] + list(range(6, len(toks))))
    cache.end([slot])
    judge(got[-40:], folders[name], toks, slice(len(toks) - 40, len(toks)), backend[1], f"{name}: the last of 325 decode steps")


# ---- the command line as a user runs it ----------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cli_greedy(folders, tmp_path, dtype):
    from test_cli_gpu import read_lines, run_cli
    name = NAMES[1]
    out = tmp_path / "tokens.jsonl"
    r = run_cli("--checkpoint_path", folders[name], "--prompt", "4,13", "--max_new_tokens", "7", "--temperature", "0",
                "--dtype", dtype, "--output", str(out))
    assert r.returncode == 0, r.stderr[-2000:]
    rows = read_lines(out)
    assert [len(x["prompt"]) for x in rows] == [4, 13]
    for x in rows:
        assert len(x["tokens"]) == 7
        seq = list(x["prompt"])
        for tok in x["tokens"]:
            logits = plain(folders[name], seq)[-1]
            margin = 1e-3 if dtype == "float32" else 0.05 * float(logits.pow(2).mean().sqrt()) + 0.05
            if tok != int(torch.argmax(logits)):
                assert logits[tok] >= logits.max() - margin, f"request {x['request']}: chose {tok}"
                break                                          # a near tie turned the other way: the sequences part here
            seq.append(tok)


# ---- other orders of layers, widths that no 16-byte kernel takes ----------------------------------------------------

@pytest.mark.parametrize("which", ["no-attention", "only-attention", "one-layer", "one-tap"])
def test_other_layer_orders(tmp_path, backend, which):
    """Models without any cached keys, without any recurrent state, of one layer, with convolutions of one tap; width 52 and
    vocabulary 97, so that the bfloat16 products take the kernels for rows that are no whole 16-byte units."""
    device, dtype = backend
    base = gf.config_from_name(NAMES[0])
    L = base["layers"]
    layers = {"no-attention": [L[0], L[2], L[0]], "only-attention": [L[1], L[1]], "one-layer": [L[2]],
              "one-tap": [dict(L[0], mixer=dict(L[0]["mixer"], conv=1)), dict(L[2], mixer=dict(L[2]["mixer"], conv=1))]}[which]
    cfg = dict(base, layers=json.loads(json.dumps(layers)), width=52, vocab=97)
    folder = str(tmp_path / which)
    gf.write_model_folder(folder, cfg, seed=3, std=0.11, jitter=0.2)
    model = gf.load(folder, dtype=dtype, device=device)
    cache = model.new_cache(max_tokens=256, max_seqs=2)
    st = Stepper(model, cache)
    toks = tokens_of(97, 70, seed=8)
    (slot,) = cache.begin(1)
    got = stepped(st, slot, toks, [33, 34])
    cache.end([slot])
    judge(got, folder, toks, slice(None), dtype, which)
