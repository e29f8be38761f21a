"""Plain, slow statement of the Lasezen decoder, the oracle of its tests.

Whole sequences only: no cache, no packing, no kernels, one function per
mechanism, all on the CPU.  It shares no code with the package under test.
`P` maps checkpoint tensor names to tensors, `cfg` is the config.json dict.

The design: an embedding; layers of two kinds, each `x += m * post(mixer(pre(x)))`
and, where the layer has a feed-forward, `x += m * post(ff(pre(x)))`, with
layer norms (weight and bias) before and after each sublayer; a span of layers
may run several times in a row with the same weights; a final layer norm and
the output product.

    attention  grouped queries, q and k divided by their root mean square per head (with a
               weight), no rotation, score = q.k * scale, a query sees the keys of its own
               block of `mask.size` positions up to itself, and the softmax denominator
               holds one more term exp(sink_h) that has no value
    retention  q, k rotated on their first `rot.dims` dimensions (pairs i, i + dims/2),
               k *= dim^-1/2, S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, o divided by
               its root mean square per head, times silu(W_g h), then W_o

`act=torch.bfloat16` rounds where the library's bfloat16 path stores an
activation, which measures the noise of the format on the model at hand.
"""
import math

import torch


def rounded(x, act):
    return x if act is None else x.to(act).to(x.dtype)


def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def block_mask(n, size):
    """seen[i, j]: j <= i and both in the same block of `size` positions (size None: plain causal)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if size:
        seen = seen & (i // size == j // size)
    return seen


def sink_softmax_attention(q, k, v, sink, scale, size):
    """q [S, H, d], k [S, G, d], v [S, G, dv], sink [H] -> [S, H, dv].  The denominator of head h holds
    exp(sink_h) besides the visible keys' terms."""
    S, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    seen = block_mask(S, size)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[h].reshape(1, 1).to(s.dtype))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + torch.exp(sink[h].to(s.dtype) - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def attention_mixer(h, P, pre, mx, eps, act=None):
    S = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    f = h.dtype
    q = rounded(h @ P[pre + "q"].to(f).T, act).view(S, H, d)
    k = rounded(h @ P[pre + "k"].to(f).T, act).view(S, G, d)
    v = rounded(h @ P[pre + "v"].to(f).T, act).view(S, G, dv)
    q = rounded(unit_rms(q, eps) * P[pre + "q.norm"].to(f), act)
    k = rounded(unit_rms(k, eps) * P[pre + "k.norm"].to(f), act)
    size = (mx.get("mask") or {}).get("size")
    y = sink_softmax_attention(q, k, v, P[pre + "sink"].to(f), float(mx["scale"]), size)
    return rounded(y.reshape(S, H * dv), act) @ P[pre + "o"].to(f).T


def rotate_front(x, dims, base):
    """x [S, heads, d]: the first `dims` dimensions of each head are rotated by the position, dimension i with
    i + dims/2, angle p * base^(-2i/dims); the rest pass."""
    S = x.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / dims)).to(torch.float32)
    ang = (torch.arange(S, dtype=torch.float32)[:, None] * freq[None, :]).to(x.dtype)   # the angle is a 32-bit product
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, w = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - w * s, w * c + u * s, x[..., dims:]], dim=-1)


def retention_scan(q, k, v, decay):
    """q, k [S, H, d], v [S, H, dv], decay [H]: the recurrence, one token after the other."""
    S, H, d = q.shape
    out = torch.zeros(S, H, v.shape[-1], dtype=q.dtype)
    state = torch.zeros(H, d, v.shape[-1], dtype=q.dtype)
    for t in range(S):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    return out


def retention_mixer(h, P, pre, mx, eps, act=None):
    S = h.shape[0]
    H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
    f = h.dtype
    q = rounded(h @ P[pre + "q"].to(f).T, act).view(S, H, d)
    k = rounded(h @ P[pre + "k"].to(f).T, act).view(S, H, d)
    v = rounded(h @ P[pre + "v"].to(f).T, act).view(S, H, dv)
    g = rounded(h @ P[pre + "g"].to(f).T, act)
    q = rotate_front(q, mx["rot"]["dims"], mx["rot"]["base"])
    k = rotate_front(k, mx["rot"]["dims"], mx["rot"]["base"]) * d ** -0.5
    o = retention_scan(q, k, v, torch.tensor(mx["decay"], dtype=f))
    o = unit_rms(o, eps).reshape(S, H * dv) * silu(g)
    return rounded(o, act) @ P[pre + "o"].to(f).T


def dense_ff(h, P, pre, act=None, round_before_gelu=True):
    z = h @ P[pre + "up"].to(h.dtype).T
    return rounded(gelu_erf(rounded(z, act) if round_before_gelu else z), act) @ P[pre + "down"].to(h.dtype).T


def layer_runs(cfg):
    """The order in which layers run: a span of layers `loop.times` times in a row, the rest once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], n))


def forward(tokens, P, cfg, dtype=torch.float64, act=None, keep_layers=False, round_before_gelu=True):
    """Logits [S, vocab] of one whole sequence (and, with keep_layers, the residual stream after every layer run).
    round_before_gelu (only with act): whether the feed-forward's first product is rounded before the activation
    (a kernel that applies the activation to its 32-bit accumulator does not)."""
    eps = float(cfg["norm"]["eps"])
    m = float(cfg["residual_mult"])
    f = dtype

    def ln(x, name):
        return layer_norm(x, P[name].to(f), P[name + ".b"].to(f), eps)
    x = P["embed"].to(f)[torch.as_tensor(tokens)]
    kept = []
    for i in layer_runs(cfg):
        L = cfg["layers"][i]
        pre = f"l{i}."
        h = rounded(ln(x, pre + "norm1"), act)
        mixer = {"attention": attention_mixer, "retention": retention_mixer}[L["type"]]
        x = x + m * ln(mixer(h, P, pre + "mix.", L["mixer"], eps, act), pre + "norm1b")
        if L.get("mlp") is not None:
            h = rounded(ln(x, pre + "norm2"), act)
            x = x + m * ln(dense_ff(h, P, pre + "mlp.", act, round_before_gelu), pre + "norm2b")
        kept.append(x)
    logits = rounded(ln(x, "final.norm"), act) @ P["head"].to(f).T
    return (logits, torch.stack(kept)) if keep_layers else logits


def greedy_generate(prompt, n_new, P, cfg, dtype=torch.float64):
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(torch.argmax(forward(seq, P, cfg, dtype)[-1])))
    return seq[len(prompt):]


def load_folder(folder):
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    return load_file(os.path.join(folder, "model.safetensors")), cfg
