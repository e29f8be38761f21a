"""The Gikepel decoder stated plainly: whole sequences, 64-bit, no cache, one function per mechanism.

It shares no code with the package; tests compare the package's results with it.  Weights come as a dict of
tensors under the checkpoint's own names, the configuration as the config.json dict.

    embedding        x_t = embed[tok_t] + bigram[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets]  (row `buckets` for t = 0)
    layer            x <- x + ls1 * mixer(LN_1(x)) + ls2 * ff(LN_2(x)),  LN = (x - mean) / sqrt(var + eps) * w,  both of the same x
    feed-forward     W_down relu(W_up h)^2
    latent_attention softmax attention whose keys and values are expanded from a normed latent c = rms(W_dkv h)[:rank],
                     with one rotated key part shared by all heads, an output gate sigmoid(W_g h)
    mamba2           selective state space with a scalar decay per head and token
    channel_delta    gated delta rule with a decay per head and key channel
    output           softcap(embed LN(x))
"""
import math

import torch

F64 = torch.float64


def layer_norm(x, w, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def embedding(tokens, embed, bigram, buckets, mul_prev, mul_cur):
    rows = [buckets] + [(tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(1, len(tokens))]
    return embed[torch.tensor(tokens)] + bigram[torch.tensor(rows)]


def yarn_frequencies(dims, base, scaling):
    """(frequencies [dims/2], amplitude on cos and sin)."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(dim_of(scaling["fast"])), 0)
    hi = min(math.ceil(dim_of(scaling["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, freqs, amplitude):
    """x [T, ..., dims]: pairs (2i, 2i+1) turned by positions[t] * freqs[i]; cos and sin times amplitude."""
    T = x.shape[0]
    ang = positions.to(F64)[:, None] * freqs[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [freqs.numel()]
    c, s = (torch.cos(ang) * amplitude).view(shape), (torch.sin(ang) * amplitude).view(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def causal_conv(x, w, bias=None):
    """x [T, C], w [C, taps] whose last column meets the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += x[:T - back] * w[:, j]
    if bias is not None:
        out = out + bias
    return out


def latent_attention(h, W, m, eps, prefix):
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[prefix + "q"].T).view(T, H, d + r)
    dkv = h @ W[prefix + "dkv"].T
    c = rms(dkv[:, :rank], eps) * W[prefix + "dkv.norm"]
    pos = torch.arange(T)
    freqs, amp = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    k_rot = rotate_interleaved(dkv[:, rank:], pos, freqs, amp)                   # [T, r], one for all heads
    q_rot = rotate_interleaved(q[..., d:].contiguous(), pos, freqs, amp)         # [T, H, r]
    k_un = (c @ W[prefix + "uk"].T).view(T, H, d)
    v = (c @ W[prefix + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], k_un) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    p = torch.softmax(s.masked_fill(~mask, -math.inf), dim=-1)
    y = torch.einsum("hij,jhv->ihv", p, v).reshape(T, H * dv)
    y = y * torch.sigmoid(h @ W[prefix + "g"].T)
    return y @ W[prefix + "o"].T


def mamba2(h, W, m, eps, prefix):
    T = h.shape[0]
    H, P, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    proj = h @ W[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[prefix + "conv"], W[prefix + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[prefix + "dt_bias"])                                     # [T, H]
    decay = torch.exp(-torch.exp(W[prefix + "A_log"]) * dt)
    y = torch.zeros(T, H, P, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W[prefix + "D"][hd] * x[t, hd]
    y = y.view(T, inner) * silu(z)
    y = rms(y.view(T, NG, inner // NG), eps).reshape(T, inner) * W[prefix + "norm"]
    return y @ W[prefix + "o"].T


def channel_delta(h, W, m, eps, prefix):
    T = h.shape[0]
    H, KH, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[prefix + "q"].T, W[prefix + "q.conv"])).view(T, KH, d)
    k = silu(causal_conv(h @ W[prefix + "k"].T, W[prefix + "k.conv"])).view(T, KH, d)
    v = silu(causal_conv(h @ W[prefix + "v"].T, W[prefix + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[prefix + "b"].T)                                   # [T, H]
    a = (h @ W[prefix + "a1"].T) @ W[prefix + "a2"].T + W[prefix + "dt_bias"]
    decay = torch.exp(-torch.exp(W[prefix + "A_log"])[None, :, None] * softplus(a).view(T, H, d))
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        kh = hd // (H // KH)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            o[t, hd] = S.T @ q[t, kh]
    o = rms(o, eps) * W[prefix + "norm"]
    gate = torch.sigmoid((h @ W[prefix + "g1"].T) @ W[prefix + "g2"].T).view(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ W[prefix + "o"].T


MIXERS = {"latent_attention": latent_attention, "mamba2": mamba2, "channel_delta": channel_delta}


def feed_forward(h, W, prefix):
    return torch.relu(h @ W[prefix + "up"].T) ** 2 @ W[prefix + "down"].T


def forward(cfg, weights, tokens, return_layers=False):
    """logits [T, vocab] of one sequence (64-bit); with return_layers also the residual stream after every layer."""
    W = {k: (v.to(F64) if v.dtype.is_floating_point else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    b = cfg["embedding"]["bigram"]
    x = embedding(list(tokens), W["embed"], W["bigram"], b["buckets"], b["mul_prev"], b["mul_cur"])
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[L["type"]](layer_norm(x, W[p + "norm1"], eps), W, L["mixer"], eps, p + "mix.") * W[p + "ls1"]
        if L.get("mlp") is not None:
            y = y + feed_forward(layer_norm(x, W[p + "norm2"], eps), W, p + "mlp.") * W[p + "ls2"]
        x = x + y
        layers.append(x)
    logits = layer_norm(x, W["final.norm"], eps) @ W["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(layers)) if return_layers else logits
