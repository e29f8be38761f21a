"""The Gikepel decoder as data: which parts each layer has and which checkpoint tensors fill which parameter.

The design: a token embedding plus a hashed bigram embedding; layers in an order that config.json lists, each a
parallel block (mixer and feed-forward read two bias-free layer norms of the same x, each result takes a learned
per-column factor, both are added at once); a final layer norm, the output product with the embedding table and a
soft cap on the logits.  Three kinds of mixer:

    'latent_attention'  softmax attention whose keys and values are expanded from a normed latent of `kv_rank`
                        numbers per token, with `rot_dim` rotated query/key dimensions (the key's shared by all heads,
                        interleaved pairs, YaRN-scaled frequencies), a given score scale and a sigmoid output gate
    'mamba2'            a selective state space with a scalar decay per head and token, a short convolution ahead of it
                        and a gated group norm behind it
    'channel_delta'     the gated delta rule with a decay per head and key channel, short convolutions on q, k, v, unit
                        q and k, a normed and gated read-out

The feed-forward is dense with the square of ReLU between its two products; a layer may have none.

config.json keys: architecture, vocab, width, norm.eps, logit_softcap, embedding.bigram {buckets, mul_prev, mul_cur},
layers [{type, mixer {...}, mlp {kind, ff} | null}].  Tensor names: embed, bigram, final.norm, l<i>.norm1 / norm2 / ls1 /
ls2, l<i>.mix.*, l<i>.mlp.{up,down}.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..config.args import ConfigError
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..weights.plan import Recipe, Source, WeightPlan
from .lasezen import _int, _num

KINDS = ("latent_attention", "mamba2", "channel_delta")


@dataclass(frozen=True)
class LayerArgs:
    kind: str
    mixer: Dict[str, Any]                  # the layer's sizes and constants, checked
    ff: Optional[int] = None               # hidden size of the feed-forward; None: the layer has none


@dataclass(frozen=True)
class GikepelArgs:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: Optional[float]
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: Tuple[LayerArgs, ...]
    source: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def to_json(self) -> Dict[str, Any]:
        return dict(self.source)


def _mixer(kind: str, m: Any, where: str) -> Dict[str, Any]:
    if kind not in KINDS:
        raise ConfigError(f"config.json: {where}'type' is {kind!r}; this design has {', '.join(KINDS)}")
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where}'mixer' must be an object")
    w = where + "mixer."
    if kind == "latent_attention":
        out = {k: _int(m, k, w) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        out["scale"] = _num(m, "scale", w)
        rot = m.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"config.json: {w}'rot' must be an object with 'dims' and 'base'")
        dims, base = _int(rot, "dims", w + "rot."), _num(rot, "base", w + "rot.")
        if dims != out["rot_dim"] or dims % 2:
            raise ConfigError(f"config.json: {w}rot.dims = {dims} must be even and equal rot_dim = {out['rot_dim']}")
        if base <= 1:
            raise ConfigError(f"config.json: {w}rot.base must exceed 1")
        scaling = rot.get("scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"config.json: {w}rot.scaling must be an object or null")
            scaling = {k: _num(scaling, k, w + "rot.scaling.") for k in ("factor", "original", "fast", "slow")}
            if scaling["factor"] <= 0 or scaling["original"] <= 0 or scaling["fast"] <= 0 or scaling["slow"] <= 0:
                raise ConfigError(f"config.json: {w}rot.scaling needs positive numbers")
        out.update(rot_base=base, rot_scaling=scaling)
        return out
    if kind == "mamba2":
        out = {k: _int(m, k, w) for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv")}
        if out["heads"] % out["groups"]:
            raise ConfigError(f"config.json: {w}{out['heads']} heads do not divide into {out['groups']} groups")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"config.json: {w}heads * vdim does not divide into {out['norm_groups']} norm_groups")
        return out
    out = {k: _int(m, k, w) for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {w}{out['heads']} heads do not divide into {out['kv_heads']} kv_heads")
    return out


def parse(cfg: Dict[str, Any]) -> GikepelArgs:
    if not isinstance(cfg, dict):
        raise ConfigError("config.json must hold one JSON object")
    layers = cfg.get("layers")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    parsed = []
    for i, L in enumerate(layers):
        where = f"layers[{i}]."
        if not isinstance(L, dict):
            raise ConfigError(f"config.json: layers[{i}] must be an object")
        mixer = _mixer(L.get("type"), L.get("mixer"), where)
        mlp, ff = L.get("mlp"), None
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {where}'mlp' must be null or an object of kind 'dense'")
            ff = _int(mlp, "ff", where + "mlp.")
        parsed.append(LayerArgs(L["type"], mixer, ff))
    norm = cfg.get("norm")
    if not isinstance(norm, dict):
        raise ConfigError("config.json: 'norm' must be an object with 'eps'")
    eps = _num(norm, "eps", "norm.")
    if eps < 0:
        raise ConfigError("config.json: norm.eps must not be negative")
    cap = cfg.get("logit_softcap")
    if cap is not None:
        cap = _num(cfg, "logit_softcap", "")
        if cap <= 0:
            raise ConfigError("config.json: logit_softcap must be positive or null")
    emb = cfg.get("embedding")
    big = emb.get("bigram") if isinstance(emb, dict) else None
    if not isinstance(big, dict):
        raise ConfigError("config.json: 'embedding.bigram' must be an object with buckets, mul_prev, mul_cur")
    return GikepelArgs(vocab=_int(cfg, "vocab", ""), width=_int(cfg, "width", ""), norm_eps=eps, logit_softcap=cap,
                       buckets=_int(big, "buckets", "embedding.bigram."), mul_prev=_int(big, "mul_prev", "embedding.bigram.", 0),
                       mul_cur=_int(big, "mul_cur", "embedding.bigram.", 0), layers=tuple(parsed), source=dict(cfg))


def build_spec(a: GikepelArgs, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> ModelSpec:
    norm = PartSpec("layernorm", dict(dim=a.width, eps=a.norm_eps, bias=False))
    layers = []
    for i, L in enumerate(a.layers):
        m, position = L.mixer, None
        if L.kind == "latent_attention":
            scaling = None if m["rot_scaling"] is None else dict(m["rot_scaling"], type="yarn")
            position = PartSpec("rope", dict(head_dim=m["rot_dim"], base=m["rot_base"], scaling=scaling, pairing="interleaved",
                                             freq_dtype="float64"))
            mixer = PartSpec("latent_attention", dict(dim=a.width, n_head=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                                                      v_head_dim=m["vdim"], rank=m["kv_rank"], scale=m["scale"], eps=a.norm_eps))
        elif L.kind == "mamba2":
            mixer = PartSpec("state_space", dict(dim=a.width, n_head=m["heads"], head_dim=m["vdim"], n_state=m["state"],
                                                 n_groups=m["groups"], norm_groups=m["norm_groups"], taps=m["conv"], eps=a.norm_eps))
        else:
            ra, rg = low_ranks(a, i, shapes)
            mixer = PartSpec("delta_rule", dict(dim=a.width, n_head=m["heads"], n_qk=m["kv_heads"], head_dim=m["dim"],
                                                v_head_dim=m["vdim"], taps=m["conv"], decay_rank=ra, gate_rank=rg, eps=a.norm_eps))
        parts = dict(mixer=mixer, mixer_norm=norm)
        if L.ff is not None:
            parts.update(feed_forward=PartSpec("dense", dict(dim=a.width, hidden=L.ff, activation="relu2")), ffn_norm=norm)
        layers.append(LayerSpec(block="parallel", parts=parts, position=position, block_params=dict(layer_scale=True)))
    spec = ModelSpec(architecture="gikepel", dim=a.width, vocab_size=a.vocab, layers=layers,
                     schedule=[ScheduleEntry(layer=i, cache=i) for i in range(len(layers))], final_norm=norm,
                     tie_embeddings=True, logit_cap=a.logit_softcap,
                     embedding=PartSpec("bigram_hash", dict(dim=a.width, buckets=a.buckets, mul_prev=a.mul_prev, mul_cur=a.mul_cur)))
    spec.validate()
    return spec


def low_ranks(a: GikepelArgs, layer: int, shapes: Optional[Dict[str, Tuple[int, ...]]]) -> Tuple[int, int]:
    """(rank of the decay projection, rank of the gate projection) of a 'channel_delta' layer.  config.json does not
    name them; the checkpoint's tensors l<i>.mix.a1 and l<i>.mix.g1 have them as their first dimension.  Without a
    checkpoint (random weights) both are a sixteenth of the width, at least 8, or `mixer.low_rank` if config.json has it."""
    if shapes is not None and f"l{layer}.mix.a1" in shapes and f"l{layer}.mix.g1" in shapes:
        return int(shapes[f"l{layer}.mix.a1"][0]), int(shapes[f"l{layer}.mix.g1"][0])
    src = a.source.get("layers", [])[layer].get("mixer", {}) if a.source else {}
    r = src.get("low_rank")
    if isinstance(r, int) and r > 0:
        return r, r
    return max(8, a.width // 16), max(8, a.width // 16)


def weight_plan(a: GikepelArgs, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> WeightPlan:
    D, V = a.width, a.vocab
    r = [Recipe("embed.weight", [Source("embed", (V, D), "embedding")]),
         Recipe("embedding.table", [Source("bigram", (a.buckets + 1, D), "embedding")]),
         Recipe("final_norm.weight", [Source("final.norm", (D,), "norm")])]
    for i, L in enumerate(a.layers):
        s, t, m = f"l{i}.", f"layers.{i}.", L.mixer
        x, y = s + "mix.", t + "mixer."
        r += [Recipe(t + "mixer_norm.weight", [Source(s + "norm1", (D,), "norm")]),
              Recipe(t + "mixer_scale.weight", [Source(s + "ls1", (D,), "norm")])]
        if L.kind == "latent_attention":
            H, d, rot, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            r += [Recipe(y + "wq", [Source(x + "q", (H * (d + rot), D))]), Recipe(y + "wdkv", [Source(x + "dkv", (R + rot, D))]),
                  Recipe(y + "latent_norm", [Source(x + "dkv.norm", (R,), "norm")]),
                  Recipe(y + "wuk", [Source(x + "uk", (H * d, R))]), Recipe(y + "wuv", [Source(x + "uv", (H * dv, R))]),
                  Recipe(y + "wg", [Source(x + "g", (H * dv, D))]), Recipe(y + "wo", [Source(x + "o", (D, H * dv))])]
        elif L.kind == "mamba2":
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, C = H * P, H * P + 2 * G * N
            r += [Recipe(y + "w_in", [Source(x + "in", (2 * inner + 2 * G * N + H, D))]),
                  Recipe(y + "conv", [Source(x + "conv", (C, taps), "conv")]), Recipe(y + "conv_bias", [Source(x + "conv.b", (C,), "bias")]),
                  Recipe(y + "dt_bias", [Source(x + "dt_bias", (H,), "bias")]), Recipe(y + "a_log", [Source(x + "A_log", (H,), "bias")]),
                  Recipe(y + "skip", [Source(x + "D", (H,), "norm")]), Recipe(y + "norm", [Source(x + "norm", (inner,), "norm")]),
                  Recipe(y + "wo", [Source(x + "o", (D, inner))])]
        else:
            H, J, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = low_ranks(a, i, shapes)
            r += [Recipe(y + "wq", [Source(x + "q", (J * d, D))]), Recipe(y + "q_conv", [Source(x + "q.conv", (J * d, taps), "conv")]),
                  Recipe(y + "wk", [Source(x + "k", (J * d, D))]), Recipe(y + "k_conv", [Source(x + "k.conv", (J * d, taps), "conv")]),
                  Recipe(y + "wv", [Source(x + "v", (H * dv, D))]), Recipe(y + "v_conv", [Source(x + "v.conv", (H * dv, taps), "conv")]),
                  Recipe(y + "wb", [Source(x + "b", (H, D))]), Recipe(y + "a_log", [Source(x + "A_log", (H,), "bias")]),
                  Recipe(y + "norm", [Source(x + "norm", (dv,), "norm")]),
                  Recipe(y + "wa1", [Source(x + "a1", (ra, D))]), Recipe(y + "wa2", [Source(x + "a2", (H * d, ra))]),
                  Recipe(y + "dt_bias", [Source(x + "dt_bias", (H * d,), "bias")]),
                  Recipe(y + "wg1", [Source(x + "g1", (rg, D))]), Recipe(y + "wg2", [Source(x + "g2", (H * dv, rg))]),
                  Recipe(y + "wo", [Source(x + "o", (D, H * dv))])]
        if L.ff is not None:
            r += [Recipe(t + "ffn_norm.weight", [Source(s + "norm2", (D,), "norm")]),
                  Recipe(t + "ffn_scale.weight", [Source(s + "ls2", (D,), "norm")]),
                  Recipe(t + "feed_forward.up", [Source(s + "mlp.up", (L.ff, D))]),
                  Recipe(t + "feed_forward.down", [Source(s + "mlp.down", (D, L.ff))])]
    return WeightPlan(recipes=r, aliases={"head.weight": "embed.weight"})


GIKEPEL = register_architecture(Architecture(
    name="gikepel", aliases=("Gikepel",), parse=parse, build_spec=build_spec, weight_plan=weight_plan, shapes_from_checkpoint=True,
))
