"""The Lasezen decoder as data: which parts each layer has, in which order layers run, and which
checkpoint tensors fill which parameter.

The design: a token embedding; layers of two kinds in an order that config.json lists, each a
sandwich block (layer norms with weight and bias before and after every sublayer, a constant
factor `residual_mult` on each branch, an optional dense GELU feed-forward); a span of layers may
run several times in a row with the same weights and a cache entry per run (`loop`); a final
layer norm and the output product.

    'attention'  grouped-query softmax attention without rotation: q and k normed per head (root mean
                 square, a weight shared by the heads), a given score scale, a block-diagonal causal mask
                 (`mask.size` positions per block) and a learned sink per head in the denominator
    'retention'  linear attention with a fixed decay per head and a 32-bit state per sequence: q and k
                 rotated on their leading `rot.dims` dimensions (half-split pairs), k times dim^-1/2,
                 the output divided by its root mean square per head and gated by silu(Wg h)

config.json keys: architecture, vocab, width, residual_mult, norm.eps, loop {start, stop, times},
layers [{type, mixer {...}, mlp {kind, ff} | null}].  Tensor names: embed, head, final.norm(.b),
l<i>.norm1 / norm1b / norm2 / norm2b (.b), l<i>.mix.{q,k,v,o,g,q.norm,k.norm,sink}, l<i>.mlp.{up,down}.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..config.args import ConfigError
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..weights.plan import Recipe, Source, WeightPlan


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be an integer >= {minimum}, found {v!r}")
    return v


def _num(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != v:
        raise ConfigError(f"config.json: {where}'{key}' must be a number, found {v!r}")
    return float(v)


@dataclass(frozen=True)
class MixerArgs:
    kind: str                              # 'attention' or 'retention'
    heads: int
    dim: int                               # per-head query/key size
    vdim: int                              # per-head value size
    kv_heads: int = 0                      # attention
    scale: float = 0.0                     # attention: factor on q . k
    chunk: Optional[int] = None            # attention: positions per mask block (None: plain causal)
    decay: Tuple[float, ...] = ()          # retention: one per head
    rot_dims: int = 0                      # retention: rotated leading dimensions of a head (0: none)
    rot_base: float = 10000.0


@dataclass(frozen=True)
class LayerArgs:
    mixer: MixerArgs
    ff: Optional[int] = None               # hidden size of the dense feed-forward; None: the layer has none


@dataclass(frozen=True)
class LasezenArgs:
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    layers: Tuple[LayerArgs, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    source: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def runs(self) -> List[int]:
        """Layer indices in running order: the loop's span `loop_times` times in a row, everything else once."""
        span = list(range(self.loop_start, self.loop_stop))
        return list(range(self.loop_start)) + span * self.loop_times + list(range(self.loop_stop, len(self.layers)))

    def to_json(self) -> Dict[str, Any]:
        return dict(self.source)


def _mixer(kind: str, m: Dict[str, Any], where: str) -> MixerArgs:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where}'mixer' must be an object")
    heads, dim, vdim = _int(m, "heads", where), _int(m, "dim", where), _int(m, "vdim", where)
    if kind == "attention":
        kv = _int(m, "kv_heads", where)
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads do not divide into {kv} kv_heads")
        mask = m.get("mask")
        chunk = None
        if mask is not None:
            if not isinstance(mask, dict):
                raise ConfigError(f"config.json: {where}'mask' must be an object or null")
            chunk = _int(mask, "size", where + "mask.")
        return MixerArgs(kind, heads, dim, vdim, kv_heads=kv, scale=_num(m, "scale", where), chunk=chunk)
    if kind == "retention":
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
            raise ConfigError(f"config.json: {where}'decay' must list one number per head ({heads})")
        rot = m.get("rot")
        rot_dims, base = 0, 10000.0
        if rot is not None:
            if not isinstance(rot, dict):
                raise ConfigError(f"config.json: {where}'rot' must be an object or null")
            rot_dims = _int(rot, "dims", where + "rot.", minimum=0)
            if rot_dims % 2 or rot_dims > dim:
                raise ConfigError(f"config.json: {where}rot.dims = {rot_dims} must be even and at most dim = {dim}")
            if rot_dims:
                base = _num(rot, "base", where + "rot.")
                if base <= 0:
                    raise ConfigError(f"config.json: {where}rot.base must be positive")
        return MixerArgs(kind, heads, dim, vdim, decay=tuple(float(x) for x in decay), rot_dims=rot_dims, rot_base=base)
    raise ConfigError(f"config.json: {where}'type' is '{kind}'; this design has 'attention' and 'retention'")


def parse(cfg: Dict[str, Any]) -> LasezenArgs:
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
        mlp = L.get("mlp")
        ff = None
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {where}'mlp' must be null or an object of kind 'dense'")
            ff = _int(mlp, "ff", where + "mlp.")
        parsed.append(LayerArgs(mixer, ff))
    norm = cfg.get("norm")
    if not isinstance(norm, dict):
        raise ConfigError("config.json: 'norm' must be an object with 'eps'")
    eps = _num(norm, "eps", "norm.")
    if eps < 0:
        raise ConfigError("config.json: norm.eps must not be negative")
    loop = cfg.get("loop")
    start = stop = 0
    times = 1
    if loop is not None:
        if not isinstance(loop, dict):
            raise ConfigError("config.json: 'loop' must be an object or null")
        start, stop = _int(loop, "start", "loop.", 0), _int(loop, "stop", "loop.", 0)
        times = _int(loop, "times", "loop.", 0)
        if not start <= stop <= len(parsed):
            raise ConfigError(f"config.json: loop spans layers {start}..{stop - 1} of {len(parsed)}")
    return LasezenArgs(vocab=_int(cfg, "vocab", ""), width=_int(cfg, "width", ""), residual_mult=_num(cfg, "residual_mult", ""),
                       norm_eps=eps, layers=tuple(parsed), loop_start=start, loop_stop=stop, loop_times=times, source=dict(cfg))


def build_spec(a: LasezenArgs) -> ModelSpec:
    norm = PartSpec("layernorm", dict(dim=a.width, eps=a.norm_eps))
    layers = []
    for L in a.layers:
        m = L.mixer
        position = None
        if m.kind == "attention":
            mixer = PartSpec("attention", dict(dim=a.width, n_head=m.heads, n_kv=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
                                               scale=m.scale, qk_norm_eps=a.norm_eps, chunk=m.chunk, sink=True))
        else:
            mixer = PartSpec("retention", dict(dim=a.width, n_head=m.heads, head_dim=m.dim, v_head_dim=m.vdim,
                                               decay=list(m.decay), eps=a.norm_eps))
            if m.rot_dims:
                position = PartSpec("rope", dict(head_dim=m.rot_dims, base=m.rot_base, pairing="half", freq_dtype="float64"))
        parts = dict(mixer=mixer, mixer_norm=norm, mixer_post_norm=norm)
        if L.ff is not None:
            parts.update(feed_forward=PartSpec("dense", dict(dim=a.width, hidden=L.ff, activation="gelu")),
                         ffn_norm=norm, ffn_post_norm=norm)
        layers.append(LayerSpec(block="sandwich", parts=parts, position=position,
                                block_params=dict(residual_mult=a.residual_mult)))
    spec = ModelSpec(architecture="lasezen", dim=a.width, vocab_size=a.vocab, layers=layers,
                     schedule=[ScheduleEntry(layer=i, cache=run) for run, i in enumerate(a.runs())],
                     final_norm=norm)
    spec.validate()
    return spec


def _norm_recipes(target: str, name: str, D: int) -> List[Recipe]:
    return [Recipe(target + ".weight", [Source(name, (D,), "norm")]), Recipe(target + ".bias", [Source(name + ".b", (D,), "bias")])]


def weight_plan(a: LasezenArgs) -> WeightPlan:
    D, V = a.width, a.vocab
    r = [Recipe("embed.weight", [Source("embed", (V, D), "embedding")]), Recipe("head.weight", [Source("head", (V, D))])]
    r += _norm_recipes("final_norm", "final.norm", D)
    for i, L in enumerate(a.layers):
        s, t, m = f"l{i}.", f"layers.{i}.", L.mixer
        r += _norm_recipes(t + "mixer_norm", s + "norm1", D) + _norm_recipes(t + "mixer_post_norm", s + "norm1b", D)
        H, d, dv = m.heads, m.dim, m.vdim
        if m.kind == "attention":
            G = m.kv_heads
            r += [Recipe(t + "mixer.wq", [Source(s + "mix.q", (H * d, D))]), Recipe(t + "mixer.wk", [Source(s + "mix.k", (G * d, D))]),
                  Recipe(t + "mixer.wv", [Source(s + "mix.v", (G * dv, D))]), Recipe(t + "mixer.wo", [Source(s + "mix.o", (D, H * dv))]),
                  Recipe(t + "mixer.q_norm", [Source(s + "mix.q.norm", (d,), "norm")]),
                  Recipe(t + "mixer.k_norm", [Source(s + "mix.k.norm", (d,), "norm")]),
                  Recipe(t + "mixer.sink", [Source(s + "mix.sink", (H,), "unit")])]
        else:
            r += [Recipe(t + "mixer.wq", [Source(s + "mix.q", (H * d, D))]), Recipe(t + "mixer.wk", [Source(s + "mix.k", (H * d, D))]),
                  Recipe(t + "mixer.wv", [Source(s + "mix.v", (H * dv, D))]), Recipe(t + "mixer.wg", [Source(s + "mix.g", (H * dv, D))]),
                  Recipe(t + "mixer.wo", [Source(s + "mix.o", (D, H * dv))])]
        if L.ff is not None:
            r += _norm_recipes(t + "ffn_norm", s + "norm2", D) + _norm_recipes(t + "ffn_post_norm", s + "norm2b", D)
            r += [Recipe(t + "feed_forward.up", [Source(s + "mlp.up", (L.ff, D))]),
                  Recipe(t + "feed_forward.down", [Source(s + "mlp.down", (D, L.ff))])]
    return WeightPlan(recipes=r)


LASEZEN = register_architecture(Architecture(
    name="lasezen", aliases=("Lasezen",), parse=parse, build_spec=build_spec, weight_plan=weight_plan,
))
