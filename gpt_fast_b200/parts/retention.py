"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

    q = Wq h, k = Wk h (heads x head_dim), v = Wv h (heads x v_head_dim), g = Wg h (heads x v_head_dim)
    q, k rotated by the token's position (the layer's position encoding; it may cover only the leading
    dimensions of a head), k *= head_dim^-1/2
    S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t           per head, S in 32-bit, zero at the start
    y = Wo (o / rms(o) per head * silu(g))                          rms with `eps` inside the root, no weight

The four projections are one product; the state S [heads, head_dim, v_head_dim] is the mixer's only memory, a
fixed-size per-sequence state of the cache (no keys or values are kept), carried from step to step."""
from typing import Optional, Sequence

import torch

from .. import ops
from ..cache.needs import CacheNeeds, StateNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual


@register_mixer("retention")
class Retention:
    def __init__(self, dim: int, n_head: int, head_dim: int, v_head_dim: int, decay: Sequence[float], eps: float,
                 dtype: torch.dtype, position=None, k_scale: Optional[float] = None):
        if len(decay) != n_head:
            raise ValueError(f"{len(decay)} decays for {n_head} heads")
        self.dim, self.n_head, self.head_dim, self.v_head_dim = dim, n_head, head_dim, v_head_dim
        self.decay_values = [float(x) for x in decay]
        self.eps, self.dtype, self.position = float(eps), dtype, position
        self.k_scale = float(k_scale) if k_scale is not None else float(head_dim) ** -0.5
        if position is not None and position.head_dim > head_dim:
            raise ValueError(f"the position encoding rotates {position.head_dim} dimensions, a head has {head_dim}")
        self.w_in = self.wo = self.decay = None

    def param_specs(self):
        H, d, dv, D = self.n_head, self.head_dim, self.v_head_dim, self.dim
        return {"wq": ParamSpec((H * d, D)), "wk": ParamSpec((H * d, D)), "wv": ParamSpec((H * dv, D)),
                "wg": ParamSpec((H * dv, D)), "wo": ParamSpec((D, H * dv))}

    def load(self, tensors):
        # rows: q heads, k heads, v heads, gate
        self.w_in = torch.cat([tensors["wq"], tensors["wk"], tensors["wv"], tensors["wg"]]).contiguous()
        self.wo = tensors["wo"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32).to(self.wo.device)

    def export(self):
        H, d, dv = self.n_head, self.head_dim, self.v_head_dim
        wq, wk, wv, wg = self.w_in.split([H * d, H * d, H * dv, H * dv])
        return {"wq": wq, "wk": wk, "wv": wv, "wg": wg, "wo": self.wo}

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateNeed((self.n_head, self.head_dim, self.v_head_dim), torch.float32))

    def forward(self, h, batch, view, residual, append: bool = True):
        if not append:
            raise ValueError("a retention layer owns its state: it cannot run on another run's cache entry")
        T = batch.n_tokens
        H, d, dv = self.n_head, self.head_dim, self.v_head_dim
        proj = torch.empty(T, 2 * H * (d + dv), dtype=self.dtype, device=h.device)
        ops.linear(h, self.w_in, proj)
        o = torch.empty(T, H, dv, dtype=torch.float32, device=h.device)
        pos = self.position
        ops.retention(proj, (0, H * d, 2 * H * d), view.state, o, batch, H, d, dv, self.decay,
                      table=None if pos is None else pos.table, rot_dims=0 if pos is None else pos.head_dim,
                      pairing="half" if pos is None else pos.pairing, k_scale=self.k_scale)
        y = torch.empty(T, H * dv, dtype=self.dtype, device=h.device)
        ops.retention_gate(o, proj, 2 * H * d + H * dv, y, H, dv, self.eps)
        as_residual(residual).add_linear(y, self.wo)
