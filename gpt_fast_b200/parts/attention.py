"""Causal grouped-query attention with a fused q/k/v projection
(gpt-fast model.py:167-216).

Steps: qkv = h Wqkv^T; prepare q and k (rotate by each token's position, or
norm per head), append k, v to the sequence's place in the cache and attend
over the cache; residual += y Wo^T.  Query head h reads key/value head
h // (n_head / n_kv); the scale is 1/sqrt(head_dim) unless given.

Options beyond gpt-fast's attention, each off by default:
  position=None    no rotation: positions do not enter the scores
  qk_norm_eps      q and k are divided by their root mean square over the head (+ eps inside the root) and
                   multiplied by a weight [head_dim] shared by the heads (parameters q_norm, k_norm)
  chunk            a query sees only keys of its own block of `chunk` positions, blocks counted from the
                   sequence's first position
  sink             a learned number per query head (parameter sink) whose exponential joins the softmax
                   denominator; it has no key and no value and is not scaled
  v_head_dim       a head size of the values that differs from the keys'
  window           only the latest `window` positions are seen
With none of them the rotate-and-append kernel and the tensor-core attention kernels run; the others go through
`ops.qkv_prepare` and the options of `ops.attention`."""
import math
from typing import Optional

import torch

from .. import ops
from ..cache.needs import CacheNeeds, KVNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual


@register_mixer("attention")
class Attention:
    def __init__(self, dim: int, n_head: int, n_kv: int, head_dim: int, dtype: torch.dtype, position,
                 window: Optional[int] = None, scale: Optional[float] = None, v_head_dim: Optional[int] = None,
                 qk_norm_eps: Optional[float] = None, chunk: Optional[int] = None, sink: bool = False):
        if n_head % n_kv:
            raise ValueError(f"{n_head} query heads do not divide into {n_kv} key/value heads")
        if chunk is not None and chunk < 1:
            raise ValueError(f"a chunk of {chunk} positions")
        self.dim, self.n_head, self.n_kv, self.head_dim = dim, n_head, n_kv, head_dim
        self.v_head_dim = int(v_head_dim) if v_head_dim else head_dim
        self.window, self.dtype, self.position = window, dtype, position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.chunk, self.has_sink = chunk, bool(sink)
        self.plain = (position is not None and self.v_head_dim == head_dim and self.qk_norm_eps is None
                      and chunk is None and not self.has_sink and getattr(position, "head_dim", head_dim) == head_dim)
        self.wqkv = self.wo = self.q_norm = self.k_norm = self.sink = None

    def param_specs(self):
        H, G, d, dv, D = self.n_head, self.n_kv, self.head_dim, self.v_head_dim, self.dim
        specs = {"wq": ParamSpec((H * d, D)), "wk": ParamSpec((G * d, D)), "wv": ParamSpec((G * dv, D)),
                 "wo": ParamSpec((D, H * dv))}
        if self.qk_norm_eps is not None:
            specs["q_norm"] = ParamSpec((d,), "vector")
            specs["k_norm"] = ParamSpec((d,), "vector")
        if self.has_sink:
            specs["sink"] = ParamSpec((H,), "vector")
        return specs

    def load(self, tensors):
        # rows: q heads, then k heads, then v heads (gpt-fast model.py:184-189)
        self.wqkv = torch.cat([tensors["wq"], tensors["wk"], tensors["wv"]]).contiguous()
        self.wo = tensors["wo"]
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors["q_norm"], tensors["k_norm"].to(tensors["q_norm"].dtype)
        if self.has_sink:
            self._sink_stored = tensors["sink"]
            self.sink = tensors["sink"].float().contiguous()        # softmax terms are 32-bit

    def export(self):
        """The parameters as `load` received them (the way back from the fused layout)."""
        H, G, d, dv = self.n_head, self.n_kv, self.head_dim, self.v_head_dim
        wq, wk, wv = self.wqkv.split([H * d, G * d, G * dv])
        out = {"wq": wq, "wk": wk, "wv": wv, "wo": self.wo}
        if self.qk_norm_eps is not None:
            out.update(q_norm=self.q_norm, k_norm=self.k_norm)
        if self.has_sink:
            out["sink"] = self._sink_stored
        return out

    def cache_needs(self) -> CacheNeeds:
        dv = self.v_head_dim if self.v_head_dim != self.head_dim else None
        return CacheNeeds(kv=KVNeed(self.n_kv, self.head_dim, self.window, dv))

    def forward(self, h, batch, view, residual, append: bool = True):
        T = batch.n_tokens
        H, G, d, dv = self.n_head, self.n_kv, self.head_dim, self.v_head_dim
        qkv = torch.empty(T, (H + G) * d + G * dv, dtype=self.dtype, device=h.device)
        partials = ops.linear(h, self.wqkv, qkv, defer=True)      # a split sum is finished by the kernel that reads it
        y = torch.empty(T, H * dv, dtype=self.dtype, device=h.device)
        if self.plain:
            ops.rope_append_attention(qkv, partials, view.kv, batch, self.position.table, y, H, G, d, self.position.pairing,
                                      append, self.scale, self.window)
        else:
            q = torch.empty(T, H, d, dtype=self.dtype, device=h.device)
            pos = self.position
            ops.qkv_prepare(qkv, partials, (0, H * d, (H + G) * d), q, view.kv, batch, H, G, d, dv,
                            table=None if pos is None else pos.table, rot_dims=0 if pos is None else pos.head_dim,
                            pairing="half" if pos is None else pos.pairing, q_norm=self.q_norm, k_norm=self.k_norm,
                            norm_eps=self.qk_norm_eps or 0.0, append=append)
            ops.attention(q, view.kv, batch, y, H, G, d, self.scale, self.window, self.chunk, self.sink, dv)
        as_residual(residual).add_linear(y, self.wo)
