"""Latent attention: keys and values of all heads are expanded from one small latent vector per token.

    q = Wq h                          per head: head_dim unrotated numbers, then rot_dim rotated ones
    (l, k_r) = Wdkv h                 l: rank numbers, k_r: rot_dim numbers shared by all heads
    c = l / rms(l) * norm             the latent (root mean square with eps inside the root)
    k_h = Wuk,h c,  v_h = Wuv,h c     expanded keys (head_dim) and values (v_head_dim)
    s_h(i, j) = scale (q_u,h,i . k_h,j + rot(q_r,h,i) . rot(k_r,j)),  causal softmax,  o_h = sum_j p v_h,j
    y = Wo (concat_h o_h * sigmoid(Wg h))

Only (c, rot(k_r)) is cached: one row of rank + rot_dim numbers per token.  Since k_h and v_h are linear in c, the
mixer attends on the latent itself: the query of head h becomes [Wuk,h^T q_u,h | rot(q_r,h)] (rank + rot_dim numbers),
all heads read the same cached rows as keys and their first rank numbers as values, and Wuv,h expands the attended
latent afterwards.  Nothing is ever expanded per cached token, in prompts or in decoding."""
from typing import Optional

import torch

from .. import ops
from ..cache.needs import CacheNeeds, KVNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual


@register_mixer("latent_attention")
class LatentAttention:
    def __init__(self, dim: int, n_head: int, head_dim: int, rot_dim: int, v_head_dim: int, rank: int, scale: float, eps: float,
                 dtype: torch.dtype, position, window: Optional[int] = None):
        if position is None or position.head_dim != rot_dim:
            raise ValueError(f"latent attention rotates {rot_dim} dimensions; its position encoding must cover exactly those")
        self.dim, self.n_head, self.head_dim, self.rot_dim, self.v_head_dim, self.rank = dim, n_head, head_dim, rot_dim, v_head_dim, rank
        self.scale, self.eps, self.dtype, self.position, self.window = float(scale), float(eps), dtype, position, window
        self.w_in = self.wuk = self.wuv = self.wo = self.latent_norm = None

    def param_specs(self):
        H, d, r, dv, R, D = self.n_head, self.head_dim, self.rot_dim, self.v_head_dim, self.rank, self.dim
        return {"wq": ParamSpec((H * (d + r), D)), "wdkv": ParamSpec((R + r, D)), "wg": ParamSpec((H * dv, D)),
                "wuk": ParamSpec((H * d, R)), "wuv": ParamSpec((H * dv, R)), "wo": ParamSpec((D, H * dv)),
                "latent_norm": ParamSpec((R,), "vector")}

    def load(self, tensors):
        # rows of the fused projection: queries, down projection, gate
        self.w_in = torch.cat([tensors["wq"], tensors["wdkv"], tensors["wg"]]).contiguous()
        self.wuk = tensors["wuk"].view(self.n_head, self.head_dim, self.rank)         # [H][k = head_dim][n = rank]
        self.wuv = tensors["wuv"].view(self.n_head, self.v_head_dim, self.rank).transpose(1, 2).contiguous()   # [H][k = rank][n = v_head_dim]
        self.wo, self.latent_norm = tensors["wo"], tensors["latent_norm"]

    def export(self):
        H, d, r, dv, R = self.n_head, self.head_dim, self.rot_dim, self.v_head_dim, self.rank
        wq, wdkv, wg = self.w_in.split([H * (d + r), R + r, H * dv])
        return {"wq": wq, "wdkv": wdkv, "wg": wg, "wuk": self.wuk.reshape(H * d, R), "wuv": self.wuv.transpose(1, 2).reshape(H * dv, R),
                "wo": self.wo, "latent_norm": self.latent_norm}

    def cache_needs(self) -> CacheNeeds:
        # one "key head" of rank + rot_dim numbers per token; values are its leading part, so no value storage
        return CacheNeeds(kv=KVNeed(1, self.rank + self.rot_dim, self.window, values=False))

    def forward(self, h, batch, view, residual, append: bool = True):
        T = batch.n_tokens
        H, d, r, dv, R = self.n_head, self.head_dim, self.rot_dim, self.v_head_dim, self.rank
        q_off, kv_off, g_off = 0, H * (d + r), H * (d + r) + R + r
        proj = torch.empty(T, g_off + H * dv, dtype=self.dtype, device=h.device)
        ops.linear(h, self.w_in, proj)
        q = torch.empty(T, H, R + r, dtype=self.dtype, device=h.device)
        ops.latent_prepare(proj, q_off, kv_off, q, view.kv, batch, H, d, r, R, self.latent_norm, self.eps,
                           self.position.table, self.position.pairing, append)
        ops.headwise_linear(proj, self.wuk, q.view(T, H * (R + r)), H, d, R, a_off=q_off, a_stride=d + r, out_stride=R + r)
        o = torch.empty(T, H * R, dtype=self.dtype, device=h.device)
        ops.attention(q, view.kv, batch, o, H, 1, R + r, self.scale, self.window, v_head_dim=R, values_in_keys=True)
        y = torch.empty(T, H * dv, dtype=self.dtype, device=h.device)
        ops.headwise_linear(o, self.wuv, y, H, R, dv, gate=proj, gate_off=g_off)
        as_residual(residual).add_linear(y, self.wo)
