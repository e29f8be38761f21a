"""A selective state-space mixer with a scalar decay per head and token (the Mamba-2 form).

    (z, x, B, C, dt) = Win h                  z, x: heads x head_dim; B, C: groups x n_state; dt: heads
    (x, B, C) <- silu(conv(x, B, C) + bias)   a causal convolution over time per channel, `taps` wide
    dt <- softplus(dt + dt_bias)
    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T,   y_t = S_t^T C_t + D_h x_t       per head, S [n_state, head_dim]
    out = Wo (rms_groups(y * silu(z)) * norm)                 root mean square over `norm_groups` equal parts, eps inside

Head h reads group h // (heads / groups).  Per sequence the cache keeps S (32-bit) and the convolution's last
taps - 1 inputs; both start at zero."""
import torch

from .. import ops
from ..cache.needs import CacheNeeds, StateNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """Rows of zeros up to a multiple: the tensor-core product takes output widths of whole 16-byte units."""
    extra = -w.shape[0] % multiple
    if extra == 0:
        return w.contiguous()
    return torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous()


@register_mixer("state_space")
class StateSpace:
    def __init__(self, dim: int, n_head: int, head_dim: int, n_state: int, n_groups: int, norm_groups: int, taps: int, eps: float,
                 dtype: torch.dtype, position=None):
        if n_head % n_groups:
            raise ValueError(f"{n_head} heads do not divide into {n_groups} groups")
        if (n_head * head_dim) % norm_groups:
            raise ValueError(f"{n_head * head_dim} inner channels do not divide into {norm_groups} norm groups")
        self.dim, self.n_head, self.head_dim, self.n_state, self.n_groups = dim, n_head, head_dim, n_state, n_groups
        self.norm_groups, self.taps, self.eps, self.dtype = norm_groups, int(taps), float(eps), dtype
        self.inner = n_head * head_dim
        self.conv_channels = self.inner + 2 * n_groups * n_state
        self.width = 2 * self.inner + 2 * n_groups * n_state + n_head
        self.state_floats = n_head * n_state * head_dim
        self.w_in = self.wo = self.conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm = None

    def param_specs(self):
        H, C = self.n_head, self.conv_channels
        return {"w_in": ParamSpec((self.width, self.dim)), "conv": ParamSpec((C, self.taps), "vector"),
                "conv_bias": ParamSpec((C,), "vector"), "dt_bias": ParamSpec((H,), "vector"), "a_log": ParamSpec((H,), "vector"),
                "skip": ParamSpec((H,), "vector"), "norm": ParamSpec((self.inner,), "vector"), "wo": ParamSpec((self.dim, self.inner))}

    def load(self, tensors):
        self._w_in_rows = tensors["w_in"].shape[0]
        self.w_in = _pad_rows(tensors["w_in"])
        self.wo = tensors["wo"]
        self.conv, self.norm = tensors["conv"], tensors["norm"]
        self.conv_bias = tensors["conv_bias"].to(self.conv.dtype)
        self.dt_bias = tensors["dt_bias"]
        self.a_log, self.skip = tensors["a_log"].to(self.dt_bias.dtype), tensors["skip"].to(self.dt_bias.dtype)

    def export(self):
        return {"w_in": self.w_in[:self._w_in_rows], "conv": self.conv, "conv_bias": self.conv_bias, "dt_bias": self.dt_bias,
                "a_log": self.a_log, "skip": self.skip, "norm": self.norm, "wo": self.wo}

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateNeed((self.state_floats + (self.taps - 1) * self.conv_channels,), torch.float32))

    def forward(self, h, batch, view, residual, append: bool = True):
        if not append:
            raise ValueError("a state-space layer owns its state: it cannot run on another run's cache entry")
        T = batch.n_tokens
        H, P, N, G, inner = self.n_head, self.head_dim, self.n_state, self.n_groups, self.inner
        proj = torch.empty(T, self.w_in.shape[0], dtype=self.dtype, device=h.device)
        ops.linear(h, self.w_in, proj)
        xbc = torch.empty(T, self.conv_channels, dtype=torch.float32, device=h.device)
        ops.short_conv(proj, inner, self.conv_channels, self.conv, self.conv_bias, view.state, self.state_floats, xbc, batch)
        y = torch.empty(T, H, P, dtype=torch.float32, device=h.device)
        ops.ssd_scan(xbc, inner, inner + G * N, proj, 2 * inner + 2 * G * N, self.dt_bias, self.a_log, self.skip, view.state, 0,
                     y, batch, H, P, N, G)
        out = torch.empty(T, inner, dtype=self.dtype, device=h.device)
        ops.gated_norm(y.view(T, inner), proj, 0, self.norm, out, inner // self.norm_groups, self.eps, act="silu", gate_first=True)
        as_residual(residual).add_linear(out, self.wo)
