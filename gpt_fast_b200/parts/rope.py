"""Rotary position encoding: the frequencies (with the llama3 rescaling rule)
and the (cos, sin) table that the fused rotate-and-append kernel reads.

gpt-fast: model.py:266-278 (base frequencies, table), model.py:244-263
(llama3 rule), model.py:281-293 (rotation of interleaved pairs).  The table
is kept in 32-bit here also for a bfloat16 model (gpt-fast rounds it to the
model's dtype, model.py:278)."""
import math
from typing import Dict, Optional

import torch

from .. import ops
from . import register_position


def rope_frequencies(head_dim: int, base: float, scaling: Optional[Dict[str, float]], freq_dtype: str = "float32") -> torch.Tensor:
    """inv_freq[i] = base^(-2i/d) in 32-bit, i < d/2 (freq_dtype 'float64': evaluated in 64-bit and rounded once to
    32-bit, which is the nearest 32-bit number to the exact power), then the llama3 rule:
    wavelengths shorter than original/high_freq_factor stay, longer than
    original/low_freq_factor are divided by `factor`, between them the two are
    blended linearly in original/wavelength."""
    if freq_dtype == "float64":
        exponent = torch.arange(0, head_dim, 2, dtype=torch.float64)[: head_dim // 2] / head_dim
        freqs = (float(base) ** -exponent).to(torch.float32)
    else:
        exponent = torch.arange(0, head_dim, 2, dtype=torch.float32)[: head_dim // 2] / head_dim
        freqs = 1.0 / (base ** exponent)
    if scaling is None:
        return freqs
    if scaling.get("type") == "yarn":
        return yarn_frequencies(head_dim, base, scaling)[0]
    factor, low, high = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    original = scaling["original_max_position_embeddings"]
    low_wavelen, high_wavelen = original / low, original / high
    out = torch.empty_like(freqs)
    for i in range(freqs.numel()):
        f = freqs[i]
        wavelen = 2 * math.pi / f
        if wavelen < high_wavelen:
            out[i] = f
        elif wavelen > low_wavelen:
            out[i] = f / factor
        else:
            smooth = (original / wavelen - low) / (high - low)
            out[i] = (1 - smooth) * f / factor + smooth * f
    return out


def yarn_frequencies(dims: int, base: float, scaling: Dict[str, float]):
    """The YaRN rule for sequences longer than the `original` length a model was made for: (frequencies, amplitude).

    Pair i has frequency f_i = base^(-2i/dims).  The pair that turns `t` times over the original length is number
    dim(t) = dims ln(original / (2 pi t)) / (2 ln base).  With lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)),
    dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pairs that turn fast (ramp 0) keep f_i, slow
    ones (ramp 1) get f_i / factor, those between a blend: f_i / factor * ramp_i + f_i (1 - ramp_i).  cos and sin are
    both multiplied by the amplitude 0.1 ln(factor) + 1.  Evaluated in 64-bit and rounded once to 32-bit."""
    factor, original = float(scaling["factor"]), float(scaling["original"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


@register_position("rope")
class Rope:
    """pairing 'interleaved': pairs (2i, 2i+1); 'half': pairs (i, i + d/2).  `head_dim` is the number of rotated
    dimensions; a mixer whose heads are larger leaves the rest as they are.  scaling: None, the llama3 rule (keys
    factor, low_freq_factor, high_freq_factor, original_max_position_embeddings) or {'type': 'yarn', factor, original,
    fast, slow} (`yarn_frequencies`), whose amplitude is part of the table."""

    def __init__(self, head_dim: int, base: float, scaling: Optional[Dict[str, float]] = None,
                 pairing: str = "interleaved", freq_dtype: str = "float32"):
        if head_dim % 2:
            raise ValueError(f"rotary pairs need an even head_dim, got {head_dim}")
        if pairing not in ("interleaved", "half"):
            raise ValueError(f"unknown rotary pairing '{pairing}'")
        if freq_dtype not in ("float32", "float64"):
            raise ValueError(f"rotary frequencies are evaluated in float32 or float64, not '{freq_dtype}'")
        self.head_dim, self.base, self.scaling, self.pairing = head_dim, float(base), scaling, pairing
        self.inv_freq = rope_frequencies(head_dim, self.base, scaling, freq_dtype)
        self.amplitude = yarn_frequencies(head_dim, self.base, scaling)[1] if scaling and scaling.get("type") == "yarn" else 1.0
        self.table = None
        self._retired = []                 # earlier, shorter tables: captured decode steps may still point at them

    def prepare(self, max_positions: int, device) -> None:
        """Build the (cos, sin) table for positions 0 .. max_positions-1."""
        if self.table is not None and self.table.shape[0] >= max_positions and self.table.device == torch.device(device):
            return
        table = torch.empty(max_positions, self.head_dim // 2, 2, dtype=torch.float32, device=device)
        ops.rope_table(self.inv_freq.to(device), table, self.amplitude)
        if self.table is not None:
            # a CUDA graph captured for an earlier cache has the old table's address and length in it; the old
            # table stays valid for as long as this part lives (a few KB to MB each, one per growth)
            self._retired.append(self.table)
        self.table = table
