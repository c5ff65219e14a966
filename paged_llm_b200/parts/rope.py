"""Rotary position encoding.

inv_freq[j] = 1 / theta^(2j/d) in float32 (reference: pagedllm/model/llama.py:104),
optionally rescaled by the llama3 rule (llama.py:86-97); the angle of position p
is p * inv_freq[j] in float32 and the table holds its cosine and sine
(llama.py:111-115).  The rotation itself pairs element i with i + d/2
("half", llama.py:117-128) or 2i with 2i+1 ("interleaved", not used by Llama),
over the first `rotary_dim` elements of a head.

Frequencies are computed on the host in float32 with the reference's order of
operations, so that angles agree with it to rounding; the table is filled on
the device by a kernel of this package.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding


def llama3_rescale(inv_freq: torch.Tensor, factor: float, low_freq_factor: float,
                   high_freq_factor: float, original_max_position_embeddings: int) -> torch.Tensor:
    """Long wavelengths are divided by `factor`, short ones kept, and the band
    between blends the two linearly in 1/wavelength (llama.py:86-97)."""
    old_len = original_max_position_embeddings
    wavelen = 2 * math.pi / inv_freq
    long_wl, short_wl = old_len / low_freq_factor, old_len / high_freq_factor
    blend = (old_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    out = torch.where(wavelen > long_wl, inv_freq / factor, inv_freq)
    band = (wavelen <= long_wl) & (wavelen >= short_wl)
    return torch.where(band, (1 - blend) * inv_freq / factor + blend * inv_freq, out)


def yarn_rescale(inv_freq: torch.Tensor, base: float, factor: float, original: float, fast: float,
                 slow: float) -> tuple[torch.Tensor, float]:
    """YaRN: pair i of r/2 keeps its frequency if it turns fast and gets 1/factor of it if it turns
    slowly, with a linear ramp between.  With pair(t) = r ln(original / (2 pi t)) / (2 ln base) the
    pair whose wave makes t turns over `original` positions, lo = max(floor(pair(fast)), 0),
    hi = min(ceil(pair(slow)), r - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    the frequency is f_i / factor * ramp_i + f_i * (1 - ramp_i).  Cosine and sine are both
    multiplied by 0.1 ln(factor) + 1, which is returned beside the frequencies."""
    f = inv_freq.double()
    r = 2 * f.numel()

    def pair(turns: float) -> float:
        return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(fast)), 0)
    hi = min(math.ceil(pair(slow)), r - 1)
    ramp = ((torch.arange(f.numel(), dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).float(), 0.1 * math.log(factor) + 1.0


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, weights: dict[str, str], head_dim: int, theta: float,
                 scaling: dict | None = None, rotary_dim: int | None = None, pairing: str = "half"):
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.theta, self.scaling, self.pairing = float(theta), scaling, pairing
        self.table = None            # [P, rotary_dim/2, 2] float32: (cos, sin)
        self.max_positions = 0

    def inv_freq(self) -> torch.Tensor:
        return self.frequencies()[0]

    def frequencies(self) -> tuple[torch.Tensor, float]:
        """(frequency of each pair in float32, the factor cosine and sine are multiplied by)."""
        rd = self.rotary_dim
        kind = (self.scaling or {}).get("rope_type", (self.scaling or {}).get("type"))
        if kind == "yarn":
            # formed in float64 and rounded once
            inv = self.theta ** (-torch.arange(0, rd, 2, dtype=torch.float64) / rd)
            sc = self.scaling
            return yarn_rescale(inv, self.theta, float(sc["factor"]), float(sc["original"]), float(sc["fast"]),
                                float(sc["slow"]))
        inv = 1.0 / (self.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        if kind == "llama3":
            inv = llama3_rescale(inv, **{k: v for k, v in self.scaling.items() if k not in ("rope_type", "type")})
        elif kind not in (None, "default"):
            raise NotImplementedError(f"rope_type={kind!r} not supported (default, llama3 and yarn only)")
        return inv, 1.0

    def prepare(self, max_positions, device, ops):
        self.max_positions = int(max_positions)
        inv, magnitude = self.frequencies()
        if magnitude == 1.0:
            self.table = ops.rope_table(inv.to(device), self.max_positions)
        else:
            self.table = ops.rope_table(inv.to(device), self.max_positions, magnitude)
