"""Rotary position encoding.

For pair p < rotary_dim / 2 of a head: angle = position * theta^(-2p / rotary_dim),
all in 32-bit; the pair's two elements are rotated by it
(crates/quantinfer-runtime/src/attention.rs:7-36, the angle :29-32;
backends/cpu/src/backend.rs:240-280, the rotation :270-275). Which two elements
form pair p is the spec's `pairing`: "half_split" (x[p], x[p + rotary_dim/2]),
the reference's rule for this architecture, or "interleaved" (x[2p], x[2p + 1]),
the order its converter writes for others
(crates/quantinfer-format/src/gguf/layout.rs:52-55). The part owns the table
and the rule: inverse frequencies are computed once in 32-bit, the cos/sin
table [max_positions, rotary_dim / 2] is built on the device, and the mixer's
kernel looks positions up in it and pairs as `pairing` says. Tables are shared
between layers with the same angles.
"""

from __future__ import annotations

import math

import torch

from .. import kernels
from ..errors import ConfigError
from .base import Part, register_part


def direct_frequencies(spec):
    """(one frequency a pair as a float32 tensor on the CPU, factor on cos and sin) of a :class:`RotarySpec` whose angles
    are computed where they are used. Plain: theta^(-2i / rotary_dim) and 1. With `stretch` = (factor, original, fast,
    slow): with where(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta) the pair's number at which a pair turns t
    times over `original` positions, lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), rotary_dim - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns by f_i / factor * ramp_i + f_i (1 - ramp_i), and cos
    and sin are multiplied by 0.1 ln(factor) + 1. Evaluated in 64-bit and rounded once."""
    dims = spec.rotary_dim
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / float(dims))
    stretch = getattr(spec, "stretch", None)
    if stretch is None:
        return f.to(torch.float32), 1.0
    factor, original, fast, slow = (float(x) for x in stretch)
    if factor <= 0.0 or original <= 0.0 or fast <= 0.0 or slow <= 0.0 or spec.theta <= 1.0:
        raise ConfigError("a stretched rotation needs positive factor, original, fast and slow, and a base above one")

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(spec.theta)))

    lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32), 0.1 * math.log(factor) + 1.0


class RopeHalfSplit(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.rotary_dim % 2 or not 0 < spec.rotary_dim <= spec.head_dim:
            raise ConfigError(f"rotary_dim {spec.rotary_dim} must be even and within head_dim {spec.head_dim}")
        self.rotary_dim = spec.rotary_dim
        self.pairing = getattr(spec, "pairing", "half_split")
        if self.pairing not in ("half_split", "interleaved"):
            raise ConfigError(f"rotary pairing {self.pairing!r} is not known (half_split or interleaved)")
        key = ("rope_half_split", spec.rotary_dim, float(spec.theta), spec.max_positions)
        if key not in runtime.shared:
            half = spec.rotary_dim // 2
            # exponent = 2p / rotary_dim and theta^(-exponent), both in 32-bit
            exponent = (2.0 * torch.arange(half, dtype=torch.float32)) / torch.tensor(float(spec.rotary_dim), dtype=torch.float32)
            inv_freq = torch.pow(torch.tensor(spec.theta, dtype=torch.float32), -exponent)
            runtime.shared[key] = kernels.rope_table(inv_freq.to(runtime.device), spec.max_positions)
        self.cos, self.sin = runtime.shared[key]
        self.max_positions = spec.max_positions


register_part("position", "rope_half_split", RopeHalfSplit)
