"""Position encodings applied inside a mixer."""

from __future__ import annotations

import math

import torch

from ..config.specs import NoPositionSpec, RotarySpec
from ..kernels import ops
from .base import Part, register_part


def scaled_frequencies(freqs, scaling):
    """Frequencies with their long wavelengths slowed (``RotarySpec.scaling`` = factor, low, high, original): a
    wavelength l = 2 pi / f below original / high keeps f, above original / low gets f / factor, and in between
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  Host arithmetic in double."""
    factor, low, high, original = (float(v) for v in scaling)
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            s = (original / wavelength - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def ramped_frequencies(freqs, theta: float, dims: int, ramp):
    """Frequencies slowed by a ramp over the pair index (``RotarySpec.index_ramp`` = factor, original, fast, slow),
    and the number that cos and sin are multiplied by.  With n(t) = dims ln(original / (2 pi t)) / (2 ln theta),
    lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1), s_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):
    f_i <- s_i f_i / factor + (1 - s_i) f_i; magnitude = 0.1 ln(factor) + 1.  Host arithmetic in double."""
    factor, original, fast, slow = (float(v) for v in ramp)

    def pair_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_index(fast)), 0)
    hi = min(math.ceil(pair_index(slow)), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        s = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(s * f / factor + (1.0 - s) * f)
    return out, 0.1 * math.log(factor) + 1.0


class Rotary(Part):
    """Rotary embedding (ondeviceinfer/layers.py:36-83); which lanes pair up (half-split or neighbours) is the
    mixer's business, the tables are the same.

    ``inv_freq[i] = 1 / theta**(2i / d)`` is evaluated once on the host in fp32 exactly
    as the reference does (ondeviceinfer/layers.py:44-46); angles, cos and sin of a
    step's positions are evaluated on the device in fp32 and shared by all layers.
    """

    def __init__(self, spec: RotarySpec) -> None:
        super().__init__(spec)
        if spec.dim % 2 != 0 or spec.dim > spec.head_dim or spec.dim <= 0:
            raise ValueError(f"rotary_dim must be even and at most head_dim, got {spec.dim} of {spec.head_dim}")
        self.rot_dim = spec.dim
        self.interleaved = spec.interleaved     # which lanes pair up; the tables are the same either way

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        exponent = torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim
        inv_freq = 1.0 / (self.spec.theta ** exponent)
        if self.spec.scaling is not None:
            inv_freq = torch.tensor(scaled_frequencies(inv_freq.double().tolist(), self.spec.scaling), dtype=torch.float32)
        self.magnitude = 1.0
        if self.spec.index_ramp is not None:
            # in double from theta itself, not from the fp32 frequencies
            exact = [float(self.spec.theta) ** (-2.0 * i / self.rot_dim) for i in range(self.rot_dim // 2)]
            ramped, self.magnitude = ramped_frequencies(exact, float(self.spec.theta), self.rot_dim, self.spec.index_ramp)
            inv_freq = torch.tensor(ramped, dtype=torch.float64).to(torch.float32)
        self.inv_freq = inv_freq.to(runtime.device)

    def rotary_tables(self, ctx):
        def make():
            n, half = ctx.n_tokens, self.rot_dim // 2
            cos = torch.empty((n, half), dtype=torch.float32, device=self.inv_freq.device)
            sin = torch.empty_like(cos)
            ops.rope_table(self.inv_freq, ctx.tok_pos, cos, sin, self.magnitude)
            return cos, sin

        return ctx.memo(("rotary", self.spec), make)


class NoPosition(Part):
    rot_dim = 0

    def rotary_tables(self, ctx):
        return None


register_part(RotarySpec, Rotary)
register_part(NoPositionSpec, NoPosition)
