"""Rotary position encoding as a table of inverse frequencies.

Half-split (NeoX) pairing: for j < rotary_dim/2, ``inv_freq[j] = theta^(-2j /
rotary_dim)`` and the pair (x[j], x[j + rotary_dim/2]) is rotated by
``pos * inv_freq[j]`` (src/backends/cuda/ops/layers.cu:80-115).  The table is
computed once in float64 and rounded to fp32; the kernel forms the angle and its
sine and cosine in fp32.  Anything that can be written as such a table (scaled
frequencies, a partial rotary dimension, no rotation at all) reuses the fused
kernel by returning a different ``rotary_table()``.
"""
from __future__ import annotations

import torch

from .registry import register_part


class RotaryEncoding:
    def __init__(self, spec, ctx, prefix: str):
        self.spec = spec
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim < 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim "
                             f"{spec.head_dim}")
        half = spec.rotary_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64),
                        -2.0 * j / float(max(spec.rotary_dim, 1)))
        factor = float(getattr(spec, "scaling_factor", 1.0))
        if factor <= 0:
            raise ValueError(f"rotary scaling factor {factor} must be positive")
        if factor != 1.0:
            inv = inv / factor        # linear position scaling, in float64 before the rounding
        self.inv_freq = inv.to(torch.float32).to(ctx.device)

    def tensors(self):
        return []

    def bind(self, weights):
        pass

    def rotary_table(self):
        return (self.inv_freq if self.spec.rotary_dim else None), self.spec.rotary_dim


register_part("position", "rope", RotaryEncoding)


class InterleavedRotary:
    """Rotation of neighbouring pairs, optionally with YaRN-stretched frequencies.

    ``pair_table()`` gives (frequency per pair as fp32 [rotary_dim/2], factor on cos and
    sin, rotary_dim).  The frequencies are formed in float64 and rounded once; the
    kernel multiplies position and frequency, and takes cos and sin, in fp32."""

    def __init__(self, spec, ctx, prefix: str):
        import math
        self.spec = spec
        r = spec.rotary_dim
        if r % 2 or r > spec.head_dim or r < 0:
            raise ValueError(f"rotary_dim {r} must be even and at most {spec.head_dim}")
        i = torch.arange(r // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / max(r, 1))
        self.magnitude = 1.0
        if spec.scaling_factor > 0:
            def pair_with_turns(turns):
                return r * math.log(spec.original_context / (2.0 * math.pi * turns)) / (
                    2.0 * math.log(spec.theta))
            lo = max(math.floor(pair_with_turns(spec.fast_turns)), 0)
            hi = min(math.ceil(pair_with_turns(spec.slow_turns)), r - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / spec.scaling_factor * ramp + f * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(spec.scaling_factor) + 1.0
        self.freq = f.to(torch.float32).to(ctx.device)

    def tensors(self):
        return []

    def bind(self, weights):
        pass

    def pair_table(self):
        return self.freq, self.magnitude, self.spec.rotary_dim


register_part("position", "rope_interleaved", InterleavedRotary)


class SinusoidAdded:
    """A position vector added to the embedding: entry 2i of position p is
    sin(p * base^(-2i/size)), entry 2i+1 the cosine of the same angle.  The frequencies
    are computed once in float64 and rounded to fp32; the kernel forms the angle, its
    sine and its cosine in fp32 with the accurate functions, in the pass that gathers and
    scales the embedding rows."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx = spec, ctx
        pairs = (spec.size + 1) // 2
        i = torch.arange(pairs, dtype=torch.float64)
        freq = torch.pow(torch.tensor(float(spec.base), dtype=torch.float64),
                         -2.0 * i / float(spec.size))
        self.freq = freq.to(torch.float32).to(ctx.device)

    def tensors(self):
        return []

    def bind(self, weights):
        pass

    def embed(self, table, token_ids, positions, scale: float):
        return self.ctx.ops.embed_sinusoid(table, token_ids, positions, self.freq, scale)


register_part("position", "sinusoid_added", SinusoidAdded)


class ScaledRotary:
    """Rotation of pairs of a head's first ``rotary_dim`` entries, in either pairing, with
    the frequencies stretched by wavelength or by a ramp over the pair index (the spec
    says how).  ``pair_table()`` gives (frequency per pair as fp32 [rotary_dim / 2], the
    factor on cos and sin, rotary_dim, whether pairs are neighbours).  The frequencies are
    formed in float64 and rounded once; the kernel multiplies position and frequency, and
    takes cos and sin, in fp32."""

    def __init__(self, spec, ctx, prefix: str):
        import math
        self.spec = spec
        r = spec.rotary_dim
        if r % 2 or r > spec.head_dim or r < 0:
            raise ValueError(f"rotary_dim {r} must be even and at most {spec.head_dim}")
        if spec.layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout {spec.layout!r} is not 'half' or 'interleaved'")
        f = [float(spec.theta) ** (-2.0 * i / max(r, 1)) for i in range(r // 2)]
        self.magnitude = 1.0
        sc = spec.scaling
        if sc is not None and sc[0] == "wavelength":
            _, factor, low, high, original = sc
            out = []
            for v in f:
                wavelength = 2.0 * math.pi / v
                if wavelength < original / high:
                    out.append(v)
                elif wavelength > original / low:
                    out.append(v / factor)
                else:
                    t = (original / wavelength - low) / (high - low)
                    out.append((1.0 - t) * v / factor + t * v)
            f = out
        elif sc is not None and sc[0] == "ramp":
            _, factor, original, fast, slow = sc

            def pair_with_turns(turns):
                return r * math.log(original / (2.0 * math.pi * turns)) / (
                    2.0 * math.log(spec.theta))
            lo = max(math.floor(pair_with_turns(fast)), 0)
            hi = min(math.ceil(pair_with_turns(slow)), r - 1)
            ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(r // 2)]
            f = [v / factor * t + v * (1.0 - t) for v, t in zip(f, ramp)]
            self.magnitude = 0.1 * math.log(factor) + 1.0
        elif sc is not None:
            raise ValueError(f"rotary scaling {sc[0]!r} is not 'wavelength' or 'ramp'")
        self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(ctx.device)

    def tensors(self):
        return []

    def bind(self, weights):
        pass

    def pair_table(self):
        return self.freq, self.magnitude, self.spec.rotary_dim, self.spec.layout == "interleaved"


register_part("position", "rope_scaled", ScaledRotary)
