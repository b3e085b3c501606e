"""Rotary position encoding, with the NeoX pairing of halves or with neighbours paired.

Table as in mercury/model/rope.py:37-47: inv_freq[i] = theta^(-2i/d), angle = position *
inv_freq, both in float32; the table is kept in float32 (the reference rounds it to the
activation dtype) and covers as many positions as the engine will serve
(mercury/model/loader.py:101). `rotary_dim` is the number of leading features of a head
that are rotated; Qwen2 rotates the whole head. `pairing` "halves" pairs feature i with
feature i + rotary_dim/2; "interleaved" pairs feature 2i with feature 2i + 1 (the pair
(u, v) becomes (u cos a - v sin a, v cos a + u sin a) either way, a = position *
theta^(-2i/rotary_dim)). The tables are the same for both; the rotate-and-store kernels of
the grouped-query attention know the halves only, so an interleaved encoding answers
`fused_form()` with None and serves the mixers that ask for `pairing` themselves.

`scaling` = {"factor", "low", "high", "original"} slows the long wavelengths down (the
frequency scaling that Llama 3.1 uses): with the wavelength l = 2 pi / f, a frequency with l < original / high is kept, one with l > original /
low becomes f / factor, and between the two it is (1 - s) f / factor + s f with s = (original
/ l - low) / (high - low).
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    capturable = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None,
                 table_precision: str = "float32", pairing: str = "halves",
                 scaling: dict | None = None):
        """`table_precision` "float64": angles, cosines and sines are computed in 64-bit and
        rounded once to the float32 tables."""
        if pairing not in ("halves", "interleaved"):
            raise ValueError(f"pairing={pairing!r} is neither 'halves' nor 'interleaved'")
        self.pairing = pairing
        self.scaling = None
        if scaling:
            self.scaling = tuple(float(scaling[key]) for key in ("factor", "low", "high", "original"))
            if min(self.scaling) <= 0 or self.scaling[1] == self.scaling[2]:
                raise ValueError(f"rotary scaling {scaling!r}: positive numbers, low != high")
        self.table_precision = table_precision
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and at most {head_dim}")
        self.cos = None
        self.sin = None

    def load(self, tensors, setup):
        def tables():
            real = torch.float64 if self.table_precision == "float64" else torch.float32
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=real) / self.rotary_dim
            inv_freq = 1.0 / (self.theta ** exponent)
            if self.scaling is not None:
                factor, low, high, original = self.scaling
                wave = 2.0 * torch.pi / inv_freq
                blend = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
                mixed = (1.0 - blend) * inv_freq / factor + blend * inv_freq
                inv_freq = torch.where(wave < original / high, inv_freq,
                                       torch.where(wave > original / low, inv_freq / factor, mixed))
            positions = torch.arange(setup.max_positions, dtype=real)
            angles = torch.outer(positions, inv_freq)
            return (angles.cos().float().to(setup.device).contiguous(),
                    angles.sin().float().to(setup.device).contiguous())

        # every layer with the same constants reads the same pair of tables
        self.cos, self.sin = setup.derived(
            ("rotary", self.rotary_dim, self.theta, setup.max_positions, str(setup.device),
             self.table_precision, self.scaling), tables)

    def fused_form(self):
        return "rotary" if self.pairing == "halves" else None

    def rotary_tables(self):
        return self.cos, self.sin

    def apply(self, qkv, layout, ctx):
        raise NotImplementedError("an interleaved rotation is applied by the mixers that ask for "
                                  "its tables and pairing; the packed q/k/v path knows halves only")


class NoPositionEncoding(PositionEncoding):
    capturable = True

    def __init__(self, **_ignored):
        pass

    def fused_form(self):
        return "identity"


register_position_encoding("rotary", RotaryEncoding)
register_position_encoding("none", NoPositionEncoding)
