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
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    capturable = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None,
                 table_precision: str = "float32", pairing: str = "halves"):
        """`table_precision` "float64": angles, cosines and sines are computed in 64-bit and
        rounded once to the float32 tables."""
        if pairing not in ("halves", "interleaved"):
            raise ValueError(f"pairing={pairing!r} is neither 'halves' nor 'interleaved'")
        self.pairing = pairing
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
            positions = torch.arange(setup.max_positions, dtype=real)
            angles = torch.outer(positions, inv_freq)
            return (angles.cos().float().to(setup.device).contiguous(),
                    angles.sin().float().to(setup.device).contiguous())

        # every layer with the same constants reads the same pair of tables
        self.cos, self.sin = setup.derived(
            ("rotary", self.rotary_dim, self.theta, setup.max_positions, str(setup.device),
             self.table_precision), tables)

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
