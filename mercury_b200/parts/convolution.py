"""What a sublayer reads when it does not read the stream itself: the stream plus a short
causal convolution of it over time, per channel,

    out_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j),   j = 0 .. taps - 1,

with zeros before a sequence's first token and no bias. The last taps - 1 rows of the
stream that the convolution has seen are per-request state (float32, in the slot the cache
manager gave the request), so a sequence may be cut into steps anywhere. The state is a
ring by position: the row of position p lies at index p modulo (taps - 1), so a step only
ever writes the rows of its own last tokens and nothing is shifted. The arithmetic is
float32 on the float32 stream; the result is stored in the activation type, as the input
of the sublayer's projections.
"""

from __future__ import annotations

import torch

from .base import Part, PartSpec, StateNeed, TensorSpec, build_part

_KINDS: dict = {}


class InputConvolution(Part):
    capturable = True

    def __init__(self, size: int, taps: int, weight_name: str, init_std: float = 0.2):
        if not 1 <= taps <= 16:
            raise ValueError(f"a convolution over {taps} tokens is not built (1 to 16)")
        self.size, self.taps, self.weight_name, self.init_std = size, int(taps), weight_name, init_std
        self.weight = None

    def state_need(self):
        if self.taps <= 1:
            return None
        # row p % (taps - 1): the stream's row at position p, for the last taps - 1 positions
        return StateNeed((self.taps - 1, self.size), torch.float32)

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.size, self.taps), std=self.init_std)]

    def load(self, tensors, setup):
        # the convolution runs on the float32 stream, so its taps are float32 in both engines
        self.weight = setup.place(tensors[self.weight_name]).float().contiguous()

    def forward(self, h, ctx, state, store_tail: bool = True):
        """`store_tail=False`: the caller keeps the step's last rows itself, before the stream
        changes (the post-norm block hands the ring to the norm behind the sublayer, whose
        kernel still sees the rows as they were read here)."""
        out = ctx.buffer("sublayer_in", h.shape[0], self.size)
        ctx.ops.stream_conv(h, self.weight, state, ctx.batch, out)
        if state is not None and store_tail:
            # behind the kernel that read the ring: the step's own last rows replace it
            ctx.ops.stream_tail_store(h, state, ctx.batch)
        return out


class StreamInput(Part):
    """The stream itself, rounded to the activation type: what a sublayer reads when nothing
    stands between it and the stream."""

    capturable = True

    def __init__(self, size: int):
        self.size = size

    def state_need(self):
        return None

    def forward(self, h, ctx, state, store_tail: bool = True):
        out = ctx.buffer("sublayer_in", h.shape[0], self.size)
        ctx.ops.stream_conv(h, None, None, ctx.batch, out)
        return out


def build_input(spec: PartSpec | None, size: int):
    """A sublayer's input part from its spec ("convolution" or "stream"); None: the stream."""
    if spec is None:
        return StreamInput(size)
    kinds = {"convolution": InputConvolution, "stream": StreamInput}
    if spec.kind not in kinds:
        raise KeyError(f"no sublayer input of kind {spec.kind!r}; known: {', '.join(sorted(kinds))}")
    return kinds[spec.kind](**spec.params)
