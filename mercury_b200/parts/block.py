"""Arrangements: how mixers, a feed-forward and their norms sit in one block.

`PreNormBlock` is mercury/model/qwen2.py:72-94: norm, mixer, norm, feed-forward, with the
residual sum deferred to the next norm. A block receives the residual stream `h` and the
delta that is still to be added to it, and returns the delta it leaves behind.
"""

from __future__ import annotations

from .base import Part, PartSpec, TensorSpec, build_part, register_arrangement
from .convolution import build_input
from .norm import scaled_add


class PreNormBlock:
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec):
        self.mixer = build_part("mixer", mixer)
        self.feed_forward = build_part("feed_forward", feed_forward)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.feed_forward_norm = build_part("norm", feed_forward_norm)

    def mixers(self):
        return [self.mixer]

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def first_norm(self):
        """The norm that opens this block (what the block before may compute ahead)."""
        return self.mixer_norm

    def forward(self, h, delta, ctx, caches, states, next_norm=None):
        mixer, ff = self.mixer, self.feed_forward
        cache, state = caches[0], states[0]
        x = self.mixer_norm.add_norm(h, delta, ctx,
                                     defer=getattr(mixer, "accepts_pending_norm", False))
        if getattr(mixer, "adds_to_residual", False):
            mixed = mixer.forward(x, ctx, cache, state, residual=h,
                                  then_norm=self.feed_forward_norm)
        else:
            mixed = mixer.forward(x, ctx, cache, state)
        x = self.feed_forward_norm.add_norm(h, mixed, ctx,
                                            defer=getattr(ff, "accepts_pending_norm", False))
        if getattr(ff, "adds_to_residual", False):
            return ff.forward(x, ctx, residual=h, then_norm=next_norm)
        return ff.forward(x, ctx)


class NormedJoin(Part):
    """How two mixers side by side become one sublayer output: each output is RMS-normed over
    the model width with a plain weight of its own (`weight_names`), and the two are added
    under `scales`."""

    capturable = True

    def __init__(self, size: int, eps: float, weight_names: tuple, scales: tuple = (0.5, 0.5)):
        self.size, self.eps = int(size), float(eps)
        self.weight_names, self.scales = tuple(weight_names), tuple(float(v) for v in scales)
        if len(self.weight_names) != 2 or len(self.scales) != 2:
            raise ValueError("a join takes two outputs")
        self.weights = None

    def tensor_specs(self):
        return [TensorSpec(name, (self.size,), init="ones_normal", std=0.05)
                for name in self.weight_names]

    def load(self, tensors, setup):
        # norms are float32 arithmetic
        self.weights = [setup.place(tensors[name]).float().contiguous() for name in self.weight_names]


class SandwichBlock:
    """A norm before AND behind each sublayer: h <- h + post(mixer(pre(h))), then, where the
    block has a feed-forward, h <- h + post'(ff(pre'(h))). The sums are made by the norm
    behind the sublayer (`normed_add`), which also computes the norm that comes next, so
    the block leaves no pending delta. With `mixers` (two) and `mixer_join` (a `NormedJoin`)
    the mixer sublayer is two mixers side by side on the same normed input, joined before
    the norm behind the sublayer. A feed-forward may return two tensors (routed experts and
    a shared expert); their sum is what the norm behind it takes."""

    def __init__(self, mixer_norm: PartSpec, mixer_post_norm: PartSpec, mixer: PartSpec | None = None,
                 feed_forward: PartSpec | None = None, feed_forward_norm: PartSpec | None = None,
                 feed_forward_post_norm: PartSpec | None = None, mixers: list | None = None,
                 mixer_join: dict | None = None):
        if (mixer is None) == (mixers is None):
            raise ValueError("a block takes `mixer` or `mixers`")
        self.side_mixers = None
        self.join = None
        if mixers is not None:
            if len(mixers) != 2 or mixer_join is None:
                raise ValueError("mixers side by side come as two, with a `mixer_join`")
            self.side_mixers = [build_part("mixer", m) for m in mixers]
            self.join = NormedJoin(**mixer_join)
        self.mixer = build_part("mixer", mixer) if mixer is not None else None
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer_post_norm = build_part("norm", mixer_post_norm)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if feed_forward is not None:
            if feed_forward_norm is None or feed_forward_post_norm is None:
                raise ValueError("a feed-forward needs the norms before and behind it")
            self.feed_forward = build_part("feed_forward", feed_forward)
            self.feed_forward_norm = build_part("norm", feed_forward_norm)
            self.feed_forward_post_norm = build_part("norm", feed_forward_post_norm)

    def mixers(self):
        return list(self.side_mixers) if self.side_mixers is not None else [self.mixer]

    def parts(self):
        out = [self.mixer_norm, *self.mixers(), self.mixer_post_norm]
        if self.join is not None:
            out.append(self.join)
        if self.feed_forward is not None:
            out += [self.feed_forward_norm, self.feed_forward, self.feed_forward_post_norm]
        return out

    def first_norm(self):
        return self.mixer_norm

    def _mix(self, h, x, ctx, caches, states, then_norm):
        if self.side_mixers is None:
            mixed = self.mixer.forward(x, ctx, caches[0], states[0])
            self.mixer_post_norm.normed_add(h, mixed, ctx, then_norm=then_norm)
            return
        outs = []
        for index, mixer in enumerate(self.side_mixers):
            ctx.side = index          # mixers side by side leave their outputs in buffers of their own
            outs.append(mixer.forward(x, ctx, caches[index], states[index]))
        ctx.side = 0
        self.mixer_post_norm.joined_add(h, outs[0], outs[1], ctx, then_norm=then_norm,
                                        norm_weights=self.join.weights, scales=self.join.scales)

    def forward(self, h, delta, ctx, caches, states, next_norm=None):
        x = self.mixer_norm.add_norm(h, delta, ctx)
        if self.feed_forward is None:
            self._mix(h, x, ctx, caches, states, next_norm)
            return None
        self._mix(h, x, ctx, caches, states, self.feed_forward_norm)
        x = self.feed_forward_norm.add_norm(h, None, ctx)
        out = self.feed_forward.forward(x, ctx)
        if isinstance(out, tuple):
            self.feed_forward_post_norm.joined_add(h, out[0], out[1], ctx, then_norm=next_norm)
        else:
            self.feed_forward_post_norm.normed_add(h, out, ctx, then_norm=next_norm)
        return None


class LayerScale(Part):
    """One learned number per feature that a sublayer's output is multiplied by before it
    joins the stream."""

    capturable = True

    def __init__(self, size: int, weight_name: str, init_std: float = 0.1):
        self.size, self.weight_name, self.init_std = size, weight_name, init_std
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.size,), init="ones_normal", std=self.init_std)]

    def load(self, tensors, setup):
        self.weight = setup.place(tensors[self.weight_name])


class LayerScaleBlock:
    """Pre-norm with a learned scale on every sublayer's output: h <- h + s1 * mixer(norm1(h)),
    then, where the block has a feed-forward, h <- h + s2 * ff(norm2(h)). The sums are made at
    once (the block leaves no pending delta), each by the kernel that also computes the norm
    that comes next."""

    def __init__(self, hidden_size: int, mixer: PartSpec, mixer_norm: PartSpec, mixer_scale: str,
                 feed_forward: PartSpec | None = None, feed_forward_norm: PartSpec | None = None,
                 feed_forward_scale: str | None = None):
        self.mixer = build_part("mixer", mixer)
        self.mixer_norm = build_part("norm", mixer_norm)
        self.mixer_scale = LayerScale(hidden_size, mixer_scale)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_scale = None
        if feed_forward is not None:
            if feed_forward_norm is None or feed_forward_scale is None:
                raise ValueError("a feed-forward needs its norm and its scale")
            self.feed_forward = build_part("feed_forward", feed_forward)
            self.feed_forward_norm = build_part("norm", feed_forward_norm)
            self.feed_forward_scale = LayerScale(hidden_size, feed_forward_scale)

    def mixers(self):
        return [self.mixer]

    def parts(self):
        out = [self.mixer_norm, self.mixer, self.mixer_scale]
        if self.feed_forward is not None:
            out += [self.feed_forward_norm, self.feed_forward, self.feed_forward_scale]
        return out

    def first_norm(self):
        return self.mixer_norm

    def forward(self, h, delta, ctx, caches, states, next_norm=None):
        x = self.mixer_norm.add_norm(h, delta, ctx)
        mixed = self.mixer.forward(x, ctx, caches[0], states[0])
        if self.feed_forward is None:
            scaled_add(h, mixed, self.mixer_scale.weight, ctx, then_norm=next_norm)
            return None
        scaled_add(h, mixed, self.mixer_scale.weight, ctx, then_norm=self.feed_forward_norm)
        x = self.feed_forward_norm.add_norm(h, None, ctx)
        scaled_add(h, self.feed_forward.forward(x, ctx), self.feed_forward_scale.weight, ctx,
                   then_norm=next_norm)
        return None


class PostNormBlock:
    """A norm on each sublayer's output only: h <- h + norm(mixers(in(h))), then, where the
    block has a feed-forward, h <- h + norm'(ff(in'(h))). What a sublayer reads is made from
    the stream by an input part (`parts/convolution.py`: the stream plus a short causal
    convolution of it, or the stream itself); those parts may keep per-request state, which
    the block declares through `state_parts()`. The block may hold several mixers side by
    side; all read the same input and their outputs are added under `mixer_scales` before
    the norm (at most two are built). The sums into the stream are made by the norm behind
    the sublayer, so the block leaves no pending delta."""

    def __init__(self, hidden_size: int, mixers: list, mixer_post_norm: PartSpec,
                 mixer_scales: list | None = None, mixer_input: PartSpec | None = None,
                 feed_forward: PartSpec | None = None,
                 feed_forward_post_norm: PartSpec | None = None,
                 feed_forward_input: PartSpec | None = None):
        if not 1 <= len(mixers) <= 2:
            raise ValueError(f"a block of {len(mixers)} mixers side by side is not built (1 or 2)")
        self._mixers = [build_part("mixer", m) for m in mixers]
        self.mixer_scales = [float(v) for v in (mixer_scales or [1.0] * len(mixers))]
        if len(self.mixer_scales) != len(self._mixers):
            raise ValueError("one scale per mixer")
        self.mixer_post_norm = build_part("norm", mixer_post_norm)
        self.mixer_input = build_input(mixer_input, hidden_size)
        self.feed_forward = self.feed_forward_post_norm = self.feed_forward_input = None
        if feed_forward is not None:
            if feed_forward_post_norm is None:
                raise ValueError("a feed-forward needs the norm behind it")
            self.feed_forward = build_part("feed_forward", feed_forward)
            self.feed_forward_post_norm = build_part("norm", feed_forward_post_norm)
            self.feed_forward_input = build_input(feed_forward_input, hidden_size)

    def mixers(self):
        return list(self._mixers)

    def _inputs(self):
        return [p for p in (self.mixer_input, self.feed_forward_input) if p is not None]

    def state_parts(self):
        return [p for p in self._inputs() if p.state_need() is not None]

    def parts(self):
        out = [self.mixer_input, *self._mixers, self.mixer_post_norm]
        if self.feed_forward is not None:
            out += [self.feed_forward_input, self.feed_forward, self.feed_forward_post_norm]
        return out

    def forward(self, h, delta, ctx, caches, states, next_norm=None):
        if delta is not None:
            raise ValueError("a post-norm block takes the stream with nothing pending")
        count = len(self._mixers)
        own = dict(zip(map(id, self.state_parts()), states[count:]))
        # the rings of the input convolutions are refilled by the norms behind the sublayers,
        # which see the stream as the convolutions read it
        ring = own.get(id(self.mixer_input))
        x = self.mixer_input.forward(h, ctx, ring, store_tail=False)
        outs = []
        for index, mixer in enumerate(self._mixers):
            # mixers side by side leave their outputs in buffers of their own
            ctx.side = index
            outs.append(mixer.forward(x, ctx, caches[index], states[index]))
        ctx.side = 0
        if count == 1 and self.mixer_scales[0] == 1.0:
            self.mixer_post_norm.normed_add(h, outs[0], ctx, tail=ring)
        else:
            self.mixer_post_norm.normed_add(h, outs[0], ctx,
                                            second=outs[1] if count == 2 else None,
                                            scales=(self.mixer_scales[0],
                                                    self.mixer_scales[1] if count == 2 else 0.0),
                                            tail=ring)
        if self.feed_forward is None:
            return None
        ring = own.get(id(self.feed_forward_input))
        x = self.feed_forward_input.forward(h, ctx, ring, store_tail=False)
        self.feed_forward_post_norm.normed_add(h, self.feed_forward.forward(x, ctx), ctx, tail=ring)
        return None


register_arrangement("pre_norm", PreNormBlock)
register_arrangement("post_norm", PostNormBlock)
register_arrangement("pre_norm_layer_scale", LayerScaleBlock)
register_arrangement("sandwich_norm", SandwichBlock)
