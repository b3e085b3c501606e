"""RMSNorm fused with the residual sum.

The formula is mercury/model/qwen2.py:27-31: the pending delta is added to the residual
stream, the sum is the new residual, and the sum is normalised by rsqrt(mean(x^2) + eps)
and scaled by the weight. The reference adds in the activation dtype on its plain path and
in float32 on its fused path (mercury/kernels/rmsnorm_quant.py:40-46); here the stream
itself is float32, so nothing is rounded between layers.
"""

from __future__ import annotations

import torch

from .base import Norm, TensorSpec, register_norm

# A norm may also stand BEHIND a sublayer (`RMSNorm.normed_add`): the sublayer's output is
# normalised and only then added to the stream.


class PendingNorm:
    """A norm that has not run yet: the float32 stream, the weight and eps (and optionally
    which rows). A consumer whose kernel can normalise its input on the fly takes this
    instead of a tensor and saves the norm's own launch; any other consumer calls
    `materialize()` and gets the normalised rows."""

    def __init__(self, h, weight, eps, rows, ctx, size):
        self.h, self.weight, self.eps, self.rows, self.ctx, self.size = h, weight, eps, rows, ctx, size
        self.shape = ((h.shape[0] if rows is None else rows.shape[0]), size)
        self.dtype = ctx.dtype

    def materialize(self):
        count = self.shape[0]
        out = self.ctx.buffer("normed" if self.rows is None else "normed_rows", count, self.size)
        self.ctx.ops.add_rmsnorm(self.h, None, self.weight, self.eps, out, self.rows)
        return out


class PendingScaled(PendingNorm):
    """A norm whose output exists up to the division by the row's rms: `x` holds the stream
    times the norm weight (bfloat16) and `ss_part` [rows, tiles] the stream's sums of
    squares per 16-column tile, both left by the product that updated the stream. A product
    that takes this multiplies its result rows by 1/rms (a row scale commutes with the
    product); any other consumer calls `materialize()`, which runs the norm from the
    stream."""

    def __init__(self, x, ss_part, h, weight, eps, ctx, size):
        super().__init__(h, weight, eps, None, ctx, size)
        self.x, self.ss_part = x, ss_part


class Computed:
    """A norm's output that a fused kernel has already written; `materialize()` hands it over."""

    def __init__(self, out):
        self.out = out
        self.shape, self.dtype = out.shape, out.dtype

    def materialize(self):
        return self.out


class RMSNorm(Norm):
    capturable = True

    def __init__(self, size: int, eps: float, weight_name: str, init_std: float = 0.05,
                 gain: str = "vector"):
        """`gain` "vector": one learned number per feature; "scalar": the checkpoint holds a
        single number for all features (it is spread over a vector when loaded, so the
        kernels are the same); "one_plus": the checkpoint holds w around zero and the norm
        multiplies by 1 + w (the sum is made once, in float32, when the weight is loaded, and
        kept in float32 in both engines: 1 + w rounded to 16 bits would lose most of w)."""
        if gain not in ("vector", "scalar", "one_plus"):
            raise ValueError(f"gain={gain!r} is none of 'vector', 'scalar', 'one_plus'")
        self.size = size
        self.eps = eps
        self.weight_name = weight_name
        self.init_std = init_std
        self.gain = gain
        self.weight = None

    def tensor_specs(self):
        if self.gain == "one_plus":
            return [TensorSpec(self.weight_name, (self.size,), std=self.init_std)]
        shape = (self.size,) if self.gain == "vector" else ()
        return [TensorSpec(self.weight_name, shape, init="ones_normal", std=self.init_std)]

    def load(self, tensors, setup):
        weight = setup.place(tensors[self.weight_name])
        if self.gain == "scalar":
            weight = weight.reshape(1).expand(self.size).contiguous()
        elif self.gain == "one_plus":
            weight = (1.0 + weight.float()).contiguous()
        self.weight = weight

    def normed_add(self, h, delta, ctx, then_norm=None, second=None, scales=None, tail=None):
        """h <- h + norm(delta): this norm applied to a sublayer's OUTPUT before it joins the
        float32 stream. With `then_norm` (an RMSNorm over the same width) the same kernel
        also leaves that norm's output of the new stream in `ctx.prenormed`. With `second`
        (the output of a mixer that ran beside the first) and `scales` (a, b) the norm is
        taken of a * delta + b * second. With `tail` (the ring of the convolution the sublayer
        read through) the same kernel first keeps the stream's rows as the sublayer found
        them, each sequence's last ones, in that ring."""
        follow = then_norm if (isinstance(then_norm, RMSNorm) and then_norm.size == self.size) else None
        if tail is not None:
            follow = None                 # the kernel that keeps the rows does not norm ahead
        out = ctx.buffer("normed", h.shape[0], self.size) if follow is not None else None
        extra = {}
        if second is not None or scales is not None:
            a, b = scales if scales is not None else (1.0, 1.0)
            extra = {"delta2": second, "scale": float(a), "scale2": float(b)}
        if tail is not None:
            extra["tail"] = (tail, ctx.batch)
        ctx.ops.rmsnorm_add(h, delta, self.weight, self.eps,
                            follow.weight if follow is not None else None,
                            follow.eps if follow is not None else 0.0, out, **extra)
        ctx.prenormed = (follow, Computed(out)) if follow is not None else None

    def joined_add(self, h, first, second, ctx, then_norm=None, norm_weights=None,
                   scales=(1.0, 1.0)):
        """h <- h + norm(a n(first) + b n(second)) with (a, b) = `scales`: two outputs that ran side
        by side, joined, then this norm, then the sum into the stream. `norm_weights` = [w1, w2]
        (float32): each output first passes an RMS norm of its own with that weight (this
        norm's eps), n(x) = rmsnorm(x) * w; without them n(x) = x. With `then_norm` the same
        kernel leaves that norm's output of the new stream in `ctx.prenormed`."""
        follow = then_norm if (isinstance(then_norm, RMSNorm) and then_norm.size == self.size) else None
        out = ctx.buffer("normed", h.shape[0], self.size) if follow is not None else None
        wx, wy = norm_weights if norm_weights is not None else (None, None)
        ctx.ops.rmsnorm_join_add(h, first, second, wx, wy, scales[0], scales[1],
                                 self._float_weight(), self.eps,
                                 follow._float_weight() if follow is not None else None,
                                 follow.eps if follow is not None else 0.0, out)
        ctx.prenormed = (follow, Computed(out)) if follow is not None else None

    def _float_weight(self):
        """The weight in float32 (made once; the weight itself where it is float32 already)."""
        if self.weight.dtype == torch.float32:
            return self.weight
        held = getattr(self, "_weight_f32", None)
        if held is None:
            held = self._weight_f32 = self.weight.float().contiguous()
        return held

    def add_norm(self, h, delta, ctx, rows=None, defer=False):
        """`defer=True` says that the consumer takes a `PendingNorm`; one is returned when
        nothing has to be added first and the kernels can fuse the norm for this many rows."""
        pre = getattr(ctx, "prenormed", None)
        if pre is not None:
            ctx.prenormed = None
            if pre[0] is self and delta is None and rows is None:
                # the product before this norm already left its output (up to the row scale)
                return pre[1] if defer else pre[1].materialize()
        count = h.shape[0] if rows is None else rows.shape[0]
        if (defer and delta is None
                and getattr(ctx.ops, "can_fuse_norm", lambda *a: False)(count, self.size, self.weight)):
            return PendingNorm(h, self.weight, self.eps, rows, ctx, self.size)
        out = ctx.buffer("normed" if rows is None else "normed_rows", count, self.size)
        ctx.ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
        return out


class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * w with a weight and no bias; mean and variance (the mean
    of the squared deviations) in float32 over the float32 stream. `add_norm` is the
    interface every norm has; `scaled_add` joins a sublayer's output to the stream under a
    per-feature scale and computes the norm that follows in the same kernel."""

    capturable = True
    center = True

    def __init__(self, size: int, eps: float, weight_name: str, init_std: float = 0.05):
        self.size = size
        self.eps = eps
        self.weight_name = weight_name
        self.init_std = init_std
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.size,), init="ones_normal", std=self.init_std)]

    def load(self, tensors, setup):
        self.weight = setup.place(tensors[self.weight_name])

    def add_norm(self, h, delta, ctx, rows=None, defer=False):
        pre = getattr(ctx, "prenormed", None)
        if pre is not None:
            ctx.prenormed = None
            if pre[0] is self and delta is None and rows is None:
                return pre[1].materialize()
        count = h.shape[0] if rows is None else rows.shape[0]
        out = ctx.buffer("normed" if rows is None else "normed_rows", count, self.size)
        ctx.ops.scaled_add_norm(h, delta, None, self.weight, self.eps, True, out, rows)
        return out


def scaled_add(h, delta, scale, ctx, then_norm=None):
    """h <- h + scale * delta in the float32 stream (`scale` one number per feature, or None).
    With `then_norm` (a `LayerNorm` or `RMSNorm` over the stream's width) the same kernel
    leaves that norm's output of the new stream in `ctx.prenormed`."""
    follow = then_norm if isinstance(then_norm, (LayerNorm, RMSNorm)) and then_norm.size == h.shape[1] else None
    out = ctx.buffer("normed", h.shape[0], h.shape[1]) if follow is not None else None
    ctx.ops.scaled_add_norm(h, delta, scale,
                            follow.weight if follow is not None else None,
                            follow.eps if follow is not None else 0.0,
                            bool(getattr(follow, "center", False)), out, None)
    ctx.prenormed = (follow, Computed(out)) if follow is not None else None


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
register_norm("rmsnorm_scalar", lambda **params: RMSNorm(gain="scalar", **params))
register_norm("rmsnorm_one_plus", lambda **params: RMSNorm(gain="one_plus", **params))
