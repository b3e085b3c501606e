"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases
(mercury/model/qwen2.py:34-42, with act = SiLU). Gate and up are held as one packed matrix
`[2 * intermediate, hidden]` (gate rows first) so that one product feeds both. `activation`
is "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))); `names` gives
the checkpoint's names of the three matrices behind `prefix`."""

from __future__ import annotations

import torch

from .base import FeedForward, PartSpec, TensorSpec, build_part, register_feed_forward


class GatedFeedForward(FeedForward):
    capturable = True
    accepts_pending_norm = True
    adds_to_residual = True

    ACTIVATIONS = ("silu", "gelu_tanh", "clamped_sigmoid")

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str,
                 activation: str = "silu",
                 names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight"),
                 float_out: bool = False, limit: float = 0.0, slope: float = 1.0,
                 out_name: str = "sublayer_out"):
        """`float_out`: the result is left in float32 (from the down-projection's accumulators)
        for a block that scales it before the sum; such a block makes the sum itself.
        "clamped_sigmoid": with g = min(gate, limit) and u = clamp(up, -limit, limit) the
        product's input is g sigmoid(slope g) (u + 1). `out_name`: the float32 buffer the result
        is left in (a feed-forward that runs beside another names its own)."""
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not built; only "
                             f"{' and '.join(self.ACTIVATIONS)}")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.prefix = prefix
        self.activation = activation
        self.names = tuple(names)
        self.float_out = bool(float_out)
        self.limit, self.slope, self.out_name = float(limit), float(slope), out_name
        if activation == "clamped_sigmoid" and self.limit <= 0:
            raise ValueError("the clamped gate needs a positive limit")
        # the fused products that add into the stream belong to the pre-norm block
        if activation != "silu" or self.float_out:
            self.adds_to_residual = False
            self.accepts_pending_norm = False
        self.gate_up_weight = self.down_weight = None

    def tensor_specs(self):
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(p + self.names[0], (i, h)),
            TensorSpec(p + self.names[1], (i, h)),
            TensorSpec(p + self.names[2], (h, i)),
        ]

    def load(self, tensors, setup):
        p = self.prefix
        gate = setup.place(tensors[p + self.names[0]])
        up = setup.place(tensors[p + self.names[1]])
        widest = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        self.gate_up_weight = torch.cat([gate.to(widest), up.to(widest)], dim=0).contiguous()
        self.down_weight = setup.place(tensors[p + self.names[2]])

    def forward(self, x, ctx, residual=None, then_norm=None):
        tokens = x.shape[0]
        act = ctx.buffer("ff_act", tokens, self.intermediate_size)
        if self.activation != "silu":
            if self.activation == "clamped_sigmoid":
                ctx.ops.linear_gated(x, self.gate_up_weight, act, ctx, self.activation,
                                     limit=self.limit, slope=self.slope)
            else:
                ctx.ops.linear_gated(x, self.gate_up_weight, act, ctx, self.activation)
            # float32: the result goes through a norm before it joins the stream
            out = ctx.buffer(self.out_name, tokens, self.hidden_size, dtype="float32")
            ctx.ops.linear(act, self.down_weight, None, out)
            return out
        ctx.ops.linear_swiglu(x, self.gate_up_weight, act, ctx, ahead=self.down_weight)
        if self.float_out:
            out = ctx.buffer(self.out_name, tokens, self.hidden_size, dtype="float32")
            ctx.ops.linear(act, self.down_weight, None, out)
            return out
        if residual is not None:
            return ctx.ops.linear_residual(act, self.down_weight, None, residual, ctx, "ff_out",
                                           then_norm=then_norm)
        out = ctx.buffer("ff_out", tokens, self.hidden_size)
        ctx.ops.linear(act, self.down_weight, None, out)
        return out


class RoutedExperts(FeedForward):
    """A mixture of SiLU-gated experts, of which each token uses `top`.

    Router: z = Wr x in float32, s = sigmoid(z). The choice is made on s + correction (a
    learned number per expert that steers the choice and nothing else): the experts form
    `group_count` equal groups of neighbours, a group's score is the sum of its two largest
    choice scores, only experts of the best `group_keep` groups can be chosen, and of those
    the `top` with the largest choice scores are. A chosen expert's weight is its s times
    `route_scale`; the weights are not renormalised. out = sum of weight_e * expert_e(x).

    `correction=False`: the checkpoint has no such numbers and the choice is made on s itself.
    `weight_on` "input": the weight multiplies what the expert reads, out = sum of expert_e(
    weight_e * x), instead of what it returns. `shared`: a feed-forward (`PartSpec`) that runs
    for every token beside the routed ones; `forward` then returns (routed, shared), two
    float32 tensors whose sum is the sublayer's output.

    The experts' matrices are held stacked, `[experts, 2 ff, hidden]` (gate rows, then up
    rows) and `[experts, hidden, ff]`, so that one grouped product serves all of them.
    """

    capturable = True

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int,
                 route_scale: float, prefix: str, group_count: int = 1, group_keep: int = 1,
                 names: dict | None = None, correction: bool = True, weight_on: str = "output",
                 shared: PartSpec | None = None):
        if experts % group_count or group_keep > group_count:
            raise ValueError(f"{experts} experts do not form {group_count} groups of which "
                             f"{group_keep} are kept")
        if top > group_keep * (experts // group_count):
            raise ValueError(f"{top} experts cannot be chosen from {group_keep} groups of "
                             f"{experts // group_count}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.experts, self.top, self.route_scale = experts, top, float(route_scale)
        self.group_count, self.group_keep, self.prefix = group_count, group_keep, prefix
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on={weight_on!r} is neither 'output' nor 'input'")
        self.has_correction, self.weight_on = bool(correction), weight_on
        self.shared = build_part("feed_forward", shared) if shared is not None else None
        self.names = {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down",
                      "router": "router", "correction": "correction"}
        self.names.update(names or {})

    def _expert(self, index: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(index) + self.names[which]

    def tensor_specs(self):
        h, f = self.hidden_size, self.intermediate_size
        specs = []
        for e in range(self.experts):
            specs += [TensorSpec(self._expert(e, "gate"), (f, h)), TensorSpec(self._expert(e, "up"), (f, h)),
                      TensorSpec(self._expert(e, "down"), (h, f))]
        specs.append(TensorSpec(self.prefix + self.names["router"], (self.experts, h), std=0.2))
        if self.has_correction:
            specs.append(TensorSpec(self.prefix + self.names["correction"], (self.experts,), std=0.2))
        return specs + (self.shared.tensor_specs() if self.shared is not None else [])

    def load(self, tensors, setup):
        placed = [[setup.place(tensors[self._expert(e, which)]) for which in ("gate", "up", "down")]
                  for e in range(self.experts)]
        widest = (torch.float32 if any(t.dtype == torch.float32 for row in placed for t in row)
                  else placed[0][0].dtype)
        self.gate_up_weight = torch.stack([torch.cat([g.to(widest), u.to(widest)], dim=0)
                                           for g, u, _d in placed]).contiguous()
        self.down_weight = torch.stack([d.to(widest) for _g, _u, d in placed]).contiguous()
        # the router is float32 in both engines
        self.router = setup.place(tensors[self.prefix + self.names["router"]]).float().contiguous()
        if self.has_correction:
            self.correction = setup.place(
                tensors[self.prefix + self.names["correction"]]).float().contiguous()
        else:
            self.correction = torch.zeros(self.experts, dtype=torch.float32, device=self.router.device)
        if self.shared is not None:
            self.shared.load(tensors, setup)

    def forward(self, x, ctx):
        tokens, ops = x.shape[0], ctx.ops
        chosen = ctx.buffer("route_experts", tokens, self.top, dtype=torch.int32)
        weights = ctx.buffer("route_weights", tokens, self.top, dtype="float32")
        ops.route_experts(x, self.router, self.correction, self.group_count, self.group_keep,
                          self.route_scale, chosen, weights)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        if self.weight_on == "input":
            ops.expert_feed_forward(x, chosen, weights, self.gate_up_weight, self.down_weight, out,
                                    ctx, weight_on="input")
        else:
            ops.expert_feed_forward(x, chosen, weights, self.gate_up_weight, self.down_weight, out, ctx)
        if self.shared is None:
            return out
        return out, self.shared.forward(x, ctx)


register_feed_forward("gated", GatedFeedForward)
register_feed_forward("routed_experts", RoutedExperts)
