"""Mixers that carry a state of fixed size from token to token instead of keys and values.

Both keep their state in float32 in the slot the cache manager gave the request, start it
at zero, and run a step's tokens of each sequence in order from where the step before
left it. Everything inside the recurrence (gates, decays, the state) is float32; the
projections around it are products like any other.

`MinGRU`:  z = sigmoid(Wz x + bz), u = Wx x + bx, c = u + 1/2 where u >= 0 and sigmoid(u)
           where u < 0;  S_t = (1 - z) S_{t-1} + z c;  out = Wo (S_t * silu(Wg x)).
`GatedLinearRecurrence` (the recurrent block of Griffin: De et al., "Griffin: Mixing Gated
Linear Recurrences with Local Attention for Efficient Language Models"):
           y = gelu_tanh(Wy x + by); u = conv(Wx x + bx), a causal convolution per channel
           over `taps` tokens; per block b of the channels r = sigmoid(Ra_b u_b + ra_b) and
           i = sigmoid(Ri_b u_b + ri_b); a = exp(-decay_scale * r * softplus(lam));
           S_t = a S_{t-1} + sqrt(1 - a^2) * i * u;  out = Wo (S_t * y).
           Its state is S and the last taps - 1 inputs of the convolution.
`Mamba2` (Dao and Gu, "Transformers are SSMs: Generalized Models and Efficient Algorithms
Through Structured State Space Duality"): [z | x | B | C | dt] = W_in h; (x, B, C) through a
           causal convolution with bias and SiLU; dt = softplus(dt + dt_bias); per head, with
           B and C of the head's group, S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T
           (S is state x head_dim), y_t = S_t^T C_t + D x_t; out = Wo (groupnorm(y * silu(z)) * w),
           the norm an RMS norm over each of `norm_groups` equal parts.
`GatedDeltaRule` (Yang, Kautz and Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with
Delta Rule"): q, k, v through causal convolutions and SiLU; q, k to unit length per head, q
           also times key_dim^-1/2; beta = sigmoid(Wb h), g = exp(-exp(A_log) softplus(Wa h +
           dt_bias)); S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q (the read-out
           sees the token's own write; S is key_dim x head_dim); out = Wo (o / rms(o) * w *
           silu(Wg h)).
Both keep S and the last taps - 1 inputs of their convolutions in one state row per
request: [S | inputs one token back | two tokens back | ...].
`GeneralizedDeltaRule`: r, k, v = Wr h, Wk h, Wv h (heads x dim each); a decay per head and key
           channel, w = exp(-decay_scale * sigmoid(W2 tanh(W1 h) + w0)) (a low-rank map of the
           input); a removal rate per head and key channel, a = sigmoid(Wa h + ba); with the unit
           key u = k / sqrt(sum k^2 + unit_eps) of each head, S_t = diag(w) S_(t-1) - (a * u)
           (u^T S_(t-1)) + k v^T, both terms reading the matrix as the token found it; o = S_t^T
           r; out = Wo (o / rms(o) per head * w_norm * sigmoid(Wg h)). Its state is S alone.
`Retention` (Sun et al., "Retentive Network: A Successor to Transformer for Large Language
           Models"): q = Wq h, k = Wk h (heads x dim), v = Wv h (heads x vdim); q and k turned by
           the position encoding, k then times key_scale (dim^-1/2); per head S_t = decay_h
           S_(t-1) + k_t v_t^T with a fixed decay per head, o_t = S_t^T q_t, neither softmax nor
           denominator; out = Wo (o / rms(o) per head * silu(Wg h)). Its state is S alone.
"""

from __future__ import annotations

import torch

from .base import Mixer, PartSpec, StateNeed, TensorSpec, build_part, register_mixer


class MinGRU(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, width: int, prefix: str, names: dict | None = None,
                 bias_suffix: str = ".b"):
        self.hidden_size, self.width, self.prefix = hidden_size, width, prefix
        self.names = {"z": "z", "x": "x", "g": "g", "o": "o"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix
        self.in_weight = self.in_bias = self.out_weight = None

    def state_need(self):
        return StateNeed((self.width,), torch.float32)

    def tensor_specs(self):
        p, n, b, h, w = self.prefix, self.names, self.bias_suffix, self.hidden_size, self.width
        return [TensorSpec(p + n["z"], (w, h)), TensorSpec(p + n["z"] + b, (w,)),
                TensorSpec(p + n["x"], (w, h)), TensorSpec(p + n["x"] + b, (w,)),
                TensorSpec(p + n["g"], (w, h)), TensorSpec(p + n["o"], (h, w))]

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix
        mats = [setup.place(tensors[p + n[k]]) for k in ("z", "x", "g")]
        biases = [setup.place(tensors[p + n["z"] + b]), setup.place(tensors[p + n["x"] + b])]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats + biases) else mats[0].dtype
        # one product feeds the gate, the candidate and the output gate: rows [z; x; g]
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()
        self.in_bias = torch.cat([t.to(widest) for t in biases]
                                 + [torch.zeros(self.width, dtype=widest, device=mats[0].device)]
                                 ).contiguous()
        self.out_weight = setup.place(tensors[p + n["o"]])

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        pre = ctx.buffer("recurrent_in", tokens, 3 * self.width, dtype="float32")
        ops.linear(x, self.in_weight, self.in_bias, pre)
        mixed = ctx.buffer("recurrent_mixed", tokens, self.width)
        ops.mingru_scan(pre, state, ctx.batch, mixed)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(mixed, self.out_weight, None, out)
        return out


class GatedLinearRecurrence(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, width: int, blocks: int, taps: int, prefix: str,
                 decay_scale: float = 8.0, names: dict | None = None, bias_suffix: str = ".b"):
        if width % blocks:
            raise ValueError(f"width {width} does not divide into {blocks} blocks")
        if not 1 <= taps <= 16:
            raise ValueError(f"a convolution over {taps} tokens is not built (1 to 16)")
        self.hidden_size, self.width, self.blocks, self.taps = hidden_size, width, blocks, taps
        self.prefix = prefix
        self.decay_scale = float(decay_scale)
        self.names = {"y": "y", "x": "x", "conv": "conv", "ra": "ra", "ri": "ri", "lam": "lam",
                      "o": "o"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix

    def state_need(self):
        # row 0: S; row j >= 1: the convolution's input j tokens back
        return StateNeed((self.taps, self.width), torch.float32)

    def tensor_specs(self):
        p, n, b, h, w = self.prefix, self.names, self.bias_suffix, self.hidden_size, self.width
        size = w // self.blocks
        return [TensorSpec(p + n["y"], (w, h)), TensorSpec(p + n["y"] + b, (w,)),
                TensorSpec(p + n["x"], (w, h)), TensorSpec(p + n["x"] + b, (w,)),
                TensorSpec(p + n["conv"], (w, self.taps), std=0.3),
                TensorSpec(p + n["conv"] + b, (w,)),
                TensorSpec(p + n["ra"], (self.blocks, size, size), std=0.1),
                TensorSpec(p + n["ra"] + b, (self.blocks, size)),
                TensorSpec(p + n["ri"], (self.blocks, size, size), std=0.1),
                TensorSpec(p + n["ri"] + b, (self.blocks, size)),
                TensorSpec(p + n["lam"], (w,), std=0.5, mean=-1.0),
                TensorSpec(p + n["o"], (h, w))]

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix
        place = lambda name: setup.place(tensors[p + name])
        mats = [place(n["y"]), place(n["x"])]
        biases = [place(n["y"] + b), place(n["x"] + b)]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats + biases) else mats[0].dtype
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()   # rows [y; x]
        self.in_bias = torch.cat([t.to(widest) for t in biases]).contiguous()
        # what stands inside the recurrence is float32: taps, gate matrices, decay
        self.conv = place(n["conv"]).float().contiguous()
        self.conv_bias = place(n["conv"] + b).float().contiguous()
        # [2][blocks][in][out]: input-major, the way the gate kernel reads it
        self.gate_weight = torch.stack([place(n["ra"]).float(), place(n["ri"]).float()]
                                       ).transpose(-1, -2).contiguous()
        self.gate_bias = torch.stack([place(n["ra"] + b).float(), place(n["ri"] + b).float()]).contiguous()
        self.softplus_lam = torch.nn.functional.softplus(place(n["lam"]).float()).contiguous()
        self.out_weight = place(n["o"])

    def forward(self, x, ctx, cache, state):
        tokens, ops, w = x.shape[0], ctx.ops, self.width
        pre = ctx.buffer("recurrent_in", tokens, 2 * w, dtype="float32")
        ops.linear(x, self.in_weight, self.in_bias, pre)
        u = ctx.buffer("recurrent_conv", tokens, w, dtype="float32")
        ops.causal_conv(pre, w, w, self.conv, self.conv_bias, state, ctx.batch, u)
        gates = ctx.buffer("recurrent_gates", tokens, 2 * w, dtype="float32")
        ops.block_gates(u, self.gate_weight, self.gate_bias, gates)
        mixed = ctx.buffer("recurrent_mixed", tokens, w)
        ops.gated_recurrence_scan(pre, u, gates, self.softplus_lam, self.decay_scale, state,
                                  ctx.batch, mixed)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(mixed, self.out_weight, None, out)
        return out


def _float(setup, tensor):
    """What stands inside a recurrence is float32 in both engines."""
    return setup.place(tensor).float().contiguous()


class Mamba2(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, heads: int, head_dim: int, state_size: int, groups: int,
                 norm_groups: int, taps: int, eps: float, prefix: str, names: dict | None = None):
        if heads % groups:
            raise ValueError(f"{heads} heads do not divide into {groups} groups")
        if (heads * head_dim) % norm_groups:
            raise ValueError(f"{heads * head_dim} channels do not divide into {norm_groups} norm groups")
        if not 1 <= taps <= 16:
            raise ValueError(f"a convolution over {taps} tokens is not built (1 to 16)")
        self.hidden_size, self.heads, self.head_dim = hidden_size, heads, head_dim
        self.state_size, self.groups, self.norm_groups, self.taps = state_size, groups, norm_groups, taps
        self.eps, self.prefix = float(eps), prefix
        self.inner = heads * head_dim
        self.channels = self.inner + 2 * groups * state_size        # what the convolution sees
        self.proj = 2 * self.inner + 2 * groups * state_size + heads
        self.cells = heads * state_size * head_dim
        self.names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias",
                      "A_log": "A_log", "D": "D", "norm": "norm", "o": "o"}
        self.names.update(names or {})

    def state_need(self):
        return StateNeed((self.cells + (self.taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self):
        p, n = self.prefix, self.names
        return [TensorSpec(p + n["in"], (self.proj, self.hidden_size)),
                TensorSpec(p + n["conv"], (self.channels, self.taps), std=0.3),
                TensorSpec(p + n["conv_bias"], (self.channels,)),
                TensorSpec(p + n["dt_bias"], (self.heads,), std=0.5, mean=-0.5),
                TensorSpec(p + n["A_log"], (self.heads,), std=0.5),
                TensorSpec(p + n["D"], (self.heads,), init="ones_normal", std=0.1),
                TensorSpec(p + n["norm"], (self.inner,), init="ones_normal", std=0.05),
                TensorSpec(p + n["o"], (self.hidden_size, self.inner))]

    def load(self, tensors, setup):
        p, n = self.prefix, self.names
        self.in_weight = setup.place(tensors[p + n["in"]])
        self.conv = _float(setup, tensors[p + n["conv"]])
        self.conv_bias = _float(setup, tensors[p + n["conv_bias"]])
        self.dt_bias = _float(setup, tensors[p + n["dt_bias"]])
        self.neg_rate = (-torch.exp(_float(setup, tensors[p + n["A_log"]]))).contiguous()
        self.skip = _float(setup, tensors[p + n["D"]])
        self.norm_weight = _float(setup, tensors[p + n["norm"]])
        self.out_weight = setup.place(tensors[p + n["o"]])

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        pre = ctx.buffer("recurrent_in", tokens, self.proj, dtype="float32")
        ops.linear(x, self.in_weight, None, pre)
        cells, tail = state[:, :self.cells], state[:, self.cells:]
        xbc = ctx.buffer("recurrent_conv", tokens, self.channels, dtype="float32")
        ops.conv_act_update(pre, self.inner, self.conv, self.conv_bias, tail, ctx.batch, xbc, "silu")
        y = ctx.buffer("recurrent_y", tokens, self.inner, dtype="float32")
        ops.mamba2_scan(xbc, pre, self.proj - self.heads, self.dt_bias, self.neg_rate, self.skip,
                        (self.heads, self.head_dim, self.state_size, self.groups), cells,
                        ctx.batch, y, precise=ctx.dtype == torch.float32)
        mixed = ctx.buffer("recurrent_mixed", tokens, self.inner)
        ops.gated_group_norm(y, pre, 0, self.norm_weight, self.norm_groups, self.eps, True, mixed)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(mixed, self.out_weight, None, out)
        return out


class GatedDeltaRule(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, heads: int, key_heads: int, key_dim: int, head_dim: int,
                 taps: int, eps: float, prefix: str, unit_eps: float = 1e-6,
                 names: dict | None = None):
        if heads % key_heads:
            raise ValueError(f"{heads} heads do not divide into {key_heads} query/key heads")
        if not 1 <= taps <= 16:
            raise ValueError(f"a convolution over {taps} tokens is not built (1 to 16)")
        self.hidden_size, self.heads, self.key_heads = hidden_size, heads, key_heads
        self.key_dim, self.head_dim, self.taps = key_dim, head_dim, taps
        self.eps, self.unit_eps, self.prefix = float(eps), float(unit_eps), prefix
        self.qk = key_heads * key_dim
        self.inner = heads * head_dim
        self.channels = 2 * self.qk + self.inner                  # [q | k | v]
        self.proj = self.channels + self.inner + 2 * heads         # ... | g | b | a
        self.cells = heads * key_dim * head_dim
        self.names = {"q": "q", "k": "k", "v": "v", "conv": ".conv", "b": "b", "a": "a", "g": "g",
                      "dt_bias": "dt_bias", "A_log": "A_log", "norm": "norm", "o": "o"}
        self.names.update(names or {})

    def state_need(self):
        return StateNeed((self.cells + (self.taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self):
        p, n, h = self.prefix, self.names, self.hidden_size
        specs = []
        for key, rows in (("q", self.qk), ("k", self.qk), ("v", self.inner)):
            specs += [TensorSpec(p + n[key], (rows, h)),
                      TensorSpec(p + n[key] + n["conv"], (rows, self.taps), std=0.3)]
        return specs + [TensorSpec(p + n["b"], (self.heads, h)), TensorSpec(p + n["a"], (self.heads, h)),
                        TensorSpec(p + n["g"], (self.inner, h)),
                        TensorSpec(p + n["dt_bias"], (self.heads,), std=0.5, mean=-0.5),
                        TensorSpec(p + n["A_log"], (self.heads,), std=0.5),
                        TensorSpec(p + n["norm"], (self.head_dim,), init="ones_normal", std=0.05),
                        TensorSpec(p + n["o"], (h, self.inner))]

    def load(self, tensors, setup):
        p, n = self.prefix, self.names
        mats = [setup.place(tensors[p + n[key]]) for key in ("q", "k", "v", "g", "b", "a")]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        # one product feeds everything that is read off the layer's input: rows [q; k; v; g; b; a]
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()
        self.conv = torch.cat([_float(setup, tensors[p + n[key] + n["conv"]])
                               for key in ("q", "k", "v")], dim=0).contiguous()
        self.dt_bias = _float(setup, tensors[p + n["dt_bias"]])
        self.neg_rate = (-torch.exp(_float(setup, tensors[p + n["A_log"]]))).contiguous()
        self.norm_weight = _float(setup, tensors[p + n["norm"]])
        self.out_weight = setup.place(tensors[p + n["o"]])

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        pre = ctx.buffer("recurrent_in", tokens, self.proj, dtype="float32")
        ops.linear(x, self.in_weight, None, pre)
        cells, tail = state[:, :self.cells], state[:, self.cells:]
        qkv = ctx.buffer("recurrent_conv", tokens, self.channels, dtype="float32")
        ops.conv_act_update(pre, 0, self.conv, None, tail, ctx.batch, qkv, "silu")
        o = ctx.buffer("recurrent_y", tokens, self.inner, dtype="float32")
        gate_at = self.channels
        ops.delta_rule_scan(qkv, pre, gate_at + self.inner, gate_at + self.inner + self.heads,
                            self.dt_bias, self.neg_rate,
                            (self.heads, self.key_heads, self.key_dim, self.head_dim),
                            self.unit_eps, cells, ctx.batch, o, precise=ctx.dtype == torch.float32)
        mixed = ctx.buffer("recurrent_mixed", tokens, self.inner)
        ops.gated_group_norm(o, pre, gate_at, self.norm_weight, self.heads, self.eps, False, mixed)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(mixed, self.out_weight, None, out)
        return out


class GeneralizedDeltaRule(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, heads: int, key_dim: int, decay_rank: int, eps: float,
                 prefix: str, head_dim: int | None = None, decay_scale: float = 0.6065306597126334,
                 unit_eps: float = 1e-6, names: dict | None = None, bias_suffix: str = ".b"):
        """`decay_scale`: the decay is exp(-decay_scale * sigmoid(.)), so a channel keeps at
        least exp(-decay_scale) of its row per token; `decay_rank`: rows of W1."""
        self.hidden_size, self.heads, self.key_dim = hidden_size, heads, key_dim
        self.head_dim = key_dim if head_dim is None else int(head_dim)
        self.decay_rank = int(decay_rank)
        self.eps, self.unit_eps, self.prefix = float(eps), float(unit_eps), prefix
        self.decay_scale = float(decay_scale)
        self.keys = heads * key_dim
        self.inner = heads * self.head_dim
        # what one product reads off the layer's input: [r | k | v | g | a | t]
        self.offsets = {"r": 0, "k": self.keys, "v": 2 * self.keys, "g": 2 * self.keys + self.inner,
                        "a": 2 * self.keys + 2 * self.inner,
                        "t": 3 * self.keys + 2 * self.inner}
        self.proj = self.offsets["t"] + self.decay_rank
        self.cells = heads * key_dim * self.head_dim
        self.names = {"r": "r", "k": "k", "v": "v", "g": "g", "a": "a", "w1": "w1", "w2": "w2",
                      "w0": "w0", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix

    def state_need(self):
        return StateNeed((self.cells,), torch.float32)

    def tensor_specs(self):
        p, n, h = self.prefix, self.names, self.hidden_size
        return [TensorSpec(p + n["r"], (self.keys, h), std=0.05),
                TensorSpec(p + n["k"], (self.keys, h), std=0.05),
                TensorSpec(p + n["v"], (self.inner, h), std=0.05),
                TensorSpec(p + n["g"], (self.inner, h), std=0.05),
                TensorSpec(p + n["a"], (self.keys, h), std=0.05),
                TensorSpec(p + n["a"] + self.bias_suffix, (self.keys,), std=0.5),
                TensorSpec(p + n["w1"], (self.decay_rank, h), std=0.05),
                TensorSpec(p + n["w2"], (self.keys, self.decay_rank), std=0.3),
                TensorSpec(p + n["w0"], (self.keys,), std=1.0),
                TensorSpec(p + n["norm"], (self.inner,), init="ones_normal", std=0.05),
                TensorSpec(p + n["o"], (h, self.inner))]

    def load(self, tensors, setup):
        p, n = self.prefix, self.names
        mats = [setup.place(tensors[p + n[key]]) for key in ("r", "k", "v", "g", "a", "w1")]
        bias = setup.place(tensors[p + n["a"] + self.bias_suffix])
        widest = (torch.float32 if any(t.dtype == torch.float32 for t in mats + [bias])
                  else mats[0].dtype)
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()
        in_bias = torch.zeros(self.proj, dtype=widest, device=bias.device)
        in_bias[self.offsets["a"]:self.offsets["a"] + self.keys] = bias.to(widest)
        self.in_bias = in_bias.contiguous()
        self.decay_weight = setup.place(tensors[p + n["w2"]])
        self.decay_bias = setup.place(tensors[p + n["w0"]]).to(self.decay_weight.dtype).contiguous()
        self.norm_weight = _float(setup, tensors[p + n["norm"]])
        self.out_weight = setup.place(tensors[p + n["o"]])

    def forward(self, x, ctx, cache, state):
        tokens, ops, at = x.shape[0], ctx.ops, self.offsets
        pre = ctx.buffer("recurrent_in", tokens, self.proj, dtype="float32")
        ops.linear(x, self.in_weight, self.in_bias, pre)
        # (float32: what makes the decay is 32-bit arithmetic)
        squashed = ctx.buffer("recurrent_decay_in", tokens, self.decay_rank, dtype="float32")
        ops.tanh_slice(pre, at["t"], self.decay_rank, squashed)
        decay = ctx.buffer("recurrent_decay", tokens, self.keys, dtype="float32")
        ops.linear(squashed, self.decay_weight, self.decay_bias, decay)
        o = ctx.buffer("recurrent_y", tokens, self.inner, dtype="float32")
        ops.general_delta_scan(pre, (at["r"], at["k"], at["v"], at["a"]), decay, self.decay_scale,
                               (self.heads, self.key_dim, self.head_dim), self.unit_eps, state,
                               ctx.batch, o, precise=ctx.dtype == torch.float32)
        mixed = ctx.buffer("recurrent_mixed", tokens, self.inner)
        ops.gated_group_norm(o, pre, at["g"], self.norm_weight, self.heads, self.eps, False, mixed,
                             gate="sigmoid")
        out = ctx.sublayer_out(tokens, self.hidden_size)
        ops.linear(mixed, self.out_weight, None, out)
        return out


class Retention(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, heads: int, key_dim: int, value_dim: int, decay: list,
                 eps: float, prefix: str, key_scale: float | None = None, names: dict | None = None,
                 position_encoding: PartSpec | None = None):
        """`decay`: one number per head; `key_scale`: what the rotated keys are multiplied by
        (default key_dim^-1/2)."""
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        self.hidden_size, self.heads, self.key_dim, self.value_dim = hidden_size, heads, key_dim, value_dim
        self.decay_values = [float(v) for v in decay]
        self.eps, self.prefix = float(eps), prefix
        self.key_scale = float(key_dim) ** -0.5 if key_scale is None else float(key_scale)
        self.position = (build_part("position_encoding", position_encoding)
                         if position_encoding is not None else None)
        self.keys, self.inner = heads * key_dim, heads * value_dim
        # what one product reads off the layer's input: [q | k | v | g]
        self.offsets = {"q": 0, "k": self.keys, "v": 2 * self.keys, "g": 2 * self.keys + self.inner}
        self.proj = 2 * self.keys + 2 * self.inner
        self.cells = heads * key_dim * value_dim
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
        self.names.update(names or {})

    def state_need(self):
        return StateNeed((self.cells,), torch.float32)

    def tensor_specs(self):
        p, n, h = self.prefix, self.names, self.hidden_size
        return [TensorSpec(p + n["q"], (self.keys, h), std=0.05),
                TensorSpec(p + n["k"], (self.keys, h), std=0.05),
                TensorSpec(p + n["v"], (self.inner, h), std=0.05),
                TensorSpec(p + n["g"], (self.inner, h), std=0.05),
                TensorSpec(p + n["o"], (h, self.inner))] + (
                    self.position.tensor_specs() if self.position is not None else [])

    def load(self, tensors, setup):
        p, n = self.prefix, self.names
        mats = [setup.place(tensors[p + n[key]]) for key in ("q", "k", "v", "g")]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=setup.device)
        # the read-out's norm has no weight: the kernel that norms and gates takes ones
        self.norm_weight = torch.ones(self.value_dim, dtype=torch.float32, device=setup.device)
        self.out_weight = setup.place(tensors[p + n["o"]])
        if self.position is not None:
            self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state):
        tokens, ops, at = x.shape[0], ctx.ops, self.offsets
        # float32: what enters the recurrence is 32-bit
        pre = ctx.buffer("recurrent_in", tokens, self.proj, dtype="float32")
        ops.linear(x, self.in_weight, None, pre)
        tables = self.position.rotary_tables() if self.position is not None else None
        pairing = getattr(self.position, "pairing", "halves")
        o = ctx.buffer("recurrent_y", tokens, self.inner, dtype="float32")
        ops.retention_scan(pre, (at["q"], at["k"], at["v"]), self.decay, self.key_scale,
                           (self.heads, self.key_dim, self.value_dim), tables, pairing, state,
                           ctx.batch, o)
        mixed = ctx.buffer("recurrent_mixed", tokens, self.inner)
        ops.gated_group_norm(o, pre, at["g"], self.norm_weight, self.heads, self.eps, False, mixed)
        out = ctx.sublayer_out(tokens, self.hidden_size)
        ops.linear(mixed, self.out_weight, None, out)
        return out


register_mixer("mingru", MinGRU)
register_mixer("retention", Retention)
register_mixer("generalized_delta_rule", GeneralizedDeltaRule)
register_mixer("mamba2", Mamba2)
register_mixer("gated_delta_rule", GatedDeltaRule)
register_mixer("gated_linear_recurrence", GatedLinearRecurrence)
