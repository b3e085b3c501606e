"""Grouped-query attention over the paged cache.

Formulas of mercury/model/qwen2.py:45-69: q, k and v projections (bias on all three when
`qkv_bias`), position encoding on q and k after the bias and before the keys are stored,
keys and values stored before attending (mercury/model/attention.py:127, :154) so that a
portion sees its own keys, softmax(q.k * scale) over the keys j <= p, query head h reading
KV head h // (heads / kv_heads), and an output projection. The three projections are held
as one packed matrix so that one product feeds them.
"""

from __future__ import annotations

import torch

from .base import CacheNeed, Mixer, PartSpec, TensorSpec, build_part, register_mixer


class GroupedQueryAttention(Mixer):
    capturable = True
    accepts_pending_norm = True
    adds_to_residual = True

    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        scale: float,
        prefix: str,
        qkv_bias: bool = True,
        out_bias: bool = False,
        window: int = 0,
        position_encoding: PartSpec | None = None,
    ):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.prefix = prefix
        self.qkv_bias = qkv_bias
        self.out_bias = out_bias
        self.window = int(window)
        self.position = build_part(
            "position_encoding", position_encoding or PartSpec("none", {})
        )
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.qkv_weight = self.qkv_b = self.out_weight = self.out_b = None

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self):
        p, h = self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "q_proj.weight", (self.q_size, h)),
            TensorSpec(p + "k_proj.weight", (self.kv_size, h)),
            TensorSpec(p + "v_proj.weight", (self.kv_size, h)),
            TensorSpec(p + "o_proj.weight", (h, self.q_size)),
        ]
        if self.qkv_bias:
            specs += [
                TensorSpec(p + "q_proj.bias", (self.q_size,)),
                TensorSpec(p + "k_proj.bias", (self.kv_size,)),
                TensorSpec(p + "v_proj.bias", (self.kv_size,)),
            ]
        if self.out_bias:
            specs.append(TensorSpec(p + "o_proj.bias", (h,)))
        return specs + self.position.tensor_specs()      # a learned encoding owns tensors too

    def load(self, tensors, setup):
        p = self.prefix

        def packed(suffix):
            parts = [setup.place(tensors[p + name + suffix]) for name in ("q_proj", "k_proj", "v_proj")]
            widest = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
            return torch.cat([t.to(widest) for t in parts], dim=0).contiguous()

        self.qkv_weight = packed(".weight")
        self.qkv_b = packed(".bias") if self.qkv_bias else None
        self.out_weight = setup.place(tensors[p + "o_proj.weight"])
        self.out_b = setup.place(tensors[p + "o_proj.bias"]) if self.out_bias else None
        self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state, residual=None, then_norm=None):
        tokens = x.shape[0]
        ops = ctx.ops
        qkv = ctx.buffer("qkv", tokens, self.q_size + 2 * self.kv_size)
        form = self.position.fused_form()
        tables = self.position.rotary_tables() if form == "rotary" else None
        attended = ctx.buffer("attended", tokens, self.q_size)
        fused = getattr(ops, "qkv_attention", None)
        if fused is not None and form is not None:
            # projection, bias, rotation, store into the pages and attention: the kernels
            # choose how to share the work between them
            fused(x, self.qkv_weight, self.qkv_b, qkv, self.num_heads, self.num_kv_heads,
                  self.head_dim, tables, ctx.batch, cache, self.scale, self.window, attended)
            return self._project_out(attended, ctx, residual, then_norm, tokens)
        if form is not None:
            # projection, bias, rotation and the store into the pages, fused where it pays
            ops.qkv_rope_store(x, self.qkv_weight, self.qkv_b, qkv, self.num_heads,
                               self.num_kv_heads, self.head_dim, tables, ctx.batch, cache)
        else:
            if hasattr(x, "materialize"):
                x = x.materialize()
            ops.linear(x, self.qkv_weight, self.qkv_b, qkv)
            self.position.apply(qkv, (self.num_heads, self.num_kv_heads, self.head_dim), ctx)
            ops.rope_cache_write(qkv, self.num_heads, self.num_kv_heads, self.head_dim, None,
                                 ctx.batch, cache)
        ops.paged_attention(
            qkv, self.num_heads, self.num_kv_heads, self.head_dim, ctx.batch, cache,
            self.scale, self.window, attended,
        )
        return self._project_out(attended, ctx, residual, then_norm, tokens)

    def _project_out(self, attended, ctx, residual, then_norm, tokens):
        ops = ctx.ops
        if residual is not None:
            return ops.linear_residual(attended, self.out_weight, self.out_b, residual, ctx,
                                       "mixer_out", then_norm=then_norm)
        out = ctx.buffer("mixer_out", tokens, self.hidden_size)
        ops.linear(attended, self.out_weight, self.out_b, out)
        return out


register_mixer("grouped_query_attention", GroupedQueryAttention)


class MixedHeadAttention(Mixer):
    """Grouped-query attention whose heads exchange their softmax weights, with key and
    value heads of different sizes and an optional blend of the values across layers.

    Per token: q, k, v projections with biases; the position encoding on q and k; the value
    blend; keys and blended values stored in the pages; w_g = softmax(q_g . k * scale) over
    the keys j <= p (and inside `window`, if one is given); when `head_mix` is set the
    weights are mixed before they meet the values, w'_h = sum_g M[h, g] w_g with M a learned
    [heads, heads] matrix, and head h applies w'_h to the values of its own key/value head;
    an output projection with bias.

    `value_blend` = ("source", key): this layer's values of the step's tokens are left in
    `ctx.carry[key]` for later layers. ("blend", key): v <- (1 - c) v + c carry[key], with c
    one learned number (`names["blend"]`); the blended values are what the pages hold.

    `names` maps q, k, v, o (biases: the name + ".b" unless `bias_suffix` says otherwise),
    mix and blend to checkpoint names behind `prefix`.
    """

    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, prefix: str, names: dict | None = None,
                 bias_suffix: str = ".b", head_mix: bool = True,
                 value_blend: tuple | None = None, window: int = 0,
                 position_encoding: PartSpec | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale = float(scale)
        self.prefix = prefix
        self.names = {"q": "q", "k": "k", "v": "v", "o": "o", "mix": "talk", "blend": "vmix"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix
        self.head_mix = bool(head_mix)
        self.value_blend = tuple(value_blend) if value_blend else None
        if self.value_blend and self.value_blend[0] not in ("source", "blend"):
            raise ValueError(f"value_blend role {self.value_blend[0]!r}")
        self.window = int(window)
        self.position = build_part("position_encoding", position_encoding or PartSpec("none", {}))
        if self.position.fused_form() is None:
            raise ValueError("this mixer takes a rotary encoding or none")
        self.q_size = num_heads * head_dim
        self.k_size = num_kv_heads * head_dim
        self.v_size = num_kv_heads * value_dim
        self.qkv_weight = self.qkv_b = self.out_weight = self.out_b = None
        self.mix = self.blend = None

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window, self.value_dim)

    def tensor_specs(self):
        p, h, n, b = self.prefix, self.hidden_size, self.names, self.bias_suffix
        specs = [TensorSpec(p + n["q"], (self.q_size, h)), TensorSpec(p + n["q"] + b, (self.q_size,)),
                 TensorSpec(p + n["k"], (self.k_size, h)), TensorSpec(p + n["k"] + b, (self.k_size,)),
                 TensorSpec(p + n["v"], (self.v_size, h)), TensorSpec(p + n["v"] + b, (self.v_size,)),
                 TensorSpec(p + n["o"], (h, self.num_heads * self.value_dim)),
                 TensorSpec(p + n["o"] + b, (h,))]
        if self.head_mix:
            specs.append(TensorSpec(p + n["mix"], (self.num_heads, self.num_heads),
                                    init="eye_normal", std=0.1))
        if self.value_blend and self.value_blend[0] == "blend":
            specs.append(TensorSpec(p + n["blend"], (), std=0.1, mean=0.4))
        return specs + self.position.tensor_specs()

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix

        def packed(suffix):
            parts = [setup.place(tensors[p + n[key] + suffix]) for key in ("q", "k", "v")]
            widest = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
            return torch.cat([t.to(widest) for t in parts], dim=0).contiguous()

        self.qkv_weight, self.qkv_b = packed(""), packed(b)
        self.out_weight = setup.place(tensors[p + n["o"]])
        self.out_b = setup.place(tensors[p + n["o"] + b])
        # the weights of the softmax are float32, and so is what mixes them
        self.mix = setup.place(tensors[p + n["mix"]]).float().contiguous() if self.head_mix else None
        if self.value_blend and self.value_blend[0] == "blend":
            self.blend = setup.place(tensors[p + n["blend"]]).float().reshape(1).contiguous()
        self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state):
        tokens = x.shape[0]
        ops = ctx.ops
        qkv = ctx.buffer("qkv_split", tokens, self.q_size + self.k_size + self.v_size)
        ops.linear(x, self.qkv_weight, self.qkv_b, qkv)
        tables = self.position.rotary_tables() if self.position.fused_form() == "rotary" else None
        keep = blend_from = None
        if self.value_blend:
            role, key = self.value_blend
            if role == "source":
                keep = ctx.carry[key] = ctx.buffer("values_" + str(key), tokens, self.v_size)
            else:
                blend_from = ctx.carry.get(key)
                if blend_from is None or blend_from.shape[1] != self.v_size:
                    raise ValueError(f"{self.prefix}: no layer before this one left values of "
                                     f"width {self.v_size} under {key!r}")
        layout = (self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim)
        ops.rope_blend_store(qkv, layout, tables, ctx.batch, cache, blend_from, self.blend, keep)
        attended = ctx.buffer("attended_v", tokens, self.num_heads * self.value_dim)
        ops.mixed_head_attention(qkv, layout, ctx.batch, cache, self.scale, self.window, self.mix,
                                 attended)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(attended, self.out_weight, self.out_b, out)
        return out


class LatentAttention(Mixer):
    """Attention over a cached low-rank latent.

    Per token: q = Wq h (heads x dim), or through a latent of its own when `q_rank` is set:
    q = Wuq (rmsnorm(Wdq h) * w_q); c = rmsnorm(Wdkv h) * w, `rank` numbers, which is what the
    cache keeps; per head k = Wuk c and v = Wuv c; weights = softmax(q.k * scale) over the keys
    j <= p (inside `window`, if one is given), with exp(sink_h) joining the denominator when
    the layer has a `sink`; an output projection.

    The keys and values are never built. Since q.(Wuk_h c) = (Wuk_h^T q).c, a head's query is
    taken into the latent space once per token and the head attends over the cached rows
    themselves, which serve as keys and as values (one shared head for all query heads);
    Wuv_h is applied to the head's weighted sum of rows afterwards.

    With `rot_dim` > 0 the down-projection has rot_dim more rows, which are not normed: one
    rotated key part that all heads share. A head's query is then [dim unrotated | rot_dim
    rotated] numbers, its score (q_u . k_u + q_r . k_r) * scale, and the cached row is
    [c | k_r after rotation]: the query that meets it is [Wuk_h^T q_u | q_r rotated], and Wuv_h
    reads the first `rank` numbers of the weighted sum of rows only. `position_encoding`
    gives the rotation of those rot_dim numbers (tables and pairing).

    `own_latent=False`: the layer has no Wdkv and reads the rows that another layer's call
    stored (its `LayerCall` names that call's cache layer with `writes_cache=False`).
    `cache_window`: what the cache layer keeps, where layers that read it look further back
    than this one (default: this layer's own window).
    """

    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, rank: int,
                 scale: float, eps: float, prefix: str, own_latent: bool = True,
                 names: dict | None = None, sink: bool = True, q_rank: int = 0, rot_dim: int = 0,
                 window: int = 0, cache_window: int | None = None,
                 position_encoding: PartSpec | None = None):
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.head_dim, self.value_dim, self.rank = head_dim, value_dim, rank
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.own_latent = bool(own_latent)
        self.has_sink = bool(sink)
        self.q_rank, self.rot_dim = int(q_rank), int(rot_dim)
        self.window = int(window)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.window and (self.cache_window and self.cache_window < self.window):
            raise ValueError(f"{prefix}: the cache keeps {self.cache_window} keys, fewer than the "
                             f"window of {self.window}")
        self.position = None
        if self.rot_dim:
            if position_encoding is None:
                raise ValueError(f"{prefix}: a rotated key part needs its position encoding")
            self.position = build_part("position_encoding", position_encoding)
            if getattr(self.position, "rotary_dim", 0) != self.rot_dim:
                raise ValueError(f"{prefix}: the encoding must rotate all {self.rot_dim} numbers of "
                                 f"the rotated part")
        self.q_head = head_dim + self.rot_dim          # a head's query as projected
        self.row = rank + self.rot_dim                 # a cached row
        self.q_size = num_heads * self.q_head
        self.names = {"q": "q", "q_down": "dq", "q_down_norm": "dq.norm", "q_up": "uq",
                      "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv",
                      "sink": "sink", "o": "o"}
        self.names.update(names or {})

    @property
    def plain(self) -> bool:
        """Neither a query latent nor a rotated part: the form whose kernels came first."""
        return not self.q_rank and not self.rot_dim

    def cache_need(self):
        return CacheNeed(1, self.row, self.cache_window, shared_values=True)

    def tensor_specs(self):
        p, n, h = self.prefix, self.names, self.hidden_size
        if self.q_rank:
            specs = [TensorSpec(p + n["q_down"], (self.q_rank, h)),
                     TensorSpec(p + n["q_down_norm"], (self.q_rank,), init="ones_normal", std=0.05),
                     TensorSpec(p + n["q_up"], (self.q_size, self.q_rank), std=0.05)]
        else:
            specs = [TensorSpec(p + n["q"], (self.q_size, h))]
        if self.own_latent:
            specs += [TensorSpec(p + n["down"], (self.row, h)),
                      TensorSpec(p + n["down_norm"], (self.rank,), init="ones_normal", std=0.05)]
        specs += [TensorSpec(p + n["up_k"], (self.num_heads * self.head_dim, self.rank),
                             std=0.02 if self.plain else 0.1),
                  TensorSpec(p + n["up_v"], (self.num_heads * self.value_dim, self.rank),
                             std=0.02 if self.plain else 0.1)]
        if self.has_sink:
            specs.append(TensorSpec(p + n["sink"], (self.num_heads,), std=1.0))
        specs.append(TensorSpec(p + n["o"], (h, self.num_heads * self.value_dim)))
        return specs + (self.position.tensor_specs() if self.position is not None else [])

    def load(self, tensors, setup):
        p, n = self.prefix, self.names
        mats = [setup.place(tensors[p + n["q_down" if self.q_rank else "q"]])]
        self.down_norm = self.q_norm = self.q_up = None
        if self.q_rank:
            self.q_norm = setup.place(tensors[p + n["q_down_norm"]])
            self.q_up = setup.place(tensors[p + n["q_up"]])
        if self.own_latent:
            mats.append(setup.place(tensors[p + n["down"]]))
            self.down_norm = setup.place(tensors[p + n["down_norm"]])
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()   # rows [q; dkv]
        up_k = setup.place(tensors[p + n["up_k"]]).view(self.num_heads, self.head_dim, self.rank)
        up_v = (setup.place(tensors[p + n["up_v"]]).view(self.num_heads, self.value_dim, self.rank)
                .transpose(1, 2))
        # both per head and input-major, [heads, in, out]: the key up-projection as stored is the
        # map that takes a query to the latent (its transpose); the value up-projection is turned
        if self.rot_dim:
            # the rotated part of a query passes into the place behind the latent unchanged,
            # and the value up-projection does not read the rotated part of a row
            absorb = torch.zeros((self.num_heads, self.q_head, self.row), dtype=up_k.dtype,
                                 device=up_k.device)
            absorb[:, :self.head_dim, :self.rank] = up_k
            index = torch.arange(self.rot_dim, device=up_k.device)
            absorb[:, self.head_dim + index, self.rank + index] = 1.0
            widened = torch.zeros((self.num_heads, self.row, self.value_dim), dtype=up_v.dtype,
                                  device=up_v.device)
            widened[:, :self.rank] = up_v
            self.absorb, self.up_v = absorb.contiguous(), widened.contiguous()
        else:
            self.absorb, self.up_v = up_k.contiguous(), up_v.contiguous()
        self.sink = (setup.place(tensors[p + n["sink"]]).float().contiguous()
                     if self.has_sink else None)
        self.out_weight = setup.place(tensors[p + n["o"]])
        if self.position is not None:
            self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        if cache.write != self.own_latent:
            raise ValueError(f"{self.prefix}: a layer stores latent rows iff it makes its own")
        pre = ctx.buffer("latent_in", tokens, self.in_weight.shape[0], dtype="float32")
        ops.linear(x, self.in_weight, None, pre)
        if self.plain:
            if self.own_latent:
                ops.latent_norm_store(pre, self.q_size, self.rank, self.down_norm, self.eps,
                                      ctx.batch, cache)
            queries = pre
        else:
            tables = self.position.rotary_tables() if self.position is not None else None
            pairing = getattr(self.position, "pairing", "halves")
            narrow = ctx.buffer("latent_cq", tokens, self.q_rank) if self.q_rank else None
            # the query latent's norm, the key latent's norm, the rotation of the shared key
            # part and the store of [c | rotated part] into the pages
            ops.latent_prepare(pre, self.q_rank, self.q_norm, narrow,
                               self.q_rank if self.q_rank else self.q_size, self.rank,
                               self.down_norm, self.rot_dim, tables, pairing, self.eps, ctx.batch,
                               cache if self.own_latent else None)
            if self.q_rank:
                queries = ctx.buffer("latent_qfull", tokens, self.q_size)
                ops.linear(narrow, self.q_up, None, queries)
            else:
                queries = pre
        q = ctx.buffer("latent_q", tokens, self.num_heads * self.row)
        ops.head_linear(queries, 0, self.absorb, q)
        if self.rot_dim:
            ops.rope_rows(q, self.num_heads, self.row, self.rank, self.rot_dim, tables, pairing,
                          ctx.batch)
        gathered = ctx.buffer("latent_sum", tokens, self.num_heads * self.row)
        ops.paged_attention(q, self.num_heads, 1, self.row, ctx.batch, cache, self.scale,
                            self.window, gathered, sinks=self.sink)
        attended = ctx.buffer("attended_v", tokens, self.num_heads * self.value_dim)
        ops.head_linear(gathered, 0, self.up_v, attended)
        out = ctx.sublayer_out(tokens, self.hidden_size)
        ops.linear(attended, self.out_weight, None, out)
        return out


class SigmoidAttention(Mixer):
    """Grouped-query attention whose weights are sigmoids and are not normalised over the keys.

    Per token: q = Wq h + bq (heads x dim), k = Wk h + bk (kv_heads x dim); the values are the
    keys as projected (`values_from_keys`; before norm and rotation) or a projection of their
    own; with `qk_norm`, q and k of each head are divided by their root mean square and
    multiplied by a weight of `dim` numbers shared by the heads (plain weight), before the
    rotation; the position encoding on q and k. Key j is seen from position p iff j <= p and
    (p - j < window or j < keep_first): a sliding window beside first tokens that stay
    visible at their true positions (window 0: every key). The weight of a seen key is
    sigmoid(q.k * scale + b_h), b_h one learned number per query head; out_h = sum_j weight_j
    v_j; an output projection.
    """

    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, eps: float, prefix: str, window: int = 0, keep_first: int = 0,
                 qk_norm: bool = True, qk_bias: bool = True, values_from_keys: bool = True,
                 value_dim: int | None = None, names: dict | None = None, bias_suffix: str = ".b",
                 position_encoding: PartSpec | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim = head_dim
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        self.values_from_keys = bool(values_from_keys)
        if self.values_from_keys and self.value_dim != head_dim:
            raise ValueError("values that are the keys have the keys' size")
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.window, self.keep_first = int(window), int(keep_first) if window else 0
        self.qk_norm, self.qk_bias = bool(qk_norm), bool(qk_bias)
        self.position = (build_part("position_encoding", position_encoding)
                         if position_encoding is not None else None)
        self.q_size = num_heads * head_dim
        self.k_size = num_kv_heads * head_dim
        self.v_size = 0 if self.values_from_keys else num_kv_heads * self.value_dim
        self.names = {"q": "q", "k": "k", "v": "v", "q_norm": "q.norm", "k_norm": "k.norm",
                      "head_bias": "pb", "o": "o"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window, self.value_dim,
                         keep_first=self.keep_first)

    def _projections(self):
        return ("q", "k") if self.values_from_keys else ("q", "k", "v")

    def tensor_specs(self):
        p, n, b, h = self.prefix, self.names, self.bias_suffix, self.hidden_size
        rows = {"q": self.q_size, "k": self.k_size, "v": self.v_size}
        specs = []
        for key in self._projections():
            specs.append(TensorSpec(p + n[key], (rows[key], h), std=0.05))
            if self.qk_bias and key != "v":
                specs.append(TensorSpec(p + n[key] + b, (rows[key],), std=0.1))
        if self.qk_norm:
            specs += [TensorSpec(p + n["q_norm"], (self.head_dim,), init="ones_normal", std=0.1),
                      TensorSpec(p + n["k_norm"], (self.head_dim,), init="ones_normal", std=0.1)]
        specs += [TensorSpec(p + n["head_bias"], (self.num_heads,), std=0.5, mean=-2.0),
                  TensorSpec(p + n["o"], (h, self.num_heads * self.value_dim))]
        return specs + (self.position.tensor_specs() if self.position is not None else [])

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix
        mats = [setup.place(tensors[p + n[key]]) for key in self._projections()]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()
        self.in_bias = None
        if self.qk_bias:
            biases = [setup.place(tensors[p + n[key] + b]) for key in ("q", "k")]
            if self.v_size:
                biases.append(torch.zeros(self.v_size, dtype=biases[0].dtype, device=biases[0].device))
            self.in_bias = torch.cat([t.to(widest) for t in biases]).contiguous()
        # norms are float32 arithmetic: their weights are held so
        self.q_norm = self.k_norm = None
        if self.qk_norm:
            self.q_norm = setup.place(tensors[p + n["q_norm"]]).float().contiguous()
            self.k_norm = setup.place(tensors[p + n["k_norm"]]).float().contiguous()
        self.head_bias = setup.place(tensors[p + n["head_bias"]]).float().contiguous()
        self.out_weight = setup.place(tensors[p + n["o"]])
        if self.position is not None:
            self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        pre = ctx.buffer("attn_in", tokens, self.in_weight.shape[0], dtype="float32")
        ops.linear(x, self.in_weight, self.in_bias, pre)
        tables = self.position.rotary_tables() if self.position is not None else None
        pairing = getattr(self.position, "pairing", "halves")
        layout = (self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim)
        q = ctx.buffer("attn_q", tokens, self.q_size)
        # per-head norms, rotation, and the store of keys and values into the pages
        ops.qk_norm_rope_store(pre, layout, self.q_norm, self.k_norm, self.eps, tables, pairing,
                               ctx.batch, cache, q, self.values_from_keys)
        attended = ctx.buffer("attended_v", tokens, self.num_heads * self.value_dim)
        ops.sigmoid_attention(q, layout, ctx.batch, cache, self.scale, self.window,
                              self.keep_first, self.head_bias, attended)
        out = ctx.sublayer_out(tokens, self.hidden_size)
        ops.linear(attended, self.out_weight, None, out)
        return out


class MaskedAttention(Mixer):
    """Grouped-query softmax attention whose mask, cap, sink and number of maps are parameters.

    Per token: q = Wq h, k = Wk h and v = Wv h (heads x dim, kv_heads x dim, kv_heads x value_dim),
    each with a bias when `bias` names it ("q", "k", "v", "o"; a bias is `name + bias_suffix`); with
    `values_from_keys` there is no Wv and the values are the keys as projected, before norm and
    rotation. `qk_norm` "projection": q over all its heads' rows at once is divided by its root
    mean square and multiplied by a weight of that many numbers, and so is k (before the
    rotation). The position encoding turns q and k. `mask` = {"kind", "size", "keep_first"}: key j
    is seen from position p iff j <= p and, for "sliding", p - j < size or j < keep_first (first
    tokens that stay visible at their true positions); for "chunked", floor(p / size) = floor(j /
    size), chunks counted from position 0; for "full", nothing more. score = q . k * scale, then
    softcap * tanh(score / softcap) when `softcap` > 0; softmax over the seen keys, with exp(sink_h)
    in the denominator when `sink` (one learned number per query head, no key, no value).

    `maps` = 2 is differential attention (Ye et al., "Differential Transformer"): q holds heads x
    2 x dim rows and k kv_heads x 2 x dim, head by head as [map 1, map 2]; each map is rotated
    and attends on its own over the same values, and with lambda = exp(lq1 . lk1) - exp(lq2 .
    lk2) + diff (four learned vectors of `dim` numbers, one lambda for the layer) a head's output
    is (a1 - lambda a2) divided by its root mean square over value_dim, times 1 - diff.

    An output projection (with a bias when `bias` names "o") closes it.
    """

    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, eps: float, prefix: str, mask: dict | None = None,
                 value_dim: int | None = None, bias: tuple = (), values_from_keys: bool = False,
                 qk_norm: str | None = None, softcap: float = 0.0, sink: bool = False, maps: int = 1,
                 diff: float = 0.0, names: dict | None = None, bias_suffix: str = ".b",
                 position_encoding: PartSpec | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        if maps not in (1, 2):
            raise ValueError(f"{maps} maps per head are not built (1 or 2)")
        if qk_norm not in (None, "projection"):
            raise ValueError(f"qk_norm={qk_norm!r} is neither None nor 'projection'")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.maps = head_dim, int(maps)
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        self.values_from_keys = bool(values_from_keys)
        if self.values_from_keys and self.value_dim != self.maps * head_dim:
            raise ValueError("values that are the keys have the keys' size")
        mask = dict(mask or {"kind": "full"})
        self.mask_kind = mask.get("kind", "full")
        if self.mask_kind not in ("full", "sliding", "chunked"):
            raise ValueError(f"mask kind {self.mask_kind!r}")
        self.mask_size = int(mask.get("size", 0)) if self.mask_kind != "full" else 0
        self.keep_first = int(mask.get("keep_first", 0)) if self.mask_kind == "sliding" else 0
        if self.mask_kind != "full" and self.mask_size <= 0:
            raise ValueError("a sliding or chunked mask needs a positive size")
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.bias = tuple(bias)
        self.qk_norm, self.softcap, self.has_sink = qk_norm, float(softcap), bool(sink)
        self.diff = float(diff)
        self.position = (build_part("position_encoding", position_encoding)
                         if position_encoding is not None else None)
        self.q_size = num_heads * self.maps * head_dim
        self.k_size = num_kv_heads * self.maps * head_dim
        self.v_size = 0 if self.values_from_keys else num_kv_heads * self.value_dim
        self.names = {"q": "q", "k": "k", "v": "v", "q_norm": "q.norm", "k_norm": "k.norm",
                      "sink": "sink", "o": "o", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix
        self.lam = 0.0

    def cache_need(self):
        # a chunk never reaches further back than its size, so the pages behind that go back
        # to the pool as they do behind a window
        return CacheNeed(self.num_kv_heads, self.maps * self.head_dim, self.mask_size, self.value_dim,
                         keep_first=self.keep_first)

    def _projections(self):
        return ("q", "k") if self.values_from_keys else ("q", "k", "v")

    def tensor_specs(self):
        p, n, b, h = self.prefix, self.names, self.bias_suffix, self.hidden_size
        rows = {"q": self.q_size, "k": self.k_size, "v": self.v_size}
        specs = []
        for key in self._projections():
            specs.append(TensorSpec(p + n[key], (rows[key], h), std=0.05))
            if key in self.bias:
                specs.append(TensorSpec(p + n[key] + b, (rows[key],), std=0.1))
        if self.qk_norm:
            specs += [TensorSpec(p + n["q_norm"], (self.q_size,), init="ones_normal", std=0.1),
                      TensorSpec(p + n["k_norm"], (self.k_size,), init="ones_normal", std=0.1)]
        if self.has_sink:
            specs.append(TensorSpec(p + n["sink"], (self.num_heads,), std=1.0))
        if self.maps == 2:
            specs += [TensorSpec(p + n[key], (self.head_dim,), std=0.1)
                      for key in ("lq1", "lk1", "lq2", "lk2")]
        specs.append(TensorSpec(p + n["o"], (h, self.num_heads * self.value_dim)))
        if "o" in self.bias:
            specs.append(TensorSpec(p + n["o"] + b, (h,), std=0.1))
        return specs + (self.position.tensor_specs() if self.position is not None else [])

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix
        keys = self._projections()
        mats = [setup.place(tensors[p + n[key]]) for key in keys]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()
        self.in_bias = None
        if any(key in self.bias for key in keys):
            pieces = [setup.place(tensors[p + n[key] + b]).to(widest) if key in self.bias
                      else torch.zeros(mat.shape[0], dtype=widest, device=mat.device)
                      for key, mat in zip(keys, mats)]
            self.in_bias = torch.cat(pieces).contiguous()
        # norms, sinks and lambda are float32 arithmetic: they are held so
        self.q_norm = self.k_norm = self.sink = None
        if self.qk_norm:
            self.q_norm = setup.place(tensors[p + n["q_norm"]]).float().contiguous()
            self.k_norm = setup.place(tensors[p + n["k_norm"]]).float().contiguous()
        if self.has_sink:
            self.sink = setup.place(tensors[p + n["sink"]]).float().contiguous()
        if self.maps == 2:
            lq1, lk1, lq2, lk2 = (tensors[p + n[key]].float() for key in ("lq1", "lk1", "lq2", "lk2"))
            self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum())) + self.diff
        self.out_weight = setup.place(tensors[p + n["o"]])
        self.out_bias = setup.place(tensors[p + n["o"] + b]) if "o" in self.bias else None
        if self.position is not None:
            self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        pre = ctx.buffer("attn_in", tokens, self.in_weight.shape[0], dtype="float32")
        ops.linear(x, self.in_weight, self.in_bias, pre)
        tables = self.position.rotary_tables() if self.position is not None else None
        pairing = getattr(self.position, "pairing", "halves")
        layout = (self.num_heads, self.num_kv_heads, self.maps, self.head_dim, self.value_dim)
        q = ctx.buffer("attn_q", tokens, self.q_size)
        # the norms over the projections, the rotation, and the store of keys and values
        ops.masked_prepare(pre, layout, self.q_norm, self.k_norm, self.eps, tables, pairing,
                           ctx.batch, cache, q, self.values_from_keys)
        attended = ctx.buffer("attended_v", tokens, self.num_heads * self.value_dim)
        ops.masked_attention(q, layout, ctx.batch, cache, self.scale,
                             (self.mask_kind, self.mask_size, self.keep_first), attended,
                             softcap=self.softcap, sinks=self.sink, lam=self.lam, sub_eps=self.eps,
                             out_scale=1.0 - self.diff if self.maps == 2 else 1.0)
        out = ctx.sublayer_out(tokens, self.hidden_size)
        ops.linear(attended, self.out_weight, self.out_bias, out)
        return out


register_mixer("mixed_head_attention", MixedHeadAttention)
register_mixer("latent_attention", LatentAttention)
register_mixer("sigmoid_attention", SigmoidAttention)
register_mixer("masked_attention", MaskedAttention)
