"""Token embedding and the output head.

Embedding: a row lookup without scaling (mercury/model/qwen2.py:100, :109), written into
the float32 residual stream. Head: hidden times a [vocab, hidden] matrix, no bias
(mercury/model/qwen2.py:128-130, :145-150); logits are float32. A head is tied to the
embedding by naming the embedding's checkpoint tensor as its own weight: both parts then
get the same buffer from `PartSetup.place_named`.

Both are registered kinds ("lookup", "linear"), so a model description chooses them like
any other part; an embedding that scales its rows or a head with a bias or a soft cap is
another registered kind, not a change to the generic model.
"""

from __future__ import annotations

import torch

from .base import Embedding, Head, StateNeed, TensorSpec, register_embedding, register_head


class TokenEmbedding(Embedding):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str, scale: float = 1.0):
        """`scale`: every row is multiplied by it on its way into the stream."""
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight_name = weight_name
        self.scale = float(scale)
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors, setup):
        self.table = setup.place_named(tensors, self.weight_name)

    def forward(self, token_ids, ctx):
        h = ctx.buffer("residual", token_ids.shape[0], self.hidden_size, dtype="float32")
        if self.scale != 1.0:
            ctx.ops.embed(token_ids, self.table, h, scale=self.scale)
        else:
            ctx.ops.embed(token_ids, self.table, h)
        return h


class PositionedEmbedding(TokenEmbedding):
    """Token row plus a learned vector per position (position counted from 0 in each
    sequence), neither scaled: stream[t] = table[token[t]] + positions[position[t]]."""

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str, position_name: str,
                 max_positions: int):
        super().__init__(vocab_size, hidden_size, weight_name)
        self.position_name = position_name
        self.max_positions = max_positions
        self.position_table = None

    def tensor_specs(self):
        return super().tensor_specs() + [
            TensorSpec(self.position_name, (self.max_positions, self.hidden_size))]

    def load(self, tensors, setup):
        super().load(tensors, setup)
        self.position_table = setup.place_named(tensors, self.position_name)

    def forward(self, token_ids, ctx):
        h = ctx.buffer("residual", token_ids.shape[0], self.hidden_size, dtype="float32")
        ctx.ops.embed(token_ids, self.table, h, positions=ctx.batch.positions,
                      position_table=self.position_table)
        return h


class BigramEmbedding(TokenEmbedding):
    """Token row plus a row of a hashed table of token pairs: stream[t] = table[token[t]] +
    pairs[(token[t-1] * mul_prev + token[t] * mul_cur) mod buckets], and for a sequence's
    first token the row behind the buckets (the table has buckets + 1 rows). The token in
    front of a step's first token is per-request state (`state_need()`): one int32 per slot,
    which the lookup kernel reads and brings up to date."""

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str, pair_name: str,
                 buckets: int, mul_prev: int, mul_cur: int):
        super().__init__(vocab_size, hidden_size, weight_name)
        self.pair_name = pair_name
        if int(buckets) <= 0 or int(buckets) >= 1 << 31:
            raise ValueError(f"buckets={buckets} must be positive and below 2^31")
        # (a x + b y) mod n = ((a mod n) x + (b mod n) y) mod n: the kernel gets multipliers below
        # the bucket count, so its 64-bit products are exact whatever the configuration names
        self.buckets = int(buckets)
        self.mul_prev, self.mul_cur = int(mul_prev) % self.buckets, int(mul_cur) % self.buckets
        self.pair_table = None

    def state_need(self):
        return StateNeed((1,), torch.int32)

    def tensor_specs(self):
        return super().tensor_specs() + [
            TensorSpec(self.pair_name, (self.buckets + 1, self.hidden_size))]

    def load(self, tensors, setup):
        super().load(tensors, setup)
        self.pair_table = setup.place_named(tensors, self.pair_name)

    def forward(self, token_ids, ctx, state=None):
        if state is None:
            raise ValueError("the bigram embedding needs its state: every sequence's last token")
        h = ctx.buffer("residual", token_ids.shape[0], self.hidden_size, dtype="float32")
        ctx.ops.embed_bigram(token_ids, self.table, self.pair_table, self.buckets, self.mul_prev,
                             self.mul_cur, state, ctx.batch, h)
        return h


class LinearHead(Head):
    capturable = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.weight_name = weight_name
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors, setup):
        self.weight = setup.place_named(tensors, self.weight_name)

    def forward(self, rows, ctx):
        logits = ctx.buffer("logits", rows.shape[0], self.vocab_size, dtype="float32")
        ctx.ops.linear(rows, self.weight, None, logits)
        return logits


class SoftCappedHead(LinearHead):
    """logits <- cap * tanh(logits / cap) behind the product (`cap` 0: none)."""

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str, cap: float):
        super().__init__(vocab_size, hidden_size, weight_name)
        self.cap = float(cap)

    def forward(self, rows, ctx):
        logits = super().forward(rows, ctx)
        if self.cap > 0.0:
            ctx.ops.softcap(logits, self.cap)
        return logits


register_embedding("lookup", TokenEmbedding)
register_embedding("lookup_learned_positions", PositionedEmbedding)
register_embedding("lookup_bigram", BigramEmbedding)
register_head("linear", LinearHead)
register_head("linear_softcap", SoftCappedHead)
