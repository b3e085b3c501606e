"""Plain PyTorch twins of the CUDA kernels, one per kernel, with the same signatures.

They have two uses: each kernel's GPU test compares the kernel with its twin, and the CPU
tests build a runner on top of `TorchOps` to exercise the step function, the cache manager,
the scheduler and the replay program without a GPU. The product never imports this file:
its only kernel set is the CUDA one.

Arithmetic is float32 throughout (float64 with `exact=True`), whatever the storage dtype.
"""

from __future__ import annotations

import torch


class TorchOps:
    def __init__(self, exact: bool = False):
        self.acc = torch.float64 if exact else torch.float32

    # ---------------------------------------------------------------- embedding and norms

    def embed(self, token_ids, table, out, positions=None, position_table=None, scale=1.0):
        rows = table[token_ids.long()].to(self.acc) * scale
        if position_table is not None:
            rows = rows + position_table[positions[:out.shape[0]].long()].to(self.acc)
        out.copy_(rows.to(out.dtype))

    def rmsnorm_add(self, h, delta, weight, eps, next_weight, next_eps, out, delta2=None,
                    scale=1.0, scale2=1.0, tail=None):
        if tail is not None:
            self.stream_tail_store(h, tail[0], tail[1])
        d = delta.to(self.acc)
        if delta2 is not None or scale != 1.0:
            d = d * scale
            if delta2 is not None:
                d = d + delta2.to(self.acc) * scale2
        normed = d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.acc)
        h.add_(normed.to(h.dtype))
        if next_weight is not None:
            x = h.to(self.acc)
            out.copy_((x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + next_eps)
                       * next_weight.to(self.acc)).to(out.dtype))

    def patch_tokens(self, token_ids, token_from, sampled):
        late = token_from >= 0
        token_ids[late] = sampled[token_from[late].long()]

    def add_rmsnorm(self, h, delta, weight, eps, out, rows=None):
        if rows is None:
            if delta is not None:
                h.add_(delta.to(h.dtype))
            x = h.to(self.acc)
        else:
            index = rows.long()
            x = h[index].to(self.acc)
            if delta is not None:
                x = x + delta[index].to(self.acc)
        rstd = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_((x * rstd * weight.to(self.acc)).to(out.dtype))

    # ---------------------------------------------------------------- products

    # inputs may be an unevaluated norm (PendingNorm); the twin simply evaluates it

    def can_fuse_norm(self, rows, hidden, weight):
        return rows <= 16

    @staticmethod
    def _x(x):
        return x.materialize() if hasattr(x, "materialize") else x

    def linear_residual(self, x, weight, bias, h, ctx, name, then_norm=None):
        y = self._x(x).to(self.acc) @ weight.to(self.acc).T
        if bias is not None:
            y = y + bias.to(self.acc)
        h.add_(y.to(h.dtype))
        return None

    def linear(self, x, weight, bias, out):
        x = self._x(x)
        y = x.to(self.acc) @ weight.to(self.acc).T
        if bias is not None:
            y = y + bias.to(self.acc)
        out.copy_(y.to(out.dtype))

    def linear_swiglu(self, x, weight, out, ctx=None, ahead=None):
        x = self._x(x)
        gate_up = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        self.linear(x, weight, None, gate_up)
        self.swiglu(gate_up, out)

    def linear_gated(self, x, weight, out, ctx, activation, limit=0.0, slope=1.0):
        x = self._x(x)
        width = out.shape[-1]
        both = x.to(self.acc) @ weight.to(self.acc).T
        both = both.to(x.dtype).to(self.acc)          # the product lands in the activation type
        gate, up = both[:, :width], both[:, width:]
        if activation == "silu":
            act = gate * torch.sigmoid(gate)
        elif activation == "gelu_tanh":
            act = 0.5 * gate * (1.0 + torch.tanh(0.7978845608028654 * (gate + 0.044715 * gate ** 3)))
        elif activation == "clamped_sigmoid":
            gate = gate.clamp(max=limit)
            act = gate * torch.sigmoid(slope * gate)
            up = up.clamp(-limit, limit) + 1.0
        else:
            raise ValueError(activation)
        out.copy_((act * up).to(out.dtype))

    # ---------------------------------------------------------------- recurrences

    @staticmethod
    def _sequences(batch):
        starts, slots = batch.q_start.tolist(), batch.slots.tolist()
        for s in range(batch.num_seqs):
            if starts[s + 1] > starts[s]:
                yield starts[s], starts[s + 1], slots[s]

    def mingru_scan(self, pre, state, batch, out):
        width = out.shape[1]
        for begin, end, slot in self._sequences(batch):
            rows = pre[begin:end].to(self.acc)
            z = torch.sigmoid(rows[:, :width])
            u = rows[:, width:2 * width]
            cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            g = rows[:, 2 * width:]
            g = g * torch.sigmoid(g)
            s = state[slot].to(self.acc)
            for t in range(end - begin):
                s = (1.0 - z[t]) * s + z[t] * cand[t]
                out[begin + t] = (s * g[t]).to(out.dtype)
            state[slot] = s.to(state.dtype)

    def causal_conv(self, pre, offset, width, conv, conv_bias, state, batch, u):
        """u[t] = sum_k conv[:, k] * x[t - (taps - 1 - k)] + bias with x = pre[:, offset:
        offset + width]; inputs before the step come from rows 1.. of the state (row j: j
        tokens back), zeros before the sequence's start. The state is left as it was."""
        taps = conv.shape[1]
        for begin, end, slot in self._sequences(batch):
            x = pre[begin:end, offset:offset + width].to(self.acc)
            past = state[slot, 1:taps].to(self.acc).flip(0)          # oldest first
            padded = torch.cat([past, x])
            acc = torch.zeros_like(x)
            for k in range(taps):
                acc = acc + padded[k:k + x.shape[0]] * conv[:, k].to(self.acc)
            u[begin:end] = (acc + conv_bias.to(self.acc)).to(u.dtype)

    def block_gates(self, u, weight, bias, gates):
        """weight [kinds][blocks][in][out], bias [kinds][blocks][out]; gates [tokens][kinds *
        width] = sigmoid of the block-diagonal products."""
        kinds, blocks, size, _ = weight.shape
        ub = u.to(self.acc).view(u.shape[0], blocks, size)
        for kind in range(kinds):
            pre = torch.einsum("bio,tbi->tbo", weight[kind].to(self.acc), ub) + bias[kind].to(self.acc)
            gates[:, kind * blocks * size:(kind + 1) * blocks * size] = \
                torch.sigmoid(pre).reshape(u.shape[0], -1).to(gates.dtype)

    def gated_recurrence_scan(self, pre, u, gates, softplus_lam, decay_scale, state, batch, out):
        width = out.shape[1]
        taps = state.shape[1]
        for begin, end, slot in self._sequences(batch):
            y = pre[begin:end, :width].to(self.acc)
            y = 0.5 * y * (1.0 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
            uu = u[begin:end].to(self.acc)
            r, i = gates[begin:end, :width].to(self.acc), gates[begin:end, width:].to(self.acc)
            a = torch.exp(-decay_scale * r * softplus_lam.to(self.acc))
            b = torch.sqrt(1.0 - a * a) * i * uu
            s = state[slot, 0].to(self.acc)
            for t in range(end - begin):
                s = a[t] * s + b[t]
                out[begin + t] = (s * y[t]).to(out.dtype)
            state[slot, 0] = s.to(state.dtype)
            if taps > 1:
                x = pre[begin:end, width:2 * width].to(state.dtype)
                history = torch.cat([state[slot, 1:taps].flip(0), x])[-(taps - 1):]
                state[slot, 1:taps] = history.flip(0)

    def qkv_rope_store(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables,
                       batch, cache):
        x = self._x(x)
        self.linear(x, weight, bias, qkv)
        self.rope_cache_write(qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache)

    def swiglu(self, gate_up, out):
        width = out.shape[-1]
        gate = gate_up[:, :width].to(self.acc)
        up = gate_up[:, width:].to(self.acc)
        out.copy_((gate * torch.sigmoid(gate) * up).to(out.dtype))

    # ---------------------------------------------------------------- attention

    def rope_cache_write(self, qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache):
        tokens = qkv.shape[0]
        q_size, kv_size = num_heads * head_dim, num_kv_heads * head_dim
        live = batch.seq_of_token[:tokens] >= 0
        pos = batch.positions[:tokens].long()
        if tables is not None:
            cos_t, sin_t = tables
            half = cos_t.shape[1]
            cos = cos_t[pos].to(self.acc).unsqueeze(1)
            sin = sin_t[pos].to(self.acc).unsqueeze(1)
            for start, heads in ((0, num_heads), (q_size, num_kv_heads)):
                x = qkv[:, start:start + heads * head_dim].view(tokens, heads, head_dim)
                a = x[..., :half].to(self.acc)
                b = x[..., half:2 * half].to(self.acc)
                first = (a * cos - b * sin).to(qkv.dtype)
                second = (b * cos + a * sin).to(qkv.dtype)
                x[..., :half] = first
                x[..., half:2 * half] = second
        if cache is None or not cache.write:
            return
        seq = batch.seq_of_token[:tokens].long().clamp(min=0)
        page = cache.table[seq, pos // cache.page_size].long()
        offset = pos % cache.page_size
        k = qkv[:, q_size:q_size + kv_size].view(tokens, num_kv_heads, head_dim)
        v = qkv[:, q_size + kv_size:].view(tokens, num_kv_heads, head_dim)
        keep = live & (page >= 0)
        cache.k[page[keep], :, offset[keep], :] = k[keep].to(cache.k.dtype)
        cache.v[page[keep], :, offset[keep], :] = v[keep].to(cache.v.dtype)

    def qkv_attention(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables, batch,
                      cache, scale, window, out):
        self.qkv_rope_store(x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables, batch,
                            cache)
        self.paged_attention(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window, out)

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale,
                        window, out, sinks=None):
        group = num_heads // num_kv_heads
        q_start = batch.q_start.tolist()
        kv_lens = batch.kv_len.tolist()
        ps = cache.page_size
        for s in range(batch.num_seqs):
            begin, end = q_start[s], q_start[s + 1]
            q_len, kv_len = end - begin, kv_lens[s]
            if q_len == 0:
                continue
            first_pos = kv_len - q_len
            low = max(0, first_pos - window + 1) if window > 0 else 0
            low_page = low // ps
            pages = cache.table[s, low_page:-(-kv_len // ps)].long()
            keys = cache.k[pages].permute(1, 0, 2, 3).reshape(num_kv_heads, -1, head_dim)
            vals = cache.v[pages].permute(1, 0, 2, 3).reshape(num_kv_heads, -1, head_dim)
            key_pos = torch.arange(low_page * ps, low_page * ps + keys.shape[1], device=qkv.device)
            q = qkv[begin:end, :num_heads * head_dim].view(q_len, num_heads, head_dim).to(self.acc)
            q_pos = torch.arange(first_pos, kv_len, device=qkv.device)
            hidden = (key_pos[None, :] > q_pos[:, None]) | (key_pos[None, :] >= kv_len)
            if window > 0:
                hidden = hidden | (key_pos[None, :] <= q_pos[:, None] - window)
            keys = keys.to(self.acc).repeat_interleave(group, dim=0)
            vals = vals.to(self.acc).repeat_interleave(group, dim=0)
            scores = torch.einsum("qhd,hkd->hqk", q, keys) * scale
            scores = scores.masked_fill(hidden[None], float("-inf"))
            if sinks is None:
                weights = torch.softmax(scores, dim=-1)
            else:
                # a sink is one more term of the denominator: no key, no value, not scaled
                sink = sinks.to(self.acc)[:, None, None]
                big = torch.maximum(scores.max(-1, keepdim=True).values, sink)
                e = torch.exp(scores - big)
                weights = e / (e.sum(-1, keepdim=True) + torch.exp(sink - big))
            weights = torch.nan_to_num(weights)  # a hidden key's value may be non-finite
            vals = torch.where(hidden.all(0)[None, :, None], torch.zeros_like(vals), vals)
            o = torch.einsum("hqk,hkd->qhd", weights, vals)
            out[begin:end] = o.reshape(q_len, num_heads * head_dim).to(out.dtype)

    def rope_blend_store(self, qkv, layout, tables, batch, cache, blend_from, blend, keep):
        """Packed rows [q heads of `dim` | k heads of `dim` | v heads of `vdim`]: q and k are
        rotated over their leading features in place; v is copied to `keep` (if given), then
        blended v <- (1 - c) v + c blend_from (if given); k and v go into the pages."""
        heads, kv_heads, dim, vdim = layout
        tokens = qkv.shape[0]
        q_size, k_size = heads * dim, kv_heads * dim
        live = batch.seq_of_token[:tokens] >= 0
        pos = batch.positions[:tokens].long()
        if tables is not None:
            cos_t, sin_t = tables
            half = cos_t.shape[1]
            cos = cos_t[pos].to(self.acc).unsqueeze(1)
            sin = sin_t[pos].to(self.acc).unsqueeze(1)
            for start, count in ((0, heads), (q_size, kv_heads)):
                x = qkv[:, start:start + count * dim].view(tokens, count, dim)
                a = x[..., :half].to(self.acc)
                b = x[..., half:2 * half].to(self.acc)
                first = (a * cos - b * sin).to(qkv.dtype)
                second = (b * cos + a * sin).to(qkv.dtype)
                x[..., :half] = first
                x[..., half:2 * half] = second
        v = qkv[:, q_size + k_size:]
        if keep is not None:
            keep.copy_(v)
        if blend_from is not None:
            c = blend.to(self.acc)
            v.copy_(((1.0 - c) * v.to(self.acc) + c * blend_from.to(self.acc)).to(qkv.dtype))
        if cache is None or not cache.write:
            return
        seq = batch.seq_of_token[:tokens].long().clamp(min=0)
        page = cache.table[seq, pos // cache.page_size].long()
        offset = pos % cache.page_size
        keep_rows = live & (page >= 0)
        k = qkv[:, q_size:q_size + k_size].view(tokens, kv_heads, dim)
        cache.k[page[keep_rows], :, offset[keep_rows], :] = k[keep_rows].to(cache.k.dtype)
        cache.v[page[keep_rows], :, offset[keep_rows], :] = \
            v.view(tokens, kv_heads, vdim)[keep_rows].to(cache.v.dtype)

    def mixed_head_attention(self, qkv, layout, batch, cache, scale, window, mix, out):
        heads, kv_heads, dim, vdim = layout
        group = heads // kv_heads
        q_start = batch.q_start.tolist()
        kv_lens = batch.kv_len.tolist()
        ps = cache.page_size
        for s in range(batch.num_seqs):
            begin, end = q_start[s], q_start[s + 1]
            q_len, kv_len = end - begin, kv_lens[s]
            if q_len == 0:
                continue
            first_pos = kv_len - q_len
            low = max(0, first_pos - window + 1) if window > 0 else 0
            low_page = low // ps
            pages = cache.table[s, low_page:-(-kv_len // ps)].long()
            keys = cache.k[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, dim)
            vals = cache.v[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, vdim)
            key_pos = torch.arange(low_page * ps, low_page * ps + keys.shape[1], device=qkv.device)
            q = qkv[begin:end, :heads * dim].view(q_len, heads, dim).to(self.acc)
            q_pos = torch.arange(first_pos, kv_len, device=qkv.device)
            hidden = (key_pos[None, :] > q_pos[:, None]) | (key_pos[None, :] >= kv_len)
            if window > 0:
                hidden = hidden | (key_pos[None, :] <= q_pos[:, None] - window)
            keys = keys.to(self.acc).repeat_interleave(group, dim=0)
            vals = vals.to(self.acc).repeat_interleave(group, dim=0)
            scores = torch.einsum("qhd,hkd->hqk", q, keys) * scale
            scores = scores.masked_fill(hidden[None], float("-inf"))
            weights = torch.nan_to_num(torch.softmax(scores, dim=-1))
            if mix is not None:
                weights = torch.einsum("hg,gqk->hqk", mix.to(self.acc), weights)
            vals = torch.where(hidden.all(0)[None, :, None], torch.zeros_like(vals), vals)
            o = torch.einsum("hqk,hkd->qhd", weights, vals)
            out[begin:end] = o.reshape(q_len, heads * vdim).to(out.dtype)

    # ---------------------------------------------------------------- layer norm, scale, cap

    def scaled_add_norm(self, h, delta, scale, weight, eps, center, out, rows=None):
        """h += delta * scale (either may be None); then, if `weight` is given, out = norm(h)
        * weight, a layer norm (`center`) or an RMS norm. With `rows` only those rows are
        normalised and h is left as it was."""
        add = None
        if delta is not None:
            add = delta.to(self.acc) * (scale.to(self.acc) if scale is not None else 1.0)
        if rows is None:
            if add is not None:
                h.add_(add.to(h.dtype))
            x = h.to(self.acc)
        else:
            index = rows.long()
            x = h[index].to(self.acc)
            if add is not None:
                x = x + add[index]
        if weight is None:
            return
        if center:
            x = x - x.mean(-1, keepdim=True)
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_((x * weight.to(self.acc)).to(out.dtype))

    def softcap(self, logits, cap):
        logits.copy_((cap * torch.tanh(logits.to(self.acc) / cap)).to(logits.dtype))

    # ---------------------------------------------------------------- state-space and delta rule

    def conv_act(self, pre, offset, conv, bias, tail, batch, out, act):
        """out[t] = act(sum_k conv[:, k] * x[t - (taps - 1 - k)] + bias), x = pre[:, offset:
        offset + channels]; inputs before the step come from `tail` [slots, (taps - 1) *
        channels] (input j tokens back at (j - 1) * channels), which is left as it was."""
        channels, taps = conv.shape
        for begin, end, slot in self._sequences(batch):
            x = pre[begin:end, offset:offset + channels].to(self.acc)
            past = tail[slot].to(self.acc).view(taps - 1, channels).flip(0)       # oldest first
            padded = torch.cat([past, x])
            acc = torch.zeros_like(x)
            for k in range(taps):
                acc = acc + padded[k:k + x.shape[0]] * conv[:, k].to(self.acc)
            if bias is not None:
                acc = acc + bias.to(self.acc)
            if act == "silu":
                acc = acc * torch.sigmoid(acc)
            out[begin:end] = acc.to(out.dtype)

    def conv_act_update(self, pre, offset, conv, bias, tail, batch, out, act):
        self.conv_act(pre, offset, conv, bias, tail, batch, out, act)
        self.conv_tail_update(pre, offset, conv.shape[0], conv.shape[1], tail, batch)

    def conv_tail_update(self, pre, offset, channels, taps, tail, batch):
        if taps <= 1:
            return
        for begin, end, slot in self._sequences(batch):
            x = pre[begin:end, offset:offset + channels].to(tail.dtype)
            old = tail[slot].view(taps - 1, channels).flip(0)
            history = torch.cat([old, x])[-(taps - 1):]
            tail[slot] = history.flip(0).reshape(-1)

    def mamba2_scan(self, xbc, pre, dt_offset, dt_bias, neg_rate, skip, layout, cells, batch, y,
                    precise=False):
        heads, vdim, n, groups = layout
        inner, per = heads * vdim, heads // groups
        for begin, end, slot in self._sequences(batch):
            rows = xbc[begin:end].to(self.acc)
            x = rows[:, :inner].view(-1, heads, vdim)
            b = rows[:, inner:inner + groups * n].view(-1, groups, n).repeat_interleave(per, dim=1)
            c = rows[:, inner + groups * n:].view(-1, groups, n).repeat_interleave(per, dim=1)
            dt = torch.nn.functional.softplus(pre[begin:end, dt_offset:dt_offset + heads].to(self.acc)
                                              + dt_bias.to(self.acc))
            decay = torch.exp(neg_rate.to(self.acc) * dt)
            s = cells[slot].to(self.acc).view(heads, n, vdim)
            for t in range(end - begin):
                s = decay[t, :, None, None] * s + dt[t, :, None, None] * b[t, :, :, None] * x[t, :, None, :]
                out = torch.einsum("hnp,hn->hp", s, c[t]) + skip.to(self.acc)[:, None] * x[t]
                y[begin + t] = out.reshape(-1).to(y.dtype)
            cells[slot] = s.reshape(-1).to(cells.dtype)

    def delta_rule_scan(self, qkv, pre, beta_offset, decay_offset, dt_bias, neg_rate, layout,
                        unit_eps, cells, batch, o, precise=False):
        heads, key_heads, dim, vdim = layout
        qk, per = key_heads * dim, heads // key_heads
        for begin, end, slot in self._sequences(batch):
            rows = qkv[begin:end].to(self.acc)
            q = rows[:, :qk].view(-1, key_heads, dim)
            k = rows[:, qk:2 * qk].view(-1, key_heads, dim)
            v = rows[:, 2 * qk:].view(-1, heads, vdim)
            q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * dim ** -0.5
            k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
            q, k = q.repeat_interleave(per, dim=1), k.repeat_interleave(per, dim=1)
            beta = torch.sigmoid(pre[begin:end, beta_offset:beta_offset + heads].to(self.acc))
            g = torch.exp(neg_rate.to(self.acc) * torch.nn.functional.softplus(
                pre[begin:end, decay_offset:decay_offset + heads].to(self.acc) + dt_bias.to(self.acc)))
            s = cells[slot].to(self.acc).view(heads, dim, vdim)
            for t in range(end - begin):
                s = g[t, :, None, None] * s
                u = beta[t, :, None] * (v[t] - torch.einsum("hdp,hd->hp", s, k[t]))
                s = s + k[t, :, :, None] * u[:, None, :]
                o[begin + t] = torch.einsum("hdp,hd->hp", s, q[t]).reshape(-1).to(o.dtype)
            cells[slot] = s.reshape(-1).to(cells.dtype)

    def gated_group_norm(self, y, pre, gate_offset, weight, groups, eps, gate_first, out,
                         gate="silu"):
        """RMS norm of y in `groups` equal parts, times `weight` (as long as a row, or as a
        part and then shared by the parts), times silu(gate) (or sigmoid(gate)) before
        (`gate_first`) or behind the norm; gate = pre[:, gate_offset : gate_offset + width]."""
        tokens, width = y.shape
        kind = gate
        gate = pre[:, gate_offset:gate_offset + width].to(self.acc)
        gate = gate * torch.sigmoid(gate) if kind == "silu" else torch.sigmoid(gate)
        x = y.to(self.acc)
        if gate_first:
            x = x * gate
        x = x.view(tokens, groups, width // groups)
        x = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)).view(tokens, width)
        x = x * weight.to(self.acc).repeat(width // weight.numel())
        if not gate_first:
            x = x * gate
        out.copy_(x.to(out.dtype))

    # ---------------------------------------------------------------- stream convolution

    def stream_conv(self, h, weight, state, batch, out):
        """out_t = h_t + sum_j weight[:, j] * h_(t - taps + 1 + j) per channel, rows before the
        step from the ring `state[slot, position % (taps - 1)]`, zeros before position 0;
        without a weight, out = h. The ring is left as it was."""
        tokens = h.shape[0]
        if weight is None:
            out.copy_(h.to(out.dtype))
            return
        taps = weight.shape[1]
        ring = taps - 1
        starts, slots, lens = batch.q_start.tolist(), batch.slots.tolist(), batch.kv_len.tolist()
        w = weight.to(self.acc)
        for s in range(batch.num_seqs):
            begin, end = starts[s], starts[s + 1]
            n = end - begin
            if n == 0:
                continue
            first = lens[s] - n
            x = h[begin:end].to(self.acc)
            past = torch.zeros((ring, h.shape[1]), dtype=self.acc, device=h.device)
            for k in range(1, ring + 1):                      # k tokens before the step's first
                if first - k >= 0:
                    past[ring - k] = state[slots[s], (first - k) % ring].to(self.acc)
            padded = torch.cat([past, x])
            acc = x.clone()
            for j in range(taps):
                acc = acc + padded[j:j + n] * w[:, j]
            out[begin:end] = acc.to(out.dtype)

    def stream_tail_store(self, h, state, batch):
        """The rows of `h` at each sequence's last taps - 1 positions into its ring."""
        ring = state.shape[1]
        starts, slots, lens = batch.q_start.tolist(), batch.slots.tolist(), batch.kv_len.tolist()
        for s in range(batch.num_seqs):
            begin, end = starts[s], starts[s + 1]
            first = lens[s] - (end - begin)
            for t in range(max(begin, end - ring), end):
                state[slots[s], (first + t - begin) % ring] = h[t].to(state.dtype)

    # ---------------------------------------------------------------- rotations of pairs

    def _rotate(self, x, pos, tables, pairing):
        """x [tokens, ..., dims] rotated over all its last axis; tables (cos, sin) [positions,
        dims / 2]."""
        cos_t, sin_t = tables
        shape = [x.shape[0]] + [1] * (x.dim() - 2) + [cos_t.shape[1]]
        cos = cos_t[pos].to(self.acc).view(shape)
        sin = sin_t[pos].to(self.acc).view(shape)
        x = x.to(self.acc)
        if pairing == "interleaved":
            a, b = x[..., 0::2], x[..., 1::2]
            return torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
        half = x.shape[-1] // 2
        a, b = x[..., :half], x[..., half:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    @staticmethod
    def _page_slots(batch, cache, tokens):
        live = batch.seq_of_token[:tokens] >= 0
        pos = batch.positions[:tokens].long()
        seq = batch.seq_of_token[:tokens].long().clamp(min=0)
        page = cache.table[seq, pos // cache.page_size].long()
        return live & (page >= 0), page, pos % cache.page_size

    def latent_prepare(self, pre, q_rank, q_norm, narrow, kv_offset, rank, down_norm, rot_dim,
                       tables, pairing, eps, batch, cache):
        """narrow = rmsnorm(pre[:, :q_rank]) * q_norm (if q_rank); with a cache, the row [c |
        rotated part] of every token into its page: c = rmsnorm(pre[:, kv_offset : kv_offset +
        rank]) * down_norm, the part pre[:, kv_offset + rank : + rot_dim] rotated."""
        tokens = pre.shape[0]
        if q_rank:
            x = pre[:, :q_rank].to(self.acc)
            narrow.copy_((x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
                          * q_norm.to(self.acc)).to(narrow.dtype))
        if cache is None:
            return
        x = pre[:, kv_offset:kv_offset + rank].to(self.acc)
        c = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * down_norm.to(self.acc)
        pos = batch.positions[:tokens].long()
        if rot_dim:
            part = self._rotate(pre[:, kv_offset + rank:kv_offset + rank + rot_dim], pos, tables, pairing)
            c = torch.cat([c, part], dim=-1)
        keep, page, offset = self._page_slots(batch, cache, tokens)
        cache.k[page[keep], 0, offset[keep], :] = c[keep].to(cache.k.dtype)

    def rope_rows(self, q, heads, row, offset, rot_dim, tables, pairing, batch):
        """In place: q[t, h * row + offset : + rot_dim] rotated by the token's position."""
        tokens = q.shape[0]
        pos = batch.positions[:tokens].long()
        view = q.view(tokens, heads, row)[:, :, offset:offset + rot_dim]
        view.copy_(self._rotate(view, pos, tables, pairing).to(q.dtype))

    # ---------------------------------------------------------------- sigmoid attention

    def qk_norm_rope_store(self, pre, layout, q_norm, k_norm, eps, tables, pairing, batch, cache, q,
                           values_from_keys):
        heads, kv_heads, dim, vdim = layout
        tokens = pre.shape[0]
        pos = batch.positions[:tokens].long()
        qs, ks = heads * dim, kv_heads * dim
        qx = pre[:, :qs].to(self.acc).view(tokens, heads, dim)
        kx = pre[:, qs:qs + ks].to(self.acc).view(tokens, kv_heads, dim)
        vx = kx if values_from_keys else pre[:, qs + ks:].to(self.acc).view(tokens, kv_heads, vdim)
        if q_norm is not None:
            qx = qx * torch.rsqrt(qx.pow(2).mean(-1, keepdim=True) + eps) * q_norm.to(self.acc)
            kn = kx * torch.rsqrt(kx.pow(2).mean(-1, keepdim=True) + eps) * k_norm.to(self.acc)
        else:
            kn = kx
        if tables is not None:
            rot = 2 * tables[0].shape[1]
            qx = torch.cat([self._rotate(qx[..., :rot], pos, tables, pairing), qx[..., rot:]], dim=-1)
            kn = torch.cat([self._rotate(kn[..., :rot], pos, tables, pairing), kn[..., rot:]], dim=-1)
        q.copy_(qx.reshape(tokens, qs).to(q.dtype))
        keep, page, offset = self._page_slots(batch, cache, tokens)
        cache.k[page[keep], :, offset[keep], :] = kn[keep].to(cache.k.dtype)
        cache.v[page[keep], :, offset[keep], :] = vx[keep].to(cache.v.dtype)

    def sigmoid_attention(self, q, layout, batch, cache, scale, window, keep_first, head_bias, out):
        heads, kv_heads, dim, vdim = layout
        group = heads // kv_heads
        q_start, kv_lens = batch.q_start.tolist(), batch.kv_len.tolist()
        ps = cache.page_size
        for s in range(batch.num_seqs):
            begin, end = q_start[s], q_start[s + 1]
            q_len, kv_len = end - begin, kv_lens[s]
            if q_len == 0:
                continue
            first_pos = kv_len - q_len
            key_pos = torch.arange(kv_len, device=q.device)
            q_pos = torch.arange(first_pos, kv_len, device=q.device)
            seen = key_pos[None, :] <= q_pos[:, None]
            if window > 0:
                seen = seen & ((key_pos[None, :] > q_pos[:, None] - window)
                               | (key_pos[None, :] < keep_first))
            pages = cache.table[s, :-(-kv_len // ps)].long()
            wanted = seen.any(0)
            got = pages[key_pos // ps] >= 0
            if bool((wanted & ~got).any()):
                raise AssertionError("a visible key's page was given back")
            pages = pages.clamp(min=0)
            keys = cache.k[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, dim)[:, :kv_len]
            vals = cache.v[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, vdim)[:, :kv_len]
            keys = keys.to(self.acc).repeat_interleave(group, dim=0)
            vals = vals.to(self.acc).repeat_interleave(group, dim=0)
            vals = torch.where(wanted[None, :, None], vals, torch.zeros_like(vals))
            keys = torch.where(wanted[None, :, None], keys, torch.zeros_like(keys))
            qs = q[begin:end].view(q_len, heads, dim).to(self.acc)
            scores = torch.einsum("qhd,hkd->hqk", qs, keys) * scale + head_bias.to(self.acc)[:, None, None]
            weights = torch.sigmoid(scores) * seen[None]
            o = torch.einsum("hqk,hkd->qhd", weights, vals)
            out[begin:end] = o.reshape(q_len, heads * vdim).to(out.dtype)

    # ---------------------------------------------------------------- masked attention

    def embed_bigram(self, token_ids, table, pairs, buckets, mul_prev, mul_cur, state, batch, out):
        ids = token_ids.long()
        rows = table[ids].to(self.acc)
        starts, slots = batch.q_start.tolist(), batch.slots.tolist()
        positions = batch.positions.tolist()
        pair_rows = torch.zeros_like(rows)
        live = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
        for s in range(batch.num_seqs):
            begin, end = starts[s], starts[s + 1]
            if end <= begin:
                continue
            prev = int(state[slots[s], 0])
            for t in range(begin, end):
                tok = int(ids[t])
                row = buckets if positions[t] == 0 else (prev * mul_prev + tok * mul_cur) % buckets
                assert 0 <= mul_prev < buckets and 0 <= mul_cur < buckets
                pair_rows[t] = pairs[row].to(self.acc)
                live[t] = True
                prev = tok
            state[slots[s], 0] = prev
        out.copy_(((rows + pair_rows) * live[:, None]).to(out.dtype))

    def rmsnorm_join_add(self, h, x, y, wx, wy, a, b, weight, eps, next_weight, next_eps, out):
        def unit(v):
            return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)

        xv, yv = x.to(self.acc), y.to(self.acc)
        if wx is not None:
            xv = unit(xv) * wx.to(self.acc)
        if wy is not None:
            yv = unit(yv) * wy.to(self.acc)
        z = a * xv + b * yv
        h.add_((unit(z) * weight.to(self.acc)).to(h.dtype))
        if next_weight is not None:
            v = h.to(self.acc)
            out.copy_((v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + next_eps)
                       * next_weight.to(self.acc)).to(out.dtype))

    def masked_prepare(self, pre, layout, q_norm, k_norm, eps, tables, pairing, batch, cache, q,
                       values_from_keys):
        heads, kv_heads, maps, dim, vdim = layout
        tokens = pre.shape[0]
        pos = batch.positions[:tokens].long()
        qs, ks = heads * maps * dim, kv_heads * maps * dim
        qx = pre[:, :qs].to(self.acc)
        kx = pre[:, qs:qs + ks].to(self.acc)
        vx = (kx if values_from_keys else pre[:, qs + ks:].to(self.acc)).view(tokens, kv_heads, vdim)
        kn = kx
        if q_norm is not None:
            qx = qx * torch.rsqrt(qx.pow(2).mean(-1, keepdim=True) + eps) * q_norm.to(self.acc)
            kn = kx * torch.rsqrt(kx.pow(2).mean(-1, keepdim=True) + eps) * k_norm.to(self.acc)
        qx, kn = qx.view(tokens, heads * maps, dim), kn.view(tokens, kv_heads * maps, dim)
        if tables is not None:
            rot = 2 * tables[0].shape[1]
            qx = torch.cat([self._rotate(qx[..., :rot], pos, tables, pairing), qx[..., rot:]], dim=-1)
            kn = torch.cat([self._rotate(kn[..., :rot], pos, tables, pairing), kn[..., rot:]], dim=-1)
        q.copy_(qx.reshape(tokens, qs).to(q.dtype))
        keep, page, offset = self._page_slots(batch, cache, tokens)
        cache.k[page[keep], :, offset[keep], :] = kn.reshape(tokens, kv_heads, maps * dim)[keep].to(cache.k.dtype)
        cache.v[page[keep], :, offset[keep], :] = vx[keep].to(cache.v.dtype)

    def masked_attention(self, q, layout, batch, cache, scale, mask, out, softcap=0.0, sinks=None,
                         lam=0.0, sub_eps=0.0, out_scale=1.0):
        heads, kv_heads, maps, dim, vdim = layout
        kind, size, keep_first = mask
        group = heads // kv_heads
        q_start, kv_lens = batch.q_start.tolist(), batch.kv_len.tolist()
        ps = cache.page_size
        for s in range(batch.num_seqs):
            begin, end = q_start[s], q_start[s + 1]
            q_len, kv_len = end - begin, kv_lens[s]
            if q_len == 0:
                continue
            key_pos = torch.arange(kv_len, device=q.device)[None, :]
            q_pos = torch.arange(kv_len - q_len, kv_len, device=q.device)[:, None]
            seen = key_pos <= q_pos
            if kind == "sliding":
                seen = seen & ((q_pos - key_pos < size) | (key_pos < keep_first))
            elif kind == "chunked":
                seen = seen & (q_pos // size == key_pos // size)
            pages = cache.table[s, :-(-kv_len // ps)].long()
            wanted = seen.any(0)
            if bool((wanted & ~(pages[key_pos[0] // ps] >= 0)).any()):
                raise AssertionError("a visible key's page was given back")
            pages = pages.clamp(min=0)
            keys = cache.k[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, maps, dim)[:, :kv_len]
            vals = cache.v[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, vdim)[:, :kv_len]
            keys = torch.where(wanted[None, :, None, None], keys.to(self.acc), torch.zeros((), dtype=self.acc))
            vals = torch.where(wanted[None, :, None], vals.to(self.acc), torch.zeros((), dtype=self.acc))
            keys = keys.repeat_interleave(group, dim=0)
            vals = vals.repeat_interleave(group, dim=0)
            qs = q[begin:end].view(q_len, heads, maps, dim).to(self.acc)
            result = None
            for mp in range(maps):
                scores = torch.einsum("qhd,hkd->hqk", qs[:, :, mp], keys[:, :, mp]) * scale
                if softcap > 0:
                    scores = softcap * torch.tanh(scores / softcap)
                scores = scores.masked_fill(~seen[None], float("-inf"))
                top = scores.max(-1, keepdim=True).values
                if sinks is not None:
                    top = torch.maximum(top, sinks.to(self.acc)[:, None, None])
                e = torch.exp(scores - top)
                den = e.sum(-1, keepdim=True)
                if sinks is not None:
                    den = den + torch.exp(sinks.to(self.acc)[:, None, None] - top)
                a = torch.einsum("hqk,hkd->qhd", e / den, vals)
                result = a if mp == 0 else result - lam * a
            if maps == 2:
                result = result * torch.rsqrt(result.pow(2).mean(-1, keepdim=True) + sub_eps) * out_scale
            out[begin:end] = result.reshape(q_len, heads * vdim).to(out.dtype)

    def retention_scan(self, pre, offsets, decay, key_scale, layout, tables, pairing, cells, batch, o):
        heads, dim, vdim = layout
        at_q, at_k, at_v = offsets
        for begin, end, slot in self._sequences(batch):
            count = end - begin
            pos = batch.positions[begin:end].long()
            qx = pre[begin:end, at_q:at_q + heads * dim].to(self.acc).view(count, heads, dim)
            kx = pre[begin:end, at_k:at_k + heads * dim].to(self.acc).view(count, heads, dim)
            vx = pre[begin:end, at_v:at_v + heads * vdim].to(self.acc).view(count, heads, vdim)
            if tables is not None:
                rot = 2 * tables[0].shape[1]
                qx = torch.cat([self._rotate(qx[..., :rot], pos, tables, pairing), qx[..., rot:]], dim=-1)
                kx = torch.cat([self._rotate(kx[..., :rot], pos, tables, pairing), kx[..., rot:]], dim=-1)
            kx = kx * key_scale
            # the matrices lie column by column: [head][vdim][dim]
            s = cells[slot].view(heads, vdim, dim).to(self.acc).clone()
            g = decay.to(self.acc)[:, None, None]
            for t in range(count):
                s = g * s + vx[t][:, :, None] * kx[t][:, None, :]
                o[begin + t] = torch.einsum("hpd,hd->hp", s, qx[t]).reshape(-1).to(o.dtype)
            cells[slot] = s.reshape(-1).to(cells.dtype)

    # ---------------------------------------------------------------- generalized delta rule

    def tanh_slice(self, pre, offset, count, out):
        out.copy_(torch.tanh(pre[:, offset:offset + count].to(self.acc)).to(out.dtype))

    def general_delta_scan(self, pre, offsets, decay, decay_scale, layout, unit_eps, cells, batch, o,
                           precise=False):
        """Per head: S <- diag(w) S - (a * u)(u^T S) + k v^T, o = S^T r with w = exp(-decay_scale
        * sigmoid(decay)), a = sigmoid(pre[a]), u = k / sqrt(sum k^2 + unit_eps)."""
        heads, dim, vdim = layout
        at_r, at_k, at_v, at_a = offsets
        keys = heads * dim
        for begin, end, slot in self._sequences(batch):
            rows = pre[begin:end].to(self.acc)
            r = rows[:, at_r:at_r + keys].view(-1, heads, dim)
            k = rows[:, at_k:at_k + keys].view(-1, heads, dim)
            v = rows[:, at_v:at_v + heads * vdim].view(-1, heads, vdim)
            a = torch.sigmoid(rows[:, at_a:at_a + keys]).view(-1, heads, dim)
            w = torch.exp(-decay_scale * torch.sigmoid(decay[begin:end].to(self.acc))).view(-1, heads, dim)
            u = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
            s = cells[slot].to(self.acc).view(heads, dim, vdim)
            for t in range(end - begin):
                us = torch.einsum("hd,hdp->hp", u[t], s)
                s = (w[t, :, :, None] * s - (a[t] * u[t])[:, :, None] * us[:, None, :]
                     + k[t, :, :, None] * v[t, :, None, :])
                o[begin + t] = torch.einsum("hdp,hd->hp", s, r[t]).reshape(-1).to(o.dtype)
            cells[slot] = s.reshape(-1).to(cells.dtype)

    # ---------------------------------------------------------------- latent attention

    def latent_norm_store(self, pre, offset, rank, weight, eps, batch, cache):
        """c = rmsnorm(pre[:, offset : offset + rank]) * weight into the pages (one shared
        head of size `rank`)."""
        tokens = pre.shape[0]
        x = pre[:, offset:offset + rank].to(self.acc)
        c = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.acc)
        live = batch.seq_of_token[:tokens] >= 0
        pos = batch.positions[:tokens].long()
        seq = batch.seq_of_token[:tokens].long().clamp(min=0)
        page = cache.table[seq, pos // cache.page_size].long()
        keep = live & (page >= 0)
        cache.k[page[keep], 0, (pos % cache.page_size)[keep], :] = c[keep].to(cache.k.dtype)

    def head_linear(self, x, offset, weight, out):
        """out[t, h] = weight[h]^T x[t, h] with weight [heads, in, out] (input-major) and x's
        heads side by side from column `offset`."""
        heads, cols, _outs = weight.shape
        xs = x[:, offset:offset + heads * cols].to(self.acc).reshape(-1, heads, cols)
        out.copy_(torch.einsum("hio,thi->tho", weight.to(self.acc), xs).reshape(out.shape).to(out.dtype))

    # ---------------------------------------------------------------- routed experts

    def route_experts(self, x, router, correction, group_count, group_keep, route_scale, chosen,
                      weights):
        tokens, top = chosen.shape
        experts = router.shape[0]
        s = torch.sigmoid(self._x(x).to(self.acc) @ router.to(self.acc).T)
        choice = s + correction.to(self.acc)
        size = experts // group_count
        grouped = choice.view(tokens, group_count, size)
        score = grouped.topk(min(2, size), -1).values.sum(-1)
        kept = score.topk(group_keep, -1).indices
        allowed = torch.zeros(tokens, group_count, dtype=torch.bool, device=x.device)
        allowed.scatter_(1, kept, True)
        allowed = allowed[:, :, None].expand(-1, -1, size).reshape(tokens, experts)
        index = choice.masked_fill(~allowed, float("-inf")).topk(top, -1).indices
        chosen.copy_(index.to(chosen.dtype))
        weights.copy_((s.gather(1, index) * route_scale).to(weights.dtype))

    def expert_feed_forward(self, x, chosen, weights, gate_up, down, out, ctx=None,
                            weight_on="output"):
        """out[t] = sum_j weights[t, j] * down[e] (silu(gate[e] x[t]) * (up[e] x[t])), e =
        chosen[t, j]; gate_up [experts, 2 ff, hidden] (gate rows first), down [experts,
        hidden, ff]."""
        x = self._x(x)
        ff = down.shape[2]
        total = torch.zeros(out.shape, dtype=self.acc, device=x.device)
        for e in range(gate_up.shape[0]):
            hit = (chosen == e)
            rows = hit.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            both = (x[rows].to(self.acc) @ gate_up[e].to(self.acc).T)
            w = (weights[rows].to(self.acc) * hit[rows]).sum(-1, keepdim=True)
            if weight_on == "input":      # the weight on what the expert reads (no biases)
                both = both * w
            act = (both[:, :ff] * torch.sigmoid(both[:, :ff]) * both[:, ff:]).to(x.dtype).to(self.acc)
            y = act @ down[e].to(self.acc).T
            total[rows] += y if weight_on == "input" else w * y
        out.copy_(total.to(out.dtype))

    # ---------------------------------------------------------------- sampling

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(out.dtype))

    def sample(self, logits, temperature, top_p, u, out):
        """Row by row: greedy where temperature <= 0 (lowest index on ties); otherwise
        softmax(logits / max(T, 1e-5)), keep the tokens whose strictly-more-probable
        predecessors hold at most top_p, renormalise, and take the first index whose
        cumulative probability exceeds u."""
        for row in range(logits.shape[0]):
            t = float(temperature[row])
            if t <= 0.0:
                out[row] = int(torch.argmax(logits[row]))
                continue
            probs = torch.softmax(logits[row].double() / max(t, 1e-5), dim=-1)
            p = float(top_p[row])
            if p < 1.0:
                ordered, index = probs.sort(descending=True)
                before = ordered.cumsum(-1) - ordered
                # ties are kept or dropped together: mass of strictly larger values
                first_of_value = torch.searchsorted(-ordered, -ordered, right=False)
                before = before[first_of_value]
                probs = torch.zeros_like(probs).scatter_(0, index, ordered.masked_fill(before > p, 0.0))
            cdf = probs.cumsum(-1)
            target = float(u[row]) * float(cdf[-1])
            choice = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype), right=True))
            out[row] = min(choice, logits.shape[1] - 1)
