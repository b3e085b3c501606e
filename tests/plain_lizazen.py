"""A plain, slow Lizazen: whole sequences in float64, no cache, no batching, one function per
mechanism. It shares no code with the package; the tests compare the engine with it.

A model is (config dictionary as config.json holds it, {tensor name: tensor}). Notation:
x[t] is the stream's row of token t, H query heads, G key/value heads, d the query/key size
of a head, dv its value size.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def bigram_rows(tokens, table, buckets, mul_prev, mul_cur):
    """Row (previous * mul_prev + token * mul_cur) mod buckets; the row behind the buckets for
    a sequence's first token."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return table[torch.tensor(rows)]


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with `scaling` the long wavelengths are slowed down: a wavelength
    below original/high keeps f, one above original/low takes f/factor, between the two the
    blend (1 - s) f/factor + s f with s = (original/wavelength - low) / (high - low)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
        original = float(scaling["original"])
        out = []
        for v in f:
            wave = 2.0 * math.pi / v
            if wave < original / high:
                out.append(v)
            elif wave > original / low:
                out.append(v / factor)
            else:
                s = (original / wave - low) / (high - low)
                out.append((1.0 - s) * v / factor + s * v)
        f = out
    return torch.tensor(f, dtype=F)


def rotate(x, rot):
    """x: [T, heads, d]; the first rot["dims"] features of every head turn by position * f_i,
    feature i paired with feature i + dims/2."""
    dims = int(rot["dims"])
    if not dims:
        return x
    f = rotary_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    angle = torch.arange(x.shape[0], dtype=F)[:, None] * f[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def seen_sliding(T, size, keep_first=0):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def seen_chunked(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_attention(q, k, v, seen, scale, softcap=0.0, sink=None):
    """q: [T, H, d], k: [T, G, d], v: [T, G, dv], seen: [T, T] -> [T, H, dv]. `sink` [H]: one
    more term exp(sink_h) in the denominator, with no key and no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def capped_window_attention(h, m, w, p, eps):
    """The mixer of an `attention` layer."""
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    T = h.shape[0]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = k.reshape(T, G, d)                                       # the keys as projected
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, d)       # one norm over all heads' rows
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, d)
    q, k = rotate(q, m["rot"]), rotate(k, m["rot"])
    o = softmax_attention(q, k, v, seen_sliding(T, int(m["mask"]["size"])), float(m["scale"]),
                          float(m.get("softcap") or 0.0), w[p + "sink"])
    return o.reshape(T, -1) @ w[p + "o"].T + w[p + "o.b"]


def differential_attention(h, m, w, p, eps):
    """The mixer of an `attention_2` layer: two softmax maps per head over the same values."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    diff = float(m["diff"])
    q = (h @ w[p + "q"].T).reshape(T, H, 2, d)
    k = (h @ w[p + "k"].T).reshape(T, G, 2, d)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    seen = seen_sliding(T, int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0)))
    maps = []
    for which in (0, 1):
        qm, km = rotate(q[:, :, which], m["rot"]), rotate(k[:, :, which], m["rot"])
        maps.append(softmax_attention(qm, km, v, seen, float(m["scale"])))
    lam = (torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum())
           + diff)
    o = rms_unit(maps[0] - lam * maps[1], eps) * (1.0 - diff)
    return o.reshape(T, -1) @ w[p + "o"].T


def chunked_attention(h, m, w, p):
    """The left side of a `parallel` layer."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q, k = rotate(q, m["rot"]), rotate(k, m["rot"])
    o = softmax_attention(q, k, v, seen_chunked(T, int(m["mask"]["size"])), float(m["scale"]))
    return o.reshape(T, -1) @ w[p + "o"].T + w[p + "o.b"]


def retention(h, m, w, p, eps):
    """The right side of a `parallel` layer: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = rotate((h @ w[p + "q"].T).reshape(T, H, d), m["rot"])
    k = rotate((h @ w[p + "k"].T).reshape(T, H, d), m["rot"]) * d ** -0.5
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = float(m["decay"][head]) * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    out = rms_unit(out, eps).reshape(T, -1)
    gate = h @ w[p + "g"].T
    return (out * gate * torch.sigmoid(gate)) @ w[p + "o"].T


def side_by_side(h, m, w, p, eps):
    left = chunked_attention(h, m["left"], w, p + "left.")
    right = retention(h, m["right"], w, p + "right.", eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


def dense_feed_forward(h, mlp, w, p):
    limit = float(mlp["limit"])
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def silu_expert(h, w, p):
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_feed_forward(h, mlp, w, p):
    """Each token's `top` experts by sigmoid score; the score multiplies the expert's input."""
    top = int(mlp["router"]["top"])
    s = torch.sigmoid(h @ w[p + "router"].T)
    out = torch.zeros_like(h)
    chosen = torch.topk(s, top, dim=-1).indices
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += silu_expert((s[t, e] * h[t])[None], w, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + silu_expert(h, w, p + "shared.")
    return out


def forward(config, tensors, tokens, layer_streams=None):
    """Logits [T, vocab] of a whole sequence; with `layer_streams` (a list) the stream after
    every layer is appended to it."""
    w = {n: (t.to(F) if t.is_floating_point() else t) for n, t in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)]
    big = (config.get("embedding") or {}).get("bigram")
    if big:
        x = x + bigram_rows(tokens, w["bigram"], int(big["buckets"]), int(big["mul_prev"]),
                            int(big["mul_cur"]))
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = capped_window_attention(h, m, w, p + "mix.", eps)
        elif kind == "attention_2":
            y = differential_attention(h, m, w, p + "mix.", eps)
        elif kind == "parallel":
            y = side_by_side(h, m, w, p + "mix.", eps)
        else:
            raise ValueError(kind)
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            y = (dense_feed_forward(h, mlp, w, p + "mlp.") if mlp["kind"] == "dense"
                 else routed_feed_forward(h, mlp, w, p + "mlp."))
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        if layer_streams is not None:
            layer_streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
