"""A plain implementation of the Sisavik decoder: float64, whole sequences, no cache, no
state carried between calls, one function per mechanism. It shares no code with the package
and is what the engine is compared with.

Notation: T tokens at positions 0 .. T-1, x the residual stream [T, width], W the tensors by
name (linear weights [out, in]).

    rms(v)        = v / sqrt(mean(v^2) + eps)
    shortconv(x)  = x + sum_j w[:, j] * x shifted by (taps - 1 - j) tokens, zeros in front
    layer:          x <- x + rms(mixer(shortconv1(x))) * (1 + n1)
                    x <- x + rms(ff(shortconv2(x))) * (1 + n2)       (where the layer has an ff)
    ff(h)         = Wdown (gelu_tanh(Wgate h) * (Wup h))
    logits        = Whead (rms(x) * (1 + n_final))
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_convolution(x, w):
    """x [T, C], w [C, taps]: x_t + sum_j w[:, j] x_(t - taps + 1 + j)."""
    taps = w.shape[1]
    count = x.shape[0]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F), x])
    out = x.clone()
    for j in range(taps):
        out = out + padded[j:j + count] * w[:, j]
    return out


def rotate_pairs(v, positions, base, dims):
    """v [T, ..., D]: features (2i, 2i + 1), i < dims / 2, turned by positions * base^(-2i/dims)."""
    if not dims:
        return v
    i = torch.arange(dims // 2, dtype=F)
    angle = positions.to(F)[:, None] * base ** (-2.0 * i / dims)
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [dims // 2]
    c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible(count, window, keep_first=0):
    """[T, T] bool: key j seen from i iff j <= i and (i - j < window or j < keep_first);
    window 0 or None: every earlier key."""
    i = torch.arange(count)[:, None]
    j = torch.arange(count)[None, :]
    seen = j <= i
    if window:
        seen = seen & ((i - j < window) | (j < keep_first))
    return seen


def latent_rows(W, p, m, h, eps):
    """What a latent-attention layer caches: the normed latent and the rotated shared key part."""
    count = h.shape[0]
    rank = m["kv_rank"]
    down = h @ W[p + "dkv"].T
    c = rms(down[:, :rank], eps) * W[p + "dkv.norm"]
    rot = m.get("rot") or {}
    shared = rotate_pairs(down[:, rank:], torch.arange(count), rot.get("base", 1.0), rot.get("dims", 0))
    return c, shared


def latent_attention(W, p, m, h, eps, rows):
    count = h.shape[0]
    heads, dim, rot_dim, vdim = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, shared = rows
    q = (rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]) @ W[p + "uq"].T
    q = q.view(count, heads, dim + rot_dim)
    rot = m.get("rot") or {}
    q_plain = q[..., :dim]
    q_turned = rotate_pairs(q[..., dim:], torch.arange(count), rot.get("base", 1.0), rot.get("dims", 0))
    k = (c @ W[p + "uk"].T).view(count, heads, dim)
    v = (c @ W[p + "uv"].T).view(count, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k)
              + torch.einsum("ihd,jd->hij", q_turned, shared)) * m["scale"]
    seen = visible(count, (m.get("mask") or {}).get("size", 0))
    weights = torch.softmax(scores.masked_fill(~seen[None], -math.inf), dim=-1)
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(count, heads * vdim)
    return out @ W[p + "o"].T


def sigmoid_attention(W, p, m, h, eps):
    count = h.shape[0]
    heads, groups, dim = m["heads"], m["kv_heads"], m["dim"]
    positions = torch.arange(count)
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(count, heads, dim)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(count, groups, dim)
    v = k                                              # the values: the keys as projected
    rot = m.get("rot") or {}
    q = rotate_pairs(rms(q, eps) * W[p + "q.norm"], positions, rot.get("base", 1.0), rot.get("dims", 0))
    k = rotate_pairs(rms(k, eps) * W[p + "k.norm"], positions, rot.get("base", 1.0), rot.get("dims", 0))
    share = heads // groups
    out = torch.zeros(count, heads, dim, dtype=F)
    mask = m.get("mask") or {}
    seen = visible(count, mask.get("size", 0), mask.get("keep_first", 0)).to(F)
    for head in range(heads):
        g = head // share
        scores = q[:, head] @ k[:, g].T * m["scale"] + W[p + "pb"][head]
        out[:, head] = (torch.sigmoid(scores) * seen) @ v[:, g]
    return out.reshape(count, heads * dim) @ W[p + "o"].T


def generalized_delta_rule(W, p, m, h, eps, decay_scale=math.exp(-0.5), unit_eps=1e-6):
    count = h.shape[0]
    heads, dim = m["heads"], m["dim"]
    r = (h @ W[p + "r"].T).view(count, heads, dim)
    k = (h @ W[p + "k"].T).view(count, heads, dim)
    v = (h @ W[p + "v"].T).view(count, heads, dim)
    decay = torch.exp(-decay_scale * torch.sigmoid(
        torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).view(count, heads, dim)
    rate = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).view(count, heads, dim)
    unit = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    state = torch.zeros(heads, dim, dim, dtype=F)           # [head, key channel, value channel]
    read = torch.zeros(count, heads, dim, dtype=F)
    for t in range(count):
        for head in range(heads):
            old = state[head]
            removed = torch.outer(rate[t, head] * unit[t, head], unit[t, head] @ old)
            state[head] = decay[t, head][:, None] * old - removed + torch.outer(k[t, head], v[t, head])
            read[t, head] = state[head].T @ r[t, head]
    read = rms(read, eps).reshape(count, heads * dim)
    return (read * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def feed_forward(W, p, h):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def forward(raw: dict, tensors: dict, tokens: list[int], layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence."""
    W = {name: t.to(F) for name, t in tensors.items()}
    eps = raw["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    cached: dict[int, tuple] = {}
    for index, layer in enumerate(raw["layers"]):
        p = f"l{index}."
        m = layer["mixer"]
        h = short_convolution(x, W[p + "canon1"])
        if layer["type"] == "latent_attention":
            source = m.get("kv_from")
            if source is None:
                cached[index] = latent_rows(W, p + "mix.", m, h, eps)
                source = index
            y = latent_attention(W, p + "mix.", m, h, eps, cached[source])
        elif layer["type"] == "parallel":
            y = (m["left_scale"] * sigmoid_attention(W, p + "mix.left.", m["left"], h, eps)
                 + m["right_scale"] * generalized_delta_rule(W, p + "mix.right.", m["right"], h, eps))
        else:
            raise ValueError(layer["type"])
        x = x + rms(y, eps) * (1.0 + W[p + "norm1"])
        if layer.get("mlp") is not None:
            h = short_convolution(x, W[p + "canon2"])
            x = x + rms(feed_forward(W, p + "mlp.", h), eps) * (1.0 + W[p + "norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * (1.0 + W["final.norm"])) @ W["head"].T
