"""The Sisavik decoder described in parts.

A token's row of the embedding table opens the stream. Every layer is a post-norm block:
each sublayer reads the stream plus a short causal convolution of it (per channel, the
stream's last rows kept per request) and its output passes an RMS norm (weight stored
around zero, applied as 1 + w) before it joins the stream. A layer's mixer is attention over
a cached low-rank latent with a query latent, a rotated key part shared by the heads and a
sliding window (a layer may read the rows an earlier layer caches instead of making its
own), or two mixers side by side under a scale each: grouped-query attention with sigmoid
weights, values that are the keys as projected, per-head query/key norms, a window and
kept first tokens, beside a generalized delta rule with a decay per key channel. The
feed-forward is gelu-gated and dense, or absent. The same kind of norm and an untied head
close the stack. Rotations pair neighbouring features. Tensor names: `embed`,
`l<i>.norm1|norm2|canon1|canon2`, `l<i>.mix.*` (`l<i>.mix.left.*` and `l<i>.mix.right.*` in
a parallel layer), `l<i>.mlp.gate|up|down`, `final.norm`, `head`.
"""

from __future__ import annotations

import math

from ..config.model_config import (SisavikConfig, register_architecture,
                                   sisavik_sizes_from_tensors)
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec

UNIT_EPS = 1e-6                      # under the root when the delta rule's key is made a unit vector
DECAY_SCALE = math.exp(-0.5)         # a channel's decay is exp(-DECAY_SCALE * sigmoid(.))


def _rotation(table: dict, size: int) -> PartSpec | None:
    rot = table.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if not dims:
        return None
    return PartSpec("rotary", {"head_dim": size, "theta": float(rot["base"]), "rotary_dim": dims,
                               "table_precision": "float64", "pairing": "interleaved"})


def _window(table: dict) -> tuple[int, int]:
    mask = table.get("mask") or {}
    size = int(mask.get("size", 0))
    return size, (int(mask.get("keep_first", 0)) if size else 0)


def _latent(config: SisavikConfig, index: int, m: dict, cache_window: int) -> PartSpec:
    rot_dim = int(m["rot_dim"])
    return PartSpec("latent_attention", {
        "hidden_size": config.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]),
        "value_dim": int(m["vdim"]), "rank": int(m["kv_rank"]), "scale": float(m["scale"]),
        "eps": config.norm_eps, "prefix": f"l{index}.mix.", "own_latent": m.get("kv_from") is None,
        "sink": False, "q_rank": int(m["q_rank"]), "rot_dim": rot_dim,
        "window": _window(m)[0], "cache_window": cache_window,
        "position_encoding": _rotation(m, rot_dim) if rot_dim else None})


def _left(config: SisavikConfig, index: int, m: dict) -> PartSpec:
    window, keep = _window(m)
    return PartSpec("sigmoid_attention", {
        "hidden_size": config.width, "num_heads": int(m["heads"]),
        "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]), "scale": float(m["scale"]),
        "eps": config.norm_eps, "prefix": f"l{index}.mix.left.", "window": window,
        "keep_first": keep, "qk_norm": True, "qk_bias": True, "values_from_keys": True,
        "position_encoding": _rotation(m, int(m["dim"]))})


def _right(config: SisavikConfig, index: int, m: dict, decay_rank: int) -> PartSpec:
    return PartSpec("generalized_delta_rule", {
        "hidden_size": config.width, "heads": int(m["heads"]), "key_dim": int(m["dim"]),
        "decay_rank": decay_rank, "eps": config.norm_eps, "prefix": f"l{index}.mix.right.",
        "decay_scale": DECAY_SCALE, "unit_eps": UNIT_EPS})


def describe_sisavik(config: SisavikConfig) -> ModelSpec:

    def norm(name):
        return PartSpec("rmsnorm_one_plus", {"size": config.width, "eps": config.norm_eps,
                                             "weight_name": name})

    def conv(name):
        return PartSpec("convolution", {"size": config.width, "taps": config.taps,
                                        "weight_name": name})

    # what a layer that makes a latent has to keep: the widest window of the layers that read
    # its rows (0, every key, if one of them has no window)
    keeps: dict[int, int] = {}
    for index, layer in enumerate(config.layers):
        if layer["type"] != "latent_attention":
            continue
        source = layer["mixer"].get("kv_from")
        source = index if source is None else int(source)
        window = _window(layer["mixer"])[0]
        if source not in keeps:
            keeps[source] = window
        elif keeps[source] and window:
            keeps[source] = max(keeps[source], window)
        else:
            keeps[source] = 0

    blocks, schedule = [], []
    cache_layers = 0
    cache_of: dict[int, int] = {}
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        m = layer["mixer"]
        params = {"hidden_size": config.width, "mixer_post_norm": norm(p + "norm1"),
                  "mixer_input": conv(p + "canon1")}
        if layer["type"] == "latent_attention":
            source = m.get("kv_from")
            source = index if source is None else int(source)
            params["mixers"] = [_latent(config, index, m, keeps[source])]
            if source == index:
                cache_of[index] = cache_layers
                cache_layers += 1
                call = LayerCall(block=index, cache=cache_of[index])
            else:
                call = LayerCall(block=index, cache=cache_of[source], writes_cache=False)
        else:
            rank = int(m["right"].get("decay_rank", 0))
            if rank <= 0:
                raise ValueError(f"layer {index}: the rows of mix.right.w1 are not known (a model "
                                 f"folder's tensors give them; a configuration made in code names "
                                 f"them as mixer.right.decay_rank)")
            params["mixers"] = [_left(config, index, m["left"]), _right(config, index, m["right"], rank)]
            params["mixer_scales"] = [float(m["left_scale"]), float(m["right_scale"])]
            call = LayerCall(block=index, cache=(cache_layers, None))
            cache_layers += 1
        if layer["mlp"] is not None:
            params["feed_forward"] = PartSpec("gated", {
                "hidden_size": config.width, "intermediate_size": int(layer["mlp"]["ff"]),
                "prefix": p + "mlp.", "activation": "gelu_tanh", "names": ("gate", "up", "down")})
            params["feed_forward_post_norm"] = norm(p + "norm2")
            params["feed_forward_input"] = conv(p + "canon2")
        blocks.append(PartSpec("post_norm", params))
        schedule.append(call)
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=config.max_positions,
        embedding=PartSpec("lookup", {"vocab_size": config.vocab, "hidden_size": config.width,
                                      "weight_name": "embed"}),
        blocks=blocks,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": config.vocab, "hidden_size": config.width,
                                 "weight_name": "head"}),
    )


register_architecture("Sisavik", SisavikConfig, describe_sisavik, sisavik_sizes_from_tensors)
