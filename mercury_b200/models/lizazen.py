"""The Lizazen decoder described in parts.

A token's row of the embedding table plus a row of a hashed table of token pairs opens the
stream. Every layer is a block with an RMS norm (plain weight) before and behind each
sublayer. A layer's mixer is one of three kinds, chosen per layer by the configuration:
`attention` (grouped-query attention with biased q/k/o projections, values that are the
keys as projected, one RMS norm over all heads' rows of q and of k, a rotation of the
leading part of each head whose long wavelengths may be slowed down, scores under a tanh
cap, a sliding window and a softmax sink), `attention_2` (differential attention: two
softmax maps per head over the same values, a sliding window beside kept first tokens), or
`parallel` (softmax attention over chunks of positions, with biases, beside retention;
each output is normed over the model width and the two are averaged). A layer's
feed-forward is dense with a clamped sigmoid gate, a mixture of SiLU-gated experts whose
router score multiplies the expert's input, with a shared expert beside them, or absent.
A norm and an untied head close the stack. Rotations pair feature i with feature i +
dims/2. Tensor names: `embed`, `bigram`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`
(`l<i>.mix.left.*`, `l<i>.mix.right.*` in a parallel layer), `l<i>.mlp.gate|up|down` or
`l<i>.mlp.e<j>.gate|up|down` with `l<i>.mlp.router` and `l<i>.mlp.shared.gate|up|down`,
`final.norm`, `head`.
"""

from __future__ import annotations

from ..config.model_config import LizazenConfig, register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec

GATE_SLOPE = 1.702      # the dense feed-forward's gate is g * sigmoid(GATE_SLOPE * g)
JOIN_SCALES = (0.5, 0.5)  # a parallel layer's output is half the sum of its two normed sides


def _rotation(table: dict) -> PartSpec | None:
    rot = table.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if not dims:
        return None
    return PartSpec("rotary", {"head_dim": int(table["dim"]), "theta": float(rot["base"]),
                               "rotary_dim": dims, "table_precision": "float64",
                               "scaling": rot.get("scaling") or None})


def _attention(config: LizazenConfig, prefix: str, m: dict, kind: str, **extra) -> PartSpec:
    mask = {"kind": kind, "size": int(m["mask"]["size"])}
    if kind == "sliding":
        mask["keep_first"] = int(m["mask"].get("keep_first", 0))
    params = {"hidden_size": config.width, "num_heads": int(m["heads"]),
              "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
              "value_dim": int(m["vdim"]), "scale": float(m["scale"]), "eps": config.norm_eps,
              "prefix": prefix, "mask": mask, "position_encoding": _rotation(m)}
    params.update(extra)
    return PartSpec("masked_attention", params)


def _mixers(config: LizazenConfig, index: int, layer: dict) -> dict:
    """The block parameters that name a layer's mixer or mixers."""
    p = f"l{index}.mix."
    kind, m = layer["type"], layer["mixer"]
    if kind == "attention":
        return {"mixer": _attention(config, p, m, "sliding", bias=("q", "k", "o"),
                                    values_from_keys=True, qk_norm="projection",
                                    softcap=float(m.get("softcap") or 0.0), sink=True)}
    if kind == "attention_2":
        return {"mixer": _attention(config, p, m, "sliding", maps=2, diff=float(m["diff"]))}
    left, right = m["left"], m["right"]
    retention = PartSpec("retention", {
        "hidden_size": config.width, "heads": int(right["heads"]), "key_dim": int(right["dim"]),
        "value_dim": int(right["vdim"]), "decay": [float(v) for v in right["decay"]],
        "eps": config.norm_eps, "prefix": p + "right.", "position_encoding": _rotation(right)})
    return {"mixers": [_attention(config, p + "left.", left, "chunked", bias=("q", "k", "v", "o")),
                       retention],
            "mixer_join": {"size": config.width, "eps": config.norm_eps,
                           "weight_names": (p + "left.out", p + "right.out"),
                           "scales": JOIN_SCALES}}


def _feed_forward(config: LizazenConfig, index: int, mlp: dict) -> PartSpec:
    prefix = f"l{index}.mlp."
    if mlp["kind"] == "dense":
        return PartSpec("gated", {
            "hidden_size": config.width, "intermediate_size": int(mlp["ff"]), "prefix": prefix,
            "activation": "clamped_sigmoid", "limit": float(mlp["limit"]), "slope": GATE_SLOPE,
            "names": ("gate", "up", "down")})
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("gated", {
            "hidden_size": config.width, "intermediate_size": int(mlp["shared"]["ff"]),
            "prefix": prefix + "shared.", "activation": "silu", "names": ("gate", "up", "down"),
            "float_out": True, "out_name": "shared_out"})
    return PartSpec("routed_experts", {
        "hidden_size": config.width, "intermediate_size": int(mlp["expert"]["ff"]),
        "experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]),
        "route_scale": 1.0, "prefix": prefix, "correction": False, "weight_on": "input",
        "shared": shared})


def describe_lizazen(config: LizazenConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("rmsnorm", {"size": config.width, "eps": config.norm_eps,
                                    "weight_name": name})

    blocks, schedule = [], []
    cache_layers = 0
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        params = {"mixer_norm": norm(p + "norm1"), "mixer_post_norm": norm(p + "norm1b")}
        params.update(_mixers(config, index, layer))
        if layer["mlp"] is not None:
            params["feed_forward"] = _feed_forward(config, index, layer["mlp"])
            params["feed_forward_norm"] = norm(p + "norm2")
            params["feed_forward_post_norm"] = norm(p + "norm2b")
        blocks.append(PartSpec("sandwich_norm", params))
        if layer["type"] == "parallel":
            schedule.append(LayerCall(block=index, cache=(cache_layers, None)))
        else:
            schedule.append(LayerCall(block=index, cache=cache_layers))
        cache_layers += 1
    if config.bigram:
        buckets, mul_prev, mul_cur = config.bigram
        embedding = PartSpec("lookup_bigram", {
            "vocab_size": config.vocab, "hidden_size": config.width, "weight_name": "embed",
            "pair_name": "bigram", "buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur})
    else:
        embedding = PartSpec("lookup", {"vocab_size": config.vocab, "hidden_size": config.width,
                                        "weight_name": "embed"})
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=config.max_positions,
        embedding=embedding,
        blocks=blocks,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": config.vocab, "hidden_size": config.width,
                                 "weight_name": "head"}),
    )


register_architecture("Lizazen", LizazenConfig, describe_lizazen)
