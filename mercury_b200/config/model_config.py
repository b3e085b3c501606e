"""Typed architecture configurations, read from the architecture's own config.json keys.

Every size and constant of a model comes from here; no part of the engine carries one.
`Qwen2Config` holds the field set of mercury/config.py:22-37 (`ModelConfig`) with the same
defaults for absent keys (mercury/config.py:56-70), plus the keys the reference silently
ignores and this engine either honours (the sliding window) or checks (`hidden_act`,
`rope_scaling`, `attention_bias`).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Callable


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the offending key named."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""

    architecture: str

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:
        """The config.json dictionary that `from_dict` reads back to an equal object."""
        raise NotImplementedError


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    hidden_act: str = "silu"

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen2Config":
        def need(key: str) -> Any:
            if key not in raw:
                raise ConfigError(f"config.json has no {key!r}, which Qwen2 needs")
            return raw[key]

        arch = (raw.get("architectures") or ["Qwen2ForCausalLM"])[0]
        heads = int(need("num_attention_heads"))
        hidden = int(need("hidden_size"))
        layers = int(need("num_hidden_layers"))
        kv_heads = int(raw.get("num_key_value_heads", heads))
        head_dim = int(raw.get("head_dim") or hidden // heads)
        eos = raw.get("eos_token_id", [])
        if eos is None:
            eos = []
        if isinstance(eos, int):
            eos = [eos]

        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r}: the Qwen2 feed-forward here is SiLU-gated only")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError("rope_scaling is set; scaled rotary embeddings are not built")
        if raw.get("attention_bias", True) is False:
            raise ConfigError("attention_bias=false: Qwen2 carries a bias on q, k and v")
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads={heads} is not a multiple of num_key_value_heads={kv_heads}"
            )
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim={head_dim} must be even for rotary embeddings")

        use_window = bool(raw.get("use_sliding_window", False))
        window = int(raw.get("sliding_window") or 0)
        if use_window and window <= 0:
            raise ConfigError("use_sliding_window is true but sliding_window is not positive")
        return cls(
            architecture=arch,
            hidden_size=hidden,
            intermediate_size=int(need("intermediate_size")),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=int(need("vocab_size")),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            rope_theta=float(raw.get("rope_theta", 10000.0)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            eos_token_ids=tuple(int(t) for t in eos),
            bos_token_id=raw.get("bos_token_id"),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=int(raw.get("max_window_layers", layers)),
            hidden_act=act,
        )

    def layer_window(self, layer: int) -> int:
        """Window of one layer in tokens, 0 for full attention: with `use_sliding_window`
        the layers from `max_window_layers` on see only the last `sliding_window` keys."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out


# --------------------------------------------------------------------------- Fegenex

_FEGENEX_MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "mingru": ("width",),
    "rglru": ("width", "blocks", "conv"),
}


@dataclass(frozen=True)
class FegenexConfig(ModelConfig):
    """A Fegenex decoder: a list of layers, each with one of three mixers (attention whose
    heads' weights are mixed, a minGRU, a real-gated linear recurrent unit behind a short
    convolution) and an optional gated feed-forward. config.json keys: `architecture`,
    `width`, `vocab`, `max_positions`, `norm.eps`, and `layers`, a list of
    `{"type", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}`. Every size and
    constant of a layer is in its own entry, so layers may differ in all of them."""

    width: int
    vocab: int
    max_positions: int
    norm_eps: float
    layers: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "FegenexConfig":
        def need(table: dict, key: str, where: str) -> Any:
            if key not in table:
                raise ConfigError(f"config.json has no {key!r} in {where}, which Fegenex needs")
            return table[key]

        layers = []
        for index, layer in enumerate(need(raw, "layers", "the model")):
            where = f"layer {index}"
            kind = need(layer, "type", where)
            if kind not in _FEGENEX_MIXER_KEYS:
                raise ConfigError(f"{where}: mixer type {kind!r} is not one of "
                                  f"{', '.join(sorted(_FEGENEX_MIXER_KEYS))}")
            mixer = dict(need(layer, "mixer", where))
            for key in _FEGENEX_MIXER_KEYS[kind]:
                need(mixer, key, f"{where}'s mixer")
            if kind == "attention":
                heads, kv_heads = int(mixer["heads"]), int(mixer["kv_heads"])
                if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
                    raise ConfigError(f"{where}: {heads} query heads do not divide into "
                                      f"{kv_heads} key/value heads")
                rot = mixer.get("rot") or {}
                dims = int(rot.get("dims", 0))
                if dims % 2 or dims > int(mixer["dim"]):
                    raise ConfigError(f"{where}: rot.dims={dims} must be even and at most "
                                      f"dim={mixer['dim']}")
                if dims and "base" not in rot:
                    raise ConfigError(f"{where}: rot.dims is set but rot.base is missing")
            if kind == "rglru":
                if int(mixer["width"]) % int(mixer["blocks"]):
                    raise ConfigError(f"{where}: width {mixer['width']} does not divide into "
                                      f"{mixer['blocks']} blocks")
                if int(mixer["conv"]) < 1:
                    raise ConfigError(f"{where}: conv={mixer['conv']} taps")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}: feed-forward kind {mlp.get('kind')!r} is not built")
                need(mlp, "ff", f"{where}'s mlp")
            layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
        if not layers:
            raise ConfigError("config.json lists no layers")
        norm = need(raw, "norm", "the model")
        return cls(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Fegenex"])[0]),
            width=int(need(raw, "width", "the model")),
            vocab=int(need(raw, "vocab", "the model")),
            max_positions=int(need(raw, "max_positions", "the model")),
            norm_eps=float(need(norm, "eps", "norm")),
            layers=tuple(layers),
        )

    def to_dict(self) -> dict:
        return {
            "architecture": self.architecture,
            "width": self.width,
            "vocab": self.vocab,
            "max_positions": self.max_positions,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l["type"], "mixer": dict(l["mixer"]),
                        "mlp": dict(l["mlp"]) if l["mlp"] is not None else None}
                       for l in self.layers],
        }


# --------------------------------------------------------------------------- Kinelix

_KINELIX_MIXER_KEYS = {
    "mamba2": ("heads", "vdim", "state", "groups", "norm_groups", "conv"),
    "delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
    "latent_attention": ("heads", "dim", "vdim", "kv_rank", "scale"),
}


@dataclass(frozen=True)
class KinelixConfig(ModelConfig):
    """A Kinelix decoder: pre-norm layers (layer norms with a weight and no bias, a learned
    scale per feature on every sublayer's output), each with one of three mixers (a Mamba-2
    state-space layer, a gated delta rule, attention over a cached low-rank latent with a
    softmax sink and no positions) and a dense or routed feed-forward or none. config.json
    keys: `architecture`, `width`, `vocab`, `embedding.scale`, `norm.eps`, `logit_softcap`
    and `layers`, a list of `{"type", "mixer": {...}, "mlp": {"kind": "dense", "ff"} |
    {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "groups":
    {"count", "keep"}}} | null}`. A latent-attention layer with `kv_from: j` has no
    down-projection of its own and reads the latent rows that layer j caches. The design has
    no positions, so nothing bounds a sequence's length but `max_positions` (not a key of
    the design; absent, `DEFAULT_POSITIONS`)."""

    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    max_positions: int = 1 << 20
    layers: tuple = ()

    DEFAULT_POSITIONS = 1 << 20

    @classmethod
    def from_dict(cls, raw: dict) -> "KinelixConfig":
        def need(table: dict, key: str, where: str) -> Any:
            if not isinstance(table, dict) or key not in table:
                raise ConfigError(f"config.json has no {key!r} in {where}, which Kinelix needs")
            return table[key]

        def positive(table: dict, key: str, where: str) -> int:
            value = int(need(table, key, where))
            if value <= 0:
                raise ConfigError(f"{where}: {key}={value} must be positive")
            return value

        layers = []
        listed = need(raw, "layers", "the model")
        for index, layer in enumerate(listed):
            where = f"layer {index}"
            kind = need(layer, "type", where)
            if kind not in _KINELIX_MIXER_KEYS:
                raise ConfigError(f"{where}: mixer type {kind!r} is not one of "
                                  f"{', '.join(sorted(_KINELIX_MIXER_KEYS))}")
            mixer = dict(need(layer, "mixer", where))
            for key in _KINELIX_MIXER_KEYS[kind]:
                if key != "scale":
                    positive(mixer, key, f"{where}'s mixer")
            if kind == "mamba2":
                if int(mixer["heads"]) % int(mixer["groups"]):
                    raise ConfigError(f"{where}: {mixer['heads']} heads do not divide into "
                                      f"{mixer['groups']} groups")
                if (int(mixer["heads"]) * int(mixer["vdim"])) % int(mixer["norm_groups"]):
                    raise ConfigError(f"{where}: heads * vdim does not divide into "
                                      f"{mixer['norm_groups']} norm groups")
            if kind == "delta" and int(mixer["heads"]) % int(mixer["kv_heads"]):
                raise ConfigError(f"{where}: {mixer['heads']} heads do not divide into "
                                  f"{mixer['kv_heads']} query/key heads")
            if kind == "latent_attention":
                float(need(mixer, "scale", f"{where}'s mixer"))
                source = mixer.get("kv_from")
                if source is not None:
                    source = int(source)
                    ok = (0 <= source < index and listed[source].get("type") == "latent_attention"
                          and listed[source].get("mixer", {}).get("kv_from") is None)
                    if not ok:
                        raise ConfigError(f"{where}: kv_from={source} must name an earlier "
                                          f"latent-attention layer with a latent of its own")
                    if int(listed[source]["mixer"].get("kv_rank", 0)) != int(mixer["kv_rank"]):
                        raise ConfigError(f"{where}: kv_rank differs from layer {source}'s, "
                                          f"whose latent it reads")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                what = need(mlp, "kind", f"{where}'s mlp")
                if what == "dense":
                    positive(mlp, "ff", f"{where}'s mlp")
                elif what == "moe":
                    positive(need(mlp, "expert", f"{where}'s mlp"), "ff", f"{where}'s expert")
                    router = dict(need(mlp, "router", f"{where}'s mlp"))
                    experts = positive(router, "experts", f"{where}'s router")
                    top = positive(router, "top", f"{where}'s router")
                    float(need(router, "scale", f"{where}'s router"))
                    groups = router.get("groups") or {"count": 1, "keep": 1}
                    count = positive(groups, "count", f"{where}'s router groups")
                    keep = positive(groups, "keep", f"{where}'s router groups")
                    if experts % count or keep > count or top > keep * (experts // count):
                        raise ConfigError(f"{where}: {experts} experts in {count} groups of which "
                                          f"{keep} are kept cannot give {top} experts a token")
                else:
                    raise ConfigError(f"{where}: feed-forward kind {what!r} is not built")
            layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
        if not layers:
            raise ConfigError("config.json lists no layers")
        return cls(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Kinelix"])[0]),
            width=positive(raw, "width", "the model"),
            vocab=positive(raw, "vocab", "the model"),
            norm_eps=float(need(need(raw, "norm", "the model"), "eps", "norm")),
            embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
            logit_softcap=float(raw.get("logit_softcap") or 0.0),
            max_positions=int(raw.get("max_positions") or cls.DEFAULT_POSITIONS),
            layers=tuple(layers),
        )

    def to_dict(self) -> dict:
        import copy

        out = {
            "architecture": self.architecture,
            "width": self.width,
            "vocab": self.vocab,
            "embedding": {"scale": self.embedding_scale},
            "norm": {"eps": self.norm_eps},
            "logit_softcap": self.logit_softcap,
            "layers": [copy.deepcopy(l) for l in self.layers],
        }
        if self.max_positions != self.DEFAULT_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


# --------------------------------------------------------------------------- Sisavik

_SISAVIK_LATENT_KEYS = ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale")
_SISAVIK_LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
_SISAVIK_RIGHT_KEYS = ("heads", "dim")


@dataclass(frozen=True)
class SisavikConfig(ModelConfig):
    """A Sisavik decoder: layers whose sublayers read the stream through a short causal
    convolution (x + conv(x), `canon.taps` taps per channel) and whose outputs pass an RMS
    norm (weight stored around zero, applied as 1 + w) before they join the stream. A
    layer's mixer is attention over a cached low-rank latent with a rotated key part shared
    by all heads and a sliding window (`latent_attention`; with `kv_from: j` it reads the
    rows layer j caches), or two mixers side by side whose outputs are added under
    `left_scale` and `right_scale` (`parallel`): grouped-query attention with sigmoid
    weights, values that are the keys as projected, a window and kept first tokens, beside
    a generalized delta rule with a decay per key channel. The feed-forward is gelu-gated
    and dense, or absent. The rows of the delta rule's low-rank decay map (`mix.right.w1`) are
    a size that only the tensor gives; `sisavik_sizes_from_tensors` writes it into the mixer as
    `right.decay_rank` when a model folder is read, and a configuration made in code names it
    there. config.json keys: `architecture`, `width`, `vocab`, `norm.eps`,
    `canon.taps` and `layers`, a list of `{"type", "mixer": {...}, "mlp": {"kind": "dense",
    "ff"} | null}`. Positions are bounded by `max_positions` alone (not a key of the design;
    absent, `DEFAULT_POSITIONS`)."""

    width: int
    vocab: int
    norm_eps: float
    taps: int = 1
    max_positions: int = 1 << 20
    layers: tuple = ()

    DEFAULT_POSITIONS = 1 << 20

    @classmethod
    def from_dict(cls, raw: dict) -> "SisavikConfig":
        def need(table, key: str, where: str) -> Any:
            if not isinstance(table, dict) or key not in table:
                raise ConfigError(f"config.json has no {key!r} in {where}, which Sisavik needs")
            return table[key]

        def positive(table, key: str, where: str) -> int:
            value = int(need(table, key, where))
            if value <= 0:
                raise ConfigError(f"{where}: {key}={value} must be positive")
            return value

        def rotation(table: dict, limit: int, where: str) -> None:
            rot = table.get("rot")
            if not rot:
                return
            dims = int(need(rot, "dims", f"{where}'s rot"))
            if dims < 0 or dims % 2 or dims > limit:
                raise ConfigError(f"{where}: rot.dims={dims} must be even and at most {limit}")
            if dims and float(need(rot, "base", f"{where}'s rot")) <= 0:
                raise ConfigError(f"{where}: rot.base must be positive")

        def mask(table: dict, where: str) -> None:
            m = table.get("mask")
            if not m:
                return
            if int(need(m, "size", f"{where}'s mask")) <= 0:
                raise ConfigError(f"{where}: mask.size must be positive")
            if int(m.get("keep_first", 0)) < 0:
                raise ConfigError(f"{where}: mask.keep_first must not be negative")

        layers = []
        listed = need(raw, "layers", "the model")
        for index, layer in enumerate(listed):
            where = f"layer {index}"
            kind = need(layer, "type", where)
            mixer = dict(need(layer, "mixer", where))
            if kind == "latent_attention":
                for key in _SISAVIK_LATENT_KEYS:
                    if key == "scale":
                        float(need(mixer, key, f"{where}'s mixer"))
                    elif key == "rot_dim":
                        if int(need(mixer, key, f"{where}'s mixer")) < 0:
                            raise ConfigError(f"{where}: rot_dim must not be negative")
                    else:
                        positive(mixer, key, f"{where}'s mixer")
                rotation(mixer, int(mixer["rot_dim"]), where)
                if int(mixer["rot_dim"]) and int((mixer.get("rot") or {}).get("dims", 0)) != int(mixer["rot_dim"]):
                    raise ConfigError(f"{where}: rot.dims must equal rot_dim, the rotated key part")
                mask(mixer, where)
                source = mixer.get("kv_from")
                if source is not None:
                    source = int(source)
                    ok = (0 <= source < index and listed[source].get("type") == "latent_attention"
                          and listed[source].get("mixer", {}).get("kv_from") is None)
                    if not ok:
                        raise ConfigError(f"{where}: kv_from={source} must name an earlier "
                                          f"latent-attention layer with a latent of its own")
                    theirs = listed[source]["mixer"]
                    same = (int(theirs.get("kv_rank", 0)) == int(mixer["kv_rank"])
                            and int(theirs.get("rot_dim", -1)) == int(mixer["rot_dim"])
                            and (theirs.get("rot") or {}) == (mixer.get("rot") or {}))
                    if not same:
                        raise ConfigError(f"{where}: kv_rank, rot_dim and rot differ from layer "
                                          f"{source}'s, whose rows it reads")
            elif kind == "parallel":
                left = dict(need(mixer, "left", f"{where}'s mixer"))
                right = dict(need(mixer, "right", f"{where}'s mixer"))
                for key in _SISAVIK_LEFT_KEYS:
                    if key == "scale":
                        float(need(left, key, f"{where}'s left mixer"))
                    else:
                        positive(left, key, f"{where}'s left mixer")
                if int(left["heads"]) % int(left["kv_heads"]):
                    raise ConfigError(f"{where}: {left['heads']} query heads do not divide into "
                                      f"{left['kv_heads']} key/value heads")
                if int(left["vdim"]) != int(left["dim"]):
                    raise ConfigError(f"{where}: the values are the keys, so vdim={left['vdim']} "
                                      f"must equal dim={left['dim']}")
                rotation(left, int(left["dim"]), f"{where}'s left mixer")
                mask(left, f"{where}'s left mixer")
                for key in _SISAVIK_RIGHT_KEYS:
                    positive(right, key, f"{where}'s right mixer")
                if "decay_rank" in right:
                    positive(right, "decay_rank", f"{where}'s right mixer")
                float(need(mixer, "left_scale", f"{where}'s mixer"))
                float(need(mixer, "right_scale", f"{where}'s mixer"))
            else:
                raise ConfigError(f"{where}: mixer type {kind!r} is not one of latent_attention, "
                                  f"parallel")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                if need(mlp, "kind", f"{where}'s mlp") != "dense":
                    raise ConfigError(f"{where}: feed-forward kind {mlp['kind']!r} is not built")
                positive(mlp, "ff", f"{where}'s mlp")
            import copy

            layers.append({"type": kind, "mixer": copy.deepcopy(layer["mixer"]), "mlp": mlp})
        if not layers:
            raise ConfigError("config.json lists no layers")
        taps = int((raw.get("canon") or {}).get("taps", 1))
        if not 1 <= taps <= 16:
            raise ConfigError(f"canon.taps={taps}: a convolution over 1 to 16 tokens is built")
        return cls(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Sisavik"])[0]),
            width=positive(raw, "width", "the model"),
            vocab=positive(raw, "vocab", "the model"),
            norm_eps=float(need(need(raw, "norm", "the model"), "eps", "norm")),
            taps=taps,
            max_positions=int(raw.get("max_positions") or cls.DEFAULT_POSITIONS),
            layers=tuple(layers),
        )

    def to_dict(self) -> dict:
        import copy

        out = {
            "architecture": self.architecture,
            "width": self.width,
            "vocab": self.vocab,
            "norm": {"eps": self.norm_eps},
            "canon": {"taps": self.taps},
            "layers": [copy.deepcopy(l) for l in self.layers],
        }
        if self.max_positions != self.DEFAULT_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


def sisavik_sizes_from_tensors(raw: dict, shapes: dict) -> dict:
    """The raw config.json with `mixer.right.decay_rank` of every parallel layer set to the
    rows of its `l<i>.mix.right.w1`, where the configuration does not name it."""
    import copy

    out = copy.deepcopy(raw)
    for index, layer in enumerate(out.get("layers") or []):
        right = (layer.get("mixer") or {}).get("right") if isinstance(layer, dict) else None
        shape = shapes.get(f"l{index}.mix.right.w1")
        if isinstance(right, dict) and "decay_rank" not in right and shape:
            right["decay_rank"] = int(shape[0])
    return out


# --------------------------------------------------------------------------- Lizazen

@dataclass(frozen=True)
class LizazenConfig(ModelConfig):
    """A Lizazen decoder: a token row plus a row of a hashed bigram table opens the stream;
    every layer has an RMS norm before and behind each sublayer. A layer's mixer is
    `attention` (grouped-query attention with biased q/k projections, values that are the keys
    as projected, one RMS norm over all heads' rows of q and of k, a partial rotation whose
    long wavelengths are slowed down, scores under a tanh cap, a sliding window and a softmax
    sink), `attention_2` (differential attention: two softmax maps per head over the same
    values, a sliding window beside kept first tokens) or `parallel` (softmax attention over
    chunks of positions beside retention, a linear attention with a fixed decay per head;
    the two outputs are normed and averaged). The feed-forward is dense with clamped gate
    and up (`kind: dense`), a mixture of experts whose router score multiplies the expert's
    input, with a shared expert (`kind: moe`), or absent. config.json keys: `architecture`,
    `width`, `vocab`, `norm.eps`, `embedding.bigram` (`buckets`, `mul_prev`, `mul_cur`; absent:
    no bigram table) and `layers`, a list of `{"type", "mixer": {...}, "mlp": {...} | null}`.
    Positions are bounded by `max_positions` alone (not a key of the design)."""

    width: int
    vocab: int
    norm_eps: float
    bigram: tuple | None = None          # (buckets, mul_prev, mul_cur)
    max_positions: int = 1 << 20
    layers: tuple = ()

    DEFAULT_POSITIONS = 1 << 20
    MIXERS = ("attention", "attention_2", "parallel")

    @classmethod
    def from_dict(cls, raw: dict) -> "LizazenConfig":
        import copy

        def need(table, key: str, where: str) -> Any:
            if not isinstance(table, dict) or key not in table:
                raise ConfigError(f"config.json has no {key!r} in {where}, which Lizazen needs")
            return table[key]

        def positive(table, key: str, where: str) -> int:
            value = int(need(table, key, where))
            if value <= 0:
                raise ConfigError(f"{where}: {key}={value} must be positive")
            return value

        def rotation(table: dict, where: str) -> None:
            rot = table.get("rot")
            if not rot:
                return
            dims = int(need(rot, "dims", f"{where}'s rot"))
            if dims < 0 or dims % 2 or dims > int(table["dim"]):
                raise ConfigError(f"{where}: rot.dims={dims} must be even and at most {table['dim']}")
            if dims and float(need(rot, "base", f"{where}'s rot")) <= 0:
                raise ConfigError(f"{where}: rot.base must be positive")
            scaling = rot.get("scaling")
            if scaling:
                for key in ("factor", "low", "high", "original"):
                    if float(need(scaling, key, f"{where}'s rot.scaling")) <= 0:
                        raise ConfigError(f"{where}: rot.scaling.{key} must be positive")
                if float(scaling["high"]) == float(scaling["low"]):
                    raise ConfigError(f"{where}: rot.scaling.high must differ from rot.scaling.low")

        def attention(table: dict, where: str, keys=("heads", "kv_heads", "dim", "vdim")) -> None:
            for key in keys:
                positive(table, key, where)
            float(need(table, "scale", where))
            if int(table["heads"]) % int(table["kv_heads"]):
                raise ConfigError(f"{where}: {table['heads']} query heads do not divide into "
                                  f"{table['kv_heads']} key/value heads")
            rotation(table, where)
            positive(need(table, "mask", where), "size", f"{where}'s mask")
            if int(table["mask"].get("keep_first", 0)) < 0:
                raise ConfigError(f"{where}: mask.keep_first must not be negative")

        def expert(table, where: str) -> None:
            positive(table, "ff", where)

        layers = []
        for index, layer in enumerate(need(raw, "layers", "the model")):
            where = f"layer {index}"
            kind = need(layer, "type", where)
            mixer = need(layer, "mixer", where)
            if kind == "attention":
                attention(mixer, f"{where}'s mixer")
                if int(mixer["vdim"]) != int(mixer["dim"]):
                    raise ConfigError(f"{where}: the values are the keys, so vdim={mixer['vdim']} "
                                      f"must equal dim={mixer['dim']}")
                if float(mixer.get("softcap") or 0.0) < 0:
                    raise ConfigError(f"{where}: softcap must not be negative")
            elif kind == "attention_2":
                attention(mixer, f"{where}'s mixer")
                float(need(mixer, "diff", f"{where}'s mixer"))
            elif kind == "parallel":
                attention(need(mixer, "left", f"{where}'s mixer"), f"{where}'s left mixer")
                right = need(mixer, "right", f"{where}'s mixer")
                for key in ("heads", "dim", "vdim"):
                    positive(right, key, f"{where}'s right mixer")
                rotation(right, f"{where}'s right mixer")
                decay = need(right, "decay", f"{where}'s right mixer")
                if len(decay) != int(right["heads"]):
                    raise ConfigError(f"{where}: {len(decay)} decays for {right['heads']} heads")
            else:
                raise ConfigError(f"{where}: mixer type {kind!r} is not one of "
                                  f"{', '.join(cls.MIXERS)}")
            mlp = layer.get("mlp")
            if mlp is not None:
                form = need(mlp, "kind", f"{where}'s mlp")
                if form == "dense":
                    positive(mlp, "ff", f"{where}'s mlp")
                    if float(need(mlp, "limit", f"{where}'s mlp")) <= 0:
                        raise ConfigError(f"{where}: mlp.limit must be positive")
                elif form == "moe":
                    expert(need(mlp, "expert", f"{where}'s mlp"), f"{where}'s mlp.expert")
                    router = need(mlp, "router", f"{where}'s mlp")
                    experts = positive(router, "experts", f"{where}'s mlp.router")
                    if not 1 <= positive(router, "top", f"{where}'s mlp.router") <= experts:
                        raise ConfigError(f"{where}: top={router['top']} of {experts} experts")
                    if mlp.get("shared") is not None:
                        expert(mlp["shared"], f"{where}'s mlp.shared")
                else:
                    raise ConfigError(f"{where}: feed-forward kind {form!r} is neither dense nor moe")
            layers.append({"type": kind, "mixer": copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)})
        if not layers:
            raise ConfigError("config.json lists no layers")
        bigram = (raw.get("embedding") or {}).get("bigram")
        if bigram:
            bigram = (positive(bigram, "buckets", "embedding.bigram"),
                      int(need(bigram, "mul_prev", "embedding.bigram")),
                      int(need(bigram, "mul_cur", "embedding.bigram")))
        return cls(
            architecture=str(raw.get("architecture") or (raw.get("architectures") or ["Lizazen"])[0]),
            width=positive(raw, "width", "the model"),
            vocab=positive(raw, "vocab", "the model"),
            norm_eps=float(need(need(raw, "norm", "the model"), "eps", "norm")),
            bigram=bigram or None,
            max_positions=int(raw.get("max_positions") or cls.DEFAULT_POSITIONS),
            layers=tuple(layers),
        )

    def to_dict(self) -> dict:
        import copy

        out = {
            "architecture": self.architecture,
            "width": self.width,
            "vocab": self.vocab,
            "norm": {"eps": self.norm_eps},
            "layers": [copy.deepcopy(l) for l in self.layers],
        }
        if self.bigram:
            out["embedding"] = {"bigram": {"buckets": self.bigram[0], "mul_prev": self.bigram[1],
                                           "mul_cur": self.bigram[2]}}
        if self.max_positions != self.DEFAULT_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


# --------------------------------------------------------------------------- the registry

@dataclass(frozen=True)
class Architecture:
    """What the engine knows about one architecture name: how to read its config.json and
    how to turn that configuration into a model description (`ModelSpec`)."""

    name: str
    config_class: type
    describe: Callable[[ModelConfig], Any]
    # optional: (raw config.json, {tensor name: shape}) -> raw config.json with the sizes
    # filled in that only a checkpoint's tensors give
    complete: Callable[[dict, dict], dict] | None = None


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, describe: Callable,
                          complete: Callable | None = None) -> None:
    """Add an architecture. `describe(config)` returns the `ModelSpec` to build. `complete(raw,
    shapes)` (optional) fills sizes into a raw config.json that only the shapes of the
    checkpoint's tensors give; it is called when a model folder is read."""
    _ARCHITECTURES[name] = Architecture(name, config_class, describe, complete)


def known_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def architecture_named(name: str) -> Architecture:
    _load_builtin()
    entry = _ARCHITECTURES.get(name)
    if entry is None:
        raise ConfigError(
            f"architecture {name!r} is not registered; known: {', '.join(sorted(_ARCHITECTURES))}"
        )
    return entry


def _load_builtin() -> None:
    # The built-in model descriptions register themselves when imported.
    from .. import models  # noqa: F401


def read_model_config(folder: str | Path) -> tuple[Architecture, ModelConfig]:
    """Parse `<folder>/config.json` with the class its `architectures[0]` is registered to.

    The reference falls back to "Qwen2ForCausalLM" when the key is absent
    (mercury/config.py:46); so does this.
    """
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    raw = json.loads(path.read_text())
    entry = architecture_named(architecture_name(raw))
    if entry.complete is not None:
        from ..weights.loader import tensor_shapes

        raw = entry.complete(raw, tensor_shapes(folder))
    return config_from_dict(raw)


def architecture_name(raw: dict) -> str:
    """The name a config.json registers under: the first of `architectures`, else the
    single `architecture`, else Qwen2 (the reference's default, mercury/config.py:46)."""
    listed = raw.get("architectures")
    if listed:
        return str(listed[0])
    return str(raw.get("architecture") or "Qwen2ForCausalLM")


def config_from_dict(raw: dict) -> tuple[Architecture, ModelConfig]:
    name = architecture_name(raw)
    entry = architecture_named(name)
    return entry, entry.config_class.from_dict(raw)


def config_fields(config: ModelConfig) -> dict:
    return {f.name: getattr(config, f.name) for f in fields(config)}
