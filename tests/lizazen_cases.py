"""Small Lizazen configurations for the tests, their random weights, and the comparison of a
replayed trace with the plain implementation."""

from __future__ import annotations

import json
import tempfile
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

import plain_lizazen
from mercury_b200.config import config_from_dict
from mercury_b200.trace_run import replay
from mercury_b200.weights import random_tensors


def _rot(dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return rot


def capped(heads, kv_heads, dim, window, rot_dims, softcap, scale=None, base=10000.0, scaling=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
            "scale": scale if scale is not None else dim ** -0.5, "softcap": softcap,
            "mask": {"size": window}, "rot": _rot(rot_dims, base, scaling)}


def differential(heads, kv_heads, dim, vdim, window, keep, rot_dims, diff, scale=None, base=10000.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
            "scale": scale if scale is not None else dim ** -0.5,
            "mask": {"size": window, "keep_first": keep}, "rot": _rot(rot_dims, base)}


def chunked(heads, kv_heads, dim, vdim, chunk, rot_dims, scale=None, base=10000.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else dim ** -0.5,
            "mask": {"size": chunk}, "rot": _rot(rot_dims, base)}


def retained(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": _rot(rot_dims, base)}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(width, vocab, layers, bigram=(53, 31, 5), eps=1e-6):
    out = {"architecture": "Lizazen", "width": width, "vocab": vocab, "norm": {"eps": eps},
           "layers": layers}
    if bigram:
        out["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
    return out


RAW = {
    # all three kinds of layer in an order of their own, twice with other sizes; two experts a
    # token, with and without a shared expert; a layer without a feed-forward; windows, kept
    # tokens and chunks that are no multiples of a page; scaled and plain rotations
    "mix": model(64, 131, [
        layer("parallel", {"left": chunked(4, 2, 16, 24, 21, 8), "right": retained(3, 16, 8, (0.9, 0.99, 0.5), 16)},
              moe(5, 2, 24, shared=40)),
        layer("attention_2", differential(4, 2, 8, 24, 19, 5, 4, 0.3), dense(80, 0.7)),
        layer("attention", capped(6, 2, 8, 37, 8, 3.0, scale=0.9, scaling=(4.0, 1.0, 3.0, 48))),
        layer("attention_2", differential(2, 1, 16, 8, 40, 18, 16, 0.75, scale=0.4, base=300.0), moe(3, 1, 32)),
        layer("attention", capped(2, 2, 24, 9, 6, 20.0, base=500.0), dense(48, 2.5)),
        layer("parallel", {"left": chunked(6, 3, 8, 8, 33, 4, base=77.0), "right": retained(2, 24, 12, (0.97, 0.8), 8)},
              dense(72, 1.0)),
    ], eps=1e-5),
    # values that may hide a fault when equal or 1: one head, as many key/value heads as query
    # heads, scales of 1, a window of 1 and a chunk of 1 (a token sees itself), no kept
    # tokens, no decay at all and a decay of nothing kept, every expert chosen, no rotation
    # on one side, no bigram table
    "ones": model(48, 77, [
        layer("attention", capped(1, 1, 16, 1, 16, 1.0, scale=1.0), dense(64, 1.0)),
        layer("attention_2", differential(3, 3, 8, 8, 1, 0, 2, 0.5, scale=1.0), moe(2, 2, 16, shared=16)),
        layer("parallel", {"left": chunked(1, 1, 32, 32, 1, 32, scale=1.0), "right": retained(1, 8, 8, (1.0,), 0)}),
        layer("parallel", {"left": chunked(2, 2, 16, 16, 25, 0), "right": retained(2, 4, 16, (0.0, 0.5), 4)},
              moe(1, 1, 24)),
        layer("attention_2", differential(1, 1, 32, 32, 30, 30, 32, 0.0), dense(24, 100.0)),
    ], bigram=None),
    "only_capped": model(48, 50, [layer("attention", capped(6, 2, 12, 17, 8, 5.0, scaling=(6.0, 1.0, 3.0, 64)),
                                        dense(64, 1.5))]),
    "only_differential": model(48, 50, [layer("attention_2", differential(6, 2, 12, 20, 17, 7, 6, 0.45),
                                              moe(4, 2, 16, shared=24))]),
    "only_parallel": model(48, 50, [layer("parallel", {"left": chunked(6, 2, 12, 20, 17, 8),
                                                       "right": retained(4, 12, 6, (0.9, 0.95, 0.99, 0.999), 12)},
                                          moe(6, 1, 16, shared=8))]),
    # nothing a multiple of 8 (or of 4, where the design allows it); kept tokens that reach
    # beyond a page; a multiplier of zero in the pair hash
    "odd": model(100, 101, [
        layer("attention", capped(6, 3, 10, 45, 6, 7.5, scale=0.3), moe(7, 3, 22, shared=26)),
        layer("parallel", {"left": chunked(6, 2, 10, 14, 23, 6, base=77.0), "right": retained(5, 6, 10, (0.9, 0.8, 0.7, 0.99, 0.95), 2)},
              dense(50, 0.9)),
        layer("attention_2", differential(3, 1, 18, 26, 23, 21, 10, 0.4), dense(34, 1.2)),
        layer("parallel", {"left": chunked(3, 1, 36, 20, 70, 18), "right": retained(3, 20, 6, (0.5, 0.6, 0.999), 20)},
              moe(3, 2, 30)),
    ], bigram=(97, 0, 3), eps=1e-4),
    # sizes at the edges of what the kernels choose between: head sizes of 64 and 128 (which
    # the tensor-core attention kernels take) beside ones they refuse, more heads than a tile
    # holds, retention heads of 96 x 160 and 160 x 40, a value size above the key size
    "wide": model(192, 300, [
        layer("attention", capped(8, 2, 64, 40, 32, 30.0), dense(200, 1.0)),
        layer("attention_2", differential(4, 2, 64, 128, 33, 17, 64, 0.5), moe(6, 2, 96, shared=64)),
        layer("parallel", {"left": chunked(16, 16, 32, 64, 50, 32), "right": retained(1, 96, 160, (0.98,), 48)}),
        layer("attention_2", differential(3, 1, 40, 72, 64, 3, 8, 0.2), dense(64, 0.5)),
        layer("parallel", {"left": chunked(4, 2, 128, 64, 48, 64), "right": retained(2, 160, 40, (0.9, 0.999), 160)},
              moe(4, 1, 48, shared=48)),
        layer("attention", capped(20, 4, 16, 25, 16, 2.0, scaling=(2.0, 0.5, 2.0, 30)), dense(48, 3.0)),
    ], bigram=(211, 13, 1)),
    # layer sizes of the order a real model has (few layers, a small vocabulary)
    "real": model(512, 1000, [
        layer("attention", capped(8, 2, 64, 128, 64, 30.0, scaling=(4.0, 1.0, 8.0, 256)), dense(1408, 7.0)),
        layer("attention_2", differential(4, 2, 64, 128, 80, 16, 32, 0.55), moe(8, 2, 352, shared=704)),
        layer("parallel", {"left": chunked(8, 4, 64, 64, 128, 64), "right": retained(4, 64, 128, (0.97, 0.99, 0.995, 0.999), 64)},
              dense(1408, 7.0)),
    ], bigram=(4093, 1021, 17)),
}
SEED = {name: 83 + i for i, name in enumerate(RAW)}
SHARPEN = 3.0     # query projections are scaled so that attention is far from uniform


@lru_cache(maxsize=None)
def lizazen_model(name: str):
    """(raw config dictionary, typed config, {name: bfloat16 tensor})."""
    raw = RAW[name]
    _entry, config = config_from_dict(raw)
    tensors = random_tensors(config, SEED[name], torch.bfloat16, std=0.03 if name == "real" else 0.08)
    for key in tensors:
        if key.endswith(".q") and ".right." not in key:
            tensors[key] = (tensors[key].float() * SHARPEN).to(torch.bfloat16)
        if key.endswith(".router"):
            # far apart, so that no choice of experts rests on a close call
            tensors[key] = (tensors[key].float() * 4.0).to(torch.bfloat16)
    return raw, config, tensors


def random_tokens(count: int, vocab: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=gen).tolist()


@lru_cache(maxsize=None)
def requests_for(name: str, lengths: tuple) -> dict:
    return {f"r{i}": random_tokens(n, RAW[name]["vocab"], 900 + i) for i, n in enumerate(lengths)}


@lru_cache(maxsize=None)
def oracle(name: str, lengths: tuple) -> dict:
    raw, _config, tensors = lizazen_model(name)
    return {rid: plain_lizazen.forward(raw, tensors, tokens).numpy()
            for rid, tokens in requests_for(name, lengths).items()}


def make_runner(name, ops, device, dtype, page=16, num_tokens=512, poison=True, tensors=None, **more):
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, own = lizazen_model(name)
    more.setdefault("max_model_len", num_tokens)     # the pool may be smaller than a request is long
    return ModelRunner(config=config, tensors=tensors if tensors is not None else own, dtype=dtype,
                       device=device, page_size=page, num_pages=num_tokens // page, max_seqs=4,
                       max_step_tokens=num_tokens, ops=ops,
                       poison_pages=poison, **more)


def compare_rows(runner, steps, rows, want, vocab, tolerance) -> float:
    """Replays `steps`; every written row against `want[request][position]`. The error of a row
    is its largest difference over the request's largest logit. Returns the worst."""
    scale = {rid: float(np.abs(w).max()) for rid, w in want.items()}
    worst = 0.0
    with tempfile.TemporaryDirectory() as tmp:
        done = []
        replay(runner, [json.dumps(s) for s in steps], Path(tmp), done.append)
        assert done == [f"done {s['step']}" for s in steps]
        for step, expected in rows.items():
            if not expected:
                continue
            got = np.fromfile(Path(tmp) / f"{step}.f32", dtype="<f4").reshape(len(expected), vocab)
            for row, (rid, pos) in enumerate(expected):
                assert np.isfinite(got[row]).all(), f"step {step} {rid}@{pos}: non-finite logits"
                err = float(np.abs(got[row].astype(np.float64) - want[rid][pos]).max() / scale[rid])
                assert err <= tolerance, (f"step {step}: request {rid} position {pos}: relative "
                                          f"error {err:.3e} exceeds {tolerance:.0e}")
                worst = max(worst, err)
    assert not runner.cache.live
    runner.cache.check_invariants()
    assert runner.cache.leaked_pages() == 0
    return worst


def replay_and_compare(runner, name, lengths, steps, rows, tolerance) -> float:
    return compare_rows(runner, steps, rows, oracle(name, lengths), RAW[name]["vocab"], tolerance)


@lru_cache(maxsize=None)
def bfloat16_bound(name: str, lengths: tuple) -> float:
    """What the bfloat16 engine may be off by on this model: twice what a bfloat16 twin of
    the plain implementation itself is off by (the PyTorch twins of the kernels, float32
    arithmetic, bfloat16 storage between them, whole prompts), and at least 1.5e-2."""
    import replay_cases
    from kernel_twins import TorchOps

    steps, rows = replay_cases.whole(requests_for(name, lengths))
    runner = make_runner(name, TorchOps(), "cpu", torch.bfloat16, poison=False)
    return max(1.5e-2, 2.0 * replay_and_compare(runner, name, lengths, steps, rows, 1.0))


def tolerance_for(dtype, name: str, lengths: tuple) -> float:
    return 3e-5 if dtype == torch.float32 else bfloat16_bound(name, lengths)
