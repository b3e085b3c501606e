"""Small Sisavik configurations for the tests, their random weights, and the comparison of a
replayed trace with the plain implementation."""

from __future__ import annotations

import json
import tempfile
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

import plain_sisavik
from mercury_b200.config import config_from_dict
from mercury_b200.trace_run import replay
from mercury_b200.weights import random_tensors


def _latent(heads, dim, rot_dim, vdim, rank, q_rank, window, base=10000.0, scale=None, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
             "q_rank": q_rank, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
             "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def _left(heads, kv_heads, dim, window, keep, rot_dims, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
            "scale": scale if scale is not None else dim ** -0.5,
            "mask": {"size": window, "keep_first": keep}, "rot": {"base": base, "dims": rot_dims}}


def _right(heads, dim, decay_rank):
    return {"heads": heads, "dim": dim, "decay_rank": decay_rank}


def _parallel(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _model(width, vocab, taps, layers, eps=1e-6):
    return {"architecture": "Sisavik", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "canon": {"taps": taps}, "layers": layers}


RAW = {
    # both kinds of layer in an order of their own; a latent read by two later layers with
    # other head sizes and windows (one wider than the source's own, one narrower); a second
    # latent of another rank; two parallel layers of different sizes; a layer without a
    # feed-forward; windows and kept tokens that are no multiples of a page
    "mix": _model(64, 131, 3, [
        _layer("parallel", _parallel(_left(4, 2, 16, 21, 5, 16), _right(3, 16, 8), 0.7, 0.4), 80),
        _layer("latent_attention", _latent(4, 16, 8, 24, 32, 24, 19, scale=0.3), 96),
        _layer("latent_attention", _latent(2, 24, 8, 8, 32, 40, 37, scale=0.25, kv_from=1)),
        _layer("latent_attention", _latent(3, 8, 4, 16, 40, 16, 50, base=500.0), 48),
        _layer("parallel", _parallel(_left(6, 3, 8, 40, 18, 4, base=300.0, scale=0.5),
                                     _right(2, 24, 5), 1.3, 0.2), 72),
        _layer("latent_attention", _latent(5, 8, 8, 8, 32, 8, 9, scale=0.4, kv_from=1), 32),
        _layer("latent_attention", _latent(2, 16, 4, 8, 40, 12, 33, base=500.0, kv_from=3)),
    ], eps=1e-5),
    # values that may hide a fault when equal or 1: one head, key/value heads as many as query
    # heads, scales of 1, a window of 1 (a token sees itself), no kept tokens, two taps, the
    # rotation over a part of the head only, value size equal to the key size
    "ones": _model(48, 77, 2, [
        _layer("latent_attention", _latent(1, 16, 16, 16, 16, 16, 1), 64),
        _layer("parallel", _parallel(_left(3, 3, 16, 1, 0, 6, scale=1.0), _right(1, 8, 1), 1.0, 1.0)),
        _layer("parallel", _parallel(_left(1, 1, 32, 25, 0, 32), _right(4, 4, 3), 1.0, 1.0), 40),
        _layer("latent_attention", _latent(1, 16, 16, 16, 16, 16, 30, kv_from=0), 24),
    ]),
    "only_latent": _model(48, 50, 3, [_layer("latent_attention", _latent(5, 12, 4, 20, 40, 28, 17), 64)]),
    "only_parallel": _model(48, 50, 3, [
        _layer("parallel", _parallel(_left(6, 2, 12, 17, 7, 8), _right(4, 12, 6), 0.6, 0.9), 64)]),
    # one tap: the convolution is a scale of the token itself and keeps no state
    "one_tap": _model(40, 50, 1, [
        _layer("latent_attention", _latent(2, 8, 4, 8, 16, 8, 12), 32),
        _layer("parallel", _parallel(_left(2, 1, 8, 12, 3, 8), _right(2, 8, 2), 0.5, 0.5), 32)]),
    # nothing a multiple of 8 (or of 4, where the design allows it); five taps; kept tokens
    # that reach beyond a page
    "odd": _model(100, 101, 5, [
        _layer("latent_attention", _latent(3, 20, 6, 12, 36, 22, 45, scale=0.3), 130),
        _layer("parallel", _parallel(_left(6, 2, 10, 23, 21, 6, base=77.0), _right(5, 6, 7), 0.9, 1.1), 50),
        _layer("latent_attention", _latent(7, 12, 6, 20, 36, 14, 11, scale=0.2, kv_from=0)),
        _layer("parallel", _parallel(_left(3, 1, 36, 70, 2, 18), _right(3, 20, 3), 0.3, 0.8), 34),
    ], eps=1e-4),
    # sizes at the edges of what the kernels choose between: cached rows of 64 and of 128
    # numbers (which the tensor-core attention kernels take) beside one they refuse, more
    # heads than a decode tile holds, head sizes of 128, matrices of 96 and of 160 rows
    "wide": _model(192, 300, 4, [
        _layer("latent_attention", _latent(20, 16, 16, 24, 48, 64, 40, scale=0.3), 200),
        _layer("parallel", _parallel(_left(4, 2, 128, 33, 17, 64), _right(2, 96, 16), 0.6, 0.5), 96),
        _layer("latent_attention", _latent(3, 40, 32, 8, 96, 32, 64)),
        _layer("latent_attention", _latent(16, 8, 32, 8, 96, 24, 100, kv_from=2), 64),
        _layer("parallel", _parallel(_left(16, 16, 32, 50, 33, 32), _right(1, 160, 4), 1.0, 0.3)),
        _layer("latent_attention", _latent(9, 24, 16, 16, 48, 48, 25, kv_from=0), 48),
        _layer("latent_attention", _latent(4, 32, 24, 32, 56, 40, 48), 48),
    ]),
    # layer sizes of the order a real model has (few layers, a small vocabulary)
    "real": _model(512, 1000, 4, [
        _layer("latent_attention", _latent(8, 64, 32, 64, 96, 192, 128), 1408),
        _layer("parallel", _parallel(_left(8, 2, 64, 128, 16, 64), _right(8, 64, 32), 0.5, 0.5), 1408),
        _layer("latent_attention", _latent(8, 64, 32, 64, 96, 192, 256, kv_from=0), 1408),
    ]),
}
SEED = {name: 61 + i for i, name in enumerate(RAW)}
SHARPEN = 3.0     # query-side projections are scaled so that attention is far from uniform


@lru_cache(maxsize=None)
def sisavik_model(name: str):
    """(raw config dictionary, typed config, {name: bfloat16 tensor})."""
    raw = RAW[name]
    _entry, config = config_from_dict(raw)
    tensors = random_tensors(config, SEED[name], torch.bfloat16, std=0.03 if name == "real" else 0.08)
    for key in tensors:
        if key.endswith(".mix.uq") or key.endswith(".mix.left.q"):
            tensors[key] = (tensors[key].float() * SHARPEN).to(torch.bfloat16)
    return raw, config, tensors


def random_tokens(count: int, vocab: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=gen).tolist()


@lru_cache(maxsize=None)
def requests_for(name: str, lengths: tuple) -> dict:
    return {f"r{i}": random_tokens(n, RAW[name]["vocab"], 700 + i) for i, n in enumerate(lengths)}


@lru_cache(maxsize=None)
def oracle(name: str, lengths: tuple) -> dict:
    raw, _config, tensors = sisavik_model(name)
    return {rid: plain_sisavik.forward(raw, tensors, tokens).numpy()
            for rid, tokens in requests_for(name, lengths).items()}


def make_runner(name, ops, device, dtype, page=16, num_tokens=512, poison=True, tensors=None, **more):
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, own = sisavik_model(name)
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
