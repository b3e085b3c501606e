"""Lizazen on the CUDA kernels: every mechanism through its part against the plain
implementation, the new kernels against their PyTorch twins at sizes of their own, and the
model through the engine's step function, cache and state manager, in float32 and bfloat16."""

from __future__ import annotations

import json
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import lizazen_mechanisms
import replay_cases
from kernel_twins import TorchOps
from lizazen_cases import (RAW, lizazen_model, make_runner, replay_and_compare, requests_for,
                           tolerance_for)
from mercury_b200.parts.base import LayerCache

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


@pytest.fixture(scope="module")
def ops():
    from mercury_b200.kernels.ops import CudaOps

    return CudaOps("cuda")


@pytest.fixture(scope="module")
def twin():
    return TorchOps(exact=True)


def rand(shape, dtype, seed, scale=1.0):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=gen) * scale).to(dtype).cuda()


def close(got, want, dtype, what="", tol32=3e-6, tol16=5e-3):
    tol = tol32 if dtype == torch.float32 else tol16
    scale = max(float(want.double().abs().max()), 1e-6)
    err = float((got.double() - want.double()).abs().max()) / scale
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite"
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.0e}"


# ------------------------------------------------------------------------------ mechanisms

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("check", lizazen_mechanisms.ALL, ids=lambda f: f.__name__[6:])
def test_mechanism(ops, check, dtype):
    check(ops, "cuda", dtype)


# ------------------------------------------------------------------------------ kernels and twins

def ragged(q_lens, kv_lens, slots=None, pad=0, page=16, scatter=7):
    """A batch of sequences with `q_lens` new tokens each, ending at `kv_lens`, and a block
    table whose pages lie scattered over the pool."""
    starts, seq_of, positions = [0], [], []
    for s, (n, kv) in enumerate(zip(q_lens, kv_lens)):
        starts.append(starts[-1] + n)
        seq_of += [s] * n
        positions += list(range(kv - n, kv))
    seq_of += [-1] * pad
    positions += [0] * pad
    per = -(-max(kv_lens) // page)
    total = per * len(q_lens)
    order = (torch.randperm(total + 1, generator=torch.Generator().manual_seed(scatter))[:total]
             if scatter else torch.arange(total))
    table = order.to(torch.int32).view(len(q_lens), per)
    dev = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return SimpleNamespace(num_seqs=len(q_lens), num_tokens=len(seq_of), q_start=dev(starts),
                           slots=dev(slots if slots is not None else list(range(len(q_lens)))),
                           seq_of_token=dev(seq_of), positions=dev(positions), kv_len=dev(list(kv_lens)),
                           max_q_len=max(q_lens), max_kv_len=max(kv_lens), table=table.cuda(),
                           pages=total + 1, attention_splits=None)


MASKS = [("full", 0, 0), ("sliding", 37, 0), ("sliding", 50, 21), ("chunked", 48, 0), ("sliding", 1, 0)]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("mask", MASKS, ids=lambda m: f"{m[0]}{m[1]}k{m[2]}")
@pytest.mark.parametrize("heads,kv_heads,maps,dim,vdim", [(4, 2, 1, 16, 16), (6, 2, 2, 24, 40),
                                                          (8, 8, 1, 64, 64), (3, 1, 2, 64, 128),
                                                          (5, 5, 1, 40, 200), (16, 2, 1, 128, 64)])
def test_masked_attention_against_its_twin(ops, twin, dtype, mask, heads, kv_heads, maps, dim, vdim):
    """Prompt portions beside decoded tokens, key ranges split over blocks and merged, a
    padded batch; sinks, a cap and both numbers of maps."""
    q_lens, kv_lens = (70, 1, 9, 1), (70, 190, 130, 33)
    batch = ragged(q_lens, kv_lens, pad=2)
    layout = (heads, kv_heads, maps, dim, vdim)
    k = rand((batch.pages, kv_heads, 16, maps * dim), dtype, 1, 0.7)
    v = rand((batch.pages, kv_heads, 16, vdim), dtype, 2)
    cache = LayerCache(k, v, 16, batch.table, True)
    q = rand((batch.num_tokens, heads * maps * dim), dtype, 3, 0.7)
    sinks = rand((heads,), torch.float32, 4) if maps == 1 else None
    extra = dict(softcap=6.0 if maps == 1 else 0.0, sinks=sinks, lam=0.45 if maps == 2 else 0.0,
                 sub_eps=1e-5, out_scale=0.7 if maps == 2 else 1.0)
    want = torch.zeros((batch.num_tokens, heads * vdim), dtype=dtype, device="cuda")
    twin.masked_attention(q, layout, batch, cache, dim ** -0.5, mask, want, **extra)
    live = batch.seq_of_token >= 0
    kernels = ["simt"]
    if dtype == torch.bfloat16 and ops.lib.mb_masked_attention_mma_supports(maps, dim, vdim):
        kernels.append("mma")
    for kernel in kernels:
        for splits in (None, 1, 3, 16):
            batch.attention_splits = splits
            got = torch.full_like(want, float("nan"))
            ops.masked_attention(q, layout, batch, cache, dim ** -0.5, mask, got, kernel=kernel, **extra)
            close(got[live], want[live], dtype, f"{kernel}, splits {splits}", tol32=1e-5, tol16=1.2e-2)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("heads,kv_heads,maps,dim,vdim,rot,from_keys,normed", [
    (4, 2, 1, 16, 16, 8, True, True), (6, 2, 2, 24, 40, 24, False, False),
    (3, 3, 1, 10, 6, 0, False, True), (8, 2, 1, 128, 64, 64, False, False)])
def test_prepare_against_its_twin(ops, twin, dtype, heads, kv_heads, maps, dim, vdim, rot, from_keys, normed):
    batch = ragged((5, 1, 40), (5, 77, 64), pad=3)
    layout = (heads, kv_heads, maps, dim, vdim)
    qs, ks = heads * maps * dim, kv_heads * maps * dim
    pre = rand((batch.num_tokens, qs + ks + (0 if from_keys else kv_heads * vdim)), torch.float32, 5)
    wq = rand((qs,), torch.float32, 6, 0.1) + 1 if normed else None
    wk = rand((ks,), torch.float32, 7, 0.1) + 1 if normed else None
    tables = None
    if rot:
        angle = torch.arange(128, dtype=torch.float64)[:, None] * 50.0 ** (-torch.arange(rot // 2) * 2.0 / rot)
        tables = (angle.cos().float().cuda(), angle.sin().float().cuda())
    out = {}
    for name, kernels in (("got", ops), ("want", twin)):
        k = torch.zeros((batch.pages, kv_heads, 16, maps * dim), dtype=dtype, device="cuda")
        v = torch.zeros((batch.pages, kv_heads, 16, vdim), dtype=dtype, device="cuda")
        q = torch.zeros((batch.num_tokens, qs), dtype=dtype, device="cuda")
        kernels.masked_prepare(pre, layout, wq, wk, 1e-5, tables, "halves", batch,
                               LayerCache(k, v, 16, batch.table, True), q, from_keys)
        out[name] = (q, k, v)
    live = batch.seq_of_token >= 0
    close(out["got"][0][live], out["want"][0][live], dtype, "queries", tol16=8e-3)
    close(out["got"][1], out["want"][1], dtype, "key pages", tol16=8e-3)
    close(out["got"][2], out["want"][2], dtype, "value pages", tol16=8e-3)


@pytest.mark.parametrize("heads,dim,vdim,rot", [(3, 12, 20, 8), (2, 64, 128, 64), (1, 160, 40, 0),
                                                (5, 6, 33, 6), (4, 128, 64, 32)])
def test_retention_over_steps_against_its_twin(ops, twin, heads, dim, vdim, rot):
    """Sequences in scattered slots over steps of unequal portions, one absent from a step."""
    decay = torch.tensor([0.999, 0.9, 0.5, 0.97, 1.0][:heads], dtype=torch.float32).cuda()
    tables = None
    if rot:
        angle = torch.arange(256, dtype=torch.float64)[:, None] * 50.0 ** (-torch.arange(rot // 2) * 2.0 / rot)
        tables = (angle.cos().float().cuda(), angle.sin().float().cuda())
    cells = torch.zeros((6, heads * dim * vdim), dtype=torch.float32, device="cuda")
    cells_want = cells.clone()
    width = 2 * heads * dim + heads * vdim
    at = [0, 0, 0]
    for step, q_lens in enumerate([(5, 1, 70), (1, 0, 2), (1, 1, 1), (33, 2, 1), (2, 9, 0)]):
        kv = [a + n for a, n in zip(at, q_lens)]
        batch = ragged(q_lens, kv, slots=[4, 0, 2], pad=3)
        pre = rand((batch.num_tokens, width + 7), torch.float32, 10 + step, 0.5)
        got = torch.zeros((batch.num_tokens, heads * vdim), dtype=torch.float32, device="cuda")
        want = torch.zeros_like(got)
        offsets = (3, 3 + heads * dim, 3 + 2 * heads * dim)
        ops.retention_scan(pre, offsets, decay, dim ** -0.5, (heads, dim, vdim), tables, "halves",
                           cells, batch, got)
        twin.retention_scan(pre, offsets, decay, dim ** -0.5, (heads, dim, vdim), tables, "halves",
                            cells_want, batch, want)
        live = batch.seq_of_token >= 0
        close(got[live], want[live], torch.float32, f"step {step}", tol32=1e-5)
        close(cells, cells_want, torch.float32, f"matrices after step {step}", tol32=1e-5)
        at = kv


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width", [72, 1024, 4100])
def test_join_against_its_twin(ops, twin, dtype, width):
    x, y = rand((37, width), torch.float32, 1, 2.0), rand((37, width), torch.float32, 2, 0.3)
    weights = [rand((width,), torch.float32, 3 + i, 0.1) + 1 for i in range(4)]
    for normed, follow in ((True, True), (True, False), (False, True)):
        h = rand((37, width), torch.float32, 9) + 3
        h_want = h.clone()
        out = torch.zeros((37, width), dtype=dtype, device="cuda") if follow else None
        out_want = torch.zeros_like(out) if follow else None
        args = (weights[0] if normed else None, weights[1] if normed else None, 0.5, 0.8, weights[2], 1e-5,
                weights[3] if follow else None, 1e-6)
        ops.rmsnorm_join_add(h, x, y, *args, out)
        twin.rmsnorm_join_add(h_want, x, y, *args, out_want)
        close(h, h_want, torch.float32, "stream")
        if follow:
            close(out, out_want, dtype, "norm computed ahead", tol16=8e-3)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("pairs,hidden,ff", [(40, 64, 24), (3000, 256, 96)])
def test_experts_weighted_on_their_input_against_the_twin(ops, twin, dtype, pairs, hidden, ff):
    """Few pairs (this package's grouped products) and many (the library's, in bfloat16)."""
    from mercury_b200.engine.runner import StepContext, Workspace

    experts, top = 6, 2
    tokens = pairs // top
    x = rand((tokens, hidden), dtype, 1)
    gate_up = rand((experts, 2 * ff, hidden), dtype, 2, 0.1)
    down = rand((experts, hidden, ff), dtype, 3, 0.1)
    gen = torch.Generator().manual_seed(4)
    chosen = torch.stack([torch.randperm(experts, generator=gen)[:top] for _ in range(tokens)]).int().cuda()
    weights = torch.rand((tokens, top), generator=gen).cuda() + 0.2
    ctx = StepContext(ops, Workspace(torch.device("cuda"), dtype, tokens), 16, dtype)
    got = torch.zeros((tokens, hidden), dtype=torch.float32, device="cuda")
    want = torch.zeros_like(got)
    ops.expert_feed_forward(x, chosen, weights, gate_up, down, got, ctx, weight_on="input")
    twin.expert_feed_forward(x, chosen, weights, gate_up, down, want, weight_on="input")
    close(got, want, dtype, "experts", tol32=1e-5, tol16=2e-2)


@pytest.mark.parametrize("tokens", [1, 5, 16, 40])
@pytest.mark.parametrize("hidden,ff", [(256, 96), (896, 4864)])
def test_clamped_gate_in_the_few_token_product(ops, twin, tokens, hidden, ff):
    """Up to 16 tokens the product and the clamped gate are one kernel; beyond, two."""
    from mercury_b200.engine.runner import StepContext, Workspace

    dtype = torch.bfloat16
    x = rand((tokens, hidden), dtype, 1)
    weight = rand((2 * ff, hidden), dtype, 2, 0.08)
    ctx = StepContext(ops, Workspace(torch.device("cuda"), dtype, tokens), 16, dtype)
    got = torch.zeros((tokens, ff), dtype=dtype, device="cuda")
    want = torch.zeros_like(got)
    before = ops.launches + ops.library_calls
    ops.linear_gated(x, weight, got, ctx, "clamped_sigmoid", limit=0.8, slope=1.702)
    assert (ops.launches + ops.library_calls - before == 1) == (tokens <= 16)
    twin.linear_gated(x, weight, want, None, "clamped_sigmoid", limit=0.8, slope=1.702)
    raw = x.float() @ weight.float().T
    assert (raw > 0.8).any() and (raw < -0.8).any()
    close(got, want, dtype, "clamped gate", tol16=1.2e-2)


# ------------------------------------------------------------------------------ the model

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 100, 41), "odd": (50, 7, 121, 33),
           "wide": (40, 110)}


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["mix", "ones", "odd", "wide"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay(ops, name, mode, dtype):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 320, seed=5) if mode == "mixed" else builder(requests)
    page = {"mix": 16, "ones": 8, "wide": 32, "odd": 4}[name]
    replay_and_compare(make_runner(name, ops, "cuda", dtype, page=page, num_tokens=320), name, lengths,
                       steps, rows, tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("mode", ["whole", "mixed"])
def test_real_layer_sizes(ops, dtype, mode):
    """Layer sizes of the order a real model has: the shapes at which the few-token, library
    and tensor-core kernels are chosen."""
    name, lengths = "real", (150, 40, 300, 17)
    requests = requests_for(name, lengths)
    steps, rows = (replay_cases.whole(requests) if mode == "whole"
                   else replay_cases.mixed(requests, 640, seed=5))
    replay_and_compare(make_runner(name, ops, "cuda", dtype, num_tokens=640), name, lengths, steps,
                       rows, tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_through_graphs(ops, dtype):
    """A short prompt and then 200 tokens one by one (replayed CUDA graphs), every window and
    chunk passing over decoded tokens, in a pool smaller than the request is long."""
    name, lengths = "mix", (230,)
    requests = requests_for(name, lengths)
    steps, rows = replay_cases.decode_tail(requests, tail=200)
    runner = make_runner(name, ops, "cuda", dtype, num_tokens=192, poison=False, max_model_len=256)
    replay_and_compare(runner, name, lengths, steps, rows, tolerance_for(dtype, name, lengths))
    assert runner.graph_replays > 100


def test_cut_does_not_change_float32_logits(ops):
    """The same request whole and in portions of two tokens: beyond rounding nothing moves."""
    import numpy as np
    from mercury_b200.engine.batch import StepEntry

    name = "mix"
    tokens = requests_for(name, (90,))["r0"]
    got = []
    for cut in (90, 2):
        runner = make_runner(name, ops, "cuda", torch.float32, poison=False, cuda_graphs=False)
        seq = runner.open("a")
        rows = []
        for at in range(0, 90, cut):
            part = tokens[at:at + cut]
            rows.append(runner.step([StepEntry(seq, part, list(range(len(part))))]).clone())
        got.append(torch.cat(rows).cpu().numpy())
    assert np.abs(got[0] - got[1]).max() <= 2e-5 * np.abs(got[0]).max()


def test_greedy_generation_through_the_engine_and_cli(ops, tmp_path):
    from mercury_b200 import Engine, EngineConfig, SamplingParams
    from mercury_b200.weights import write_random_model
    from test_lizazen_cpu import greedy

    name = "mix"
    raw, config, tensors = lizazen_model(name)
    runner = make_runner(name, ops, "cuda", torch.float32, num_tokens=256, poison=False)
    cfg = EngineConfig(model="(memory)", device="cuda", dtype="float32", block_size=16, num_blocks=16,
                       max_running=4, max_batched_tokens=256, prefill_chunk=24, max_model_len=256,
                       debug_invariants=True)
    engine = Engine(cfg, runner=runner)
    prompts = [requests_for(name, (37, 70, 20))[f"r{i}"] for i in range(3)]
    outs = engine.generate(prompts, SamplingParams(), 8)
    for prompt, out in zip(prompts, outs):
        assert out == greedy(raw, tensors, prompt, 8)
    assert engine.leaked_pages() == 0
    # the command line on a model folder written by the random-weights mode
    folder = write_random_model(tmp_path / "model", config, seed=3)
    from safetensors.torch import load_file
    stored = load_file(str(folder / "model.safetensors"))
    stored_raw = json.loads((folder / "config.json").read_text())
    done = subprocess.run(
        [sys.executable, "-m", "mercury_b200.generate", "--model", str(folder), "--dtype", "float32",
         "--prompt-ids", ",".join(map(str, prompts[2])), "--max-tokens", "5", "--num-blocks", "32",
         "--max-model-len", "128", "--max-running", "2", "--max-batched-tokens", "128"],
        capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert json.loads(done.stdout.strip().splitlines()[-1])["output_ids"] == greedy(stored_raw, stored, prompts[2], 5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_on_a_model_folder(dtype, tmp_path):
    """The replay program as a user runs it: a model folder, steps on standard input, a pool
    for the live requests only."""
    from pathlib import Path

    import numpy as np
    from safetensors.torch import save_file

    from lizazen_cases import oracle

    name = "odd"
    raw, _config, tensors = lizazen_model(name)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    lengths = (50, 7, 121, 33, 90, 64)
    requests = requests_for(name, lengths)
    steps, rows = replay_cases.mixed(requests, 320, seed=2)
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    done = subprocess.run(
        [str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
         "--max-tokens", "320"],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
        timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.split("\n") if l.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    want = oracle(name, lengths)
    tol = tolerance_for(torch.float32 if dtype == "float32" else torch.bfloat16, name, lengths)
    for step, expected in rows.items():
        if not expected:
            continue
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(expected), -1)
        for row, (rid, pos) in enumerate(expected):
            err = np.abs(got[row] - want[rid][pos]).max() / np.abs(want[rid]).max()
            assert err <= tol, (step, rid, pos, err)
