"""Sisavik on the CUDA kernels: every mechanism through its part against the plain
implementation, the new kernels against their PyTorch twins at sizes of their own, and the
model through the engine's step function, cache and state manager, in float32 and bfloat16."""

from __future__ import annotations

import json
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import replay_cases
import sisavik_mechanisms
from kernel_twins import TorchOps
from mercury_b200.parts.base import LayerCache
from sisavik_cases import (RAW, make_runner, replay_and_compare, requests_for, sisavik_model,
                           tolerance_for)

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
@pytest.mark.parametrize("check", sisavik_mechanisms.ALL, ids=lambda f: f.__name__[6:])
def test_mechanism(ops, check, dtype):
    check(ops, "cuda", dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_reader_looks_further_back_than_the_layer_that_caches(ops, dtype):
    sisavik_mechanisms.check_latent_attention(ops, "cuda", dtype, own_window=19, cache_window=44)


# ------------------------------------------------------------------------------ kernels and twins

def ragged(q_lens, kv_lens, slots=None, pad=0):
    """A batch of sequences with `q_lens` new tokens each, ending at `kv_lens`."""
    starts, seq_of, positions = [0], [], []
    for s, (n, kv) in enumerate(zip(q_lens, kv_lens)):
        starts.append(starts[-1] + n)
        seq_of += [s] * n
        positions += list(range(kv - n, kv))
    seq_of += [-1] * pad
    positions += [0] * pad
    dev = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return SimpleNamespace(num_seqs=len(q_lens), num_tokens=len(seq_of), q_start=dev(starts),
                           slots=dev(slots if slots is not None else list(range(len(q_lens)))),
                           seq_of_token=dev(seq_of), positions=dev(positions), kv_len=dev(list(kv_lens)),
                           max_q_len=max(q_lens), max_kv_len=max(kv_lens))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("fused", [False, True], ids=["store", "store-in-norm"])
@pytest.mark.parametrize("width,taps", [(200, 3), (1024, 4), (72, 2), (136, 7)])
def test_stream_convolution_over_steps(ops, twin, dtype, width, taps, fused):
    """Sequences in scattered slots over steps of unequal portions, shorter and longer than
    the convolution's reach, one of them absent from a step; the ring carries over. `fused`:
    the step's last rows are kept by the norm behind the sublayer, which then changes the
    stream."""
    weight = rand((width, taps), torch.float32, 1, 0.5)
    state = torch.zeros((6, taps - 1, width), dtype=torch.float32, device="cuda")
    state_want = state.clone()
    at = [0, 0, 0]
    for step, q_lens in enumerate([(5, 1, 70), (1, 0, 2), (1, 1, 1), (33, 2, 1), (2, 9, 0)]):
        kv = [a + n for a, n in zip(at, q_lens)]
        batch = ragged(q_lens, kv, slots=[4, 0, 2], pad=3)
        h = rand((batch.num_tokens, width), torch.float32, 10 + step)
        got = torch.zeros((batch.num_tokens, width), dtype=dtype, device="cuda")
        want = torch.zeros_like(got)
        ops.stream_conv(h, weight, state, batch, got)
        twin.stream_conv(h, weight, state_want, batch, want)
        live = batch.seq_of_token >= 0
        if fused:
            delta = rand((batch.num_tokens, width), dtype, 20 + step)
            delta2 = rand((batch.num_tokens, width), dtype, 30 + step) if step % 2 else None
            gain = rand((width,), torch.float32, 3) + 1
            h_want = h.clone()
            ops.rmsnorm_add(h, delta, gain, 1e-5, None, 0.0, None, delta2=delta2, scale=0.7,
                            scale2=1.3, tail=(state, batch))
            twin.rmsnorm_add(h_want, delta, gain, 1e-5, None, 0.0, None, delta2=delta2, scale=0.7,
                             scale2=1.3, tail=(state_want, batch))
            close(h[live], h_want[live], torch.float32, f"stream after step {step}")
        else:
            ops.stream_tail_store(h, state, batch)
            twin.stream_tail_store(h, state_want, batch)
        close(got[live], want[live], dtype, f"step {step}")
        assert torch.equal(state, state_want), f"ring after step {step}"
        at = kv


@pytest.mark.parametrize("heads,dim,vdim", [(3, 12, 12), (6, 32, 32), (2, 64, 64), (1, 128, 128),
                                             (5, 20, 20), (2, 96, 96)])
@pytest.mark.parametrize("precise", [False, True], ids=["fast", "precise"])
def test_general_delta_scan_over_steps(ops, twin, heads, dim, vdim, precise):
    width = heads * dim
    cells = rand((5, heads * dim * vdim), torch.float32, 3, 0.1)
    cells_want = cells.clone()
    offsets = (0, width, 2 * width, 3 * width)
    for step, q_lens in enumerate([(40, 1, 3), (1, 1, 0), (2, 17, 1)]):
        batch = ragged(q_lens, q_lens, slots=[3, 0, 1])
        pre = rand((batch.num_tokens, 4 * width + 5), torch.float32, 20 + step)
        decay = rand((batch.num_tokens, width), torch.float32, 30 + step, 2.0)
        got = torch.zeros((batch.num_tokens, heads * vdim), dtype=torch.float32, device="cuda")
        want = torch.zeros_like(got)
        ops.general_delta_scan(pre, offsets, decay, 0.6, (heads, dim, vdim), 1e-6, cells, batch, got,
                               precise=precise)
        twin.general_delta_scan(pre, offsets, decay, 0.6, (heads, dim, vdim), 1e-6, cells_want, batch,
                                want)
        close(got, want, torch.float32, f"read-outs, step {step}", 2e-5)
        close(cells, cells_want, torch.float32, f"matrices, step {step}", 2e-5)
    assert torch.equal(cells[2], cells_want[2]) and torch.equal(cells[4], cells_want[4])


SIGMOID_CASES = [
    # heads, kv heads, dim, page, q_lens, kv_lens, window, keep
    (6, 3, 64, 16, (5, 1, 33), (5, 140, 33), 50, 13),
    (6, 2, 32, 16, (1, 1, 1, 1), (1, 9, 240, 400), 50, 7),
    (8, 8, 16, 8, (70, 2), (200, 66), 33, 0),
    (3, 1, 128, 32, (40, 1, 2), (100, 777, 50), 64, 64),
    (16, 2, 64, 16, (130, 1), (130, 2000), 0, 0),
    (5, 5, 24, 16, (1, 2), (300, 301), 1, 3),
    (2, 1, 40, 64, (1,), (1500,), 1024, 1),
    (14, 2, 64, 16, (300, 1, 70), (300, 500, 331), 100, 70),
    (4, 4, 128, 16, (129, 64), (400, 64), 65, 64),
    (8, 1, 64, 32, (200,), (1000,), 128, 129),
]


@pytest.mark.parametrize("kernel,dtype", [("simt", torch.float32), ("simt", torch.bfloat16),
                                          ("mma", torch.bfloat16)], ids=["f32", "bf16", "bf16-mma"])
@pytest.mark.parametrize("splits", [0, 1, 5])
@pytest.mark.parametrize("case", range(len(SIGMOID_CASES)), ids=lambda i: f"case{i}")
def test_sigmoid_attention_against_its_twin(ops, twin, kernel, dtype, splits, case):
    """`splits`: the keys of a row tile divided over that many blocks (0: the kernel's own
    choice), summed afterwards. Pages behind the window and not among the kept first tokens
    are absent from the table."""
    from test_kernels_gpu import make_batch

    heads, kv_heads, dim, page, q_lens, kv_lens, window, keep = SIGMOID_CASES[case]
    if kernel == "mma" and not ops.lib.mb_sigmoid_attention_mma_supports(dim):
        pytest.skip("head sizes left to the CUDA-core kernel")
    num_pages = sum(-(-kv // page) for kv in kv_lens) + 3
    batch, table = make_batch(q_lens, kv_lens, page, num_pages, pad_tokens=2, seed=case)
    if window:
        for s, (q, kv) in enumerate(zip(q_lens, kv_lens)):
            first_needed = max(0, kv - q - window + 1) // page
            for p in range(-(-keep // page), first_needed):
                table[s, p] = -1
    batch.attention_splits = splits or None
    k = rand((num_pages, kv_heads, page, dim), dtype, 40 + case, 0.5)
    q = rand((batch.num_tokens, heads * dim), dtype, 50 + case, 0.5)
    bias = rand((heads,), torch.float32, 60 + case)
    cache = LayerCache(k, k, page, table, False)
    got = torch.zeros((batch.num_tokens, heads * dim), dtype=dtype, device="cuda")
    want = torch.zeros_like(got)
    layout = (heads, kv_heads, dim, dim)
    ops.sigmoid_attention(q, layout, batch, cache, dim ** -0.5, window, keep, bias, got, kernel=kernel)
    twin.sigmoid_attention(q, layout, batch, cache, dim ** -0.5, window, keep, bias, want)
    live = batch.seq_of_token >= 0
    close(got[live], want[live], dtype, "sigmoid attention", 2e-5, 8e-3)


# ------------------------------------------------------------------------------ the model

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 150, 41, 90), "wide": (40, 300),
           "odd": (50, 7, 121, 33)}


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["only_latent", "only_parallel", "one_tap"])
def test_each_layer_kind_alone(ops, dtype, name):
    lengths = (1, 2, 60)
    requests = requests_for(name, lengths)
    for builder in (replay_cases.whole, replay_cases.portions):
        steps, rows = builder(requests)
        replay_and_compare(make_runner(name, ops, "cuda", dtype), name, lengths, steps, rows,
                           tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["mix", "ones", "wide", "odd"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay(ops, dtype, name, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 512, seed=3) if mode == "mixed" else builder(requests)
    page = {"mix": 16, "ones": 8, "wide": 32, "odd": 4}[name]
    replay_and_compare(make_runner(name, ops, "cuda", dtype, page=page), name, lengths, steps, rows,
                       tolerance_for(dtype, name, lengths))


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
    """A short prompt and then 200 tokens one by one (replayed CUDA graphs), every window
    passing over decoded tokens, in a pool smaller than the request is long."""
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
    from test_sisavik_cpu import greedy

    name = "mix"
    raw, config, tensors = sisavik_model(name)
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
    """The replay program as a user runs it: a folder whose config.json does not name the
    decay map's rows (the tensors give them), steps on standard input, a pool for the live
    requests only."""
    import copy
    from pathlib import Path

    import numpy as np
    from safetensors.torch import save_file

    name = "odd"
    raw, _config, tensors = sisavik_model(name)
    bare = copy.deepcopy(raw)
    for layer in bare["layers"]:
        if layer["type"] == "parallel":
            del layer["mixer"]["right"]["decay_rank"]
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(bare))
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
    from sisavik_cases import oracle

    want = oracle(name, lengths)
    tol = tolerance_for(torch.float32 if dtype == "float32" else torch.bfloat16, name, lengths)
    for step, expected in rows.items():
        if not expected:
            continue
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(expected), -1)
        for row, (rid, pos) in enumerate(expected):
            err = np.abs(got[row] - want[rid][pos]).max() / np.abs(want[rid]).max()
            assert err <= tol, (step, rid, pos, err)
