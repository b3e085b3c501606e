"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl mercury_b200|reference]

The default run has the layer sizes of Qwen2.5-0.5B (24 layers, hidden 896, 14 query heads,
2 KV heads of 64, feed-forward 4864, vocabulary 151936, tied head) with seeded random
weights in bfloat16, pages of 16 tokens, a model length of 4096, and decodes a batch of 8
requests whose contexts hold 2048 tokens. One "step" is one decode step of the whole batch.

It prints ONE JSON line:
  value      decoded tokens per second, timed on the device with CUDA events over K steps
             issued back to back (after W warm-up steps); the block of K steps is timed five
             times and the median block gives `value` and `ms_per_step` (`repeats` holds the
             minimum, median and maximum);
  e2e        the same through `Engine.step()`: every step copies its inputs from pinned host
             memory, samples on the device and reads the tokens back to the host;
  prefill    one 2048-token prompt in one step: tokens/s, ms, and flops / time / peak;
             `prefill_512x4` is the same prompt in four portions of 512;
  roofline   for the decode step: bytes it has to read (every weight once, the cache of
             the live requests) / time, against the measured copy bandwidth;
  points     decode tokens per second at batch 1 and 64, `point_rooflines` their fractions;
  kernels    per class of kernel call, for the decode step and for the prompt step: the
             milliseconds it takes (CUDA events around every call of a step launched eagerly
             behind a device-side delay, so that the launches queue up), what the model needs
             of it (bytes to read, or flops) and that over time over the measured peak.
Weights (about 1 GB) are far larger than the 126 MB L2, so every step streams them from
HBM again; no extra L2 flush is needed ("l2" in config says so).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN25_05B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 24, "hidden_size": 896,
    "num_attention_heads": 14, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 4864, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "use_sliding_window": False,
    "max_position_embeddings": 32768,
}
SIZES = {
    "0.5b": QWEN25_05B,
    "1.5b": {**QWEN25_05B, "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12,
             "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 8960},
    "7b": {**QWEN25_05B, "num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28,
           "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
           "vocab_size": 152064, "tie_word_embeddings": False},
}
BATCH = 8
CONTEXT = 2048        # tokens each request holds when decoding starts
MODEL_LEN = 4096      # benchmark context length: the most a request may reach
PREFILL_TOKENS = 2048
BLOCK = 16
SEED = 0
REPEATS = 5           # how often the block of K decode steps is timed
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
METRIC = "decode tok/s at batch 8 (Qwen2.5-0.5B sizes, 2048-token contexts)"


def bench_config(peak_kind: str) -> dict:
    """The `config` of the JSON line: every size of the run, flat; the same for both arms."""
    c = QWEN25_05B
    return {"model": "Qwen2.5-0.5B sizes", "layers": c["num_hidden_layers"],
            "layers_of_model": c["num_hidden_layers"], "hidden": c["hidden_size"],
            "q_heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
            "head_dim": c["head_dim"], "intermediate": c["intermediate_size"],
            "vocab": c["vocab_size"], "tied": c["tie_word_embeddings"], "global_batch": BATCH,
            "seq_len": CONTEXT, "max_model_len": MODEL_LEN, "kv_block": BLOCK,
            "parallelism": "single GPU", "l2": "inputs>L2 (1 GB of weights streamed per step)",
            "peaks": peak_kind}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        raw = json.loads(path.read_text())
        out = dict(FALLBACK_PEAKS)
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if isinstance(raw.get(key), (int, float)):
                out[key] = float(raw[key])
        return out, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background while a timed region runs."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except OSError:
            self.proc = None

    def stop(self, window: tuple[float, float] | None = None) -> dict:
        """Median SM clock and the throttle reasons seen; with `window` (start, end in
        time.time() seconds) only the samples taken inside it count."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        self.proc.wait()
        import datetime

        clocks, top, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7 or not parts[1].isdigit():
                continue
            if window is not None:
                try:
                    stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                except ValueError:
                    continue
                if not window[0] <= stamp <= window[1]:
                    continue
            clocks.append(int(parts[1]))
            top = int(parts[2]) if parts[2].isdigit() else top
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": top,
                "reasons": sorted(reasons), "samples": len(clocks)}


def class_costs(cfg: dict, batch: int, context: int, tokens: int) -> dict:
    """What each class of kernel call has to move or compute: for a decode step of `batch`
    requests at `context` tokens ("decode": bytes read) and for a prompt step of `tokens`
    tokens ("prefill": flops, or bytes for the classes that only move data)."""
    h, i, v, layers = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (n_q + 2 * n_kv) * d
    kv_layer = 2 * n_kv * d * 2                   # bytes of keys and values per token and layer
    decode = {
        "q/k/v product": ("hbm", layers * 2 * (qkv * h + qkv)),
        "q/k/v + rotary + store": ("hbm", layers * 2 * (qkv * h + qkv)),
        "attention": ("hbm", layers * batch * context * kv_layer),
        "residual product": ("hbm", layers * 2 * (n_q * d * h + h * i)),
        "gated product": ("hbm", layers * 2 * 2 * i * h),
        "product": ("hbm", 2 * v * h),
        "norm": ("hbm", 2 * batch * h * 6),
        "embedding": ("hbm", batch * h * 6),
        "sampling": ("hbm", batch * v * 4),
    }
    t = tokens
    prefill = {
        "q/k/v product": ("tensor", layers * 2 * t * qkv * h),
        "q/k/v + rotary + store": ("tensor", layers * 2 * t * qkv * h),
        "rotary + store": ("hbm", layers * t * (2 * qkv * 2 + 2 * n_kv * d * 2)),
        "attention": ("tensor", 2 * t * t * n_q * d * layers),
        "residual product": ("tensor", layers * 2 * t * (n_q * d * h + h * i)),
        "gated product": ("tensor", layers * 2 * t * 2 * i * h),
        "gate": ("hbm", layers * t * 3 * i * 2),
        "product": ("hbm", 2 * v * h),
        # every norm reads the float32 stream and a bfloat16 delta, writes both back
        "norm": ("hbm", (2 * layers + 1) * t * h * (4 + 2 + 4 + 2)),
        "embedding": ("hbm", t * h * 6),
    }
    return {"decode": decode, "prefill": prefill}


def model_numbers(cfg: dict) -> dict:
    """Bytes a decode step must read and flops a prefill must do, from the sizes alone."""
    h, i, v, layers = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    n_q, n_kv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    qkv = (n_q + 2 * n_kv) * d
    per_layer = qkv * h + qkv + n_q * d * h + 2 * i * h + h * i + 2 * h
    head = v * h
    params_read = layers * per_layer + head + h   # tied table read once by the head
    if not cfg["tie_word_embeddings"]:
        pass  # the embedding table is only gathered from, not streamed
    kv_per_token = 2 * layers * n_kv * d * 2
    gemm_flops_per_token = 2 * layers * (qkv * h + n_q * d * h + 3 * i * h)
    return {"weight_bytes": 2 * params_read, "kv_bytes_per_token": kv_per_token,
            "gemm_flops_per_token": gemm_flops_per_token,
            "attn_flops": lambda t: 2 * t * t * n_q * d * layers, "head_flops_per_row": 2 * head}


def make_runner(torch, config, tensors, batch, page_tokens, graphs=True, gemm=None):
    from mercury_b200.engine.runner import ModelRunner
    from mercury_b200.kernels.ops import CudaOps

    ops = CudaOps("cuda", gemm=gemm) if gemm else None
    return ModelRunner(config=config, tensors=tensors, dtype=torch.bfloat16, device="cuda",
                       page_size=BLOCK, num_pages=page_tokens // BLOCK, max_seqs=batch,
                       max_step_tokens=max(PREFILL_TOKENS, batch), max_model_len=MODEL_LEN,
                       cuda_graphs=graphs, ops=ops)


def timed(torch, fn, reps: int) -> float:
    """Milliseconds per call of fn over `reps` calls, by CUDA events."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps


def fill_contexts(torch, runner, batch, context, vocab):
    from mercury_b200.engine.batch import StepEntry

    gen = torch.Generator().manual_seed(SEED + 1)
    seqs = []
    for b in range(batch):
        seq = runner.open(f"bench-{b}")
        tokens = torch.randint(0, vocab, (context,), generator=gen).tolist()
        for at in range(0, context, PREFILL_TOKENS):
            runner.step([StepEntry(seq, tokens[at:at + PREFILL_TOKENS], [])])
        seqs.append(seq)
    torch.cuda.synchronize()
    return seqs


def decode_rate(torch, runner, batch, context, vocab, steps, warmup, load_window=None, repeats=1):
    """(tokens/s, ms per step, launches per step, [ms per step of every repeat]) of `steps`
    decode steps of `batch`, timed `repeats` times in a row (the median repeat counts). With
    `load_window` (a list) the same steps keep running, untimed, until a second has passed
    since the timed region began, and [start, end] of that stretch is appended: the clock
    sampler needs more than the few dozen milliseconds the timed steps take."""
    from mercury_b200.engine.batch import StepEntry

    seqs = fill_contexts(torch, runner, batch, context, vocab)
    out = torch.empty(batch, dtype=torch.int32, device="cuda")
    gen = torch.Generator().manual_seed(SEED + 2)
    feed = torch.randint(0, vocab, (steps * repeats + warmup + 1, batch), generator=gen).tolist()
    turn = [0]

    def one():
        tokens = feed[turn[0]]
        turn[0] += 1
        logits = runner.step([StepEntry(s, [tokens[i]], [0]) for i, s in enumerate(seqs)])
        runner.ops.argmax(logits, out)

    if load_window is not None:
        feed += feed * (int(1.2 / 0.0005) // len(feed) + 1)
    for _ in range(warmup):
        one()
    before = runner.launch_count()
    began = time.time()
    samples = [timed(torch, one, steps) for _ in range(repeats)]
    ms = statistics.median(samples)
    launches = (runner.launch_count() - before) / (steps * repeats)
    if load_window is not None:
        while time.time() - began < 1.0 and turn[0] < len(feed) - 1 and \
                seqs[0].num_computed + 2 < runner.max_model_len:
            one()
        torch.cuda.synchronize()
        load_window.extend([began, time.time()])
    for s in seqs:
        runner.close(s)
    return batch * 1e3 / ms, ms, launches, samples


def kernel_classes(torch, runner, batch, context, vocab, cfg, peak) -> dict:
    """Milliseconds per class of kernel call of one decode step of `batch` requests and of
    one prompt step, each launched eagerly with CUDA events around every call; a delay on
    the device lets the launches queue up first, so that the events see kernels back to
    back and not the host's launch loop. Beside each: what the model needs of the class
    (bytes or flops), and that over time over the measured peak."""
    from mercury_b200.engine.batch import StepEntry

    costs = class_costs(cfg, batch, context, PREFILL_TOKENS)
    out = {}
    seqs = fill_contexts(torch, runner, batch, context, vocab)
    gen = torch.Generator().manual_seed(SEED + 6)
    tokens = torch.randint(0, vocab, (8, batch), generator=gen).tolist()
    prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    sampled = torch.empty(batch, dtype=torch.int32, device="cuda")
    runner.time_kernels = True
    try:
        rows = []
        for turn in range(4):                      # the first two are warm-up
            torch.cuda._sleep(20_000_000)          # about 10 ms: the step's launches queue up behind it
            logits = runner.step([StepEntry(s, [tokens[turn][i]], [0]) for i, s in enumerate(seqs)])
            rows.append(dict(runner.last_kernel_ms))
        decode = {k: statistics.median(r.get(k, 0.0) for r in rows[2:]) for k in rows[-1]}
        torch.cuda._sleep(20_000_000)
        runner.ops.begin_timing()
        runner.ops.argmax(logits, sampled)
        decode["sampling"] = runner.ops.end_timing().get("sampling", 0.0)
        for s in seqs:
            runner.close(s)
        rows = []
        for turn in range(3):
            seq = runner.open(f"classes-{turn}")
            torch.cuda._sleep(40_000_000)
            runner.step([StepEntry(seq, prompt, [PREFILL_TOKENS - 1])])
            rows.append(dict(runner.last_kernel_ms))
            runner.close(seq)
        prefill = {k: statistics.median(r.get(k, 0.0) for r in rows[1:]) for k in rows[-1]}
    finally:
        runner.time_kernels = False
    for name, measured in (("decode", decode), ("prefill", prefill)):
        block = {}
        for kind, ms in sorted(measured.items()):
            bound, amount = costs[name].get(kind, ("hbm", 0))
            top = peak["hbm_gbs"] * 1e9 if bound == "hbm" else peak["bf16_tflops"] * 1e12
            block[kind] = {"ms": round(ms, 4), "bound": bound,
                           "frac": round(amount / (ms * 1e-3) / top, 4) if ms > 0 and amount else None}
        block["sum_ms"] = round(sum(measured.values()), 4)
        out[name] = block
    return out


def prefill_rate(torch, runner, vocab, reps=5):
    from mercury_b200.engine.batch import StepEntry

    gen = torch.Generator().manual_seed(SEED + 3)
    tokens = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    times = []
    for rep in range(reps + 2):
        seq = runner.open(f"prefill-{rep}")
        ms = timed(torch, lambda: runner.step([StepEntry(seq, tokens, [PREFILL_TOKENS - 1])]), 1)
        runner.close(seq)
        if rep >= 2:
            times.append(ms)
    return statistics.median(times)


def prefill_portions_rate(torch, runner, vocab, portion=512, reps=5):
    """The 2048-token prompt as portions of `portion` tokens, one step each; ms for all."""
    from mercury_b200.engine.batch import StepEntry

    gen = torch.Generator().manual_seed(SEED + 3)
    tokens = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    times = []

    def run(seq):
        for at in range(0, PREFILL_TOKENS, portion):
            last = at + portion >= PREFILL_TOKENS
            runner.step([StepEntry(seq, tokens[at:at + portion], [portion - 1] if last else [])])

    for rep in range(reps + 2):
        seq = runner.open(f"portions-{rep}")
        ms = timed(torch, lambda: run(seq), 1)
        runner.close(seq)
        if rep >= 2:
            times.append(ms)
    return statistics.median(times)


def e2e_rate(torch, config, tensors, batch, context, vocab, steps, warmup):
    """Decode tokens/s through Engine.step(): host tokens in, host tokens out."""
    from mercury_b200 import Engine, EngineConfig, SamplingParams
    runner = make_runner(torch, config, tensors, batch, batch * (context + 256))
    cfg = EngineConfig(model="(in memory)", dtype="bfloat16", block_size=BLOCK,
                       num_blocks=runner.cache.pools[0].num_pages, max_running=batch,
                       max_batched_tokens=max(PREFILL_TOKENS, batch), prefill_chunk=PREFILL_TOKENS,
                       max_model_len=MODEL_LEN, prefix_caching=False, seed=SEED)
    engine = Engine(cfg, runner=runner)
    gen = torch.Generator().manual_seed(SEED + 4)
    produced = []
    started = set()

    def sink(event):
        produced.append(event.kind)
        started.add(event.rid)

    for b in range(batch):
        prompt = torch.randint(0, vocab, (context,), generator=gen).tolist()
        engine.submit(f"e2e-{b}", prompt, steps + warmup + batch + 8, sink,
                      SamplingParams(ignore_eos=True))
    while len(started) < batch:          # prompts first: until every request decodes
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    size_before = len(produced)
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    tokens = sum(1 for kind in produced[size_before:] if kind == "token")
    assert tokens == batch * steps, (tokens, batch, steps)
    lay = runner.buffers._layout(batch, batch, -(-(context + steps + warmup + batch + 8) // BLOCK), batch)
    return tokens / seconds, lay["size"] * 4, batch * 4


def other_sizes(torch, args) -> dict:
    """The side workloads of the benchmark description, one flat block: decode at batch 8 and
    the 2048-token prompt at Qwen2.5-1.5B and 7B sizes (all their layers, random weights), and
    the mixed serving workload at 1.5B sizes. A size that fails says so and does not take the
    line with it."""
    from types import SimpleNamespace

    from mercury_b200.config import config_from_dict
    from mercury_b200.weights import random_tensors

    out = {}
    for name in ("1.5b", "7b"):
        try:
            raw = SIZES[name]
            _entry, config = config_from_dict(raw)
            tensors = random_tensors(config, SEED, torch.bfloat16)
            runner = make_runner(torch, config, tensors, BATCH, BATCH * (CONTEXT + 256))
            steps = min(args.steps, 32)
            rate, ms, _l, _s = decode_rate(torch, runner, BATCH, CONTEXT, raw["vocab_size"], steps,
                                           max(3, min(args.warmup, 8)))
            out[f"{name}_decode_b8"] = round(rate, 1)
            out[f"{name}_decode_ms"] = round(ms, 4)
            out[f"{name}_prefill_ms"] = round(prefill_rate(torch, runner, raw["vocab_size"], reps=3), 3)
            out[f"{name}_layers"] = raw["num_hidden_layers"]
            del runner
            torch.cuda.empty_cache()
            if name == "1.5b":
                mixed = run_mixed(SimpleNamespace(size=name, policy="lpm"), prepared=(config, tensors))
                out["1.5b_mixed_output_tokens_per_s"] = mixed["output_tokens_per_s"]
                out["1.5b_mixed_prefix_hit_tokens"] = mixed["prefix_hit_tokens"]
                out["1.5b_mixed_requests"] = 32
            del tensors
            torch.cuda.empty_cache()
        except Exception as exc:      # a side workload must not cost the headline its line
            out[f"{name}_error"] = f"{type(exc).__name__}: {exc}"[:200]
    return out


def run_ours(args) -> dict:
    import torch

    from mercury_b200.config import config_from_dict
    from mercury_b200.weights import random_tensors

    peak, peak_kind = peaks()
    _entry, config = config_from_dict(QWEN25_05B)
    tensors = random_tensors(config, SEED, torch.bfloat16)
    vocab = QWEN25_05B["vocab_size"]
    numbers = model_numbers(QWEN25_05B)

    sampler = ClockSampler()
    sampler.start()
    runner = make_runner(torch, config, tensors, 64, 64 * (CONTEXT + 256))
    window: list[float] = []
    value, ms, launches, samples = decode_rate(torch, runner, BATCH, CONTEXT, vocab, args.steps,
                                               args.warmup, load_window=window, repeats=REPEATS)
    clocks = sampler.stop(tuple(window))
    b1, ms1, _, _ = decode_rate(torch, runner, 1, CONTEXT, vocab, args.steps, args.warmup, repeats=3)
    b64, ms64, _, _ = decode_rate(torch, runner, 64, CONTEXT, vocab, args.steps, args.warmup, repeats=3)
    prefill_ms = prefill_rate(torch, runner, vocab)
    portions_ms = prefill_portions_rate(torch, runner, vocab)
    kernels = kernel_classes(torch, runner, BATCH, CONTEXT, vocab, QWEN25_05B, peak)
    del runner
    torch.cuda.empty_cache()
    e2e, h2d, d2h = e2e_rate(torch, config, tensors, BATCH, CONTEXT, vocab, args.steps, args.warmup)
    del tensors
    torch.cuda.empty_cache()
    sizes = {} if args.no_sizes else other_sizes(torch, args)

    def step_bytes(batch, steps_before):
        return numbers["weight_bytes"] + batch * (CONTEXT + steps_before) * numbers["kv_bytes_per_token"]

    def fraction(batch, step_ms, steps_before):
        return round(step_bytes(batch, steps_before) / (step_ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)

    middle = args.warmup + REPEATS * args.steps // 2
    achieved = step_bytes(BATCH, middle) / (ms * 1e-3) / 1e9
    flops = (PREFILL_TOKENS * numbers["gemm_flops_per_token"] + numbers["attn_flops"](PREFILL_TOKENS)
             + numbers["head_flops_per_row"])
    return {
        "metric": METRIC,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform-random token ids, random N(0,0.02) weights",
        "config": bench_config(peak_kind),
        "repeats": {"n": REPEATS, "ms_min": round(min(samples), 4),
                    "ms_median": round(statistics.median(samples), 4), "ms_max": round(max(samples), 4)},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "prefill_512x4": {"value": round(PREFILL_TOKENS * 1e3 / portions_ms, 1),
                          "tokens": PREFILL_TOKENS, "ms": round(portions_ms, 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1)},
        "point_rooflines": {"decode_b1": {"ms": round(ms1, 4), "frac": fraction(1, ms1, args.warmup + 3 * args.steps // 2)},
                            "decode_b64": {"ms": round(ms64, 4), "frac": fraction(64, ms64, args.warmup + 3 * args.steps // 2)}},
        "kernels": kernels,
        "sizes": sizes,
        "clocks": clocks,
    }


def run_part(args) -> dict:
    """`--only decode|prefill|products`: one small workload for profilers, with the same
    model, weights and shapes as the full run. Prints what it measured, not the bench line."""
    import torch

    from mercury_b200.config import config_from_dict
    from mercury_b200.weights import random_tensors

    if args.only == "mixed":
        return run_mixed(args)
    if args.only == "designs":
        return run_designs(args)
    raw = SIZES[args.size]
    _entry, config = config_from_dict(raw)
    vocab = raw["vocab_size"]
    if args.only == "products":
        from types import SimpleNamespace

        from mercury_b200.kernels.ops import CudaOps

        def replayed(fn, calls=10):
            """Microseconds per call of fn, `calls` of them replayed from a CUDA graph: the
            device's time without the host's share (a product of a few microseconds is
            launched more slowly than it runs)."""
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(calls):
                    fn()
            graph.replay()
            return timed(torch, graph.replay, max(args.steps, 3)) / calls * 1e3

        out = {}
        for name, (m, n, k) in {"qkv": (2048, 1152, 896), "o": (2048, 896, 896),
                                "gate_up": (2048, 9728, 896), "down": (2048, 896, 4864),
                                "qkv_7b": (2048, 4608, 3584), "down_7b": (2048, 3584, 18944)}.items():
            x = torch.randn(m, k).bfloat16().cuda()
            w = torch.randn(n, k).bfloat16().cuda()
            y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            for gemm in ("library", "tcgen05"):
                ops = CudaOps("cuda", gemm=gemm)
                us = replayed(lambda: ops.linear(x, w, None, y))
                ops.check_errors()
                out[f"{name}_{gemm}_us"] = round(us, 1)
                out[f"{name}_{gemm}_tflops"] = round(2 * m * n * k / us / 1e6, 1)
            ops = CudaOps("cuda")
            error = torch.zeros(1, dtype=torch.int32, device="cuda")
            stream = torch.cuda.current_stream

            def pairs():
                assert ops.lib.mb_gemm_pair(x.data_ptr(), w.data_ptr(), None, y.data_ptr(), 0, m, n, k,
                                            None, 0, 0.0, 0, None, None, None, None, error.data_ptr(),
                                            stream().cuda_stream) == 0
            us = replayed(pairs)
            assert int(error.item()) == 0
            out[f"{name}_pairs_us"] = round(us, 1)
            out[f"{name}_pairs_tflops"] = round(2 * m * n * k / us / 1e6, 1)
        # the gated product: gate/up with the SiLU gate in the epilogue, one CTA per tile against
        # pairs of CTAs, and the library's product followed by the gate kernel
        for name, (m, width, k) in {"gated_0.5b": (2048, 4864, 896), "gated_1.5b": (2048, 8960, 1536),
                                    "gated_7b": (2048, 18944, 3584)}.items():
            x = torch.randn(m, k).bfloat16().cuda()
            w = (torch.randn(2 * width, k) * 0.05).bfloat16().cuda()
            y = torch.empty(m, width, dtype=torch.bfloat16, device="cuda")
            both = torch.empty(m, 2 * width, dtype=torch.bfloat16, device="cuda")
            ctx = SimpleNamespace(buffer=lambda *_a, **_k: both)
            for label, gemm, min_k in (("one_cta", "auto", 1 << 30), ("pairs", "auto", 0),
                                       ("library_and_gate", "library", 0)):
                ops = CudaOps("cuda", gemm=gemm)
                ops.pair_min_k = min_k
                ops.gated_max_elements = 1 << 40
                us = replayed(lambda: ops.linear_swiglu(x, w, y, ctx))
                ops.check_errors()
                out[f"{name}_{label}_us"] = round(us, 1)
                out[f"{name}_{label}_tflops"] = round(4 * m * width * k / us / 1e6, 1)
        return out
    tensors = random_tensors(config, SEED, torch.bfloat16)
    batch = args.batch
    runner = make_runner(torch, config, tensors, max(batch, 2), max(batch, 2) * (CONTEXT + 256),
                         graphs=not args.no_graphs, gemm=args.gemm)
    if args.only == "prefill":
        return {"prefill_ms": round(prefill_rate(torch, runner, vocab, reps=args.steps), 3)}
    if args.only == "kernels":
        return kernel_classes(torch, runner, batch, CONTEXT, vocab, raw, peaks()[0])
    rate, ms, launches, _samples = decode_rate(torch, runner, batch, CONTEXT, vocab, args.steps,
                                               args.warmup)
    return {"decode_tokens_per_s": round(rate, 1), "ms_per_step": round(ms, 4), "batch": batch,
            "launches_per_step": launches, "graphs": not args.no_graphs}


# ------------------------------------------------------------------------------ other designs

DESIGN_SIZES = {
    # width, query heads, key/value heads, head size, feed-forward, recurrent blocks
    "0.5b": (896, 14, 2, 64, 4864, 7),
    "1.5b": (1536, 12, 2, 128, 8960, 12),
}
DESIGN_LAYERS = 8
DESIGN_VOCAB = 32768


def design_configs(size: str) -> tuple[dict, dict]:
    """A Fegenex model at the layer sizes of `size` (attention with a feed-forward, minGRU,
    gated linear recurrence, attention with a feed-forward, twice over) and the Qwen2 model
    of the same width, heads, feed-forward, depth and vocabulary beside it."""
    width, heads, kv_heads, dim, ff, blocks = DESIGN_SIZES[size]
    attention = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                           "rot": {"dims": dim // 2, "base": 10000.0}, "scale": dim ** -0.5,
                           "v_mix": True}}
    order = [attention, {"type": "mingru", "mixer": {"width": width}, "mlp": None},
             {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": 4}, "mlp": None},
             attention]
    fegenex = {"architecture": "Fegenex", "width": width, "vocab": DESIGN_VOCAB,
               "max_positions": MODEL_LEN, "norm": {"eps": 1e-6},
               "layers": [order[i % len(order)] for i in range(DESIGN_LAYERS)]}
    qwen2 = {**SIZES[size], "num_hidden_layers": DESIGN_LAYERS, "vocab_size": DESIGN_VOCAB,
             "tie_word_embeddings": False}
    return fegenex, qwen2


def design_costs(raw: dict, batch: int, context: int, tokens: int) -> dict:
    """Per class of kernel call, what a Fegenex model has to read (decode step, bytes) or
    compute (prompt step, flops; bytes for the classes that only move data)."""
    w, v = raw["width"], raw["vocab"]
    products = head = 2 * v * w
    gated = kv_token = att_flops = mix_flops = rec_tokens = 0
    norms = 1
    for layer in raw["layers"]:
        m = layer["mixer"]
        norms += 2
        if layer["type"] == "attention":
            qkv = (m["heads"] + m["kv_heads"]) * m["dim"] + m["kv_heads"] * m["vdim"]
            products += 2 * (qkv * w + m["heads"] * m["vdim"] * w)
            kv_token += 2 * m["kv_heads"] * (m["dim"] + m["vdim"])
            att_flops += m["heads"] * (m["dim"] + m["vdim"])
            mix_flops += m["heads"] * m["heads"]
        elif layer["type"] == "mingru":
            products += 2 * 4 * m["width"] * w
            rec_tokens += 4 * 3 * m["width"] + 2 * m["width"]
        else:
            products += 2 * 3 * m["width"] * w
            rec_tokens += 4 * 9 * m["width"] + 2 * m["width"]
        if layer["mlp"]:
            norms += 2
            gated += 2 * 2 * layer["mlp"]["ff"] * w
            products += 2 * layer["mlp"]["ff"] * w
    t = tokens
    return {
        "decode": {"product": ("hbm", products), "gated product": ("hbm", gated),
                   "attention": ("hbm", batch * context * kv_token),
                   "recurrence": ("hbm", batch * rec_tokens), "norm": ("hbm", norms * batch * w * 12)},
        "prefill": {"product": ("tensor", t * (products - head) + head),
                    "gated product": ("tensor", t * gated),
                    "attention": ("tensor", t * t * (att_flops + mix_flops)),
                    "recurrence": ("hbm", t * rec_tokens), "norm": ("hbm", norms * t * w * 14)},
    }


KINELIX_SIZES = {
    # width, heads, head size, latent rank, feed-forward, experts, experts a token uses
    "0.5b": (896, 14, 64, 128, 4864, 16, 4),
    "1.5b": (1536, 12, 128, 128, 8960, 16, 4),
}


def kinelix_config(size: str) -> dict:
    """A Kinelix model at the layer sizes of `size`: attention over a cached latent with a
    dense feed-forward, a Mamba-2 layer and a gated delta rule with routed experts (whose
    active width equals the dense feed-forward's), and an attention layer that reads the
    first one's latent, twice over."""
    width, heads, dim, rank, ff, experts, top = KINELIX_SIZES[size]
    moe = {"kind": "moe", "expert": {"ff": ff // top},
           "router": {"experts": experts, "top": top, "scale": 1.0, "groups": {"count": 4, "keep": 2}}}

    def latent(source=None):
        mixer = {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": rank, "scale": dim ** -0.5}
        if source is not None:
            mixer["kv_from"] = source
        return mixer

    layers = []
    for base in range(0, DESIGN_LAYERS, 4):
        layers += [
            {"type": "latent_attention", "mixer": latent(), "mlp": {"kind": "dense", "ff": ff}},
            {"type": "mamba2", "mlp": moe,
             "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 2,
                       "norm_groups": 2, "conv": 4}},
            {"type": "delta", "mlp": moe,
             "mixer": {"heads": width // 128, "kv_heads": width // 128, "dim": 128, "vdim": 128,
                       "conv": 4}},
            {"type": "latent_attention", "mixer": latent(base), "mlp": {"kind": "dense", "ff": ff}},
        ]
    return {"architecture": "Kinelix", "width": width, "vocab": DESIGN_VOCAB,
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "max_positions": MODEL_LEN, "layers": layers[:DESIGN_LAYERS]}


def kinelix_costs(raw: dict, batch: int, context: int, tokens: int) -> dict:
    """Per class of kernel call, what a Kinelix model has to read (decode step, bytes) or
    compute (prompt step, flops; bytes for the classes that only move data)."""
    w, v = raw["width"], raw["vocab"]
    products = head = 2 * v * w
    gated = latent_token = att_flops = head_products = 0
    expert_all = expert_active = router = state_bytes = scan_flops = rec_tokens = 0
    norms = 1
    for layer in raw["layers"]:
        m = layer["mixer"]
        norms += 1
        if layer["type"] == "latent_attention":
            own = m.get("kv_from") is None
            rows = m["heads"] * m["dim"] + (m["kv_rank"] if own else 0)
            products += 2 * (rows * w + m["heads"] * m["vdim"] * w)
            head_products += 2 * m["heads"] * m["kv_rank"] * (m["dim"] + m["vdim"])
            latent_token += 2 * m["kv_rank"]
            att_flops += m["heads"] * 2 * m["kv_rank"]
        elif layer["type"] == "mamba2":
            inner = m["heads"] * m["vdim"]
            proj = 2 * inner + 2 * m["groups"] * m["state"] + m["heads"]
            products += 2 * (proj * w + inner * w)
            state_bytes += 2 * 4 * m["heads"] * m["state"] * m["vdim"]
            scan_flops += 6 * m["heads"] * m["state"] * m["vdim"]
            rec_tokens += 4 * (2 * proj + 2 * inner) + 2 * inner
        else:
            qk, inner = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            proj = 2 * qk + 2 * inner + 2 * m["heads"]
            products += 2 * (proj * w + inner * w)
            state_bytes += 2 * 4 * m["heads"] * m["dim"] * m["vdim"]
            scan_flops += 8 * m["heads"] * m["dim"] * m["vdim"]
            rec_tokens += 4 * (2 * proj + 2 * inner) + 2 * inner
        mlp = layer["mlp"]
        if mlp is None:
            continue
        norms += 1
        if mlp["kind"] == "dense":
            gated += 2 * 2 * mlp["ff"] * w
            products += 2 * mlp["ff"] * w
        else:
            r = mlp["router"]
            expert_all += 2 * 3 * r["experts"] * mlp["expert"]["ff"] * w
            expert_active += 2 * 3 * r["top"] * mlp["expert"]["ff"] * w
            router += 4 * r["experts"] * w
    t = tokens
    # a decode step reads the experts its tokens chose, at most all of them
    touched = min(expert_all, batch * expert_active)
    return {
        "decode": {"product": ("hbm", products), "gated product": ("hbm", gated),
                   "attention": ("hbm", batch * context * latent_token),
                   "head product": ("hbm", head_products),
                   "expert products": ("hbm", touched), "router": ("hbm", router),
                   "recurrence": ("hbm", batch * (state_bytes + rec_tokens)),
                   "norm": ("hbm", norms * batch * w * 14)},
        "prefill": {"product": ("tensor", t * (products - head) + head),
                    "gated product": ("tensor", t * gated),
                    "attention": ("tensor", t * t * att_flops),
                    "head product": ("tensor", t * head_products),
                    "expert products": ("tensor", t * expert_active),
                    "router": ("hbm", router + t * w * 2),
                    "recurrence": ("tensor", t * scan_flops),
                    "norm": ("hbm", norms * t * w * 14)},
    }


SISAVIK_SIZES = {
    # width, heads, unrotated and rotated query/key size, value size, key latent, query latent,
    # feed-forward, key/value heads of the sigmoid attention, window, kept first tokens
    "0.5b": (896, 14, 64, 32, 64, 96, 448, 4864, 2, 1024, 64),
    "1.5b": (1536, 12, 128, 32, 128, 96, 768, 8960, 2, 1024, 64),
}


def sisavik_config(size: str) -> dict:
    """A Sisavik model at the layer sizes of `size`: attention over a cached latent (a row of
    128 numbers with its rotated part, as Kinelix's latent has) with a query latent and a
    window, sigmoid attention beside a generalized delta rule, and two attention layers
    that read the first one's rows, twice over; every layer with a dense feed-forward."""
    width, heads, dim, rot, vdim, rank, q_rank, ff, kv_heads, window, keep = SISAVIK_SIZES[size]

    def latent(source=None):
        mixer = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
                 "q_rank": q_rank, "scale": (dim + rot) ** -0.5, "mask": {"size": window},
                 "rot": {"base": 10000.0, "dims": rot}}
        if source is not None:
            mixer["kv_from"] = source
        return mixer

    parallel = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                         "scale": dim ** -0.5, "mask": {"size": window, "keep_first": keep},
                         "rot": {"base": 10000.0, "dims": dim}},
                "right": {"heads": width // dim, "dim": dim, "decay_rank": 64},
                "left_scale": 0.5, "right_scale": 0.5}
    mlp = {"kind": "dense", "ff": ff}
    layers = []
    for base in range(0, DESIGN_LAYERS, 4):
        layers += [{"type": "latent_attention", "mixer": latent(), "mlp": mlp},
                   {"type": "parallel", "mixer": parallel, "mlp": mlp},
                   {"type": "latent_attention", "mixer": latent(base), "mlp": mlp},
                   {"type": "latent_attention", "mixer": latent(base), "mlp": mlp}]
    return {"architecture": "Sisavik", "width": width, "vocab": DESIGN_VOCAB,
            "max_positions": MODEL_LEN, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "layers": layers[:DESIGN_LAYERS]}


def seen_pairs(tokens: int, before: int, window: int, keep: int = 0) -> int:
    """How many (query, key) pairs a portion of `tokens` behind `before` cached tokens has
    under a window with kept first tokens."""
    total = 0
    for p in range(before, before + tokens):
        total += p + 1 if not window or p < window else window + min(keep, p + 1 - window)
    return total


def sisavik_costs(raw: dict, batch: int, context: int, tokens: int) -> dict:
    """Per class of kernel call, what a Sisavik model has to read (decode step, bytes) or
    compute (prompt step, flops; bytes for the classes that only move data)."""
    w, v = raw["width"], raw["vocab"]
    taps = raw["canon"]["taps"]
    products = head = 2 * v * w
    gated = head_products = att_bytes = att_flops = state_bytes = scan_flops = rec_tokens = 0
    rotary = 0
    norms = 1
    for layer in raw["layers"]:
        m = layer["mixer"]
        norms += 2                                   # the input convolution and the norm behind
        if layer["type"] == "latent_attention":
            own = m.get("kv_from") is None
            row, q_head = m["kv_rank"] + m["rot_dim"], m["dim"] + m["rot_dim"]
            rows = m["q_rank"] + (row if own else 0)
            products += 2 * (rows * w + m["heads"] * q_head * m["q_rank"] + m["heads"] * m["vdim"] * w)
            head_products += 2 * m["heads"] * row * (q_head + m["vdim"])
            reach = min(context + 1, m["mask"]["size"] or context + 1)
            att_bytes += batch * reach * 2 * row
            att_flops += m["heads"] * 4 * row * seen_pairs(tokens, 0, m["mask"]["size"])
            rotary += 4 * rows + 2 * (m["q_rank"] + (row if own else 0)) + 4 * m["heads"] * row
        else:
            left, right = m["left"], m["right"]
            qk = (left["heads"] + left["kv_heads"]) * left["dim"]
            products += 2 * (qk * w + left["heads"] * left["dim"] * w)
            mask = left["mask"]
            reach = min(context + 1, (mask["size"] + mask["keep_first"]) if mask["size"] else context + 1)
            att_bytes += batch * reach * 2 * 2 * left["kv_heads"] * left["dim"]
            att_flops += left["heads"] * 4 * left["dim"] * seen_pairs(tokens, 0, mask["size"],
                                                                      mask["keep_first"])
            rotary += 4 * qk + 2 * (left["heads"] + 2 * left["kv_heads"]) * left["dim"]
            keys = right["heads"] * right["dim"]
            proj = 5 * keys + right["decay_rank"]
            products += 2 * (proj * w + keys * right["decay_rank"] + keys * w)
            state_bytes += 2 * 4 * right["heads"] * right["dim"] * right["dim"]
            scan_flops += 10 * right["heads"] * right["dim"] * right["dim"]
            rec_tokens += 4 * (5 * keys + 2 * right["decay_rank"] + 2 * keys) + 2 * keys
        if layer["mlp"] is not None:
            norms += 2
            gated += 2 * 2 * layer["mlp"]["ff"] * w
            products += 2 * layer["mlp"]["ff"] * w
    t = tokens
    # a convolution reads the float32 stream and writes activations; a norm reads the float32
    # stream and the sublayer's output and writes the stream
    per_row = w * (4 + 2 + 4 + 2 + 4) // 2
    return {
        "decode": {"product": ("hbm", products), "gated product": ("hbm", gated),
                   "attention": ("hbm", att_bytes), "head product": ("hbm", head_products),
                   "recurrence": ("hbm", batch * (state_bytes + rec_tokens)),
                   "rotary + store": ("hbm", batch * rotary),
                   "norm": ("hbm", norms * batch * per_row)},
        "prefill": {"product": ("tensor", t * (products - head) + head),
                    "gated product": ("tensor", t * gated),
                    "attention": ("tensor", att_flops),
                    "head product": ("tensor", t * head_products),
                    "recurrence": ("tensor", t * scan_flops),
                    "rotary + store": ("hbm", t * rotary),
                    "norm": ("hbm", norms * t * per_row)},
    }


LIZAZEN_SIZES = {
    # width, query heads, key/value heads, head size, feed-forward, experts, experts a token
    # uses, window / chunk, kept first tokens
    "0.5b": (896, 14, 2, 64, 4864, 16, 4, 1024, 64),
    "1.5b": (1536, 12, 2, 128, 8960, 16, 4, 1024, 64),
}


def lizazen_config(size: str) -> dict:
    """A Lizazen model at the layer sizes of `size`: capped window attention with a dense
    feed-forward, differential attention (two maps of 64 over values of 128) with routed
    experts and a shared expert (active width: the dense feed-forward's), differential
    attention with a dense feed-forward, and chunked attention beside retention with routed
    experts, twice over."""
    width, heads, kv_heads, dim, ff, experts, top, window, keep = LIZAZEN_SIZES[size]
    moe = {"kind": "moe", "expert": {"ff": ff // top}, "router": {"experts": experts, "top": top - 1},
           "shared": {"ff": ff // top}}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    capped = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
              "softcap": 30.0, "mask": {"size": window},
              "rot": {"base": 100000.0, "dims": dim,
                      "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 4096}}}
    maps = width // 128
    differential = {"heads": maps, "kv_heads": max(1, maps // 7) if maps % 7 == 0 else 2, "dim": 64,
                    "vdim": 128, "diff": 0.5, "scale": 0.125,
                    "mask": {"size": window, "keep_first": keep}, "rot": {"base": 10000.0, "dims": 32}}
    parallel = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                         "scale": dim ** -0.5, "mask": {"size": window},
                         "rot": {"base": 10000.0, "dims": dim // 2}},
                "right": {"heads": width // 128, "dim": 64, "vdim": 128,
                          "decay": [1.0 - 2.0 ** (-5 - i % 8) for i in range(width // 128)],
                          "rot": {"base": 10000.0, "dims": 64}}}
    layers = []
    for _ in range(0, DESIGN_LAYERS, 4):
        layers += [{"type": "attention", "mixer": capped, "mlp": dense},
                   {"type": "attention_2", "mixer": differential, "mlp": moe},
                   {"type": "attention_2", "mixer": differential, "mlp": dense},
                   {"type": "parallel", "mixer": parallel, "mlp": moe}]
    return {"architecture": "Lizazen", "width": width, "vocab": DESIGN_VOCAB,
            "max_positions": MODEL_LEN, "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 31337, "mul_cur": 7}},
            "layers": layers[:DESIGN_LAYERS]}


def chunk_pairs(tokens: int, chunk: int) -> int:
    """(query, key) pairs of a prompt of `tokens` under chunks of `chunk` positions."""
    return sum(p % chunk + 1 for p in range(tokens))


def lizazen_costs(raw: dict, batch: int, context: int, tokens: int) -> dict:
    """Per class of kernel call, what a Lizazen model has to read (decode step, bytes) or
    compute (prompt step, flops; bytes for the classes that only move data)."""
    w, v = raw["width"], raw["vocab"]
    products = head = 2 * v * w
    gated = att_bytes = att_flops = state_bytes = scan_flops = rec_tokens = rotary = 0
    expert_bytes = expert_flops = router = 0
    norms = 1

    def attention(m, kind, maps=1, from_keys=False):
        nonlocal products, att_bytes, att_flops, rotary
        qk = (m["heads"] + m["kv_heads"]) * maps * m["dim"]
        values = 0 if from_keys else m["kv_heads"] * m["vdim"]
        products += 2 * ((qk + values) * w + m["heads"] * m["vdim"] * w)
        size, keep = m["mask"]["size"], m["mask"].get("keep_first", 0)
        reach = min(context + 1, size + keep) if kind == "sliding" else context % size + 1
        att_bytes += batch * reach * 2 * m["kv_heads"] * (maps * m["dim"] + m["vdim"])
        pairs = seen_pairs(tokens, 0, size, keep) if kind == "sliding" else chunk_pairs(tokens, size)
        att_flops += m["heads"] * maps * 2 * (m["dim"] + m["vdim"]) * pairs
        rotary += 4 * (qk + values) + 2 * (qk + m["kv_heads"] * m["vdim"])

    for layer in raw["layers"]:
        m = layer["mixer"]
        norms += 2
        if layer["type"] == "attention":
            attention(m, "sliding", from_keys=True)
        elif layer["type"] == "attention_2":
            attention(m, "sliding", maps=2)
        else:
            attention(m["left"], "chunked")
            right = m["right"]
            keys, inner = right["heads"] * right["dim"], right["heads"] * right["vdim"]
            products += 2 * ((2 * keys + 2 * inner) * w + inner * w)
            state_bytes += 2 * 4 * right["heads"] * right["dim"] * right["vdim"]
            scan_flops += 4 * right["heads"] * right["dim"] * right["vdim"]
            rec_tokens += 4 * (2 * keys + 2 * inner) + 4 * inner + 2 * inner
        mlp = layer["mlp"]
        if mlp is None:
            continue
        norms += 2
        if mlp["kind"] == "dense":
            gated += 2 * 2 * mlp["ff"] * w
            products += 2 * mlp["ff"] * w
        else:
            experts, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            router += 4 * experts * w
            per_expert = 2 * 3 * ff * w
            expert_bytes += min(experts, batch * top) * per_expert
            expert_flops += top * per_expert
            if mlp.get("shared"):
                gated += 2 * 2 * mlp["shared"]["ff"] * w
                products += 2 * mlp["shared"]["ff"] * w
    t = tokens
    per_row = w * (4 + 2 + 4 + 2 + 4) // 2
    return {
        "decode": {"product": ("hbm", products), "gated product": ("hbm", gated),
                   "attention": ("hbm", att_bytes), "expert products": ("hbm", expert_bytes),
                   "router": ("hbm", router),
                   "recurrence": ("hbm", batch * (state_bytes + rec_tokens)),
                   "rotary + store": ("hbm", batch * rotary),
                   "norm": ("hbm", norms * batch * per_row)},
        "prefill": {"product": ("tensor", t * (products - head) + head),
                    "gated product": ("tensor", t * gated),
                    "attention": ("tensor", att_flops),
                    "expert products": ("tensor", t * expert_flops),
                    "recurrence": ("tensor", t * scan_flops),
                    "rotary + store": ("hbm", t * rotary),
                    "norm": ("hbm", norms * t * per_row)},
    }


def classes_of(torch, runner, batch, context, vocab, costs, peak) -> dict:
    """Milliseconds per class of kernel call of a decode step and of a prompt step (events
    around every call, the launches queued behind a delay on the device), with the fraction
    of the measured peak where `costs` names what the class has to do."""
    from mercury_b200.engine.batch import StepEntry

    seqs = fill_contexts(torch, runner, batch, context, vocab)
    gen = torch.Generator().manual_seed(SEED + 6)
    tokens = torch.randint(0, vocab, (4, batch), generator=gen).tolist()
    prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
    runner.time_kernels = True
    try:
        rows = []
        for turn in range(4):
            torch.cuda._sleep(20_000_000)
            runner.step([StepEntry(s, [tokens[turn][i]], [0]) for i, s in enumerate(seqs)])
            rows.append(dict(runner.last_kernel_ms))
        decode = {k: statistics.median(r.get(k, 0.0) for r in rows[2:]) for k in rows[-1]}
        for s in seqs:
            runner.close(s)
        rows = []
        for turn in range(3):
            seq = runner.open(f"classes-{turn}")
            torch.cuda._sleep(40_000_000)
            runner.step([StepEntry(seq, prompt, [PREFILL_TOKENS - 1])])
            rows.append(dict(runner.last_kernel_ms))
            runner.close(seq)
        prefill = {k: statistics.median(r.get(k, 0.0) for r in rows[1:]) for k in rows[-1]}
    finally:
        runner.time_kernels = False
    out = {}
    for name, measured in (("decode", decode), ("prefill", prefill)):
        block = {}
        for kind, ms in sorted(measured.items()):
            bound, amount = costs[name].get(kind, ("hbm", 0))
            top = peak["hbm_gbs"] * 1e9 if bound == "hbm" else peak["bf16_tflops"] * 1e12
            block[kind] = {"ms": round(ms, 4), "bound": bound,
                           "frac": round(amount / (ms * 1e-3) / top, 4) if ms > 0 and amount else None}
        block["sum_ms"] = round(sum(measured.values()), 4)
        out[name] = block
    return out


def run_designs(args) -> dict:
    """`--only designs`: prefill and decode throughput of Fegenex at a few layer sizes of
    real models (random weights, 8 layers), beside Qwen2 at the same sizes, with every
    class of kernel call against its roofline."""
    import torch

    from mercury_b200.config import config_from_dict
    from mercury_b200.weights import random_tensors

    peak, peak_kind = peaks()
    out = {"workload": f"{DESIGN_LAYERS} layers, vocabulary {DESIGN_VOCAB}, decode batch {args.batch} "
                       f"at {CONTEXT}-token contexts, prompt of {PREFILL_TOKENS} tokens, bfloat16",
           "peaks": peak_kind, "sizes": {}}
    for size in ([args.size] if args.size_given else list(DESIGN_SIZES)):
        row = {}
        fegenex, qwen2 = design_configs(size)
        # the design asked for, beside the closest models this engine has at the same sizes
        models = ((("fegenex", fegenex), ("qwen2", qwen2)) if args.design == "fegenex" else
                  (("kinelix", kinelix_config(size)), ("fegenex", fegenex), ("qwen2", qwen2))
                  if args.design == "kinelix" else
                  (("sisavik", sisavik_config(size)), ("kinelix", kinelix_config(size)),
                   ("qwen2", qwen2)) if args.design == "sisavik" else
                  (("lizazen", lizazen_config(size)), ("sisavik", sisavik_config(size)),
                   ("kinelix", kinelix_config(size)), ("qwen2", qwen2)))
        for label, raw in models:
            _entry, config = config_from_dict(raw)
            tensors = random_tensors(config, SEED, torch.bfloat16)
            vocab = DESIGN_VOCAB
            batch = args.batch
            runner = make_runner(torch, config, tensors, max(batch, 2),
                                 max(batch, 2) * (CONTEXT + 256), graphs=not args.no_graphs)
            prefill_ms = prefill_rate(torch, runner, vocab)
            rate, ms, launches, _ = decode_rate(torch, runner, batch, CONTEXT, vocab, args.steps,
                                                max(3, args.warmup))
            costs = (design_costs(raw, batch, CONTEXT, PREFILL_TOKENS) if label == "fegenex"
                     else kinelix_costs(raw, batch, CONTEXT, PREFILL_TOKENS) if label == "kinelix"
                     else sisavik_costs(raw, batch, CONTEXT, PREFILL_TOKENS) if label == "sisavik"
                     else lizazen_costs(raw, batch, CONTEXT, PREFILL_TOKENS) if label == "lizazen"
                     else class_costs(raw, batch, CONTEXT, PREFILL_TOKENS))
            row[label] = {"prefill_ms": round(prefill_ms, 3),
                          "prefill_tokens_per_s": round(PREFILL_TOKENS / prefill_ms * 1e3, 1),
                          "decode_ms_per_step": round(ms, 4), "decode_tokens_per_s": round(rate, 1),
                          "launches_per_decode_step": launches,
                          "classes": classes_of(torch, runner, batch, CONTEXT, vocab, costs, peak)}
            del runner, tensors
            torch.cuda.empty_cache()
        out["sizes"][size] = row
    return out



def run_mixed(args, prepared=None) -> dict:
    """`--only mixed`: 32 requests through Engine.generate, prompt lengths uniform in
    [64, 2048], half of them sharing one 512-token prefix, 128 greedy tokens each (the
    benchmark description's serving workload, by default at Qwen2.5-1.5B sizes)."""
    import torch

    from mercury_b200 import Engine, EngineConfig, SamplingParams
    from mercury_b200.config import config_from_dict
    from mercury_b200.engine.runner import ModelRunner
    from mercury_b200.weights import random_tensors

    raw = SIZES[args.size]
    if prepared is None:
        _entry, config = config_from_dict(raw)
        tensors = random_tensors(config, SEED, torch.bfloat16)
    else:
        config, tensors = prepared
    gen = torch.Generator().manual_seed(SEED + 5)
    shared = torch.randint(0, raw["vocab_size"], (512,), generator=gen).tolist()
    prompts = []
    for i in range(32):
        n = int(torch.randint(64, 2049, (1,), generator=gen))
        body = torch.randint(0, raw["vocab_size"], (n,), generator=gen).tolist()
        prompts.append((shared + body[512:]) if (i % 2 == 0 and n > 512) else body)
    pool_tokens = 32 * (2048 + 128 + BLOCK)
    runner = ModelRunner(config=config, tensors=tensors, dtype=torch.bfloat16, device="cuda",
                         page_size=BLOCK, num_pages=pool_tokens // BLOCK, max_seqs=32,
                         max_step_tokens=4096, max_model_len=MODEL_LEN)
    cfg = EngineConfig(model="(in memory)", dtype="bfloat16", block_size=BLOCK,
                       num_blocks=pool_tokens // BLOCK, max_running=32, max_batched_tokens=4096,
                       prefill_chunk=2048, max_model_len=MODEL_LEN, policy=args.policy, seed=SEED)
    engine = Engine(cfg, runner=runner)
    engine.generate([prompts[0][:64]], SamplingParams(ignore_eos=True), 4)      # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, SamplingParams(ignore_eos=True), 128)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    produced = sum(len(o) for o in outs)
    snap = engine.snapshot()
    return {"workload": "mixed: 32 requests, prompts 64..2048, 16 share a 512-token prefix, 128 tokens each",
            "size": args.size, "policy": args.policy, "output_tokens": produced,
            "prompt_tokens": sum(len(p) for p in prompts), "seconds": round(seconds, 3),
            "output_tokens_per_s": round(produced / seconds, 1),
            "prefix_hit_tokens": snap["cache"]["hit_tokens"], "steps": snap["engine"]["steps"],
            "preemptions": snap["scheduler"]["preemptions"], "leaked_pages": engine.leaked_pages()}


def run_reference(args) -> dict:
    """The unmodified reference (installed under baseline/_ref) on the same model folder,
    batch and context, through its own Engine.submit/step."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "mercury").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed on this box"}
    try:
        import torch

        from mercury_b200.config import config_from_dict
        from mercury_b200.weights import write_random_model

        sys.path.insert(0, str(ref))
        from mercury.config import EngineConfig as RefConfig
        from mercury.engine import Engine as RefEngine
        from mercury.request import SamplingParams as RefParams
    except Exception as err:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"import failed: {type(err).__name__}: {err}"}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device on this box"}
    try:
        return _time_reference(args, torch, config_from_dict, write_random_model, RefConfig,
                               RefEngine, RefParams)
    except Exception as err:  # noqa: BLE001
        return {"impl": "reference",
                "unavailable": " ".join(f"the reference failed while running: "
                                        f"{type(err).__name__}: {err}".split())[:300]}


def _time_reference(args, torch, config_from_dict, write_random_model, RefConfig, RefEngine,
                    RefParams) -> dict:
    _entry, config = config_from_dict(QWEN25_05B)
    vocab = QWEN25_05B["vocab_size"]
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(Path(tmp) / "model", config, SEED)
        cfg = RefConfig(model=str(folder), device="cuda", dtype="bfloat16", block_size=BLOCK,
                        num_blocks=BATCH * (CONTEXT + 256) // BLOCK, max_running=BATCH,
                        max_model_len=MODEL_LEN, prefill_budget=BATCH * CONTEXT, seed=SEED)
        engine = RefEngine(cfg)
        gen = torch.Generator().manual_seed(SEED + 4)
        produced = []
        for b in range(BATCH):
            prompt = torch.randint(0, vocab, (CONTEXT,), generator=gen).tolist()
            engine.submit(f"ref-{b}", prompt, args.steps + args.warmup + 8,
                          lambda ev: produced.append(ev.kind), RefParams(ignore_eos=True))
        engine.step()                       # admits and prefills every prompt
        for _ in range(args.warmup):
            engine.step()
        sampler = ClockSampler()
        sampler.start()
        torch.cuda.synchronize()
        before = len(produced)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            engine.step()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        clocks = sampler.stop()
        tokens = sum(1 for kind in produced[before:] if kind == "token")
    rate = round(tokens / seconds, 1)
    return {"impl": "reference", "metric": METRIC,
            "value": rate, "unit": "tokens/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(1e3 * seconds / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random N(0,0.02) weights",
            "config": bench_config(peaks()[1]),
            # the reference has no device-timed number: its only clock is the wall clock around
            # its own Engine.step, host tokens in and out, which is an end-to-end number by
            # nature; the bytes it copies per step are its own business and not counted here
            "timing": "wall clock around Engine.step, host tokens in and out",
            "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": None,
                    "d2h_bytes_per_step": None},
            "clocks": clocks}


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="mercury_b200", choices=("mercury_b200", "reference"))
    p.add_argument("--only", default="all",
                   choices=("all", "decode", "prefill", "products", "mixed", "kernels", "designs"),
                   help="run one part only (for profilers and side workloads); prints its own JSON")
    p.add_argument("--size", default=None, choices=tuple(SIZES),
                   help="layer sizes of --only decode/prefill/mixed (default 0.5b; mixed: 1.5b)")
    p.add_argument("--design", default="fegenex", choices=("fegenex", "kinelix", "sisavik", "lizazen"),
                   help="which design --only designs measures beside the closest existing models")
    p.add_argument("--policy", default="lpm", choices=("fcfs", "lpm", "lpm_aging"))
    p.add_argument("--batch", type=int, default=BATCH, help="decode batch of --only decode")
    p.add_argument("--no-graphs", action="store_true", help="launch kernels one by one")
    p.add_argument("--no-sizes", action="store_true",
                   help="leave the 1.5B and 7B side workloads out of the full run (about a minute)")
    p.add_argument("--gemm", default=None, choices=("library", "tcgen05", "auto"),
                   help="many-token product of --only prefill/decode (default: the engine's)")
    args = p.parse_args()
    if args.gpus != 1:
        print("bench.py measures a single-GPU engine; --gpus must be 1", flush=True)
        return 2
    args.size_given = args.size is not None
    if args.size is None:
        args.size = "1.5b" if args.only == "mixed" else "0.5b"
    if args.only != "all":
        print(json.dumps(run_part(args)), flush=True)
        return 0
    args.warmup = max(3, args.warmup)
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
