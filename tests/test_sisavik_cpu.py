"""Sisavik through the engine's step function, cache and state manager on the CPU (PyTorch
kernel twins) against the plain implementation: each mechanism alone, every layer kind alone,
whole prompts, prompts cut into portions down to two tokens, decoding token by token, mixed
batches with pages and state slots used again, and greedy generation through the engine."""

from __future__ import annotations

import pytest
import torch

import plain_sisavik
import replay_cases
import sisavik_mechanisms
from kernel_twins import TorchOps
from sisavik_cases import RAW, make_runner, replay_and_compare, requests_for, sisavik_model

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 100, 41), "odd": (50, 7, 121, 33),
           "wide": (40, 110)}


@pytest.mark.parametrize("check", sisavik_mechanisms.ALL, ids=lambda f: f.__name__[6:])
def test_mechanism(check):
    check(TorchOps(), "cpu", torch.float32)


def test_a_reader_looks_further_back_than_the_layer_that_caches():
    sisavik_mechanisms.check_latent_attention(TorchOps(), "cpu", torch.float32, own_window=19, cache_window=44)


@pytest.mark.parametrize("name", ["only_latent", "only_parallel", "one_tap"])
def test_each_layer_kind_alone(name):
    lengths = (1, 2, 60)
    requests = requests_for(name, lengths)
    for builder in (replay_cases.whole, replay_cases.portions):
        steps, rows = builder(requests)
        replay_and_compare(make_runner(name, TorchOps(), "cpu", torch.float32), name, lengths,
                           steps, rows, 3e-5)


@pytest.mark.parametrize("name", ["mix", "ones", "odd", "wide"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay(name, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 320, seed=5) if mode == "mixed" else builder(requests)
    replay_and_compare(make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=320),
                       name, lengths, steps, rows, 3e-5)


def test_decoding_far_beyond_every_window():
    """A window passes over decoded tokens: pages behind it go back to the pool while the kept
    first tokens' pages stay, and the pool is smaller than the request is long."""
    name, lengths = "mix", (20, 150)
    steps, rows = replay_cases.decode_tail(requests_for(name, lengths), tail=120)
    runner = make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=192)
    replay_and_compare(runner, name, lengths, steps, rows, 3e-5)


def test_config_round_trip_and_refusals():
    from mercury_b200.config import ConfigError, config_from_dict

    entry, config = config_from_dict(RAW["mix"])
    assert entry.name == "Sisavik" and config.to_dict() == RAW["mix"]
    assert config_from_dict(config.to_dict())[1] == config

    def broken(change):
        raw = config.to_dict()
        change(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)

    broken(lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3))   # 4 heads over 3
    broken(lambda r: r["layers"][0]["mixer"]["left"].update(vdim=8))       # values are the keys
    broken(lambda r: r["layers"][0].update(type="lstm"))
    broken(lambda r: r["layers"][2]["mixer"].update(kv_from=0))            # not a latent layer
    broken(lambda r: r["layers"][2]["mixer"].update(kv_from=3))            # a later layer
    broken(lambda r: r["layers"][5]["mixer"].update(kv_from=2))            # a reader, no latent of its own
    broken(lambda r: r["layers"][2]["mixer"].update(kv_rank=16))           # another rank than its source
    broken(lambda r: r["layers"][1]["mixer"]["rot"].update(dims=4))        # not the rotated part's size
    broken(lambda r: r["layers"][1]["mlp"].update(kind="sparse"))
    broken(lambda r: r["canon"].update(taps=0))


def test_sizes_that_only_tensors_give(tmp_path):
    """The rows of the decay map's first matrix are not in config.json: a model folder's
    tensors give them."""
    import copy
    import json

    from safetensors.torch import save_file

    from mercury_b200.config import read_model_config

    raw, _config, tensors = sisavik_model("only_parallel")
    bare = copy.deepcopy(raw)
    del bare["layers"][0]["mixer"]["right"]["decay_rank"]
    (tmp_path / "config.json").write_text(json.dumps(bare))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    _entry, config = read_model_config(tmp_path)
    assert config.layers[0]["mixer"]["right"]["decay_rank"] == raw["layers"][0]["mixer"]["right"]["decay_rank"]


def test_layout_of_caches_and_state():
    from mercury_b200.config import architecture_named
    from mercury_b200.models.model import Model

    _raw, config, _tensors = sisavik_model("mix")
    spec = architecture_named("Sisavik").describe(config)
    model = Model(spec)
    names = {s.name for s in model.tensor_specs()}
    assert "l1.mix.dkv" in names and "l2.mix.dkv" not in names and "l2.mix.uk" in names
    assert "l0.mix.left.q.b" in names and "l0.mix.left.v" not in names and "l0.mix.right.w1" in names
    assert "l2.canon1" in names and "l2.canon2" not in names and "l2.norm2" not in names
    assert spec.schedule[2].cache == spec.schedule[1].cache and not spec.schedule[2].writes_cache
    assert spec.schedule[6].cache == spec.schedule[3].cache != spec.schedule[1].cache
    # the first latent keeps the widest window of its three readers; the kept first tokens of
    # the two sigmoid-attention layers make groups of their own
    latents = [l for l in model.cache_layers.values() if l.need.shared_values]
    assert sorted(l.need.window for l in latents) == [37, 50]
    assert sorted(zip(model.group_windows, model.group_keeps)) == [(21, 5), (37, 0), (40, 18), (50, 0)]
    assert not model.skips_cached_prefix          # state of its own: every token has to be run
    # per layer: the delta rule's matrices (parallel layers) and a ring per convolution
    assert len(model.state_needs) == 2 + 7 + 5


def greedy(raw, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits = plain_sisavik.forward(raw, tensors, tokens)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]


def test_greedy_generation_through_the_engine():
    from mercury_b200 import Engine, EngineConfig, SamplingParams

    name = "mix"
    raw, config, tensors = sisavik_model(name)
    runner = make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=256, poison=False)
    cfg = EngineConfig(model="(memory)", device="cpu", dtype="float32", block_size=16, num_blocks=16,
                       max_running=4, max_batched_tokens=256, prefill_chunk=24, max_model_len=256,
                       debug_invariants=True)
    engine = Engine(cfg, runner=runner)
    prompts = [requests_for(name, (37, 70, 20))[f"r{i}"] for i in range(3)]
    outs = engine.generate(prompts, SamplingParams(), 6)
    for prompt, out in zip(prompts, outs):
        assert out == greedy(raw, tensors, prompt, 6)
    assert engine.leaked_pages() == 0


def test_preempted_requests_start_again_from_an_empty_state():
    """A pool too small for all requests at once: the newest is put back (its pages and its
    state slot given up) and recomputed later in a slot that another request has used."""
    from mercury_b200 import Engine, EngineConfig, SamplingParams

    name = "odd"
    raw, config, tensors = sisavik_model(name)
    runner = make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=160, poison=True)
    cfg = EngineConfig(model="(memory)", device="cpu", dtype="float32", block_size=16, num_blocks=10,
                       max_running=4, max_batched_tokens=160, prefill_chunk=32, max_model_len=160,
                       debug_invariants=True)
    engine = Engine(cfg, runner=runner)
    prompts = [requests_for(name, (33, 64, 41, 50))[f"r{i}"] for i in range(4)]
    outs = engine.generate(prompts, SamplingParams(), 12)
    for prompt, out in zip(prompts, outs):
        assert out == greedy(raw, tensors, prompt, 12)
    assert engine.snapshot()["scheduler"]["preemptions"] > 0
    assert engine.leaked_pages() == 0
