"""Lizazen through the engine's step function, cache and state manager on the CPU (PyTorch
kernel twins) against the plain implementation: each mechanism alone, every layer kind alone,
whole prompts, prompts cut into portions down to two tokens, decoding token by token, mixed
batches with pages and state slots used again, and greedy generation through the engine."""

from __future__ import annotations

import pytest
import torch

import lizazen_mechanisms
import plain_lizazen
import replay_cases
from kernel_twins import TorchOps
from lizazen_cases import RAW, lizazen_model, make_runner, replay_and_compare, requests_for

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 100, 41), "odd": (50, 7, 121, 33),
           "wide": (40, 110)}


@pytest.mark.parametrize("check", lizazen_mechanisms.ALL, ids=lambda f: f.__name__[6:])
def test_mechanism(check):
    check(TorchOps(), "cpu", torch.float32)


@pytest.mark.parametrize("name", ["only_capped", "only_differential", "only_parallel"])
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


def test_decoding_far_beyond_every_window_and_chunk():
    """Windows and chunks pass over decoded tokens: pages behind them go back to the pool while
    the kept first tokens' pages stay, and the pool is smaller than the request is long."""
    name, lengths = "mix", (20, 150)
    steps, rows = replay_cases.decode_tail(requests_for(name, lengths), tail=120)
    runner = make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=192)
    replay_and_compare(runner, name, lengths, steps, rows, 3e-5)


def test_config_round_trip_and_refusals():
    from mercury_b200.config import ConfigError, config_from_dict

    entry, config = config_from_dict(RAW["mix"])
    assert entry.name == "Lizazen" and config.to_dict() == RAW["mix"]
    assert config_from_dict(config.to_dict())[1] == config
    assert config_from_dict(RAW["ones"])[1].bigram is None

    def broken(change):
        raw = config.to_dict()
        change(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)

    broken(lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3))   # 4 heads over 3
    broken(lambda r: r["layers"][2]["mixer"].update(vdim=16))              # values are the keys
    broken(lambda r: r["layers"][0].update(type="lstm"))
    broken(lambda r: r["layers"][0]["mixer"]["right"].update(decay=[0.5]))  # a decay per head
    broken(lambda r: r["layers"][1]["mixer"]["rot"].update(dims=10))       # beyond the head
    broken(lambda r: r["layers"][1]["mixer"].pop("diff"))
    broken(lambda r: r["layers"][1]["mlp"].update(kind="sparse"))
    broken(lambda r: r["layers"][1]["mlp"].update(limit=0.0))
    broken(lambda r: r["layers"][0]["mlp"]["router"].update(top=6))        # of five experts
    broken(lambda r: r["layers"][2]["mixer"]["mask"].update(size=0))
    broken(lambda r: r["embedding"]["bigram"].update(buckets=0))


def test_layout_of_caches_and_state():
    from mercury_b200.config import architecture_named
    from mercury_b200.models.model import Model

    _raw, config, _tensors = lizazen_model("mix")
    spec = architecture_named("Lizazen").describe(config)
    model = Model(spec)
    names = {s.name for s in model.tensor_specs()}
    assert {"bigram", "l0.mix.left.q.b", "l0.mix.left.v.b", "l0.mix.right.g", "l0.mix.left.out",
            "l0.mlp.e4.down", "l0.mlp.shared.up", "l0.mlp.router", "l1.mix.lq2", "l2.mix.k.norm",
            "l2.mix.sink", "l2.mix.o.b", "l2.norm1b"} <= names
    assert not {"l2.mix.v", "l1.mix.q.b", "l1.mix.sink", "l2.norm2", "l3.mlp.shared.up",
                "l0.mlp.correction", "l0.mix.right.q.b"} & names
    # a cache layer per layer; windows, kept first tokens and chunks decide the groups
    assert sorted(zip(model.group_windows, model.group_keeps)) == [(9, 0), (19, 5), (21, 0), (33, 0),
                                                                   (37, 0), (40, 18)]
    need = {c: l.need for c, l in model.cache_layers.items()}
    assert (need[1].head_dim, need[1].value_head_dim) == (16, 24)       # two maps of 8 side by side
    assert (need[2].head_dim, need[2].value_head_dim) == (8, 8)
    assert not model.skips_cached_prefix          # state of its own: every token has to be run
    # the matrices of the two retention layers and the last token of the embedding
    assert sorted(model.state_needs) == [(-1, 0), (0, 1), (5, 1)]
    assert model.state_needs[(0, 1)].shape == (3 * 16 * 8,)
    assert Model(architecture_named("Lizazen").describe(lizazen_model("ones")[1])).state_needs.keys() \
        == {(2, 1), (3, 1)}


def greedy(raw, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits = plain_lizazen.forward(raw, tensors, tokens)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]


def test_greedy_generation_through_the_engine():
    from mercury_b200 import Engine, EngineConfig, SamplingParams

    name = "mix"
    raw, config, tensors = lizazen_model(name)
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
    raw, config, tensors = lizazen_model(name)
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
