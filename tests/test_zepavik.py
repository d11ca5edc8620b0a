"""The Zepavik decoder off the GPU: its configuration and description as parts, the engine's bookkeeping for it
(the embedding's per-sequence state, cache groups per window, the parallel layer) with the torch stand-in for
the kernels, and that the plain implementation the GPU tests compare with can tell a fault from rounding."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_zepavik
from helpers import random_tokens
from ops_double import double_loader
from zepavik_models import ZEPAVIK, make_folder
from stratakv_b200 import EngineConfig, StepEntry
from stratakv_b200.config import ConfigError, ZepavikConfig, load_config
from stratakv_b200.engine.engine import Engine
from stratakv_b200.engine.model import cache_requests, expected_tensors
from stratakv_b200.weights import load_checkpoint


def test_config_round_trip_and_what_it_refuses(tmp_path):
    for raw in ZEPAVIK.values():
        typed = ZepavikConfig.from_dict(raw)
        assert typed.to_dict() == raw
    (tmp_path / "config.json").write_text(json.dumps(ZEPAVIK["ZB"]))
    arch, typed = load_config(tmp_path)
    assert arch.name == "Zepavik" and typed.layers[1].window == 130 and typed.layers[2].window == 0
    assert typed.layers[0].ff == 100 and typed.bigram.buckets == 1 and typed.logit_scale == 0.5
    for path, value, message in ((("layers", 0, "type"), "recurrent", "not a mixer"),
                                 (("layers", 0, "mixer", "kv_heads"), 4, "multiple"),
                                 (("layers", 1, "mlp", "kind"), "routed", "not a feed-forward"),
                                 (("layers", 0, "mixer", "dim"), 0, "positive"),
                                 (("vocab",), None, "missing"), (("norm",), None, "missing")):
        raw = copy.deepcopy(ZEPAVIK["ZB"])
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=message):
            ZepavikConfig.from_dict(raw)


def test_description_names_the_checkpoint_tensors_and_groups_the_cache():
    from stratakv_b200.models.zepavik import zepavik_spec
    spec = zepavik_spec(ZepavikConfig.from_dict(ZEPAVIK["ZB"]))
    shapes = {name: tuple(request.shape) for name, request in expected_tensors(spec).items()}
    assert shapes["embed"] == (131, 72) and shapes["bigram"] == (2, 72) and shapes["pos"] == (512, 72)
    assert shapes["l0.mix.q"] == (120, 72) and shapes["l0.mix.k"] == (40, 72) and shapes["l0.mix.v"] == (24, 72)
    assert shapes["l0.mix.q.b"] == (120,) and shapes["l0.mix.v.b"] == (24,) and shapes["l0.mix.o"] == (72, 72)
    assert shapes["l1.mix.o"] == (72, 120) and shapes["l1.mix.g"] == (3, 72) and shapes["l1.mix.r1"] == (3,)
    assert shapes["l2.mlp.up"] == (8, 72) and shapes["l2.mlp.down"] == (72, 8) and shapes["head"] == (131, 72)
    assert "l0.norm2" not in shapes and shapes["final.norm"] == (72,)
    no_mlp = zepavik_spec(ZepavikConfig.from_dict(ZEPAVIK["ZA"]))
    assert not any(name.startswith("l1.mlp") for name in expected_tensors(no_mlp))
    requests = cache_requests(spec)
    assert [r.kind for r in requests] == ["kv_window", "kv_window", "kv", "none"]
    assert (requests[0].head_dim, requests[0].v_head_dim, requests[0].window) == (20, 12, 7)
    assert requests[2].v_head_dim == 0 and requests[3].state_bytes == 8          # the embedding's two last ids
    assert spec.positions_are_tabled and spec.head.logit_scale == 0.5


def cpu_engine(folder, max_tokens=512, block_size=16, max_batch=0):
    arch, config = load_config(folder)
    spec = arch.build_spec(config)
    tensors = load_checkpoint(folder, {n: r.shape for n, r in expected_tensors(spec).items()}, spec.ignorable)
    return Engine(spec, tensors, EngineConfig(max_tokens=max_tokens, dtype="float32", device="cpu", block_size=block_size,
                                              max_batch=max_batch), kernel_loader=double_loader())


@pytest.mark.parametrize("name", ["ZA", "ZB"])
def test_bookkeeping_portions_batches_and_slots_used_again(tmp_path, name):
    folder = make_folder(tmp_path / name, ZEPAVIK[name], seed=3)
    config, weights = plain_zepavik.load_folder(folder)
    engine = cpu_engine(folder, max_tokens=16 * 14, max_batch=3)
    vocab = ZEPAVIK[name]["vocab"]
    for round_ in range(2):                                   # the second round takes the slots and pages of the first
        prompts = [random_tokens(vocab, n, seed=10 * round_ + n) for n in (5, 40, 18)]
        refs = [plain_zepavik.logits_of(config, weights, p).numpy() for p in prompts]
        slots = [engine.open_sequence() for _ in prompts]
        cut = [1, 20, 17]
        got = engine.step([StepEntry(s, p[:c], list(range(c))) for s, p, c in zip(slots, prompts, cut)])
        np.testing.assert_allclose(got.numpy(), np.concatenate([r[:c] for r, c in zip(refs, cut)]), rtol=1e-4, atol=2e-5)
        got = engine.step([StepEntry(slots[0], prompts[0][1:], [3]), StepEntry(slots[1], prompts[1][20:22], [0, 1]),
                           StepEntry(slots[2], prompts[2][17:], [0])])
        np.testing.assert_allclose(got.numpy(), np.stack([refs[0][4], refs[1][20], refs[1][21], refs[2][17]]), rtol=1e-4, atol=2e-5)
        engine.close_sequence(slots[0]); engine.close_sequence(slots[2])
        for position in range(22, 40):                        # past the window of 7 (ZB) and over page borders
            got = engine.step([StepEntry(slots[1], [prompts[1][position]], [0])])
            np.testing.assert_allclose(got.numpy()[0], refs[1][position], rtol=1e-4, atol=2e-5)
        engine.close_sequence(slots[1])
        assert engine.cache.all_free()


def test_a_window_gives_its_pages_back_while_the_sequence_runs(tmp_path):
    folder = make_folder(tmp_path / "ZB", ZEPAVIK["ZB"], seed=3)
    engine = cpu_engine(folder, max_tokens=16 * 12, max_batch=1)
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, random_tokens(131, 100, seed=1), [])])
    record = engine.cache.sequences[slot]
    groups = {group.request.window: group.index for group in engine.cache.groups}
    assert len(record.blocks[groups[7]]) == 2 and record.dropped[groups[7]] == 5      # positions 94.. are live
    assert len(record.blocks[groups[130]]) == 7 and len(record.blocks[groups[0]]) == 7
    engine.close_sequence(slot)
    assert engine.cache.all_free()


def test_the_plain_implementation_tells_faults_from_rounding(tmp_path):
    """Each fault that the GPU tests are there to catch moves the plain logits by far more than they allow."""
    name = "ZA"
    folder = make_folder(tmp_path / name, ZEPAVIK[name], seed=5)
    config, weights = plain_zepavik.load_folder(folder)
    tokens = random_tokens(ZEPAVIK[name]["vocab"], 90, seed=2)
    right = plain_zepavik.logits_of(config, weights, tokens).numpy()
    allowed = 0.06 * right.std()             # what tests/test_zepavik_gpu.py allows a position in bfloat16

    def moved(change):
        """The most a position's logits move, root mean square over the vocabulary."""
        other_config, other_weights = copy.deepcopy(config), dict(weights)
        change(other_config, other_weights)
        difference = plain_zepavik.logits_of(other_config, other_weights, tokens).numpy() - right
        return np.sqrt((difference ** 2).mean(axis=-1)).max()

    def window_off_by_one(c, w): c["layers"][0]["mixer"]["mask"]["size"] += 1
    def no_distance_bias(c, w): w["l0.mix.r1"] = torch.zeros_like(w["l0.mix.r1"])
    def no_query_bias(c, w): w["l1.mix.q.b"] = torch.zeros_like(w["l1.mix.q.b"])
    def no_value_bias(c, w): w["l0.mix.v.b"] = torch.zeros_like(w["l0.mix.v.b"])
    def no_gate(c, w): w["l0.mix.g"] = torch.zeros_like(w["l0.mix.g"])
    def other_pair_hash(c, w): c["embedding"]["bigram"]["mul_prev"] += 1
    def shifted_positions(c, w): w["pos"] = torch.roll(w["pos"], 1, dims=0)
    for change in (window_off_by_one, no_distance_bias, no_query_bias, no_value_bias, no_gate, other_pair_hash, shifted_positions):
        assert moved(change) > 2 * allowed, change.__name__
    # (a bias on the keys adds the same number to all of a query's scores and cancels in the softmax)
    # the value norm: without it the values keep their own length
    v = torch.randn(5, 2, 16, dtype=torch.float64) * 3
    assert torch.allclose((plain_zepavik.rms_divide(v, 0.0) ** 2).mean(-1), torch.ones(5, 2, dtype=torch.float64))
    # first token reads the last row; rows repeat with the hash
    assert plain_zepavik.pair_rows([4, 9, 4, 9], 13, 31, 7) == [13, (4 * 31 + 9 * 7) % 13, (9 * 31 + 4 * 7) % 13, (4 * 31 + 9 * 7) % 13]
    seen = plain_zepavik.visible(6, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True] and seen[1].tolist() == [True, True] + [False] * 4
