"""The Povusun decoder off the GPU: its configuration and description as parts, the engine's bookkeeping for it
(recurrent state per slot, a latent cache, borrowed keys, the sandwich layer) with the torch stand-in for the
kernels, and that the plain implementation the GPU tests compare with can tell a fault from rounding."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_povusun
from helpers import random_tokens
from ops_double import double_loader
from povusun_models import POVUSUN, make_folder
from stratakv_b200 import EngineConfig, StepEntry
from stratakv_b200.config import ConfigError, PovusunConfig, load_config
from stratakv_b200.engine.engine import Engine
from stratakv_b200.engine.model import cache_requests, expected_tensors
from stratakv_b200.weights import load_checkpoint


def test_config_round_trip_and_what_it_refuses(tmp_path):
    for raw in POVUSUN.values():
        assert PovusunConfig.from_dict(raw).to_dict() == raw
    (tmp_path / "config.json").write_text(json.dumps(POVUSUN["PA"]))
    arch, typed = load_config(tmp_path)
    assert arch.name == "Povusun" and [layer.type for layer in typed.layers] == ["rglru", "attention", "latent_attention", "attention"]
    assert typed.layers[3].kv_from == 1 and typed.layers[1].softcap == 6.0 and typed.layers[3].softcap == 0.0
    assert typed.layers[2].mlp is None and typed.layers[0].mlp.limit == 0.5 and typed.side_dim == 8
    for path, value, message in ((("layers", 0, "type"), "convolution", "not a mixer"),
                                 (("layers", 1, "mixer", "kv_heads"), 3, "multiple"),
                                 (("layers", 1, "mlp", "kind"), "routed", "not a feed-forward"),
                                 (("layers", 0, "mixer", "blocks"), 5, "multiple"),
                                 (("layers", 3, "mixer", "kv_from"), 2, "no keys and values"),
                                 (("layers", 3, "mixer", "kv_from"), 3, "earlier layer"),
                                 (("layers", 3, "mixer", "vdim"), 16, "differs"),
                                 (("layers", 1, "mlp", "limit"), 0.0, "positive"),
                                 (("layers", 1, "mixer", "q_temp", "every"), 0, "positive"),
                                 (("vocab",), None, "missing"), (("norm",), None, "missing")):
        raw = copy.deepcopy(POVUSUN["PA"])
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=message):
            PovusunConfig.from_dict(raw)


def test_description_names_the_checkpoint_tensors_and_the_cache():
    from stratakv_b200.models.povusun import povusun_spec
    spec = povusun_spec(PovusunConfig.from_dict(POVUSUN["PA"]))
    shapes = {name: tuple(request.shape) for name, request in expected_tensors(spec).items()}
    assert shapes["embed"] == (97, 64) and shapes["side.embed"] == (97, 32) and "head" not in shapes
    assert shapes["l0.mix.y"] == (48, 64) and shapes["l0.mix.conv"] == (48, 3) and shapes["l0.mix.ra"] == (3, 16, 16)
    assert shapes["l0.mix.ri.b"] == (3, 16) and shapes["l0.mix.lam"] == (48,) and shapes["l0.mix.o"] == (64, 48)
    assert shapes["l1.mix.q"] == (64, 64) and shapes["l1.mix.k"] == (16, 64) and shapes["l1.mix.v"] == (24, 64)
    assert shapes["l1.mix.g"] == (96, 64) and shapes["l1.mix.o"] == (64, 96)
    assert shapes["l2.mix.dkv"] == (40, 64) and shapes["l2.mix.dkv.norm"] == (40,) and shapes["l2.mix.uk"] == (48, 40)
    assert shapes["l2.mix.uv"] == (24, 40) and shapes["l2.mix.o"] == (64, 24)
    assert "l3.mix.k" not in shapes and "l3.mix.v" not in shapes and shapes["l3.mix.q"] == (64, 64)
    assert "l2.mlp.gate" not in shapes and "l2.norm2" not in shapes and shapes["l2.norm1b"] == (64,)
    assert shapes["l1.mlp.gate"] == (96, 64) and shapes["l1.side.gate"] == (8, 64) and shapes["l1.side.proj"] == (64, 8)
    requests = cache_requests(spec)
    assert [r.kind for r in requests] == ["none", "kv", "latent"]
    assert requests[0].state_bytes == 4 * (2 + 3) * 48 and (requests[1].head_dim, requests[1].v_head_dim) == (16, 24)
    assert requests[2].head_dim == 40
    assert [(e.cache, e.writes_cache) for e in spec.schedule] == [(0, True), (1, True), (2, True), (1, False)]
    without_side = povusun_spec(PovusunConfig.from_dict(POVUSUN["PB"]))
    assert not any("side" in name for name in expected_tensors(without_side))


def cpu_engine(folder, max_tokens=512, block_size=16, max_batch=0):
    arch, config = load_config(folder)
    spec = arch.build_spec(config)
    tensors = load_checkpoint(folder, {n: r.shape for n, r in expected_tensors(spec).items()}, spec.ignorable)
    return Engine(spec, tensors, EngineConfig(max_tokens=max_tokens, dtype="float32", device="cpu", block_size=block_size,
                                              max_batch=max_batch), kernel_loader=double_loader())


@pytest.mark.parametrize("name", ["PA", "PB"])
def test_bookkeeping_portions_batches_and_slots_used_again(tmp_path, name):
    folder = make_folder(tmp_path / name, POVUSUN[name], seed=3)
    config, weights = plain_povusun.load_folder(folder)
    engine = cpu_engine(folder, max_tokens=16 * 14, max_batch=3)
    vocab = POVUSUN[name]["vocab"]
    for turn in range(2):                     # the second turn takes the slots, pages and states of the first
        prompts = [random_tokens(vocab, n, seed=10 * turn + n) for n in (5, 40, 18)]
        refs = [plain_povusun.logits_of(config, weights, p).numpy() for p in prompts]
        slots = [engine.open_sequence() for _ in prompts]
        cut = [1, 20, 17]
        got = engine.step([StepEntry(s, p[:c], list(range(c))) for s, p, c in zip(slots, prompts, cut)])
        np.testing.assert_allclose(got.numpy(), np.concatenate([r[:c] for r, c in zip(refs, cut)]), rtol=1e-4, atol=2e-5)
        got = engine.step([StepEntry(slots[0], prompts[0][1:], [3]), StepEntry(slots[1], prompts[1][20:22], [0, 1]),
                           StepEntry(slots[2], prompts[2][17:], [0])])
        np.testing.assert_allclose(got.numpy(), np.stack([refs[0][4], refs[1][20], refs[1][21], refs[2][17]]), rtol=1e-4, atol=2e-5)
        engine.close_sequence(slots[0]); engine.close_sequence(slots[2])
        for position in range(22, 40):
            got = engine.step([StepEntry(slots[1], [prompts[1][position]], [0])])
            np.testing.assert_allclose(got.numpy()[0], refs[1][position], rtol=1e-4, atol=2e-5)
        engine.close_sequence(slots[1])
        assert engine.cache.all_free()


def test_a_step_that_runs_twice_leaves_the_recurrent_state_as_one_run_does(tmp_path):
    """A decode graph's warm-up and its first replay run the same one-token step twice: the state a step reads is
    not the state it writes."""
    name = "PA"
    folder = make_folder(tmp_path / name, POVUSUN[name], seed=4)
    config, weights = plain_povusun.load_folder(folder)
    engine = cpu_engine(folder)
    tokens = random_tokens(POVUSUN[name]["vocab"], 12, seed=1)
    ref = plain_povusun.logits_of(config, weights, tokens).numpy()
    slot = engine.open_sequence()
    engine.step([StepEntry(slot, tokens[:6], [])])
    for position in range(6, 12):
        step, rows, n = engine.prepare([StepEntry(slot, [tokens[position]], [0])])
        engine.model.forward(step, rows, n)                                  # once for nothing
        got = engine.model.forward(step, rows, n).clone()
        engine.cache.advance(slot, position + 1)
        np.testing.assert_allclose(got.numpy()[0], ref[position], rtol=1e-4, atol=2e-5)


def test_the_plain_implementation_tells_faults_from_rounding(tmp_path):
    """Each fault that the GPU tests are there to catch moves the plain logits by far more than they allow."""
    name = "PA"
    folder = make_folder(tmp_path / name, POVUSUN[name], seed=5)
    config, weights = plain_povusun.load_folder(folder)
    tokens = random_tokens(POVUSUN[name]["vocab"], 90, seed=2)
    right = plain_povusun.logits_of(config, weights, tokens).numpy()
    allowed = 0.08 * right.std()             # what tests/test_povusun_gpu.py allows a position in bfloat16

    def moved(change):
        other_config, other_weights = copy.deepcopy(config), dict(weights)
        change(other_config, other_weights)
        difference = plain_povusun.logits_of(other_config, other_weights, tokens).numpy() - right
        return np.sqrt((difference ** 2).mean(axis=-1)).max()

    def no_cap(c, w): c["layers"][1]["mixer"].pop("softcap")
    def no_temperature(c, w): c["layers"][3]["mixer"].pop("q_temp")
    def no_gate(c, w): w["l1.mix.g"] = torch.zeros_like(w["l1.mix.g"])
    def own_keys_of_another_layer(c, w): w["l1.mix.k"] = torch.roll(w["l1.mix.k"], 1, dims=0)
    def no_latent_norm_weight(c, w): w["l2.mix.dkv.norm"] = torch.ones_like(w["l2.mix.dkv.norm"])
    def faster_decay(c, w): w["l0.mix.lam"] = w["l0.mix.lam"] + 1.0
    def shifted_taps(c, w): w["l0.mix.conv"] = torch.roll(w["l0.mix.conv"], 1, dims=1)
    def no_conv_bias(c, w): w["l0.mix.conv.b"] = torch.zeros_like(w["l0.mix.conv.b"])
    def other_limit(c, w): c["layers"][1]["mlp"]["limit"] = 0.2
    def no_side_input(c, w): w["side.embed"] = torch.zeros_like(w["side.embed"])
    def side_of_another_layer(c, w): w["side.embed"] = torch.roll(w["side.embed"], 8, dims=1)
    def no_second_norm(c, w): w["l1.norm1b"] = w["l1.norm1b"] * 2.0
    for change in (no_cap, no_temperature, no_gate, own_keys_of_another_layer, no_latent_norm_weight,
                   faster_decay, shifted_taps, no_conv_bias, other_limit, no_side_input, side_of_another_layer, no_second_norm):
        assert moved(change) > 2 * allowed, f"{change.__name__}: {moved(change) / right.std():.3f} of the spread"


def test_mechanisms_of_the_plain_implementation():
    """The small functions against numbers worked out by hand."""
    p = plain_povusun
    t = torch.tensor
    assert torch.allclose(p.query_temperature(t([0, 5, 6, 13, 14]), 0.5, 7),
                          1.0 + 0.5 * torch.log(t([1.0, 1.0, 2.0, 3.0, 3.0], dtype=torch.float64)))
    assert torch.allclose(p.soft_cap(t([0.0, 100.0, -100.0], dtype=torch.float64), 5.0), t([0.0, 5.0, -5.0], dtype=torch.float64))
    x = t([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=torch.float64)
    conv = p.causal_conv(x, t([[10.0, 1.0], [0.0, 2.0]], dtype=torch.float64), t([0.5, 0.0], dtype=torch.float64))
    assert torch.allclose(conv, t([[1.5, 4.0], [13.5, 8.0], [35.5, 12.0]], dtype=torch.float64))
    v = torch.randn(5, 2, 16, dtype=torch.float64) * 3
    assert torch.allclose((p.unit_rms(v, 0.0) ** 2).mean(-1), torch.ones(5, 2, dtype=torch.float64))
    weights = p.causal_softmax(torch.zeros(1, 3, 3, dtype=torch.float64))[0]
    assert torch.allclose(weights, t([[1, 0, 0], [0.5, 0.5, 0], [1 / 3, 1 / 3, 1 / 3]], dtype=torch.float64))
