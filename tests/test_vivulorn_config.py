"""Host-side parts of the Vivulorn design: its configuration class, the order in which layers run, the names and shapes of
its tensors, the caches and states its layers ask for, and the plain implementation's own mechanisms on hand-made cases."""

from __future__ import annotations

import copy
import json
import math

import numpy as np
import pytest
import torch

import plain_vivulorn as plain
from lalamo_b200.config import (
    AttentionSpec, BlockSpec, ConfigError, DenseMLPSpec, GatedDeltaSpec, LatentAttentionSpec, LayerNormSpec, VivulornConfig, config_from_dict, load_config,
)
from lalamo_b200.parts.model import plan_tensor_decls
from lalamo_b200.weights.loader import WeightsError, load_weights
from tiny_vivulorn import CONFIG_A, CONFIG_B, CONFIG_C, CONFIG_E, CONFIGS, tensor_shapes, write_model


def test_every_size_and_constant_comes_from_the_configuration():
    config = config_from_dict(CONFIG_A)
    assert isinstance(config, VivulornConfig)
    plan = config.to_plan()
    assert plan.vocab_size == 160 and plan.model_dim == 64 and plan.embedding.scale == 2.0 and plan.head.tied and plan.head.softcap == 5.0
    assert isinstance(plan.final_norm, LayerNormSpec) and plan.final_norm.eps == 1e-5 and plan.stream_mix.model_dim == 64
    assert all(isinstance(layer, BlockSpec) and isinstance(layer.pre_mixer_norm, LayerNormSpec) for layer in plan.layers)
    first, second, third, fourth = plan.layers
    assert isinstance(first.mixer, GatedDeltaSpec)
    assert (first.mixer.num_heads, first.mixer.num_groups, first.mixer.key_dim, first.mixer.value_dim, first.mixer.conv_taps) == (4, 2, 16, 24, 4)
    assert not first.mixer.decay_per_channel and first.mixer.decay_rank == 0 and first.mixer.gate_rank == 0 and first.mixer.gate_activation == "silu"
    assert first.mixer.norm_eps == 1e-5 and first.mixer.unit_eps == 1e-6
    assert isinstance(first.ffn, DenseMLPSpec) and (first.ffn.hidden_dim, first.ffn.activation, first.ffn.has_bias) == (48, "gelu", True)
    assert isinstance(second.mixer, LatentAttentionSpec)
    assert (second.mixer.num_heads, second.mixer.head_dim, second.mixer.rope_dim, second.mixer.value_dim, second.mixer.latent_dim) == (4, 16, 8, 24, 32)
    assert (second.mixer.window, second.mixer.scale, second.mixer.gated, second.mixer.sink) == (None, 0.2, False, True)
    assert second.mixer.position.pairing == "interleaved" and second.mixer.position.theta == 500.0 and second.mixer.position.scaling is None
    assert second.mixer.latent_norm.eps == 1e-5 and second.mixer.latent_norm.scale_offset == 0.0
    assert isinstance(third.mixer, AttentionSpec)
    assert (third.mixer.num_heads, third.mixer.num_groups, third.mixer.head_dim, third.mixer.value_dim, third.mixer.scale) == (4, 2, 16, 32, 0.3)
    assert third.mixer.qk_norm_whole and third.mixer.gated and third.mixer.window is None and not third.mixer.has_bias
    rope = third.mixer.position
    assert (rope.pairing, rope.rotary_dim, rope.theta) == ("half", 8, 100.0)
    assert (rope.scaling.factor, rope.scaling.original, rope.scaling.fast, rope.scaling.slow) == (4.0, 64.0, 8.0, 2.0)
    assert fourth.ffn is None and fourth.pre_ffn_norm is None and fourth.mixer.conv_taps == 2
    plain_b = config_from_dict(CONFIG_B).to_plan()
    assert plain_b.layers[0].mixer.position is None and plain_b.stream_mix is None and plain_b.head.softcap == 0.0 and plain_b.embedding.scale == 1.0
    assert plain_b.layers[3].mixer.position.scaling.factor == 1.5 and plain_b.layers[2].mixer.conv_taps == 1


def test_the_order_in_which_layers_run():
    for name, config in CONFIGS.items():
        schedule = config_from_dict(config).to_plan().schedule
        assert [(entry.layer, entry.mix_embedding) for entry in schedule] == plain.layer_runs(config), name
        assert all(entry.cache_from is None and not entry.add_embedding for entry in schedule)   # every run has a cache of its own
    runs = [(entry.layer, entry.mix_embedding) for entry in config_from_dict(CONFIG_A).to_plan().schedule]
    assert runs == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    whole = [(entry.layer, entry.mix_embedding) for entry in config_from_dict(CONFIG_C).to_plan().schedule]
    assert whole == [(0, True), (1, False), (2, False)] * 3
    once = copy.deepcopy(CONFIG_A)
    once["loop"] = {"start": 3, "stop": 4, "times": 1}   # one pass still renews the stream before its first layer
    assert [(entry.layer, entry.mix_embedding) for entry in config_from_dict(once).to_plan().schedule] == [(0, False), (1, False), (2, False), (3, True)]


@pytest.mark.parametrize("path,value,key", [
    (("layers", 0, "type"), "recurrent", "layers[0].type"),
    (("layers", 2, "mixer", "kv_heads"), 3, "layers[2].mixer.kv_heads"),
    (("layers", 0, "mixer", "kv_heads"), 3, "layers[0].mixer.kv_heads"),
    (("layers", 2, "mixer", "rot", "dims"), 18, "layers[2].mixer.rot.dims"),
    (("layers", 2, "mixer", "rot", "scaling", "factor"), None, "layers[2].mixer.rot.scaling.factor"),
    (("layers", 2, "mixer", "scale"), None, "layers[2].mixer.scale"),
    (("layers", 1, "mixer", "rot_dim"), 7, "layers[1].mixer.rot_dim"),
    (("layers", 1, "mixer", "kv_rank"), None, "layers[1].mixer.kv_rank"),
    (("layers", 0, "mixer", "conv"), 0, "layers[0].mixer.conv"),
    (("layers", 1, "mlp", "kind"), "moe", "layers[1].mlp.kind"),
    (("layers", 1, "mlp", "ff"), None, "layers[1].mlp.ff"),
    (("loop", "stop"), 9, "loop"),
    (("norm", "eps"), None, "config.norm.eps"),
    (("width",), None, "config.width"),
])
def test_errors_name_the_key(path, value, key):
    raw = copy.deepcopy(CONFIG_A)
    node = raw
    for step in path[:-1]:
        node = node[step]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        config_from_dict(raw)
    assert key in str(error.value)


def test_tensor_names_and_shapes_and_loading(tmp_path):
    for name in ("A", "B", "E"):
        config = CONFIGS[name]
        folder, _ = write_model(tmp_path / name, config, 3)
        typed = load_config(folder)
        plan = typed.to_plan()
        declared = {typed.checkpoint_names(*key)[0]: tuple(decl.shape) for key, decl in plan_tensor_decls(plan).items()}
        assert declared == tensor_shapes(config), name
        tensors = load_weights(folder, typed, plan)
        assert len(tensors) == len(declared)
    missing = copy.deepcopy(CONFIG_A)
    missing["layers"][1]["mixer"]["kv_rank"] = 40   # the checkpoint's tensors do not fit
    (tmp_path / "A" / "config.json").write_text(json.dumps(missing))
    with pytest.raises(WeightsError):
        load_weights(tmp_path / "A", load_config(tmp_path / "A"))


def test_random_weights_round_trip(tmp_path):
    from lalamo_b200.weights.random_init import write_random_model

    folder = write_random_model(tmp_path / "random", CONFIG_A, seed=5)
    typed = load_config(folder)
    assert typed.to_json_dict()["loop"] == CONFIG_A["loop"]
    tensors = load_weights(folder, typed)
    assert (tensors[(("layers", 1, "mixer"), "latent_norm")] - 1).abs().max() < 0.5 and tensors[(("stream_mix",), "weight")].shape == (64, 128)


def test_the_caches_and_states_the_layers_ask_for():
    from lalamo_b200.parts.attention import Attention
    from lalamo_b200.parts.base import PagedKVNeed
    from lalamo_b200.parts.latent_attention import LatentAttention

    plan = config_from_dict(CONFIG_A).to_plan()
    holder = lambda spec, **more: type("Holder", (), {"spec": spec, **more})()
    need = LatentAttention.cache_need(holder(plan.layers[1].mixer))
    assert need == PagedKVNeed(num_groups=1, head_dim=40, window=None, value_dim=32, values_in_keys=True)   # the latent and the shared key part, nothing per head
    need = Attention.cache_need(holder(plan.layers[2].mixer, keep_first=0))
    assert (need.num_groups, need.head_dim, need.value_dim, need.window) == (2, 16, 32, None)
    assert len(plan.schedule) == 6   # a cache or state per run: the repeated layers hold two each


# ------------------------------------------------------------------ the plain implementation by hand
def test_plain_norms_by_hand():
    x = np.array([[1.0, 3.0]])
    assert np.allclose(plain.layer_norm(x, np.array([2.0, 2.0]), np.array([0.5, -0.5]), 0.0), [[-1.5, 1.5]])
    assert np.allclose(plain.layer_norm(x, np.ones(2), np.zeros(2), 3.0), [[-0.5, 0.5]])   # var 1, eps 3 under the root
    assert np.allclose(plain.rms_norm(x, np.array([1.0, 2.0]), 4.0), [[1 / 3, 2.0]])       # mean square 5, + 4
    assert np.allclose(plain.gelu_erf(np.array([0.0, 1.0])), [0.0, 0.5 * (1 + math.erf(2 ** -0.5))])
    assert np.allclose(plain.softcap(np.array([0.0, 1e9, -1e9, 0.1]), 5.0), [0.0, 5.0, -5.0, 5.0 * math.tanh(0.02)])


def test_plain_rotations_agree_on_reordered_channels():
    """Pairs (2i, 2i + 1) are pairs (i, i + dims / 2) of the channels taken evens first, odds second."""
    generator = np.random.default_rng(0)
    x = generator.standard_normal((5, 3, 12))
    positions = np.array([0, 1, 7, 100, 4000])
    freq = plain.plain_frequencies(8, 50.0)
    order = np.concatenate([np.arange(0, 8, 2), np.arange(1, 8, 2), np.arange(8, 12)])
    pairs = plain.rotate_pairs(x, positions, 8, freq)
    halves = plain.rotate_half(x[..., order], positions, 8, freq)
    assert np.allclose(pairs[..., order], halves)
    assert np.allclose(pairs[..., 8:], x[..., 8:]) and np.allclose(pairs[0], x[0])   # the rest passes; position 0 turns nothing
    assert np.allclose(np.linalg.norm(pairs, axis=-1), np.linalg.norm(x, axis=-1))
    one = plain.rotate_half(np.array([[[1.0, 0.0]]]), np.array([3]), 2, np.array([0.5]), 2.0)   # angle 1.5, lengths doubled
    assert np.allclose(one, [[[2 * math.cos(1.5), 2 * math.sin(1.5)]]])


def test_stretched_frequencies_by_hand():
    """dims 8, base 100: pair(t) = 8 ln(original / (2 pi t)) / (2 ln 100).  original 64, fast 8, slow 2 put the ramp between
    pair floor(0.21) = 0 and pair ceil(1.41) = 2: pair 0 keeps its frequency, pair 1 is half way, pairs 2 and 3 are divided."""
    scaling = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}
    freq, magnitude = plain.yarn_frequencies(8, 100.0, scaling)
    base = 100.0 ** (-np.arange(4) / 4)
    assert np.allclose(freq, [base[0], base[1] * (0.5 / 4 + 0.5), base[2] / 4, base[3] / 4])
    assert math.isclose(magnitude, 0.1 * math.log(4.0) + 1.0)
    # a ramp of no width: hi = lo, the division is by 0.001 and the ramp is a step
    step, _ = plain.yarn_frequencies(8, 100.0, {"factor": 2.0, "original": 64, "fast": 3.0, "slow": 2.5})
    lo = math.floor(8 * math.log(64 / (2 * math.pi * 3.0)) / (2 * math.log(100.0)))
    assert lo == 1 and np.allclose(step, [base[0], base[1], base[2] / 2, base[3] / 2])
    # the package's table is the same
    from lalamo_b200.config.plan import YarnScaling
    from lalamo_b200.parts.rope import stretched_frequencies

    got, factor = stretched_frequencies(8, 100.0, YarnScaling(4.0, 64.0, 8.0, 2.0))
    assert np.allclose(got.double().numpy(), freq, rtol=1e-6) and math.isclose(factor, magnitude, rel_tol=1e-6)


def test_plain_softmax_with_a_sink_by_hand():
    scores = np.log(np.array([[1.0, 2.0, 5.0]]))
    mask = np.array([[True, True, False]])
    assert np.allclose(plain.sink_softmax(scores, mask), [[1 / 3, 2 / 3, 0.0]])
    assert np.allclose(plain.sink_softmax(scores, mask, sink=math.log(3.0)), [[1 / 6, 2 / 6, 0.0]])   # counts once, carries nothing
    assert np.allclose(plain.sink_softmax(scores, mask, sink=800.0), 0.0)                              # a large sink takes all the weight, without overflow


def test_plain_convolution_and_delta_rule_by_hand():
    x = np.array([[1.0], [2.0], [3.0]])
    taps = np.array([[100.0, 10.0, 1.0]])   # the last column is the current token's
    assert np.allclose(plain.short_convolution(x, taps), [[1.0], [12.0], [123.0]])
    assert np.allclose(plain.short_convolution(x[2:], taps, before=x[:2]), [[123.0]])
    # one key direction: the state learns v where beta = 1, forgets by g, and the read-out sees the write of its own token
    k = np.array([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0]])
    v = np.array([[2.0], [4.0], [7.0]])
    out, state = plain.delta_rule(q=k, k=k, v=v, beta=np.array([1.0, 0.5, 1.0]), g=np.array([1.0, 0.5, 1.0]))
    # t0: S = [[2],[0]] -> 2.  t1: S = 0.5 S = [[1],[0]]; u = 0.5 (4 - 1) = 1.5; S = [[2.5],[0]] -> 2.5.  t2: u = 7 on the other row -> 7.
    assert np.allclose(out, [[2.0], [2.5], [7.0]]) and np.allclose(state, [[2.5], [7.0]])
    resumed, _ = plain.delta_rule(k[2:], k[2:], v[2:], np.array([1.0]), np.array([1.0]), state=np.array([[2.5], [0.0]]))
    assert np.allclose(resumed, [[7.0]])


def test_plain_forward_renews_the_stream_once_a_pass(tmp_path):
    """With a renewal that keeps the stream and drops the embedding's output ([I 0]) a model whose one layer runs twice equals the
    two-layer model of the same layer twice; with [0 I] every pass starts over and the result is that of one pass."""
    config = copy.deepcopy(CONFIG_E)
    _, weights = write_model(tmp_path / "e", config, 9)
    tokens = [5, 9, 2, 77, 31, 5, 5, 60]
    twice = copy.deepcopy(config)
    twice["layers"] = config["layers"] * 2
    del twice["loop"]
    doubled = dict(weights, **{name.replace("l0.", "l1."): value for name, value in weights.items() if name.startswith("l0.")})
    eye, zero = np.eye(64), np.zeros((64, 64))
    keep = dict(weights, **{"loop.in": np.concatenate([eye, zero], axis=1)})
    assert np.allclose(plain.forward(tokens, keep, config), plain.forward(tokens, doubled, twice))
    restart = dict(weights, **{"loop.in": np.concatenate([zero, eye], axis=1)})
    single = copy.deepcopy(config)
    del single["loop"]
    assert np.allclose(plain.forward(tokens, restart, config), plain.forward(tokens, weights, single))
    runs: list[np.ndarray] = []
    plain.forward(tokens, weights, config, runs)
    assert len(runs) == 2 and runs[0].shape == (8, 64)
