"""Host-side parts of the Zozenex design: its configuration class, the names and shapes of its tensors, the caches and states its
layers ask for, and the plain implementation's own mechanisms on hand-made cases."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_zozenex as plain
from lalamo_b200.config import (
    BlockSpec, ConfigError, DenseMLPSpec, LinearAttentionSpec, ParallelMixerSpec, PooledWindowAttentionSpec, RMSNormSpec, RoutedMLPSpec, ZozenexConfig,
    config_from_dict, load_config,
)
from lalamo_b200.parts.model import plan_tensor_decls
from lalamo_b200.weights.loader import WeightsError, load_weights
from tiny_zozenex import CONFIG_A, CONFIG_B, CONFIGS, DECAY_RANK, tensor_shapes, write_model


def test_every_size_and_constant_comes_from_the_configuration():
    config = config_from_dict(CONFIG_A)
    assert isinstance(config, ZozenexConfig)
    plan = config.to_plan()
    assert plan.vocab_size == 160 and plan.model_dim == 64 and not plan.head.tied and plan.embedding.learned_positions == 2048 and plan.embedding.scale == 1.0
    assert isinstance(plan.final_norm, RMSNormSpec) and plan.final_norm.eps == 1e-5 and plan.final_norm.exact
    assert all(isinstance(layer, BlockSpec) and layer.pre_mixer_norm.exact for layer in plan.layers)
    first, second, third, fourth = plan.layers
    assert isinstance(first.mixer, LinearAttentionSpec)
    assert (first.mixer.num_heads, first.mixer.key_dim, first.mixer.value_dim, first.mixer.decay, first.mixer.scaled, first.mixer.norm_weight) == (4, 16, 24, "fixed", "key", False)
    assert first.mixer.decay_values == tuple(CONFIG_A["layers"][0]["mixer"]["decay"]) and first.mixer.norm_eps == 1e-5 and first.mixer.gate_activation == "silu"
    ffn = first.ffn
    assert isinstance(ffn, RoutedMLPSpec) and (ffn.num_experts, ffn.top, ffn.hidden_dim, ffn.weight_scale, ffn.activation) == (6, 2, 24, 1.5, "gelu")
    assert not ffn.gated and ffn.choice_bias and ffn.shared_gate and not ffn.renormalize and ffn.score == "sigmoid" and ffn.group_count == 1
    assert isinstance(ffn.shared, DenseMLPSpec) and (ffn.shared.hidden_dim, ffn.shared.activation, ffn.shared.has_bias) == (32, "gelu", False)
    assert isinstance(second.mixer, ParallelMixerSpec) and [(name, scale) for name, _, scale in second.mixer.branches] == [("left", 0.5), ("right", 0.5)]
    assert second.mixer.branch_norm == RMSNormSpec(dim=64, eps=1e-5, exact=True)
    left, right = second.mixer.branches[0][1], second.mixer.branches[1][1]
    assert isinstance(left, PooledWindowAttentionSpec)
    assert (left.num_heads, left.num_groups, left.head_dim, left.value_dim, left.window, left.pool, left.scale, left.softcap) == (4, 2, 16, 24, 37, 5, 0.3, 15.0)
    assert left.rotate_values and left.head_bias and (left.position.rotary_dim, left.position.theta, left.position.pairing) == (8, 500.0, "half")
    assert isinstance(right, LinearAttentionSpec)
    assert (right.num_heads, right.key_dim, right.value_dim, right.decay, right.tau, right.scaled, right.norm_weight) == (2, 16, 8, "channel", 6.0, "query", True)
    assert third.ffn is None and third.pre_ffn_norm is None
    assert fourth.ffn.shared is None and not fourth.ffn.shared_gate and fourth.ffn.top == 4
    plain_b = config_from_dict(CONFIG_B).to_plan()
    assert plain_b.layers[0].mixer.branches[0][1].position.rotary_dim == 0 and plain_b.layers[0].mixer.branches[0][1].pool == 21


def test_the_bottleneck_rank_and_the_positions_come_from_the_tensors(tmp_path):
    other = copy.deepcopy(CONFIG_A)
    other["max_positions"] = 300
    folder, _ = write_model(tmp_path / "a", other, 1, rank=6)
    config = load_config(folder)
    assert config.layers[1].mixer.branches[1][1].decay_rank == 6 and config.layers[2].mixer.branches[1][1].decay_rank == 6
    assert config.to_plan().embedding.learned_positions == 300
    assert config_from_dict(other).layers[1].mixer.branches[1][1].decay_rank == 16   # no checkpoint and no key: the default
    assert config.to_json_dict()["max_positions"] == 300 and config.to_json_dict()["architecture"] == "Zozenex"


@pytest.mark.parametrize("path,value,key", [
    (("layers", 0, "type"), "attention", "layers[0].type"),
    (("layers", 0, "mixer", "decay"), [0.5], "layers[0].mixer.decay"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "layers[1].mixer.left.kv_heads"),
    (("layers", 1, "mixer", "left", "vdim"), 7, "layers[1].mixer.left.vdim"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18, "layers[1].mixer.left.rot.dims"),
    (("layers", 1, "mixer", "left", "scale"), None, "layers[1].mixer.left.scale"),
    (("layers", 1, "mixer", "left", "mask", "size"), 0, "layers[1].mixer.left.mask.size"),
    (("layers", 1, "mixer", "right", "tau"), 0.0, "layers[1].mixer.right.tau"),
    (("layers", 0, "mlp", "kind"), "dense", "layers[0].mlp.kind"),
    (("layers", 0, "mlp", "router", "top"), 7, "layers[0].mlp.router.top"),
    (("layers", 0, "mlp", "expert", "ff"), None, "layers[0].mlp.expert.ff"),
    (("norm", "eps"), None, "config.norm.eps"),
    (("max_positions",), None, "config.max_positions"),
])
def test_a_bad_configuration_names_its_key(path, value, key):
    raw = copy.deepcopy(CONFIG_A)
    at = raw
    for step in path[:-1]:
        at = at[step]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as caught:
        config_from_dict(raw)
    assert key in str(caught.value)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_tensor_names_and_shapes(tmp_path, name):
    """Every tensor of a model folder written from the design's own names is asked for under that name with that shape, and nothing else is."""
    config = CONFIGS[name]
    folder, _ = write_model(tmp_path / name, config, 3, DECAY_RANK[name])
    typed = load_config(folder)
    plan = typed.to_plan()
    asked = {typed.checkpoint_names(path, local)[0]: decl.shape for (path, local), decl in plan_tensor_decls(plan).items()}
    written = tensor_shapes(config, DECAY_RANK[name])
    assert set(asked) == set(written)
    for tensor_name, shape in written.items():
        assert tuple(extent for extent in asked[tensor_name] if extent != 1) == tuple(extent for extent in shape if extent != 1), tensor_name
    assert len(load_weights(folder, typed, plan)) == len(written)


def test_a_checkpoint_that_does_not_fit_is_reported_whole(tmp_path):
    from lalamo_b200.weights.safetensors_io import write_safetensors

    folder, weights = write_model(tmp_path / "a", CONFIG_A, 3, DECAY_RANK["A"])
    broken = {name: tensor.to(torch.bfloat16) for name, tensor in weights.items() if name != "l1.mix.left.pb"}
    broken["l0.mlp.correction"] = torch.zeros(5, dtype=torch.bfloat16)
    broken["l9.extra"] = torch.zeros(2, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", broken)
    with pytest.raises(WeightsError) as caught:
        load_weights(folder, load_config(folder))
    assert caught.value.missing == ["l1.mix.left.pb"] and caught.value.unexpected == ["l9.extra"] and caught.value.wrong_shape[0][0] == "l0.mlp.correction"


def test_caches_and_states_the_layers_ask_for():
    """Retention: one 32-bit matrix state.  The pair of mixers: the attention's pages under the window's rule (no shorter than a block),
    its blocks' pages kept for good with one row for every ``pool`` positions (a row holds a key and its value), and the linear attention's matrix state."""
    from lalamo_b200.cache.manager import CacheManager
    from lalamo_b200.parts.base import CompositeNeed, PagedKVNeed, SlotStateNeed

    # what the parts would declare, spelled out here for CONFIG_A's second and third layer and CONFIG_B's first
    def needs(heads, groups, dim, vdim, size, pool, linear):
        return CompositeNeed((CompositeNeed((PagedKVNeed(groups, dim + vdim, window=max(size, pool), values_in_keys=True),
                                             PagedKVNeed(groups, dim + vdim, window=None, values_in_keys=True, tokens_per_row=pool))),
                              SlotStateNeed(linear, torch.float32)))

    all_needs = [SlotStateNeed((4, 16, 24), torch.float32), needs(4, 2, 16, 24, 37, 5, (2, 16, 8)), needs(2, 2, 32, 16, 16, 16, (4, 8, 16)), needs(3, 3, 24, 10, 9, 21, (1, 12, 20))]
    manager = CacheManager(all_needs, [None] * 4, None, page_size=16, num_pages=12, num_slots=2)
    assert {group.window: len(group.entries) for group in manager.groups} == {37: 1, 16: 1, 21: 1, None: 3}
    manager.admit("a")
    manager.reserve("a", 100)
    manager.commit("a", 100)
    held = {group.window: sum(page >= 0 for page in manager.requests["a"].blocks[index]) for index, group in enumerate(manager.groups)}
    # positions 0 .. 100 - window are behind every later query's window: their whole pages are given back; the blocks' pages all stay
    assert held == {None: 7, 37: 7 - (100 - 37 + 1) // 16, 16: 7 - (100 - 16 + 1) // 16, 21: 7 - (100 - 21 + 1) // 16}
    manager.release("a")
    manager.check()
    assert manager.free_pages() == 12


def test_the_plain_mechanisms_on_hand_made_cases():
    # a block is seen once all of it lies behind the window: with a window of 3 and blocks of 2, position 4 sees block 0 (positions 0, 1)
    # and positions 2 .. 4; position 3 sees positions 1 .. 3 and no block (position 0 is not seen at all)
    h = torch.eye(6, dtype=torch.float64)
    cfg = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "softcap": 1e7, "rot": {"dims": 0, "base": 10.0}, "mask": {"size": 3, "pool": 2}}
    keys = torch.tensor([[8.0, 0.0], [0.0, 0.0], [0.0, 0.0], [0.0, 0.0], [0.0, 0.0], [0.0, 0.0]], dtype=torch.float64)
    w = {"q": torch.tensor([[1.0] * 6, [0.0] * 6], dtype=torch.float64), "k": keys.T.contiguous(), "v": torch.zeros(2, 6, dtype=torch.float64), "pb": torch.tensor([-2.0], dtype=torch.float64),
         "o": torch.eye(2, dtype=torch.float64)}
    w["v"][0, 0] = 1.0   # only position 0 has a value; it is rotated by position 0, that is not at all
    out = plain.pooled_sigmoid_attention(h, w, cfg)
    weight_alone, weight_in_block = (float(torch.sigmoid(torch.tensor(x, dtype=torch.float64))) for x in (8.0 - 2.0, 4.0 - 2.0))
    length = lambda row: float(row.norm())   # the sum is turned back by the query's position: its length stays
    assert abs(length(out[0]) - weight_alone) < 1e-9 and abs(length(out[2]) - weight_alone) < 1e-9
    assert length(out[3]) < 1e-9                                        # left the window, its block not yet behind it
    assert abs(length(out[4]) - 0.5 * weight_in_block) < 1e-9           # the block's mean key (half the score) and mean value (half the value)
    assert abs(length(out[5]) - 0.5 * weight_in_block) < 1e-9
    # the recurrence against its closed form for a fixed decay: o_t = sum_j a^(t - j) (q_t . k_j) v_j
    q, k, v = torch.rand(5, 1, 3, dtype=torch.float64), torch.rand(5, 1, 3, dtype=torch.float64), torch.rand(5, 1, 2, dtype=torch.float64)
    out = plain.linear_recurrence(q, k, v, torch.full((5, 1, 3), 0.5, dtype=torch.float64))
    closed = sum(0.5 ** (4 - j) * (q[4, 0] @ k[j, 0]) * v[j, 0] for j in range(5))
    assert torch.allclose(out[4, 0], closed)
    # experts are chosen by score plus correction and weighed by the score alone
    w = {"router": torch.tensor([[2.0], [0.0], [-2.0]], dtype=torch.float64), "correction": torch.tensor([-1.0, 0.0, 0.9], dtype=torch.float64)}
    for e in range(3):
        w[f"e{e}.up"], w[f"e{e}.down"] = torch.ones(1, 1, dtype=torch.float64), torch.full((1, 1), float(e + 1), dtype=torch.float64)
    cfg = {"router": {"experts": 3, "top": 1, "scale": 2.0}, "expert": {"ff": 1}, "shared": None}
    out = plain.routed_experts(torch.ones(1, 1, dtype=torch.float64), w, cfg)
    # choice scores: 0.88 - 1, 0.5, 0.12 + 0.9 -> the third expert, weighed by sigmoid(-2) * 2
    assert torch.allclose(out, torch.sigmoid(torch.tensor(-2.0, dtype=torch.float64)) * 2.0 * 3.0 * plain.gelu(torch.ones(1, 1, dtype=torch.float64)))


def test_how_the_tensor_core_attention_divides_a_step():
    """A CTA's eight warps are one query head's 16 tokens each: the fewer heads a K/V head has, the longer the tiles; launches of few CTAs
    share out a tile's rows, by the launch's shape alone."""
    from lalamo_b200 import ops

    assert [ops.pooled_attention_tiling(heads, groups) for heads, groups in ((8, 8), (8, 4), (6, 2), (16, 4), (40, 2))] == [(1, 128), (2, 64), (3, 32), (4, 32), (4, 32)]
    assert ops.pooled_attention_supported(torch.bfloat16, 64, 48) and ops.pooled_attention_supported(torch.bfloat16, 128, 16)
    assert not ops.pooled_attention_supported(torch.float32, 64, 64) and not ops.pooled_attention_supported(torch.bfloat16, 24, 64)
    assert not ops.pooled_attention_supported(torch.bfloat16, 64, 144)
    for shares_of in (lambda n: ops.pooled_attention_shares(n, 16, 4, sms=148), lambda n: ops.pooled_single_shares(n, 16, 4, sms=148)):
        counts = [shares_of(n) for n in (1, 8, 64, 148, 1000)]
        assert counts[0] == 16 and counts[-1] == 1 and all(a >= b for a, b in zip(counts, counts[1:])) and all(1 <= c <= 16 for c in counts)
