"""The Vivulorn design on the GPU against the plain NumPy restatement (``plain_vivulorn.py``): each mechanism's kernels
alone, then whole models through the engine: prompts at once, decoding through the cache and the recurrent state,
portions of every size, mixed batches with pages and slots that are freed and used again, keys far back, long
decoding, and greedy generation through the Python entry point and the command line."""

from __future__ import annotations

import copy
import json

import numpy as np
import pytest
import torch

import plain_vivulorn as plain
from tiny_vivulorn import CONFIGS, attention, delta, latent, layer, model, write_model

pytestmark = pytest.mark.gpu

FLOAT32_LIMIT = 2e-4   # of the logits' spread; 32-bit sums of a few hundred terms stay far below
BFLOAT16_LIMIT = 0.08


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("vivulorn")
    return {name: write_model(root / name, config, 70 + seed) for seed, (name, config) in enumerate(CONFIGS.items())}


def tokens_for(config: dict, count: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, config["vocab"], size=count).tolist()


def load_engine(folder, dtype: str, max_tokens: int = 1024, **options):
    from lalamo_b200.engine.engine import Engine, EngineConfig

    return Engine.load(folder, EngineConfig(dtype=dtype, page_size=16, max_tokens=max_tokens, max_requests=4, poison_freed=True, **options))


def row_errors(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: the spread of the difference (its mean taken off) over the spread of the wanted logits."""
    difference = got - want
    difference = difference - difference.mean(axis=-1, keepdims=True)
    centred = want - want.mean(axis=-1, keepdims=True)
    return np.sqrt((difference**2).mean(axis=-1)) / np.sqrt((centred**2).mean())


def run_schedule(engine, requests: dict[str, list[int]], schedule: list[list[tuple[str, int]]]) -> dict[str, np.ndarray]:
    """Feeds the requests' tokens in the schedule's portions (every step one batch), asks for every position's logits,
    ends a request with its last token, and checks the cache's books after every step."""
    from lalamo_b200.engine.executor import StepEntry

    done = {name: 0 for name in requests}
    rows: dict[str, list[np.ndarray]] = {name: [] for name in requests}
    for step in schedule:
        entries = []
        for name, count in step:
            if done[name] == 0:
                engine.admit(name)
            entries.append(StepEntry(name, requests[name][done[name] : done[name] + count], list(range(count))))
        logits = engine.step(entries).float().cpu().numpy()
        offset = 0
        for name, count in step:
            rows[name].append(logits[offset : offset + count])
            offset += count
            done[name] += count
            if done[name] == len(requests[name]):
                engine.release(name)
        engine.executor.check_status()
        engine.cache.check()
    assert all(done[name] == len(tokens) for name, tokens in requests.items())
    return {name: np.concatenate(parts) for name, parts in rows.items()}


def close_enough(got: np.ndarray, want: np.ndarray, dtype: str) -> bool:
    """Nothing in this design makes a discrete choice, so every row is held to the limit, in bfloat16 too."""
    errors = row_errors(got, want)
    return bool(errors.max() < (FLOAT32_LIMIT if dtype == "float32" else BFLOAT16_LIMIT))


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_a_prompt_at_once_and_token_by_token(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 90, 5)
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, dtype)
    whole = run_schedule(engine, {"a": tokens}, [[("a", len(tokens))]])["a"]
    assert close_enough(whole, want, dtype)
    # the first 21 at once, the rest one by one: the state and the cache carry everything, steps replay from recordings
    decoded = run_schedule(engine, {"b": tokens}, [[("b", 21)]] + [[("b", 1)]] * (len(tokens) - 21))["b"]
    assert close_enough(decoded, want, dtype)
    # from the very first token on, one by one: convolutions that start among zeros, an empty state, a cache of one key
    single = run_schedule(engine, {"c": tokens[:40]}, [[("c", 1)]] * 40)["c"]
    assert close_enough(single, want[:40], dtype)
    assert engine.cache.free_pages() == engine.cache.num_pages


@pytest.mark.parametrize("name", ["A", "C"])
def test_the_stream_after_every_layer_run(models, name):
    """The 32-bit stream after every run of a layer (a repeated layer counts each time) against the plain implementation's."""
    from lalamo_b200 import ops

    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 30, 8)
    wanted: list[np.ndarray] = []
    plain.forward(tokens, weights, config, wanted)
    engine = load_engine(folder, "float32", cuda_graphs=False)
    seen: list[torch.Tensor] = []
    for block in engine.model.blocks:
        def tapped(residual, pending, step, cache, inner=block.forward):
            result = inner(residual, pending, step, cache)
            stream = residual.clone()
            if result is not None:   # what the block leaves for the next norm to add
                ops.residual_add(stream, result)
            seen.append(stream)
            return result
        block.forward = tapped
    run_schedule(engine, {"a": tokens}, [[("a", len(tokens))]])
    assert len(seen) == len(wanted) == len(plain.layer_runs(config))
    for index, (got, want) in enumerate(zip(seen, wanted)):
        assert np.abs(got.cpu().numpy() - want).max() < 2e-4 * np.abs(want).max(), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 150, 6)
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, dtype)
    for cuts in ([2, 3, 2, 5, 1, 17, 1, 1, 33, 2, 16, 31, 36], [64, 2, 2, 2, 48, 32], [7] * 21 + [3], [1, 2, 147]):
        assert sum(cuts) == len(tokens)
        got = run_schedule(engine, {"a": tokens}, [[("a", count)] for count in cuts])["a"]
        assert close_enough(got, want, dtype), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Up to four live requests of unequal lengths, portions beside single tokens; requests end and others take their
    slots and pages (which were overwritten with NaN when they were given back); a pool smaller than the sum."""
    folder, weights = models[name]
    config = CONFIGS[name]
    lengths = {"a": 70, "b": 1, "c": 33, "d": 2, "e": 95, "f": 18, "g": 64}
    requests = {key: tokens_for(config, count, 10 + index) for index, (key, count) in enumerate(lengths.items())}
    schedule = [
        [("a", 30), ("b", 1), ("c", 2)],
        [("a", 1), ("c", 1), ("d", 1), ("e", 17)],
        [("a", 1), ("c", 14), ("d", 1), ("e", 1)],
        [("a", 16), ("c", 1), ("e", 40), ("f", 3)],
        [("a", 1), ("c", 15), ("e", 1), ("f", 15)],
        [("a", 21), ("e", 2), ("g", 33)],
        [("e", 33), ("g", 1)],
        [("e", 1), ("g", 30)],
    ]
    engine = load_engine(folder, dtype, max_tokens=288)
    got = run_schedule(engine, requests, schedule)
    for key, tokens in requests.items():
        assert close_enough(got[key], plain.forward(tokens, weights, config), dtype), key
    # each request alone, in one piece, on the same engine: what the batch and the cutting change is rounding
    for key in ("a", "e"):
        alone = run_schedule(engine, {key: requests[key]}, [[(key, len(requests[key]))]])[key]
        assert row_errors(got[key], alone).max() < 5e-5 if dtype == "float32" else close_enough(got[key], alone, dtype), key
    assert engine.cache.free_pages() == engine.cache.num_pages


def test_a_request_left_out_of_steps_goes_on_later(models):
    """A request that sits out steps while others run and end keeps its pages, its state and its convolutions' inputs."""
    folder, weights = models["A"]
    config = CONFIGS["A"]
    requests = {key: tokens_for(config, count, 90 + count) for key, count in (("a", 40), ("b", 25), ("c", 12))}
    schedule = [[("a", 9)], [("b", 20)], [("b", 5), ("c", 3)], [("a", 1), ("c", 9)], [("a", 30)]]
    got = run_schedule(load_engine(folder, "float32", max_tokens=128), requests, schedule)
    for key, tokens in requests.items():
        assert close_enough(got[key], plain.forward(tokens, weights, config), "float32"), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    folder, weights = models["C"]
    config = CONFIGS["C"]
    tokens = tokens_for(config, 420, 22)
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, dtype)
    got = run_schedule(engine, {"a": tokens}, [[("a", 4)]] + [[("a", 1)]] * 416)["a"]
    assert close_enough(got, want, dtype) and close_enough(got[-50:], want[-50:], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_portions_beside_a_short_request(models, name, dtype):
    """Portions long enough for the recurrence to run as chunks side by side and for attention to run in tiles on the tensor cores."""
    folder, weights = models[name]
    config = CONFIGS[name]
    requests = {"a": tokens_for(config, 1300, 41), "b": tokens_for(config, 30, 42)}
    schedule = [[("a", 700), ("b", 5)], [("a", 1), ("b", 20)], [("a", 590), ("b", 1)], [("b", 4), ("a", 9)]]
    engine = load_engine(folder, dtype, max_tokens=2048)
    got = run_schedule(engine, requests, schedule)
    for key, tokens in requests.items():
        assert close_enough(got[key], plain.forward(tokens, weights, config), dtype), key


# Scores that spread over tens of units: every query gives nearly all its weight to one or two keys, which lie anywhere in the
# context, so that a key that is lost or misplaced far back changes the logits by far more than rounding does.
SHARP = {
    "attention": model(96, 64, [layer("attention", attention(heads=4, kv_heads=2, dim=32, vdim=16, rot_dims=16, base=50.0, scale=1.0, scaling=(3.0, 40, 6.0, 1.0)), None)]),
    "attention-64": model(96, 128, [layer("attention", attention(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=64, base=1000.0, scale=0.7, scaling=(2.0, 128, 16.0, 1.0)), None)]),
    "latent": model(96, 64, [layer("latent_attention", latent(heads=3, dim=24, rot_dim=12, vdim=20, kv_rank=40, base=50.0, scale=0.8), None)]),
    "latent-64": model(96, 128, [layer("latent_attention", latent(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=64, base=300.0, scale=0.5), None)]),
}


def attention_weights_of(config: dict, weights: dict, tokens: list[int]) -> np.ndarray:
    """The plain implementation's largest softmax weight per query and head of the one layer, and where it lies: [queries, heads, 2]."""
    entry = config["layers"][0]
    c, eps, n = entry["mixer"], config["norm"]["eps"], len(tokens)
    x = weights["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    h = plain.layer_norm(x, weights["l0.norm1"], weights["l0.norm1.b"], eps)
    positions = np.arange(n)
    if entry["type"] == "attention":
        q = plain.rms_norm(h @ weights["l0.mix.q"].T, weights["l0.mix.q.norm"], eps).reshape(n, c["heads"], c["dim"])
        k = plain.rms_norm(h @ weights["l0.mix.k"].T, weights["l0.mix.k.norm"], eps).reshape(n, c["kv_heads"], c["dim"])
        freq, magnitude = plain.yarn_frequencies(c["rot"]["dims"], c["rot"]["base"], c["rot"].get("scaling"))
        q, k = (plain.rotate_half(a, positions, c["rot"]["dims"], freq, magnitude) for a in (q, k))
        scores = np.stack([q[:, head] @ k[:, head // (c["heads"] // c["kv_heads"])].T for head in range(c["heads"])], axis=1) * c["scale"]
        sink = None
    else:
        q = (h @ weights["l0.mix.q"].T).reshape(n, c["heads"], c["dim"] + c["rot_dim"])
        down = h @ weights["l0.mix.dkv"].T
        normed = plain.rms_norm(down[:, : c["kv_rank"]], weights["l0.mix.dkv.norm"], eps)
        freq = plain.plain_frequencies(c["rot_dim"], c["rot"]["base"])
        k_rot = plain.rotate_pairs(down[:, None, c["kv_rank"] :], positions, c["rot_dim"], freq)[:, 0]
        q_rot = plain.rotate_pairs(q[..., c["dim"] :], positions, c["rot_dim"], freq)
        k_plain = (normed @ weights["l0.mix.uk"].T).reshape(n, c["heads"], c["dim"])
        scores = (np.einsum("qhd,khd->qhk", q[..., : c["dim"]], k_plain) + np.einsum("qhd,kd->qhk", q_rot, k_rot)) * c["scale"]
        sink = weights["l0.mix.sink"][None, :, None]
    p = plain.sink_softmax(scores, plain.causal_mask(n)[:, None, :], sink)
    return np.stack([p.max(-1), p.argmax(-1)], axis=-1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SHARP))
def test_keys_far_back_and_at_page_borders_decide_the_logits(tmp_path, name, dtype):
    config = SHARP[name]
    folder, weights = write_model(tmp_path / name, config, 5)
    tokens = tokens_for(config, 700, 3)
    # the test shows what it is meant to: late queries mostly give most of their weight to one key, and those keys lie all over
    # the context, also hundreds of tokens back and on both sides of page borders
    top = attention_weights_of(config, weights, tokens)[500:]
    assert np.median(top[..., 0]) > 0.5
    distance = (np.arange(500, 700)[:, None] - top[..., 1])[top[..., 0] > 0.5]
    assert (distance > 300).sum() > 20 and {int(p) % 16 for p in top[..., 1].reshape(-1)} >= {0, 15}
    want = plain.forward(tokens, weights, config)
    engine = load_engine(folder, dtype)
    whole = run_schedule(engine, {"a": tokens}, [[("a", 700)]])["a"]
    assert close_enough(whole, want, dtype)
    cut = run_schedule(engine, {"a": tokens}, [[("a", 333)], [("a", 2)], [("a", 300)]] + [[("a", 1)]] * 65)["a"]
    assert close_enough(cut, want, dtype)


def test_a_sink_takes_its_share_and_no_more(tmp_path):
    """A sink far above the scores silences its head, one far below them changes nothing; both through the engine's kernels."""
    config = CONFIGS["E"]
    folder, weights = write_model(tmp_path / "sink", config, 8)
    tokens = tokens_for(config, 80, 1)
    from lalamo_b200.weights.safetensors_io import write_safetensors

    for sinks in ([60.0, -60.0, 0.0], [-60.0, 2.0, 60.0]):
        changed = dict(weights, **{"l0.mix.sink": np.asarray(sinks)})
        write_safetensors(folder / "model.safetensors", {key: torch.from_numpy(np.asarray(value)).to(torch.bfloat16) for key, value in changed.items()})
        want = plain.forward(tokens, changed, config)
        assert row_errors(plain.forward(tokens, weights, config), want).max() > 0.05   # the sinks matter
        for dtype in ("float32", "bfloat16"):
            engine = load_engine(folder, dtype)
            got = run_schedule(engine, {"a": tokens}, [[("a", 50)]] + [[("a", 1)]] * 30)["a"]
            assert close_enough(got, want, dtype), (sinks, dtype)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(models, name):
    from lalamo_b200 import GenerationConfig, LanguageModel

    folder, weights = models[name]
    config = CONFIGS[name]
    model_ = LanguageModel.load(folder, dtype="float32", max_tokens=1024, max_requests=4)
    prompts = [tokens_for(config, count, 30 + count) for count in (1, 9, 30, 47, 2, 18)]
    produced = model_.generate_tokens(prompts, GenerationConfig(temperature=0.0), max_output_length=12, eos_token_ids=[])
    compared = 0
    for prompt, generated in zip(prompts, produced):
        assert len(generated) == 12
        sequence = list(prompt)
        for token in generated:
            logits = plain.forward(sequence, weights, config)[-1]
            best = np.sort(logits)[-2:]
            if best[1] - best[0] < 1e-4:
                break   # a tie within 32-bit rounding: either token is right, and what follows depends on it
            assert token == int(np.argmax(logits))
            sequence.append(token)
        else:
            compared += 1
    assert compared >= 4   # sequences compared to their end
    model_.engine.executor.check_status()
    assert model_.engine.cache.free_pages() == model_.engine.cache.num_pages


def test_command_line_and_step_replay(models, tmp_path):
    """The same model through the two programs a user runs: `generate` (greedy ids of the plain implementation) and the
    step replay that writes logits (portions, two live requests, a request that ends and another in its slot)."""
    import subprocess
    import sys
    from pathlib import Path

    from trace_client import TraceRun

    root = Path(__file__).resolve().parent.parent
    folder, weights = models["B"]
    config = CONFIGS["B"]
    prompt = tokens_for(config, 11, 77)
    prompt_file = tmp_path / "prompts.txt"
    prompt_file.write_text(" ".join(str(token) for token in prompt) + "\n")
    command = [sys.executable, "-m", "lalamo_b200", "generate", str(folder), "--prompt-ids-file", str(prompt_file), "--max-tokens", "5", "--temperature", "0",
               "--dtype", "float32", "--max-cache-tokens", "256"]
    result = subprocess.run(command, cwd=root, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    produced = [json.loads(line) for line in result.stdout.splitlines() if line.startswith("{")][0]["token_ids"]
    sequence = list(prompt)
    for token in produced:
        logits = plain.forward(sequence, weights, config)[-1]
        best = np.sort(logits)[-2:]
        if best[1] - best[0] < 1e-4:
            break
        assert token == int(np.argmax(logits))
        sequence.append(token)

    requests = {name: tokens_for(config, count, 80 + count) for name, count in (("a", 40), ("b", 9), ("c", 21))}
    wanted = {name: plain.forward(tokens, weights, config) for name, tokens in requests.items()}
    run = TraceRun(folder, "float32", tmp_path / "out", 128, config["vocab"])
    steps = [([("a", 0, 17), ("b", 0, 2)], []), ([("a", 17, 18), ("b", 2, 9)], ["b"]), ([("a", 18, 40), ("c", 0, 21)], ["a", "c"])]
    for entries, ended in steps:
        got = run.step([{"id": name, "tokens": requests[name][lo:hi], "want": list(range(hi - lo))} for name, lo, hi in entries], ended)
        want = np.concatenate([wanted[name][lo:hi] for name, lo, hi in entries])
        assert row_errors(got, want).max() < FLOAT32_LIMIT
    assert run.close() == 0
