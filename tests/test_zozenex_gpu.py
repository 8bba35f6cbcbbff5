"""The Zozenex design on the GPU against the plain restatement (``plain_zozenex.py``): each mechanism's kernels alone, then
whole models through the engine: prompts at once, decoding through the caches and the recurrent states, portions of every
size, mixed batches with pages and slots that are freed and used again, keys far back and at every edge (page, window,
block), long decoding, and greedy generation through the Python entry point and the command line."""

from __future__ import annotations

import copy
import json

import numpy as np
import pytest
import torch

import plain_zozenex as plain
from tiny_zozenex import CONFIGS, DECAY_RANK, layer, left, model, moe, retention, right, write_model

pytestmark = pytest.mark.gpu

FLOAT32_LIMIT = 2e-4   # of the logits' spread; 32-bit sums of a few hundred terms stay far below
BFLOAT16_LIMIT = 0.08


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("zozenex")
    return {name: write_model(root / name, config, 40 + seed, DECAY_RANK[name]) for seed, (name, config) in enumerate(CONFIGS.items())}


def tokens_for(config: dict, count: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, config["vocab"], size=count).tolist()


MAX_SLACK = 0.05   # by how much a left-out expert's choice score may beat a chosen one's where bfloat16 rounding turned a close call


def expected(config: dict, weights: dict, tokens: list[int], choices: dict | None = None) -> np.ndarray:
    """The plain implementation's logits.  With ``choices`` (what :func:`run_schedule` recorded of the engine's routers) the plain
    experts are the engine's, and the engine's choice must be the plain one up to close calls."""
    slack: list[float] = []
    logits = plain.forward(config, weights, tokens, choices=choices, slack=slack).numpy()
    assert not slack or max(slack) < MAX_SLACK, max(slack)
    return logits


def routed(config: dict) -> bool:
    return any(entry["mlp"] is not None for entry in config["layers"])


def follows_choices(config: dict, dtype: str) -> bool:
    """bfloat16 rounding of a router's input can turn a close call between two experts, which no limit on rounding errors covers (and
    random weights make a few in a hundred tokens, whose effect the recurrent states then carry on): there the plain implementation
    is given the engine's choices, which are checked against its own scores, and every row is held to the limit all the same."""
    return dtype == "bfloat16" and routed(config)


def load_engine(folder, dtype: str, max_tokens: int = 1024, config: dict | None = None, **options):
    from lalamo_b200.engine.engine import Engine, EngineConfig

    if config is not None and follows_choices(config, dtype):
        options.setdefault("cuda_graphs", False)   # the routers' choices are read after every launch
    return Engine.load(folder, EngineConfig(dtype=dtype, page_size=16, max_tokens=max_tokens, max_requests=4, poison_freed=True, **options))


def row_errors(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: the spread of the difference (its mean taken off) over the spread of the wanted logits."""
    difference = got - want
    difference = difference - difference.mean(axis=-1, keepdims=True)
    centred = want - want.mean(axis=-1, keepdims=True)
    return np.sqrt((difference**2).mean(axis=-1)) / np.sqrt((centred**2).mean())


def run_schedule(engine, requests: dict[str, list[int]], schedule: list[list[tuple[str, int]]], choices: dict | None = None) -> dict[str, np.ndarray]:
    """Feeds the requests' tokens in the schedule's portions (every step one batch), asks for every position's logits,
    ends a request with its last token, and checks the cache's books after every step.  ``choices`` (a dict) receives what the
    routers chose: request -> router (in the order they run) -> [tokens, top]; needs an engine that replays nothing."""
    from lalamo_b200 import ops
    from lalamo_b200.engine.executor import StepEntry

    done = {name: 0 for name in requests}
    rows: dict[str, list[np.ndarray]] = {name: [] for name in requests}
    seen: list[torch.Tensor] = []
    route = ops.moe_route

    def recording_route(*args, **kwargs):
        result = route(*args, **kwargs)
        seen.append(result[0])
        return result

    if choices is not None:
        ops.moe_route = recording_route
    try:
        for step in schedule:
            entries = []
            for name, count in step:
                if done[name] == 0:
                    engine.admit(name)
                entries.append(StepEntry(name, requests[name][done[name] : done[name] + count], list(range(count))))
            seen.clear()
            logits = engine.step(entries).float().cpu().numpy()
            offset = 0
            for name, count in step:
                rows[name].append(logits[offset : offset + count])
                if choices is not None:
                    for router, chosen in enumerate(seen):
                        choices.setdefault(name, {}).setdefault(router, []).append(chosen[offset : offset + count].cpu())
                offset += count
                done[name] += count
                if done[name] == len(requests[name]):
                    engine.release(name)
            engine.executor.check_status()
            engine.cache.check()
    finally:
        ops.moe_route = route
    assert all(done[name] == len(tokens) for name, tokens in requests.items())
    return {name: np.concatenate(parts) for name, parts in rows.items()}


def compare(engine, config: dict, weights: dict, requests: dict[str, list[int]], schedule: list, dtype: str, first_rows: int | None = None) -> dict[str, np.ndarray]:
    """Runs the schedule and holds every row of every request to the limit of the type against the plain implementation."""
    follow = follows_choices(config, dtype)
    recorded: dict = {}
    got = run_schedule(engine, requests, schedule, recorded if follow else None)
    routers = [index for index, entry in enumerate(config["layers"]) if entry["mlp"] is not None]
    for name, tokens in requests.items():
        choices = {layer_index: torch.cat(recorded[name][router]) for router, layer_index in enumerate(routers)} if follow else None
        want = expected(config, weights, tokens, choices)
        errors = row_errors(got[name], want)
        assert errors.max() < (FLOAT32_LIMIT if dtype == "float32" else BFLOAT16_LIMIT), (name, int(errors.argmax()), float(errors.max()))
    return got


# ----------------------------------------------------------------------------- mechanisms alone
def test_linear_recurrence_kernels_with_both_kinds_of_decay():
    """The recurrence's kernels against the plain recurrence: portions of unequal lengths from states that are not zero, heads whose key
    and value sizes differ and fit no vector width, a fixed decay per head and a decay per channel made from logits."""
    from lalamo_b200 import ops

    device = torch.device("cuda")
    generator = torch.Generator().manual_seed(3)
    for heads, dk, dv, fixed in ((3, 12, 20, True), (2, 40, 8, False), (1, 64, 64, False), (4, 32, 32, True)):
        lengths = [5, 1, 37]
        tokens = sum(lengths)
        gate_offset = -(-(2 * heads * dk + heads * dv) // 8) * 8
        proj = torch.randn(tokens, gate_offset + heads * dv, generator=generator)
        logits = 2.0 + torch.randn(tokens, heads * dk, generator=generator)
        bias = torch.randn(heads * dk, generator=generator)
        decays = torch.tensor([0.9 - 0.1 * h for h in range(heads)])
        weight = 1.0 + 0.1 * torch.randn(dv, generator=generator)
        state = torch.randn(5, heads, dk, dv, generator=generator)
        slots = [3, 0, 4]
        starts = np.cumsum([0] + lengths[:-1]).tolist()
        on = lambda t, dtype=torch.float32: t.to(device=device, dtype=dtype).contiguous()
        device_state = on(state)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        out = ops.linear_attention(on(proj), device_state, num_heads=heads, key_dim=dk, value_dim=dv, decay_logits=None if fixed else on(logits),
                                   decay_bias=None if fixed else on(bias), fixed_decay=on(decays) if fixed else None, tau=3.0, query_scale=dk ** -0.5,
                                   norm_weight=on(weight), norm_eps=1e-5, gate_offset=gate_offset, gate_activation="silu",
                                   segment_start=on(torch.tensor(starts), torch.int32), segment_length=on(torch.tensor(lengths), torch.int32),
                                   segment_slot=on(torch.tensor(slots), torch.int32), segments=3, status=status)
        assert int(status.item()) == 0
        p = proj.double()
        for start, length, slot in zip(starts, lengths, slots):
            rows = p[start : start + length]
            q = rows[:, : heads * dk].reshape(length, heads, dk) * dk ** -0.5
            k = rows[:, heads * dk : 2 * heads * dk].reshape(length, heads, dk)
            v = rows[:, 2 * heads * dk : 2 * heads * dk + heads * dv].reshape(length, heads, dv)
            if fixed:
                decay = decays.double()[None, :, None].expand(length, heads, dk)
            else:
                decay = torch.sigmoid(logits[start : start + length].double() + bias.double()).pow(1.0 / 3.0).reshape(length, heads, dk)
            s = state[slot].double().clone()
            want = torch.zeros(length, heads, dv, dtype=torch.float64)
            for t in range(length):
                s = decay[t][:, :, None] * s + k[t][:, :, None] * v[t][:, None, :]
                want[t] = torch.einsum("hkv,hk->hv", s, q[t])
            gate = rows[:, gate_offset : gate_offset + heads * dv]
            want = (plain.rms_norm(want, weight.double(), 1e-5).reshape(length, heads * dv) * plain.silu(gate))
            assert torch.allclose(out[start : start + length].double().cpu(), want, rtol=2e-4, atol=2e-4), (heads, dk, dv, fixed)
            assert torch.allclose(device_state[slot].double().cpu(), s, rtol=1e-4, atol=1e-4)


def test_branch_norms_and_learned_positions():
    from lalamo_b200 import ops

    device = torch.device("cuda")
    generator = torch.Generator().manual_seed(4)
    a, b = torch.randn(7, 72, generator=generator), 3.0 * torch.randn(7, 72, generator=generator)
    wa, wb = torch.randn(72, generator=generator), torch.randn(72, generator=generator)
    residual = torch.randn(7, 72, generator=generator)
    for dtype in (torch.float32, torch.bfloat16):
        a_, b_ = a.to(dtype), b.to(dtype)
        stream = residual.to(device).clone()
        ops.branch_norms_accumulate(stream, [(a_.to(device), wa.to(device), 0.5), (b_.to(device), wb.to(device), 0.25)], 1e-5)
        want = residual.double() + 0.5 * plain.rms_norm(a_.double(), wa.double(), 1e-5) + 0.25 * plain.rms_norm(b_.double(), wb.double(), 1e-5)
        assert torch.allclose(stream.double().cpu(), want, rtol=1e-5, atol=1e-5)
    table, position_table = torch.randn(11, 16, generator=generator), torch.randn(9, 16, generator=generator)
    ids, positions = torch.tensor([3, 10, 0, 3], dtype=torch.int32), torch.tensor([0, 8, 5, 1], dtype=torch.int32)
    out = torch.empty(4, 16, dtype=torch.float32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ops.embed(table.to(device), ids.to(device), out, 1.0, status)
    ops.embed(position_table.to(device), positions.to(device), out, 1.0, status, accumulate=True)
    assert torch.equal(out.cpu(), table[ids.long()] + position_table[positions.long()]) and int(status.item()) == 0


def test_router_with_a_choice_bias_and_experts_without_a_gate():
    """Experts ranked by score plus correction and weighed by the score alone; a gate row behind the experts' rows; experts without a
    gate on all three paths (streamed, grouped on the tensor cores, plain) against the plain sum."""
    from lalamo_b200 import ops

    device = torch.device("cuda")
    generator = torch.Generator().manual_seed(5)
    tokens, width, experts, top, ff = 70, 64, 6, 2, 24
    x = torch.randn(tokens, width, generator=generator).to(torch.bfloat16)
    router = torch.randn(experts + 1, width, generator=generator) / 4
    correction = torch.tensor([0.4, -0.3, 0.0, 0.9, -0.9, 0.2])
    up = (torch.randn(experts, ff, width, generator=generator) / 8).to(torch.bfloat16)
    down = (torch.randn(experts, width, ff, generator=generator) / 5).to(torch.bfloat16)
    chosen, weights, gate = ops.moe_route(x.to(device), router.to(device), top=top, score="sigmoid", weight_scale=1.5, choice_bias=correction.to(device), extra=1)
    scores = torch.sigmoid(x.double() @ router.double().T)
    order = torch.argsort(-(scores[:, :experts] + correction.double()), dim=1, stable=True)[:, :top]
    assert torch.equal(chosen.cpu().long(), order)
    assert torch.allclose(weights.cpu().double(), 1.5 * torch.gather(scores[:, :experts], 1, order), rtol=1e-5)
    assert torch.allclose(gate.cpu().double()[:, 0], scores[:, experts], rtol=1e-5)
    assert not torch.equal(order, torch.argsort(-scores[:, :experts], dim=1, stable=True)[:, :top])   # the correction decides somewhere
    want = torch.zeros(tokens, width, dtype=torch.float64)
    for t in range(tokens):
        for j in range(top):
            e = int(order[t, j])
            hidden = plain.gelu(x[t].double() @ up[e].double().T).to(torch.bfloat16).double()
            want[t] += weights[t, j].cpu().double() * (hidden @ down[e].double().T)
    for path in ("grouped", "stream", "plain"):
        out = ops.moe_experts(x.to(device), None, up.to(device), down.to(device), chosen, weights, "gelu", path=path)
        assert torch.allclose(out.double().cpu(), want, rtol=2e-2, atol=2e-2), path
    shared = torch.randn(tokens, width, generator=generator).to(torch.bfloat16)
    stream = torch.zeros(tokens, width, dtype=torch.float32, device=device)
    routed_sum = ops.moe_experts(x.to(device), None, up.to(device), down.to(device), chosen, weights, "gelu", combine=False)
    ops.moe_combine_add(routed_sum, stream, shared.to(device), gate)
    assert torch.allclose(stream.double().cpu(), want + scores[:, experts : experts + 1] * shared.double(), rtol=2e-2, atol=2e-2)


def pooled_case(dtype, heads, groups, dk, dv, window, pool, rot_dims, page_size, contexts, lengths, cap, seed, tensor_cores=False, shares=None, alone=True):
    """One step of the pooled attention's kernels over requests that hold ``contexts`` tokens already and bring ``lengths`` more (the
    earlier tokens go through the same kernels, one request a step, in uneven portions), against the plain attention over each
    request's whole sequence.  Pages are handed out in a scattered order.  ``tensor_cores``: the last step's attention on the tensor-core
    kernels: portions in tiles of consecutive tokens, portions of one token on the kernel of tokens that attend alone (``alone=False``: as
    tiles of one token too); ``shares``: so many CTAs share out a tile's rows; left out, the launch's shape decides."""
    from lalamo_b200 import ops

    device = torch.device("cuda")
    generator = torch.Generator().manual_seed(seed)
    totals = [c + n for c, n in zip(contexts, lengths)]
    width = heads * dk + groups * (dk + dv)
    rows = [(3.0 * torch.randn(total, width, generator=generator)).to(dtype) for total in totals]
    bias = -2.0 + torch.randn(heads, generator=generator)
    base, scale = 200.0, 0.3
    blocks_per_request = -(-max(totals) // page_size)
    pages = blocks_per_request * len(totals) + 3
    pool_rows = -(-page_size // pool)
    order = torch.randperm(pages, generator=generator).tolist()
    table = torch.tensor([[order[r * blocks_per_request + b] for b in range(blocks_per_request)] for r in range(len(totals))], dtype=torch.int32, device=device)
    token_pages = torch.full((pages, page_size, groups, dk + dv), float("nan"), dtype=dtype, device=device)   # a row: key | value
    pool_pages = torch.full((pages, pool_rows, groups, dk + dv), float("nan"), dtype=dtype, device=device)
    qk_freq = (1.0 / (torch.tensor(base) ** (torch.arange(0, rot_dims, 2, dtype=torch.float32) / rot_dims))).to(device) if rot_dims else None
    v_freq = (1.0 / (torch.tensor(base) ** (torch.arange(0, dv, 2, dtype=torch.float32) / dv))).to(device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    as_int = lambda values: torch.tensor(values, dtype=torch.int32, device=device)

    def step(portions, on_tensor_cores=False):   # [(request, first position, count)]
        tokens = sum(count for _, _, count in portions)
        qkv = torch.cat([rows[r][first : first + count] for r, first, count in portions]).to(device)
        positions = as_int([p for _, first, count in portions for p in range(first, first + count)])
        segment = as_int([index for index, (_, _, count) in enumerate(portions) for _ in range(count)])
        step_table = table[[r for r, _, _ in portions]].contiguous()
        q = torch.empty(tokens, heads * dk, dtype=dtype, device=device)
        shape = dict(num_heads=heads, num_groups=groups, head_dim=dk, value_dim=dv)
        ops.pooled_rewrite(qkv, q, token_pages, qk_freq=qk_freq, rotary_dim=rot_dims, value_freq=v_freq, positions=positions, token_segment=segment,
                           block_table=step_table, write_kv=True, status=status, **shape)
        ops.pooled_means(token_pages, pool_pages, segment_length=as_int([count for _, _, count in portions]),
                         segment_context=as_int([first for _, first, _ in portions]), block_table=step_table, pool_table=step_table, segments=len(portions),
                         max_length=max(count for _, _, count in portions), num_groups=groups, head_dim=dk, value_dim=dv, pool=pool, status=status)
        out = torch.empty(tokens, heads * dv, dtype=dtype, device=device)
        common = dict(positions=positions, token_segment=segment, block_table=step_table, pool_table=step_table, scale=scale, softcap=cap,
                      head_bias=bias.to(device), window=window, pool=pool, value_freq=v_freq, status=status, **shape)
        if on_tensor_cores:
            size = ops.pooled_attention_tiling(heads, groups)[1]
            starts = np.cumsum([0] + [count for _, _, count in portions[:-1]]).tolist()
            tiles = [(first, min(size, start + count - first)) for start, (_, _, count) in zip(starts, portions) if count > 1 or not alone
                     for first in range(start, start + count, size)]
            singles = [start for start, (_, _, count) in zip(starts, portions) if count == 1 and alone]
            # what the allocator hands out next holds NaN: a kernel that reads 32-bit sums which no CTA of its launch wrote shows it
            for size in range(1, 17):
                junk = torch.full((size, tokens, heads * dv), float("nan"), dtype=torch.float32, device=device)
                del junk
            if tiles:
                ops.pooled_attention(q, token_pages, pool_pages, out, tiles=as_int([v for tile in tiles for v in tile]), num_tiles=len(tiles), shares=shares, **common)
            for size in range(1, 17):
                junk = torch.full((size, tokens, heads * dv), float("nan"), dtype=torch.float32, device=device)
                del junk
            if singles:
                ops.pooled_attention_single(q, token_pages, pool_pages, out, singles=as_int(singles), num_singles=len(singles), shares=shares, **common)
        else:
            ops.pooled_attention_plain(q, token_pages, pool_pages, out, **common)
        return out

    for r, context in enumerate(contexts):
        first = 0
        for count in (3, 1, 2, 11, 1, 40):
            count = min(count, context - first)
            if count > 0:
                step([(r, first, count)])
                first += count
        while first < context:
            count = min(64, context - first)
            step([(r, first, count)])
            first += count
    got = step([(r, context, count) for r, (context, count) in enumerate(zip(contexts, lengths))], tensor_cores).double().cpu()
    assert int(status.item()) == 0
    offset = 0
    worst = 0.0
    for r, (context, count) in enumerate(zip(contexts, lengths)):
        whole = rows[r].double()
        total = totals[r]
        positions = torch.arange(total)
        q = plain.rotate_halves(whole[:, : heads * dk].reshape(total, heads, dk), positions, rot_dims, base)
        k = plain.rotate_halves(whole[:, heads * dk : heads * dk + groups * dk].reshape(total, groups, dk), positions, rot_dims, base)
        v = plain.rotate_halves(whole[:, heads * dk + groups * dk :].reshape(total, groups, dv), positions, dv, base)
        k, v = k.to(dtype).double(), v.to(dtype).double()   # as the cache holds them
        want = torch.zeros(count, heads, dv, dtype=torch.float64)
        for n in range(count):
            i = context + n
            first = max(0, i - window + 1)
            seen = max(0, (i - window + 1) // pool)
            keys = torch.cat([k[: seen * pool].reshape(seen, pool, groups, dk).mean(1).to(dtype).double(), k[first : i + 1]])
            values = torch.cat([v[: seen * pool].reshape(seen, pool, groups, dv).mean(1).to(dtype).double(), v[first : i + 1]])
            for head in range(heads):
                g = head // (heads // groups)
                score = (keys[:, g] @ q[i, head].to(dtype).double()) * scale
                if cap > 0:
                    score = cap * torch.tanh(score / cap)
                want[n, head] = torch.sigmoid(score + bias[head].double()) @ values[:, g]
        want = plain.rotate_halves(want, positions[context:], dv, base, sign=-1.0).reshape(count, heads * dv)
        error = (got[offset : offset + count] - want).abs().max() / want.abs().max()
        worst = max(worst, float(error))
        offset += count
    return worst


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pooled_attention_kernels_at_every_edge(dtype):
    """Single tokens and portions whose first, last or only token lies just before, on and just after a window's edge, a block's last
    position and a page's border; blocks longer than a page, than the window, and blocks that divide neither."""
    limit = 2e-5 if dtype == torch.float32 else 2e-2
    cases = [
        dict(heads=4, groups=2, dk=16, dv=24, window=10, pool=4, rot_dims=8, page_size=16, contexts=[0, 9, 10, 13, 14, 31, 32, 47], lengths=[1] * 8, cap=20.0),
        dict(heads=2, groups=2, dk=24, dv=8, window=16, pool=16, rot_dims=0, page_size=16, contexts=[15, 16, 31, 32, 33, 95], lengths=[1, 1, 1, 1, 1, 1], cap=0.0),
        dict(heads=3, groups=1, dk=8, dv=12, window=7, pool=24, rot_dims=8, page_size=16, contexts=[22, 23, 29, 30, 31, 54], lengths=[1, 2, 1, 1, 5, 40], cap=5.0),
        dict(heads=2, groups=1, dk=32, dv=32, window=1, pool=3, rot_dims=16, page_size=16, contexts=[0, 1, 2, 3, 4, 50], lengths=[1, 1, 1, 1, 33, 2], cap=30.0),
        dict(heads=6, groups=6, dk=64, dv=40, window=100, pool=12, rot_dims=64, page_size=16, contexts=[0, 99, 111, 112, 200], lengths=[130, 1, 1, 1, 17], cap=28.0),
    ]
    for index, case in enumerate(cases):
        assert pooled_case(dtype, seed=20 + index, **case) < limit, case


def test_pooled_attention_on_the_tensor_cores_at_every_edge():
    """The tensor-core kernel over the same kinds of edges: heads of 16 to 128 channels with keys and values of different sizes, one
    to eight query heads a K/V head, tiles that end inside a portion, windows and blocks that begin and end inside a tile of 64 rows."""
    cases = [
        dict(heads=4, groups=2, dk=16, dv=32, window=10, pool=4, rot_dims=8, page_size=16, contexts=[0, 9, 10, 13, 14, 31, 32, 47], lengths=[1] * 8, cap=20.0),
        dict(heads=2, groups=2, dk=32, dv=16, window=16, pool=16, rot_dims=0, page_size=16, contexts=[15, 16, 31, 32, 33, 95], lengths=[1, 1, 1, 1, 1, 70], cap=0.0),
        dict(heads=3, groups=1, dk=16, dv=16, window=7, pool=24, rot_dims=8, page_size=16, contexts=[22, 23, 29, 30, 31, 54], lengths=[1, 2, 1, 1, 5, 40], cap=5.0),
        dict(heads=8, groups=1, dk=32, dv=32, window=1, pool=3, rot_dims=16, page_size=16, contexts=[0, 1, 2, 3, 4, 50], lengths=[1, 1, 1, 1, 33, 2], cap=30.0),
        dict(heads=6, groups=6, dk=64, dv=32, window=100, pool=12, rot_dims=64, page_size=16, contexts=[0, 99, 111, 112, 200, 700], lengths=[130, 1, 1, 1, 17, 1], cap=28.0),
        dict(heads=4, groups=1, dk=128, dv=128, window=70, pool=5, rot_dims=64, page_size=16, contexts=[0, 69, 330], lengths=[150, 3, 1], cap=30.0),
        dict(heads=6, groups=3, dk=80, dv=96, window=130, pool=2, rot_dims=80, page_size=32, contexts=[0, 260], lengths=[200, 66], cap=12.0),
        dict(heads=40, groups=2, dk=32, dv=48, window=33, pool=7, rot_dims=16, page_size=16, contexts=[0, 1, 32, 33, 39, 40, 41, 200], lengths=[1] * 8, cap=25.0),
        dict(heads=9, groups=1, dk=48, dv=16, window=50, pool=6, rot_dims=48, page_size=16, contexts=[49, 55, 56, 120], lengths=[1, 1, 1, 1], cap=0.0),
    ]
    for index, case in enumerate(cases):
        for shares, alone in ((1, True), (None, True), (5, True), (1, False), (5, False)):   # every tile's rows in one CTA, as the launch's shape decides, shared out over five
            assert pooled_case(torch.bfloat16, seed=40 + index, tensor_cores=True, shares=shares, alone=alone, **case) < 2e-2, (case, shares, alone)


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_a_prompt_at_once_and_token_by_token(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 90, 5)
    engine = load_engine(folder, dtype, config=config)
    compare(engine, config, weights, {"a": tokens}, [[("a", len(tokens))]], dtype)
    # the first 21 at once, the rest one by one: windows and blocks pass over decoded tokens, steps replay from recordings
    compare(engine, config, weights, {"b": tokens}, [[("b", 21)]] + [[("b", 1)]] * (len(tokens) - 21), dtype)
    # from the very first token on, one by one: an empty state, a cache of one key, no block yet
    compare(engine, config, weights, {"c": tokens[:40]}, [[("c", 1)]] * 40, dtype)
    assert engine.cache.free_pages() == engine.cache.num_pages


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_stream_after_every_layer(models, name):
    from lalamo_b200 import ops

    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 70, 8)
    wanted: list = []
    plain.forward(config, weights, tokens, wanted)
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
    assert len(seen) == len(wanted) == len(config["layers"])
    for index, (got, want) in enumerate(zip(seen, wanted)):
        assert np.abs(got.cpu().numpy() - want.numpy()).max() < 2e-4 * np.abs(want.numpy()).max(), index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_every_size(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    tokens = tokens_for(config, 150, 6)
    engine = load_engine(folder, dtype, config=config)
    for cuts in ([2, 3, 2, 5, 1, 17, 1, 1, 33, 2, 16, 31, 36], [64, 2, 2, 2, 48, 32], [7] * 21 + [3], [1, 2, 147]):
        assert sum(cuts) == len(tokens)
        compare(engine, config, weights, {"a": tokens}, [[("a", count)] for count in cuts], dtype)


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
    engine = load_engine(folder, dtype, max_tokens=288, config=config)
    got = compare(engine, config, weights, requests, schedule, dtype)
    if dtype == "float32":
        # each request alone, in one piece, on the same engine: what the batch and the cutting change is rounding
        for key in ("a", "e"):
            alone = run_schedule(engine, {key: requests[key]}, [[(key, len(requests[key]))]])[key]
            assert row_errors(got[key], alone).max() < 5e-5, key
    assert engine.cache.free_pages() == engine.cache.num_pages


def test_a_request_left_out_of_steps_goes_on_later(models):
    folder, weights = models["A"]
    config = CONFIGS["A"]
    requests = {key: tokens_for(config, count, 90 + count) for key, count in (("a", 60), ("b", 45), ("c", 12))}
    schedule = [[("a", 9)], [("b", 40)], [("b", 5), ("c", 3)], [("a", 1), ("c", 9)], [("a", 50)]]
    compare(load_engine(folder, "float32", max_tokens=160), config, weights, requests, schedule, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    folder, weights = models["C"]
    config = CONFIGS["C"]
    tokens = tokens_for(config, 420, 22)
    compare(load_engine(folder, dtype, config=config), config, weights, {"a": tokens}, [[("a", 4)]] + [[("a", 1)]] * 416, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_portions_beside_a_short_request(models, name, dtype):
    folder, weights = models[name]
    config = CONFIGS[name]
    requests = {"a": tokens_for(config, 1300, 41), "b": tokens_for(config, 30, 42)}
    # 900 tokens at once: long enough for a recurrence to run as chunks side by side where its head shape makes that pay
    schedule = [[("a", 900), ("b", 5)], [("a", 1), ("b", 20)], [("a", 390), ("b", 1)], [("b", 4), ("a", 9)]]
    compare(load_engine(folder, dtype, max_tokens=2048, config=config), config, weights, requests, schedule, dtype)


@pytest.mark.parametrize("name", ["D", "E"])
def test_recorded_steps_in_bfloat16(models, name):
    """Decoding replayed from recordings in bfloat16, in models that choose no experts (the routed ones run unrecorded in bfloat16
    above, and recorded in 32-bit)."""
    folder, weights = models[name]
    config = CONFIGS[name]
    requests = {"a": tokens_for(config, 80, 51), "b": tokens_for(config, 50, 52)}
    schedule = [[("a", 30), ("b", 1)]] + [[("a", 1), ("b", 1)]] * 49 + [[("a", 1)]]
    compare(load_engine(folder, "bfloat16", cuda_graphs=True), config, weights, requests, schedule, "bfloat16")


# One key that stands out.  The weights are made so that a key's score is far above the cap if its token is the marker and zero
# otherwise, under a bias far below zero: a marker weighs one wherever it is seen (as itself inside the window; through its
# block's mean key, which keeps a quarter of its score, once the whole block lies behind the window), everything else weighs nearly
# nothing.  So a row's output is the sum of the few markers it sees, and a marker or a block that is seen one position early or late,
# or lost (far back, at a page's border, among the first tokens), changes that row's logits by about their whole spread.
MARKER, MARKER_WINDOW, MARKER_POOL = 7, 19, 4
MARKER_CONFIGS = {
    "narrow": model(96, 64, [layer("parallel", {"left": left(heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=8, base=50.0, scale=1.0, softcap=30.0,
                                                             size=MARKER_WINDOW, pool=MARKER_POOL), "right": right(heads=1, dim=8, vdim=8, tau=4.0)}, None)]),
    "heads-of-64": model(96, 128, [layer("parallel", {"left": left(heads=4, kv_heads=4, dim=64, vdim=64, rot_dims=32, base=1000.0, scale=1.0, softcap=30.0,
                                                                  size=MARKER_WINDOW, pool=MARKER_POOL), "right": right(heads=1, dim=8, vdim=8, tau=4.0)}, None)]),
}
MARKER_POSITIONS = (0, 1, 15, 16, 40, 47, 48, 130, 131, 200, 263)


def marker_model(directory, config: dict):
    """Weights as described above: channel 0 of the stream holds the marker (embedding 40 for the marker, 0 otherwise), channel 1 a
    constant; the last channel of every key head reads channel 0, the last channel of every query head channel 1, all other rows of
    the query and key projections are zero ( the last channel of a head is not rotated); the branch's output is made large beside the stream."""
    from lalamo_b200.weights.safetensors_io import write_safetensors

    folder, weights = write_model(directory, config, 9, rank=4)
    c = config["layers"][0]["mixer"]["left"]
    weights["embed"][:, 0] = 0.0
    weights["embed"][MARKER, 0] = 40.0
    weights["embed"][:, 1] = 4.0
    weights["pos"] *= 0.25
    weights["pos"][:, :2] = 0.0
    weights["l0.norm1"][:2] = 1.0
    for name, heads, source in (("l0.mix.left.q", c["heads"], 1), ("l0.mix.left.k", c["kv_heads"], 0)):
        weights[name].zero_()
        for head in range(heads):
            weights[name][head * c["dim"] + c["dim"] - 1, source] = 16.0
    weights["l0.mix.left.pb"].fill_(-15.0)
    weights["l0.mix.left.out"] *= 8.0   # this branch's output decides the logits
    weights["l0.mix.right.out"] *= 0.25
    write_safetensors(folder / "model.safetensors", {name: tensor.to(torch.bfloat16) for name, tensor in weights.items()})
    return folder, weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(MARKER_CONFIGS))
def test_single_keys_and_blocks_decide_the_logits(tmp_path, name, dtype):
    config = MARKER_CONFIGS[name]
    folder, weights = marker_model(tmp_path / name, config)
    length = 330
    tokens = [token if token != MARKER else MARKER + 1 for token in tokens_for(config, length, 3)]
    for position in MARKER_POSITIONS:
        tokens[position] = MARKER
    want = expected(config, weights, tokens)
    # the rows at which a marker leaves the window, and at which its block is first seen
    leaving = sorted({position + MARKER_WINDOW for position in MARKER_POSITIONS})
    appearing = sorted({position // MARKER_POOL * MARKER_POOL + MARKER_POOL - 1 + MARKER_WINDOW for position in MARKER_POSITIONS})
    # the test shows what it is meant to: a window one position longer keeps a marker at the row where it should have left, and
    # blocks that come into sight one position late are missed at the row where they should appear; either changes those rows'
    # logits by several times the bfloat16 limit, a thousand times the 32-bit one (and blocks of other positions change nearly every late row)
    longer = copy.deepcopy(config)
    longer["layers"][0]["mixer"]["left"]["mask"]["size"] += 1
    changed = row_errors(expected(longer, weights, tokens), want)
    assert changed[leaving].min() > 2 * BFLOAT16_LIMIT and np.median(changed[appearing]) > 3 * BFLOAT16_LIMIT
    shorter = copy.deepcopy(config)
    shorter["layers"][0]["mixer"]["left"]["mask"]["size"] -= 1
    assert np.median(row_errors(expected(shorter, weights, tokens), want)[[row - 1 for row in leaving]]) > 3 * BFLOAT16_LIMIT
    other = copy.deepcopy(config)
    other["layers"][0]["mixer"]["left"]["mask"]["pool"] += 1
    assert np.median(row_errors(expected(other, weights, tokens), want)[100:]) > 3 * BFLOAT16_LIMIT
    engine = load_engine(folder, dtype)
    compare(engine, config, weights, {"a": tokens}, [[("a", length)]], dtype)
    compare(engine, config, weights, {"a": tokens}, [[("a", 2)], [("a", 15)], [("a", 118)], [("a", 2)], [("a", 100)]] + [[("a", 1)]] * 93, dtype)
    compare(engine, config, weights, {"a": tokens[:120]}, [[("a", 1)]] * 120, dtype)


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
            logits = expected(config, weights, sequence)[-1]
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
        logits = expected(config, weights, sequence)[-1]
        best = np.sort(logits)[-2:]
        if best[1] - best[0] < 1e-4:
            break
        assert token == int(np.argmax(logits))
        sequence.append(token)

    requests = {name: tokens_for(config, count, 80 + count) for name, count in (("a", 40), ("b", 9), ("c", 21))}
    wanted = {name: expected(config, weights, tokens) for name, tokens in requests.items()}
    run = TraceRun(folder, "float32", tmp_path / "out", 128, config["vocab"], poison_freed=True)
    steps = [([("a", 0, 17), ("b", 0, 2)], []), ([("a", 17, 18), ("b", 2, 9)], ["b"]), ([("a", 18, 40), ("c", 0, 21)], ["a", "c"])]
    for entries, ended in steps:
        got = run.step([{"id": name, "tokens": requests[name][lo:hi], "want": list(range(hi - lo))} for name, lo, hi in entries], ended)
        want = np.concatenate([wanted[name][lo:hi] for name, lo, hi in entries])
        assert row_errors(got, want).max() < FLOAT32_LIMIT
    assert run.close() == 0
