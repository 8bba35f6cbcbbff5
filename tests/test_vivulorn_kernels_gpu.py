"""The kernels Vivulorn added to the shared ones, each alone against plain arithmetic in float64: the layer norm with the
residual sum and a sublayer's bias, the stream laid beside the embedding's output, capped logits, and a sink in the latent
attention's denominator on the plain kernel, the tensor-core kernel and its split merge."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def as_int(values) -> torch.Tensor:
    return torch.tensor(values, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,dim", [(1, 64), (7, 72), (33, 1000), (300, 2048)])
def test_layer_norm_with_the_residual_sum_and_a_bias(tokens, dim, dtype):
    """Mean and variance over a row of the 32-bit stream after a sublayer's output and its bias were added; the sum is written
    back; a row whose mean dwarfs its spread keeps its spread (two passes, not a difference of means of squares)."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(tokens + dim)
    stream = generator.standard_normal((tokens, dim)).astype(np.float32)
    stream[0] = 1000.0 + 0.01 * generator.standard_normal(dim)
    delta = torch.from_numpy(generator.standard_normal((tokens, dim))).to(dtype)
    delta_bias = generator.standard_normal(dim).astype(np.float32)
    weight = (1 + 0.3 * generator.standard_normal(dim)).astype(np.float32)
    bias = generator.standard_normal(dim).astype(np.float32)
    eps = 1e-5
    total = stream.astype(np.float64) + delta.double().numpy() + delta_bias
    centred = total - total.mean(axis=-1, keepdims=True)
    want = centred / np.sqrt((centred**2).mean(axis=-1, keepdims=True) + eps) * weight + bias

    x = torch.from_numpy(stream).cuda()
    out = torch.empty(tokens, dim, dtype=dtype, device="cuda")
    ops.rmsnorm(x, torch.from_numpy(weight).cuda(), out, eps, delta=ops.BiasedSum(delta.cuda(), torch.from_numpy(delta_bias).cuda()), write_back=True,
                exact=True, bias=torch.from_numpy(bias).cuda(), centred=True)
    assert np.abs(x.double().cpu().numpy() - total).max() < 4e-7 * max(1.0, np.abs(total).max())
    got = out.double().cpu().numpy()
    # the first row's spread is 0.01 around 1000 plus the delta's: float32 holds it to a few parts in 1e4 of the spread
    limit = 2e-3 if dtype == torch.float32 else 0.05
    assert np.abs(got - want).max() < limit * max(1.0, np.abs(want).max())

    # without a delta, for chosen rows only
    rows = [tokens - 1, 0] if tokens > 1 else [0]
    out = torch.empty(len(rows), dim, dtype=dtype, device="cuda")
    ops.rmsnorm(x, torch.from_numpy(weight).cuda(), out, eps, rows=as_int(rows), exact=True, bias=torch.from_numpy(bias).cuda(), centred=True)
    assert np.abs(out.double().cpu().numpy() - want[rows]).max() < limit * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_stream_beside_the_embedding_output(dtype):
    from lalamo_b200 import ops

    generator = np.random.default_rng(4)
    tokens, dim, vocab, scale = 19, 72, 50, 2.5
    stream = torch.from_numpy(generator.standard_normal((tokens, dim)).astype(np.float32))
    table = torch.from_numpy(generator.standard_normal((vocab, dim))).to(dtype)
    ids = generator.integers(0, vocab, tokens)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.stream_concat(stream.cuda(), table.cuda(), as_int(ids.tolist()), scale, status)
    assert int(status.item()) == 0 and got.shape == (tokens, 2 * dim) and got.dtype == dtype
    want = torch.cat([stream.to(dtype), (table[ids].float() * scale).to(dtype)], dim=1)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("factor,cap", [(1.0, 5.0), (0.25, 30.0), (2.0, 0.0)])
def test_capped_logits(factor, cap):
    from lalamo_b200 import ops

    logits = torch.tensor([[0.0, 0.1, -0.1, 4.0, -7.0, 60.0, -1e4, 1e30]], dtype=torch.float32)
    got = logits.cuda().clone()
    ops.scale_(got, factor, cap)
    scaled = logits.double() * factor
    want = cap * torch.tanh(scaled / cap) if cap > 0 else scaled
    assert torch.allclose(got.cpu().double(), want, rtol=1e-5, atol=1e-6)
    if cap > 0:
        assert float(got.abs().max()) <= cap


def rows_in_pages(rows: np.ndarray, page_size: int, dtype: torch.dtype, seed: int):
    """Rows ``[n, latent + rope]`` of one request in shuffled pages among NaN."""
    n, full = rows.shape
    blocks = -(-n // page_size)
    order = np.random.default_rng(seed).permutation(blocks + 5)[:blocks]
    pages = torch.full((blocks + 5, page_size, 1, full), float("nan"), dtype=dtype, device="cuda")
    source = torch.from_numpy(rows).to(dtype).cuda()
    for block, page in enumerate(order.tolist()):
        count = min(page_size, n - block * page_size)
        pages[page, :count, 0] = source[block * page_size : block * page_size + count]
    return pages, as_int(order.tolist()).reshape(1, -1)


def sums_with_a_sink(q: np.ndarray, rows: np.ndarray, latent: int, scale: float, sink: np.ndarray) -> np.ndarray:
    """``out[t, h] = sum_{j <= t} e^{s_j} row_j[:latent] / (sum_{j <= t} e^{s_j} + e^{sink_h})``, ``s_j = q[t, h] . row_j * scale``."""
    out = np.zeros((q.shape[0], q.shape[1], latent))
    for t in range(q.shape[0]):
        seen = rows[: t + 1]
        for head in range(q.shape[1]):
            scores = seen @ q[t, head] * scale
            top = max(scores.max(), sink[head])
            weights = np.exp(scores - top)
            out[t, head] = weights @ seen[:, :latent] / (weights.sum() + math.exp(sink[head] - top))
    return out


@pytest.mark.parametrize("splits", [0, 1, 3, 32])
@pytest.mark.parametrize("latent,rope,heads", [(64, 32, 4), (256, 32, 16), (32, 16, 3)])
def test_a_sink_in_the_latent_attention_denominator(latent, rope, heads, splits):
    """Every position of a 300-token request with sinks below, among and far above the scores, one head with a sink so large
    that its output vanishes; on the plain kernel (``splits`` 0, also in 32-bit) and on the tensor-core kernel with the
    cached rows in one CTA or shared out over several, whose merge must count the sink once."""
    from lalamo_b200 import ops

    generator = np.random.default_rng(latent + heads)
    n, page_size, full, scale = 300, 16, latent + rope, 0.5
    sink = np.linspace(-6.0, 6.0, heads)
    sink[-1] = 60.0
    for dtype in ([torch.float32, torch.bfloat16] if splits == 0 else [torch.bfloat16]):
        rows = 0.4 * generator.standard_normal((n, full))
        q = 0.6 * generator.standard_normal((n, heads, full))
        rows, q = (torch.from_numpy(a).to(dtype).double().numpy() for a in (rows, q))
        want = sums_with_a_sink(q, rows, latent, scale, sink)
        assert np.abs(want[:, -1]).max() < 1e-12 and np.abs(want[:, 0]).max() > 0.05
        pages, table = rows_in_pages(rows, page_size, dtype, heads)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = torch.full((n, heads, latent), float("nan"), dtype=dtype, device="cuda")
        common = dict(positions=torch.arange(n, dtype=torch.int32, device="cuda"), token_segment=torch.zeros(n, dtype=torch.int32, device="cuda"),
                      block_table=table, num_heads=heads, latent=latent, rope=rope, scale=scale, window=None, status=status,
                      sink=torch.from_numpy(sink).float().cuda())
        if splits == 0:
            ops.latent_attention_plain(torch.from_numpy(q).to(dtype).cuda().contiguous(), pages, out, **common)
        else:
            run = ops.latent_attention_tiling(heads)[1]
            items = [(first, min(run, n - first)) for first in range(0, n, run)]
            ops.latent_attention(torch.from_numpy(q).to(dtype).cuda().contiguous(), pages, out, items=as_int(np.asarray(items).reshape(-1)),
                                 num_items=len(items), splits=splits, **common)
        assert int(status.item()) == 0
        got = out.double().cpu().numpy()
        worst = np.abs(got - want).max(axis=(1, 2))
        assert worst.max() < (1e-4 if dtype == torch.float32 else 0.03), (dtype, int(worst.argmax()), float(worst.max()))
