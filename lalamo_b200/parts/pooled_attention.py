"""Grouped attention with sigmoid weights under a sliding window, with one mean key and mean value for every whole block
of positions before the window (see :class:`~lalamo_b200.config.plan.PooledWindowAttentionSpec`).

The mixer holds two paged caches whose rows hold a key and its value side by side: the positions' under the window's
retention rule (pages go back once the window and every unfinished block have passed them), and the blocks' means, one
row per block, which are kept for good.  A step rotates q, k and v and writes the pages, computes the mean of every block it completed from the pages, and
then attends: the visible blocks first, then the window's positions upwards, the weights ``sigmoid(cap(q . k scale) +
bias_h)`` summed with the values in 32-bit without any normalisation; rotated values are turned back by the query's
position at the end.  In bfloat16, for heads of multiples of 16 channels, the attention runs on the tensor cores: portions in tiles of
consecutive tokens, tokens that attend alone (decoding) on a kernel of their own whose products have the cache's rows as rows and the
query heads as columns; otherwise, and in 32-bit, a block per token and head computes it plainly."""

from __future__ import annotations

from typing import Mapping

import numpy as np
import torch

from .. import ops
from ..config.plan import PooledWindowAttentionSpec, RopeSpec
from .base import CacheNeed, CompositeNeed, CompositeView, HostSegments, Mixer, PagedKVNeed, PagedKVView, Runtime, StepInputs, TensorDecl, register_part

__all__ = ["PooledWindowAttention"]


def _frequencies(dims: int, theta: float) -> torch.Tensor:
    """``theta ** (-2m / dims)`` for the pairs ``m`` of ``dims`` channels, as the 32-bit table the kernels multiply positions with."""
    channel = torch.arange(0, dims, 2, dtype=torch.float32)
    return 1.0 / (torch.tensor(theta, dtype=torch.float32) ** (channel / dims))


@register_part(PooledWindowAttentionSpec)
class PooledWindowAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: PooledWindowAttentionSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if spec.num_heads % spec.num_groups:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_groups={spec.num_groups}")
        if spec.window < 1 or spec.pool < 0 or spec.softcap < 0.0:
            raise ValueError("the window must be positive, the block size and the cap not negative")
        if spec.position is not None and not isinstance(spec.position, RopeSpec):
            raise ValueError(f"pooled window attention applies rotary position encodings, not {type(spec.position).__name__}")
        if spec.rotate_values and (spec.position is None or spec.value_dim % 2):
            raise ValueError("rotated values need a rotary specification (for the base) and an even value_dim")
        if spec.position is not None and spec.position.pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {spec.position.pairing!r}; known: 'half', 'interleaved'")
        if spec.position is not None and spec.position.scaling is not None:
            raise ValueError("stretched frequencies are not supported here")
        self.qkv = runtime.matrix(torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0))
        self.out_proj = runtime.matrix(tensors["out_proj"])
        self.head_bias = runtime.vector(tensors["head_bias"]) if spec.head_bias else None
        self.rotary_dim = spec.position.rotary_dim if spec.position is not None else 0
        self.interleaved = spec.position is not None and spec.position.pairing == "interleaved"
        self.qk_freq = _frequencies(self.rotary_dim, spec.position.theta).to(runtime.device) if self.rotary_dim else None
        self.value_freq = _frequencies(spec.value_dim, spec.position.theta).to(runtime.device) if spec.rotate_values else None
        self.scale = spec.scale if spec.scale is not None else spec.head_dim ** -0.5
        self.on_tensor_cores = ops.pooled_attention_supported(runtime.dtype, spec.head_dim, spec.value_dim)
        self.tile_tokens = ops.pooled_attention_tiling(spec.num_heads, spec.num_groups)[1]

    @classmethod
    def tensor_decls(cls, spec: PooledWindowAttentionSpec) -> dict[str, TensorDecl]:
        decls = {
            "q_proj": TensorDecl((spec.num_heads * spec.head_dim, spec.model_dim)),
            "k_proj": TensorDecl((spec.num_groups * spec.head_dim, spec.model_dim)),
            "v_proj": TensorDecl((spec.num_groups * spec.value_dim, spec.model_dim)),
            "out_proj": TensorDecl((spec.model_dim, spec.num_heads * spec.value_dim)),
        }
        if spec.head_bias:
            decls["head_bias"] = TensorDecl((spec.num_heads,), role="vector")
        return decls

    def cache_need(self) -> CacheNeed | None:
        spec = self.spec
        # A block's mean is taken when its last position is written: until then its positions stay, also behind the window.
        row = spec.head_dim + spec.value_dim   # a row holds a key and its value
        tokens = PagedKVNeed(num_groups=spec.num_groups, head_dim=row, window=max(spec.window, spec.pool), values_in_keys=True)
        if not spec.pool:
            return tokens
        blocks = PagedKVNeed(num_groups=spec.num_groups, head_dim=row, window=None, values_in_keys=True, tokens_per_row=spec.pool)
        return CompositeNeed((tokens, blocks))

    # The tensor-core kernel's tiles depend on where the portions start and how long they are, not on what the cache holds,
    # and are the same for every layer of this kind with the same number of tokens a tile.
    step_plan_uses_context = False

    def step_plan_key(self) -> object:
        return ("pooled_window_attention", self.tile_tokens)   # tiles and single tokens

    def plan_step(self, segments: HostSegments) -> dict[str, np.ndarray]:
        """``singles``: the rows of portions of one token (they attend alone); ``tiles``: ``(first row, count)`` of each run of at most
        ``tile_tokens`` consecutive tokens of a longer portion."""
        singles = [start for start, length in zip(segments.start, segments.length) if length == 1]
        tiles = [(first, min(self.tile_tokens, start + length - first)) for start, length in zip(segments.start, segments.length) if length > 1
                 for first in range(start, start + length, self.tile_tokens)]
        return {"singles": np.asarray(singles, dtype=np.int32), "tiles": np.asarray(tiles, dtype=np.int32).reshape(-1)}

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs, cache: "PagedKVView | CompositeView", residual: torch.Tensor | None = None) -> torch.Tensor | None:  # type: ignore[override]
        spec = self.spec
        status = self.runtime.status
        if spec.pool:
            tokens_view, blocks_view = cache.views
        else:
            tokens_view, blocks_view = cache, None
        qkv = ops.linear(x, self.qkv, status=status)
        queries = self.runtime.empty(step.tokens, spec.num_heads * spec.head_dim)
        shape = dict(num_heads=spec.num_heads, num_groups=spec.num_groups, head_dim=spec.head_dim, value_dim=spec.value_dim)
        ops.pooled_rewrite(qkv, queries, tokens_view.k_pages, qk_freq=self.qk_freq, rotary_dim=self.rotary_dim, value_freq=self.value_freq,
                           interleaved=self.interleaved, positions=step.positions, token_segment=step.token_segment, block_table=tokens_view.block_table,
                           write_kv=tokens_view.owns, status=status, **shape)
        if blocks_view is not None and blocks_view.owns:
            ops.pooled_means(tokens_view.k_pages, blocks_view.k_pages, segment_length=step.segment_length,
                             segment_context=step.segment_context, block_table=tokens_view.block_table, pool_table=blocks_view.block_table,
                             segments=step.segments, max_length=step.max_segment_length, num_groups=spec.num_groups, head_dim=spec.head_dim,
                             value_dim=spec.value_dim, pool=spec.pool, status=status)
        mixed = self.runtime.empty(step.tokens, spec.num_heads * spec.value_dim)
        common = dict(positions=step.positions, token_segment=step.token_segment, block_table=tokens_view.block_table,
                      pool_table=blocks_view.block_table if blocks_view is not None else None, scale=self.scale, softcap=spec.softcap, head_bias=self.head_bias,
                      window=spec.window, pool=spec.pool, value_freq=self.value_freq, interleaved=self.interleaved, status=status, **shape)
        pool_pages = blocks_view.k_pages if blocks_view is not None else None
        if self.on_tensor_cores:
            lists, host_lists = step.plan_of(self)
            if host_lists["singles"].size:
                ops.pooled_attention_single(queries, tokens_view.k_pages, pool_pages, mixed, singles=lists["singles"], num_singles=host_lists["singles"].size, **common)
            if host_lists["tiles"].size:
                ops.pooled_attention(queries, tokens_view.k_pages, pool_pages, mixed, tiles=lists["tiles"], num_tiles=host_lists["tiles"].size // 2, **common)
        else:
            ops.pooled_attention_plain(queries, tokens_view.k_pages, pool_pages, mixed, **common)
        if residual is not None:
            return ops.linear_accumulate(mixed, self.out_proj, residual, status=status)
        return ops.linear(mixed, self.out_proj, status=status)
