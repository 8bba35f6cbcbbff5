"""Latent attention over a paged cache: a token leaves one row ``[latent | rope]`` behind (its normed latent vector and
one rotated key part shared by all heads), from which every head's keys and values are made.

The heads' key and value projections are not applied to the cached rows.  A query head's unrotated part is taken into
the latent's space instead (``W_uk_h^T q_h``), so that the score against a cached row is one dot product over
``latent + rope`` channels; the attention sums the rows' latent parts, and the head's value projection is applied to
that sum.  Both are exact rearrangements of ``(q . W_uk c)`` and ``sum_j p_j W_uv c_j``."""

from __future__ import annotations

from typing import Mapping

import numpy as np
import torch

from .. import ops
from ..config.plan import LatentAttentionSpec, RMSNormSpec, RopeSpec
from .base import CacheNeed, HostSegments, Mixer, PagedKVNeed, PagedKVView, Runtime, StepInputs, TensorDecl, build_part, register_part

__all__ = ["LatentAttention"]


@register_part(LatentAttentionSpec)
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: LatentAttentionSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if spec.window is not None and spec.window < 1:
            raise ValueError(f"window must be positive, got {spec.window}")
        if not isinstance(spec.latent_norm, RMSNormSpec) or spec.latent_norm.dim != spec.latent_dim:
            raise ValueError("the latent vector's norm must be an RMS norm over latent_dim")
        if not isinstance(spec.position, RopeSpec) or spec.position.rotary_dim != spec.rope_dim or spec.position.pairing not in ("half", "interleaved"):
            raise ValueError("latent attention rotates all rope_dim channels of the rotated parts, in halves or in pairs of neighbours")
        heads, dim, rope = spec.num_heads, spec.head_dim, spec.rope_dim
        q_proj, down_proj = tensors["q_proj"], tensors["down_proj"]
        if spec.position.pairing == "interleaved":
            # The kernels rotate channel i with i + rope / 2.  A score sums over the rotated channels of the query and of the
            # shared key part, so taking both in the same other order (even channels first, then the odd ones) changes no
            # score, and pair (2i, 2i + 1) becomes pair (i, i + rope / 2) with its angle.
            order = torch.cat([torch.arange(0, rope, 2), torch.arange(1, rope, 2)])
            per_head = q_proj.reshape(heads, dim + rope, -1)
            q_proj = torch.cat([per_head[:, :dim], per_head[:, dim:][:, order]], dim=1).reshape(q_proj.shape)
            down_proj = torch.cat([down_proj[: spec.latent_dim], down_proj[spec.latent_dim :][order]], dim=0)
        # One product for everything that reads the mixer's input: queries, the gate, the latent's down-projection.
        rows = [q_proj] + ([tensors["gate_proj"]] if spec.gated else []) + [down_proj]
        self.in_proj = runtime.matrix(torch.cat(rows, dim=0))
        self.q_width = heads * (dim + rope)
        self.gate_width = heads * spec.value_dim if spec.gated else 0
        self.key_up = runtime.matrix(tensors["key_up_proj"].reshape(heads, dim, spec.latent_dim))        # [head][channel][latent]
        self.value_up = runtime.matrix(tensors["value_up_proj"].reshape(heads, spec.value_dim, spec.latent_dim))
        self.out_proj = runtime.matrix(tensors["out_proj"])
        self.latent_norm = runtime.vector(tensors["latent_norm"])
        self.sink = runtime.vector(tensors["sink"]) if spec.sink else None
        self.position = build_part(spec.position, {}, runtime)
        if self.position.magnitude != 1.0:
            raise ValueError("latent attention takes no factor on sines and cosines")
        self.scale = spec.scale if spec.scale is not None else (dim + rope) ** -0.5

    @classmethod
    def tensor_decls(cls, spec: LatentAttentionSpec) -> dict[str, TensorDecl]:
        heads = spec.num_heads
        decls = {
            "q_proj": TensorDecl((heads * (spec.head_dim + spec.rope_dim), spec.model_dim)),
            "down_proj": TensorDecl((spec.latent_dim + spec.rope_dim, spec.model_dim)),
            "latent_norm": TensorDecl((spec.latent_dim,), role="vector", init="ones"),
            "key_up_proj": TensorDecl((heads * spec.head_dim, spec.latent_dim)),
            "value_up_proj": TensorDecl((heads * spec.value_dim, spec.latent_dim)),
            "out_proj": TensorDecl((spec.model_dim, heads * spec.value_dim)),
        }
        if spec.gated:
            decls["gate_proj"] = TensorDecl((heads * spec.value_dim, spec.model_dim))
        if spec.sink:
            decls["sink"] = TensorDecl((heads,), role="vector")
        return decls

    def cache_need(self) -> CacheNeed | None:
        spec = self.spec
        return PagedKVNeed(num_groups=1, head_dim=spec.latent_dim + spec.rope_dim, window=spec.window, value_dim=spec.latent_dim, values_in_keys=True)

    # The tensor-core kernel's items depend on where the portions start and how long they are, not on what the cache
    # holds, and they are the same for every latent layer with as many heads.
    step_plan_uses_context = False

    def step_plan_key(self) -> object:
        return ("latent_attention", ops.latent_attention_tiling(self.spec.num_heads))

    def plan_step(self, segments: HostSegments) -> dict[str, np.ndarray]:
        """``items``: ``(first row, count)`` of every run of consecutive tokens that one CTA takes."""
        _, run = ops.latent_attention_tiling(self.spec.num_heads)
        items = [(first, min(run, start + length - first)) for start, length in zip(segments.start, segments.length) for first in range(start, start + length, run)]
        return {"items": np.asarray(items, dtype=np.int32).reshape(-1)}

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs, cache: PagedKVView, residual: torch.Tensor | None = None) -> torch.Tensor | None:  # type: ignore[override]
        spec, runtime = self.spec, self.runtime
        heads, dim, rope, latent = spec.num_heads, spec.head_dim, spec.rope_dim, spec.latent_dim
        tokens = step.tokens
        projected = ops.linear(x, self.in_proj, status=runtime.status)
        q = projected[:, : self.q_width]
        gate = projected[:, self.q_width : self.q_width + self.gate_width] if spec.gated else None
        down = projected[:, self.q_width + self.gate_width :]
        queries = runtime.empty(tokens, heads, latent + rope)
        per_head = q.view(tokens, heads, dim + rope)
        # the heads' unrotated query parts into the latent's space: the framework's own kernel writes them where the attention
        # reads them; sizes it does not take (and the 32-bit path) go through a batched library product, [head][token][latent]
        own_products = ops.heads_product_supported(runtime.dtype, dim, latent) and ops.heads_product_supported(runtime.dtype, latent, spec.value_dim) \
            and projected.shape[1] % 8 == 0 and (dim + rope) % 8 == 0 and self.q_width % 2 == 0
        q_latent = None
        if own_products:
            ops.heads_product(per_head[:, :, :dim], self.key_up, queries[:, :, :latent], weight_is_kn=True)
        else:
            q_latent = ops.heads_linear(per_head[:, :, :dim].transpose(0, 1), self.key_up)
        ops.latent_prepare(q, q_latent, down, queries, cache.k_pages, norm_weight=self.latent_norm, eps=spec.latent_norm.eps,
                           scale_offset=spec.latent_norm.scale_offset, inv_freq=self.position.inv_freq, positions=step.positions,
                           token_segment=step.token_segment, block_table=cache.block_table, num_heads=heads, head_dim=dim, latent=latent, rope=rope,
                           write_kv=cache.owns, status=runtime.status)
        summed = runtime.empty(tokens, heads, latent)
        common = dict(positions=step.positions, token_segment=step.token_segment, block_table=cache.block_table, num_heads=heads, latent=latent, rope=rope,
                      scale=self.scale, window=spec.window, status=runtime.status, sink=self.sink)
        if ops.latent_attention_supported(runtime.dtype, latent, rope, cache.k_pages.shape[1]):
            lists, host_lists = step.plan_of(self)
            num_items = host_lists["items"].size // 2
            splits = ops.latent_attention_splits(num_items, heads, latent, spec.window, step.max_context)
            ops.latent_attention(queries, cache.k_pages, summed, items=lists["items"], num_items=num_items, splits=splits, **common)
        else:
            ops.latent_attention_plain(queries, cache.k_pages, summed, **common)
        mixed = runtime.empty(tokens, heads * spec.value_dim)
        if own_products:
            # the heads' value projections applied to the sums, times the gate, laid out for the out-projection
            ops.heads_product(summed, self.value_up, mixed.view(tokens, heads, spec.value_dim), weight_is_kn=False,
                              gate=gate.view(tokens, heads, spec.value_dim) if gate is not None else None)
        else:
            values = ops.heads_linear(summed.transpose(0, 1), self.value_up, transpose_weight=True)   # [head][token][vdim]
            ops.gate_heads(values, gate, mixed)
        if residual is not None:
            return ops.linear_accumulate(mixed, self.out_proj, residual, status=runtime.status)
        return ops.linear(mixed, self.out_proj, status=runtime.status)
