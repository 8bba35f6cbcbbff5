"""Linear attention with a decaying matrix state per head: ``S_t = diag(a_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t``, no softmax
and no denominator.  The decay is one fixed number per head (retention) or one number per head and key channel made from
the token through a bottleneck, ``a = sigmoid(W_a2 (W_a1 h) + b) ** (1 / tau)`` (gated linear attention).  The read-out is
RMS-normed per head, multiplied by an activated gate and projected out.

One product gives q, k, v and the gate's logits (rows padded to a multiple of 8); the decay's logits come from two small
products (the bottleneck padded with zeros to a multiple of 32 columns).  A kernel lays the recurrence's inputs out in 32-bit
with the scale on q or k and the decays; the recurrence is the scan the gated delta rule uses, without that rule's correction;
the read-out kernel is shared with it too.  Per request the mixer holds the matrix state in 32-bit."""

from __future__ import annotations

from typing import Mapping

import numpy as np
import torch

from .. import ops
from ..config.plan import LinearAttentionSpec
from .base import CacheNeed, HostSegments, Mixer, Runtime, SlotStateNeed, SlotStateView, StepInputs, TensorDecl, register_part

__all__ = ["LinearAttention"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_part(LinearAttentionSpec)
class LinearAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: LinearAttentionSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        heads, dk, dv = spec.num_heads, spec.key_dim, spec.value_dim
        if spec.decay not in ("fixed", "channel"):
            raise ValueError(f"unknown decay {spec.decay!r}; known: 'fixed', 'channel'")
        if spec.scaled not in ("query", "key"):
            raise ValueError(f"unknown place of the scale {spec.scaled!r}; known: 'query', 'key'")
        if spec.gate_activation not in ("sigmoid", "silu"):
            raise ValueError(f"unknown gate activation {spec.gate_activation!r}; known: 'sigmoid', 'silu'")
        rows = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0)
        self.gate_offset = _round_up(rows.shape[0], 8)
        padded = torch.zeros(_round_up(self.gate_offset + heads * dv, 8), spec.model_dim, dtype=rows.dtype)
        padded[: rows.shape[0]] = rows
        padded[self.gate_offset : self.gate_offset + heads * dv] = tensors["gate_proj"]
        self.in_proj = runtime.matrix(padded)
        self.fixed_decay = self.decay_down = self.decay_up = self.decay_bias = None
        if spec.decay == "fixed":
            if len(spec.decay_values) != heads:
                raise ValueError(f"{len(spec.decay_values)} fixed decays for {heads} heads")
            self.fixed_decay = runtime.vector(torch.tensor(spec.decay_values, dtype=torch.float64))
        else:
            if spec.decay_rank < 1 or spec.tau <= 0.0:
                raise ValueError("a decay made from the token needs a bottleneck of positive rank and a positive tau")
            rank = _round_up(spec.decay_rank, 32)
            down = torch.zeros(rank, spec.model_dim, dtype=rows.dtype)
            down[: spec.decay_rank] = tensors["decay_down"]
            up = torch.zeros(_round_up(heads * dk, 8), rank, dtype=rows.dtype)
            up[: heads * dk, : spec.decay_rank] = tensors["decay_up"]
            self.decay_down, self.decay_up = runtime.matrix(down), runtime.matrix(up)
            self.decay_bias = runtime.vector(tensors["decay_bias"])
        self.norm_weight = runtime.vector(tensors["out_norm"] if spec.norm_weight else torch.ones(dv))
        self.out_proj = runtime.matrix(tensors["out_proj"])
        scale = dk ** -0.5
        self.query_scale, self.key_scale = (scale, 1.0) if spec.scaled == "query" else (1.0, scale)

    @classmethod
    def tensor_decls(cls, spec: LinearAttentionSpec) -> dict[str, TensorDecl]:
        heads, dk, dv = spec.num_heads, spec.key_dim, spec.value_dim
        decls = {
            "q_proj": TensorDecl((heads * dk, spec.model_dim)),
            "k_proj": TensorDecl((heads * dk, spec.model_dim)),
            "v_proj": TensorDecl((heads * dv, spec.model_dim)),
            "gate_proj": TensorDecl((heads * dv, spec.model_dim)),
            "out_proj": TensorDecl((spec.model_dim, heads * dv)),
        }
        if spec.decay == "channel":
            decls["decay_down"] = TensorDecl((spec.decay_rank, spec.model_dim))
            decls["decay_up"] = TensorDecl((heads * dk, spec.decay_rank))
            decls["decay_bias"] = TensorDecl((heads * dk,), role="vector")
        if spec.norm_weight:
            decls["out_norm"] = TensorDecl((dv,), role="vector", init="ones")
        return decls

    def cache_need(self) -> CacheNeed | None:
        spec = self.spec
        return SlotStateNeed(shape=(spec.num_heads, spec.key_dim, spec.value_dim), dtype=torch.float32)

    # Long portions run in chunks side by side (the plan the gated delta rule's layers make, shared with them): which rows belong
    # to which chunk depends on the portions' lengths only.
    step_plan_uses_context = False

    def step_plan_key(self) -> object:
        return ("gated_delta", ops.GDR_CHUNK_TOKENS, ops.GDR_LONG_PORTION)

    def plan_step(self, segments: HostSegments) -> dict[str, np.ndarray]:
        return ops.gated_delta_chunk_plan(segments.start, segments.length)

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs, cache: SlotStateView, residual: torch.Tensor | None = None) -> torch.Tensor | None:  # type: ignore[override]
        spec = self.spec
        if not cache.owns:
            raise ValueError("a linear-attention layer cannot read another layer's state")
        status = self.runtime.status
        lists, host_lists = step.plan_of(self)
        chunk_plan = dict(lists, num_chunks=host_lists["chunk_start"].size, num_long=host_lists["long_table"].size // 3, num_direct=host_lists["direct"].size)
        proj = ops.linear(x, self.in_proj, status=status)
        logits = None
        if self.decay_down is not None:
            logits = ops.linear(ops.linear(x, self.decay_down, status=status), self.decay_up, status=status)
        read_out = ops.linear_attention(
            proj,
            cache.state,
            num_heads=spec.num_heads,
            key_dim=spec.key_dim,
            value_dim=spec.value_dim,
            decay_logits=logits,
            decay_bias=self.decay_bias,
            fixed_decay=self.fixed_decay,
            tau=spec.tau,
            query_scale=self.query_scale,
            key_scale=self.key_scale,
            norm_weight=self.norm_weight,
            norm_eps=spec.norm_eps,
            gate_offset=self.gate_offset,
            gate_activation=spec.gate_activation,
            segment_start=step.segment_start,
            segment_length=step.segment_length,
            segment_slot=cache.segment_slot,
            segments=step.segments,
            status=status,
            chunk_plan=chunk_plan,
        )
        if residual is not None:
            return ops.linear_accumulate(read_out, self.out_proj, residual, status=status)
        return ops.linear(read_out, self.out_proj, status=status)
