"""The gated-delta-rule mixer: a matrix state per head, ``S <- diag(g) S; S <- S + k (beta (v - S^T k))^T;
o = S^T q`` with one decay per head and key channel, fed by short causal convolutions of q, k and v and
followed by a per-head RMS norm, a low-rank sigmoid gate and the out-projection.

Three products feed the recurrence's kernels: ``[q ; k ; v ; beta]`` (rows padded to a multiple of 8),
the two bottlenecks ``[a1 ; g1]`` (each padded to a multiple of 32 columns for the next product), and
the block-diagonal ``[a2 0 ; 0 g2]`` that turns the bottlenecks into decay and gate logits; the padding
is zeros and changes no sum.  Without bottlenecks (``decay_rank = gate_rank = 0``) the decay and gate logits are
rows of the first product, ``[q ; k ; v ; beta ; a ; g]``, and that product is the only one.  The decay is one number
per head and key channel, or one per head.  Per request the mixer holds the matrix state in 32-bit and the
convolutions' last ``taps - 1`` inputs in the activation type."""

from __future__ import annotations

from typing import Mapping

import numpy as np
import torch

from .. import ops
from ..config.plan import GatedDeltaSpec
from .base import CacheNeed, CompositeNeed, CompositeView, HostSegments, Mixer, Runtime, SlotStateNeed, StepInputs, TensorDecl, register_part

__all__ = ["GatedDelta"]


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


@register_part(GatedDeltaSpec)
class GatedDelta(Mixer):
    graph_safe = True

    def __init__(self, spec: GatedDeltaSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if spec.num_heads % spec.num_groups:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_groups={spec.num_groups}")
        if spec.conv_taps < 1 or spec.decay_rank < 0 or spec.gate_rank < 0:
            raise ValueError("conv_taps must be positive, decay_rank and gate_rank not negative")
        if (spec.decay_rank == 0) != (spec.gate_rank == 0):
            raise ValueError("the decay and the gate both go through a bottleneck, or neither does")
        if spec.gate_activation not in ("sigmoid", "silu"):
            raise ValueError(f"unknown gate activation {spec.gate_activation!r}; known: 'sigmoid', 'silu'")
        heads, groups, dk, dv = spec.num_heads, spec.num_groups, spec.key_dim, spec.value_dim
        self.channels = 2 * groups * dk + heads * dv
        self.direct = spec.decay_rank == 0
        decay_columns = heads * dk if spec.decay_per_channel else heads
        rows = torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"], tensors["beta_proj"]], dim=0)
        if self.direct:
            # [q ; k ; v ; beta | a | g], each part starting at a multiple of 8 rows
            self.decay_offset = _round_up(rows.shape[0], 8)
            self.gate_offset = _round_up(decay_columns, 8)   # counted from the decay logits
            padded = torch.zeros(_round_up(self.decay_offset + self.gate_offset + heads * dv, 8), spec.model_dim, dtype=rows.dtype)
            padded[: rows.shape[0]] = rows
            padded[self.decay_offset : self.decay_offset + decay_columns] = tensors["decay_proj"]
            padded[self.decay_offset + self.gate_offset : self.decay_offset + self.gate_offset + heads * dv] = tensors["gate_proj"]
            self.in_proj = runtime.matrix(padded)
        else:
            self.gate_offset = decay_columns
            padded = torch.zeros(_round_up(rows.shape[0], 8), spec.model_dim, dtype=rows.dtype)
            padded[: rows.shape[0]] = rows
            self.in_proj = runtime.matrix(padded)
            decay_rank, gate_rank = _round_up(spec.decay_rank, 32), _round_up(spec.gate_rank, 32)
            down = torch.zeros(decay_rank + gate_rank, spec.model_dim, dtype=rows.dtype)
            down[: spec.decay_rank] = tensors["decay_down"]
            down[decay_rank : decay_rank + spec.gate_rank] = tensors["gate_down"]
            self.low_rank_down = runtime.matrix(down)
            up = torch.zeros(decay_columns + heads * dv, decay_rank + gate_rank, dtype=rows.dtype)
            up[:decay_columns, : spec.decay_rank] = tensors["decay_up"]
            up[decay_columns:, decay_rank : decay_rank + spec.gate_rank] = tensors["gate_up"]
            self.low_rank_up = runtime.matrix(up)
        self.conv_weight = runtime.vector(torch.cat([tensors["q_conv"], tensors["k_conv"], tensors["v_conv"]], dim=0).reshape(self.channels, spec.conv_taps))
        self.a_log = runtime.vector(tensors["a_log"])
        self.dt_bias = runtime.vector(tensors["dt_bias"])
        self.norm_weight = runtime.vector(tensors["out_norm"])
        self.out_proj = runtime.matrix(tensors["out_proj"])

    @classmethod
    def tensor_decls(cls, spec: GatedDeltaSpec) -> dict[str, TensorDecl]:
        heads, groups, dk, dv = spec.num_heads, spec.num_groups, spec.key_dim, spec.value_dim
        decay_columns = heads * dk if spec.decay_per_channel else heads
        if spec.decay_rank == 0:
            logits = {"decay_proj": TensorDecl((decay_columns, spec.model_dim)), "gate_proj": TensorDecl((heads * dv, spec.model_dim))}
        else:
            logits = {
                "decay_down": TensorDecl((spec.decay_rank, spec.model_dim)),
                "decay_up": TensorDecl((decay_columns, spec.decay_rank)),
                "gate_down": TensorDecl((spec.gate_rank, spec.model_dim)),
                "gate_up": TensorDecl((heads * dv, spec.gate_rank)),
            }
        return {
            "q_proj": TensorDecl((groups * dk, spec.model_dim)),
            "k_proj": TensorDecl((groups * dk, spec.model_dim)),
            "v_proj": TensorDecl((heads * dv, spec.model_dim)),
            "q_conv": TensorDecl((groups * dk, spec.conv_taps), role="vector"),
            "k_conv": TensorDecl((groups * dk, spec.conv_taps), role="vector"),
            "v_conv": TensorDecl((heads * dv, spec.conv_taps), role="vector"),
            "beta_proj": TensorDecl((heads, spec.model_dim)),
            "a_log": TensorDecl((heads,), role="vector", init="zeros"),
            "dt_bias": TensorDecl((decay_columns,), role="vector"),
            **logits,
            "out_norm": TensorDecl((dv,), role="vector", init="ones"),
            "out_proj": TensorDecl((spec.model_dim, heads * dv)),
        }

    def cache_need(self) -> CacheNeed | None:
        spec = self.spec
        matrix = SlotStateNeed(shape=(spec.num_heads, spec.key_dim, spec.value_dim), dtype=torch.float32)
        conv = SlotStateNeed(shape=(max(spec.conv_taps - 1, 1), self.channels))
        return CompositeNeed((matrix, conv))

    # Long portions run in chunks side by side; which rows belong to which chunk depends on the portions' lengths
    # only, and is the same for every layer of this kind.
    step_plan_uses_context = False

    def step_plan_key(self) -> object:
        return ("gated_delta", ops.GDR_CHUNK_TOKENS, ops.GDR_LONG_PORTION)

    def plan_step(self, segments: HostSegments) -> dict[str, np.ndarray]:
        return ops.gated_delta_chunk_plan(segments.start, segments.length)

    def forward(self, x: torch.Tensor, step: StepInputs, cache: CompositeView) -> torch.Tensor:  # type: ignore[override]
        spec = self.spec
        matrix_view, conv_view = cache.views
        if not cache.owns:
            raise ValueError("a gated-delta layer cannot read another layer's state")
        status = self.runtime.status
        lists, host_lists = step.plan_of(self)
        chunk_plan = dict(lists, num_chunks=host_lists["chunk_start"].size, num_long=host_lists["long_table"].size // 3, num_direct=host_lists["direct"].size)
        proj = ops.linear(x, self.in_proj, status=status)
        if self.direct:
            logits = proj[:, self.decay_offset :]
        else:
            low = ops.linear(x, self.low_rank_down, status=status)
            logits = ops.linear(low, self.low_rank_up, status=status)
        read_out = ops.gated_delta_rule(
            proj,
            logits,
            conv_view.state if spec.conv_taps > 1 else None,
            matrix_view.state,
            conv_weight=self.conv_weight,
            a_log=self.a_log,
            dt_bias=self.dt_bias,
            norm_weight=self.norm_weight,
            norm_eps=spec.norm_eps,
            num_heads=spec.num_heads,
            num_groups=spec.num_groups,
            key_dim=spec.key_dim,
            value_dim=spec.value_dim,
            unit_eps=spec.unit_eps,
            token_segment=step.token_segment,
            segment_start=step.segment_start,
            segment_length=step.segment_length,
            segment_slot=matrix_view.segment_slot,
            segments=step.segments,
            status=status,
            chunk_plan=chunk_plan,
            decay_per_head=not spec.decay_per_channel,
            gate_activation=spec.gate_activation,
            gate_offset=self.gate_offset,
        )
        return ops.linear(read_out, self.out_proj, status=status)
