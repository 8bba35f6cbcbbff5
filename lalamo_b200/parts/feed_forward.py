"""Dense gated feed-forward (``lalamo/modules/mlp.py:233-262``): ``down(up(x) * act(gate(x)))``
with the up and gate projections fused into one product, rows ordered ``[up ; gate]``."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import DenseMLPSpec, GatedMLPSpec
from .base import FeedForward, Runtime, StepInputs, TensorDecl, register_part

__all__ = ["DenseMLP", "GatedMLP"]


@register_part(GatedMLPSpec)
class GatedMLP(FeedForward):
    def __init__(self, spec: GatedMLPSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.up_gate = runtime.matrix(torch.cat([tensors["up_proj"], tensors["gate_proj"]], dim=0))
        self.down = runtime.matrix(tensors["down_proj"])

    @classmethod
    def tensor_decls(cls, spec: GatedMLPSpec) -> dict[str, TensorDecl]:
        return {
            "gate_proj": TensorDecl((spec.hidden_dim, spec.model_dim)),
            "up_proj": TensorDecl((spec.hidden_dim, spec.model_dim)),
            "down_proj": TensorDecl((spec.model_dim, spec.hidden_dim)),
        }

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs | None = None, residual: torch.Tensor | None = None) -> torch.Tensor | None:
        hidden = ops.gated_linear(x, self.up_gate, self.spec.activation, status=self.runtime.status, limit=self.spec.limit)
        if residual is not None:
            early = ops.gated_linear_starts_successor_early(x.shape[0], self.up_gate.shape[0], x.shape[1])
            return ops.linear_accumulate(hidden, self.down, residual, status=self.runtime.status, started_early=early)
        return ops.linear(hidden, self.down, status=self.runtime.status)


@register_part(DenseMLPSpec)
class DenseMLP(FeedForward):
    """``down(act(up(x) + b_up)) + b_down``: two projections around an activation, no gate.  The up-projection's bias and the
    activation are the product's epilogue (the weight-streaming product's for steps of few tokens, the tcgen05 product's
    otherwise; one elementwise kernel after a library product in 32-bit); the down-projection's bias is added with the
    product, onto the 32-bit stream, by whoever adds it."""

    def __init__(self, spec: DenseMLPSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.up = runtime.matrix(tensors["up_proj"])
        self.down = runtime.matrix(tensors["down_proj"])
        self.up_bias = runtime.vector(tensors["up_bias"]) if spec.has_bias else None
        self.down_bias = runtime.vector(tensors["down_bias"]) if spec.has_bias else None

    @classmethod
    def tensor_decls(cls, spec: DenseMLPSpec) -> dict[str, TensorDecl]:
        decls = {
            "up_proj": TensorDecl((spec.hidden_dim, spec.model_dim)),
            "down_proj": TensorDecl((spec.model_dim, spec.hidden_dim)),
        }
        if spec.has_bias:
            decls["up_bias"] = TensorDecl((spec.hidden_dim,), role="vector")
            decls["down_bias"] = TensorDecl((spec.model_dim,), role="vector")
        return decls

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs | None = None, residual: torch.Tensor | None = None):
        hidden = ops.linear_bias_activation(x, self.up, self.up_bias, self.spec.activation, status=self.runtime.status)
        if residual is not None:
            return ops.linear_accumulate(hidden, self.down, residual, status=self.runtime.status, bias=self.down_bias)
        out = ops.linear(hidden, self.down, status=self.runtime.status)
        if isinstance(out, ops.SlicedSum):
            out = out.sum()
        if self.down_bias is not None:
            ops.add_bias(out, self.down_bias)
        return out
