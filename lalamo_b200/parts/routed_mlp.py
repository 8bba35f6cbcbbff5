"""A routed feed-forward (mixture of experts): the router's scores in 32-bit, the choice of experts under a
limit on groups of experts, the chosen experts' feed-forwards (gated or not), and their weighted sum; optionally a
shared feed-forward that every token runs, plainly added or times a sigmoid gate of one number per token (whose logit
is one more row of the router's 32-bit product)."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import RoutedMLPSpec
from .base import FeedForward, Part, Runtime, StepInputs, TensorDecl, build_part, part_type, register_part

__all__ = ["RoutedMLP"]


@register_part(RoutedMLPSpec)
class RoutedMLP(FeedForward):
    def __init__(self, spec: RoutedMLPSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if not (1 <= spec.top <= spec.num_experts and spec.num_experts % spec.group_count == 0 and 1 <= spec.group_keep <= spec.group_count):
            raise ValueError(f"top {spec.top} of {spec.num_experts} experts in {spec.group_count} groups of which {spec.group_keep} are kept is not a valid choice")
        if spec.top > spec.group_keep * (spec.num_experts // spec.group_count):
            raise ValueError("the kept groups hold fewer experts than a token uses")
        if spec.shared_gate and spec.shared is None:
            raise ValueError("a gate on the shared feed-forward needs a shared feed-forward")
        router = tensors["router"]
        if spec.shared_gate:
            router = torch.cat([router, tensors["shared_gate"].reshape(1, spec.model_dim).to(router.dtype)], dim=0)   # its logit is one more row of the router's product
        self.router = runtime.vector(router)  # the router's logits are 32-bit
        self.router_bias = runtime.vector(tensors["router_bias"]) if spec.router_bias else None
        self.choice_bias = runtime.vector(tensors["choice_bias"]) if spec.choice_bias else None
        self.shared: FeedForward | None = None
        if spec.shared is not None:
            self.shared = build_part(spec.shared, {local[len("shared."):]: tensor for local, tensor in tensors.items() if local.startswith("shared.")}, runtime)  # type: ignore[assignment]
        experts = range(spec.num_experts)
        self.gate = runtime.matrix(torch.stack([tensors[f"experts.{e}.gate_proj"] for e in experts])) if spec.gated else None
        self.up = runtime.matrix(torch.stack([tensors[f"experts.{e}.up_proj"] for e in experts]))
        self.down = runtime.matrix(torch.stack([tensors[f"experts.{e}.down_proj"] for e in experts]))

    @classmethod
    def tensor_decls(cls, spec: RoutedMLPSpec) -> dict[str, TensorDecl]:
        decls = {"router": TensorDecl((spec.num_experts, spec.model_dim))}
        if spec.router_bias:
            decls["router_bias"] = TensorDecl((spec.num_experts,), role="vector")
        if spec.choice_bias:
            decls["choice_bias"] = TensorDecl((spec.num_experts,), role="vector", init="zeros")
        if spec.shared_gate:
            decls["shared_gate"] = TensorDecl((1, spec.model_dim))
        if spec.shared is not None:
            for local, decl in part_type(spec.shared).tensor_decls(spec.shared).items():
                decls[f"shared.{local}"] = decl
        for e in range(spec.num_experts):
            if spec.gated:
                decls[f"experts.{e}.gate_proj"] = TensorDecl((spec.hidden_dim, spec.model_dim))
            decls[f"experts.{e}.up_proj"] = TensorDecl((spec.hidden_dim, spec.model_dim))
            decls[f"experts.{e}.down_proj"] = TensorDecl((spec.model_dim, spec.hidden_dim))
        return decls

    def sub_parts(self) -> list[Part]:
        return [self.shared] if self.shared is not None else []

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs | None = None, residual: torch.Tensor | None = None) -> "torch.Tensor | ops.ScaledSum | None":
        """The experts' weighted sum; with a shared feed-forward the two terms are handed on un-summed
        (``ops.ScaledSum``), for a consumer that adds them in 32-bit.  With ``residual`` (the 32-bit stream) everything is
        added to it by one kernel, nothing rounded on the way, and ``None`` is returned."""
        spec = self.spec
        routing = ops.moe_route(x, self.router, top=spec.top, group_count=spec.group_count, group_keep=spec.group_keep, score=spec.score,
                                renormalize=spec.renormalize, bias=self.router_bias, chosen_softmax=spec.chosen_softmax, weight_scale=spec.weight_scale,
                                choice_bias=self.choice_bias, extra=1 if spec.shared_gate else 0)
        chosen, weights = routing[0], routing[1]
        shared_gate = routing[2] if spec.shared_gate else None
        # with a shared feed-forward the consumer adds two terms anyway: the experts' weighted sum is left to it as well
        routed = ops.moe_experts(x, self.gate, self.up, self.down, chosen, weights, spec.activation, limit=spec.limit,
                                 combine=self.shared is None and residual is None)
        everyone = None
        if self.shared is not None:
            everyone = self.shared.forward(x, step)
            if isinstance(everyone, (ops.SlicedSum, ops.BiasedSum)):
                everyone = everyone.sum()
        if residual is not None:
            ops.moe_combine_add(routed, residual, everyone, shared_gate)
            return None
        if self.shared is None:
            return routed
        if shared_gate is not None:
            # no stream to add to: the gated sum in 32-bit, rounded once
            total = torch.zeros(x.shape[0], spec.model_dim, dtype=torch.float32, device=x.device)
            ops.moe_combine_add(routed, total, everyone, shared_gate)
            out = self.runtime.empty(*total.shape)
            ops.cast_rows(total, out)
            return out
        return ops.ScaledSum([(routed, 1.0, None), (everyone, 1.0, None)])
