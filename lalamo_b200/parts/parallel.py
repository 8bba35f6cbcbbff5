"""Mixers side by side: every branch reads the same input with a cache of its own, and the result is the
weighted sum of the branches' outputs.  The sum is handed on un-summed (``ops.ScaledSum``) where the
consumer can add the terms itself; a branch's output bias travels with its term.  Where every branch's output passes a
norm of its own before the sum (``branch_norm``), norms, weights and the sum onto the residual stream are one 32-bit kernel."""

from __future__ import annotations

from typing import Mapping

import numpy as np
import torch

from .. import ops
from ..config.plan import ParallelMixerSpec, RMSNormSpec
from .base import CacheNeed, CompositeNeed, CompositeView, HostSegments, Mixer, Part, Runtime, StepInputs, TensorDecl, build_part, part_type, register_part

__all__ = ["ParallelMixer"]


@register_part(ParallelMixerSpec)
class ParallelMixer(Mixer):
    def __init__(self, spec: ParallelMixerSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if not spec.branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.branches: list[Mixer] = []
        self.scales: list[float] = []
        for name, branch_spec, scale in spec.branches:
            prefix = name + "."
            own = {local[len(prefix):]: tensor for local, tensor in tensors.items() if local.startswith(prefix)}
            self.branches.append(build_part(branch_spec, own, runtime))  # type: ignore[arg-type]
            self.scales.append(float(scale))
        self.graph_safe = all(getattr(branch, "graph_safe", False) for branch in self.branches)
        self.branch_weights: list[torch.Tensor] | None = None
        if spec.branch_norm is not None:
            norm = spec.branch_norm
            if not isinstance(norm, RMSNormSpec) or not norm.exact or norm.scale_offset != 0.0:
                raise ValueError("the norm of the branches' outputs must be an exact RMS norm with a plain weight")
            self.branch_weights = [runtime.vector(tensors[f"{name}.out_norm.scale"]) for name, _, _ in spec.branches]
            self.can_accumulate = True   # norms and sum go straight onto the residual stream
        # The step's plan is the branches' plans side by side, each under its branch's own key.
        self._planners = [branch for branch in self.branches if type(branch).plan_step is not Part.plan_step]

    @classmethod
    def tensor_decls(cls, spec: ParallelMixerSpec) -> dict[str, TensorDecl]:
        decls: dict[str, TensorDecl] = {}
        for name, branch_spec, _ in spec.branches:
            for local, decl in part_type(branch_spec).tensor_decls(branch_spec).items():
                decls[f"{name}.{local}"] = decl
            if spec.branch_norm is not None:
                for local, decl in part_type(spec.branch_norm).tensor_decls(spec.branch_norm).items():
                    decls[f"{name}.out_norm.{local}"] = decl
        return decls

    def cache_need(self) -> CacheNeed | None:
        return CompositeNeed(tuple(branch.cache_need() for branch in self.branches))

    def sub_parts(self) -> list[Part]:
        """The branches, for whoever walks a model's parts (step planners, weight accounting)."""
        return list(self.branches)

    def _normed_sum(self, x: torch.Tensor, step: StepInputs, cache: CompositeView, residual: torch.Tensor | None) -> torch.Tensor | None:
        """``sum_i scale_i * norm_i(branch_i(x))``: added to ``residual`` (32-bit, nothing rounded on the way) if that is
        given, else returned in the activation type."""
        outputs = []
        for branch, view in zip(self.branches, cache.views):
            out = branch.forward(x, step, view)
            if isinstance(out, (ops.SlicedSum, ops.ScaledSum, ops.BiasedSum)):
                out = out.sum()
            outputs.append(out)
        target = residual if residual is not None else torch.zeros(x.shape[0], self.spec.branch_norm.dim, dtype=torch.float32, device=x.device)
        terms = list(zip(outputs, self.branch_weights, self.scales))
        for first in range(0, len(terms), 2):
            ops.branch_norms_accumulate(target, terms[first : first + 2], self.spec.branch_norm.eps)
        if residual is not None:
            return None
        rounded = self.runtime.empty(*target.shape)
        ops.cast_rows(target, rounded)
        return rounded

    def forward(self, x: torch.Tensor, step: StepInputs, cache: CompositeView, residual: torch.Tensor | None = None) -> "torch.Tensor | ops.ScaledSum | None":  # type: ignore[override]
        if self.branch_weights is not None:
            return self._normed_sum(x, step, cache, residual)
        terms = []
        for branch, scale, view in zip(self.branches, self.scales, cache.views):
            bias = getattr(branch, "output_bias", None)
            if bias is not None:
                out = branch.forward(x, step, view, add_output_bias=False)
            else:
                out = branch.forward(x, step, view)
            if isinstance(out, ops.SlicedSum):
                out = out.sum()
            terms.append((out, scale, bias))
        if len(terms) <= 2:
            return ops.ScaledSum(terms)
        return ops.ScaledSum([(ops.ScaledSum(terms).sum(), 1.0, None)])
