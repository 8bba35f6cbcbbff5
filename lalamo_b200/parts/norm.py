"""RMS norm (``lalamo/modules/normalization.py:89-126``): statistics in 32-bit, the
normalised value rounded to the activation type before the multiplication by the scale."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import LayerNormSpec, RMSNormSpec
from .base import Norm, Runtime, TensorDecl, register_part

__all__ = ["LayerNorm", "RMSNorm"]


@register_part(RMSNormSpec)
class RMSNorm(Norm):
    def __init__(self, spec: RMSNormSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.scale = runtime.vector(tensors["scale"])

    @classmethod
    def tensor_decls(cls, spec: RMSNormSpec) -> dict[str, TensorDecl]:
        # a weight that is used as ``w + offset`` is made small
        return {"scale": TensorDecl((spec.dim,), role="vector", init="ones" if spec.scale_offset == 0.0 else "normal")}

    def _out(self, x: torch.Tensor, rows: torch.Tensor | None, num_rows: int | None) -> torch.Tensor:
        count = x.shape[0] if rows is None else (rows.numel() if num_rows is None else num_rows)
        return self.runtime.empty(count, self.spec.dim)

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None, num_rows: int | None = None) -> torch.Tensor:
        out = self._out(x, rows, num_rows)
        ops.rmsnorm(x, self.scale, out, self.spec.eps, rows=rows, scale_offset=self.spec.scale_offset, exact=self.spec.exact)
        return out

    def residual_forward(
        self,
        residual: torch.Tensor,
        delta: "torch.Tensor | ops.SlicedSum | None",
        rows: torch.Tensor | None = None,
        num_rows: int | None = None,
    ) -> torch.Tensor:
        out = self._out(residual, rows, num_rows)
        ops.rmsnorm(
            residual,
            self.scale,
            out,
            self.spec.eps,
            delta=delta,
            rows=rows,
            scale_offset=self.spec.scale_offset,
            write_back=delta is not None and rows is None,
            exact=self.spec.exact,
        )
        return out

    def accumulate(self, residual: torch.Tensor, delta: "torch.Tensor | ops.ScaledSum", rounded: torch.Tensor | None = None,
                   then: "RMSNorm | None" = None) -> None:
        """``residual += norm(delta)`` on the 32-bit stream, the norm itself in 32-bit too (no rounding of the
        normalised value); ``rounded`` receives the new stream in the activation type or, with ``then`` (an exact RMS
        norm), that norm of the new stream: the same kernel computes both norms."""
        next_norm = None
        if then is not None:
            if not then.spec.exact or then.spec.dim != self.spec.dim:
                raise ValueError("only an exact RMS norm of the same width can follow in the same kernel")
            next_norm = (then.scale, then.spec.eps, then.spec.scale_offset)
        ops.norm_accumulate(residual, delta, self.scale, self.spec.eps, scale_offset=self.spec.scale_offset, rounded=rounded, next_norm=next_norm)


@register_part(LayerNormSpec)
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * scale + bias``: statistics, norm, scale and bias in 32-bit on the 32-bit stream, rounded
    once to the activation type.  The residual sum is fused in like the RMS norm's (one kernel serves both)."""

    def __init__(self, spec: LayerNormSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.scale = runtime.vector(tensors["scale"])
        self.bias = runtime.vector(tensors["bias"])

    @classmethod
    def tensor_decls(cls, spec: LayerNormSpec) -> dict[str, TensorDecl]:
        return {"scale": TensorDecl((spec.dim,), role="vector", init="ones"), "bias": TensorDecl((spec.dim,), role="vector")}

    def _out(self, x: torch.Tensor, rows: torch.Tensor | None, num_rows: int | None) -> torch.Tensor:
        count = x.shape[0] if rows is None else (rows.numel() if num_rows is None else num_rows)
        return self.runtime.empty(count, self.spec.dim)

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None, num_rows: int | None = None) -> torch.Tensor:
        out = self._out(x, rows, num_rows)
        ops.rmsnorm(x, self.scale, out, self.spec.eps, rows=rows, exact=True, bias=self.bias, centred=True)
        return out

    def residual_forward(
        self,
        residual: torch.Tensor,
        delta: "torch.Tensor | ops.SlicedSum | ops.BiasedSum | None",
        rows: torch.Tensor | None = None,
        num_rows: int | None = None,
    ) -> torch.Tensor:
        out = self._out(residual, rows, num_rows)
        ops.rmsnorm(residual, self.scale, out, self.spec.eps, delta=delta, rows=rows, write_back=delta is not None and rows is None,
                    exact=True, bias=self.bias, centred=True)
        return out
