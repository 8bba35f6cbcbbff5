"""The parts at the model's two ends: the token embedding (``lalamo/modules/embedding.py``) that
starts the 32-bit residual stream, and the read-out that turns normed rows into 32-bit logits.

A read-out declares ``tied = True`` if it has no table of its own; the model then hands it the
embedding's table under the local name ``"weight"``."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import EmbeddingSpec, HeadSpec, StreamMixSpec
from .base import Part, Runtime, TensorDecl, register_part

__all__ = ["Embedding", "Head", "LMHead", "StreamMix", "TokenEmbedding"]


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, tokens: int, positions: torch.Tensor | None = None) -> torch.Tensor:
        """The residual stream ``[tokens, model_dim]`` in 32-bit for these token ids (at these positions, for an embedding
        that looks at them)."""
        raise NotImplementedError

    def add_to(self, residual: torch.Tensor, token_ids: torch.Tensor) -> None:
        """``residual += forward(token_ids)``."""
        ops.residual_add(residual, self.forward(token_ids, residual.shape[0]))


class Head(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """32-bit logits ``[rows, vocab]`` for normed rows ``x``."""
        raise NotImplementedError


@register_part(EmbeddingSpec)
class TokenEmbedding(Embedding):
    def __init__(self, spec: EmbeddingSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.weight = runtime.matrix(tensors["weight"])
        self.positions = runtime.matrix(tensors["positions"]) if spec.learned_positions else None

    @classmethod
    def tensor_decls(cls, spec: EmbeddingSpec) -> dict[str, TensorDecl]:
        decls = {"weight": TensorDecl((spec.vocab_size, spec.model_dim))}
        if spec.learned_positions:
            decls["positions"] = TensorDecl((spec.learned_positions, spec.model_dim))
        return decls

    def forward(self, token_ids: torch.Tensor, tokens: int, positions: torch.Tensor | None = None) -> torch.Tensor:
        residual = self.runtime.empty(tokens, self.spec.model_dim, dtype=torch.float32)
        ops.embed(self.weight, token_ids, residual, self.spec.scale, self.runtime.status)
        if self.positions is not None:
            if positions is None:
                raise ValueError("an embedding with learned position vectors needs the tokens' positions")
            # the same gather with the positions as indices, unscaled and added; a position past the table is reported like a bad token id
            ops.embed(self.positions, positions, residual, 1.0, self.runtime.status, accumulate=True)
        return residual

    def add_to(self, residual: torch.Tensor, token_ids: torch.Tensor) -> None:
        """``residual += forward(token_ids)``: a model that feeds its input again further up gathers the rows again."""
        ops.embed(self.weight, token_ids, residual, self.spec.scale, self.runtime.status, accumulate=True)


@register_part(HeadSpec)
class LMHead(Head):
    def __init__(self, spec: HeadSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        weight = tensors["weight"]
        # a tied read-out is handed the embedding's table as the embedding holds it: no second copy
        self.weight = weight if weight.is_cuda and weight.dtype == runtime.dtype and weight.is_contiguous() else runtime.matrix(weight)

    @classmethod
    def tensor_decls(cls, spec: HeadSpec) -> dict[str, TensorDecl]:
        return {} if spec.tied else {"weight": TensorDecl((spec.vocab_size, spec.model_dim))}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(x, self.weight, out_dtype=torch.float32, status=self.runtime.status)
        if self.spec.scale != 1.0 or self.spec.softcap > 0.0:
            ops.scale_(logits, self.spec.scale, self.spec.softcap)
        return logits


@register_part(StreamMixSpec)
class StreamMix(Part):
    """``x <- W [x ; x0]``: the residual stream renewed from itself and the embedding's output.  The two are laid side by side,
    rounded to the activation type (the embedding's rows are gathered again, nothing is kept), and one product with 32-bit
    results writes the new stream."""

    def __init__(self, spec: StreamMixSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.weight = runtime.matrix(tensors["weight"])

    @classmethod
    def tensor_decls(cls, spec: StreamMixSpec) -> dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.model_dim, 2 * spec.model_dim))}

    def forward(self, residual: torch.Tensor, embedding: "TokenEmbedding", token_ids: torch.Tensor) -> torch.Tensor:
        """The new 32-bit stream for the stream ``residual`` (everything added) and the tokens' embeddings."""
        both = ops.stream_concat(residual, embedding.weight, token_ids, embedding.spec.scale, self.runtime.status)
        return ops.linear(both, self.weight, out_dtype=torch.float32, status=self.runtime.status)
