"""The arrangement of norms, mixer and feed-forward in one block, and the registry of arrangements.

An arrangement is a :class:`Block` subclass registered under the name a layer's specification
carries in ``arrangement``.  It names the *roles* of its parts (fields of the specification that
hold part specifications), gets them built, and says in ``forward`` how they are wired around the
residual stream.  The built-in one is ``"pre_norm"`` (``lalamo/modules/transformer_layer.py:220-377``):
``h = x + mixer(norm1(x)); y = h + ffn(norm2(h))``.

The residual stream is a 32-bit tensor that the block updates in place.  A block returns its last
sub-block's output *not yet added* (or ``None`` if it added it itself): the next norm (the next
block's, or the model's final norm) adds it while it normalises, which saves one pass over the stream.
What is not yet added is a tensor of the activation type or an ``ops.SlicedSum`` (a product left as the
partial sums of its K slices); ``Norm.residual_forward`` and ``ops.residual_add`` take either.
"""

from __future__ import annotations

from typing import Any, Callable, ClassVar, Mapping

import torch

from .base import CacheView, FeedForward, Mixer, Norm, Part, Runtime, StepInputs, TensorDecl, build_part, part_type

__all__ = ["Block", "OutputNormBlock", "PreNormBlock", "SandwichNormBlock", "block_tensor_decls", "block_type", "build_block", "register_arrangement"]

_ARRANGEMENTS: dict[str, type["Block"]] = {}


def register_arrangement(name: str) -> Callable[[type["Block"]], type["Block"]]:
    """Class decorator: layers whose specification says ``arrangement == name`` are run by the class."""

    def decorate(block_class: type[Block]) -> type[Block]:
        _ARRANGEMENTS[name] = block_class
        return block_class

    return decorate


def block_type(spec: Any) -> type["Block"]:
    name = getattr(spec, "arrangement", None)
    if name not in _ARRANGEMENTS:
        raise ValueError(f"unknown block arrangement {name!r}; known: {sorted(_ARRANGEMENTS)}")
    return _ARRANGEMENTS[name]


def _role_specs(spec: Any) -> list[tuple[str, Any]]:
    """The part specifications of a layer, by role; roles whose field is ``None`` are left out."""
    return [(role, getattr(spec, role)) for role in block_type(spec).roles if getattr(spec, role, None) is not None]


def block_tensor_decls(spec: Any) -> dict[tuple[str, str], TensorDecl]:
    """``(role, local name) -> declaration`` for every tensor of the block's parts."""
    decls: dict[tuple[str, str], TensorDecl] = {}
    for role, part_spec in _role_specs(spec):
        for local, decl in part_type(part_spec).tensor_decls(part_spec).items():
            decls[(role, local)] = decl
    return decls


class Block:
    """Base of the arrangements.  Building sets one attribute per role (the built part, or ``None``
    where the specification leaves the role empty); one of the roles must be ``"mixer"``, since the
    model asks the block's mixer what cache it needs."""

    roles: ClassVar[tuple[str, ...]] = ()
    mixer: Mixer

    def __init__(self, spec: Any, tensors: Mapping[tuple[str, str], torch.Tensor], runtime: Runtime) -> None:
        if "mixer" not in self.roles:
            raise TypeError(f"{type(self).__name__}.roles must contain 'mixer'")
        self.spec = spec
        self.runtime = runtime
        for role in self.roles:
            setattr(self, role, None)
        for role, part_spec in _role_specs(spec):
            role_tensors = {local: tensor for (owner, local), tensor in tensors.items() if owner == role}
            setattr(self, role, build_part(part_spec, role_tensors, runtime))

    def parts(self) -> list[Part]:
        return [getattr(self, role) for role in self.roles if getattr(self, role) is not None]

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, step: StepInputs, cache: CacheView | None) -> torch.Tensor | None:
        """``residual`` holds the stream minus ``pending`` (the previous block's last output, or
        ``None`` if that was added already).  Returns this block's last output, to be added by the
        next norm, or ``None`` if the block added it itself."""
        raise NotImplementedError


@register_arrangement("pre_norm")
class PreNormBlock(Block):
    roles = ("pre_mixer_norm", "mixer", "pre_ffn_norm", "ffn")
    pre_mixer_norm: Norm
    pre_ffn_norm: Norm | None
    ffn: FeedForward | None

    def __init__(self, spec: Any, tensors: Mapping[tuple[str, str], torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if (self.ffn is None) != (self.pre_ffn_norm is None):
            raise ValueError("a pre-norm block has a feed-forward with its norm, or neither")

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, step: StepInputs, cache: CacheView | None) -> torch.Tensor | None:
        normed = self.pre_mixer_norm.residual_forward(residual, pending)
        if self.mixer.can_accumulate:
            mixed = self.mixer.forward(normed, step, cache, residual=residual)
        else:
            mixed = self.mixer.forward(normed, step, cache)
        if self.ffn is None:
            return mixed   # the next block's norm (or the model's last) adds it
        normed = self.pre_ffn_norm.residual_forward(residual, mixed)
        if self.ffn.can_accumulate:
            return self.ffn.forward(normed, step, residual=residual)
        return self.ffn.forward(normed, step)


@register_arrangement("output_norm")
class OutputNormBlock(Block):
    """``x <- x + mixer_norm(mixer(x)); x <- x + ffn_norm(ffn(x))``: the sublayers read the stream itself
    (rounded to the activation type), the norms sit on their outputs.  Norm and residual sum are one
    32-bit kernel, which also hands the new stream, rounded, to the next sublayer."""

    roles = ("mixer", "mixer_norm", "ffn", "ffn_norm")
    mixer_norm: Norm
    ffn: FeedForward | None
    ffn_norm: Norm | None

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, step: StepInputs, cache: CacheView | None) -> torch.Tensor | None:
        from .. import ops

        if pending is not None:
            ops.residual_add(residual, pending)
        runtime = self.runtime
        carried = step.carry.pop("rounded_stream", None)   # (the stream it is a copy of, the copy), left by the block before
        if runtime.dtype == torch.float32:
            x = residual  # the sublayers read the stream in place; what they return is added only after they have read it
        elif pending is None and carried is not None and carried[0] is residual:
            x = carried[1]
        else:
            x = runtime.empty(*residual.shape)
            ops.cast_rows(residual, x)
        mixed = self.mixer.forward(x, step, cache)
        if isinstance(mixed, ops.SlicedSum):
            mixed = mixed.sum()
        has_ffn = self.ffn is not None
        rounded = x if x is not residual else None   # the kernel that adds to the stream also rounds it for the next reader
        self._accumulate(self.mixer_norm, residual, mixed, rounded)
        if has_ffn:
            out = self.ffn.forward(x, step)
            if isinstance(out, ops.SlicedSum):
                out = out.sum()
            self._accumulate(self.ffn_norm, residual, out, rounded)
        if rounded is not None:
            step.carry["rounded_stream"] = (residual, rounded)
        return None

    @staticmethod
    def _accumulate(norm: Norm, residual: torch.Tensor, delta: "torch.Tensor", rounded: torch.Tensor | None) -> None:
        from .. import ops

        accumulate = getattr(norm, "accumulate", None)
        if accumulate is not None:
            accumulate(residual, delta, rounded)
            return
        if isinstance(delta, ops.ScaledSum):
            delta = delta.sum()
        ops.residual_add(residual, norm.forward(delta))
        if rounded is not None:
            ops.cast_rows(residual, rounded)


@register_arrangement("sandwich_norm")
class SandwichNormBlock(Block):
    """``x <- x + mixer_out_norm(mixer(mixer_norm(x))); x <- x + ffn_out_norm(ffn(ffn_norm(x)))``: a norm before and
    after each sublayer, all of them 32-bit on the 32-bit stream.  The norm after a sublayer, the residual sum and the
    norm before the next sublayer are one kernel (``RMSNorm.accumulate(..., then=...)``), also across blocks: the model
    tells a block which norm the next block begins with (``step.carry["next_norm"]``), and the block leaves that norm
    of its final stream in ``step.carry["normed_stream"]``."""

    roles = ("mixer_norm", "mixer", "mixer_out_norm", "ffn_norm", "ffn", "ffn_out_norm")
    mixer_norm: Norm
    mixer_out_norm: Norm
    ffn_norm: Norm | None
    ffn: FeedForward | None
    ffn_out_norm: Norm | None

    def __init__(self, spec: Any, tensors: Mapping[tuple[str, str], torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if (self.ffn is None) != (self.ffn_norm is None) or (self.ffn is None) != (self.ffn_out_norm is None):
            raise ValueError("a sandwich block has a feed-forward with both of its norms, or none of the three")

    @property
    def first_norm(self) -> Norm:
        """The norm this block begins with (a block before it may compute it on the way)."""
        return self.mixer_norm

    @staticmethod
    def _fusable(norm: Norm | None) -> bool:
        return norm is not None and getattr(norm.spec, "exact", False) and hasattr(norm, "accumulate")

    def _add_normed(self, out_norm: Norm, residual: torch.Tensor, delta: "torch.Tensor", then: Norm | None) -> torch.Tensor | None:
        """``residual += out_norm(delta)``; returns ``then(residual)`` if ``then`` is given."""
        from .. import ops

        if isinstance(delta, ops.SlicedSum):
            delta = delta.sum()
        if self._fusable(out_norm):
            if then is not None and self._fusable(then) and then.spec.dim == out_norm.spec.dim:
                normed = self.runtime.empty(*residual.shape)
                out_norm.accumulate(residual, delta, normed, then=then)   # type: ignore[attr-defined]
                return normed
            out_norm.accumulate(residual, delta)   # type: ignore[attr-defined]
        else:
            if isinstance(delta, ops.ScaledSum):
                delta = delta.sum()
            ops.residual_add(residual, out_norm.forward(delta))
        return then.forward(residual) if then is not None else None

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, step: StepInputs, cache: CacheView | None) -> torch.Tensor | None:
        from .. import ops

        following = step.carry.pop("next_norm", None)
        carried = step.carry.pop("normed_stream", None)   # (the stream, the norm, that norm of the stream), left by the block before
        if pending is not None:
            ops.residual_add(residual, pending)
            carried = None
        if carried is not None and carried[0] is residual and carried[1] is self.mixer_norm:
            normed = carried[2]
        else:
            normed = self.mixer_norm.forward(residual)
        mixed = self.mixer.forward(normed, step, cache)
        last_norm, last = self.mixer_out_norm, mixed
        if self.ffn is not None:
            normed = self._add_normed(self.mixer_out_norm, residual, mixed, self.ffn_norm)
            last_norm, last = self.ffn_out_norm, self.ffn.forward(normed, step)
        ahead = following if following is not None and self._fusable(following) and self._fusable(last_norm) else None
        normed = self._add_normed(last_norm, residual, last, ahead)
        if ahead is not None:
            step.carry["normed_stream"] = (residual, ahead, normed)
        return None


def build_block(spec: Any, tensors: Mapping[tuple[str, str], torch.Tensor], runtime: Runtime) -> Block:
    return block_type(spec)(spec, tensors, runtime)
