"""Python bindings of the CUDA kernels: tensors in, launches on the current stream.

Every function checks what the kernel cannot check for itself (device, dtype, contiguity,
size limits) and raises :class:`KernelError` with a clear message instead of launching with
arguments the kernel does not support.  Matrix products of the 32-bit path go to the library
(cuBLAS through ``torch.matmul``, with TF32 and reduced-precision reductions switched off), as
the reference's go to XLA (``lalamo/weight_matrix.py:418-432``).
"""

from __future__ import annotations

from dataclasses import dataclass

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import native

__all__ = ["BiasedSum", "ExpertSum", "KernelError", "ScaledSum", "SlicedSum", "dtype_code", "launch_count", "reset_launch_count"]


class KernelError(RuntimeError):
    pass


@dataclass
class SlicedSum:
    """A product ``x @ weight.T`` left as the partial sums of its K slices, ``partials[slice, token, row]``
    in float32.  Whoever consumes it adds the slices in order and rounds the sum to ``dtype``, as the
    product's own epilogue would have: :func:`rmsnorm` and :func:`residual_add` take it as their
    ``delta``, :meth:`sum` gives the plain tensor."""

    partials: torch.Tensor
    dtype: torch.dtype

    @property
    def shape(self) -> torch.Size:
        return self.partials.shape[1:]

    def sum(self) -> torch.Tensor:
        slices, tokens, rows = self.partials.shape
        out = torch.empty(tokens, rows, dtype=self.dtype, device=self.partials.device)
        _sum_slices(self.partials, out, "store")
        return out


@dataclass
class BiasedSum:
    """A product ``tensor`` (or a :class:`SlicedSum`) whose bias, a 32-bit vector over its columns, is still to be added:
    :func:`rmsnorm` adds both to the residual stream on its way, :func:`residual_add` likewise; :meth:`sum` gives the
    plain tensor."""

    tensor: "torch.Tensor | SlicedSum"
    bias: torch.Tensor

    @property
    def shape(self) -> torch.Size:
        return self.tensor.shape

    def sum(self) -> torch.Tensor:
        out = self.tensor.sum() if isinstance(self.tensor, SlicedSum) else self.tensor.clone()
        add_bias(out, self.bias)
        return out


@dataclass
class ScaledSum:
    """A sum ``scale_0 * (tensor_0 + bias_0) + scale_1 * (tensor_1 + bias_1)`` left to its consumer
    (:func:`norm_accumulate` computes it in 32-bit on the way): ``terms`` holds one or two
    ``(tensor, scale, bias or None)`` of equal shape, biases 32-bit vectors over the last dimension."""

    terms: list

    @property
    def shape(self) -> torch.Size:
        return self.terms[0][0].shape

    def sum(self) -> torch.Tensor:
        """The plain tensor, in the terms' type (32-bit arithmetic, one rounding)."""
        total = None
        for tensor, scale, bias in self.terms:
            if isinstance(tensor, ExpertSum):
                tensor = tensor.sum()
            value = tensor.float() if bias is None else tensor.float() + bias
            total = value * scale if total is None else total + value * scale
        return total.to(self.terms[0][0].dtype)   # (an ExpertSum carries its dtype too)


@dataclass
class ExpertSum:
    """The weighted sum of a token's routed experts left to its consumer: ``sum_k weights[t, k] * pair_out[t * top + k]`` over the
    pairs whose expert exists, in the order of ``k`` and in 32-bit (:func:`norm_accumulate` adds them on its way; :meth:`sum`
    gives the plain tensor in ``dtype``)."""

    pair_out: torch.Tensor  # float32 [tokens * top, width]
    weights: torch.Tensor  # float32 [tokens, top]
    chosen: torch.Tensor  # int32 [tokens, top]
    experts: int
    dtype: torch.dtype

    @property
    def shape(self) -> torch.Size:
        return torch.Size((self.chosen.shape[0], self.pair_out.shape[1]))

    def sum(self) -> torch.Tensor:
        tokens, top = self.chosen.shape
        out = torch.empty(tokens, self.pair_out.shape[1], dtype=self.dtype, device=self.pair_out.device)
        code = _lib().lb_moe_combine(_ptr(self.pair_out), _ptr(self.weights), _ptr(self.chosen), c_int(self.experts), _ptr(out), c_int(tokens), c_int(top),
                                     c_int(self.pair_out.shape[1]), c_int(dtype_code(self.dtype)), _stream())
        _done(code, "moe_combine")
        return out


_ACTIVATIONS = {"silu": 0, "gelu": 1, "identity": 2, "sigmoid_limit": 3}  # the last takes a `limit`, see csrc/common.cuh
_launches = 0


def launch_count() -> int:
    """Kernels of this library launched since the last reset."""
    return _launches


def add_launches(count: int) -> None:
    """Counts launches that did not go through these bindings (replays of a recorded graph)."""
    global _launches
    _launches += count


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


# The current stream's handle straight from torch's bindings where they exist: the public
# torch.cuda.current_stream() builds a Stream object and costs 3 us a call, which a step of a
# hundred-odd launches feels.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    if _raw_stream is not None and _raw_device is not None:
        return c_void_p(_raw_stream(_raw_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    if tensor is None:
        return c_void_p(0)
    return c_void_p(tensor.data_ptr())


def _check(tensor: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")


def _done(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code != 0:
        if code == -1:
            raise KernelError(f"{what}: unsupported element type")
        if code == -2:
            raise KernelError(f"{what}: a size is outside what the kernel supports")
        raise KernelError(f"{what}: CUDA error {code} at launch")
    _launches += launches


def _lib() -> ctypes.CDLL:
    return native.library()


# --------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float, status: torch.Tensor, accumulate: bool = False) -> None:
    """``out[t] = float(table[ids[t]]) * scale`` into the 32-bit residual stream (``accumulate``: added to it)."""
    _check(table, "table")
    _check(ids, "ids", torch.int32)
    _check(out, "out", torch.float32)
    tokens, dim = out.shape
    vocab = table.shape[0]
    if table.shape[1] != dim or ids.numel() < tokens:
        raise KernelError("embed: shapes of table, ids and out do not agree")
    code = _lib().lb_embed(_ptr(table), _ptr(ids), _ptr(out), c_int(tokens), c_int(dim), c_int(vocab), c_float(scale),
                           c_int(dtype_code(table.dtype)), _ptr(status), _stream(), c_int(1 if accumulate else 0))
    _done(code, "embed")


def rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    *,
    delta: "torch.Tensor | SlicedSum | BiasedSum | None" = None,
    rows: torch.Tensor | None = None,
    scale_offset: float = 0.0,
    write_back: bool = False,
    exact: bool = False,
    bias: torch.Tensor | None = None,
    centred: bool = False,
) -> None:
    """``out[r] = rms_norm(x[src] + delta[src]) * (weight + offset)``, ``src = rows[r]`` or ``r``.
    ``exact``: 32-bit throughout and rounded once (otherwise the normalised value and the scale are each rounded first).
    ``bias`` (32-bit, with ``exact``) is added to the output; ``centred`` (with ``exact``) makes it a layer norm,
    ``(h - mean) * rsqrt(mean((h - mean)^2) + eps) * (weight + offset) + bias``.  ``delta`` may carry a bias of its own
    (:class:`BiasedSum`), added to the stream with it.

    ``x`` is the 32-bit residual stream or has ``out``'s type.  With ``write_back`` the sum is
    stored back into ``x``.  ``delta`` may be a :class:`SlicedSum`: its slices are added here.
    """
    _check(x, "x")
    _check(weight, "weight", torch.float32)
    _check(out, "out")
    dim = x.shape[-1]
    out_rows = out.numel() // dim if dim else 0
    if out.shape[-1] != dim or weight.numel() != dim:
        raise KernelError("rmsnorm: the last dimensions of x, weight and out differ")
    if x.dtype != torch.float32 and x.dtype != out.dtype:
        raise KernelError("rmsnorm: x must be float32 or of out's type")
    partials, slices, slice_stride = None, 0, 0
    delta_bias = None
    if isinstance(delta, BiasedSum):
        delta, delta_bias = delta.tensor, delta.bias
        _check(delta_bias, "delta bias", torch.float32)
        if delta_bias.numel() != dim:
            raise KernelError("rmsnorm: the delta's bias must have one element per column")
    if (bias is not None or centred) and not exact:
        raise KernelError("rmsnorm: an output bias and the layer norm exist in the exact (32-bit) form only")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != dim:
            raise KernelError("rmsnorm: bias must have one element per column")
    if isinstance(delta, SlicedSum):
        _check(delta.partials, "delta.partials", torch.float32)
        if delta.shape != x.shape or delta.dtype != out.dtype:
            raise KernelError("rmsnorm: the sliced delta and x differ in shape, or its type is not out's")
        partials, slices, slice_stride = delta.partials, delta.partials.shape[0], delta.partials.shape[1] * delta.partials.shape[2]
        delta = None
    elif delta is not None:
        _check(delta, "delta", out.dtype)
        if delta.shape != x.shape:
            raise KernelError("rmsnorm: delta and x differ in shape")
    if rows is not None:
        _check(rows, "rows", torch.int32)
        if rows.numel() < out_rows:
            raise KernelError("rmsnorm: fewer row indices than output rows")
    elif out_rows != x.numel() // dim:
        raise KernelError("rmsnorm: x and out differ in rows")
    if dim > 50000:
        raise KernelError(f"rmsnorm: rows of {dim} elements exceed the supported 50000")
    code = _lib().lb_rmsnorm(_ptr(x), c_int(1 if x.dtype == torch.float32 else 0),
                             _ptr(delta), _ptr(partials), c_int(slices), c_longlong(slice_stride), _ptr(weight), _ptr(rows), _ptr(out), c_int(out_rows), c_int(dim), c_float(eps),
                             c_float(scale_offset), c_int(1 if write_back else 0), c_int(dtype_code(out.dtype)), _stream(), c_int(1 if exact else 0),
                             _ptr(bias), c_int(1 if centred else 0), _ptr(delta_bias))
    _done(code, "rmsnorm")


def _sum_slices(partials: torch.Tensor, out: torch.Tensor, epilogue: str) -> None:
    _check(partials, "partials", torch.float32)
    slices, tokens, rows = partials.shape
    if out.shape != (tokens, rows):
        raise KernelError("sum_slices: out must be [tokens, rows]")
    code = _lib().lb_sum_slices(_ptr(partials), _ptr(out), c_int(tokens), c_int(rows), c_int(slices), c_int(_TC_EPILOGUES[epilogue]), _stream())
    _done(code, "sum_slices")


def residual_add(x: torch.Tensor, delta: torch.Tensor | SlicedSum) -> None:
    """``x += delta`` on the 32-bit residual stream (a :class:`SlicedSum` is summed and rounded first)."""
    _check(x, "x", torch.float32)
    if isinstance(delta, BiasedSum):
        delta = delta.sum()
    if isinstance(delta, SlicedSum):
        if delta.dtype != torch.bfloat16:
            raise KernelError("residual_add: a sliced sum is rounded to bfloat16")
        _sum_slices(delta.partials, x, "residual_add")
        return
    _check(delta, "delta")
    if x.shape != delta.shape:
        raise KernelError("residual_add: shapes differ")
    code = _lib().lb_residual_add(_ptr(x), _ptr(delta), c_longlong(x.numel()), c_int(dtype_code(delta.dtype)), _stream())
    _done(code, "residual_add")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x`` rounded to ``out``'s type: the 32-bit residual stream as a sublayer's input."""
    _check(x, "x", torch.float32)
    _check(out, "out")
    if x.shape != out.shape:
        raise KernelError("cast_rows: shapes differ")
    code = _lib().lb_cast_rows(_ptr(x), _ptr(out), c_longlong(x.numel()), c_int(dtype_code(out.dtype)), _stream())
    _done(code, "cast_rows")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """``x[r, :] += bias`` in place (the sum in 32-bit, rounded to ``x``'s type)."""
    _check(x, "x")
    _check(bias, "bias", torch.float32)
    if x.dim() != 2 or bias.numel() != x.shape[1]:
        raise KernelError("add_bias: bias must have one element per column of x")
    code = _lib().lb_add_bias(_ptr(x), _ptr(bias), c_int(x.shape[0]), c_int(x.shape[1]), c_int(dtype_code(x.dtype)), _stream())
    _done(code, "add_bias")


def norm_accumulate(residual: torch.Tensor, delta: "torch.Tensor | ScaledSum", weight: torch.Tensor, eps: float, *,
                    scale_offset: float = 0.0, rounded: torch.Tensor | None = None, next_norm: tuple | None = None) -> None:
    """``residual += rms_norm(delta) * (weight + offset)`` on the 32-bit residual stream, everything in 32-bit;
    ``delta`` may be a :class:`ScaledSum` of one or two terms, summed here.  ``rounded`` (optional, of
    ``delta``'s type) receives the new stream rounded to that type or, with ``next_norm = (weight, eps, offset)``,
    the RMS norm of the new stream under that weight (32-bit, rounded once): what the next sublayer begins with."""
    _check(residual, "residual", torch.float32)
    _check(weight, "weight", torch.float32)
    terms = list(delta.terms) if isinstance(delta, ScaledSum) else [(delta, 1.0, None)]
    if not 1 <= len(terms) <= 2:
        raise KernelError("norm_accumulate: one or two terms")
    terms = [(tensor.sum() if index > 0 and isinstance(tensor, ExpertSum) else tensor, scale, bias) for index, (tensor, scale, bias) in enumerate(terms)]
    routed = terms[0][0] if isinstance(terms[0][0], ExpertSum) else None
    if routed is not None:
        # the first term comes as the experts' un-summed outputs: the kernel adds them; a stand-in of the right type and shape for the checks below
        for name, tensor, dtype in (("pair_out", routed.pair_out, torch.float32), ("weights", routed.weights, torch.float32), ("chosen", routed.chosen, torch.int32)):
            _check(tensor, name, dtype)
        if routed.shape != residual.shape or routed.pair_out.shape[0] != routed.chosen.numel() or routed.weights.shape != routed.chosen.shape:
            raise KernelError("norm_accumulate: the experts' outputs, weights and choices do not fit the residual stream")
        stand_in = terms[1][0] if len(terms) == 2 else torch.empty(residual.shape, dtype=routed.dtype, device=residual.device)
        terms[0] = (stand_in, terms[0][1], terms[0][2])
    first = terms[0][0]
    for tensor, _, bias in terms:
        _check(tensor, "delta", first.dtype)
        if tensor.shape != residual.shape:
            raise KernelError("norm_accumulate: delta and the residual stream differ in shape")
        if bias is not None:
            _check(bias, "bias", torch.float32)
            if bias.numel() != residual.shape[1]:
                raise KernelError("norm_accumulate: a bias must have one element per column")
    if weight.numel() != residual.shape[1]:
        raise KernelError("norm_accumulate: weight must have one element per column")
    if rounded is not None:
        _check(rounded, "rounded", first.dtype)
        if rounded.shape != residual.shape:
            raise KernelError("norm_accumulate: rounded and the residual stream differ in shape")
    second = terms[1] if len(terms) == 2 else (None, 0.0, None)
    next_weight, next_eps, next_offset = next_norm if next_norm is not None else (None, 0.0, 0.0)
    if next_weight is not None:
        _check(next_weight, "next_norm weight", torch.float32)
        if rounded is None or next_weight.numel() != residual.shape[1]:
            raise KernelError("norm_accumulate: the next norm needs `rounded` and a weight of one element per column")
    code = _lib().lb_norm_accumulate(_ptr(residual), _ptr(first), _ptr(terms[0][2]), c_float(terms[0][1]), _ptr(second[0]), _ptr(second[2]), c_float(second[1]),
                                     _ptr(weight), _ptr(rounded), c_int(residual.shape[0]), c_int(residual.shape[1]), c_float(eps), c_float(scale_offset),
                                     c_int(dtype_code(first.dtype)), _stream(), _ptr(next_weight), c_float(next_eps), c_float(next_offset),
                                     _ptr(routed.pair_out if routed is not None else None), _ptr(routed.weights if routed is not None else None),
                                     _ptr(routed.chosen if routed is not None else None), c_int(routed.chosen.shape[1] if routed is not None else 0),
                                     c_int(routed.experts if routed is not None else 0))
    _done(code, "norm_accumulate")


def scale_(x: torch.Tensor, factor: float, softcap: float = 0.0) -> None:
    """``x *= factor`` in place on a 32-bit tensor; with ``softcap`` > 0 then ``x = softcap * tanh(x / softcap)``."""
    _check(x, "x", torch.float32)
    if softcap < 0.0:
        raise KernelError("scale_: the cap must not be negative")
    _done(_lib().lb_scale(_ptr(x), c_float(factor), c_longlong(x.numel()), _stream(), c_float(softcap)), "scale")


def bias_activation(x: torch.Tensor, bias: torch.Tensor | None, activation: str) -> torch.Tensor:
    """``act(x + bias)`` (32-bit arithmetic, rounded once to ``x``'s type); ``activation``: ``"silu"``, ``"gelu"`` (exact) or ``"identity"``."""
    _check(x, "x")
    if activation not in ("silu", "gelu", "identity"):
        raise KernelError(f"bias_activation: unknown activation {activation!r}")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if x.dim() != 2 or bias.numel() != x.shape[1]:
            raise KernelError("bias_activation: bias must have one element per column of x")
    out = torch.empty_like(x)
    code = _lib().lb_bias_activation(_ptr(x), _ptr(bias), _ptr(out), c_int(x.shape[0]), c_int(x.shape[1]), c_int(_ACTIVATIONS[activation]),
                                     c_int(dtype_code(x.dtype)), _stream())
    _done(code, "bias_activation")
    return out


def stream_concat(stream: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float, status: torch.Tensor) -> torch.Tensor:
    """``[stream[t] | float(table[ids[t]]) * scale]`` per token, rounded to the table's type: the 32-bit residual stream and
    the embedding's output side by side, ``[tokens, 2 * dim]``."""
    _check(stream, "stream", torch.float32)
    _check(table, "table")
    _check(ids, "ids", torch.int32)
    tokens, dim = stream.shape
    if table.shape[1] != dim or ids.numel() < tokens:
        raise KernelError("stream_concat: shapes of stream, table and ids do not agree")
    out = torch.empty(tokens, 2 * dim, dtype=table.dtype, device=stream.device)
    code = _lib().lb_stream_concat(_ptr(stream), _ptr(table), _ptr(ids), _ptr(out), c_int(tokens), c_int(dim), c_int(table.shape[0]), c_float(scale),
                                   c_int(dtype_code(table.dtype)), _ptr(status), _stream())
    _done(code, "stream_concat")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _check(src, "src")
    _check(rows, "rows", torch.int32)
    _check(out, "out", src.dtype)
    dim = src.shape[-1]
    if out.shape[-1] != dim or rows.numel() < out.shape[0]:
        raise KernelError("gather_rows: shapes do not agree")
    code = _lib().lb_gather_rows(_ptr(src), _ptr(rows), _ptr(out), c_int(out.shape[0]), c_int(dim), c_int(src.element_size()), _stream())
    _done(code, "gather_rows")


def fill_slots(table: torch.Tensor, largest_bytes: int, slot: int, pattern: int = 0) -> None:
    """Fills slot ``slot`` of every per-request state tensor with the 32-bit ``pattern`` in one launch.
    ``table`` is int64 ``[states, 2]`` on the device: each state's base address and bytes per slot."""
    _check(table, "table", torch.int64)
    if table.dim() != 2 or table.shape[1] != 2:
        raise KernelError("fill_slots: table must be [states, 2]")
    if slot < 0:
        raise KernelError("fill_slots: negative slot")
    code = _lib().lb_fill_slots(_ptr(table), c_int(table.shape[0]), c_longlong(largest_bytes), c_int(slot), ctypes.c_uint(pattern & 0xFFFFFFFF), _stream())
    _done(code, "fill_slots")


def feed_tokens(token_ids: torch.Tensor, segment_start: torch.Tensor, segment_length: torch.Tensor, source: torch.Tensor,
                sampled: torch.Tensor, status: torch.Tensor | None = None) -> None:
    """Writes token ids that the step before sampled on the device into this step's ``token_ids``: the last
    token of segment ``s`` becomes ``sampled[source[s]]`` wherever ``source[s] >= 0``."""
    for name, tensor in (("token_ids", token_ids), ("segment_start", segment_start), ("segment_length", segment_length), ("source", source), ("sampled", sampled)):
        _check(tensor, name, torch.int32)
    segments = source.numel()
    if segment_start.numel() != segments or segment_length.numel() != segments:
        raise KernelError("feed_tokens: one start, length and source per segment")
    if status is not None:
        _check(status, "status", torch.int32)
    code = _lib().lb_feed_tokens(_ptr(token_ids), _ptr(segment_start), _ptr(segment_length), _ptr(source), _ptr(sampled), c_int(sampled.numel()),
                                 c_int(segments), _ptr(status), _stream())
    _done(code, "feed_tokens")


def gated_activation(fused: torch.Tensor, out: torch.Tensor, activation: str, limit: float = 0.0) -> None:
    """``out = up * act(gate)`` for ``fused = [up ; gate]`` along the last dimension (``"sigmoid_limit"``:
    ``g * sigmoid(1.702 g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``)."""
    _check(fused, "fused")
    _check(out, "out", fused.dtype)
    if activation not in _ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}; known: {sorted(_ACTIVATIONS)}")
    tokens, hidden = out.shape
    if fused.shape != (tokens, 2 * hidden):
        raise KernelError("gated_activation: fused must be [tokens, 2 * hidden]")
    code = _lib().lb_gated_activation(_ptr(fused), _ptr(out), c_int(tokens), c_int(hidden), c_int(_ACTIVATIONS[activation]),
                                      c_int(dtype_code(out.dtype)), _stream(), c_float(limit))
    _done(code, "gated_activation")


# ----------------------------------------------------------------------------- attention
def _check_paged(k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor, num_groups: int, head_dim: int,
                 value_dim: int | None = None) -> tuple[int, int, int]:
    _check(k_pages, "k_pages")
    _check(v_pages, "v_pages", k_pages.dtype)
    _check(block_table, "block_table", torch.int32)
    if k_pages.dim() != 4 or k_pages.shape[2:] != (num_groups, head_dim):
        raise KernelError("the key cache must be [pages, page_size, groups, head_dim]")
    if v_pages.shape != (k_pages.shape[0], num_groups, value_dim or head_dim, k_pages.shape[1]):
        raise KernelError("the value cache must be [pages, groups, value_dim, page_size] (values are stored transposed)")
    if block_table.dim() != 2:
        raise KernelError("block_table must be [segments, max_blocks]")
    return k_pages.shape[1], k_pages.shape[0], block_table.shape[1]


def qk_norm_rope_write(
    qkv: torch.Tensor,
    q_out: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    *,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    scale_offset: float,
    inv_freq: torch.Tensor | None,
    rotary_dim: int,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    write_kv: bool,
    status: torch.Tensor,
    value_dim: int | None = None,
    bias: torch.Tensor | None = None,
    whole_norm: bool = False,
    turn_scale: float = 1.0,
) -> None:
    """Splits ``qkv`` rows into heads, applies per-head norm and rotary embedding to queries and
    keys, writes queries to ``q_out`` and keys/values into their pages.  ``value_dim``: the size of a
    value head where it differs from ``head_dim``; ``bias``: a 32-bit vector over ``qkv``'s columns,
    added before the norm.  ``whole_norm``: the norm runs over all of a token's query columns at once (and
    over all of its key columns), with weights of one element per column, in 32-bit with no rounding before the
    rotation.  ``turn_scale`` multiplies sines and cosines.  ``qkv`` may be the first columns of a wider product."""
    if not qkv.is_cuda or qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("qk_norm_rope_write: qkv must be a [tokens, .] CUDA tensor with unit column stride")
    _check(q_out, "q_out", qkv.dtype)
    tokens = qkv.shape[0]
    value_dim = value_dim or head_dim
    if qkv.shape[1] != (num_heads + num_groups) * head_dim + num_groups * value_dim or q_out.numel() != tokens * num_heads * head_dim:
        raise KernelError("qk_norm_rope_write: qkv / q_out widths do not match the head counts")
    if whole_norm and (q_weight is None or bias is not None):
        raise KernelError("qk_norm_rope_write: a norm over the whole projection needs weights and takes no bias")
    row_inv = torch.empty(tokens, 2, dtype=torch.float32, device=qkv.device) if whole_norm else None
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != qkv.shape[1]:
            raise KernelError("qk_norm_rope_write: bias must have one element per column of qkv")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim, value_dim)
    if k_pages.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_write: cache and activations differ in type")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_norm_rope_write: give both norm weights or neither")
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _check(weight, name, torch.float32)
            if weight.numel() != (head_dim if not whole_norm else head_dim * (num_heads if name == "q_weight" else num_groups)):
                raise KernelError(f"{name} must have head_dim elements (one per column of the projection for a norm over the whole of it)")
    if rotary_dim:
        if inv_freq is None:
            raise KernelError("qk_norm_rope_write: rotary_dim > 0 needs inv_freq")
        _check(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2 or rotary_dim % 2 or rotary_dim > head_dim:
            raise KernelError("qk_norm_rope_write: inv_freq must have rotary_dim / 2 elements, rotary_dim even and <= head_dim")
    _check(positions, "positions", torch.int32)
    _check(token_segment, "token_segment", torch.int32)
    code = _lib().lb_qk_norm_rope_write(
        _ptr(qkv), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(q_weight), _ptr(k_weight), c_float(eps), c_float(scale_offset),
        _ptr(inv_freq), c_int(rotary_dim), _ptr(positions), _ptr(token_segment), _ptr(block_table), c_int(tokens), c_int(num_heads),
        c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks), c_int(1 if write_kv else 0),
        c_int(dtype_code(qkv.dtype)), _ptr(status), _stream(), c_int(value_dim), _ptr(bias), _ptr(row_inv), c_float(turn_scale), c_int(qkv.stride(0)))
    _done(code, "qk_norm_rope_write", 2 if whole_norm and tokens > 64 else 1)   # few tokens: the statistic is computed in the rewrite itself


def paged_attention_plain(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    *,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    scale: float,
    window: int | None,
    status: torch.Tensor,
    value_dim: int | None = None,
    keep_first: int = 0,
) -> None:
    """Causal (optionally windowed) attention of every token over its request's pages.  Under a window
    the first ``keep_first`` keys of a request stay visible.  ``value_dim``: the size of a value head
    (and of an output head) where it differs from ``head_dim``."""
    _check(q, "q")
    _check(out, "out", q.dtype)
    tokens = q.shape[0]
    value_dim = value_dim or head_dim
    if q.numel() != tokens * num_heads * head_dim or out.numel() != tokens * num_heads * value_dim:
        raise KernelError("paged_attention: q / out sizes do not match the head counts")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim, value_dim)
    if k_pages.dtype != q.dtype:
        raise KernelError("paged_attention: cache and queries differ in type")
    if value_dim > 512:
        raise KernelError(f"paged_attention: value_dim {value_dim} exceeds the supported 512")
    if keep_first < 0:
        raise KernelError("paged_attention: keep_first must not be negative")
    if num_heads % num_groups:
        raise KernelError("paged_attention: num_heads must be a multiple of num_groups")
    code = _lib().lb_paged_attention_plain(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(positions), _ptr(token_segment), _ptr(block_table), c_int(tokens),
        c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks), c_float(scale),
        c_int(window if window else 0), c_int(dtype_code(q.dtype)), _ptr(status), _stream(), c_int(value_dim), c_int(keep_first))
    _done(code, "paged_attention_plain")


DECODE_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128)
_sm_counts: dict[int, int] = {}
_decode_ctas_per_sm: dict[tuple[int, int], int] = {}


def sm_count() -> int:
    """Multiprocessors of the current device (asked once per device)."""
    device = torch.cuda.current_device()
    if device not in _sm_counts:
        _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[device]


def decode_ctas_per_sm(head_dim: int) -> int:
    """CTAs of the split-key attention kernel an SM of the current device holds at this head size
    (the library asks the runtime; registers and the ring's shared memory decide)."""
    key = (torch.cuda.current_device(), head_dim)
    if key not in _decode_ctas_per_sm:
        _decode_ctas_per_sm[key] = max(1, int(_lib().lb_attention_decode_ctas_per_sm(c_int(head_dim))))
    return _decode_ctas_per_sm[key]


def decode_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in DECODE_HEAD_DIMS and page_size % 16 == 0


def decode_attention_plan(tokens: int, num_heads: int, num_groups: int, max_context: int, window: int | None, head_dim: int = 64,
                          resident_ctas: int | None = None, keep_first: int = 0) -> tuple[int, int]:
    """``(splits, blocks_per_split)`` in 16-key blocks.  Depends on the batch's size and longest
    context only.  The grid has ``splits * pairs`` CTAs of four warps, of which the device holds
    ``resident_ctas`` to a round (default: its multiprocessors times three quarters of the CTAs each
    holds at this head size, rounded: measured, plans made for every resident CTA at once run 3 to
    9 % longer at batch 64, since the CTAs of a round do not start and end together); a CTA costs
    about six blocks' time beside the blocks each of its warps walks.  The number of splits that
    makes the fewest rounds' worth of that is taken, with at least eight blocks to a split."""
    span = min(max_context, window + 15) if window else max_context
    blocks_total = span // 16 + 1
    if window and keep_first:
        blocks_total = min(max_context // 16 + 1, blocks_total + -(-keep_first // 16))  # the blocks of the kept first keys come before the window's
    pairs = max(1, tokens * num_groups * -(-(num_heads // num_groups) // 16))
    slots = resident_ctas if resident_ctas is not None else sm_count() * ((3 * decode_ctas_per_sm(head_dim) + 2) // 4)
    best, best_cost = 1, None
    for splits in range(1, max(1, blocks_total // 8) + 1):
        per_warp = -(-(-(-blocks_total // splits)) // 4)
        cost = -(-pairs * splits // slots) * (per_warp + 6)
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    blocks_per_split = -(-blocks_total // best)
    return -(-blocks_total // blocks_per_split), blocks_per_split


def attention_decode(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    *,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    scale: float,
    window: int | None,
    max_context: int,
    status: torch.Tensor,
    scratch: torch.Tensor | None = None,
    token_list: torch.Tensor | None = None,
    num_listed: int | None = None,
    fresh_keys: int | None = None,
    keep_first: int = 0,
) -> None:
    """Split-key tensor-core attention for tokens that attend alone (bfloat16 only).  Under a window the
    first ``keep_first`` keys of a request stay visible.  ``max_context``
    is the largest position + 1 in the batch; it sizes the grid.  ``token_list`` (its first
    ``num_listed`` entries) restricts the call to some tokens of the batch.  ``fresh_keys``: the kernel
    launched just before on this stream is :func:`qk_norm_rope_write` (which lets its successor start
    early) and writes at most that many of the newest positions each token sees; the attention then
    starts early and reads the older keys while that kernel runs.  ``None``: an ordinary launch."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    if q.numel() != q.shape[0] * num_heads * head_dim or out.numel() != q.numel():
        raise KernelError("attention_decode: q / out sizes do not match the head counts")
    tokens = q.shape[0]
    if token_list is not None:
        _check(token_list, "token_list", torch.int32)
        tokens = token_list.numel() if num_listed is None else num_listed
        if tokens > token_list.numel():
            raise KernelError("attention_decode: token_list is shorter than num_listed")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim)
    if k_pages.dtype != torch.bfloat16:
        raise KernelError("attention_decode: the cache must be bfloat16")
    if not decode_attention_supported(q.dtype, head_dim, page_size):
        raise KernelError(f"attention_decode: head_dim {head_dim} (supported: {DECODE_HEAD_DIMS}) or page_size {page_size} (a multiple of 16) is not supported")
    if num_heads % num_groups:
        raise KernelError("attention_decode: num_heads must be a multiple of num_groups")
    keep_first = keep_first if window else 0
    splits, blocks_per_split = decode_attention_plan(tokens, num_heads, num_groups, max_context, window, head_dim, keep_first=keep_first)
    needed = tokens * num_heads * splits * (head_dim + 2)
    if scratch is None:
        scratch = torch.empty(needed, dtype=torch.float32, device=q.device)
    else:
        _check(scratch, "scratch", torch.float32)
        if scratch.numel() < needed:
            raise KernelError(f"attention_decode: scratch holds {scratch.numel()} floats, {needed} are needed")
    code = _lib().lb_attention_decode(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(scratch), _ptr(positions), _ptr(token_segment), _ptr(block_table),
        _ptr(token_list), c_int(tokens), c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks),
        c_float(scale), c_int(window if window else 0), c_int(splits), c_int(blocks_per_split), c_int(-1 if fresh_keys is None else fresh_keys),
        _ptr(status), _stream(), c_int(keep_first))
    _done(code, "attention_decode", 2 if splits > 1 else 1)   # the kernel and the merge of its splits


PREFILL_TILE = 32
PREFILL_MAX_HEADS_PER_CTA = 8


def prefill_attention_supported(dtype: torch.dtype, num_heads: int, num_groups: int, head_dim: int, page_size: int) -> bool:
    heads_per_group = num_heads // max(num_groups, 1)
    chunks = -(-heads_per_group // PREFILL_MAX_HEADS_PER_CTA)
    return decode_attention_supported(dtype, head_dim, page_size) and heads_per_group % chunks == 0


def attention_prefill(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    *,
    tiles: torch.Tensor,
    num_tiles: int,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    scale: float,
    window: int | None,
    status: torch.Tensor,
    kernel: str | None = None,
    split_tiles: int = 0,
    keep_first: int = 0,
) -> None:
    """Tensor-core attention for portions of prompts (bfloat16 only).  Under a window the first
    ``keep_first`` keys of a request stay visible.  ``tiles`` is ``[num_tiles, 2]``:
    first token and count (at most 32) of runs of consecutive tokens of one request.  Head size 64 runs
    on the tcgen05 kernel (scores and output in tensor memory), the other sizes on the ``mma.sync``
    one; ``kernel="mma"`` or ``"tcgen05"`` forces one of them.  ``split_tiles`` > 1 (tcgen05 kernel only):
    a tile that sees at least that many tiles of 64 keys is worked on by two CTAs, half of the keys each,
    for launches of few tiles that the longest tile's chain of keys would bound."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    _check(tiles, "tiles", torch.int32)
    if q.numel() != q.shape[0] * num_heads * head_dim or out.numel() != q.numel():
        raise KernelError("attention_prefill: q / out sizes do not match the head counts")
    if tiles.numel() < 2 * num_tiles:
        raise KernelError("attention_prefill: fewer tile records than num_tiles")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim)
    if not prefill_attention_supported(k_pages.dtype, num_heads, num_groups, head_dim, page_size):
        raise KernelError(f"attention_prefill: head_dim {head_dim} (supported: {DECODE_HEAD_DIMS}), page_size {page_size} (a multiple of 16) "
                          f"or {num_heads} heads over {num_groups} groups is not supported")
    if kernel not in (None, "mma", "tcgen05"):
        raise KernelError(f"attention_prefill: unknown kernel {kernel!r}")
    takes_tcgen05 = head_dim == 64 and num_heads // num_groups <= 128
    if kernel == "tcgen05" and not takes_tcgen05:
        raise KernelError(f"attention_prefill: the tcgen05 kernel takes head size 64 and up to 128 query heads per K/V head, not {head_dim} and {num_heads // num_groups}")
    if kernel == "tcgen05" or (kernel is None and takes_tcgen05 and USE_TCGEN05_ATTENTION):
        code = _lib().lb_attention_prefill_tcgen05(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tiles), c_int(num_tiles), c_int(q.shape[0]), _ptr(positions), _ptr(token_segment),
            _ptr(block_table), c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks),
            c_float(scale), c_int(window if window else 0), c_int(split_tiles), _ptr(status), _stream(), c_int(keep_first if window else 0))
        if code == -5:
            raise KernelError("attention_prefill: the driver made no tensor map for these tensors")
        _done(code, "attention_prefill (tcgen05)")
        return
    code = _lib().lb_attention_prefill(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tiles), c_int(num_tiles), _ptr(positions), _ptr(token_segment), _ptr(block_table),
        c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks), c_float(scale),
        c_int(window if window else 0), _ptr(status), _stream(), c_int(keep_first if window else 0))
    _done(code, "attention_prefill")


# ---------------------------------------------------------------------------- short conv
def short_conv(
    proj: torch.Tensor | SlicedSum,
    state: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    out: torch.Tensor,
    *,
    token_segment: torch.Tensor,
    segment_start: torch.Tensor,
    segment_length: torch.Tensor,
    segment_slot: torch.Tensor,
    segments: int,
    status: torch.Tensor,
) -> None:
    """Gated depthwise causal convolution of every portion, reading and updating each request's
    state slot (``state`` is ``[slots, kernel_size - 1, dim]``).  ``proj`` may be a :class:`SlicedSum`
    (the in-projection left in its K slices): a step of single tokens adds them in the convolution's own
    kernel, any other step sums them first."""
    _check(out, "out")
    _check(weight, "weight", torch.float32)
    tokens, dim = out.shape
    kernel_size = weight.shape[1]
    single_tokens = segments == tokens and out.dtype == torch.bfloat16 and dim % 8 == 0 and dim >= 8
    if isinstance(proj, SlicedSum):
        if proj.dtype != out.dtype:
            raise KernelError("short_conv: the sliced in-projection is rounded to another type than out's")
        if not single_tokens:
            proj = proj.sum()
    sliced = isinstance(proj, SlicedSum)
    if sliced:
        _check(proj.partials, "proj.partials", torch.float32)
    else:
        _check(proj, "proj", out.dtype)
    if tuple(proj.shape) != (tokens, 3 * dim) or weight.shape[0] != dim:
        raise KernelError("short_conv: proj must be [tokens, 3 * dim] and weight [dim, kernel_size]")
    if kernel_size > 1:
        _check(state, "state", out.dtype)
        if state.dim() != 3 or state.shape[1:] != (kernel_size - 1, dim):
            raise KernelError("short_conv: state must be [slots, kernel_size - 1, dim]")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != dim:
            raise KernelError("short_conv: bias must have dim elements")
    if single_tokens:
        # every portion is one token: one kernel for the slices' sum, the convolution and the state
        code = _lib().lb_short_conv_single(
            _ptr(proj.partials if sliced else None), c_int(proj.partials.shape[0] if sliced else 0), _ptr(None if sliced else proj), _ptr(state), _ptr(weight),
            _ptr(bias), _ptr(out), _ptr(token_segment), _ptr(segment_slot), c_int(tokens), c_int(dim), c_int(kernel_size), c_int(state.shape[0]), _ptr(status),
            _stream())
        _done(code, "short_conv_single")
        return
    code = _lib().lb_short_conv(
        _ptr(proj), _ptr(state), _ptr(weight), _ptr(bias), _ptr(out), _ptr(token_segment), _ptr(segment_start), _ptr(segment_length),
        _ptr(segment_slot), c_int(tokens), c_int(segments), c_int(dim), c_int(kernel_size), c_int(state.shape[0]),
        c_int(dtype_code(proj.dtype)), _ptr(status), _stream())
    _done(code, "short_conv", 2 if kernel_size > 1 else 1)


# ---------------------------------------------------------------------- gated delta rule
GDR_CHUNK_TOKENS = 256  # long portions are scanned in chunks of this many tokens, side by side
GDR_LONG_PORTION = 768  # portions of at least this many tokens count as long


def gated_delta_chunks_pay(key_dim: int, value_dim: int) -> bool:
    """Whether long portions should run as chunks: a chunk's scan carries ``key_dim`` further columns beside the
    ``value_dim`` of the state, and the chunks' states are put together in order afterwards.  Measured on 2,048-token
    portions: 64 x 128 heads 0.36 against 0.56 ms a layer, 128 x 128 heads 0.93 against 0.69 ms."""
    return 2 * key_dim <= value_dim


def gated_delta_chunk_plan(starts, lengths, chunk_tokens: int = GDR_CHUNK_TOKENS, long_portion: int = GDR_LONG_PORTION) -> dict:
    """The host's part of the chunked gated delta rule, from the portions' first rows and lengths alone: ``direct``
    (the portions scanned whole), ``chunk_start`` / ``chunk_length`` / ``chunk_slot`` (the chunks of the long portions,
    each with a temporary state of its own) and ``long_table`` (per long portion: its index, its first chunk, its number of
    chunks).  NumPy int32 arrays."""
    import numpy as np

    direct, chunk_start, chunk_length, long_table = [], [], [], []
    for index, (start, length) in enumerate(zip(starts, lengths)):
        if length < long_portion:
            direct.append(index)
            continue
        first = len(chunk_start)
        for offset in range(0, length, chunk_tokens):
            count = min(chunk_tokens, length - offset)
            chunk_start.append(start + offset)
            chunk_length.append(count)
        long_table.append((index, first, len(chunk_start) - first))
    as_array = lambda values: np.asarray(values, dtype=np.int32).reshape(-1)
    return {"direct": as_array(direct), "chunk_start": as_array(chunk_start), "chunk_length": as_array(chunk_length),
            "chunk_slot": np.arange(len(chunk_start), dtype=np.int32), "long_table": as_array(long_table)}


def gated_delta_rule(
    proj: torch.Tensor,
    low_rank: torch.Tensor,
    conv_state: torch.Tensor | None,
    matrix_state: torch.Tensor,
    *,
    conv_weight: torch.Tensor,
    a_log: torch.Tensor,
    dt_bias: torch.Tensor,
    norm_weight: torch.Tensor,
    norm_eps: float,
    num_heads: int,
    num_groups: int,
    key_dim: int,
    value_dim: int,
    unit_eps: float,
    token_segment: torch.Tensor,
    segment_start: torch.Tensor,
    segment_length: torch.Tensor,
    segment_slot: torch.Tensor,
    segments: int,
    status: torch.Tensor,
    chunk_plan: dict | None = None,
    decay_per_head: bool = False,
    gate_activation: str = "sigmoid",
    gate_offset: int | None = None,
) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel over the step's portions, from each
    request's state slot and back into it.  ``chunk_plan`` (see :func:`gated_delta_chunk_plan`; int32 arrays on
    the device with their sizes) lets long portions run as chunks side by side; without it every portion is
    scanned from its first token to its last.

    ``proj`` ``[tokens, >= C + heads]`` holds, per token, the pre-convolution q (``groups x key_dim``), k
    (the same) and v (``heads x value_dim``), ``C`` channels in all, then one beta logit per head;
    ``low_rank`` ``[tokens, heads * key_dim + heads * value_dim]`` the decay logits and the output gate's
    logits.  ``conv_weight`` is ``[C, taps]`` (last column: the current token), ``conv_state``
    ``[slots, taps - 1, C]`` (the convolutions' last inputs, in the activation type), ``matrix_state``
    ``[slots, heads, key_dim, value_dim]`` in 32-bit.  Returns the gated, normed read-out
    ``[tokens, heads * value_dim]`` in the activation type.

    ``decay_per_head``: one decay per head; ``low_rank`` then begins with ``heads`` decay logits and ``dt_bias`` has ``heads``
    elements.  ``gate_offset``: the column of ``low_rank`` at which the gate's logits begin (default: right after the decay
    logits).  ``gate_activation``: ``"sigmoid"`` or ``"silu"``.  ``low_rank`` may be a column slice of a wider product
    (of ``proj`` itself, for instance)."""
    _check(proj, "proj")
    if not low_rank.is_cuda or low_rank.dim() != 2 or low_rank.stride(1) != 1 or low_rank.dtype != proj.dtype:
        raise KernelError("gated_delta_rule: low_rank must be a [tokens, .] CUDA tensor of proj's type with unit column stride")
    if gate_activation not in ("sigmoid", "silu"):
        raise KernelError(f"gated_delta_rule: unknown gate activation {gate_activation!r}")
    _check(matrix_state, "matrix_state", torch.float32)
    for name, tensor in (("conv_weight", conv_weight), ("a_log", a_log), ("dt_bias", dt_bias), ("norm_weight", norm_weight)):
        _check(tensor, name, torch.float32)
    for name, tensor in (("token_segment", token_segment), ("segment_start", segment_start), ("segment_length", segment_length), ("segment_slot", segment_slot)):
        _check(tensor, name, torch.int32)
    tokens = proj.shape[0]
    channels = 2 * num_groups * key_dim + num_heads * value_dim
    taps = conv_weight.shape[1]
    if num_heads % num_groups or key_dim < 1 or key_dim > 256 or value_dim < 1:
        raise KernelError(f"gated_delta_rule: {num_heads} heads over {num_groups} groups with key size {key_dim} (at most 256) is not supported")
    decay_columns = num_heads if decay_per_head else num_heads * key_dim
    gate_offset = decay_columns if gate_offset is None else gate_offset
    if proj.shape[1] < channels + num_heads or low_rank.shape[0] != tokens or gate_offset < decay_columns or low_rank.shape[1] < gate_offset + num_heads * value_dim:
        raise KernelError("gated_delta_rule: proj or low_rank is too narrow for the head counts")
    if conv_weight.shape != (channels, taps) or a_log.numel() != num_heads or dt_bias.numel() != decay_columns or norm_weight.numel() != value_dim:
        raise KernelError("gated_delta_rule: conv_weight, a_log, dt_bias or norm_weight has the wrong size")
    num_slots = matrix_state.shape[0]
    if matrix_state.shape != (num_slots, num_heads, key_dim, value_dim):
        raise KernelError("gated_delta_rule: matrix_state must be [slots, heads, key_dim, value_dim]")
    if taps > 1:
        if conv_state is None:
            raise KernelError("gated_delta_rule: a convolution of more than one tap needs its state")
        _check(conv_state, "conv_state", proj.dtype)
        if conv_state.shape != (num_slots, taps - 1, channels):
            raise KernelError("gated_delta_rule: conv_state must be [slots, taps - 1, channels]")
    device = proj.device
    q = torch.empty(tokens, num_groups, key_dim, dtype=torch.float32, device=device)
    k = torch.empty_like(q)
    v = torch.empty(tokens, num_heads, value_dim, dtype=torch.float32, device=device)
    beta = torch.empty(tokens, num_heads, dtype=torch.float32, device=device)
    decay = torch.empty(tokens, num_heads, key_dim, dtype=torch.float32, device=device)
    lib = _lib()
    single_tokens = segments == tokens   # every portion is one token: the convolutions' kernel also writes their new state
    code = lib.lb_gdr_prepare(_ptr(proj), c_int(proj.shape[1]), _ptr(low_rank), c_int(low_rank.stride(0)), _ptr(conv_state), _ptr(conv_weight), _ptr(a_log),
                              _ptr(dt_bias), _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(decay), _ptr(token_segment), _ptr(segment_start), _ptr(segment_slot),
                              c_int(tokens), c_int(num_heads), c_int(num_groups), c_int(key_dim), c_int(value_dim), c_int(taps), c_int(num_slots),
                              c_float(unit_eps), c_float(key_dim ** -0.5), c_int(dtype_code(proj.dtype)), _ptr(status), _stream(), c_int(1 if single_tokens else 0),
                              c_int(1 if decay_per_head else 0))
    _done(code, "gdr_prepare")
    if taps > 1 and not single_tokens:
        code = lib.lb_gdr_conv_state(_ptr(proj), c_int(proj.shape[1]), _ptr(conv_state), _ptr(segment_start), _ptr(segment_length), _ptr(segment_slot),
                                     c_int(segments), c_int(channels), c_int(taps), c_int(num_slots), c_int(dtype_code(proj.dtype)), _stream())
        _done(code, "gdr_conv_state")
    read_out = torch.empty(tokens, num_heads, value_dim, dtype=torch.float32, device=device)
    direct_list, num_direct = None, segments
    if chunk_plan is not None and chunk_plan["num_chunks"] > 0 and not gated_delta_chunks_pay(key_dim, value_dim):
        chunk_plan = None
    if chunk_plan is not None and chunk_plan["num_chunks"] > 0:
        # Long portions: their chunks are scanned side by side from zero states, with key_dim further columns that carry
        # each chunk's transition; then the chunks' incoming states in order, and the read-outs' second term.
        num_chunks, num_long = chunk_plan["num_chunks"], chunk_plan["num_long"]
        wide_dim = value_dim + key_dim
        wide = torch.empty(tokens, num_heads, wide_dim, dtype=torch.float32, device=device)
        chunk_state = torch.empty(num_chunks, num_heads, key_dim, wide_dim, dtype=torch.float32, device=device)
        chunk_in = torch.empty(num_chunks, num_heads, key_dim, value_dim, dtype=torch.float32, device=device)
        _done(lib.lb_gdr_chunk_init(_ptr(chunk_state), c_int(num_chunks), c_int(num_heads), c_int(key_dim), c_int(value_dim), _stream()), "gdr_chunk_init")
        code = lib.lb_gdr_scan(_ptr(q), _ptr(k), _ptr(decay), _ptr(v), _ptr(beta), _ptr(chunk_state), _ptr(wide), _ptr(chunk_plan["chunk_start"]),
                               _ptr(chunk_plan["chunk_length"]), _ptr(chunk_plan["chunk_slot"]), c_int(num_chunks), c_int(num_heads), c_int(num_groups),
                               c_int(key_dim), c_int(wide_dim), c_int(num_chunks), _ptr(status), _stream(), _ptr(None), c_int(value_dim))
        _done(code, "gdr_scan (chunks)")
        code = lib.lb_gdr_chunk_finish(_ptr(chunk_state), _ptr(chunk_in), _ptr(matrix_state), _ptr(wide), _ptr(read_out), _ptr(chunk_plan["long_table"]),
                                       c_int(num_long), _ptr(segment_slot), _ptr(chunk_plan["chunk_start"]), _ptr(chunk_plan["chunk_length"]), c_int(num_chunks),
                                       c_int(chunk_plan.get("chunk_tokens", GDR_CHUNK_TOKENS)), c_int(num_heads), c_int(key_dim), c_int(value_dim), c_int(num_slots),
                                       _stream())
        _done(code, "gdr_chunk_finish", 2)
        direct_list, num_direct = chunk_plan["direct"], chunk_plan["num_direct"]
    if num_direct > 0:
        code = lib.lb_gdr_scan(_ptr(q), _ptr(k), _ptr(decay), _ptr(v), _ptr(beta), _ptr(matrix_state), _ptr(read_out), _ptr(segment_start), _ptr(segment_length),
                               _ptr(segment_slot), c_int(num_direct), c_int(num_heads), c_int(num_groups), c_int(key_dim), c_int(value_dim), c_int(num_slots),
                               _ptr(status), _stream(), _ptr(direct_list), c_int(value_dim))
        _done(code, "gdr_scan")
    out = torch.empty(tokens, num_heads * value_dim, dtype=proj.dtype, device=device)
    code = lib.lb_gdr_output(_ptr(read_out), _ptr(low_rank), c_int(low_rank.stride(0)), c_int(gate_offset), _ptr(norm_weight), _ptr(out), c_int(tokens),
                             c_int(num_heads), c_int(value_dim), c_float(norm_eps), c_int(dtype_code(proj.dtype)), _stream(), c_int(1 if gate_activation == "silu" else 0))
    _done(code, "gdr_output")
    return out


# ---------------------------------------------------------------------- latent attention
def heads_linear(x: torch.Tensor, weight: torch.Tensor, transpose_weight: bool = False) -> torch.Tensor:
    """One small product per head: ``out[h] = x[h] @ weight[h]`` (``transpose_weight``: ``x[h] @ weight[h].T``) for
    ``x [heads, tokens, k]`` (any strides with the last one 1) and ``weight [heads, k, n]`` (``[heads, n, k]``);
    32-bit accumulation, ``out [heads, tokens, n]`` contiguous in ``x``'s type.  A library product (batched)."""
    if x.dim() != 3 or weight.dim() != 3 or x.shape[0] != weight.shape[0] or x.dtype != weight.dtype or not x.is_cuda:
        raise KernelError("heads_linear: x [heads, tokens, k] and weight [heads, ., .] must agree in heads, type and device")
    return torch.bmm(x, weight.transpose(1, 2) if transpose_weight else weight)


def heads_product_supported(dtype: torch.dtype, k: int, n: int) -> bool:
    """Whether :func:`heads_product` (the framework's own kernel) takes a per-head product of these sizes."""
    return dtype == torch.bfloat16 and k >= 16 and n >= 16 and k % 16 == 0 and n % 16 == 0 and (64 * (k + 8) + max(k * 72, 64 * (k + 8))) * 2 <= 227 * 1024


def heads_product(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, *, weight_is_kn: bool, gate: torch.Tensor | None = None) -> None:
    """``out[t, h] = x[t, h] @ weight[h]`` (``weight [heads, k, n]``, ``weight_is_kn``) or ``x[t, h] @ weight[h].T`` (``weight [heads, n, k]``),
    optionally times ``sigmoid(gate[t, h])``; bfloat16 on the tensor cores with 32-bit sums.  ``x [tokens, heads, k]``, ``out`` and ``gate``
    ``[tokens, heads, n]`` may be views with any token and head strides (column slices of wider products, parts of wider rows)."""
    _check(weight, "weight", torch.bfloat16)
    tokens, heads, k = x.shape
    n = weight.shape[2] if weight_is_kn else weight.shape[1]
    if weight.shape != ((heads, k, n) if weight_is_kn else (heads, n, k)) or out.shape != (tokens, heads, n) or not heads_product_supported(x.dtype, k, n):
        raise KernelError(f"heads_product: x {tuple(x.shape)}, weight {tuple(weight.shape)} and out {tuple(out.shape)} are not shapes the kernel takes")
    for name, tensor in (("x", x), ("out", out), ("gate", gate)):
        if tensor is not None and (not tensor.is_cuda or tensor.dtype != torch.bfloat16 or tensor.stride(2) != 1 or (name == "gate" and tensor.shape != out.shape)):
            raise KernelError(f"heads_product: {name} must be a bfloat16 CUDA tensor [tokens, heads, .] with unit stride along the last dimension")
    code = _lib().lb_heads_product(_ptr(x), c_longlong(x.stride(0)), c_int(x.stride(1)), _ptr(weight), c_int(1 if weight_is_kn else 0), _ptr(out),
                                   c_longlong(out.stride(0)), c_int(out.stride(1)), _ptr(gate), c_longlong(gate.stride(0) if gate is not None else 0),
                                   c_int(gate.stride(1) if gate is not None else 0), c_int(tokens), c_int(heads), c_int(k), c_int(n), _stream())
    _done(code, "heads_product")


def _check_latent_pages(pages: torch.Tensor, block_table: torch.Tensor, latent: int, rope: int) -> tuple[int, int, int]:
    _check(pages, "pages")
    _check(block_table, "block_table", torch.int32)
    if pages.dim() != 4 or pages.shape[2:] != (1, latent + rope):
        raise KernelError("the latent cache must be [pages, page_size, 1, latent + rope]")
    if block_table.dim() != 2:
        raise KernelError("block_table must be [segments, max_blocks]")
    return pages.shape[1], pages.shape[0], block_table.shape[1]


def latent_prepare(q: torch.Tensor, q_latent: torch.Tensor | None, down: torch.Tensor, q_out: torch.Tensor, pages: torch.Tensor, *, norm_weight: torch.Tensor,
                   eps: float, scale_offset: float, inv_freq: torch.Tensor, positions: torch.Tensor, token_segment: torch.Tensor,
                   block_table: torch.Tensor, num_heads: int, head_dim: int, latent: int, rope: int, write_kv: bool, status: torch.Tensor) -> None:
    """Latent attention's step between the projections and the attention.  ``q [tokens, heads * (head_dim + rope)]`` and
    ``down [tokens, latent + rope]`` may be column slices of a wider product (row strides are passed on).  Writes the
    row ``[norm(down[:latent]) * (norm_weight + scale_offset) | rope(down[latent:])]`` into the token's page and the
    queries ``[q_latent[h, t] | rope(q[t, h, head_dim:])]`` into ``q_out [tokens, heads, latent + rope]`` (``q_latent=None``:
    the latent parts are in ``q_out`` already and stay); the rotation pairs channel ``i`` with ``i + rope / 2``."""
    tokens = q_out.shape[0]
    for name, tensor in (("q", q), ("down", down)):
        if not tensor.is_cuda or tensor.dim() != 2 or tensor.stride(1) != 1 or tensor.dtype != q_out.dtype or tensor.shape[0] != tokens:
            raise KernelError(f"latent_prepare: {name} must be a [tokens, .] CUDA tensor of q_out's type with unit column stride")
    if q_latent is not None:
        _check(q_latent, "q_latent", q_out.dtype)
    _check(q_out, "q_out")
    _check(norm_weight, "norm_weight", torch.float32)
    _check(inv_freq, "inv_freq", torch.float32)
    _check(positions, "positions", torch.int32)
    _check(token_segment, "token_segment", torch.int32)
    if (q.shape[1] != num_heads * (head_dim + rope) or down.shape[1] != latent + rope or (q_latent is not None and q_latent.shape != (num_heads, tokens, latent))
            or q_out.shape != (tokens, num_heads, latent + rope) or norm_weight.numel() != latent or inv_freq.numel() != rope // 2 or rope % 2):
        raise KernelError("latent_prepare: the sizes of q, q_latent, down, q_out, the norm's weight and the frequencies do not agree")
    page_size, num_pages, max_blocks = _check_latent_pages(pages, block_table, latent, rope)
    if pages.dtype != q_out.dtype:
        raise KernelError("latent_prepare: cache and activations differ in type")
    code = _lib().lb_latent_prepare(_ptr(q), c_int(q.stride(0)), _ptr(q_latent), _ptr(down), c_int(down.stride(0)), _ptr(q_out), _ptr(pages), _ptr(norm_weight),
                                    c_float(eps), c_float(scale_offset), _ptr(inv_freq), _ptr(positions), _ptr(token_segment), _ptr(block_table), c_int(tokens),
                                    c_int(num_heads), c_int(head_dim), c_int(latent), c_int(rope), c_int(page_size), c_int(num_pages), c_int(max_blocks),
                                    c_int(1 if write_kv else 0), c_int(dtype_code(q_out.dtype)), _ptr(status), _stream())
    _done(code, "latent_prepare")


def _check_sink(sink: torch.Tensor | None, num_heads: int) -> None:
    if sink is not None:
        _check(sink, "sink", torch.float32)
        if sink.numel() != num_heads:
            raise KernelError("latent attention: the sink must have one number per head")


def latent_attention_plain(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, *, positions: torch.Tensor, token_segment: torch.Tensor,
                           block_table: torch.Tensor, num_heads: int, latent: int, rope: int, scale: float, window: int | None,
                           status: torch.Tensor, sink: torch.Tensor | None = None) -> None:
    """Causal (optionally windowed) attention of queries ``[tokens, heads, latent + rope]`` over their requests' cached rows
    ``[latent | rope]``: ``out[t, h] = sum_j softmax_j(q[t, h] . row_j * scale) row_j[:latent]``, all in 32-bit.  ``sink``
    (32-bit, one number per head): ``exp(sink[h])`` joins the softmax's denominator, unscaled and with no row behind it."""
    _check_sink(sink, num_heads)
    _check(q, "q")
    _check(out, "out", q.dtype)
    tokens = q.shape[0]
    if q.shape != (tokens, num_heads, latent + rope) or out.shape != (tokens, num_heads, latent):
        raise KernelError("latent_attention: q must be [tokens, heads, latent + rope] and out [tokens, heads, latent]")
    page_size, num_pages, max_blocks = _check_latent_pages(pages, block_table, latent, rope)
    if pages.dtype != q.dtype:
        raise KernelError("latent_attention: cache and queries differ in type")
    if latent > 1024 or (latent + rope) * 4 > 40 * 1024:
        raise KernelError(f"latent_attention: latent {latent} + rope {rope} exceed what the kernel supports")
    code = _lib().lb_latent_attention_plain(_ptr(q), _ptr(pages), _ptr(out), _ptr(positions), _ptr(token_segment), _ptr(block_table), c_int(tokens),
                                            c_int(num_heads), c_int(latent), c_int(rope), c_int(page_size), c_int(num_pages), c_int(max_blocks),
                                            c_float(scale), c_int(window if window else 0), c_int(dtype_code(q.dtype)), _ptr(status), _stream(), _ptr(sink))
    _done(code, "latent_attention_plain")


LATENT_MMA_ROWS = 64  # query rows (tokens x heads) of one CTA of the tensor-core latent attention


def latent_attention_supported(dtype: torch.dtype, latent: int, rope: int, page_size: int) -> bool:
    """Whether :func:`latent_attention` (tensor cores) takes these sizes; :func:`latent_attention_plain` takes the rest."""
    return dtype == torch.bfloat16 and latent >= 16 and latent % 16 == 0 and rope % 16 == 0 and page_size % 16 == 0 and 3 * 64 * (latent + rope + 8) * 2 <= 227 * 1024


def latent_attention_tiling(num_heads: int) -> tuple[int, int]:
    """``(heads, tokens)`` of one CTA's query rows: all heads of as many consecutive tokens as fit (blocks of 64 heads beyond that)."""
    heads = min(num_heads, LATENT_MMA_ROWS)
    return heads, max(1, LATENT_MMA_ROWS // heads)


def latent_attention_splits(num_items: int, num_heads: int, latent: int, window: int | None, max_context: int, sms: int | None = None) -> int:
    """Over how many CTAs an item's cached rows are shared out: 1 where the items fill the GPU by themselves."""
    heads, tokens = latent_attention_tiling(num_heads)
    ctas = num_items * -(-num_heads // heads) * -(-latent // (256 if latent > 128 else 128))
    sms = sms or sm_count()
    rows = min(window, max_context) if window else max_context
    blocks = -(-(rows + tokens) // 64) + 1
    if ctas >= 2 * sms or blocks <= 2:
        return 1
    return max(1, min(blocks // 2, -(-2 * sms // ctas), 32))   # two blocks a CTA: one block each was measured 1 % slower


def latent_attention(q: torch.Tensor, pages: torch.Tensor, out: torch.Tensor, *, items: torch.Tensor, num_items: int, positions: torch.Tensor,
                     token_segment: torch.Tensor, block_table: torch.Tensor, num_heads: int, latent: int, rope: int, scale: float, window: int | None,
                     status: torch.Tensor, splits: int = 1, sink: torch.Tensor | None = None) -> None:
    """:func:`latent_attention_plain` on the tensor cores (bfloat16).  ``items``: int32 ``[num_items, 2]`` (first token row,
    count), each at most ``latent_attention_tiling(num_heads)[1]`` consecutive tokens of one request, together all tokens.
    ``splits`` > 1 shares an item's cached rows out over that many CTAs, merged in split order.  ``sink``: as for
    :func:`latent_attention_plain`."""
    _check_sink(sink, num_heads)
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    _check(items, "items", torch.int32)
    tokens = q.shape[0]
    if q.shape != (tokens, num_heads, latent + rope) or out.shape != (tokens, num_heads, latent) or items.numel() < 2 * num_items:
        raise KernelError("latent_attention: q must be [tokens, heads, latent + rope], out [tokens, heads, latent], items [num_items, 2]")
    page_size, num_pages, max_blocks = _check_latent_pages(pages, block_table, latent, rope)
    if pages.dtype != q.dtype or not latent_attention_supported(q.dtype, latent, rope, page_size):
        raise KernelError(f"latent_attention: latent {latent}, rope {rope}, pages of {page_size} are not sizes the tensor-core kernel takes")
    heads_per_cta, tokens_per_cta = latent_attention_tiling(num_heads)
    partial = torch.empty(tokens, num_heads, splits, latent + 2, dtype=torch.float32, device=q.device) if splits > 1 else None
    code = _lib().lb_latent_attention_mma(_ptr(q), _ptr(pages), _ptr(out), _ptr(partial), _ptr(items), c_int(num_items), _ptr(positions), _ptr(token_segment),
                                          _ptr(block_table), c_int(tokens), c_int(num_heads), c_int(latent), c_int(rope), c_int(page_size), c_int(num_pages),
                                          c_int(max_blocks), c_float(scale), c_int(window if window else 0), c_int(heads_per_cta), c_int(tokens_per_cta),
                                          c_int(splits), _ptr(status), _stream(), _ptr(sink))
    _done(code, "latent_attention_mma", 2 if splits > 1 else 1)


def gate_heads(values: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor) -> None:
    """``out[t, h * vdim + j] = values[h, t, j] * sigmoid(gate[t, h * vdim + j])`` (``gate=None``: no gate); ``gate`` may
    be a column slice of a wider product."""
    _check(values, "values")
    _check(out, "out", values.dtype)
    heads, tokens, value_dim = values.shape
    if out.shape != (tokens, heads * value_dim):
        raise KernelError("gate_heads: out must be [tokens, heads * vdim]")
    stride = 0
    if gate is not None:
        if not gate.is_cuda or gate.dtype != values.dtype or gate.shape != out.shape or gate.stride(1) != 1:
            raise KernelError("gate_heads: gate must be [tokens, heads * vdim] of the values' type with unit column stride")
        stride = gate.stride(0)
    code = _lib().lb_gate_heads(_ptr(values), _ptr(gate), c_int(stride), _ptr(out), c_int(tokens), c_int(heads), c_int(value_dim),
                                c_int(dtype_code(values.dtype)), _stream())
    _done(code, "gate_heads")


# ------------------------------------------------------------------------ routed experts
_ROUTER_SCORES = {"sigmoid": 0, "softmax": 1, "logits": 2}


def moe_route(x: torch.Tensor, router: torch.Tensor, *, top: int, group_count: int = 1, group_keep: int = 1, score: str = "sigmoid",
              renormalize: bool = False, weight_scale: float = 1.0, bias: torch.Tensor | None = None,
              chosen_softmax: bool = False, choice_bias: torch.Tensor | None = None, extra: int = 0) -> tuple:
    """Chooses ``top`` experts per token: 32-bit router logits ``x @ router.T``, scores (``"sigmoid"`` or
    ``"softmax"``), only experts of the ``group_keep`` best of ``group_count`` groups of neighbours eligible
    (a group's score: the sum of its two largest scores).  Returns ``(chosen int32 [tokens, top], weights
    float32 [tokens, top])``, the weights being the chosen scores (over their sum if ``renormalize``; their softmax
    if ``chosen_softmax``) times ``weight_scale``.  ``bias`` (32-bit, one per expert) is added to the logits;
    ``score="logits"`` ranks by the logits themselves.  ``choice_bias`` (32-bit, one per expert) is added to the scores where
    experts are ranked, not where they weigh.  ``extra``: the router's last ``extra`` rows are no experts but gates; the
    sigmoids of their logits are returned as a third value, float32 ``[tokens, extra]``."""
    _check(x, "x")
    _check(router, "router", torch.float32)
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != router.shape[0] - extra:
            raise KernelError("moe_route: the bias must have one element per expert")
    if score not in _ROUTER_SCORES:
        raise KernelError(f"moe_route: unknown score {score!r}; known: {sorted(_ROUTER_SCORES)}")
    tokens, width = x.shape
    if extra < 0 or extra >= router.shape[0]:
        raise KernelError("moe_route: the router must have rows for the experts besides the extra ones")
    experts = router.shape[0] - extra
    if router.shape[1] != width:
        raise KernelError("moe_route: the router's width is not x's")
    if choice_bias is not None:
        _check(choice_bias, "choice_bias", torch.float32)
        if choice_bias.numel() != experts:
            raise KernelError("moe_route: the choice bias must have one element per expert")
    if not (1 <= top <= experts and group_count >= 1 and experts % group_count == 0 and 1 <= group_keep <= group_count):
        raise KernelError(f"moe_route: top {top} of {experts} experts in {group_count} groups of which {group_keep} are kept is not a valid choice")
    if 4 * (2 * experts + extra + group_count) * 4 > 48 * 1024:
        raise KernelError(f"moe_route: {experts} experts exceed the kernel's shared memory")
    chosen = torch.empty(tokens, top, dtype=torch.int32, device=x.device)
    weights = torch.empty(tokens, top, dtype=torch.float32, device=x.device)
    extra_out = torch.empty(tokens, extra, dtype=torch.float32, device=x.device) if extra else None
    code = _lib().lb_moe_route(_ptr(x), _ptr(router), _ptr(chosen), _ptr(weights), c_int(tokens), c_int(width), c_int(experts), c_int(top), c_int(group_count),
                               c_int(group_keep), c_int(_ROUTER_SCORES[score]), c_int(2 if chosen_softmax else 1 if renormalize else 0), c_float(weight_scale),
                               c_int(dtype_code(x.dtype)), _stream(), _ptr(bias), _ptr(choice_bias), c_int(extra), _ptr(extra_out))
    _done(code, "moe_route")
    if extra:
        return chosen, weights, extra_out
    return chosen, weights


MOE_STREAM_MAX_PAIRS = 32  # up to this many (token, expert) pairs each pair streams its expert's weights; more are grouped by expert (measured: 24 pairs 30 % faster streamed, 48 pairs as fast either way)


def moe_experts(x: torch.Tensor, gate: "torch.Tensor | None", up: torch.Tensor, down: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor,
                activation: str = "silu", path: str | None = None, limit: float = 0.0, combine: bool = True) -> "torch.Tensor | ExpertSum":
    """``out[t] = sum_k weights[t, k] * down[e] (act(gate[e] x[t]) * (up[e] x[t]))`` with ``e = chosen[t, k]``;
    ``gate`` and ``up`` are ``[experts, ff, width]``, ``down`` ``[experts, width, ff]``.  The weighted sum is
    32-bit, in the order of ``k``; a pair whose expert is no expert counts nothing.  ``path`` forces one of the
    three ways the pairs' products are computed (``"grouped"``, ``"stream"``, ``"plain"``); left out, the sizes
    choose.  ``combine=False`` leaves the weighted sum to the consumer (an :class:`ExpertSum`).  ``gate=None``: experts
    without a gate, ``down[e] act(up[e] x[t])`` (the activation in 32-bit on the 32-bit sums, rounded once)."""
    _check(x, "x")
    for name, tensor in (("gate", gate), ("up", up), ("down", down)):
        if tensor is not None:
            _check(tensor, name, x.dtype)
    _check(chosen, "chosen", torch.int32)
    _check(weights, "weights", torch.float32)
    if activation not in _ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}; known: {sorted(_ACTIVATIONS)}")
    tokens, width = x.shape
    experts, ff = up.shape[0], up.shape[1]
    top = chosen.shape[1]
    if up.shape != (experts, ff, width) or (gate is not None and gate.shape != up.shape) or down.shape != (experts, width, ff) or chosen.shape != (tokens, top) or weights.shape != chosen.shape:
        raise KernelError("moe_experts: shapes of x, the experts' weights, chosen and weights do not agree")
    if (width + ff) * 4 > 200 * 1024:
        raise KernelError("moe_experts: width + ff exceed the kernel's shared memory")
    pairs = tokens * top
    pair_out = torch.empty(pairs, width, dtype=torch.float32, device=x.device)
    vector = 8 if x.dtype == torch.bfloat16 else 4
    wide_rows = width % vector == 0 and ff % vector == 0 and max(width, ff) * 4 <= 160 * 1024
    lib = _lib()
    if path is None:
        path = "grouped" if x.dtype == torch.bfloat16 and wide_rows and experts <= 1024 and pairs > MOE_STREAM_MAX_PAIRS else "stream" if wide_rows else "plain"
    if path == "grouped":
        # many pairs: sorted by expert, 64 at a time on the tensor cores, every expert's weights read once per 64 pairs
        if not (x.dtype == torch.bfloat16 and wide_rows and experts <= 1024):
            raise KernelError("moe_experts: the grouped kernels take bfloat16, rows of 16-byte multiples and at most 1024 experts")
        offsets = torch.empty(experts + 1, dtype=torch.int32, device=x.device)
        order = torch.empty(pairs, dtype=torch.int32, device=x.device)
        hidden = torch.empty(pairs, ff, dtype=x.dtype, device=x.device)
        code = lib.lb_moe_experts_grouped(_ptr(x), _ptr(gate), _ptr(up), _ptr(down), _ptr(chosen), _ptr(offsets), _ptr(order), _ptr(hidden), _ptr(pair_out),
                                          c_int(pairs), c_int(top), c_int(width), c_int(ff), c_int(experts), c_int(_ACTIVATIONS[activation]), _stream(), c_float(limit))
        _done(code, "moe_experts_grouped", 3)
    elif path == "stream":
        # few pairs: each streams its expert's rows, 16 bytes a lane, the rows shared out over many blocks
        if not wide_rows:
            raise KernelError("moe_experts: the streaming kernels take rows of 16-byte multiples")
        hidden = torch.empty(pairs, ff, dtype=x.dtype, device=x.device)
        code = lib.lb_moe_expert_stream_wide(_ptr(x), _ptr(gate), _ptr(up), _ptr(down), _ptr(chosen), _ptr(hidden), _ptr(pair_out), c_int(pairs), c_int(top),
                                             c_int(width), c_int(ff), c_int(experts), c_int(_ACTIVATIONS[activation]), c_int(dtype_code(x.dtype)), _stream(), c_float(limit))
        _done(code, "moe_expert_stream_wide", 2)
    elif path == "plain":
        code = lib.lb_moe_expert_stream(_ptr(x), _ptr(gate), _ptr(up), _ptr(down), _ptr(chosen), _ptr(pair_out), c_int(pairs), c_int(top), c_int(width),
                                        c_int(ff), c_int(experts), c_int(_ACTIVATIONS[activation]), c_int(dtype_code(x.dtype)), _stream(), c_float(limit))
        _done(code, "moe_expert_stream")
    else:
        raise KernelError(f"moe_experts: unknown path {path!r}")
    if not combine:
        return ExpertSum(pair_out, weights, chosen, experts, x.dtype)   # the consumer adds the pairs' outputs
    out = torch.empty(tokens, width, dtype=x.dtype, device=x.device)
    code = lib.lb_moe_combine(_ptr(pair_out), _ptr(weights), _ptr(chosen), c_int(experts), _ptr(out), c_int(tokens), c_int(top), c_int(width),
                              c_int(dtype_code(x.dtype)), _stream())
    _done(code, "moe_combine")
    return out


def moe_combine_add(routed: ExpertSum, residual: torch.Tensor, every: torch.Tensor | None = None, every_gate: torch.Tensor | None = None) -> None:
    """``residual[t] += sum_k weights[t, k] * pair_out[t * top + k] + every_gate[t] * every[t]`` on the 32-bit residual stream, in
    32-bit: the routed experts' weighted sum, what every token runs besides (``every``, optional, in the activation type) times
    a 32-bit number per token (``every_gate`` ``[tokens, 1]`` or ``[tokens]``; left out: 1)."""
    _check(residual, "residual", torch.float32)
    for name, tensor, dtype in (("pair_out", routed.pair_out, torch.float32), ("weights", routed.weights, torch.float32), ("chosen", routed.chosen, torch.int32)):
        _check(tensor, name, dtype)
    tokens, top = routed.chosen.shape
    width = routed.pair_out.shape[1]
    if residual.shape != (tokens, width) or routed.pair_out.shape[0] != tokens * top or routed.weights.shape != routed.chosen.shape:
        raise KernelError("moe_combine_add: the experts' outputs, weights and choices do not fit the residual stream")
    if every is not None:
        _check(every, "every", routed.dtype)
        if every.shape != residual.shape:
            raise KernelError("moe_combine_add: `every` must have the residual stream's shape")
    if every_gate is not None:
        _check(every_gate, "every_gate", torch.float32)
        if every is None or every_gate.numel() != tokens:
            raise KernelError("moe_combine_add: the gate needs `every` and one element per token")
    code = _lib().lb_moe_combine_add(_ptr(routed.pair_out), _ptr(routed.weights), _ptr(routed.chosen), c_int(routed.experts), _ptr(every), _ptr(every_gate), c_int(1),
                                     _ptr(residual), c_int(tokens), c_int(top), c_int(width), c_int(dtype_code(routed.dtype)), _stream())
    _done(code, "moe_combine_add")


# ----------------------------------------------------------------------- branch norms
def branch_norms_accumulate(residual: torch.Tensor, terms: list, eps: float) -> None:
    """``residual += sum_i scale_i * rms_norm(tensor_i) * weight_i`` on the 32-bit residual stream, all in 32-bit; ``terms`` holds
    one or two ``(tensor, weight, scale)``: the outputs of mixers side by side, each normed over the model's width."""
    _check(residual, "residual", torch.float32)
    if not 1 <= len(terms) <= 2:
        raise KernelError("branch_norms_accumulate: one or two terms")
    first = terms[0][0]
    for tensor, weight, _ in terms:
        _check(tensor, "branch output", first.dtype)
        _check(weight, "branch weight", torch.float32)
        if tensor.shape != residual.shape or weight.numel() != residual.shape[1]:
            raise KernelError("branch_norms_accumulate: a branch's output or weight does not fit the residual stream")
    second = terms[1] if len(terms) == 2 else (None, None, 0.0)
    code = _lib().lb_branch_norms_accumulate(_ptr(residual), _ptr(first), _ptr(terms[0][1]), c_float(terms[0][2]), _ptr(second[0]), _ptr(second[1]), c_float(second[2]),
                                             c_int(residual.shape[0]), c_int(residual.shape[1]), c_float(eps), c_int(dtype_code(first.dtype)), _stream())
    _done(code, "branch_norms_accumulate")


# ---------------------------------------------------------------------- linear attention
def linear_attention(proj: torch.Tensor, matrix_state: torch.Tensor, *, num_heads: int, key_dim: int, value_dim: int, decay_logits: torch.Tensor | None = None,
                     decay_bias: torch.Tensor | None = None, fixed_decay: torch.Tensor | None = None, tau: float = 1.0, query_scale: float = 1.0,
                     key_scale: float = 1.0, norm_weight: torch.Tensor, norm_eps: float, gate_offset: int, gate_activation: str = "silu",
                     segment_start: torch.Tensor, segment_length: torch.Tensor, segment_slot: torch.Tensor, segments: int, status: torch.Tensor,
                     chunk_plan: dict | None = None) -> torch.Tensor:
    """Linear attention ``S_t = diag(a_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t`` over the step's portions, from each request's state
    slot and back into it, then the per-head RMS norm of the read-out (times ``norm_weight``) times the gate.

    ``proj`` ``[tokens, >= gate_offset + heads * value_dim]`` holds per token q (``heads x key_dim``), k (the same), v
    (``heads x value_dim``) and, from column ``gate_offset`` on, the gate's logits.  The decay is ``fixed_decay`` (32-bit, one per
    head) or ``sigmoid(decay_logits + decay_bias) ** (1 / tau)`` (``decay_logits`` ``[tokens, heads * key_dim]`` in the
    activation type, the bias 32-bit).  ``matrix_state`` is ``[slots, heads, key_dim, value_dim]`` in 32-bit.  Returns
    ``[tokens, heads * value_dim]`` in the activation type.  ``chunk_plan`` (see :func:`gated_delta_chunk_plan`) lets long portions run as
    chunks side by side, as the gated delta rule's do: the recurrence is linear in the state, and the chunks' further columns carry
    their decays' products."""
    _check(proj, "proj")
    _check(matrix_state, "matrix_state", torch.float32)
    _check(norm_weight, "norm_weight", torch.float32)
    for name, tensor in (("segment_start", segment_start), ("segment_length", segment_length), ("segment_slot", segment_slot)):
        _check(tensor, name, torch.int32)
    if gate_activation not in ("sigmoid", "silu"):
        raise KernelError(f"linear_attention: unknown gate activation {gate_activation!r}")
    tokens = proj.shape[0]
    if key_dim < 1 or key_dim > 256 or value_dim < 1 or num_heads < 1:
        raise KernelError(f"linear_attention: {num_heads} heads with key size {key_dim} (at most 256) and value size {value_dim} are not supported")
    if gate_offset < 2 * num_heads * key_dim + num_heads * value_dim or proj.shape[1] < gate_offset + num_heads * value_dim:
        raise KernelError("linear_attention: proj is too narrow for the head counts")
    num_slots = matrix_state.shape[0]
    if matrix_state.shape != (num_slots, num_heads, key_dim, value_dim) or norm_weight.numel() != value_dim:
        raise KernelError("linear_attention: matrix_state must be [slots, heads, key_dim, value_dim] and norm_weight [value_dim]")
    if (decay_logits is None) == (fixed_decay is None):
        raise KernelError("linear_attention: the decay is either fixed per head or made from logits")
    if decay_logits is not None:
        if not decay_logits.is_cuda or decay_logits.dim() != 2 or decay_logits.stride(1) != 1 or decay_logits.dtype != proj.dtype or decay_logits.shape[0] != tokens \
                or decay_logits.shape[1] < num_heads * key_dim:
            raise KernelError("linear_attention: decay_logits must be [tokens, >= heads * key_dim] of proj's type with unit column stride")
        if decay_bias is not None:
            _check(decay_bias, "decay_bias", torch.float32)
            if decay_bias.numel() != num_heads * key_dim:
                raise KernelError("linear_attention: decay_bias must have heads * key_dim elements")
        if tau <= 0.0:
            raise KernelError("linear_attention: tau must be positive")
    else:
        _check(fixed_decay, "fixed_decay", torch.float32)
        if fixed_decay.numel() != num_heads:
            raise KernelError("linear_attention: fixed_decay must have one element per head")
    device = proj.device
    q = torch.empty(tokens, num_heads, key_dim, dtype=torch.float32, device=device)
    k = torch.empty_like(q)
    decay = torch.empty_like(q)
    v = torch.empty(tokens, num_heads, value_dim, dtype=torch.float32, device=device)
    lib = _lib()
    code = lib.lb_linear_attention_prepare(_ptr(proj), c_int(proj.shape[1]), _ptr(decay_logits), c_int(decay_logits.stride(0) if decay_logits is not None else 0),
                                           _ptr(decay_bias), _ptr(fixed_decay), c_float(1.0 / tau), c_float(query_scale), c_float(key_scale), _ptr(q), _ptr(k), _ptr(v),
                                           _ptr(decay), c_int(tokens), c_int(num_heads), c_int(key_dim), c_int(value_dim), c_int(dtype_code(proj.dtype)), _stream())
    _done(code, "linear_attention_prepare")
    read_out = torch.empty(tokens, num_heads, value_dim, dtype=torch.float32, device=device)
    # the scan of the gated delta rule without its correction (no beta), long portions in chunks where that pays
    direct_list, num_direct = None, segments
    if chunk_plan is not None and chunk_plan["num_chunks"] > 0 and gated_delta_chunks_pay(key_dim, value_dim):
        num_chunks, num_long = chunk_plan["num_chunks"], chunk_plan["num_long"]
        wide_dim = value_dim + key_dim
        wide = torch.empty(tokens, num_heads, wide_dim, dtype=torch.float32, device=device)
        chunk_state = torch.empty(num_chunks, num_heads, key_dim, wide_dim, dtype=torch.float32, device=device)
        chunk_in = torch.empty(num_chunks, num_heads, key_dim, value_dim, dtype=torch.float32, device=device)
        _done(lib.lb_gdr_chunk_init(_ptr(chunk_state), c_int(num_chunks), c_int(num_heads), c_int(key_dim), c_int(value_dim), _stream()), "gdr_chunk_init")
        code = lib.lb_gdr_scan(_ptr(q), _ptr(k), _ptr(decay), _ptr(v), _ptr(None), _ptr(chunk_state), _ptr(wide), _ptr(chunk_plan["chunk_start"]),
                               _ptr(chunk_plan["chunk_length"]), _ptr(chunk_plan["chunk_slot"]), c_int(num_chunks), c_int(num_heads), c_int(num_heads),
                               c_int(key_dim), c_int(wide_dim), c_int(num_chunks), _ptr(status), _stream(), _ptr(None), c_int(value_dim))
        _done(code, "linear_attention_scan (chunks)")
        code = lib.lb_gdr_chunk_finish(_ptr(chunk_state), _ptr(chunk_in), _ptr(matrix_state), _ptr(wide), _ptr(read_out), _ptr(chunk_plan["long_table"]),
                                       c_int(num_long), _ptr(segment_slot), _ptr(chunk_plan["chunk_start"]), _ptr(chunk_plan["chunk_length"]), c_int(num_chunks),
                                       c_int(chunk_plan.get("chunk_tokens", GDR_CHUNK_TOKENS)), c_int(num_heads), c_int(key_dim), c_int(value_dim), c_int(num_slots),
                                       _stream())
        _done(code, "gdr_chunk_finish", 2)
        direct_list, num_direct = chunk_plan["direct"], chunk_plan["num_direct"]
    if num_direct > 0:
        code = lib.lb_gdr_scan(_ptr(q), _ptr(k), _ptr(decay), _ptr(v), _ptr(None), _ptr(matrix_state), _ptr(read_out), _ptr(segment_start), _ptr(segment_length),
                               _ptr(segment_slot), c_int(num_direct), c_int(num_heads), c_int(num_heads), c_int(key_dim), c_int(value_dim), c_int(num_slots),
                               _ptr(status), _stream(), _ptr(direct_list), c_int(value_dim))
        _done(code, "linear_attention_scan")
    out = torch.empty(tokens, num_heads * value_dim, dtype=proj.dtype, device=device)
    code = lib.lb_gdr_output(_ptr(read_out), _ptr(proj), c_int(proj.shape[1]), c_int(gate_offset), _ptr(norm_weight), _ptr(out), c_int(tokens),
                             c_int(num_heads), c_int(value_dim), c_float(norm_eps), c_int(dtype_code(proj.dtype)), _stream(), c_int(1 if gate_activation == "silu" else 0))
    _done(code, "linear_attention_output")
    return out


# ------------------------------------------------------------- pooled window attention
def _check_pooled(pages: torch.Tensor, block_table: torch.Tensor, groups: int, head_dim: int, value_dim: int, what: str) -> tuple[int, int, int]:
    _check(pages, f"{what} pages")
    _check(block_table, f"{what} block table", torch.int32)
    count, rows = pages.shape[0], pages.shape[1]
    if pages.shape != (count, rows, groups, head_dim + value_dim) or block_table.dim() != 2:
        raise KernelError(f"pooled attention: the {what} pages must be [pages, rows, groups, head_dim + value_dim] (a row holds key and value)")
    return count, rows, block_table.shape[1]


def pooled_rewrite(qkv: torch.Tensor, q_out: torch.Tensor, pages: torch.Tensor, *, qk_freq: torch.Tensor | None, rotary_dim: int,
                   value_freq: torch.Tensor | None, interleaved: bool = False, positions: torch.Tensor, token_segment: torch.Tensor, block_table: torch.Tensor,
                   num_heads: int, num_groups: int, head_dim: int, value_dim: int, write_kv: bool, status: torch.Tensor) -> None:
    """Splits the rows of ``qkv`` (q ``heads x head_dim`` | k ``groups x head_dim`` | v ``groups x value_dim``; a column slice of a wider
    product will do) into heads, rotates the first ``rotary_dim`` channels of q and k by the token's position (``qk_freq``: a 32-bit
    frequency per pair) and, with ``value_freq`` (``value_dim / 2`` frequencies), all channels of v; q goes to ``q_out``, k and v
    into the token's page row (``pages`` ``[pages, page_size, groups, head_dim + value_dim]``).  Angles, sines and cosines in 32-bit,
    one rounding."""
    if not qkv.is_cuda or qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("pooled_rewrite: qkv must be a [tokens, .] CUDA tensor with unit column stride")
    _check(q_out, "q_out", qkv.dtype)
    count, page_size, max_blocks = _check_pooled(pages, block_table, num_groups, head_dim, value_dim, "token")
    if pages.dtype != qkv.dtype:
        raise KernelError("pooled_rewrite: the pages must have qkv's type")
    tokens = qkv.shape[0]
    if qkv.shape[1] < num_heads * head_dim + num_groups * (head_dim + value_dim) or q_out.shape != (tokens, num_heads * head_dim):
        raise KernelError("pooled_rewrite: qkv or q_out does not fit the head counts")
    if rotary_dim:
        _check(qk_freq, "qk_freq", torch.float32)
        if rotary_dim % 2 or rotary_dim > head_dim or qk_freq.numel() != rotary_dim // 2:
            raise KernelError("pooled_rewrite: rotary_dim must be even, at most head_dim, with one frequency per pair")
    if value_freq is not None:
        _check(value_freq, "value_freq", torch.float32)
        if value_dim % 2 or value_freq.numel() != value_dim // 2:
            raise KernelError("pooled_rewrite: rotated values need an even value_dim and one frequency per pair")
    for name, tensor in (("positions", positions), ("token_segment", token_segment)):
        _check(tensor, name, torch.int32)
    code = _lib().lb_pooled_rewrite(_ptr(qkv), c_int(qkv.stride(0)), _ptr(q_out), _ptr(pages), _ptr(qk_freq if rotary_dim else None), c_int(rotary_dim),
                                    c_int(1 if interleaved else 0), _ptr(value_freq), c_int(1 if interleaved else 0), _ptr(positions), _ptr(token_segment),
                                    _ptr(block_table), c_int(tokens), c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(value_dim), c_int(page_size),
                                    c_int(count), c_int(max_blocks), c_int(1 if write_kv else 0), c_int(dtype_code(qkv.dtype)), _ptr(status), _stream())
    _done(code, "pooled_rewrite")


def pooled_means(pages: torch.Tensor, pool_pages: torch.Tensor, *, segment_length: torch.Tensor, segment_context: torch.Tensor, block_table: torch.Tensor,
                 pool_table: torch.Tensor, segments: int, max_length: int, num_groups: int, head_dim: int, value_dim: int, pool: int, status: torch.Tensor) -> None:
    """For every block of ``pool`` positions whose last position this step wrote: the mean of its keys and of its values as the
    token pages hold them (32-bit sums in the order of the positions, one rounding) into row ``b % rows`` of the request's pooled
    page ``pool_table[b / rows]``.  ``max_length``: the step's longest portion."""
    count, page_size, max_blocks = _check_pooled(pages, block_table, num_groups, head_dim, value_dim, "token")
    pool_count, pool_rows, pool_blocks = _check_pooled(pool_pages, pool_table, num_groups, head_dim, value_dim, "pooled")
    if pool_pages.dtype != pages.dtype or pool < 1:
        raise KernelError("pooled_means: pages of one type and a positive block size")
    for name, tensor in (("segment_length", segment_length), ("segment_context", segment_context)):
        _check(tensor, name, torch.int32)
    code = _lib().lb_pooled_means(_ptr(pages), _ptr(pool_pages), _ptr(segment_length), _ptr(segment_context), _ptr(block_table),
                                  _ptr(pool_table), c_int(segments), c_int(max_length), c_int(num_groups), c_int(head_dim), c_int(value_dim), c_int(page_size),
                                  c_int(count), c_int(max_blocks), c_int(pool_rows), c_int(pool_count), c_int(pool_blocks), c_int(pool), c_int(dtype_code(pages.dtype)),
                                  _ptr(status), _stream())
    _done(code, "pooled_means")


POOLED_MMA_HEADS = 4  # query heads of one K/V head that a CTA of the tensor-core kernel takes at most


def pooled_attention_tiling(num_heads: int, num_groups: int) -> tuple[int, int]:
    """``(query heads of a K/V head per CTA, tokens per tile)`` of the tensor-core kernel: a CTA's eight warps are one head's 16 tokens each."""
    head_block = min(num_heads // num_groups, POOLED_MMA_HEADS)
    return head_block, 16 * (8 // head_block)


def pooled_attention_shares(num_tiles: int, num_heads: int, num_groups: int, sms: int | None = None) -> int:
    """How many CTAs share out a tile's rows of the cache: one where the launch has four CTAs a multiprocessor anyway, else enough
    for that many, 16 at most.  It depends on the launch's shape alone (a recorded step keeps it)."""
    head_block, _ = pooled_attention_tiling(num_heads, num_groups)
    ctas = num_tiles * num_groups * -(-(num_heads // num_groups) // head_block)
    sms = sms or sm_count()
    return 1 if ctas >= 4 * sms else max(1, min(16, -(-4 * sms // ctas)))


POOLED_SINGLE_HEADS = 16  # query heads of one K/V head that a CTA of the single-token kernel takes at most


def pooled_single_shares(num_singles: int, num_heads: int, num_groups: int, sms: int | None = None) -> int:
    """As :func:`pooled_attention_shares`, for the kernel of tokens that attend alone."""
    ctas = num_singles * num_groups * -(-(num_heads // num_groups) // POOLED_SINGLE_HEADS)
    sms = sms or sm_count()
    return 1 if ctas >= 4 * sms else max(1, min(16, -(-4 * sms // ctas)))


def pooled_attention_supported(dtype: torch.dtype, head_dim: int, value_dim: int) -> bool:
    """Whether the tensor-core kernel takes these sizes (bfloat16, heads of multiples of 16 up to 128 channels)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and value_dim % 16 == 0 and 16 <= head_dim <= 128 and 16 <= value_dim <= 128


def _pooled_arguments(q, pages, pool_pages, out, positions, token_segment, block_table, pool_table, num_heads, num_groups, head_dim, value_dim, head_bias,
                      window, pool, value_freq, what):
    _check(q, "q")
    _check(out, "out", q.dtype)
    count, page_size, max_blocks = _check_pooled(pages, block_table, num_groups, head_dim, value_dim, "token")
    if pool:
        pool_count, pool_rows, pool_blocks = _check_pooled(pool_pages, pool_table, num_groups, head_dim, value_dim, "pooled")
    else:
        pool_count, pool_rows, pool_blocks = 0, 1, 0
    tokens = q.shape[0]
    if q.shape != (tokens, num_heads * head_dim) or out.shape != (tokens, num_heads * value_dim) or pages.dtype != q.dtype or num_heads % num_groups:
        raise KernelError(f"{what}: q, out or the pages do not fit the head counts")
    if head_bias is not None:
        _check(head_bias, "head_bias", torch.float32)
        if head_bias.numel() != num_heads:
            raise KernelError(f"{what}: one bias per head")
    if value_freq is not None:
        _check(value_freq, "value_freq", torch.float32)
        if value_dim % 2 or value_freq.numel() != value_dim // 2:
            raise KernelError(f"{what}: rotated values need an even value_dim and one frequency per pair")
    if window < 1 or pool < 0 or value_dim > 512:
        raise KernelError(f"{what}: a positive window, a block size that is not negative and values of at most 512 channels")
    for name, tensor in (("positions", positions), ("token_segment", token_segment)):
        _check(tensor, name, torch.int32)
    return tokens, (count, page_size, max_blocks), (pool_count, pool_rows, pool_blocks)


def pooled_attention_plain(q: torch.Tensor, pages: torch.Tensor, pool_pages: torch.Tensor | None, out: torch.Tensor, *, positions: torch.Tensor,
                           token_segment: torch.Tensor, block_table: torch.Tensor, pool_table: torch.Tensor | None, num_heads: int, num_groups: int,
                           head_dim: int, value_dim: int, scale: float, softcap: float, head_bias: torch.Tensor | None, window: int, pool: int,
                           value_freq: torch.Tensor | None, interleaved: bool = False, status: torch.Tensor) -> None:
    """Sigmoid-weighted attention of every token over the positions of its window and the pooled blocks wholly before it:
    ``out[t, h] = sum_x sigmoid(cap(q . k_x * scale) + head_bias[h]) v_x`` (no normalisation), blocks first, then positions
    upwards, all in 32-bit; with ``value_freq`` the sum is turned back by the token's position.  One block per token and head."""
    tokens, (count, page_size, max_blocks), (pool_count, pool_rows, pool_blocks) = _pooled_arguments(
        q, pages, pool_pages, out, positions, token_segment, block_table, pool_table, num_heads, num_groups, head_dim, value_dim, head_bias, window, pool,
        value_freq, "pooled_attention_plain")
    code = _lib().lb_pooled_attention_plain(_ptr(q), _ptr(pages), _ptr(pool_pages if pool else None), _ptr(out),
                                            _ptr(positions), _ptr(token_segment), _ptr(block_table), _ptr(pool_table if pool else None), c_int(tokens), c_int(num_heads),
                                            c_int(num_groups), c_int(head_dim), c_int(value_dim), c_int(page_size), c_int(count), c_int(max_blocks), c_int(pool_rows),
                                            c_int(pool_count), c_int(pool_blocks), c_float(scale), c_float(softcap), _ptr(head_bias), c_int(window), c_int(pool),
                                            _ptr(value_freq), c_int(1 if interleaved else 0), c_int(dtype_code(q.dtype)), _ptr(status), _stream())
    _done(code, "pooled_attention_plain")


def pooled_attention(q: torch.Tensor, pages: torch.Tensor, pool_pages: torch.Tensor | None, out: torch.Tensor, *, tiles: torch.Tensor, num_tiles: int, shares: int | None = None,
                     positions: torch.Tensor, token_segment: torch.Tensor, block_table: torch.Tensor, pool_table: torch.Tensor | None, num_heads: int,
                     num_groups: int, head_dim: int, value_dim: int, scale: float, softcap: float, head_bias: torch.Tensor | None, window: int, pool: int,
                     value_freq: torch.Tensor | None, interleaved: bool = False, status: torch.Tensor) -> None:
    """The same attention on the tensor cores (bfloat16; see :func:`pooled_attention_supported`).  ``tiles``: int32 ``(first row, count)``
    per tile of consecutive tokens of one portion, at most :func:`pooled_attention_tiling`'s tokens each.  Weights in 32-bit (the cap's
    tanh and the sigmoid through the fast exponential and reciprocal), rounded to bfloat16 for the product with the values; sums in 32-bit.  Launches
    of few CTAs share out every tile's rows of the cache over several CTAs (:func:`pooled_attention_shares`), whose 32-bit sums a second
    kernel adds in order."""
    tokens, (count, page_size, max_blocks), (pool_count, pool_rows, pool_blocks) = _pooled_arguments(
        q, pages, pool_pages, out, positions, token_segment, block_table, pool_table, num_heads, num_groups, head_dim, value_dim, head_bias, window, pool,
        value_freq, "pooled_attention")
    if not pooled_attention_supported(q.dtype, head_dim, value_dim):
        raise KernelError("pooled_attention: the tensor-core kernel takes bfloat16 and heads of multiples of 16 up to 128 channels")
    _check(tiles, "tiles", torch.int32)
    if tiles.numel() < 2 * num_tiles:
        raise KernelError("pooled_attention: fewer tile records than tiles")
    head_block, _ = pooled_attention_tiling(num_heads, num_groups)
    if shares is None:
        shares = pooled_attention_shares(num_tiles, num_heads, num_groups)
    if not 1 <= shares <= 64:
        raise KernelError("pooled_attention: 1 to 64 shares")
    partial = torch.empty(shares, tokens, num_heads * value_dim, dtype=torch.float32, device=q.device) if shares > 1 else None
    code = _lib().lb_pooled_attention_mma(_ptr(q), _ptr(pages), _ptr(pool_pages if pool else None), _ptr(out), _ptr(tiles), c_int(num_tiles), _ptr(positions),
                                          _ptr(token_segment), _ptr(block_table), _ptr(pool_table if pool else None), c_int(num_heads), c_int(num_groups),
                                          c_int(head_dim), c_int(value_dim), c_int(page_size), c_int(count), c_int(max_blocks), c_int(pool_rows), c_int(pool_count),
                                          c_int(pool_blocks), c_int(head_block), c_float(scale), c_float(softcap), _ptr(head_bias), c_int(window), c_int(pool),
                                          _ptr(value_freq), c_int(1 if interleaved else 0), _ptr(status), _stream(), c_int(shares), _ptr(partial), c_int(tokens))
    _done(code, "pooled_attention", 2 if shares > 1 else 1)


def pooled_attention_single(q: torch.Tensor, pages: torch.Tensor, pool_pages: torch.Tensor | None, out: torch.Tensor, *, singles: torch.Tensor, num_singles: int,
                            shares: int | None = None, positions: torch.Tensor, token_segment: torch.Tensor, block_table: torch.Tensor,
                            pool_table: torch.Tensor | None, num_heads: int, num_groups: int, head_dim: int, value_dim: int, scale: float, softcap: float,
                            head_bias: torch.Tensor | None, window: int, pool: int, value_freq: torch.Tensor | None, interleaved: bool = False,
                            status: torch.Tensor) -> None:
    """The same attention for tokens that attend alone (``singles``: their rows, int32), on the tensor cores with the products turned
    round: 16 rows of the cache are a product's rows, up to 16 query heads of a K/V head its columns.  Same sizes, arithmetic and
    order of the rows as :func:`pooled_attention`; other rows of ``out`` are left alone."""
    tokens, (count, page_size, max_blocks), (pool_count, pool_rows, pool_blocks) = _pooled_arguments(
        q, pages, pool_pages, out, positions, token_segment, block_table, pool_table, num_heads, num_groups, head_dim, value_dim, head_bias, window, pool,
        value_freq, "pooled_attention_single")
    if not pooled_attention_supported(q.dtype, head_dim, value_dim):
        raise KernelError("pooled_attention_single: the tensor-core kernel takes bfloat16 and heads of multiples of 16 up to 128 channels")
    _check(singles, "singles", torch.int32)
    if singles.numel() < num_singles:
        raise KernelError("pooled_attention_single: fewer rows listed than announced")
    if shares is None:
        shares = pooled_single_shares(num_singles, num_heads, num_groups)
    if not 1 <= shares <= 64:
        raise KernelError("pooled_attention_single: 1 to 64 shares")
    partial = torch.empty(shares, tokens, num_heads * value_dim, dtype=torch.float32, device=q.device) if shares > 1 else None
    code = _lib().lb_pooled_attention_single(_ptr(q), _ptr(pages), _ptr(pool_pages if pool else None), _ptr(out), _ptr(singles), c_int(num_singles), _ptr(positions),
                                             _ptr(token_segment), _ptr(block_table), _ptr(pool_table if pool else None), c_int(num_heads), c_int(num_groups),
                                             c_int(head_dim), c_int(value_dim), c_int(page_size), c_int(count), c_int(max_blocks), c_int(pool_rows), c_int(pool_count),
                                             c_int(pool_blocks), c_float(scale), c_float(softcap), _ptr(head_bias), c_int(window), c_int(pool),
                                             _ptr(value_freq), c_int(1 if interleaved else 0), _ptr(status), _stream(), c_int(shares), _ptr(partial), c_int(tokens))
    _done(code, "pooled_attention_single", 2 if shares > 1 else 1)


# ------------------------------------------------------------------------------ sampling
SAMPLE_PARAM_WORDS = 27


def sample(logits: torch.Tensor, work: torch.Tensor, counts: torch.Tensor | None, params: torch.Tensor, out_tokens: torch.Tensor) -> None:
    _check(logits, "logits", torch.float32)
    _check(work, "work", torch.float32)
    _check(params, "params", torch.int32)
    _check(out_tokens, "out_tokens", torch.int32)
    rows, vocab = logits.shape
    if work.numel() < rows * vocab or params.shape != (rows, SAMPLE_PARAM_WORDS) or out_tokens.numel() < rows:
        raise KernelError("sample: work, params or out_tokens are too small for the logits")
    if counts is not None:
        _check(counts, "counts", torch.int32)
        if counts.shape[1] != vocab:
            raise KernelError("sample: counts must be [slots, vocab]")
    lib = _lib()
    if lib.lb_sample_params_size() != 4 * SAMPLE_PARAM_WORDS:
        raise KernelError("sample: parameter record sizes of the library and the bindings differ")
    code = lib.lb_sample(_ptr(logits), _ptr(work), _ptr(counts), _ptr(params), _ptr(out_tokens), c_int(rows), c_int(vocab), _stream())
    _done(code, "sample")


def argmax(logits: torch.Tensor, out_tokens: torch.Tensor) -> None:
    _check(logits, "logits", torch.float32)
    _check(out_tokens, "out_tokens", torch.int32)
    rows, vocab = logits.shape
    if out_tokens.numel() < rows:
        raise KernelError("argmax: out_tokens is too small")
    if vocab >= 8192 and rows <= 256:
        # Few long rows: spread each over many blocks.
        chunks = max(2, min(64, vocab // 2048))
        scratch = torch.empty(2 * rows * chunks, dtype=torch.float32, device=logits.device)
        code = _lib().lb_argmax_chunked(_ptr(logits), _ptr(scratch), _ptr(out_tokens), c_int(rows), c_int(vocab), c_int(chunks), _stream())
        _done(code, "argmax", 2)
        return
    code = _lib().lb_argmax(_ptr(logits), _ptr(out_tokens), c_int(rows), c_int(vocab), _stream())
    _done(code, "argmax")


def update_counts(counts: torch.Tensor, slots: torch.Tensor, add: torch.Tensor, remove: torch.Tensor) -> None:
    _check(counts, "counts", torch.int32)
    for name, tensor in (("slots", slots), ("add", add), ("remove", remove)):
        _check(tensor, name, torch.int32)
    rows = slots.numel()
    if add.numel() != rows or remove.numel() != rows:
        raise KernelError("update_counts: slots, add and remove differ in length")
    code = _lib().lb_update_counts(_ptr(counts), _ptr(slots), _ptr(add), _ptr(remove), c_int(rows), c_int(counts.shape[1]), _stream())
    _done(code, "update_counts")


# --------------------------------------------------------------------------------- linear
def configure_matmul_precision() -> None:
    """Makes library float32 products true 32-bit (no TF32, no reduced-precision reductions)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.set_float32_matmul_precision("highest")


_SKINNY_EPILOGUES = {"store": 0, "store_float": 1, "residual_add": 2, "gated": 3, "short_conv": 4}
SKINNY_MAX_TOKENS = 16


def skinny_supported(x: torch.Tensor, rows: int) -> bool:
    """Whether the weight-streaming kernel takes this product: bfloat16, 1..16 tokens, an input width
    that is a multiple of 32 and a multiple of 8 output rows."""
    return (
        x.dtype == torch.bfloat16
        and x.dim() == 2
        and 1 <= x.shape[0] <= SKINNY_MAX_TOKENS
        and x.shape[1] % 32 == 0
        and x.shape[1] >= 32
        and rows % 8 == 0
        and rows > 0
    )


def _skinny(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n: int, epilogue: str, activation: str = "identity", conv: dict | None = None,
            prefetch: bool = True, limit: float = 0.0, bias: torch.Tensor | None = None) -> None:
    """``prefetch``: the kernel asks for its weights towards L2 before it waits for the kernel before it; off where
    that kernel does not let it start early (see :func:`successor_starts_early`)."""
    conv = conv or {}
    code = _lib().lb_gemm_skinny(
        _ptr(x), _ptr(weight), _ptr(out), c_int(x.shape[0]), c_int(x.shape[1]), c_int(n), c_int(_SKINNY_EPILOGUES[epilogue]),
        c_int(_ACTIVATIONS[activation]), _ptr(conv.get("state")), _ptr(conv.get("weight")), _ptr(conv.get("bias")), _ptr(conv.get("token_segment")),
        _ptr(conv.get("segment_start")), _ptr(conv.get("segment_length")), _ptr(conv.get("segment_slot")), c_int(conv.get("segments", 0)),
        c_int(conv.get("taps", 0)), c_int(conv.get("num_slots", 0)), c_int(1 if prefetch else 0), _ptr(conv.get("status")), _stream(), c_float(limit),
        _ptr(bias))
    _done(code, f"gemm_skinny[{epilogue}]")


# Products of more than 16 tokens run on the tcgen05 kernel when this is on (LALAMO_B200_TCGEN05=0
# sends them to the library instead).
USE_TCGEN05 = os.environ.get("LALAMO_B200_TCGEN05", "1") != "0"
# Prefill attention with head size 64 runs on the tcgen05 kernel when this is on
# (LALAMO_B200_TCGEN05_ATTENTION=0 keeps it on the mma.sync kernel).
USE_TCGEN05_ATTENTION = os.environ.get("LALAMO_B200_TCGEN05_ATTENTION", "1") != "0"
# With at most 16 tokens, products of at least this many rows of W fill the GPU with 128-row tiles and
# stream faster through the TMA pipeline than through the register-direct kernel.
TCGEN05_MIN_ROWS_FEW_TOKENS = 16384
_TC_EPILOGUES = {"store": 0, "store_float": 1, "residual_add": 2, "gated": 4}
_tc_scratch: dict[int, torch.Tensor] = {}
_tc_retired: list[torch.Tensor] = []  # outgrown scratch buffers, kept: a recorded graph may hold their address
# Products cut into K slices hand their partial sums to the next norm instead of summing them in a launch of their own
# (LALAMO_B200_DEFER_SLICE_SUMS=0 sums at once).
DEFER_SLICE_SUMS = os.environ.get("LALAMO_B200_DEFER_SLICE_SUMS", "1") != "0"


def tcgen05_supported(x: torch.Tensor, rows: int) -> bool:
    """Whether the tcgen05 kernel takes this product: bfloat16, rows of 16-byte multiples."""
    return x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] >= 1 and x.shape[1] % 8 == 0 and x.shape[1] >= 8 and rows >= 1


def tcgen05_slices(tokens: int, rows: int, width: int, sms: int | None = None) -> int:
    """K slices for a product whose tiles alone would leave most of the multiprocessors idle."""
    blocks = -(-width // 64)
    sms = sms or sm_count()
    if tokens > 128:
        # The walking kernel with tiles of 128 rows x 256 tokens: slices until the tiles fill the SMs, of at least 16
        # blocks each.  Measured against one slice: 1024 x 4608 at 2,048 tokens 22.6 against 28.5 us, at 512 tokens 14.0
        # against 25.5; 2048 x 8192 at 512 tokens 21.5 against 43.2, at 1,024 tokens 33.6 against 46.7; 1024 x 1024 at
        # 2,048 tokens (16 blocks in all) 12.5 against 9.8, hence the floor.
        tiles = -(-rows // 128) * -(-tokens // 256)
        return max(1, min(sms // tiles, blocks // 16, 12))
    tile = 32 if tokens <= 32 else 64 if tokens <= 64 else 128
    ctas = -(-rows // 128) * -(-tokens // tile)
    if ctas >= 96 or blocks < 8:
        return 1
    # more than a dozen slices cost more in partial sums than they gain in CTAs (1024 x 4608 at 64 tokens: 8.7 us with 12,
    # 9.4 with 18)
    return max(1, min(-(-sms // ctas), blocks // 4, 12))


def _settled_slices(slices: int, width: int) -> int:
    """The number of K slices the kernel makes of ``slices`` asked for (whole blocks of 64 columns each)."""
    blocks = -(-width // 64)
    slices = max(1, min(slices, blocks))
    per_slice = -(-blocks // slices)
    return -(-blocks // per_slice)


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, epilogue: str = "store", residual: torch.Tensor | None = None,
                   slices: int | None = None, activation: str = "identity", status: torch.Tensor | None = None,
                   defer_sum: bool = False, limit: float = 0.0) -> torch.Tensor | SlicedSum:
    """``x @ weight.T`` on the tcgen05 tensor cores.  ``epilogue``: ``"store"`` (bfloat16),
    ``"store_float"``, ``"residual_add"`` (into ``residual``, float32, which is returned) or ``"gated"``
    (``weight`` is ``[up ; gate]``, the result ``up * activation(gate)`` of half as many columns).
    ``status``: the int32 word in which the kernel reports a wait that gave up.  ``defer_sum``: if the
    product is cut into K slices, return them as a :class:`SlicedSum` (nothing is stored or added) for a
    consumer that adds them itself."""
    if status is not None:
        _check(status, "status", torch.int32)
    _check(x, "x", torch.bfloat16)
    _check(weight, "weight", torch.bfloat16)
    tokens, width = x.shape
    rows = weight.shape[0]
    if weight.shape[1] != width or not tcgen05_supported(x, rows):
        raise KernelError(f"linear_tcgen05: a [{tokens}, {width}] x [{rows}, {weight.shape[1]}] product is not supported (widths must agree and be multiples of 8)")
    if epilogue == "residual_add":
        if residual is None:
            raise KernelError("linear_tcgen05: residual_add needs the residual stream")
        _check(residual, "residual", torch.float32)
        if residual.shape != (tokens, rows):
            raise KernelError("linear_tcgen05: residual must be [tokens, rows]")
        out = residual
    elif epilogue == "gated":
        if rows % 2 or activation not in _ACTIVATIONS:
            raise KernelError("linear_tcgen05: gated needs an even number of rows and a known activation")
        out = torch.empty(tokens, rows // 2, dtype=torch.bfloat16, device=x.device)
        slices = 1
    else:
        out = torch.empty(tokens, rows, dtype=torch.float32 if epilogue == "store_float" else torch.bfloat16, device=x.device)
    slices = tcgen05_slices(tokens, rows, width) if slices is None else slices
    slices = 1 if epilogue == "gated" else _settled_slices(slices, width)
    deferred = defer_sum and slices > 1 and epilogue in ("store", "residual_add")
    scratch = None
    if deferred:
        scratch = torch.empty(slices, tokens, rows, dtype=torch.float32, device=x.device)
    elif slices > 1:
        needed = slices * tokens * rows
        index = x.device.index if x.device.index is not None else torch.cuda.current_device()
        if index not in _tc_scratch or _tc_scratch[index].numel() < needed:
            if index in _tc_scratch:
                _tc_retired.append(_tc_scratch[index])  # recorded graphs may still write there
            _tc_scratch[index] = torch.empty(max(needed, 1 << 22), dtype=torch.float32, device=x.device)
        scratch = _tc_scratch[index]
    code = _lib().lb_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), _ptr(scratch), c_longlong(scratch.numel() if scratch is not None else 0),
                                  c_int(tokens), c_int(width), c_int(rows), c_int(_TC_EPILOGUES[epilogue]), c_int(_ACTIVATIONS[activation]), c_int(slices),
                                  c_int(1 if deferred else 0), _ptr(status), _stream(), c_float(limit))
    if code == -5:
        raise KernelError("linear_tcgen05: the driver gave no tensor map (cuTensorMapEncodeTiled)")
    _done(code, "gemm_tcgen05", 2 if slices > 1 and not deferred else 1)
    if deferred:
        return SlicedSum(scratch, torch.bfloat16)
    return out


def tcgen05_wait_probe(status: torch.Tensor, nanoseconds: int = 1_000_000) -> None:
    """Lets the tcgen05 kernels' bounded barrier wait run out on a barrier that nothing completes
    (after ``nanoseconds``, at most 0.1 s) and report it in ``status``, as a product would whose
    copy or arrival got lost."""
    _check(status, "status", torch.int32)
    _done(_lib().lb_tcgen05_wait_probe(_ptr(status), c_longlong(nanoseconds), _stream()), "tcgen05_wait_probe")


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T`` with 32-bit accumulation; ``out_dtype`` float32 gives 32-bit results from
    bfloat16 operands (the LM head's logits).  Steps of up to 16 tokens go to the weight-streaming
    kernel, everything else to the library."""
    _check(x, "x")
    _check(weight, "weight", x.dtype)
    if x.shape[-1] != weight.shape[1]:
        raise KernelError(f"linear: input width {x.shape[-1]} does not match the weight's {weight.shape[1]}")
    wants_float = out_dtype is not None and out_dtype != x.dtype
    if USE_TCGEN05 and x.shape[0] <= SKINNY_MAX_TOKENS and weight.shape[0] >= TCGEN05_MIN_ROWS_FEW_TOKENS and tcgen05_supported(x, weight.shape[0]):
        return linear_tcgen05(x, weight, "store_float" if wants_float else "store", slices=1, status=status)
    if skinny_supported(x, weight.shape[0]):
        out = torch.empty(x.shape[0], weight.shape[0], dtype=torch.float32 if wants_float else x.dtype, device=x.device)
        _skinny(x, weight, out, weight.shape[0], "store_float" if wants_float else "store")
        return out
    if USE_TCGEN05 and tcgen05_supported(x, weight.shape[0]):
        return linear_tcgen05(x, weight, "store_float" if wants_float else "store", status=status)
    if wants_float:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    return torch.mm(x, weight.t())


def linear_bias_activation(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, activation: str,
                           status: torch.Tensor | None = None) -> torch.Tensor:
    """``act(x @ weight.T + bias)`` in ``x``'s type (the sum and the activation in 32-bit, rounded once).  Steps of up to 16
    tokens compute it in the weight-streaming product's epilogue, other bfloat16 steps in the tcgen05 product's; what neither takes
    (32-bit, widths that are no multiples of 8) runs the product, then one elementwise kernel."""
    _check(x, "x")
    _check(weight, "weight", x.dtype)
    if activation not in ("silu", "gelu", "identity"):
        raise KernelError(f"linear_bias_activation: unknown activation {activation!r}")
    if x.shape[-1] != weight.shape[1]:
        raise KernelError(f"linear_bias_activation: input width {x.shape[-1]} does not match the weight's {weight.shape[1]}")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != weight.shape[0]:
            raise KernelError("linear_bias_activation: bias must have one element per row of the weight")
    if skinny_supported(x, weight.shape[0]):
        out = torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)
        _skinny(x, weight, out, weight.shape[0], "store", activation, bias=bias)
        return out
    if USE_TCGEN05 and tcgen05_supported(x, weight.shape[0]):
        out = torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)
        code = _lib().lb_gemm_tcgen05_bias_activation(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), c_int(x.shape[0]), c_int(x.shape[1]), c_int(weight.shape[0]),
                                                      c_int(_ACTIVATIONS[activation]), _ptr(status), _stream())
        if code == -5:
            raise KernelError("linear_bias_activation: the driver gave no tensor map (cuTensorMapEncodeTiled)")
        _done(code, "gemm_tcgen05_bias_activation")
        return out
    product = linear(x, weight, status=status)
    if isinstance(product, SlicedSum):
        product = product.sum()
    return bias_activation(product, bias, activation)


def gated_linear_starts_successor_early(tokens: int, rows: int, width: int) -> bool:
    """Whether the kernel :func:`gated_linear` runs for these sizes lets the kernel after it start before it has
    finished (the weight-streaming kernel does; the TMA kernel only with more than 16 tokens): a successor that
    cannot start early has nothing to gain from asking for its weights before it waits."""
    on_tcgen05 = USE_TCGEN05 and tokens <= SKINNY_MAX_TOKENS and rows >= TCGEN05_MIN_ROWS_FEW_TOKENS and width % 8 == 0
    return not on_tcgen05


def linear_accumulate(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, status: torch.Tensor | None = None,
                      started_early: bool = True, bias: torch.Tensor | None = None) -> "torch.Tensor | SlicedSum | BiasedSum | None":
    """``residual += x @ weight.T`` (the product rounded to the activation type first) when the fused
    kernel takes the product: returns ``None``.  Otherwise returns the product, not yet added: a tensor,
    or a :class:`SlicedSum` when the product was cut into K slices (the norm that follows adds them).
    ``started_early=False``: the kernel before this one does not let its successor start early.
    ``bias`` (32-bit, one element per row of the weight) is added with the product: in the fused kernel's epilogue,
    or by whoever adds what is returned (a :class:`BiasedSum`)."""
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != weight.shape[0]:
            raise KernelError("linear_accumulate: bias must have one element per row of the weight")
        if skinny_supported(x, weight.shape[0]) and x.shape[-1] == weight.shape[1] and residual.shape == (x.shape[0], weight.shape[0]):
            _check(x, "x")
            _check(weight, "weight", x.dtype)
            _check(residual, "residual", torch.float32)
            _skinny(x, weight, residual, weight.shape[0], "residual_add", prefetch=started_early, bias=bias)
            return None
        return BiasedSum(linear(x, weight, status=status), bias)
    _check(x, "x")
    _check(weight, "weight", x.dtype)
    _check(residual, "residual", torch.float32)
    if x.shape[-1] != weight.shape[1] or residual.shape != (x.shape[0], weight.shape[0]):
        raise KernelError("linear_accumulate: shapes of x, weight and residual do not agree")
    if skinny_supported(x, weight.shape[0]):
        _skinny(x, weight, residual, weight.shape[0], "residual_add", prefetch=started_early)
        return None
    if USE_TCGEN05 and tcgen05_supported(x, weight.shape[0]):
        result = linear_tcgen05(x, weight, "residual_add", residual, status=status, defer_sum=DEFER_SLICE_SUMS)
        return result if isinstance(result, SlicedSum) else None
    return torch.mm(x, weight.t())


def gated_linear(x: torch.Tensor, up_gate: torch.Tensor, activation: str, status: torch.Tensor | None = None, limit: float = 0.0) -> torch.Tensor:
    """``up * act(gate)`` for ``[up ; gate] = x @ up_gate.T`` (``up_gate``: ``[2 * hidden, width]``); ``limit``: of the
    ``"sigmoid_limit"`` activation."""
    _check(x, "x")
    _check(up_gate, "up_gate", x.dtype)
    if activation not in _ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}; known: {sorted(_ACTIVATIONS)}")
    hidden = up_gate.shape[0] // 2
    if x.shape[-1] != up_gate.shape[1] or up_gate.shape[0] != 2 * hidden:
        raise KernelError("gated_linear: shapes of x and up_gate do not agree")
    if USE_TCGEN05 and x.shape[0] <= SKINNY_MAX_TOKENS and up_gate.shape[0] >= TCGEN05_MIN_ROWS_FEW_TOKENS and tcgen05_supported(x, up_gate.shape[0]):
        return linear_tcgen05(x, up_gate, "gated", activation=activation, status=status, limit=limit)
    out = torch.empty(x.shape[0], hidden, dtype=x.dtype, device=x.device)
    if skinny_supported(x, hidden):
        _skinny(x, up_gate, out, hidden, "gated", activation, limit=limit)
        return out
    if USE_TCGEN05 and tcgen05_supported(x, up_gate.shape[0]):
        return linear_tcgen05(x, up_gate, "gated", activation=activation, status=status, limit=limit)
    fused = linear(x, up_gate, status=status)
    gated_activation(fused.sum() if isinstance(fused, SlicedSum) else fused, out, activation, limit)
    return out


def short_conv_linear(
    x: torch.Tensor,
    in_proj: torch.Tensor,
    state: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    *,
    token_segment: torch.Tensor,
    segment_start: torch.Tensor,
    segment_length: torch.Tensor,
    segment_slot: torch.Tensor,
    segments: int,
    status: torch.Tensor,
) -> torch.Tensor:
    """The in-projection and the gated short convolution (with its state update) in one:
    ``in_proj`` is ``[3 * dim, width]`` with row blocks (B, C, x)."""
    _check(x, "x")
    _check(in_proj, "in_proj", x.dtype)
    dim = in_proj.shape[0] // 3
    if x.shape[-1] != in_proj.shape[1] or in_proj.shape[0] != 3 * dim:
        raise KernelError("short_conv_linear: shapes of x and in_proj do not agree")
    out = torch.empty(x.shape[0], dim, dtype=x.dtype, device=x.device)
    taps = weight.shape[1]
    if skinny_supported(x, dim) and segments <= x.shape[0]:
        _check(weight, "weight", torch.float32)
        if weight.shape[0] != dim:
            raise KernelError("short_conv_linear: weight must be [dim, taps]")
        if taps > 1:
            _check(state, "state", x.dtype)
            if state.dim() != 3 or state.shape[1:] != (taps - 1, dim):
                raise KernelError("short_conv_linear: state must be [slots, taps - 1, dim]")
        if bias is not None:
            _check(bias, "bias", torch.float32)
        _skinny(x, in_proj, out, dim, "short_conv", conv=dict(
            state=state, weight=weight, bias=bias, token_segment=token_segment, segment_start=segment_start, segment_length=segment_length,
            segment_slot=segment_slot, segments=segments, taps=taps, num_slots=state.shape[0], status=status))
        return out
    if segments == x.shape[0] and x.dtype == torch.bfloat16 and dim % 8 == 0 and USE_TCGEN05 and not skinny_supported(x, dim) and tcgen05_supported(x, in_proj.shape[0]):
        # a step of single tokens: the product's K slices, if it has any, are added by the convolution's kernel
        proj = linear_tcgen05(x, in_proj, "store", status=status, defer_sum=DEFER_SLICE_SUMS)
    else:
        proj = linear(x, in_proj, status=status)
    short_conv(proj, state, weight, bias, out, token_segment=token_segment, segment_start=segment_start,
               segment_length=segment_length, segment_slot=segment_slot, segments=segments, status=status)
    return out
