"""Part specifications: the data from which a model is put together.

A model is described by a :class:`ModelPlan`: a tuple of :class:`BlockSpec` (each naming
its norm, mixer and feed-forward by a spec object) plus a *schedule*, the list that says
in which order blocks run.  Every size and constant lives in a spec; no part reads the
architecture's ``config.json`` and no part knows which model it is in.

The reference keeps the same information in a tree of ``*Config`` dataclasses
(``lalamo/modules/transformer_layer.py:164-207``, ``lalamo/modules/transformer.py:31-41``,
``lalamo/modules/decoder.py:158-207``).  Here the tree is flat, and the order of execution
is data as well.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar

__all__ = [
    "AttentionSpec",
    "BlockSpec",
    "DenseMLPSpec",
    "EmbeddingSpec",
    "HeadSpec",
    "FeedForwardSpec",
    "GatedDeltaSpec",
    "GatedMLPSpec",
    "LatentAttentionSpec",
    "LayerNormSpec",
    "LinearAttentionSpec",
    "MixerSpec",
    "ModelPlan",
    "NormSpec",
    "OutputNormBlockSpec",
    "ParallelMixerSpec",
    "PooledWindowAttentionSpec",
    "PositionSpec",
    "RMSNormSpec",
    "RopeSpec",
    "RoutedMLPSpec",
    "SandwichBlockSpec",
    "ScheduleEntry",
    "ShortConvSpec",
    "StreamMixSpec",
    "YarnScaling",
]


@dataclass(frozen=True)
class NormSpec:
    """Base of all normalisation specs.  ``kind`` selects the part class."""

    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class RMSNormSpec(NormSpec):
    """Root-mean-square norm: ``x * rsqrt(mean(x^2) + eps) * (w + scale_offset)``.

    Mirrors ``NormalizationConfig`` with ``subtract_mean=False``
    (``lalamo/modules/normalization.py:49-76``).
    """

    kind: ClassVar[str] = "rms_norm"
    dim: int = 0
    eps: float = 1e-5
    scale_offset: float = 0.0
    # True: the whole norm in 32-bit, ``x * rsqrt(mean(x^2) + eps) * (w + scale_offset)`` rounded once to the
    # activation type (False: the normalised value and the scale are each rounded first, as the reference does).
    exact: bool = False


@dataclass(frozen=True)
class LayerNormSpec(NormSpec):
    """Layer norm with weight and bias: ``(x - mean) / sqrt(var + eps) * w + b``, the variance being the mean of the
    squared deviations; 32-bit throughout, rounded once to the activation type."""

    kind: ClassVar[str] = "layer_norm"
    dim: int = 0
    eps: float = 1e-5


@dataclass(frozen=True)
class PositionSpec:
    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class YarnScaling:
    """Frequencies stretched for contexts beyond the ``original`` one: pair ``i`` of ``n`` rotated channels turns
    ``original * f_i / (2 pi)`` times within the original context; with ``pair(t) = n ln(original / (2 pi t)) / (2 ln theta)``
    the pair that turns ``t`` times, ``lo = max(floor(pair(fast)), 0)``, ``hi = min(ceil(pair(slow)), n - 1)`` and
    ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``, the frequency becomes ``f_i / factor * ramp_i + f_i (1 - ramp_i)``,
    and sines and cosines are multiplied by ``0.1 ln(factor) + 1``."""

    factor: float = 1.0
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0


@dataclass(frozen=True)
class RopeSpec(PositionSpec):
    """Unscaled rotary embedding over the first ``rotary_dim`` channels of a head
    (``lalamo/modules/rope.py:58-102``).  ``pairing``: ``"half"`` rotates channel ``i`` with channel
    ``i + rotary_dim / 2`` (NeoX), ``"interleaved"`` channel ``2i`` with ``2i + 1``; pair ``i`` turns by
    ``position * theta ** (-2i / rotary_dim)`` either way."""

    kind: ClassVar[str] = "rope"
    rotary_dim: int = 0
    theta: float = 10000.0
    pairing: str = "half"
    scaling: YarnScaling | None = None  # stretched frequencies and a factor on sines and cosines


@dataclass(frozen=True)
class MixerSpec:
    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Grouped-query causal attention with optional per-head q/k norm, position encoding
    and sliding window (``lalamo/modules/token_mixers/attention.py:332-447``)."""

    kind: ClassVar[str] = "attention"
    model_dim: int = 0
    num_heads: int = 0
    num_groups: int = 0
    head_dim: int = 0
    qk_norm: NormSpec | None = None
    position: PositionSpec | None = None
    window: int | None = None
    scale: float | None = None  # None -> head_dim ** -0.5
    value_dim: int | None = None  # size of a value head; None -> head_dim
    keep_first: int = 0  # under a window, the first tokens of a request that stay visible (at their true positions)
    has_bias: bool = False  # biases on the q, k, v and output projections
    # ``qk_norm`` over all rows of the q projection (and of the k projection) at once, before they are split into heads
    # (its ``dim`` is then ``head_dim`` still; the weights have one element per row of the projection); 32-bit, no rounding
    # between the norm and the rotation.
    qk_norm_whole: bool = False
    gated: bool = False  # the concatenated heads are multiplied by ``sigmoid(W_gate h)`` before the out-projection


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Causal attention whose keys and values are made from one latent vector per token: ``c = norm(W_down h)[:latent_dim]``
    (RMS norm with a plain weight) and one rotated key part ``r = rope(W_down h)[latent_dim:]`` of ``rope_dim`` channels
    shared by all heads; per head the unrotated key is ``W_uk c`` (``head_dim`` channels), the value ``W_uv c``
    (``value_dim``); a query head is ``[head_dim unrotated, rope_dim rotated]``; the score is
    ``(q_plain . k_plain + q_rot . r) * scale``.  Only ``c`` and ``r`` are cached.  ``gated``: the heads' outputs are
    multiplied by ``sigmoid(W_gate h)`` before the out-projection."""

    kind: ClassVar[str] = "latent_attention"
    model_dim: int = 0
    num_heads: int = 0
    head_dim: int = 0
    rope_dim: int = 0
    value_dim: int = 0
    latent_dim: int = 0
    latent_norm: NormSpec | None = None
    position: PositionSpec | None = None
    window: int | None = None
    scale: float | None = None  # None -> (head_dim + rope_dim) ** -0.5
    gated: bool = False
    sink: bool = False  # a learned number per head whose exponential joins the softmax's denominator (no key, no value, not scaled)


@dataclass(frozen=True)
class GatedDeltaSpec(MixerSpec):
    """A linear-attention mixer with a matrix state per head updated by the gated delta rule,
    ``S <- diag(g) S; S <- S + k (beta (v - S^T k))^T; o = S^T q``, one decay ``g`` per head and key
    channel.  q, k (``num_groups`` heads of ``key_dim``) and v (``num_heads`` heads of ``value_dim``)
    pass a causal depthwise convolution of ``conv_taps`` taps and silu; q and k are made unit vectors
    (``x / sqrt(sum x^2 + unit_eps)``, q times ``key_dim ** -0.5``); ``beta = sigmoid(W_b h)``;
    ``g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))`` through a bottleneck of ``decay_rank``; the
    read-out is RMS-normed per head (``norm_eps``) and multiplied by ``sigmoid(W_g2 W_g1 h)`` through a
    bottleneck of ``gate_rank``, then projected out.

    ``decay_per_channel=False``: one decay per head, ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))`` with one row of
    ``W_a`` and one ``dt_bias`` per head.  ``decay_rank=0`` / ``gate_rank=0``: no bottleneck, the logits are a plain
    projection of the mixer's input.  ``gate_activation``: ``"sigmoid"`` or ``"silu"``."""

    kind: ClassVar[str] = "gated_delta"
    model_dim: int = 0
    num_heads: int = 0
    num_groups: int = 0
    key_dim: int = 0
    value_dim: int = 0
    conv_taps: int = 1
    decay_rank: int = 0
    gate_rank: int = 0
    norm_eps: float = 1e-6
    unit_eps: float = 1e-6
    decay_per_channel: bool = True
    gate_activation: str = "sigmoid"


@dataclass(frozen=True)
class LinearAttentionSpec(MixerSpec):
    """Linear attention with a decaying matrix state per head and neither softmax nor denominator:
    ``S_t = diag(a_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t`` with q, k of ``key_dim`` and v of ``value_dim`` channels per head,
    plain projections of the mixer's input; one of q and k (``scaled``: ``"query"`` or ``"key"``) is multiplied by
    ``key_dim ** -0.5``.  The decay is fixed, one number per head (``decay="fixed"``, ``decay_values``), or made from the
    token, one number per head and key channel (``decay="channel"``): ``a = sigmoid(z) ** (1 / tau)`` with
    ``z = W_a2 (W_a1 h) + b`` through a bottleneck of ``decay_rank``.  Each head's read-out is divided by its root mean
    square (``norm_eps``; times a weight of ``value_dim`` elements shared by the heads if ``norm_weight``), the heads are
    multiplied by ``silu(W_g h)`` (or ``sigmoid``, ``gate_activation``) and projected out.  State, decays and their logarithms,
    the recurrence's inputs and the read-out norm are 32-bit."""

    kind: ClassVar[str] = "linear_attention"
    model_dim: int = 0
    num_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    decay: str = "fixed"
    decay_values: tuple[float, ...] = ()
    decay_rank: int = 0
    tau: float = 1.0
    scaled: str = "key"
    norm_weight: bool = False
    norm_eps: float = 1e-5
    gate_activation: str = "silu"


@dataclass(frozen=True)
class PooledWindowAttentionSpec(MixerSpec):
    """Grouped attention whose weights are sigmoids, not a softmax, under a sliding window with pooled blocks behind it.
    Position ``i`` sees the positions ``j`` with ``0 <= i - j < window`` and one mean key and mean value for every block of
    ``pool`` consecutive positions that lies wholly before the window (block ``b`` covers ``b pool .. b pool + pool - 1`` and
    is seen if ``b pool + pool - 1 <= i - window``; means of the keys and values as the cache holds them; ``pool=0``: no
    blocks).  A visible key weighs ``sigmoid(c tanh(q . k scale / c) + bias_h)`` (``softcap`` c, 0: none; ``head_bias``: a
    learned number per head); the weights are not normalised.  ``position`` rotates q and k; ``rotate_values``: a value is
    turned by its position over all of its channels (pair ``m`` by ``j theta ** (-2m / value_dim)``, the pairing of
    ``position``) before it is cached, and a head's sum is turned back by the query's position."""

    kind: ClassVar[str] = "pooled_window_attention"
    model_dim: int = 0
    num_heads: int = 0
    num_groups: int = 0
    head_dim: int = 0
    value_dim: int = 0
    position: PositionSpec | None = None
    rotate_values: bool = False
    window: int = 1
    pool: int = 0
    scale: float | None = None  # None -> head_dim ** -0.5
    softcap: float = 0.0
    head_bias: bool = False


@dataclass(frozen=True)
class ParallelMixerSpec(MixerSpec):
    """Several mixers side by side on the same input; the result is ``sum_i scale_i * branch_i(x)``.
    ``branches``: ``(name, specification, scale)``; the name prefixes the branch's tensors.  With ``branch_norm`` every
    branch's output passes a norm of that specification (a weight of its own per branch, ``<name>.out_norm``) before the sum."""

    kind: ClassVar[str] = "parallel"
    branches: tuple[tuple[str, MixerSpec, float], ...] = ()
    branch_norm: NormSpec | None = None


@dataclass(frozen=True)
class ShortConvSpec(MixerSpec):
    """Gated depthwise causal convolution of ``kernel_size`` taps
    (``lalamo/modules/token_mixers/short_conv.py:51-157``)."""

    kind: ClassVar[str] = "short_conv"
    model_dim: int = 0
    kernel_size: int = 0
    has_bias: bool = False


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: ClassVar[str] = "abstract"


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """``down(up(x) * act(gate(x)))`` (``lalamo/modules/mlp.py:233-262``).  With ``activation="sigmoid_limit"`` the hidden
    value is ``g * sigmoid(1.702 g) * (u + 1)`` for ``g = min(gate(x), limit)`` and ``u = clamp(up(x), -limit, limit)``."""

    kind: ClassVar[str] = "gated_mlp"
    model_dim: int = 0
    hidden_dim: int = 0
    activation: str = "silu"
    limit: float = 0.0  # of the "sigmoid_limit" activation


@dataclass(frozen=True)
class DenseMLPSpec(FeedForwardSpec):
    """``down(act(up(x) + b_up)) + b_down``: two projections, no gate.  ``activation``: ``"gelu"`` (the exact gelu,
    ``0.5 z (1 + erf(z / sqrt 2))``), ``"silu"`` or ``"identity"``."""

    kind: ClassVar[str] = "dense_mlp"
    model_dim: int = 0
    hidden_dim: int = 0
    activation: str = "gelu"
    has_bias: bool = True


@dataclass(frozen=True)
class RoutedMLPSpec(FeedForwardSpec):
    """A mixture of ``num_experts`` gated feed-forward layers of width ``hidden_dim`` of which each token
    uses ``top``: router scores ``score(W_router h)`` in 32-bit; experts in ``group_count`` equal groups of
    neighbours, a group scored by the sum of its two largest scores, only the best ``group_keep`` groups
    eligible; the chosen scores (over their sum if ``renormalize``) weigh the experts' outputs.
    ``router_bias``: a bias on the router's logits.  ``score="logits"`` ranks experts by the logits themselves;
    ``chosen_softmax``: the weights are the softmax over the chosen scores only.  ``limit``: of the experts'
    ``"sigmoid_limit"`` activation (see :class:`GatedMLPSpec`).  ``shared``: a dense feed-forward that every token
    runs besides, added to the experts' weighted sum (``shared_gate``: times ``sigmoid(w_sg . h)``, one number per token).
    ``gated=False``: the experts are ``down(act(up(x)))`` without a gate.  ``choice_bias``: a learned number per expert added to
    the scores where experts (and groups) are ranked, not where they weigh.  ``weight_scale`` multiplies the weights."""

    kind: ClassVar[str] = "routed_mlp"
    model_dim: int = 0
    hidden_dim: int = 0
    num_experts: int = 0
    top: int = 1
    group_count: int = 1
    group_keep: int = 1
    score: str = "sigmoid"
    renormalize: bool = False
    activation: str = "silu"
    router_bias: bool = False
    chosen_softmax: bool = False
    limit: float = 0.0
    shared: FeedForwardSpec | None = None
    gated: bool = True
    choice_bias: bool = False
    weight_scale: float = 1.0
    shared_gate: bool = False


@dataclass(frozen=True)
class OutputNormBlockSpec:
    """A block whose sublayers read the residual stream itself and whose norms sit on the sublayers'
    outputs: ``x <- x + mixer_norm(mixer(x)); x <- x + ffn_norm(ffn(x))`` (``ffn=None``: no second half)."""

    mixer: MixerSpec
    mixer_norm: NormSpec
    ffn: FeedForwardSpec | None = None
    ffn_norm: NormSpec | None = None
    arrangement: str = "output_norm"


@dataclass(frozen=True)
class SandwichBlockSpec:
    """A block with a norm before and after each sublayer: ``x <- x + mixer_out_norm(mixer(mixer_norm(x)));
    x <- x + ffn_out_norm(ffn(ffn_norm(x)))`` (``ffn=None``: no second half)."""

    mixer_norm: NormSpec
    mixer: MixerSpec
    mixer_out_norm: NormSpec
    ffn_norm: NormSpec | None = None
    ffn: FeedForwardSpec | None = None
    ffn_out_norm: NormSpec | None = None
    arrangement: str = "sandwich_norm"


@dataclass(frozen=True)
class BlockSpec:
    """Pre-norm residual block: ``h = x + mixer(norm1(x)); y = h + ffn(norm2(h))``
    (``lalamo/modules/transformer_layer.py:220-377``); ``ffn=None`` (with ``pre_ffn_norm=None``): no second half."""

    pre_mixer_norm: NormSpec
    mixer: MixerSpec
    pre_ffn_norm: NormSpec | None = None
    ffn: FeedForwardSpec | None = None
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token embedding: a row of the table per token id, times ``scale``, into the residual stream
    (``lalamo/modules/embedding.py``); optionally plus a learned vector per position."""

    kind: ClassVar[str] = "token_embedding"
    vocab_size: int = 0
    model_dim: int = 0
    scale: float = 1.0
    learned_positions: int = 0  # > 0: a table of this many learned position vectors; row ``p`` is added (unscaled) to the token at position ``p``


@dataclass(frozen=True)
class HeadSpec:
    """The read-out: logits ``(x @ W.T) * scale`` in 32-bit, with ``W`` the embedding table when ``tied``."""

    kind: ClassVar[str] = "lm_head"
    vocab_size: int = 0
    model_dim: int = 0
    tied: bool = True
    scale: float = 1.0  # the logits are multiplied by this (in 32-bit)
    softcap: float = 0.0  # > 0: the logits become ``softcap * tanh(logits / softcap)`` (in 32-bit, after the scale)


@dataclass(frozen=True)
class StreamMixSpec:
    """A projection that renews the residual stream from itself and the embedding's output: ``x <- W [x ; x0]`` with
    ``W [model_dim, 2 model_dim]`` (the stream's columns first) and ``x0`` the stream as the embedding left it.  Schedule
    entries with ``mix_embedding`` run it right before their block."""

    kind: ClassVar[str] = "stream_mix"
    model_dim: int = 0


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a block.

    ``layer`` indexes ``ModelPlan.layers`` (a layer may appear in several entries).
    ``cache_from`` names an earlier schedule entry whose cache this execution reads
    instead of owning one (the reference's ``kv_source_layer_index``,
    ``lalamo/modules/transformer.py:210-217``).
    """

    layer: int
    cache_from: int | None = None
    # True: the embedding's output (the stream as it was before the first block) is added to the stream
    # right before this execution (a model that runs a stretch of its layers several times re-feeds its input).
    add_embedding: bool = False
    # True: the stream is renewed from itself and the embedding's output by the plan's ``stream_mix`` projection
    # right before this execution (see :class:`StreamMixSpec`).
    mix_embedding: bool = False


@dataclass(frozen=True)
class ModelPlan:
    vocab_size: int
    model_dim: int
    layers: tuple[BlockSpec | OutputNormBlockSpec | SandwichBlockSpec, ...]
    final_norm: NormSpec
    tie_embeddings: bool = True
    embedding_scale: float | None = None
    schedule: tuple[ScheduleEntry, ...] = field(default=())
    # The parts at the model's two ends.  Left ``None`` they are the plain token embedding and the
    # plain (tied or untied) read-out made from the fields above; an architecture with, say, scaled or
    # capped logits gives a specification of its own, for which a part is registered.
    embedding: EmbeddingSpec | None = None
    head: HeadSpec | None = None
    stream_mix: StreamMixSpec | None = None  # needed by schedule entries with ``mix_embedding``

    def __post_init__(self) -> None:
        if self.embedding is None:
            object.__setattr__(self, "embedding", EmbeddingSpec(self.vocab_size, self.model_dim, self.embedding_scale or 1.0))
        if self.head is None:
            object.__setattr__(self, "head", HeadSpec(self.vocab_size, self.model_dim, self.tie_embeddings))
        if not self.schedule:
            object.__setattr__(
                self, "schedule", tuple(ScheduleEntry(i) for i in range(len(self.layers)))
            )
        for position, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{position}] names layer {entry.layer}, but there are {len(self.layers)}")
            if entry.mix_embedding and self.stream_mix is None:
                raise ValueError(f"schedule[{position}] mixes the embedding into the stream, but the plan has no stream_mix")
            if entry.cache_from is not None and not 0 <= entry.cache_from < position:
                raise ValueError(
                    f"schedule[{position}].cache_from={entry.cache_from} must name an earlier schedule entry"
                )
