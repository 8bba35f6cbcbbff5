"""Typed configuration of the Vivulorn architecture (``"architecture": "Vivulorn"`` in ``config.json``).

A pre-norm decoder, ``x <- x + mixer(norm1(x)); x <- x + ff(norm2(x))``, whose norms are layer norms with weight and
bias.  A layer's mixer is one of three: grouped softmax attention (an RMS norm over the whole q and the whole k
projection, rotation in halves with stretched frequencies, a sigmoid gate from the mixer's input on the heads'
outputs); latent attention (keys and values made from one normed latent vector per token plus one key part shared by
all heads and rotated in pairs of neighbouring channels; a learned sink per head in the softmax's denominator); or a
gated-delta-rule recurrence with one decay per head, fed by short causal convolutions and read out through a per-head
RMS norm and a silu gate.  The feed-forward is two projections with biases around the exact gelu, or absent.  A stretch
of the layers may run several times in a row with the same weights, every pass with a cache of its own; each pass
begins by renewing the stream from itself and the embedding's output through one projection.  The embedding is scaled;
the read-out is the embedding table itself, and the logits are soft-capped.

``config.json``: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap``, ``loop`` (``start``, ``stop``,
``times``; optional) and ``layers``, one entry per layer: ``type`` (``"attention"`` with ``mixer``: ``heads, kv_heads, dim,
vdim, scale, rot.dims, rot.base, rot.scaling.{factor, original, fast, slow}``; ``"latent_attention"`` with ``mixer``: ``heads,
dim, rot_dim, vdim, kv_rank, scale, rot.base``; ``"delta"`` with ``mixer``: ``heads, kv_heads, dim, vdim, conv``) and ``mlp``
(``null`` or ``{"kind": "dense", "ff"}``).

Checkpoint names: ``embed``, ``loop.in``, ``final.norm`` (``.b``: its bias), and per layer ``l<i>.norm1``, ``l<i>.norm2`` (with
``.b``), ``l<i>.mix.{q,k,v,q.norm,k.norm,g,o}``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,o}`` or
``l<i>.mix.{q,k,v}`` with ``.conv``, ``l<i>.mix.{b,a,A_log,dt_bias,norm,g,o}``, and ``l<i>.mlp.{up,down}`` with ``.b``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .plan import (
    AttentionSpec,
    BlockSpec,
    DenseMLPSpec,
    EmbeddingSpec,
    GatedDeltaSpec,
    HeadSpec,
    LatentAttentionSpec,
    LayerNormSpec,
    ModelPlan,
    RMSNormSpec,
    RopeSpec,
    ScheduleEntry,
    StreamMixSpec,
    YarnScaling,
)

__all__ = ["VivulornConfig"]

UNIT_EPS = 1e-6  # the design fixes the epsilon under the root that makes the recurrence's q and k unit vectors
LAYER_TYPES = ("attention", "latent_attention", "delta")


def _get(raw: Mapping[str, Any], path: str, kind: type | tuple[type, ...], where: str) -> Any:
    value: Any = raw
    for key in path.split("."):
        if not isinstance(value, Mapping) or key not in value or value[key] is None:
            raise ConfigError(f"{where}.{path}", "is required but missing")
        value = value[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"{where}.{path}", f"has the wrong type: {value!r}")
    return value


def _has(raw: Mapping[str, Any], path: str) -> bool:
    value: Any = raw
    for key in path.split("."):
        if not isinstance(value, Mapping) or value.get(key) is None:
            return False
        value = value[key]
    return True


def _positive(raw: Mapping[str, Any], path: str, where: str) -> int:
    value = _get(raw, path, int, where)
    if value < 1:
        raise ConfigError(f"{where}.{path}", f"must be positive, got {value}")
    return value


def _number(raw: Mapping[str, Any], path: str, where: str) -> float:
    return float(_get(raw, path, (int, float), where))


@dataclass(frozen=True)
class VivulornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float  # 0: the logits are not capped
    layers: tuple[BlockSpec, ...]
    loop: tuple[int, int, int] | None  # start, stop, times: layers start .. stop - 1 run `times` times in a row
    raw: dict

    architecture = "Vivulorn"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VivulornConfig":
        name = raw.get("architecture")
        if name is not None and name != "Vivulorn":
            raise ConfigError("architecture", f"expected 'Vivulorn', got {name!r}")
        vocab = _positive(raw, "vocab", "config")
        width = _positive(raw, "width", "config")
        eps = _number(raw, "norm.eps", "config")
        layer_list = raw.get("layers")
        if not isinstance(layer_list, list) or not layer_list:
            raise ConfigError("layers", "must be a non-empty list")
        layers = tuple(cls._layer(entry, index, width, eps) for index, entry in enumerate(layer_list))
        loop = None
        if raw.get("loop") is not None:
            start, stop = _get(raw, "loop.start", int, "config"), _get(raw, "loop.stop", int, "config")
            times = _positive(raw, "loop.times", "config")
            if not 0 <= start <= stop <= len(layers):
                raise ConfigError("loop", f"start={start} and stop={stop} must satisfy 0 <= start <= stop <= {len(layers)} layers")
            if start < stop:
                loop = (start, stop, times)
        softcap = _number(raw, "logit_softcap", "config") if raw.get("logit_softcap") is not None else 0.0
        if softcap < 0.0:
            raise ConfigError("logit_softcap", f"must not be negative, got {softcap}")
        return cls(
            vocab=vocab,
            width=width,
            norm_eps=eps,
            embedding_scale=_number(raw, "embedding.scale", "config") if _has(raw, "embedding.scale") else 1.0,
            logit_softcap=softcap,
            layers=layers,
            loop=loop,
            raw=copy.deepcopy(dict(raw)),
        )

    @staticmethod
    def _rope(mixer: Mapping[str, Any], at: str, dims: int, pairing: str) -> RopeSpec | None:
        if dims == 0:
            return None
        scaling = None
        if _has(mixer, "rot.scaling"):
            scaling = YarnScaling(
                factor=_number(mixer, "rot.scaling.factor", at),
                original=_number(mixer, "rot.scaling.original", at),
                fast=_number(mixer, "rot.scaling.fast", at),
                slow=_number(mixer, "rot.scaling.slow", at),
            )
            if scaling.factor <= 0.0 or scaling.original <= 0.0 or scaling.fast <= 0.0 or scaling.slow <= 0.0:
                raise ConfigError(f"{at}.rot.scaling", "factor, original, fast and slow must be positive")
        base = _number(mixer, "rot.base", at)
        if base <= 1.0:
            raise ConfigError(f"{at}.rot.base", f"must exceed 1, got {base}")
        return RopeSpec(rotary_dim=dims, theta=base, pairing=pairing, scaling=scaling)

    @classmethod
    def _layer(cls, entry: Any, index: int, width: int, eps: float) -> BlockSpec:
        where = f"layers[{index}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(where, "must be an object")
        kind = entry.get("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}.type", f"unknown layer type {kind!r}; known: {list(LAYER_TYPES)}")
        mixer = _get(entry, "mixer", Mapping, where)
        at = where + ".mixer"
        heads = _positive(mixer, "heads", at)
        if kind == "attention":
            groups, dim = _positive(mixer, "kv_heads", at), _positive(mixer, "dim", at)
            if heads % groups:
                raise ConfigError(f"{at}.kv_heads", f"{groups} does not divide heads={heads}")
            rot_dims = _get(mixer, "rot.dims", int, at) if _has(mixer, "rot.dims") else 0
            if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
                raise ConfigError(f"{at}.rot.dims", f"must be even and at most dim={dim}, got {rot_dims}")
            mixer_spec: Any = AttentionSpec(
                model_dim=width,
                num_heads=heads,
                num_groups=groups,
                head_dim=dim,
                qk_norm=RMSNormSpec(dim=dim, eps=eps, exact=True),
                qk_norm_whole=True,
                position=cls._rope(mixer, at, rot_dims, "half"),
                scale=_number(mixer, "scale", at),
                value_dim=_positive(mixer, "vdim", at),
                gated=True,
            )
        elif kind == "latent_attention":
            rot_dim = _positive(mixer, "rot_dim", at)
            if rot_dim % 2:
                raise ConfigError(f"{at}.rot_dim", f"must be even, got {rot_dim}")
            if _has(mixer, "rot.dims") and mixer["rot"]["dims"] != rot_dim:
                raise ConfigError(f"{at}.rot.dims", f"the rotated part has rot_dim={rot_dim} channels, got {mixer['rot']['dims']}")
            rank = _positive(mixer, "kv_rank", at)
            mixer_spec = LatentAttentionSpec(
                model_dim=width,
                num_heads=heads,
                head_dim=_positive(mixer, "dim", at),
                rope_dim=rot_dim,
                value_dim=_positive(mixer, "vdim", at),
                latent_dim=rank,
                latent_norm=RMSNormSpec(dim=rank, eps=eps, exact=True),
                position=cls._rope(mixer, at, rot_dim, "interleaved"),
                scale=_number(mixer, "scale", at),
                sink=True,
            )
        else:
            groups = _positive(mixer, "kv_heads", at)
            if heads % groups:
                raise ConfigError(f"{at}.kv_heads", f"{groups} does not divide heads={heads}")
            mixer_spec = GatedDeltaSpec(
                model_dim=width,
                num_heads=heads,
                num_groups=groups,
                key_dim=_positive(mixer, "dim", at),
                value_dim=_positive(mixer, "vdim", at),
                conv_taps=_positive(mixer, "conv", at),
                decay_rank=0,
                gate_rank=0,
                norm_eps=eps,
                unit_eps=UNIT_EPS,
                decay_per_channel=False,
                gate_activation="silu",
            )
        norm = LayerNormSpec(dim=width, eps=eps)
        mlp = entry.get("mlp")
        if mlp is None:
            return BlockSpec(pre_mixer_norm=norm, mixer=mixer_spec)
        at = where + ".mlp"
        if not isinstance(mlp, Mapping):
            raise ConfigError(at, "must be an object or null")
        if mlp.get("kind") != "dense":
            raise ConfigError(f"{at}.kind", f"unknown feed-forward kind {mlp.get('kind')!r}; known: ['dense']")
        ffn = DenseMLPSpec(model_dim=width, hidden_dim=_positive(mlp, "ff", at), activation="gelu", has_bias=True)
        return BlockSpec(pre_mixer_norm=norm, mixer=mixer_spec, pre_ffn_norm=norm, ffn=ffn)

    # --------------------------------------------------------------------- plan
    def schedule(self) -> tuple[ScheduleEntry, ...]:
        """Layers before the repeated stretch once, the stretch ``times`` times (every pass, the first too, begins by
        renewing the stream from itself and the embedding's output; every execution owns its cache), then the rest."""
        if self.loop is None:
            return tuple(ScheduleEntry(index) for index in range(len(self.layers)))
        start, stop, times = self.loop
        entries = [ScheduleEntry(index) for index in range(start)]
        for _ in range(times):
            entries += [ScheduleEntry(index, mix_embedding=index == start) for index in range(start, stop)]
        entries += [ScheduleEntry(index) for index in range(stop, len(self.layers))]
        return tuple(entries)

    def to_plan(self) -> ModelPlan:
        return ModelPlan(
            vocab_size=self.vocab,
            model_dim=self.width,
            layers=self.layers,
            final_norm=LayerNormSpec(dim=self.width, eps=self.norm_eps),
            tie_embeddings=True,
            schedule=self.schedule(),
            embedding=EmbeddingSpec(self.vocab, self.width, self.embedding_scale),
            head=HeadSpec(self.vocab, self.width, tied=True, softcap=self.logit_softcap),
            stream_mix=StreamMixSpec(self.width) if self.loop is not None else None,
        )

    # ---------------------------------------------------------- checkpoint names
    _ATTENTION = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "q_norm": "q.norm", "k_norm": "k.norm", "gate_proj": "g", "out_proj": "o"}
    _LATENT = {"q_proj": "q", "down_proj": "dkv", "latent_norm": "dkv.norm", "key_up_proj": "uk", "value_up_proj": "uv", "sink": "sink", "out_proj": "o"}
    _DELTA = {
        "q_proj": "q", "k_proj": "k", "v_proj": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta_proj": "b", "a_log": "A_log",
        "dt_bias": "dt_bias", "decay_proj": "a", "gate_proj": "g", "out_norm": "norm", "out_proj": "o",
    }
    _MLP = {"up_proj": "up", "up_bias": "up.b", "down_proj": "down", "down_bias": "down.b"}
    _NORMS = {"pre_mixer_norm": "norm1", "pre_ffn_norm": "norm2"}
    _NORM = {"scale": "", "bias": ".b"}

    def checkpoint_names(self, path: tuple, local: str) -> list[str]:
        if path == ("embedding",):
            return ["embed"]
        if path == ("stream_mix",):
            return ["loop.in"]
        if path == ("final_norm",) and local in self._NORM:
            return ["final.norm" + self._NORM[local]]
        if path[0] == "layers":
            index, role = path[1], path[2]
            root = f"l{index}"
            if role in self._NORMS and local in self._NORM:
                return [f"{root}.{self._NORMS[role]}{self._NORM[local]}"]
            if role == "mixer":
                mixer = self.layers[index].mixer
                table = self._LATENT if isinstance(mixer, LatentAttentionSpec) else self._DELTA if isinstance(mixer, GatedDeltaSpec) else self._ATTENTION
                if local in table:
                    return [f"{root}.mix.{table[local]}"]
            if role == "ffn" and local in self._MLP:
                return [f"{root}.mlp.{self._MLP[local]}"]
        raise KeyError(f"Vivulorn has no tensor {local!r} at {path!r}")

    def to_json_dict(self) -> dict[str, Any]:
        raw = copy.deepcopy(self.raw)
        raw["architecture"] = "Vivulorn"
        return raw
