"""Typed configuration of the Zozenex architecture (``"architecture": "Zozenex"`` in ``config.json``).

A pre-norm decoder over a token embedding plus a learned vector per position, ``x <- x + mixer(norm1(x)); x <- x +
ff(norm2(x))`` with RMS norms.  A layer's mixer is one of two, in an order the configuration lists:

* ``"retention"``: linear attention with one fixed decay per head, ``S_t = a_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t``, keys
  scaled by ``dim ** -0.5``, each head's read-out divided by its root mean square, times ``silu(W_g h)``, projected out;
* ``"parallel"``: two mixers side by side on the same input, each output RMS-normed over the model's width under a weight
  of its own, the result half their sum.  ``left``: grouped attention with sigmoid weights (no softmax), a capped score,
  a learned number per head added to it, rotary positions on part of q and k, values rotated by their own position and
  the sum turned back by the query's, under a sliding window with one mean key and value for every whole block of
  ``mask.pool`` positions before it.  ``right``: linear attention with a decay per head and key channel,
  ``a = sigmoid(W_a2 (W_a1 h) + b) ** (1 / tau)``, queries scaled, the read-out RMS-normed under a weight, a silu gate.

The feed-forward is a mixture of experts ``W_down gelu(W_up h)`` (exact gelu, no gate): sigmoid scores, the ``top`` experts
of largest score plus a learned correction chosen, weighed by their scores (without it) times ``router.scale``; a shared
expert of the same form runs for every token, times ``sigmoid(w_sg . h)``.  ``mlp: null`` leaves a layer without one.

``config.json``: ``vocab``, ``width``, ``max_positions``, ``norm.eps`` and ``layers``, one entry per layer: ``type``, ``mixer``
(``retention``: ``heads, dim, vdim, decay`` (a list, one per head); ``parallel``: ``left.{heads, kv_heads, dim, vdim, scale, softcap,
rot.dims, rot.base, mask.size, mask.pool}``, ``right.{heads, dim, vdim, tau}``) and ``mlp`` (``null`` or ``{"kind": "moe", "expert.ff",
"router.{experts, top, scale}", "shared.ff"}``).  The rank of the decay's bottleneck is the checkpoint's (rows of ``a1``).

Checkpoint names: ``embed``, ``pos``, ``final.norm``, ``head`` and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q,k,v,g,o}`` or
``l<i>.mix.left.{q,k,v,pb,o,out}`` with ``l<i>.mix.right.{q,k,v,g,o,norm,a1,a2,a2.b,out}``, and ``l<i>.mlp.{router,correction}``,
``l<i>.mlp.e<j>.{up,down}``, ``l<i>.mlp.shared.{up,down,sg}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError
from .plan import (
    BlockSpec,
    DenseMLPSpec,
    EmbeddingSpec,
    HeadSpec,
    LinearAttentionSpec,
    ModelPlan,
    ParallelMixerSpec,
    PooledWindowAttentionSpec,
    RMSNormSpec,
    RopeSpec,
    RoutedMLPSpec,
)

__all__ = ["ZozenexConfig"]

LAYER_TYPES = ("retention", "parallel")
DEFAULT_DECAY_RANK = 16  # of a configuration without a checkpoint (random weights) that names none


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
class ZozenexConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: tuple[BlockSpec, ...]
    raw: dict

    architecture = "Zozenex"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], ranks: Mapping[int, int] | None = None, max_positions: int | None = None) -> "ZozenexConfig":
        """``ranks``: per layer the rank of the decay's bottleneck found in a checkpoint; ``max_positions``: the rows of
        its position table."""
        name = raw.get("architecture")
        if name is not None and name != "Zozenex":
            raise ConfigError("architecture", f"expected 'Zozenex', got {name!r}")
        vocab = _positive(raw, "vocab", "config")
        width = _positive(raw, "width", "config")
        eps = _number(raw, "norm.eps", "config")
        if max_positions is None:
            max_positions = _positive(raw, "max_positions", "config")
        layer_list = raw.get("layers")
        if not isinstance(layer_list, list) or not layer_list:
            raise ConfigError("layers", "must be a non-empty list")
        layers = tuple(cls._layer(entry, index, width, eps, (ranks or {}).get(index)) for index, entry in enumerate(layer_list))
        return cls(vocab=vocab, width=width, max_positions=max_positions, norm_eps=eps, layers=layers, raw=copy.deepcopy(dict(raw)))

    @classmethod
    def from_model_dir(cls, model_dir: str | Path, raw: Mapping[str, Any]) -> "ZozenexConfig":
        """The configuration of a model folder: what ``config.json`` leaves to the tensors' shapes is read there."""
        from ..weights.safetensors_io import open_checkpoint

        ranks: dict[int, int] = {}
        positions = None
        try:
            checkpoint = open_checkpoint(model_dir)
        except (FileNotFoundError, OSError):
            checkpoint = None
        if checkpoint is not None:
            for index in range(len(raw.get("layers") or [])):
                name = f"l{index}.mix.right.a1"
                if name in checkpoint:
                    ranks[index] = checkpoint[name].shape[0]
            if "pos" in checkpoint:
                positions = checkpoint["pos"].shape[0]
        return cls.from_dict(raw, ranks, positions)

    @staticmethod
    def _retention(mixer: Mapping[str, Any], at: str, width: int, eps: float) -> LinearAttentionSpec:
        heads = _positive(mixer, "heads", at)
        decay = _get(mixer, "decay", list, at)
        if len(decay) != heads or any(isinstance(value, bool) or not isinstance(value, (int, float)) for value in decay):
            raise ConfigError(f"{at}.decay", f"must list one number per head ({heads}), got {decay!r}")
        return LinearAttentionSpec(
            model_dim=width,
            num_heads=heads,
            key_dim=_positive(mixer, "dim", at),
            value_dim=_positive(mixer, "vdim", at),
            decay="fixed",
            decay_values=tuple(float(value) for value in decay),
            scaled="key",
            norm_weight=False,
            norm_eps=eps,
            gate_activation="silu",
        )

    @staticmethod
    def _parallel(mixer: Mapping[str, Any], at: str, width: int, eps: float, rank: int | None) -> ParallelMixerSpec:
        left, right = _get(mixer, "left", Mapping, at), _get(mixer, "right", Mapping, at)
        where = at + ".left"
        heads, groups, dim, vdim = _positive(left, "heads", where), _positive(left, "kv_heads", where), _positive(left, "dim", where), _positive(left, "vdim", where)
        if heads % groups:
            raise ConfigError(f"{where}.kv_heads", f"{groups} does not divide heads={heads}")
        if vdim % 2:
            raise ConfigError(f"{where}.vdim", f"values are rotated in pairs: vdim must be even, got {vdim}")
        rot_dims = _get(left, "rot.dims", int, where) if _has(left, "rot.dims") else 0
        if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"{where}.rot.dims", f"must be even and at most dim={dim}, got {rot_dims}")
        base = _number(left, "rot.base", where)
        if base <= 0.0:
            raise ConfigError(f"{where}.rot.base", f"must be positive, got {base}")
        softcap = _number(left, "softcap", where) if _has(left, "softcap") else 0.0
        if softcap < 0.0:
            raise ConfigError(f"{where}.softcap", f"must not be negative, got {softcap}")
        pool = _get(left, "mask.pool", int, where) if _has(left, "mask.pool") else 0
        if pool < 0:
            raise ConfigError(f"{where}.mask.pool", f"must not be negative, got {pool}")
        attention = PooledWindowAttentionSpec(
            model_dim=width,
            num_heads=heads,
            num_groups=groups,
            head_dim=dim,
            value_dim=vdim,
            # the values' rotation takes its base from here also where no channel of q and k is rotated
            position=RopeSpec(rotary_dim=rot_dims, theta=base, pairing="half"),
            rotate_values=True,
            window=_positive(left, "mask.size", where),
            pool=pool,
            scale=_number(left, "scale", where),
            softcap=softcap,
            head_bias=True,
        )
        where = at + ".right"
        tau = _number(right, "tau", where)
        if tau <= 0.0:
            raise ConfigError(f"{where}.tau", f"must be positive, got {tau}")
        if rank is None:
            rank = _positive(right, "rank", where) if _has(right, "rank") else DEFAULT_DECAY_RANK
        linear = LinearAttentionSpec(
            model_dim=width,
            num_heads=_positive(right, "heads", where),
            key_dim=_positive(right, "dim", where),
            value_dim=_positive(right, "vdim", where),
            decay="channel",
            decay_rank=rank,
            tau=tau,
            scaled="query",
            norm_weight=True,
            norm_eps=eps,
            gate_activation="silu",
        )
        return ParallelMixerSpec(branches=(("left", attention, 0.5), ("right", linear, 0.5)), branch_norm=RMSNormSpec(dim=width, eps=eps, exact=True))

    @classmethod
    def _layer(cls, entry: Any, index: int, width: int, eps: float, rank: int | None) -> BlockSpec:
        where = f"layers[{index}]"
        if not isinstance(entry, Mapping):
            raise ConfigError(where, "must be an object")
        kind = entry.get("type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}.type", f"unknown layer type {kind!r}; known: {list(LAYER_TYPES)}")
        mixer = _get(entry, "mixer", Mapping, where)
        at = where + ".mixer"
        mixer_spec: Any = cls._retention(mixer, at, width, eps) if kind == "retention" else cls._parallel(mixer, at, width, eps, rank)
        norm = RMSNormSpec(dim=width, eps=eps, exact=True)
        mlp = entry.get("mlp")
        if mlp is None:
            return BlockSpec(pre_mixer_norm=norm, mixer=mixer_spec)
        at = where + ".mlp"
        if not isinstance(mlp, Mapping):
            raise ConfigError(at, "must be an object or null")
        if mlp.get("kind") != "moe":
            raise ConfigError(f"{at}.kind", f"unknown feed-forward kind {mlp.get('kind')!r}; known: ['moe']")
        experts, top = _positive(mlp, "router.experts", at), _positive(mlp, "router.top", at)
        if top > experts:
            raise ConfigError(f"{at}.router.top", f"{top} experts a token of {experts}")
        shared = None
        if mlp.get("shared") is not None:
            shared = DenseMLPSpec(model_dim=width, hidden_dim=_positive(mlp, "shared.ff", at), activation="gelu", has_bias=False)
        ffn = RoutedMLPSpec(
            model_dim=width,
            hidden_dim=_positive(mlp, "expert.ff", at),
            num_experts=experts,
            top=top,
            score="sigmoid",
            renormalize=False,
            activation="gelu",
            gated=False,
            choice_bias=True,
            weight_scale=_number(mlp, "router.scale", at) if _has(mlp, "router.scale") else 1.0,
            shared=shared,
            shared_gate=shared is not None,
        )
        return BlockSpec(pre_mixer_norm=norm, mixer=mixer_spec, pre_ffn_norm=norm, ffn=ffn)

    # --------------------------------------------------------------------- plan
    def to_plan(self) -> ModelPlan:
        return ModelPlan(
            vocab_size=self.vocab,
            model_dim=self.width,
            layers=self.layers,
            final_norm=RMSNormSpec(dim=self.width, eps=self.norm_eps, exact=True),
            tie_embeddings=False,
            embedding=EmbeddingSpec(self.vocab, self.width, 1.0, learned_positions=self.max_positions),
            head=HeadSpec(self.vocab, self.width, tied=False),
        )

    # ---------------------------------------------------------- checkpoint names
    _RETENTION = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "gate_proj": "g", "out_proj": "o"}
    _LEFT = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "head_bias": "pb", "out_proj": "o", "out_norm.scale": "out"}
    _RIGHT = {**_RETENTION, "out_norm": "norm", "decay_down": "a1", "decay_up": "a2", "decay_bias": "a2.b", "out_norm.scale": "out"}
    _MLP = {"router": "router", "choice_bias": "correction", "shared.up_proj": "shared.up", "shared.down_proj": "shared.down", "shared_gate": "shared.sg"}
    _NORMS = {"pre_mixer_norm": "norm1", "pre_ffn_norm": "norm2"}

    def checkpoint_names(self, path: tuple, local: str) -> list[str]:
        if path == ("embedding",):
            if local == "weight":
                return ["embed"]
            if local == "positions":
                return ["pos"]
        if path == ("lm_head",) and local == "weight":
            return ["head"]
        if path == ("final_norm",) and local == "scale":
            return ["final.norm"]
        if path[0] == "layers":
            index, role = path[1], path[2]
            root = f"l{index}"
            if role in self._NORMS and local == "scale":
                return [f"{root}.{self._NORMS[role]}"]
            if role == "mixer":
                if isinstance(self.layers[index].mixer, LinearAttentionSpec):
                    if local in self._RETENTION:
                        return [f"{root}.mix.{self._RETENTION[local]}"]
                else:
                    for branch, table in (("left", self._LEFT), ("right", self._RIGHT)):
                        if local.startswith(branch + ".") and local[len(branch) + 1 :] in table:
                            return [f"{root}.mix.{branch}.{table[local[len(branch) + 1 :]]}"]
            if role == "ffn":
                if local in self._MLP:
                    return [f"{root}.mlp.{self._MLP[local]}"]
                parts = local.split(".")
                if len(parts) == 3 and parts[0] == "experts" and parts[2] in ("up_proj", "down_proj"):
                    return [f"{root}.mlp.e{parts[1]}.{parts[2][:-5]}"]
        raise KeyError(f"Zozenex has no tensor {local!r} at {path!r}")

    def to_json_dict(self) -> dict[str, Any]:
        raw = copy.deepcopy(self.raw)
        raw["architecture"] = "Zozenex"
        raw["max_positions"] = self.max_positions
        return raw
