"""The known models of the supported architecture, for ``list-models`` and for random-weight presets.

Mirrors ``lalamo/model_registry.py:45-58`` and ``lalamo/model_import/model_specs/lfm2.py:21-67``
(full-precision LiquidAI repositories only; the quantised MLX variants are out of scope), with the
default generation options the reference gives each family.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .sampling.policy import GenerationConfig

__all__ = ["ModelRegistry", "ModelSpec", "PRESETS"]


@dataclass(frozen=True)
class ModelSpec:
    vendor: str
    family: str
    name: str
    size: str
    repo: str
    architecture: str
    generation_config: GenerationConfig

    @property
    def description(self) -> str:
        return self.repo


def _size_to_number(size: str) -> float:
    factors = {"K": 1e3, "M": 1e6, "B": 1e9, "T": 1e12}
    return float(size[:-1]) * factors[size[-1].upper()]


_LFM2 = [
    ModelSpec("LiquidAI", "LFM2", f"LFM2-{size}", size, f"LiquidAI/LFM2-{size}", "Lfm2ForCausalLM",
              GenerationConfig(temperature=0.3, min_p=0.15))
    for size in ("350M", "700M", "1.2B", "2.6B")
]
_LFM25 = [
    ModelSpec("LiquidAI", "LFM2.5", name, size, f"LiquidAI/{name}", "Lfm2ForCausalLM",
              GenerationConfig(temperature=0.1, top_k=50, top_p=0.1))
    for name, size in (("LFM2.5-350M", "350M"), ("LFM2.5-1.2B-Instruct", "1.2B"), ("LFM2.5-1.2B-Thinking", "1.2B"))
]


class ModelRegistry:
    def __init__(self, specs: list[ModelSpec]) -> None:
        self.repo_to_model = {spec.repo: spec for spec in specs}

    @classmethod
    def build(cls) -> "ModelRegistry":
        return cls(_LFM2 + _LFM25)

    def find(self, name: str) -> ModelSpec | None:
        """The spec of a repository (``"LiquidAI/LFM2-1.2B"``) or of a folder named after one
        (``"LFM2-1.2B"``, any case)."""
        if name in self.repo_to_model:
            return self.repo_to_model[name]
        wanted = name.rstrip("/").split("/")[-1].lower()
        for spec in self.repo_to_model.values():
            if spec.name.lower() == wanted:
                return spec
        return None

    def sorted_specs(self) -> list[ModelSpec]:
        """Sorted as the reference's ``list-models`` sorts (``lalamo/main.py:591-599``)."""
        return sorted(
            self.repo_to_model.values(),
            key=lambda spec: (spec.vendor.lower(), spec.family.lower(), _size_to_number(spec.size), spec.name.lower()),
        )


def _lfm2_shape(hidden: int, heads: int, ff_dim: int) -> dict[str, Any]:
    return {
        "architectures": ["Lfm2ForCausalLM"],
        "model_type": "lfm2",
        "vocab_size": 65536,
        "hidden_size": hidden,
        "num_hidden_layers": 16,
        "num_attention_heads": heads,
        "num_heads": heads,
        "num_key_value_heads": 8,
        "full_attn_idxs": [2, 5, 8, 10, 12, 14],
        "block_auto_adjust_ff_dim": True,
        "block_ff_dim": ff_dim,
        "block_ffn_dim_multiplier": 1.0,
        "block_multiple_of": 256,
        "conv_L_cache": 3,
        "conv_bias": False,
        "rope_theta": 1000000.0,
        "block_norm_eps": 1e-5,
        "norm_eps": 1e-5,
        "tie_embedding": True,
        "max_position_embeddings": 128000,
        "bos_token_id": 1,
        "eos_token_id": 7,
        "pad_token_id": 0,
    }


def _vuvulorn_shape(width: int, layers: int, left_heads: int, left_kv_heads: int, right_heads: int, right_dim: int, right_vdim: int, ff: int,
                    experts: int, top: int, rank: int) -> dict[str, Any]:
    """A Vuvulorn shape for the random-weights mode: head size 64 on the attention side under a window of 1,024 tokens
    that keeps the first 4, dense and routed feed-forwards in turn, the routed ones with as many active columns
    (``top`` experts of ``ff / top``) as the dense ones have."""
    def mixer() -> dict[str, Any]:
        return {
            "left": {"heads": left_heads, "kv_heads": left_kv_heads, "dim": 64, "vdim": 64, "scale": 0.125,
                     "mask": {"size": 1024, "keep_first": 4}, "rot": {"dims": 64, "base": 1000000.0}},
            "right": {"heads": right_heads, "kv_heads": right_heads, "dim": right_dim, "vdim": right_vdim, "conv": 4, "decay_rank": rank, "gate_rank": rank},
            "left_scale": 1.0,
            "right_scale": 1.0,
        }

    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": ff // top}, "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}}
    return {
        "architecture": "Vuvulorn",
        "vocab": 65536,
        "width": width,
        "norm": {"eps": 1e-6},
        "layers": [{"type": "parallel", "mixer": mixer(), "mlp": routed if index % 2 else dense} for index in range(layers)],
    }


def _tudulix_shape(width: int, layers: int, heads: int, kv_heads: int, ff: int, experts: int, top: int, rank: int) -> dict[str, Any]:
    """A Tudulix shape for the random-weights mode: grouped attention with heads of 64 under a window of 1,024 tokens in turn
    with latent attention (heads of 64 + 32 rotated channels over a latent of ``rank``) under a window of 2,048, every layer
    with ``top`` routed experts of ``ff`` columns and a shared one of as many; the third and fourth layer run twice."""
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 1024}, "rot": {"dims": 64, "base": 1000000.0}}
    latent = {"heads": heads, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": rank, "scale": 96 ** -0.5, "mask": {"size": 2048}, "rot": {"dims": 32, "base": 10000.0}}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top}, "shared": {"ff": ff, "limit": 7.0}}
    return {
        "architecture": "Tudulix",
        "vocab": 65536,
        "width": width,
        "norm": {"eps": 1e-6},
        "embedding": {"scale": float(width) ** 0.5},
        "logit_scale": 1.0,
        "loop": {"start": 2, "stop": 4, "times": 2},
        "layers": [{"type": "latent_attention" if index % 2 else "attention", "mixer": latent if index % 2 else attention, "mlp": mlp} for index in range(layers)],
    }


def _vivulorn_shape(width: int, layers: int, heads: int, kv_heads: int, delta_heads: int, delta_dim: int, delta_vdim: int, ff: int, rank: int) -> dict[str, Any]:
    """A Vivulorn shape for the random-weights mode: layers in the order attention, delta rule, latent attention, delta rule;
    attention with heads of 64 and stretched rotation, latent attention with heads of 64 + 32 rotated channels over a latent of
    ``rank``, the delta rule with ``delta_heads`` heads over half as many key heads behind convolutions of four taps; every layer
    but each second delta layer with a dense feed-forward of ``ff`` columns; the third and fourth layer run twice."""
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125,
                 "rot": {"dims": 64, "base": 1000000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    latent = {"heads": heads, "dim": 64, "rot_dim": 32, "vdim": 64, "kv_rank": rank, "scale": 96 ** -0.5, "rot": {"dims": 32, "base": 10000.0}}
    delta = {"heads": delta_heads, "kv_heads": delta_heads // 2, "dim": delta_dim, "vdim": delta_vdim, "conv": 4}
    kinds = [("attention", attention), ("delta", delta), ("latent_attention", latent), ("delta", delta)]
    dense = {"kind": "dense", "ff": ff}
    return {
        "architecture": "Vivulorn",
        "vocab": 65536,
        "width": width,
        "norm": {"eps": 1e-5},
        "embedding": {"scale": float(width) ** 0.5},
        "logit_softcap": 30.0,
        "loop": {"start": 2, "stop": 4, "times": 2},
        "layers": [{"type": kinds[index % 4][0], "mixer": kinds[index % 4][1], "mlp": None if index % 8 == 7 else dense} for index in range(layers)],
    }


def _zozenex_shape(width: int, layers: int, heads: int, kv_heads: int, linear_heads: int, linear_dim: int, linear_vdim: int, ff: int, experts: int, top: int) -> dict[str, Any]:
    """A Zozenex shape for the random-weights mode: retention layers in turn with layers of two mixers side by side: sigmoid attention
    with heads of 64 under a window of 1,024 tokens with one mean key and value for every 8 positions before it, and gated linear
    attention; ``linear_heads`` heads of ``linear_dim`` x ``linear_vdim`` in both kinds of recurrence; every layer with ``top`` routed
    experts of ``ff`` columns and a shared one of as many (no gates: two matrices each)."""
    retention = {"heads": linear_heads, "dim": linear_dim, "vdim": linear_vdim, "decay": [1.0 - 2.0 ** (-5 - head) for head in range(linear_heads)]}
    parallel = {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 30.0, "mask": {"size": 1024, "pool": 8},
                 "rot": {"dims": 64, "base": 1000000.0}},
        "right": {"heads": linear_heads, "dim": linear_dim, "vdim": linear_vdim, "tau": 16.0, "rank": 64},
    }
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": 2.0}, "shared": {"ff": ff}}
    return {
        "architecture": "Zozenex",
        "vocab": 65536,
        "width": width,
        "max_positions": 16384,
        "norm": {"eps": 1e-5},
        "layers": [{"type": "parallel" if index % 2 else "retention", "mixer": parallel if index % 2 else retention, "mlp": mlp} for index in range(layers)],
    }


# Shapes of the published checkpoints, and Vuvulorn shapes of the same widths and depths, for the random-weights mode
# (no weights are downloaded).
PRESETS: dict[str, dict[str, Any]] = {
    "lfm2-350m": _lfm2_shape(1024, 16, 6656),
    "lfm2-700m": _lfm2_shape(1536, 24, 10240),
    "lfm2-1.2b": _lfm2_shape(2048, 32, 12288),
    "vuvulorn-350m": _vuvulorn_shape(1024, 16, 16, 4, 8, 64, 128, 4608, 16, 4, 64),
    "vuvulorn-1.2b": _vuvulorn_shape(2048, 16, 16, 4, 8, 128, 128, 8192, 16, 4, 64),
    # 14 layers of which two run twice: 16 layer runs, and per token as many feed-forward columns (3 routed experts + the shared one) as the shapes above
    "tudulix-350m": _tudulix_shape(1024, 14, 16, 4, 1152, 16, 3, 256),
    "tudulix-1.2b": _tudulix_shape(2048, 14, 16, 4, 2048, 16, 3, 256),
    # 14 layers of which two run twice (16 layer runs); the two projections of the plain feed-forward hold what the three of a gated one of 4,608 (8,192) columns hold
    "vivulorn-350m": _vivulorn_shape(1024, 14, 16, 4, 8, 64, 128, 6912, 256),
    "vivulorn-1.2b": _vivulorn_shape(2048, 14, 16, 4, 8, 128, 128, 12288, 256),
    # 16 layers; 3 routed experts + the shared one hold in their two matrices each what the three of a gated feed-forward of 4,608 (8,192) columns hold
    "zozenex-350m": _zozenex_shape(1024, 16, 16, 4, 8, 64, 128, 1728, 16, 3),
    "zozenex-1.2b": _zozenex_shape(2048, 16, 16, 4, 8, 128, 128, 3072, 16, 3),
}
