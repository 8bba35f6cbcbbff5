"""Small Vivulorn configurations for the tests, and a writer of model folders whose tensor names and shapes are spelled
out here from the configuration (not taken from the package), with weights large enough that every mechanism matters
in the logits."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from lalamo_b200.weights.safetensors_io import write_safetensors


def attention(heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=16, base=10000.0, scale=0.25, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}


def latent(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=32, base=10000.0, scale=0.2):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": {"dims": rot_dim, "base": base}}


def delta(heads=4, kv_heads=2, dim=16, vdim=8, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


def model(vocab, width, layers, eps=1e-6, embedding_scale=1.0, softcap=None, loop=None):
    config = {"architecture": "Vivulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embedding_scale}, "layers": layers}
    if softcap is not None:
        config["logit_softcap"] = softcap
    if loop is not None:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
    return config


# A: a recurrent layer first, then a latent layer and an attention layer that run twice, then a recurrent layer without a
# feed-forward; value heads wider and narrower than key heads, rotation over part of a head, stretched frequencies whose ramp
# lies inside the pairs, a convolution of four taps and one of two.
CONFIG_A = model(160, 64, [
    layer("delta", delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4), dense(48)),
    layer("latent_attention", latent(heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=32, base=500.0), dense(40)),
    layer("attention", attention(heads=4, kv_heads=2, dim=16, vdim=32, rot_dims=8, base=100.0, scale=0.3, scaling=(4.0, 64, 8.0, 2.0)), dense(72)),
    layer("delta", delta(heads=2, kv_heads=2, dim=8, vdim=16, conv=2), None),
], eps=1e-5, embedding_scale=2.0, softcap=5.0, loop=(1, 3, 2))

# B: sizes that fit no kernel's favourite shape (a width and a vocabulary that are multiples of nothing much), no rotation at all in
# the attention, one head, one tap (no convolution state), no repeated stretch, no cap, an embedding scale of one, no stretched
# frequencies.
CONFIG_B = model(131, 72, [
    layer("attention", attention(heads=3, kv_heads=3, dim=24, vdim=8, rot_dims=0, scale=0.5), dense(20)),
    layer("latent_attention", latent(heads=1, dim=10, rot_dim=6, vdim=12, kv_rank=20, scale=0.4), None),
    layer("delta", delta(heads=3, kv_heads=1, dim=12, vdim=20, conv=1), dense(30)),
    layer("attention", attention(heads=2, kv_heads=1, dim=12, vdim=20, rot_dims=12, scale=0.3, scaling=(1.5, 32, 4.0, 0.5)), dense(16)),
])

# C: the sizes the tensor-core kernels take (heads of 64 with keys and values of one size, widths in multiples of 64, a latent of
# 64 with 32 rotated channels), the whole model three times.
CONFIG_C = model(256, 128, [
    layer("attention", attention(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=64, base=1000.0, scale=0.125, scaling=(2.0, 128, 16.0, 1.0)), dense(192)),
    layer("delta", delta(heads=4, kv_heads=2, dim=32, vdim=64, conv=3), None),
    layer("latent_attention", latent(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=64, scale=0.1), dense(128)),
], embedding_scale=3.0, softcap=12.0, loop=(0, 3, 3))

# D, E, F: one layer of each kind without a feed-forward: the mixers alone (E in a repeated stretch of its own).
CONFIG_D = model(96, 64, [layer("attention", attention(heads=4, kv_heads=1, dim=32, vdim=16, rot_dims=20, base=300.0, scale=0.2, scaling=(3.0, 40, 6.0, 1.0)), None)])
CONFIG_E = model(96, 64, [layer("latent_attention", latent(heads=3, dim=24, rot_dim=12, vdim=20, kv_rank=40, base=300.0, scale=0.15), None)], loop=(0, 1, 2))
CONFIG_F = model(96, 64, [layer("delta", delta(heads=6, kv_heads=2, dim=24, vdim=12, conv=5), None)], softcap=3.0)

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E, "F": CONFIG_F}


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    width = config["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (config["vocab"], width), "final.norm": (width,), "final.norm.b": (width,)}
    if "loop" in config:
        shapes["loop.in"] = (width, 2 * width)
    for index, entry in enumerate(config["layers"]):
        root = f"l{index}."
        shapes[root + "norm1"] = shapes[root + "norm1.b"] = (width,)
        mix, p = entry["mixer"], root + "mix."
        if entry["type"] == "attention":
            shapes[p + "q"] = (mix["heads"] * mix["dim"], width)
            shapes[p + "k"] = (mix["kv_heads"] * mix["dim"], width)
            shapes[p + "v"] = (mix["kv_heads"] * mix["vdim"], width)
            shapes[p + "q.norm"] = (mix["heads"] * mix["dim"],)
            shapes[p + "k.norm"] = (mix["kv_heads"] * mix["dim"],)
            shapes[p + "g"] = (mix["heads"] * mix["vdim"], width)
        elif entry["type"] == "latent_attention":
            shapes[p + "q"] = (mix["heads"] * (mix["dim"] + mix["rot_dim"]), width)
            shapes[p + "dkv"] = (mix["kv_rank"] + mix["rot_dim"], width)
            shapes[p + "dkv.norm"] = (mix["kv_rank"],)
            shapes[p + "uk"] = (mix["heads"] * mix["dim"], mix["kv_rank"])
            shapes[p + "uv"] = (mix["heads"] * mix["vdim"], mix["kv_rank"])
            shapes[p + "sink"] = (mix["heads"],)
        else:
            shapes[p + "q"] = shapes[p + "k"] = (mix["kv_heads"] * mix["dim"], width)
            shapes[p + "v"] = (mix["heads"] * mix["vdim"], width)
            shapes[p + "q.conv"] = shapes[p + "k.conv"] = (mix["kv_heads"] * mix["dim"], mix["conv"])
            shapes[p + "v.conv"] = (mix["heads"] * mix["vdim"], mix["conv"])
            shapes[p + "b"] = shapes[p + "a"] = (mix["heads"], width)
            shapes[p + "A_log"] = shapes[p + "dt_bias"] = (mix["heads"],)
            shapes[p + "norm"] = (mix["vdim"],)
            shapes[p + "g"] = (mix["heads"] * mix["vdim"], width)
        shapes[p + "o"] = (width, mix["heads"] * mix["vdim"])
        mlp = entry["mlp"]
        if mlp is None:
            continue
        shapes[root + "norm2"] = shapes[root + "norm2.b"] = (width,)
        shapes[root + "mlp.up"], shapes[root + "mlp.up.b"] = (mlp["ff"], width), (mlp["ff"],)
        shapes[root + "mlp.down"], shapes[root + "mlp.down.b"] = (width, mlp["ff"]), (width,)
    return shapes


def random_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in); norm weights around one, their biases and the projections' biases of a size
    that shows; sinks around the scores' size; decay rates that forget over tens of tokens."""
    generator = np.random.default_rng(seed)
    tensors: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last == "b" and len(shape) == 1:
            values = 0.3 * generator.standard_normal(shape)
        elif last in ("norm", "norm1", "norm2"):
            values = 1.0 + 0.2 * generator.standard_normal(shape)
        elif last == "sink":
            values = 1.5 * generator.standard_normal(shape)
        elif last == "A_log":
            values = generator.uniform(-3.0, 0.0, shape)
        elif last == "dt_bias":
            values = generator.uniform(-2.0, 1.0, shape)
        elif last == "conv":
            values = generator.standard_normal(shape) / np.sqrt(shape[1])
        elif last == "embed":
            values = generator.standard_normal(shape)
        elif name == "loop.in":
            values = generator.standard_normal(shape) / np.sqrt(shape[1] / 2)
        elif last in ("q", "k") and ".mix." in name:
            values = 2.0 * generator.standard_normal(shape) / np.sqrt(shape[1])   # scores that spread
        else:
            values = generator.standard_normal(shape) / np.sqrt(shape[1])
        tensors[name] = torch.from_numpy(np.asarray(values)).to(torch.bfloat16)
    return tensors


def write_model(directory: Path, config: dict, seed: int) -> tuple[Path, dict[str, np.ndarray]]:
    """Writes the folder; returns it and the weights as float64 arrays (the bfloat16 values) for the plain implementation."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    tensors = random_weights(config, seed)
    (directory / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(directory / "model.safetensors", tensors)
    return directory, {name: tensor.to(torch.float64).numpy() for name, tensor in tensors.items()}
