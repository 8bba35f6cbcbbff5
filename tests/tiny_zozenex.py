"""Small Zozenex configurations for the tests, and a writer of model folders whose tensor names and shapes are spelled
out here from the configuration (not taken from the package), with weights large enough that every mechanism matters
in the logits."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from lalamo_b200.weights.safetensors_io import write_safetensors


def retention(heads=4, dim=16, vdim=16, decay=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay or [1.0 - 2.0 ** (-2 - h) for h in range(heads)]}


def left(heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=8, base=10000.0, scale=0.25, softcap=20.0, size=24, pool=4):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "rot": {"dims": rot_dims, "base": base},
            "mask": {"size": size, "pool": pool}}


def right(heads=2, dim=16, vdim=16, tau=8.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def moe(experts=6, top=2, ff=24, scale=1.5, shared_ff=32):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}, "shared": None if shared_ff is None else {"ff": shared_ff}}


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


def model(vocab, width, layers, eps=1e-5, max_positions=2048):
    return {"architecture": "Zozenex", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps}, "layers": layers}


# A: the two kinds of layer in turn; fewer key/value heads than query heads, value heads wider and narrower than key heads,
# rotation over part of a head, a block size that divides neither the page nor the window, heads of the two branches that differ.
CONFIG_A = model(160, 64, [
    layer("retention", retention(heads=4, dim=16, vdim=24), moe(experts=6, top=2, ff=24, scale=1.5, shared_ff=32)),
    layer("parallel", {"left": left(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, base=500.0, scale=0.3, softcap=15.0, size=37, pool=5),
                       "right": right(heads=2, dim=16, vdim=8, tau=6.0)}, moe(experts=5, top=1, ff=16, scale=2.5, shared_ff=8)),
    layer("parallel", {"left": left(heads=2, kv_heads=2, dim=32, vdim=16, rot_dims=32, base=100.0, scale=0.2, softcap=8.0, size=16, pool=16),
                       "right": right(heads=4, dim=8, vdim=16, tau=2.0)}, None),
    layer("retention", retention(heads=2, dim=8, vdim=16, decay=[0.9, 0.995]), moe(experts=4, top=4, ff=40, scale=0.5, shared_ff=None)),
], eps=1e-5)

# B: sizes that fit no kernel's favourite shape, no rotation of q and k, a block longer than the window and than a page, a window of
# one, one head, one expert chosen of two.
CONFIG_B = model(131, 72, [
    layer("parallel", {"left": left(heads=3, kv_heads=3, dim=24, vdim=10, rot_dims=0, base=50.0, scale=0.5, softcap=5.0, size=9, pool=21),
                       "right": right(heads=1, dim=12, vdim=20, tau=1.0)}, moe(experts=2, top=1, ff=20, scale=1.0, shared_ff=12)),
    layer("retention", retention(heads=3, dim=12, vdim=20, decay=[0.5, 0.97, 1.0]), None),
    layer("parallel", {"left": left(heads=1, kv_heads=1, dim=12, vdim=6, rot_dims=4, base=7.0, scale=0.7, softcap=50.0, size=1, pool=2),
                       "right": right(heads=3, dim=20, vdim=12, tau=30.0)}, moe(experts=7, top=3, ff=8, scale=3.0, shared_ff=24)),
])

# C: the sizes the tensor-core kernels take (heads of 64, widths in multiples of 64), a window and blocks like a real model's in small.
CONFIG_C = model(256, 128, [
    layer("parallel", {"left": left(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, base=1000.0, scale=0.125, softcap=30.0, size=64, pool=8),
                       "right": right(heads=2, dim=64, vdim=64, tau=16.0)}, moe(experts=8, top=2, ff=64, scale=2.0, shared_ff=64)),
    layer("retention", retention(heads=2, dim=64, vdim=128), moe(experts=8, top=2, ff=64, scale=2.0, shared_ff=64)),
    layer("parallel", {"left": left(heads=4, kv_heads=4, dim=32, vdim=64, rot_dims=32, base=5e5, scale=0.2, softcap=25.0, size=80, pool=10),
                       "right": right(heads=2, dim=32, vdim=64, tau=12.0)}, None),
])

# D, E, F, G: one layer each without a feed-forward (the mixers alone), and a feed-forward behind the smallest mixer.
CONFIG_D = model(96, 64, [layer("retention", retention(heads=4, dim=16, vdim=8, decay=[0.8, 0.9, 0.99, 0.999]), None)])
CONFIG_E = model(96, 64, [layer("parallel", {"left": left(heads=4, kv_heads=1, dim=16, vdim=12, rot_dims=10, base=300.0, scale=0.4, softcap=10.0, size=20, pool=3),
                                             "right": right(heads=2, dim=8, vdim=8, tau=4.0)}, None)])
CONFIG_F = model(96, 64, [layer("retention", retention(heads=1, dim=8, vdim=8, decay=[0.9]), moe(experts=9, top=3, ff=24, scale=2.0, shared_ff=16))])

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D, "E": CONFIG_E, "F": CONFIG_F}

DECAY_RANK = {"A": 6, "B": 3, "C": 16, "D": 4, "E": 5, "F": 4}   # of the right branch's bottleneck: only the tensors' shapes say it


def tensor_shapes(config: dict, rank: int) -> dict[str, tuple[int, ...]]:
    width = config["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (config["vocab"], width), "pos": (config["max_positions"], width), "final.norm": (width,),
                                          "head": (config["vocab"], width)}
    for index, entry in enumerate(config["layers"]):
        root = f"l{index}."
        shapes[root + "norm1"] = (width,)
        mix, p = entry["mixer"], root + "mix."
        if entry["type"] == "retention":
            shapes[p + "q"] = shapes[p + "k"] = (mix["heads"] * mix["dim"], width)
            shapes[p + "v"] = shapes[p + "g"] = (mix["heads"] * mix["vdim"], width)
            shapes[p + "o"] = (width, mix["heads"] * mix["vdim"])
        else:
            a, b = mix["left"], mix["right"]
            shapes[p + "left.q"] = (a["heads"] * a["dim"], width)
            shapes[p + "left.k"] = (a["kv_heads"] * a["dim"], width)
            shapes[p + "left.v"] = (a["kv_heads"] * a["vdim"], width)
            shapes[p + "left.pb"] = (a["heads"],)
            shapes[p + "left.o"] = (width, a["heads"] * a["vdim"])
            shapes[p + "right.q"] = shapes[p + "right.k"] = (b["heads"] * b["dim"], width)
            shapes[p + "right.v"] = shapes[p + "right.g"] = (b["heads"] * b["vdim"], width)
            shapes[p + "right.o"] = (width, b["heads"] * b["vdim"])
            shapes[p + "right.norm"] = (b["vdim"],)
            shapes[p + "right.a1"] = (rank, width)
            shapes[p + "right.a2"] = (b["heads"] * b["dim"], rank)
            shapes[p + "right.a2.b"] = (b["heads"] * b["dim"],)
            shapes[p + "left.out"] = shapes[p + "right.out"] = (width,)
        mlp = entry["mlp"]
        if mlp is None:
            continue
        shapes[root + "norm2"] = (width,)
        m = root + "mlp."
        for e in range(mlp["router"]["experts"]):
            shapes[m + f"e{e}.up"] = (mlp["expert"]["ff"], width)
            shapes[m + f"e{e}.down"] = (width, mlp["expert"]["ff"])
        shapes[m + "router"] = (mlp["router"]["experts"], width)
        shapes[m + "correction"] = (mlp["router"]["experts"],)
        if mlp["shared"] is not None:
            shapes[m + "shared.up"] = (mlp["shared"]["ff"], width)
            shapes[m + "shared.down"] = (width, mlp["shared"]["ff"])
            shapes[m + "shared.sg"] = (1, width)
    return shapes


def random_weights(config: dict, seed: int, rank: int, sharp: bool = False) -> dict[str, torch.Tensor]:
    """bfloat16 tensors: matrices N(0, 1/in); norm weights around one; per-head biases of the sigmoid weights below zero, so that few
    keys weigh much (``sharp``: far below, with scores that spread over tens of units: single keys decide); decay logits that forget
    over tens of tokens; corrections of the size of the differences between scores."""
    generator = np.random.default_rng(seed)
    tensors: dict[str, torch.Tensor] = {}
    for name, shape in tensor_shapes(config, rank).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2", "out"):
            values = 1.0 + 0.2 * generator.standard_normal(shape)
        elif last == "pb":
            values = (-14.0 if sharp else -2.0) + 0.5 * generator.standard_normal(shape)
        elif name.endswith("a2.b"):
            values = 3.0 + generator.standard_normal(shape)
        elif last == "correction":
            values = 0.3 * generator.standard_normal(shape)
        elif last in ("embed", "pos"):
            values = generator.standard_normal(shape) * (1.0 if last == "embed" else 0.5)
        elif last == "router":
            values = 3.0 * generator.standard_normal(shape) / np.sqrt(shape[1])
        elif last in ("q", "k") and ".left." in name:
            values = (6.0 if sharp else 2.0) * generator.standard_normal(shape) / np.sqrt(shape[1])   # scores that spread
        else:
            values = generator.standard_normal(shape) / np.sqrt(shape[-1])
        tensors[name] = torch.from_numpy(np.asarray(values)).to(torch.bfloat16)
    return tensors


def write_model(directory: Path, config: dict, seed: int, rank: int = 4, sharp: bool = False) -> tuple[Path, dict[str, torch.Tensor]]:
    """Writes the folder; returns it and the weights in float64 (the bfloat16 values) for the plain implementation."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    tensors = random_weights(config, seed, rank, sharp)
    (directory / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(directory / "model.safetensors", tensors)
    return directory, {name: tensor.to(torch.float64) for name, tensor in tensors.items()}
