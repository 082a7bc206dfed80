"""Random-weights mode for the Masezen decoder: the names and shapes of the tensors a configuration asks for, and a
writer of a model folder (config.json, model.safetensors in bfloat16) from a configuration and a seed.

Made for models of several gigabytes: matrices are cut out of one pool of random bfloat16 values at offsets drawn
per tensor, so a folder is written at the speed of the disk.  Constants that must be sane for the model to run
(the norms' single gains, the branches' gains per channel, the query and key weights, the mix of the heads near the
identity, small convolution taps) get values of their own.  numpy only.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


def tensor_shapes(config: dict) -> dict:
    d, vocab, count = config["width"], config["vocab"], len(config["layers"])
    side = (config.get("token_side") or {}).get("dim", 0)
    taps = (config.get("canon") or {}).get("taps", 0)
    shapes = {"embed": (vocab, d), "final.norm": (), "head": (vocab, d)}
    if side:
        shapes["side.embed"] = (vocab, count * side)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] != "attention":
            raise ValueError(f"layers[{i}].type '{layer['type']}' is no mixer of this design")
        heads, groups, dk = m["heads"], m["kv_heads"], m["dim"]
        shapes.update({p + "norm1": (), p + "ls1": (d,), p + "mix.q": (heads * dk, d), p + "mix.k": (groups * dk, d), p + "mix.g": (heads * dk, d),
                       p + "mix.o": (d, heads * dk), p + "mix.q.norm": (dk,), p + "mix.k.norm": (dk,), p + "mix.talk": (heads, heads)})
        if taps:
            shapes[p + "canon1"] = (d, taps)
        if side:
            shapes.update({p + "side.gate": (side, d), p + "side.proj": (d, side), p + "side.norm": (d,)})
        mlp = layer.get("mlp")
        if not mlp:
            continue
        shapes[p + "ls2"] = (d,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        elif mlp["kind"] == "moe":
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], d)
            groups_ = [(f"e{e}", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                groups_.append(("shared", mlp["shared"]["ff"]))
            for name, ff in groups_:
                shapes.update({f"{p}mlp.{name}.gate": (ff, d), f"{p}mlp.{name}.up": (ff, d), f"{p}mlp.{name}.down": (d, ff)})
        else:
            raise ValueError(f"layers[{i}].mlp.kind '{mlp['kind']}' is no feed-forward of this design")
    return shapes


def _bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_random_model(folder, config: dict, seed: int, std: float = 0.02) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    shapes = tensor_shapes(config)
    rng = np.random.default_rng(seed)
    pool = _bf16_bits(rng.standard_normal(1 << 24) * std)
    (folder / "config.json").write_text(json.dumps(config, indent=1))

    def values(name, shape):
        n = int(np.prod(shape))
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1", "ls1", "ls2"):
            return _bf16_bits(np.ones(n))
        if leaf == "canon1":
            return _bf16_bits(rng.standard_normal(n) * 0.3)
        if leaf == "talk":
            return _bf16_bits((np.eye(shape[0]) + rng.standard_normal(shape) * 0.1).reshape(-1))
        if name == "side.embed":
            return _bf16_bits(rng.standard_normal(n))
        out = np.empty(n, dtype=np.uint16)
        at = 0
        while at < n:
            take = min(n - at, len(pool) // 2)
            start = int(rng.integers(0, len(pool) - take))
            out[at:at + take] = pool[start:start + take]
            at += take
        return out

    header, at = {}, 0
    for name, shape in shapes.items():
        size = int(np.prod(shape)) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [at, at + size]}
        at += size
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head)
        for name, shape in shapes.items():
            f.write(values(name, shape).tobytes())
    return folder
