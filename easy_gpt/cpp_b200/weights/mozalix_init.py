"""Random-weights mode for the Mozalix decoder: the names and shapes of the tensors a configuration asks for, and a
writer of a model folder (config.json, model.safetensors in bfloat16) from a configuration and a seed.

Made for models of several gigabytes: matrices are cut out of one pool of random bfloat16 values at offsets drawn
per tensor, so a folder is written at the speed of the disk.  Constants that must be sane for the model to run
(norm gains, the decays' logarithms, the step sizes' biases) get values of their own.  A layer with "weights_of" has no
tensors.  The inner size of a delta mixer's low-rank maps is its entry's "rank" (default 64).  numpy only.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


def _attention(shapes, p, m, d, maps):
    heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    shapes.update({p + "q": (heads * maps * dk, d), p + "k": (groups * maps * dk, d), p + "v": (groups * dv, d), p + "o": (d, heads * dv)})


def tensor_shapes(config: dict) -> dict:
    d, vocab = config["width"], config["vocab"]
    shapes = {"embed": (vocab, d), "final.norm": (d,), "head": (vocab, d)}
    for i, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (d,)
        if layer["type"] == "attention":
            _attention(shapes, p + "mix.", m, d, 1)
            shapes.update({p + "mix.q.norm": (m["dim"],), p + "mix.k.norm": (m["dim"],), p + "mix.sink": (m["heads"],)})
        elif layer["type"] == "attention_2":
            _attention(shapes, p + "mix.", m, d, 2)
            for name in ("q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2"):
                shapes[p + "mix." + name] = (m["dim"],)
        elif layer["type"] == "parallel":
            _attention(shapes, p + "mix.left.", m["left"], d, 1)
            r, q = m["right"], p + "mix.right."
            heads, groups, dk, dv, taps, rank = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"], r.get("rank", 64)
            shapes.update({q + "q": (groups * dk, d), q + "q.conv": (groups * dk, taps), q + "k": (groups * dk, d), q + "k.conv": (groups * dk, taps),
                           q + "v": (heads * dv, d), q + "v.conv": (heads * dv, taps), q + "b": (heads, d), q + "A_log": (heads,), q + "norm": (dv,),
                           q + "a1": (rank, d), q + "a2": (heads * dk, rank), q + "dt_bias": (heads * dk,), q + "g1": (rank, d), q + "g2": (heads * dv, rank),
                           q + "o": (d, heads * dv)})
        else:
            raise ValueError(f"layers[{i}].type '{layer['type']}' is no mixer of this design")
        mlp = layer.get("mlp")
        if mlp:
            ff = mlp["ff"]
            shapes[p + "norm2"] = (d,)
            shapes.update({p + "mlp.gate": (ff, d), p + "mlp.gate.b": (ff,), p + "mlp.up": (ff, d), p + "mlp.up.b": (ff,), p + "mlp.down": (d, ff),
                           p + "mlp.down.b": (d,)})
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
        if leaf in ("norm1", "norm2") or name == "final.norm" or leaf == "sink":
            return _bf16_bits(np.zeros(n))                                       # the gain is one plus the tensor; a sink of exp(0)
        if leaf == "norm":
            return _bf16_bits(np.ones(n))
        if leaf == "A_log":
            return _bf16_bits(np.log(rng.uniform(1.0, 16.0, n)))
        if leaf == "dt_bias":
            return _bf16_bits(np.log(np.expm1(rng.uniform(1e-3, 1e-1, n))))      # step sizes between 1e-3 and 1e-1 at zero input
        if leaf == "conv":
            return _bf16_bits(rng.standard_normal(n) * 0.3)
        if leaf in ("lq1", "lk1", "lq2", "lk2"):
            return _bf16_bits(rng.standard_normal(n) * 0.1)
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
