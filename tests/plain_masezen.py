"""Plain, slow restatement of the Masezen decoder in numpy float64: whole sequences, no cache, no batching, one
function per mechanism.  It shares nothing with the engine and is what the engine's results are held against.

A model is (config, weights): ``config`` the parsed config.json, ``weights`` a dict name -> float64 array.

Notation: n tokens, d the model width; a linear map stored [out, in] is applied as ``x @ W.T``; positions count from 0.

The layer:  h = g1 * unit(x);  x' = x + s1 * mixer(h + conv(h)) + s2 * ff(h);  x'' = x' + side(x', token), with g1 ONE
number, s1 and s2 vectors of the width, conv a causal convolution over time on each channel, and side a small gated
map of a per-token vector that every layer has a slice of.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# ---- elementwise pieces -------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def causal_conv(x, taps_w):
    """x [n, channels], taps_w [channels, taps]; the last column weighs the current token, zeros before the start."""
    n, c = x.shape
    k = taps_w.shape[1]
    padded = np.vstack([np.zeros((k - 1, c)), x])
    out = np.zeros((n, c))
    for j in range(k):
        out += padded[j:j + n] * taps_w[:, j]
    return out


# ---- rotation -------------------------------------------------------------------------------------------------------------
def rotation_frequencies(rot):
    """Angular frequency of each of the dims/2 pairs, and the factor on cos and sin."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def turn(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(sc["fast"])), 0)
    hi = min(math.ceil(turn(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(v, positions, rot):
    """v [n, heads, dim]: value i of the first dims is paired with value i + dims/2; the rest pass."""
    if not rot or not rot.get("dims"):
        return v
    dims = rot["dims"]
    f, m = rotation_frequencies(rot)
    a = positions[:, None].astype(np.float64) * f[None, :]
    cos, sin = (np.cos(a) * m)[:, None, :], (np.sin(a) * m)[:, None, :]
    out = v.copy()
    u, w = v[..., :dims // 2], v[..., dims // 2:dims]
    out[..., :dims // 2] = u * cos - w * sin
    out[..., dims // 2:dims] = w * cos + u * sin
    return out


# ---- the mixer --------------------------------------------------------------------------------------------------------------
def mixed_head_attention(h, w, p, m, eps, positions=None):
    """Grouped-query attention whose values are the projected keys themselves, whose queries and keys are normed per
    head before they are turned, whose scores are mixed across the heads before the softmax, and whose output is gated."""
    n = h.shape[0]
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(n) if positions is None else positions
    q = (h @ w[p + "q"].T).reshape(n, H, dk)
    k = (h @ w[p + "k"].T).reshape(n, G, dk)
    v = k.copy()                                          # as projected: no norm, no turn
    q = rotate_half(rms_unit(q, eps) * w[p + "q.norm"], pos, m.get("rot"))
    k = rotate_half(rms_unit(k, eps) * w[p + "k.norm"], pos, m.get("rot"))
    s = np.zeros((H, n, n))
    for head in range(H):
        s[head] = (q[:, head] @ k[:, head // (H // G)].T) * m["scale"]
    s = np.einsum("hg,gij->hij", w[p + "talk"], s)         # every head's score is a mix of all heads' scores
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    s = np.where((j <= i)[None], s, -np.inf)
    e = np.exp(s - s.max(axis=2, keepdims=True))
    a = e / e.sum(axis=2, keepdims=True)
    out = np.zeros((n, H, dk))
    for head in range(H):
        out[:, head] = a[head] @ v[:, head // (H // G)]
    return (out.reshape(n, H * dk) * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---- feed-forwards ------------------------------------------------------------------------------------------------------------
def squared_relu_ff(h, w, p):
    z = np.maximum(h @ w[p + "up"].T, 0.0)
    return (z * z) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    """down(g sigmoid(1.702 g) (u + 1)) with g = min(gate h, limit) and u = clamp(up h, -limit, limit)."""
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def routed_ff(h, w, p, mlp):
    """The `top` experts with the largest sigmoid(router h) each get the row TIMES that score as their input; a shared
    expert, if there is one, gets the row itself."""
    n = h.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = sigmoid(h @ w[p + "router"].T)
    out = np.zeros((n, w[p + "e0.down"].shape[0]))
    for t in range(n):
        for e in np.argsort(-s[t], kind="stable")[:top]:
            out[t] += clamped_expert(s[t, e] * h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return squared_relu_ff(h, w, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, w, p, mlp)
    raise ValueError(mlp["kind"])


# ---- the per-layer token input ---------------------------------------------------------------------------------------------
def token_side(x, tokens, w, p, layer, dim, eps):
    """A vector per token and layer, gated by the stream, mapped to the width and normed with a gain."""
    e = w["side.embed"][np.asarray(tokens), layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms_unit(y, eps) * w[p + "norm"]


# ---- the model ---------------------------------------------------------------------------------------------------------------
def layer_forward(config, w, i, x, tokens, positions=None):
    eps = config["norm"]["eps"]
    layer, p = config["layers"][i], f"l{i}."
    h = rms_unit(x, eps) * w[p + "norm1"]
    if layer["type"] != "attention":
        raise ValueError(layer["type"])
    branch = mixed_head_attention(h + causal_conv(h, w[p + "canon1"]), w, p + "mix.", layer["mixer"], eps, positions) * w[p + "ls1"]
    if layer.get("mlp"):
        branch = branch + feed_forward(h, w, p + "mlp.", layer["mlp"]) * w[p + "ls2"]
    x = x + branch
    return x + token_side(x, tokens, w, p + "side.", i, config["token_side"]["dim"], eps)


def forward(config, w, tokens, return_layers=False):
    """Logits [n, vocab] of a whole sequence (and the stream after every layer)."""
    x = w["embed"][np.asarray(tokens)]
    streams = []
    for i in range(len(config["layers"])):
        x = layer_forward(config, w, i, x, tokens)
        streams.append(x.copy())
    logits = (rms_unit(x, config["norm"]["eps"]) * w["final.norm"]) @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits


# ---- model folders ------------------------------------------------------------------------------------------------------
def tensor_shapes(config):
    """name -> shape of every tensor a model of this configuration has."""
    d, V, L, sd = config["width"], config["vocab"], len(config["layers"]), config["token_side"]["dim"]
    shapes = {"embed": (V, d), "side.embed": (V, L * sd), "final.norm": (), "head": (V, d)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, dk = m["heads"], m["kv_heads"], m["dim"]
        shapes.update({p + "norm1": (), p + "ls1": (d,), p + "canon1": (d, config["canon"]["taps"]),
                       p + "mix.q": (H * dk, d), p + "mix.k": (G * dk, d), p + "mix.q.norm": (dk,), p + "mix.k.norm": (dk,), p + "mix.talk": (H, H),
                       p + "mix.g": (H * dk, d), p + "mix.o": (d, H * dk),
                       p + "side.gate": (sd, d), p + "side.proj": (d, sd), p + "side.norm": (d,)})
        mlp = layer.get("mlp")
        if not mlp:
            continue
        shapes[p + "ls2"] = (d,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        else:
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], d)
            groups = [(f"e{e}", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                groups.append(("shared", mlp["shared"]["ff"]))
            for name, ff in groups:
                shapes.update({f"{p}mlp.{name}.gate": (ff, d), f"{p}mlp.{name}.up": (ff, d), f"{p}mlp.{name}.down": (d, ff)})
    return shapes


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def random_weights(config, seed, overrides=None):
    """Random weights (rounded to bfloat16, as a model file stores them) of sizes that keep activations of order one."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if leaf == "norm1" or name == "final.norm" or name.endswith("q.norm") or name.endswith("k.norm"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith("side.norm"):
            v = 0.3 + 0.1 * rng.standard_normal(shape)
        elif leaf in ("ls1", "ls2"):
            v = 0.7 + 0.3 * rng.standard_normal(shape)
        elif leaf == "canon1":
            v = rng.standard_normal(shape) * 0.4
        elif leaf == "talk":
            v = np.eye(shape[0]) + rng.standard_normal(shape) * 0.4
        elif name == "embed":
            v = rng.standard_normal(shape) * 0.5
        elif name == "side.embed":
            v = rng.standard_normal(shape)
        elif leaf == "router":
            v = rng.standard_normal(shape) * (3.0 / math.sqrt(shape[-1]))
        else:
            v = rng.standard_normal(shape) * (1.5 / math.sqrt(shape[-1]))
        w[name] = from_bf16_bits(to_bf16_bits(v)).astype(np.float64).reshape(shape)
    for name, v in (overrides or {}).items():
        w[name] = from_bf16_bits(to_bf16_bits(v)).astype(np.float64).reshape(np.shape(v))
    return w


def write_model_dir(folder, config, w):
    """config.json and model.safetensors (bfloat16) as the engine reads them."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    header, blobs, at = {}, [], 0
    for name in sorted(w):
        raw = to_bf16_bits(w[name]).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(np.shape(w[name])), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder


def read_model_dir(folder):
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    w = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = raw[8 + n + lo:8 + n + hi]
        if meta["dtype"] == "BF16":
            a = from_bf16_bits(np.frombuffer(buf, dtype=np.uint16))
        elif meta["dtype"] == "F32":
            a = np.frombuffer(buf, dtype=np.float32)
        else:
            a = np.frombuffer(buf, dtype=np.int32)
        w[name] = a.reshape(meta["shape"]).astype(np.float64)
    return config, w
