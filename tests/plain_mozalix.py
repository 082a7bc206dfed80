"""Plain, slow restatement of the Mozalix decoder in numpy float64: whole sequences, no cache, no batching, one
function per mechanism.  It shares nothing with the engine and is what the engine's results are held against.

A model is (config, weights): ``config`` the parsed config.json, ``weights`` a dict name -> float64 array.

Notation: n tokens, d the model width; a linear map stored [out, in] is applied as ``x @ W.T``; positions count from 0.
A layer is  x += N1(mixer(x)); x += N2(ff(x))  with N(y) = y / rms(y) * (1 + w): the branches read the stream itself and
are normed on their way back into it.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# ---- elementwise pieces -------------------------------------------------------------------------------------------
def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def offset_norm(y, gain, eps):
    """The layer's norm: the tensor holds the gain's distance from one."""
    return rms_unit(y, eps) * (1.0 + gain)


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
def rotate_half(v, positions, rot):
    """v [n, heads, dim]: value i of the first dims is paired with value i + dims/2, the pair turned by the angle
    position * base^(-2 i / dims); the rest pass."""
    if not rot or not rot.get("dims"):
        return v
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = base ** (-2.0 * np.arange(half, dtype=np.float64) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = v.copy()
    lo, hi = v[..., :half], v[..., half:dims]
    out[..., :half] = lo * c - hi * s
    out[..., half:dims] = hi * c + lo * s
    return out


# ---- which keys a query sees ---------------------------------------------------------------------------------------------
def seen_chunk(n, size):
    """Keys of the query's own block of `size` positions, blocks counted from position 0."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return (j <= i) & (i // size == j // size)


def seen_window(n, size, keep_first=0):
    """The last `size` positions (the query's own among them) and the first `keep_first` of the sequence."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def seen_by(n, m, kind):
    """The mask of a mixer's configuration; without a "mask" entry every earlier key is seen."""
    mask = m.get("mask")
    if not mask:
        return seen_window(n, n)
    return seen_chunk(n, mask["size"]) if kind == "chunk" else seen_window(n, mask["size"], mask.get("keep_first", 0))


def softmax_rows(s, seen, sink=None):
    """Weights over the seen keys of every row; a sink is one more term of the sum, with no key and no value."""
    s = np.where(seen, s, -np.inf)
    top = s.max(axis=1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink)
    e = np.exp(s - top)
    total = e.sum(axis=1, keepdims=True)
    if sink is not None:
        total = total + np.exp(sink - top)
    return e / total


# ---- the mixers -----------------------------------------------------------------------------------------------------------
def chunked_sink_attention(h, w, p, m, eps):
    """Grouped heads, q and k normed per head with a shared gain and then turned, keys of the query's block only, a
    learned sink per head in the softmax's sum."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = (h @ w[p + "q"].T).reshape(n, H, dk)
    k = (h @ w[p + "k"].T).reshape(n, G, dk)
    v = (h @ w[p + "v"].T).reshape(n, G, dv)
    q = rotate_half(rms_unit(q, eps) * w[p + "q.norm"], pos, m.get("rot"))
    k = rotate_half(rms_unit(k, eps) * w[p + "k.norm"], pos, m.get("rot"))
    seen = seen_by(n, m, "chunk")
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        out[:, head] = softmax_rows(s, seen, sink=w[p + "sink"][head]) @ v[:, g]
    return out.reshape(n, H * dv) @ w[p + "o"].T


def differential_lambda(w, p, m):
    return math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"]))) + m["diff"]


def differential_attention(h, w, p, m, eps):
    """Two attention maps per head over the same values, the second taken off the first with one weight for the layer;
    the difference is brought to unit root mean square per head and scaled."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = (h @ w[p + "q"].T).reshape(n, H * 2, dk)
    k = (h @ w[p + "k"].T).reshape(n, G * 2, dk)
    v = (h @ w[p + "v"].T).reshape(n, G, dv)
    q = rotate_half(rms_unit(q, eps) * w[p + "q.norm"], pos, m.get("rot"))
    k = rotate_half(rms_unit(k, eps) * w[p + "k.norm"], pos, m.get("rot"))
    seen = seen_by(n, m, "window")
    lam = differential_lambda(w, p, m)
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            s = (q[:, 2 * head + which] @ k[:, 2 * g + which].T) * m["scale"]
            maps.append(softmax_rows(s, seen) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, head] = rms_unit(o, eps) * (1.0 - m["diff"])
    return out.reshape(n, H * dv) @ w[p + "o"].T


def capped_window_attention(h, w, p, m, eps):
    """No positions; unit-rms q and k; scores squashed by cap * tanh(s / cap); the last positions and the sequence's first."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit((h @ w[p + "q"].T).reshape(n, H, dk), eps)
    k = rms_unit((h @ w[p + "k"].T).reshape(n, G, dk), eps)
    v = (h @ w[p + "v"].T).reshape(n, G, dv)
    seen = seen_by(n, m, "window")
    cap = m.get("softcap")
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        out[:, head] = softmax_rows(s, seen) @ v[:, g]
    return out.reshape(n, H * dv) @ w[p + "o"].T


def channel_gated_delta(h, w, p, m, eps):
    """The gated delta rule, token by token, with a decay per head AND key channel: per head a matrix S [dim, vdim] has its
    rows decayed, is corrected towards the token's value along the token's key, and is read with the token's query."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(n, G, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(n, G, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(n, H, dv)
    q = q / np.sqrt((q * q).sum(axis=-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)
    step = softplus((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(n, H, dk)
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * step)
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(n, H, dv)
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        S = np.zeros((dk, dv))
        for t in range(n):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms_unit(out, eps) * w[p + "norm"] * gate
    return out.reshape(n, H * dv) @ w[p + "o"].T


def side_by_side(h, w, p, m, eps):
    """Two mixers read the same rows; their outputs are summed with a weight each."""
    left = capped_window_attention(h, w, p + "left.", m["left"], eps)
    right = channel_gated_delta(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


MIXERS = {"attention": chunked_sink_attention, "attention_2": differential_attention, "parallel": side_by_side}


# ---- feed-forward ---------------------------------------------------------------------------------------------------------
def clamped_glu(h, w, p, mlp):
    """gate capped from above, up clipped on both sides; gate * sigmoid(1.702 gate) * (up + 1); every map has a bias."""
    lim = mlp["limit"]
    g = np.minimum(h @ w[p + "gate"].T + w[p + "gate.b"], lim)
    u = np.clip(h @ w[p + "up"].T + w[p + "up.b"], -lim, lim)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T + w[p + "down.b"]


# ---- the model --------------------------------------------------------------------------------------------------------------
def weights_layer(config, i):
    """The layer whose tensors layer i uses."""
    return config["layers"][i].get("weights_of", i)


def forward(config, w, tokens, return_layers=False):
    """Logits [n, vocab] of a whole sequence (and the stream after every layer)."""
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    streams = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{weights_layer(config, i)}."
        y = MIXERS[layer["type"]](x, w, p + "mix.", layer["mixer"], eps)
        x = x + offset_norm(y, w[p + "norm1"], eps)
        if layer.get("mlp"):
            y = clamped_glu(x, w, p + "mlp.", layer["mlp"])
            x = x + offset_norm(y, w[p + "norm2"], eps)
        streams.append(x.copy())
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits


# ---- model folders ------------------------------------------------------------------------------------------------------
def attention_shapes(p, m, d, maps):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {p + "q": (H * maps * dk, d), p + "k": (G * maps * dk, d), p + "v": (G * dv, d), p + "o": (d, H * dv)}


def delta_shapes(p, m, d, rank):
    H, G, dk, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    ra, rg = rank if isinstance(rank, tuple) else (rank, rank)
    return {p + "q": (G * dk, d), p + "q.conv": (G * dk, K), p + "k": (G * dk, d), p + "k.conv": (G * dk, K), p + "v": (H * dv, d),
            p + "v.conv": (H * dv, K), p + "b": (H, d), p + "A_log": (H,), p + "norm": (dv,), p + "a1": (ra, d), p + "a2": (H * dk, ra),
            p + "dt_bias": (H * dk,), p + "g1": (rg, d), p + "g2": (H * dv, rg), p + "o": (d, H * dv)}


def tensor_shapes(config, ranks=None):
    """name -> shape of every tensor a model of this configuration has.  The inner sizes of the two-step maps of a delta
    mixer are no keys of the configuration (the tensors' shapes give them): ``ranks`` maps a layer index to one size for
    both maps or to a pair (decay map, gate map); default 8."""
    d, V = config["width"], config["vocab"]
    shapes = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    for i, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (d,)
        if layer["type"] == "attention":
            shapes.update(attention_shapes(p + "mix.", m, d, 1))
            shapes.update({p + "mix.q.norm": (m["dim"],), p + "mix.k.norm": (m["dim"],), p + "mix.sink": (m["heads"],)})
        elif layer["type"] == "attention_2":
            shapes.update(attention_shapes(p + "mix.", m, d, 2))
            for name in ("q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2"):
                shapes[p + "mix." + name] = (m["dim"],)
        else:
            shapes.update(attention_shapes(p + "mix.left.", m["left"], d, 1))
            shapes.update(delta_shapes(p + "mix.right.", m["right"], d, (ranks or {}).get(i, 8)))
        mlp = layer.get("mlp")
        if mlp:
            shapes[p + "norm2"] = (d,)
            shapes.update({p + "mlp.gate": (mlp["ff"], d), p + "mlp.gate.b": (mlp["ff"],), p + "mlp.up": (mlp["ff"], d), p + "mlp.up.b": (mlp["ff"],),
                           p + "mlp.down": (d, mlp["ff"]), p + "mlp.down.b": (d,)})
    return shapes


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def random_weights(config, seed, overrides=None, ranks=None):
    """Random weights (rounded to bfloat16, as a model file stores them) of sizes that keep activations of order one."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(config, ranks).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            v = 0.2 * rng.standard_normal(shape)                 # the gain is one plus this
        elif leaf == "norm":
            v = 1.0 + 0.2 * rng.standard_normal(shape)           # q.norm, k.norm, the delta mixer's output gain
        elif leaf == "sink":
            v = rng.standard_normal(shape)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            v = rng.standard_normal(shape) * 0.1
        elif leaf == "A_log":
            v = np.log(rng.uniform(0.3, 4.0, shape))
        elif leaf == "dt_bias":
            v = np.log(np.expm1(rng.uniform(0.01, 0.5, shape)))
        elif leaf == "conv":
            v = rng.standard_normal(shape) * 0.5
        elif leaf == "b" and name.split(".")[-2] in ("gate", "up", "down"):
            v = rng.standard_normal(shape) * 0.2
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            v = rng.standard_normal(shape) * (1.5 / math.sqrt(shape[-1]))
        w[name] = from_bf16_bits(to_bf16_bits(v)).astype(np.float64)
    for name, v in (overrides or {}).items():
        w[name] = from_bf16_bits(to_bf16_bits(v)).astype(np.float64)
    return w


def write_model_dir(folder, config, w):
    """config.json and model.safetensors (bfloat16) as the engine reads them."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    header, blobs, at = {}, [], 0
    for name in sorted(w):
        raw = to_bf16_bits(w[name]).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(w[name].shape), "data_offsets": [at, at + len(raw)]}
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
