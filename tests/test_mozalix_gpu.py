"""The Mozalix decoder in the native engine against the plain numpy restatement (tests/plain_mozalix.py): each mechanism
alone, prompts cut in every way, batches, reused pages and slots, the edges of every mask, far keys, long decoding, odd
sizes, generation.

Every test makes its own small configuration and random weights.  Errors are the largest difference of a logit over
the largest logit: float32 must stay within 1e-4.  In bfloat16 every branch's input and output is rounded to eight bits
of mantissa before it joins the stream: there the bound is 3e-2 on the root mean square of all differences (over the root
mean square of the logits) and 8e-2 on the largest one; the faults that the pointed tests plant move logits by far more.
"""
import copy
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_mozalix as pm

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
LARGEST = {"float32": 1e-4, "bfloat16": 8e-2}


def sizes(heads, kv_heads, dim, vdim, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}


def chunked(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size=20, rot_dims=8, base=10000.0):
    m = sizes(heads, kv_heads, dim, vdim, scale)
    if size:
        m["mask"] = {"size": size}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": m}


def two_maps(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size=20, rot_dims=4, base=5000.0, diff=0.35):
    m = dict(sizes(heads, kv_heads, dim, vdim, scale), diff=diff)
    if size:
        m["mask"] = {"size": size}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention_2", "mixer": m}


def side(left=None, right=None, left_scale=0.8, right_scale=1.3, size=24, keep_first=5, softcap=15.0):
    l = dict(sizes(*(left or (4, 2, 16, 24, 0.3))))
    if size:
        l["mask"] = {"size": size, "keep_first": keep_first} if keep_first is not None else {"size": size}
    if softcap:
        l["softcap"] = softcap
    heads, kv_heads, dim, vdim, conv = right or (4, 2, 16, 24, 4)
    r = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}}


def model(layers, width=64, vocab=131, eps=1e-5, embedding_scale=0.7, limit=2.5):
    """layers: (mixer entry, ff or None) or ("same", j) for a layer that runs layer j's tensors."""
    cfg = {"architecture": "Mozalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": []}
    for mixer, ff in layers:
        if mixer == "same":
            cfg["layers"].append({**copy.deepcopy(cfg["layers"][ff]), "weights_of": cfg["layers"][ff].get("weights_of", ff)})
        else:
            cfg["layers"].append({**copy.deepcopy(mixer), "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None})
    if embedding_scale:
        cfg["embedding"] = {"scale": embedding_scale}
    return cfg


GENERAL = model([(two_maps(), 96), (side(), 80), (chunked(heads=3, kv_heads=1, dim=8, vdim=8, scale=0.5, size=33, rot_dims=8), None), ("same", 1), ("same", 0),
                 (side(left=(2, 1, 24, 8, 0.2), right=(2, 2, 24, 8, 3), size=9, keep_first=11, softcap=None), 48)])
GENERAL_RANKS = {1: (5, 12), 5: 3}
# keys and values of one size (32, 64, 128): in bfloat16 the attention then runs on the tiled tensor-core kernel, prompt portions and single tokens alike
TENSOR = model([(two_maps(heads=4, kv_heads=2, dim=32, vdim=32, size=20, rot_dims=16), 96), (side(left=(4, 2, 64, 64, 0.2), right=(2, 1, 32, 64, 4), size=24, keep_first=5), 80),
                (chunked(heads=4, kv_heads=1, dim=128, vdim=128, scale=0.09, size=33, rot_dims=64), None), ("same", 1), ("same", 0)], width=128)
BOTH = {"general": GENERAL, "tensor": TENSOR}
# widths that leave the decode product's alignment rule, head sizes that are no powers of two, two taps, a rotation over part of an odd-sized head
ODD = model([(side(left=(3, 3, 12, 10, 0.4), right=(3, 1, 20, 10, 2), size=7, keep_first=3), 52), (chunked(heads=3, kv_heads=3, dim=12, vdim=10, scale=0.4, size=7, rot_dims=6, base=300.0), 36),
             (two_maps(heads=3, kv_heads=1, dim=10, vdim=6, scale=0.4, size=9, rot_dims=10, diff=0.2), None)], width=72, vocab=77, embedding_scale=None)
# values that are one or equal: one head, one key head, one tap (no convolution state), masks of one position (a token sees itself, the sink and
# the kept first token), inner sizes of one, equal key and value sizes, the whole head rotated, scales of one
ONES = model([(side(left=(1, 1, 16, 16, 1.0), right=(1, 1, 16, 16, 1), left_scale=1.0, right_scale=1.0, size=1, keep_first=1, softcap=1.0), None),
              (chunked(heads=1, kv_heads=1, dim=16, vdim=16, scale=1.0, size=1, rot_dims=16), 32),
              (two_maps(heads=1, kv_heads=1, dim=8, vdim=8, scale=0.7, size=1, rot_dims=None, diff=0.5), None), ("same", 2)], width=48, vocab=64, embedding_scale=None)
ONES_RANKS = {0: 1}

ALONE = {
    "chunked": model([(chunked(), None)]),
    "chunked_all_keys": model([(chunked(size=None), None)]),
    "chunked_no_rotation": model([(chunked(rot_dims=None), None)]),
    "chunked_wide": model([(chunked(heads=8, kv_heads=2, dim=64, vdim=48, scale=0.11, size=40, rot_dims=24, base=5e5), None)], width=128),
    "chunked_planes": model([(chunked(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=48, rot_dims=32), None)], width=128),
    "chunked_large_values": model([(chunked(heads=2, kv_heads=1, dim=24, vdim=136, scale=0.25, size=50), None)]),
    "two_maps": model([(two_maps(), None)]),
    "two_maps_all_keys": model([(two_maps(size=None, rot_dims=None), None)]),
    "two_maps_wide": model([(two_maps(heads=6, kv_heads=3, dim=64, vdim=128, scale=0.11, size=40, rot_dims=16, diff=0.8), None)], width=128),
    "two_maps_equal_sizes": model([(two_maps(heads=2, kv_heads=2, dim=32, vdim=32, scale=0.2, size=17, rot_dims=32, diff=0.1), None)]),
    "two_maps_planes_64": model([(two_maps(heads=6, kv_heads=2, dim=64, vdim=64, scale=0.12, size=70, rot_dims=24, diff=0.45), None)], width=128),
    "two_maps_planes_128": model([(two_maps(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, size=None, rot_dims=64, diff=0.3), None)], width=128),
    "side_planes_128": model([(side(left=(2, 1, 128, 128, 0.09), right=(2, 2, 64, 64, 3), size=65, keep_first=70, softcap=4.0), None)], width=128),
    "side_planes_32": model([(side(left=(6, 3, 32, 32, 0.2), right=(2, 1, 16, 16, 2), size=33, keep_first=1, softcap=None), 64)]),
    "side": model([(side(), None)]),
    "side_all_keys": model([(side(size=None, keep_first=None), None)]),
    "side_no_first": model([(side(keep_first=None), None)]),
    "side_first_longer_than_window": model([(side(size=6, keep_first=21), None)]),
    "side_wide": model([(side(left=(8, 2, 64, 64, 0.11), right=(4, 2, 128, 64, 4), size=40, keep_first=17), None)], width=128),
    "side_long_keys": model([(side(left=(2, 1, 40, 200, 0.2), right=(2, 1, 200, 40, 5), softcap=3.0), None)]),
    "side_many_values": model([(side(left=(2, 2, 8, 8, 0.5), right=(2, 2, 40, 200, 2)), None)]),
    # a width that is no multiple of four, sizes that are no multiples of four either
    "odd_width": model([(chunked(heads=3, kv_heads=1, dim=10, vdim=6, scale=0.4, size=9, rot_dims=4), 27), (side(left=(2, 1, 6, 10, 0.4), right=(2, 1, 6, 10, 3)), None)],
                       width=90, vocab=53),
    "feed_forward": model([(chunked(heads=2, kv_heads=2, dim=8, vdim=8), 100)], limit=0.6),
    "shared_tensors": model([(side(), 40), (two_maps(), None), ("same", 0), ("same", 1), ("same", 2)]),
}
RANKS = {"general": GENERAL_RANKS, "ones": ONES_RANKS, "side_wide": {0: (24, 40)}, "side": {0: (16, 7)}, "tensor": {1: (9, 16)}}


def tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg, seed=0, overrides=None):
        if name not in made:
            w = pm.random_weights(cfg, seed, overrides, ranks=RANKS.get(name))
            made[name] = (pm.write_model_dir(tmp_path_factory.mktemp(name), cfg, w), cfg, w)
        return made[name]

    return get


def runner(folder, dtype, pool_tokens=512, page_size=16, slots=4, graphs=True, most_tokens=None):
    from easy_gpt.cpp_b200.native import NativeStepRunner

    return NativeStepRunner(folder, dtype, page_size=page_size, num_pages=pool_tokens // page_size, max_slots=slots,
                            max_tokens_per_request=most_tokens or pool_tokens, use_graphs=graphs)


def close(got, want, dtype, what=""):
    diff = np.asarray(got, dtype=np.float64) - want
    largest = float(np.abs(diff).max() / np.abs(want).max())
    assert largest <= LARGEST[dtype], f"{what}: largest error {largest:.3g} over {LARGEST[dtype]:.3g}"
    spread = float(np.sqrt((diff * diff).mean()) / np.sqrt((want * want).mean()))
    assert spread <= TOL[dtype] or dtype == "float32", f"{what}: error {spread:.3g} over {TOL[dtype]:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(folders, name, dtype):
    folder, cfg, w = folders(name, ALONE[name], seed=3)
    toks = tokens(cfg["vocab"], 75, 1)
    got = runner(folder, dtype).run([("a", toks, list(range(75)))])
    close(got, pm.forward(cfg, w, toks), dtype, name)


def test_the_restatement_itself():
    """The restatement's own pieces against each other: a layer that runs another's tensors names them; the stream comes out
    after every layer; the masks are what their names say."""
    cfg = GENERAL
    assert [pm.weights_layer(cfg, i) for i in range(6)] == [0, 1, 2, 1, 0, 5]
    w = pm.random_weights(cfg, 1, ranks=GENERAL_RANKS)
    assert "l3.norm1" not in w and w["l1.mix.right.a1"].shape == (5, 64) and w["l1.mix.right.g2"].shape == (4 * 24, 12)
    logits, streams = pm.forward(cfg, w, tokens(cfg["vocab"], 9, 0), return_layers=True)
    assert streams.shape == (6, 9, cfg["width"]) and logits.shape == (9, cfg["vocab"])
    assert pm.seen_chunk(7, 3).astype(int).tolist()[4] == [0, 0, 0, 1, 1, 0, 0] and pm.seen_chunk(7, 3).astype(int).tolist()[6] == [0, 0, 0, 0, 0, 0, 1]
    assert pm.seen_window(7, 3, 2).astype(int).tolist()[6] == [1, 1, 0, 0, 1, 1, 1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("general", GENERAL), ("odd", ODD), ("ones", ONES), ("alone_chunked_wide", None), ("alone_two_maps_wide", None),
                                      ("alone_side_wide", None), ("alone_side_long_keys", None), ("alone_side_many_values", None), ("alone_chunked_planes", None),
                                      ("alone_side_first_longer_than_window", None), ("alone_odd_width", None), ("alone_shared_tensors", None), ("tensor", TENSOR),
                                      ("alone_two_maps_planes_64", None), ("alone_two_maps_planes_128", None), ("alone_side_planes_128", None), ("alone_side_planes_32", None)])
def test_prompt_whole_and_token_by_token(folders, name, cfg, dtype):
    if cfg is None:
        name = name[len("alone_"):]
        cfg = ALONE[name]
    folder, cfg, w = folders(name, cfg, seed=3 if name in ALONE else 5)
    toks = tokens(cfg["vocab"], 70, 2)
    want = pm.forward(cfg, w, toks)
    r = runner(folder, dtype)
    close(r.run([("whole", toks, list(range(70)))]), want, dtype, "whole")
    r.end("whole")
    rows = [r.run([("single", [t], [0])])[0] for t in toks]
    close(np.stack(rows), want, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cuts", [[2] * 20, [3, 1, 2, 17, 1, 1, 30, 5, 2, 2, 16, 15, 1, 33], [16, 16, 16, 16, 1, 15, 48], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]])
@pytest.mark.parametrize("which", sorted(BOTH))
def test_portions(folders, cuts, dtype, which):
    """Portions down to two tokens, shorter than the convolution's reach, than the windows, the chunks and the kept first tokens,
    ending on and beside page borders."""
    folder, cfg, w = folders(which, BOTH[which], seed=5)
    toks = tokens(cfg["vocab"], sum(cuts), 7)
    want = pm.forward(cfg, w, toks)
    r = runner(folder, dtype, page_size=16)
    at, rows = 0, []
    for n in cuts:
        rows.append(r.run([("p", toks[at:at + n], list(range(n)))]))
        at += n
    close(np.concatenate(rows), want, dtype, f"portions {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(BOTH))
def test_batches_of_unequal_requests(folders, dtype, which):
    """Four requests of different lengths advance together, portions beside single tokens; each must come out as alone."""
    folder, cfg, w = folders(which, BOTH[which], seed=5)
    lengths = {"a": 61, "b": 9, "c": 130, "d": 33}
    toks = {k: tokens(cfg["vocab"], n, 10 + i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: pm.forward(cfg, w, v) for k, v in toks.items()}
    plans = {"a": [40] + [1] * 21, "b": [1] * 9, "c": [2, 64, 31, 1, 1, 30, 1], "d": [16, 17]}
    r = runner(folder, dtype, pool_tokens=512)
    at = {k: 0 for k in toks}
    got = {k: [] for k in toks}
    step = 0
    while any(plans.values()):
        entries, names = [], []
        for k in sorted(plans):
            if plans[k] and (step % 3 != 2 or k != "b"):            # b sits out every third step
                n = plans[k].pop(0)
                entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
                names.append((k, n))
                at[k] += n
        if entries:
            out = r.run(entries)
            row = 0
            for k, n in names:
                got[k].append(out[row:row + n])
                row += n
        step += 1
    for k in toks:
        close(np.concatenate(got[k]), want[k], dtype, f"request {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(BOTH))
def test_pages_and_slots_are_used_again(folders, dtype, which):
    """Two slots and a pool of four pages: every request takes a slot (convolution inputs, delta states) and pages that
    another one has left full."""
    folder, cfg, w = folders(which, BOTH[which], seed=5)
    r = runner(folder, dtype, pool_tokens=64, page_size=16, slots=2)
    for i in range(6):
        a, b = tokens(cfg["vocab"], 20 + i, 40 + i), tokens(cfg["vocab"], 31 - i, 60 + i)
        out = r.run([(f"a{i}", a[:7], []), (f"b{i}", b, [len(b) - 1])])
        close(out, pm.forward(cfg, w, b)[-1:], dtype, f"b{i}")
        r.end(f"b{i}")
        out = r.run([(f"a{i}", a[7:], list(range(len(a) - 7)))])
        close(out, pm.forward(cfg, w, a)[7:], dtype, f"a{i}")
        r.end(f"a{i}")
    assert r.info("live_requests") == 0


def test_windowed_pool_holds_long_requests(folders):
    """A request far longer than the pool: windows and chunks give pages back while it runs, and the pages of the kept first
    tokens (here 21 of them: two pages) stay to the end, where they are still read."""
    cfg = model([(two_maps(size=20), 32), (side(size=18, keep_first=21), None), (chunked(heads=2, kv_heads=1, dim=8, vdim=8, size=33, rot_dims=4), None)])
    folder, cfg, w = folders("windows_only", cfg, seed=8)
    toks = tokens(cfg["vocab"], 300, 3)
    want = pm.forward(cfg, w, toks)
    r = runner(folder, "float32", pool_tokens=112, page_size=16, slots=2, most_tokens=512)
    rows, at = [], 0
    for n in [30, 17, 2, 31] + [20] * 11:
        rows.append(r.run([("long", toks[at:at + n], list(range(n)))]))
        at += n
    close(np.concatenate(rows), want, "float32", "300 tokens through seven pages")


def aimed(cfg, seed, a, b, sharp=12.0, ranks=None):
    """Weights under which one score stands out in the first layer: the key map is the query map of its group's first head
    (for two maps: of that head's first map) behind a reflection of the model's width that carries token b's embedding onto
    token a's.  Token b is then the key that token a looks for, whatever lies between them; b's value is its own.  The score
    of that pair is `sharp`, the others' a fraction of it.  Delta states hardly decay."""
    cfg = copy.deepcopy(cfg)
    base = pm.random_weights(cfg, seed, ranks=ranks)
    layer = cfg["layers"][0]
    m, p = (layer["mixer"]["left"], "l0.mix.left.") if layer["type"] == "parallel" else (layer["mixer"], "l0.mix.")
    maps = 2 if layer["type"] == "attention_2" else 1
    m["scale"] = sharp / m["dim"]
    for l in cfg["layers"]:                                       # a layer that runs the first layer's tensors has the same entry
        if l.get("weights_of") == 0:
            l["mixer"] = copy.deepcopy(layer["mixer"])
    ea, eb = base["embed"][a], base["embed"][b]
    u = ea / np.linalg.norm(ea) - eb / np.linalg.norm(eb)
    u /= np.linalg.norm(u)
    q = base[p + "q"].reshape(m["heads"], maps, m["dim"], -1)[::m["heads"] // m["kv_heads"], 0]          # [kv_heads, dim, width]
    k = base[p + "k"].reshape(m["kv_heads"], maps, m["dim"], -1).copy()
    k[:, 0] = q - 2.0 * np.einsum("gdw,w,v->gdv", q, u, u)
    over = {p + "k": k.reshape(base[p + "k"].shape)}
    for name in (p + "q.norm", p + "k.norm"):
        if name in base:
            over[name] = np.ones_like(base[name])
    for i, l in enumerate(cfg["layers"]):
        if l["type"] == "parallel" and "weights_of" not in l:
            over[f"l{i}.mix.right.A_log"] = np.log(np.full_like(base[f"l{i}.mix.right.A_log"], 2e-3))
    return cfg, over


EDGES = {
    # (first layer, where the key lies relative to the query at `end`, the same configuration with the mask moved by one)
    "window": (lambda dim: two_maps(heads=2, kv_heads=1, dim=dim, vdim=dim, size=20, rot_dims=4, diff=0.3),
               {"inside": lambda end: end - 19, "outside": lambda end: end - 20},
               lambda m, which: m["mask"].update(size=19 if which == "inside" else 21)),
    "chunk": (lambda dim: chunked(heads=2, kv_heads=1, dim=dim, vdim=dim, size=20, rot_dims=4),
              {"inside": lambda end: end // 20 * 20, "outside": lambda end: end // 20 * 20 - 1},
              lambda m, which: None),
    "kept_window": (lambda dim: side(left=(2, 1, dim, dim, 0.3), right=(2, 1, 8, 8, 3), size=20, keep_first=5, softcap=30.0 if dim == 16 else None),
                    {"inside": lambda end: end - 19, "outside": lambda end: end - 20},
                    lambda m, which: m["left"]["mask"].update(size=19 if which == "inside" else 21)),
    "kept_first": (lambda dim: side(left=(2, 1, dim, dim, 0.3), right=(2, 1, 8, 8, 3), size=20, keep_first=5, softcap=30.0 if dim == 16 else None),
                   {"inside": lambda end: 4, "outside": lambda end: 5},
                   lambda m, which: m["left"]["mask"].update(keep_first=4 if which == "inside" else 6)),
}


def with_chunks_moved(by, cfg, w, toks):
    """The restatement's logits with every chunk starting `by` positions later."""
    saved = pm.seen_chunk

    def moved(n, size):
        i, j = np.arange(n)[:, None], np.arange(n)[None, :]
        return (j <= i) & ((i - by) // size == (j - by) // size)

    pm.seen_chunk = moved
    try:
        return pm.forward(cfg, w, toks)
    finally:
        pm.seen_chunk = saved


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("offset", ["inside", "outside"])
@pytest.mark.parametrize("how", ["prompt", "decoded"])
@pytest.mark.parametrize("dim", [16, 64])
@pytest.mark.parametrize("edge", sorted(EDGES))
def test_mask_edges(folders, dtype, offset, how, edge, dim):
    """The one key that the last token looks for lies on the last position its mask still holds, or on the first it does not:
    a window's far end, a chunk's first position and the one before it, the last kept first token and the one behind it.
    The restatement with the mask moved by one gives other logits at that place (checked), so a mask that is one off shows."""
    make, places, move = EDGES[edge]
    cfg, over = aimed(model([(make(dim), None)], vocab=90), 4, 88, 89)
    folder, cfg, w = folders(f"{edge}{dim}", cfg, seed=4, overrides=over)
    n = 70                                                        # the key lies on and beside a page border in turn
    for end in (n - 1, n - 2, n - 6):
        toks = tokens(80, n, 100 + end)                           # ids 80.. are kept for the two tokens
        toks[end] = 88
        toks[places[offset](end)] = 89
        want = pm.forward(cfg, w, toks)
        if edge == "chunk":                                       # chunks that start one position later or earlier
            other_row = with_chunks_moved(1 if offset == "inside" else -1, cfg, w, toks)[end]
        else:
            other = copy.deepcopy(cfg)
            move(other["layers"][0]["mixer"], offset)
            other_row = pm.forward(other, w, toks)[end]
        moved = np.abs(other_row - want[end]).max() / np.abs(want).max()
        assert moved > 4 * TOL[dtype], f"the test's weights do not show the edge ({moved:.3g})"
        r = runner(folder, dtype, pool_tokens=128)
        if how == "prompt":
            got = r.run([("e", toks, [end])])
        else:
            r.run([("e", toks[:end - 3], [])])
            got = np.concatenate([r.run([("e", [t], [0])]) for t in toks[end - 3:end + 1]])[-1:]
        close(got, want[end:end + 1], dtype, f"{edge} {offset} {how} end {end}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [16, 64])
def test_far_keys_sinks_and_slow_states(folders, dtype, dim):
    """Sharp attention over many pages: one kept first token far back that the last tokens look for beside a short window,
    delta states that hardly decay, a chunk of 256 positions, then decoding; and checks that the far key, the sinks, the soft
    cap and the second map matter."""
    left = (4, 2, dim, dim + 8 if dim == 16 else dim, 0.3)                    # heads of 64 and 64: the tiled tensor-core kernel in bfloat16
    cfg, over = aimed(model([(side(left=left, size=12, keep_first=16, softcap=6.0), 64), (chunked(dim=dim, vdim=dim, size=256, rot_dims=4), None),
                             (two_maps(dim=dim * 2, vdim=dim * 2 if dim == 64 else 24, size=300), 32), ("same", 0)], vocab=140, width=128 if dim == 64 else 64), 9, 138, 139)
    folder, cfg, w = folders(f"pointed{dim}", cfg, seed=9, overrides=over)
    toks = tokens(130, 400, 21)
    toks[15] = 139                                                # the key: the last kept position, at a page's border
    toks[350] = toks[395] = 138                                   # looked for in the prompt's tail and again while decoding
    want = pm.forward(cfg, w, toks)
    r = runner(folder, dtype, pool_tokens=448, page_size=16)
    ask = [0, 1, 15, 16, 17, 255, 256, 257, 330, 339]
    rows = [r.run([("f", toks[:340], ask)])] + [r.run([("f", [t], [0])]) for t in toks[340:]]
    close(np.concatenate(rows), np.concatenate([want[ask], want[340:]]), dtype, "pointed weights")
    # the far key carries weight: with it replaced the logits at the places that look for it are elsewhere
    changed = list(toks)
    changed[15] = 1
    for place in (350, 395):
        assert np.abs(pm.forward(cfg, w, changed)[place] - want[place]).max() > 4 * TOL[dtype] * np.abs(want).max()
    # so do the sinks, the cap and the second map: the restatement without each gives other logits
    short = toks[:64]
    for name, change in (("sinks", lambda c, v: v.update({"l1.mix.sink": np.full_like(v["l1.mix.sink"], -60.0)})),
                         ("cap", lambda c, v: c["layers"][0]["mixer"]["left"].pop("softcap")),
                         ("second map", lambda c, v: v.update({"l2.mix.lq1": v["l2.mix.lq1"] * 0.0, "l2.mix.lq2": v["l2.mix.lq2"] * 0.0}) or
                          c["layers"][2]["mixer"].update(diff=1e-9))):
        c2, w2 = copy.deepcopy(cfg), dict(w)
        change(c2, w2)
        for l in c2["layers"]:                                    # a layer that runs another's tensors has that layer's entry
            if "weights_of" in l:
                l["mixer"] = copy.deepcopy(c2["layers"][l["weights_of"]]["mixer"])
        assert np.abs(pm.forward(c2, w2, short) - want[:64]).max() > 4 * TOL[dtype] * np.abs(want).max(), name


@pytest.mark.parametrize("cap", [14.0, None])
def test_long_masks_over_several_ctas(folders, cap):
    """Masks of hundreds of positions on the tensor-core path: a single token's keys are then dealt to several CTAs, the tiles of
    the kept first keys among them, and a prompt tile walks kept tiles, then its window's.  One kept key far back is the one
    that the last tokens look for (sharp weights), in a portion's tail and while two requests decode side by side.  With a cap the
    first layer's prompt portions run on the tiled kernel, without on tcgen05, where the tile's keys are cut into parts."""
    cfg, over = aimed(model([(side(left=(4, 2, 64, 64, 0.3), right=(2, 1, 16, 16, 3), size=700, keep_first=70, softcap=cap), None),
                             (chunked(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=640, rot_dims=16), None),
                             (two_maps(heads=2, kv_heads=1, dim=32, vdim=32, scale=0.2, size=800, rot_dims=8), None)], vocab=140, width=128), 9, 138, 139)
    folder, cfg, w = folders(f"long_masks{cap}", cfg, seed=9, overrides=over)
    n = 1440
    toks = tokens(130, n, 77)
    toks[69] = 139                                                # the last kept position
    for place in (1290, 1399, 1439):
        toks[place] = 138
    want = pm.forward(cfg, w, toks)
    changed = list(toks)
    changed[69] = 1
    assert np.abs(pm.forward(cfg, w, changed)[1439] - want[1439]).max() > 4 * TOL["bfloat16"] * np.abs(want).max()
    r = runner(folder, "bfloat16", pool_tokens=4096, most_tokens=2048)
    ask = [0, 69, 70, 639, 640, 700, 769, 770, 899]
    rows = [r.run([("a", toks[:900], ask)]), r.run([("a", toks[900:1300], [389, 390, 399])])]
    r.run([("b", toks[:1300], [])])                              # a second request with the same tokens decodes beside the first
    for t in toks[1300:]:
        out = r.run([("a", [t], [0]), ("b", [t], [0])])
        close(out[1:], out[:1], "bfloat16", "two requests with the same tokens")
        rows.append(out[:1])
    close(np.concatenate(rows), np.concatenate([want[ask], want[[1289, 1290, 1299]], want[1300:]]), "bfloat16", "long masks")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["odd", "tensor"])
def test_long_decoding_through_captured_steps(folders, dtype, which):
    folder, cfg, w = folders(which, ODD if which == "odd" else TENSOR, seed=5)
    toks = tokens(cfg["vocab"], 240, 31)
    want = pm.forward(cfg, w, toks)
    r = runner(folder, dtype, pool_tokens=512)
    rows = [r.run([("x", toks[:5], [4]), ("y", toks[:3], [])])]
    rows += [r.run([("x", [t], [0]), ("y", [u], [0])])[:1] for t, u in zip(toks[5:], toks[3:])]
    close(np.concatenate(rows), want[4:], dtype, "decoding")
    assert r.info("graph_replays") > 200


def test_first_tokens_of_a_sequence(folders):
    """Position 0 alone, then position 1: nothing before the sequence leaks in (zeros before the convolution, an empty state, a
    softmax over one key, with and without a sink), also in a slot that another request has used."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    r = runner(folder, "float32", slots=1)
    for seed in range(3):
        toks = tokens(cfg["vocab"], 2, 80 + seed)
        want = pm.forward(cfg, w, toks)
        close(r.run([(seed, toks[:1], [0])]), want[:1], "float32", "first token")
        close(r.run([(seed, toks[1:], [0])]), want[1:], "float32", "second token")
        r.end(seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """The scheduler's own entry point: prompts in portions beside decoding requests, greedy; each generated token must be
    (within the tolerance) the plain implementation's best token after the same prefix."""
    from easy_gpt.cpp_b200.native import NativeEngine

    folder, cfg, w = folders("general", GENERAL, seed=5)
    prompts = [tokens(cfg["vocab"], n, 90 + n) for n in (3, 41, 18, 70, 9, 26)]
    engine = NativeEngine(folder, dtype=dtype, page_size=16, cache_tokens=512, max_active=4, chunk_size=16, max_batch_tokens=48)
    outputs = engine.generate(prompts, max_new_tokens=12, greedy=True)
    for prompt, out in zip(prompts, outputs):
        assert len(out) == 12
        logits = pm.forward(cfg, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= 4 * TOL[dtype] * np.abs(row).max(), (dtype, i, tok, int(row.argmax()))


def test_trace_replay_program(folders, tmp_path):
    """bin/trace_run on a model folder of this design: steps in, logits files out."""
    folder, cfg, w = folders("odd", ODD, seed=5)
    toks = tokens(cfg["vocab"], 40, 55)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[30:], "want": [9]}, {"id": "z", "tokens": toks[:2], "want": []}], "end": ["q", "z"]}]
    out = tmp_path / "out"
    run = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want = pm.forward(cfg, w, toks)
    close(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), want[[0, 29]], "float32", "step 0")
    close(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1), want[[39]], "float32", "step 1")


def test_command_line_with_random_weights(tmp_path):
    """The engine's own program on this design: random-weights mode writes a folder from a config.json (with the per-tensor
    hints that keep norms, decays and step sizes sane, and the inner size of the low-rank maps that the configuration names),
    then prompts of token ids are decoded greedily; the tokens must be the plain implementation's for the weights that were
    written."""
    cfg = model([(side(left=(2, 1, 16, 8, 0.3), right=(2, 1, 16, 16, 3), size=12, keep_first=2), 40), (chunked(heads=2, kv_heads=1, dim=16, vdim=8, size=12), None),
                 ("same", 0), (two_maps(heads=2, kv_heads=1, dim=8, vdim=16, size=10), 24)], width=64, vocab=97)
    cfg["layers"][0]["mixer"]["right"]["rank"] = 6
    cfg["layers"][2]["mixer"]["right"]["rank"] = 6
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("5 17 3\n9,8,7,6\n")
    folder = tmp_path / "model"
    folder.mkdir()
    cmd = [sys.executable, str(ROOT / "bin" / "easy_llm"), "--model", str(folder), "--random-weights", "7", "--config", str(tmp_path / "config.json"),
           "--token-ids", "--greedy", "--max-steps", "10", "--dtype", "float32", "-f", str(prompts)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    outs = [[int(t) for t in line.split()] for line in (tmp_path / "prompts_output.txt").read_text().splitlines()]
    assert len(outs) == 2 and len(outs[0]) == 8 and len(outs[1]) == 7
    cfg_read, w = pm.read_model_dir(folder)
    assert np.all(w["l0.norm1"] == 0.0) and np.all(w["l0.mix.right.norm"] == 1.0) and w["l0.mix.right.A_log"].min() >= 0.0 and w["l0.mix.right.a1"].shape == (6, 64)
    assert "l2.norm1" not in w
    for prompt, out in zip([[5, 17, 3], [9, 8, 7, 6]], outs):
        logits = pm.forward(cfg_read, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= 4e-4 * np.abs(row).max(), (i, tok, int(row.argmax()))
