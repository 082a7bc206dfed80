"""The Masezen decoder in the native engine against the plain numpy restatement (tests/plain_masezen.py): each mechanism
alone, prompts cut in every way, batches, reused pages and slots, far keys on and beside page borders, the first tokens,
long decoding, odd sizes, sizes that are one, the tensor-core paths, generation, replay and the command line.

Every test makes its own small configuration and random weights.  Errors are the largest difference of a logit over
the largest logit: float32 must stay within 1e-4.  In bfloat16 every branch's input and output is rounded to eight bits
of mantissa, and these untrained models pass nothing else on: there the bound is 3e-2 on the root mean square of all
differences (over the root mean square of the logits) and 8e-2 on the largest one; the faults that the pointed tests
plant move logits by far more.
"""
import copy
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_masezen as pm

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
LARGEST = {"float32": 1e-4, "bfloat16": 8e-2}


def attention(heads=4, kv_heads=2, dim=16, scale=0.3, rot_dims=8, base=10000.0, scaling=(4.0, 64, 16.0, 2.0)):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, limit=1.2, shared=(40, 0.9)):
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


def model(layers, width=64, vocab=131, taps=3, side=6, eps=1e-5):
    cfg = {"architecture": "Masezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "token_side": {"dim": side}, "layers": []}
    for mixer, mlp in layers:
        cfg["layers"].append({**copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)})
    return cfg


GENERAL = model([(attention(), dense(96)), (attention(heads=6, kv_heads=3, dim=8, scale=0.5, rot_dims=4, scaling=None), moe()),
                 (attention(heads=2, kv_heads=1, dim=24, scale=0.2, rot_dims=24, base=5e5, scaling=(8.0, 32, 8.0, 1.0)), None),
                 (attention(heads=4, kv_heads=4, dim=12, scale=0.35, rot_dims=None), moe(experts=3, top=1, ff=16, limit=2.5, shared=None))])
# widths that leave the decode product's alignment rule, head sizes that are no powers of two, two taps, three of five experts
ODD = model([(attention(heads=3, kv_heads=1, dim=20, scale=0.4, rot_dims=6, base=300.0), moe(experts=5, top=3, ff=10, limit=0.7, shared=(14, 3.0))),
             (attention(heads=5, kv_heads=5, dim=10, scale=0.3, rot_dims=10, scaling=None), dense(52))], width=72, vocab=77, taps=2, side=5)
# values that are one or equal: one head, one key head, one tap (no convolution, no state), one expert of which one is taken,
# one side value, the whole head rotated or nothing
ONES = model([(attention(heads=1, kv_heads=1, dim=16, scale=1.0, rot_dims=16), moe(experts=1, top=1, ff=8, limit=1.0, shared=(8, 1.0))),
              (attention(heads=2, kv_heads=2, dim=8, scale=0.7, rot_dims=None), None)], width=48, vocab=64, taps=1, side=1)

ALONE = {
    "attention": model([(attention(), None)]),
    "attention_no_rotation": model([(attention(rot_dims=None), None)]),
    "attention_no_stretching": model([(attention(scaling=None), None)]),
    "attention_many_heads": model([(attention(heads=8, kv_heads=2, dim=64, scale=0.11, rot_dims=24, base=5e5, scaling=(6.0, 1024, 24.0, 2.0)), None)], width=128),
    "attention_24_heads": model([(attention(heads=24, kv_heads=3, dim=16, scale=0.3, rot_dims=8), None)], width=96),
    "attention_heads_of_48": model([(attention(heads=4, kv_heads=2, dim=48, scale=0.15, rot_dims=48, scaling=None), None)]),
    "attention_wide_keys": model([(attention(heads=6, kv_heads=3, dim=256, scale=0.06, rot_dims=32), None)], width=96),
    "attention_five_key_heads": model([(attention(heads=10, kv_heads=5, dim=128, scale=0.09, rot_dims=128, scaling=None), None)], width=96),
    "attention_ten_key_heads": model([(attention(heads=10, kv_heads=10, dim=64, scale=0.12, rot_dims=16), None)], width=96),
    "attention_one_key_head": model([(attention(heads=4, kv_heads=1, dim=32, scale=0.2, rot_dims=32), None)]),
    "attention_large_heads": model([(attention(heads=2, kv_heads=2, dim=128, scale=0.09, rot_dims=64, scaling=None), None)], width=96),
    "attention_heads_of_256": model([(attention(heads=2, kv_heads=1, dim=256, scale=0.06, rot_dims=128, scaling=None), None)], width=96),
    "odd_width": model([(attention(heads=3, kv_heads=1, dim=10, scale=0.4, rot_dims=4), dense(27))], width=90, vocab=53, taps=4, side=3),
    "dense": model([(attention(heads=2, kv_heads=1, dim=8), dense(100))]),
    "routed": model([(attention(heads=2, kv_heads=1, dim=8), moe())]),
    "routed_without_shared": model([(attention(heads=2, kv_heads=1, dim=8), moe(experts=9, top=4, shared=None))]),
    # sizes that the grouped tensor-core products take in bfloat16 (prompts of 33 tokens and more)
    "routed_wide": model([(attention(heads=2, kv_heads=1, dim=32), moe(experts=4, top=2, ff=64, limit=1.5, shared=(128, 1.0)))], width=128),
    "eight_taps": model([(attention(heads=2, kv_heads=1, dim=8), None)], taps=8),
    "no_convolution_state": model([(attention(heads=2, kv_heads=1, dim=8), dense(32))], taps=1),
}


def tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg, seed=0, overrides=None):
        if name not in made:
            w = pm.random_weights(cfg, seed, overrides)
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


@pytest.mark.parametrize("name", ["attention_many_heads", "attention_24_heads", "attention_heads_of_48", "attention_wide_keys", "attention_five_key_heads",
                                  "attention_ten_key_heads", "attention_large_heads", "attention_heads_of_256", "attention_one_key_head"])
def test_attention_sizes_in_portions_and_single_tokens(folders, name):
    """Every form of the tensor-core attention kernels (heads of up to 64, 128 and 256 values, padded heads, one CTA or two a listed
    tile, more than 16 heads): a prompt over two listed tiles, single tokens beside another request's portion, steps of short
    entries only, and decoding, against the restatement of each request alone."""
    folder, cfg, w = folders(name, ALONE[name], seed=3)
    a, b = tokens(cfg["vocab"], 166, 5), tokens(cfg["vocab"], 150, 6)
    want_a, want_b = pm.forward(cfg, w, a), pm.forward(cfg, w, b)
    r = runner(folder, "bfloat16", pool_tokens=512)
    close(r.run([("a", a[:150], list(range(150)))]), want_a[:150], "bfloat16", name + ": two tiles")
    got = r.run([("a", a[150:151], [0]), ("b", b[:137], list(range(137)))])
    close(got, np.concatenate([want_a[150:151], want_b[:137]]), "bfloat16", name + ": a token beside a portion")
    got = r.run([("a", a[151:154], [0, 1, 2]), ("b", b[137:139], [0, 1])])
    close(got, np.concatenate([want_a[151:154], want_b[137:139]]), "bfloat16", name + ": short entries")
    for i in range(11):
        got = r.run([("a", [a[154 + i]], [0]), ("b", [b[139 + i]], [0])])
        close(got, np.stack([want_a[154 + i], want_b[139 + i]]), "bfloat16", name + f": decoding {i}")


def test_the_restatements_own_pieces():
    """The restatement against itself: the stream after every layer, the convolution against its sum written out, the routed
    feed-forward with every expert chosen against the sum of all experts, and a mix that is the identity against plain heads."""
    cfg = GENERAL
    w = pm.random_weights(cfg, 1)
    logits, streams = pm.forward(cfg, w, tokens(cfg["vocab"], 9, 0), return_layers=True)
    assert streams.shape == (4, 9, cfg["width"]) and logits.shape == (9, cfg["vocab"])
    rng = np.random.default_rng(0)
    x, taps = rng.standard_normal((7, 5)), rng.standard_normal((5, 3))
    want = np.array([[sum(taps[c, j] * (x[t - 2 + j, c] if t - 2 + j >= 0 else 0.0) for j in range(3)) for c in range(5)] for t in range(7)])
    assert np.allclose(pm.causal_conv(x, taps), want)
    mlp = moe(experts=3, top=3, ff=16, limit=2.0, shared=None)
    one = model([(attention(heads=2, kv_heads=1, dim=8), mlp)])
    w1 = pm.random_weights(one, 2)
    h = rng.standard_normal((4, one["width"]))
    s = pm.sigmoid(h @ w1["l0.mlp.router"].T)
    every = sum(pm.clamped_expert(s[:, e:e + 1] * h, w1, f"l0.mlp.e{e}.", 2.0) for e in range(3))
    assert np.allclose(pm.routed_ff(h, w1, "l0.mlp.", mlp), every)
    m = one["layers"][0]["mixer"]
    mixed = pm.mixed_head_attention(h, w1, "l0.mix.", m, 1e-5)
    plain = dict(w1)
    plain["l0.mix.talk"] = np.eye(2)
    swapped = dict(w1)
    swapped["l0.mix.talk"] = np.eye(2)[::-1]
    assert not np.allclose(mixed, pm.mixed_head_attention(h, plain, "l0.mix.", m, 1e-5))
    assert not np.allclose(pm.mixed_head_attention(h, swapped, "l0.mix.", m, 1e-5), pm.mixed_head_attention(h, plain, "l0.mix.", m, 1e-5))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("general", GENERAL), ("odd", ODD), ("ones", ONES), ("alone_attention_many_heads", None), ("alone_attention_large_heads", None),
                                      ("alone_attention_heads_of_256", None), ("alone_attention_one_key_head", None), ("alone_routed_wide", None),
                                      ("alone_odd_width", None), ("alone_eight_taps", None)])
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
@pytest.mark.parametrize("sizes", [[2] * 20, [3, 1, 2, 17, 1, 1, 30, 5, 2, 2, 16, 15, 1, 33], [16, 16, 16, 16, 1, 15, 48], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]])
@pytest.mark.parametrize("which", ["general", "eight_taps"])
def test_portions(folders, sizes, dtype, which):
    """Portions down to two tokens, shorter than the convolution's reach (eight taps: seven rows of state, of which a portion
    of two replaces two), ending on and beside page borders."""
    folder, cfg, w = folders(which, GENERAL if which == "general" else ALONE[which], seed=5 if which == "general" else 3)
    toks = tokens(cfg["vocab"], sum(sizes), 7)
    want = pm.forward(cfg, w, toks)
    r = runner(folder, dtype, page_size=16)
    at, rows = 0, []
    for n in sizes:
        rows.append(r.run([("p", toks[at:at + n], list(range(n)))]))
        at += n
    close(np.concatenate(rows), want, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests(folders, dtype):
    """Four requests of different lengths advance together, portions beside single tokens; each must come out as alone."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
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
def test_pages_and_slots_are_used_again(folders, dtype):
    """Two slots and a pool of four pages: every request takes a slot (the convolutions' inputs) and pages that another one
    has left full."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
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


def aimed(cfg, seed, a, b, sharp=6.0):
    """Weights under which one score stands out in the first layer: the key maps are the query maps of their groups' first
    heads behind a reflection of the model's width that carries what the mixer reads of a run of tokens b onto what it reads of
    a run of tokens a.  After `taps` equal tokens the convolution multiplies the normed embedding channel by channel by one
    plus the sum of its taps, so a run of b is the key that a run of a looks for, whatever lies between them; b's value is its
    own key.  The mix of the heads keeps its random part."""
    cfg = copy.deepcopy(cfg)
    base = pm.random_weights(cfg, seed)
    m = cfg["layers"][0]["mixer"]
    m["scale"] = sharp / float(np.sqrt(m["dim"]))
    eps = cfg["norm"]["eps"]
    reach = 1.0 + base["l0.canon1"].sum(axis=1)
    na, nb = (pm.rms_unit(base["embed"][t], eps) * base["l0.norm1"] * reach for t in (a, b))
    u = na / np.linalg.norm(na) - nb / np.linalg.norm(nb)
    u /= np.linalg.norm(u)
    q = base["l0.mix.q"].reshape(m["heads"], m["dim"], -1)[::m["heads"] // m["kv_heads"]].reshape(m["kv_heads"] * m["dim"], -1)
    return cfg, {"l0.mix.k": q - 2.0 * np.outer(q @ u, u), "l0.mix.q.norm": np.abs(base["l0.mix.q.norm"]), "l0.mix.k.norm": np.abs(base["l0.mix.k.norm"])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [16, 64])
def test_far_keys_at_page_borders(folders, dtype, dim):
    """Sharp attention over many pages: one run of a token far back, ending on, before and behind a page's border in turn, that the
    last tokens look for, in the prompt's tail and again while decoding; and checks that the far key and the mix of the heads matter."""
    taps = 3
    cfg, over = aimed(model([(attention(heads=4, kv_heads=2, dim=dim, rot_dims=4), dense(64)), (attention(heads=2, kv_heads=2, dim=8, rot_dims=None), moe())],
                            vocab=140, taps=taps, width=64 if dim == 16 else 128), 9, 138, 139, sharp=9.0)
    folder, cfg, w = folders(f"pointed{dim}", cfg, seed=9, overrides=over)
    for key_end in (15, 16, 17):                                 # the last token of the run of b: a page's last place, the next page's first two
        toks = tokens(130, 400, 21 + key_end)
        toks[key_end - taps + 1:key_end + 1] = [139] * taps
        toks[350 - taps + 1:351] = toks[395 - taps + 1:396] = [138] * taps
        want = pm.forward(cfg, w, toks)
        r = runner(folder, dtype, pool_tokens=448, page_size=16)
        ask = [0, 1, 15, 16, 17, 255, 256, 330, 339]
        rows = [r.run([("f", toks[:340], ask)])] + [r.run([("f", [t], [0])]) for t in toks[340:]]
        close(np.concatenate(rows), np.concatenate([want[ask], want[340:]]), dtype, f"pointed weights, key at {key_end}")
        r.end("f")
        # the same places out of one prompt
        close(r.run([("g", toks, [350, 395, 399])]), want[[350, 395, 399]], dtype, f"pointed weights in a prompt, key at {key_end}")
        # the far key carries weight: with it replaced the logits at the places that look for it are elsewhere
        changed = list(toks)
        changed[key_end - taps + 1:key_end + 1] = [1, 2, 3]
        for place in (350, 395):
            assert np.abs(pm.forward(cfg, w, changed)[place] - want[place]).max() > LARGEST[dtype] * np.abs(want).max()
    # the mix matters: with the identity in its place the logits are elsewhere
    unmixed = dict(w)
    unmixed["l0.mix.talk"] = np.eye(4)
    assert np.abs(pm.forward(cfg, unmixed, toks[:64]) - want[:64]).max() > 4 * TOL[dtype] * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(folders, dtype):
    folder, cfg, w = folders("odd", ODD, seed=5)
    toks = tokens(cfg["vocab"], 240, 31)
    want = pm.forward(cfg, w, toks)
    r = runner(folder, dtype, pool_tokens=512)
    rows = [r.run([("x", toks[:5], [4]), ("y", toks[:3], [])])]
    rows += [r.run([("x", [t], [0]), ("y", [u], [0])])[:1] for t, u in zip(toks[5:], toks[3:])]
    close(np.concatenate(rows), want[4:], dtype, "decoding")
    assert r.info("graph_replays") > 200


def test_first_tokens_of_a_sequence(folders):
    """Position 0 alone, then position 1: nothing before the sequence leaks in (zeros before the convolution, a softmax over one
    key), also in a slot that another request has used."""
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
    hints that keep the gains at one and the mix of the heads near the identity), then prompts of token ids are decoded greedily;
    the tokens must be the plain implementation's for the weights that were written."""
    cfg = model([(attention(heads=4, kv_heads=2, dim=16), dense(40)), (attention(heads=2, kv_heads=1, dim=16, rot_dims=None), moe(experts=4, top=2, ff=16))],
                width=64, vocab=97)
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
    assert np.all(w["l0.norm1"] == 1.0) and np.all(w["l1.ls1"] == 1.0) and np.all(w["l0.mix.q.norm"] == 1.0)
    assert np.abs(w["l0.mix.talk"] - np.eye(4)).max() < 0.5 and np.abs(np.diag(w["l0.mix.talk"]) - 1.0).max() < 0.5
    for prompt, out in zip([[5, 17, 3], [9, 8, 7, 6]], outs):
        logits = pm.forward(cfg_read, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= 4e-4 * np.abs(row).max(), (i, tok, int(row.argmax()))
