"""Shared pieces of the Fudulix tests: small configurations, model folders, the plain
model's rows and the error bounds."""
import random

import torch

import plain_fudulix as plain
from inferx_b200.weights.random_model import write_random_model


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, groups=None, shared=0):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def first_kind(heads, kv_heads, dim, vdim, scale, window, rot=None, v_mix=True, mlp=None):
    """A layer of type "attention"; rot = (dims, base, (factor, low, high, original) or None)."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": window}, "v_mix": v_mix}
    if rot is not None:
        dims, base, sc = rot
        m["rot"] = {"dims": dims, "base": base}
        if sc is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), sc))
    return {"type": "attention", "mixer": m, "mlp": mlp}


def second_kind(heads, kv_heads, dim, vdim, scale, window, keep_first, conv, rot=None,
                v_mix=True, mlp=None):
    """A layer of type "attention_2"; rot = (dims, base, (factor, original, fast, slow) or
    None)."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": window, "keep_first": keep_first}, "conv": conv, "v_mix": v_mix}
    if rot is not None:
        dims, base, sc = rot
        m["rot"] = {"dims": dims, "base": base}
        if sc is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def top(vocab, width, eps, buckets, mul_prev, mul_cur, layers):
    return {"architecture": "Fudulix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev,
                                     "mul_cur": mul_cur}}, "layers": layers}


# the second kind leaves the values, both others mix; part of a head rotated in both kinds,
# both stretchings; windows shorter than the prompts and three kept tokens; one identity
# expert, two of three groups; a last layer that mixes nothing and has no feed-forward
FA = top(211, 96, 1e-6, 53, 5, 3, [
    second_kind(4, 2, 24, 16, 0.3, 9, 3, 3, rot=(12, 5000.0, (3.0, 64, 8.0, 1.0)),
                mlp=dense(72)),
    first_kind(6, 2, 16, 16, 0.4, 7, rot=(8, 300.0, (4.0, 1.0, 4.0, 32)),
               mlp=moe(5, 2, 24, identity=1, groups=(3, 2), shared=40)),
    second_kind(2, 1, 12, 32, 0.25, 11, 0, 2, rot=(12, 100.0, None),
                mlp=moe(4, 1, 20, identity=2, groups=(2, 1))),
    second_kind(3, 3, 8, 4, 0.5, 64, 0, 0, v_mix=False),
])

# the first kind leaves the values; odd sizes, nothing a multiple of 8; one key/value head;
# a convolution of one tap and one of five; more kept tokens than the window holds and
# than a page; a window of one token; no groups, no identity experts, no shared expert;
# every expert chosen
FB = top(101, 60, 1e-5, 17, 1, 9, [
    first_kind(3, 1, 10, 6, 0.45, 5, rot=(10, 50.0, None), mlp=moe(3, 3, 18)),
    second_kind(5, 1, 6, 6, 0.6, 4, 6, 5, rot=(4, 20.0, (2.0, 16, 4.0, 1.0)), mlp=dense(33)),
    first_kind(2, 2, 14, 3, 0.35, 1, v_mix=False, mlp=dense(25)),
    second_kind(3, 1, 10, 6, 0.5, 6, 1, 1, rot=(6, 1000.0, (8.0, 32, 2.0, 0.5)),
                mlp=moe(2, 1, 12, identity=4, groups=(3, 2), shared=10)),
])

# sizes of the kind a served model has; value heads as wide as the keys; every entry
# rotated; groups of two
FC = top(512, 256, 1e-5, 1021, 131, 17, [
    second_kind(8, 2, 64, 64, 0.125, 48, 4, 4, rot=(64, 10000.0, (4.0, 128, 16.0, 1.0)),
                mlp=dense(384)),
    first_kind(8, 2, 128, 64, 0.09, 40, rot=(64, 20000.0, (8.0, 1.0, 4.0, 64)),
               mlp=moe(6, 3, 128, identity=2, groups=(4, 2), shared=128)),
    second_kind(4, 4, 32, 32, 0.18, 24, 2, 2, rot=(16, 1e6, None), mlp=dense(512)),
    first_kind(4, 1, 64, 128, 0.1, 33, rot=(32, 1000.0, None), mlp=moe(8, 2, 64, shared=64)),
])

CONFIGS = {"FA": FA, "FB": FB, "FC": FC}


def sharpen(name, t):
    """N(0, 0.02) weights would give uniform attention, routers without an opinion,
    corrections and biases that change nothing and convolutions of nothing; make each of
    them matter."""
    if name in ("embed", "bigram"):
        return t * 40.0
    if name.endswith((".mix.q", ".mix.k")):
        return t * 6.0
    if name.endswith(".mix.v"):
        return t * 5.0
    if name.endswith(".conv"):
        return t * 25.0
    if name.endswith(".vmix"):
        return t * 10.0 + 0.4
    if name.endswith(".router"):
        return t * 12.0
    if name.endswith(".correction"):
        return t * 8.0
    if name.endswith(".b"):
        return t * 15.0
    if name.endswith((".gate", ".up")):
        return t * 6.0
    return t


def make_model_dir(cfg, path, seed, dtype="float32", adjust=sharpen):
    write_random_model(cfg, str(path), seed=seed, dtype=dtype, adjust=adjust)
    return str(path)


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)]
            for i, n in enumerate(lengths)}


def reference_rows(model_dir, requests):
    cfg, w = plain.read_model_folder(model_dir)
    rows = {}
    for rid, toks in requests.items():
        lg = plain.forward(cfg, w, toks).to(torch.float32)
        for p in range(len(toks)):
            rows[(rid, p)] = lg[p]
    return rows


def _bound(model_dir, requests, store, factor, floor):
    cfg, w = plain.read_model_folder(model_dir)
    worst = 0.0
    for toks in requests.values():
        a = plain.forward(cfg, w, toks)
        b = plain.forward(cfg, w, toks, store=store)
        worst = max(worst, float((a - b).abs().max()) / float(a.abs().max()))
    return max(floor, factor * worst)


def bound_for(dtype, model_dir, requests):
    """Three times what storing activations in the run's element type costs the plain
    model itself, relative to the largest logit; the floors stand for sums of hundreds of
    products in that precision, which the plain model does not have."""
    if dtype == "float32":
        return _bound(model_dir, requests, plain.round_f32, 3.0, 3e-5)
    return _bound(model_dir, requests, plain.round_bf16, 3.0, 5e-3)


def decisive_rows(model_dir, requests, least=1e-3):
    """{(request, position)} whose logits cannot have been changed by a router's close
    call: no router of this or an earlier token of the request chose with a margin below
    ``least``, neither in the plain model nor in the plain model that rounds what it stores
    to bfloat16 (a choice that rounding can turn changes the token's stream, and through
    the keys and values every later token's).  Tests of bfloat16 runs compare these rows;
    the 32-bit runs compare all."""
    cfg, w = plain.read_model_folder(model_dir)
    keep = set()
    for rid, toks in requests.items():
        exact, rounded = [], []
        plain.forward(cfg, w, toks, margins=exact)
        plain.forward(cfg, w, toks, store=plain.round_bf16, margins=rounded)
        for p, (a, b) in enumerate(zip(exact, rounded)):
            if min(a, b) < least:
                break
            keep.add((rid, p))
    return keep


def rows_to_compare(dtype, model_dir, requests, rows, share=0.25):
    """The produced rows a run in ``dtype`` is held to (see ``decisive_rows``)."""
    if dtype == "float32":
        return rows
    keep = decisive_rows(model_dir, requests)
    kept = {k: v for k, v in rows.items() if k in keep}
    assert len(kept) >= share * len(rows), "too many close calls: the test compares too little"
    return kept
