"""Shared pieces of the Mapovik tests: small configurations, model folders, the plain
model's rows and the error bounds."""
import random

import torch

import plain_mapovik as plain
from inferx_b200.weights.random_model import write_random_model


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention(heads, kv_heads, dim, vdim, scale, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        dims, base, factor = rot
        m["rot"] = {"dims": dims, "base": base}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def ssd(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
            "norm_groups": norm_groups}


def parallel(left, right, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, rank=6, gate_rank=5, mlp=None):
    return {"type": "channel_delta",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                      "conv": conv, "rank": rank, "gate_rank": gate_rank}, "mlp": mlp}


# a loop over the first two layers; half of each head rotated with scaled frequencies; value
# heads wider than the keys; two experts per token; a layer without feed-forward
MA = {
    "architecture": "Mapovik", "vocab": 200, "width": 96, "norm": {"eps": 1e-6},
    "residual_mult": 0.5, "logit_scale": 2.0,
    "layers": [
        parallel(attention(4, 2, 20, 28, 0.3, rot=(10, 5000.0, 3.0)), ssd(3, 8, 12, 1, 4, 3),
                 dense(72)),
        delta(4, 2, 12, 20, 3, mlp=moe(5, 2, 24)),
        delta(2, 2, 16, 8, 4),
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}

# no loop; no residual factor and no logit factor; as many key/value heads as heads, value
# size equal to the key size, every entry rotated without scaling; one head; convolutions
# of two taps; every expert chosen
MB = {
    "architecture": "Mapovik", "vocab": 384, "width": 128, "norm": {"eps": 1e-5},
    "residual_mult": 1.0, "logit_scale": 1.0,
    "layers": [
        delta(1, 1, 24, 24, 2, rank=3, gate_rank=9, mlp=dense(100)),
        parallel(attention(2, 2, 36, 36, 0.2, rot=(36, 10000.0, None)), ssd(2, 16, 8, 2, 2, 1),
                 moe(3, 3, 40)),
        parallel(attention(3, 1, 16, 8, 0.25), ssd(1, 40, 20, 1, 5, 2), None),
    ],
}

# nothing a multiple of 8, odd head sizes, an odd vocabulary; the middle layer repeated;
# a convolution of one tap (no convolution state)
MC = {
    "architecture": "Mapovik", "vocab": 101, "width": 60, "norm": {"eps": 1e-5},
    "residual_mult": 0.7, "logit_scale": 0.5,
    "layers": [
        delta(3, 1, 7, 5, 1, rank=2, gate_rank=2, mlp=moe(7, 3, 18)),
        parallel(attention(3, 1, 9, 11, 0.45, rot=(6, 300.0, 1.5)), ssd(5, 3, 7, 5, 3, 5),
                 moe(4, 1, 26)),
        delta(6, 3, 5, 9, 4, rank=4, gate_rank=3, mlp=dense(33)),
    ],
    "loop": {"start": 1, "stop": 2, "times": 2},
}

# sizes of the kind a served model has; the whole model runs twice
MD = {
    "architecture": "Mapovik", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
    "residual_mult": 0.5, "logit_scale": 1.5,
    "layers": [
        parallel(attention(8, 2, 64, 128, 0.125, rot=(32, 10000.0, 2.0)),
                 ssd(8, 64, 64, 2, 4, 4), moe(8, 2, 128)),
        delta(4, 2, 64, 128, 4, rank=16, gate_rank=16, mlp=moe(8, 2, 128)),
        delta(2, 2, 128, 64, 4, rank=32, gate_rank=8, mlp=dense(512)),
        parallel(attention(4, 1, 128, 128, 0.09, rot=(64, 1e6, 3.0)), ssd(4, 32, 128, 1, 4, 1),
                 dense(384)),
    ],
    "loop": {"start": 0, "stop": 4, "times": 2},
}

CONFIGS = {"MA": MA, "MB": MB, "MC": MC, "MD": MD}


def sharpen(name, t):
    """N(0, 0.02) weights would give uniform attention, decays that never differ, dead
    gates and convolutions of nothing; make each of them matter."""
    if name == "embed":
        return t * 40.0
    if name.endswith((".left.q", ".left.k")):
        return t * 8.0
    if name.endswith((".mix.q", ".mix.k", ".mix.v", ".left.v", ".right.in")):
        return t * 5.0
    if name.endswith(".conv"):
        return t * 20.0
    if name.endswith(".conv.b"):
        return t * 10.0
    if name.endswith((".mix.a1", ".mix.g1")):
        return t * 8.0
    if name.endswith((".mix.a2", ".mix.g2")):
        return t * 30.0
    if name.endswith(".mix.b"):
        return t * 20.0
    if name.endswith(".dt_bias"):
        return t * 40.0
    if name.endswith(".A_log"):
        return t * 40.0 - 0.5
    if name.endswith((".gate", ".up")):
        return t * 6.0
    if name in ("loop.step",):
        return t * 20.0
    if name == "loop.in":
        return t * 4.0
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
