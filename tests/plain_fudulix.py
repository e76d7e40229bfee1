"""The Fudulix design stated plainly, in float64, one function per mechanism.

Nothing here is shared with the engine: no part, no kernel face, no cache.  A model is a
``config`` (the parsed config.json) and ``weights`` (name -> tensor); ``forward`` runs a
whole sequence from position 0 and returns the logits of every position.  ``store`` is
applied wherever a run in a narrower element type would store an activation (the
identity by default; a rounding to bfloat16 imitates such a run, from which tests derive
their bounds).

Notation: h is a sublayer's input [T, width]; W x means x @ W.T for a stored [out, in];
eps is the configuration's norm.eps everywhere.
"""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


def read_model_folder(path):
    """(config.json as a dict, name -> tensor) of a model folder."""
    from inferx_b200.weights.safetensors_io import Checkpoint
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    ck = Checkpoint(path)
    w = {n: ck.get(n).clone() for n in ck.names()}
    ck.close()
    return cfg, w


def _w(weights, name):
    return weights[name].to(F64)


def ident(x):
    return x


def round_bf16(x):
    return x.to(torch.bfloat16).to(F64)


def round_f32(x):
    return x.to(torch.float32).to(F64)


# -- small functions ---------------------------------------------------------
def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_div(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_div(x, eps) * w


# -- embedding -----------------------------------------------------------------
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token: a hash of (previous, current); the row after
    the hashed ones for a sequence's first token."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * mul_prev + cur * mul_cur) % buckets)
    return rows


def embed(cfg, weights, tokens):
    b = cfg["embedding"]["bigram"]
    x = _w(weights, "embed")[torch.tensor(tokens)]
    x = x + _w(weights, "bigram")[torch.tensor(
        bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"]))]
    return rms_norm(x, _w(weights, "embed.norm"), cfg["norm"]["eps"])


# -- rotation --------------------------------------------------------------------
def base_frequencies(dims, base):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def stretched_by_wavelength(freqs, sc):
    """Frequencies whose wavelength is short against the original context stay, long ones
    are divided by the factor, those between are blended."""
    out = []
    for f in freqs:
        wl = 2.0 * math.pi / f
        if wl < sc["original"] / sc["high"]:
            out.append(f)
        elif wl > sc["original"] / sc["low"]:
            out.append(f / sc["factor"])
        else:
            s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * f / sc["factor"] + s * f)
    return out


def stretched_by_ramp(freqs, dims, base, sc):
    """(frequencies, factor on cos and sin): a ramp over the pair index between the pairs
    that make ``fast`` and ``slow`` turns within the original context."""
    def pair_at(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_at(sc["fast"])), 0)
    hi = min(math.ceil(pair_at(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(freqs):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / sc["factor"] * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, freqs, dims, interleaved, magnitude=1.0):
    """x [T, heads, dim]: the first ``dims`` entries of each head are turned pairwise by
    position * frequency; pairs are (2i, 2i+1) when interleaved, else (i, i + dims/2)."""
    if not dims:
        return x
    half = dims // 2
    ang = torch.tensor(positions, dtype=F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    c, s = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


# -- short convolution over time ---------------------------------------------------
def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before 0."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


# -- attention ---------------------------------------------------------------------
def visible(i, j, size, keep_first=0):
    return j <= i and (i - j < size or j < keep_first)


def attend(q, k, v, scale, size, keep_first, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv].  ``sink``: one is added to the
    softmax's denominator (a key with score 0 and no value)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, size, keep_first)]
            s = (k[js, g] @ q[i, h]) * scale
            m = max(float(s.max()), 0.0) if sink else float(s.max())
            e = torch.exp(s - m)
            den = e.sum() + (math.exp(-m) if sink else 0.0)
            out[i, h] = (e / den) @ v[js, g]
    return out.reshape(T, -1)


def mix_values(v, v_first, lam):
    """Entry by entry over a token's values (layers that mix have as many of them, however
    they split them into heads)."""
    return v if v_first is None else (1.0 - lam) * v + lam * v_first.reshape(v.shape)


def attention(h, weights, p, m, eps, positions, v_first, store=ident):
    """The mixer "attention": interleaved rotation with wavelength-stretched frequencies,
    unit root mean square per head, a window, a sink.  Returns (output, values)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ _w(weights, f"{p}.q").T).reshape(T, H, d)
    k = store(h @ _w(weights, f"{p}.k").T).reshape(T, G, d)
    v = store(h @ _w(weights, f"{p}.v").T).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        f = base_frequencies(rot["dims"], rot["base"])
        if rot.get("scaling"):
            f = stretched_by_wavelength(f, rot["scaling"])
        q = rotate(q, positions, f, rot["dims"], True)
        k = rotate(k, positions, f, rot["dims"], True)
    q, k = store(rms_div(q, eps)), store(rms_div(k, eps))
    if m.get("v_mix"):
        v = store(mix_values(v, v_first, _w(weights, f"{p}.vmix")))
    o = store(attend(q, k, v, m["scale"], m["mask"]["size"], 0, True))
    return o @ _w(weights, f"{p}.o").T, v


def attention_2(h, weights, p, m, eps, positions, v_first, store=ident):
    """The mixer "attention_2": short convolutions after the projections, a norm over the
    whole projection, rotate-half with ramp-stretched frequencies, a window that keeps
    the first tokens, plain softmax.  Returns (output, values)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ _w(weights, f"{p}.q").T)
    k = store(h @ _w(weights, f"{p}.k").T)
    v = store(h @ _w(weights, f"{p}.v").T)
    if m.get("conv", 0):
        q = store(causal_conv(q, _w(weights, f"{p}.q.conv")))
        k = store(causal_conv(k, _w(weights, f"{p}.k.conv")))
        v = store(causal_conv(v, _w(weights, f"{p}.v.conv")))
    q = rms_norm(q, _w(weights, f"{p}.q.norm"), eps).reshape(T, H, d)
    k = rms_norm(k, _w(weights, f"{p}.k.norm"), eps).reshape(T, G, d)
    v = v.reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        f, mag = base_frequencies(rot["dims"], rot["base"]), 1.0
        if rot.get("scaling"):
            f, mag = stretched_by_ramp(f, rot["dims"], rot["base"], rot["scaling"])
        q = rotate(q, positions, f, rot["dims"], False, mag)
        k = rotate(k, positions, f, rot["dims"], False, mag)
    q, k = store(q), store(k)
    if m.get("v_mix"):
        v = store(mix_values(v, v_first, _w(weights, f"{p}.vmix")))
    o = store(attend(q, k, v, m["scale"], m["mask"]["size"], m["mask"].get("keep_first", 0),
                     False))
    return o @ _w(weights, f"{p}.o").T, v


# -- feed-forward --------------------------------------------------------------------
def dense_ff(h, weights, p, store=ident):
    g = h @ _w(weights, f"{p}.gate").T + _w(weights, f"{p}.gate.b")
    u = h @ _w(weights, f"{p}.up").T + _w(weights, f"{p}.up.b")
    return store(gelu_tanh(g) * u) @ _w(weights, f"{p}.down").T + _w(weights, f"{p}.down.b")


def gated_silu(h, weights, p, store=ident):
    g = h @ _w(weights, f"{p}.gate").T
    u = h @ _w(weights, f"{p}.up").T
    return store(silu(g) * u) @ _w(weights, f"{p}.down").T


def choose(scores, correction, top, group_count, group_keep):
    """scores [n] (softmax over all outputs of the router).  Returns (indices, weights):
    the ``top`` largest of scores + correction among the outputs of the ``group_keep``
    groups whose best such value is largest; weights are the plain scores over their sum."""
    n = scores.numel()
    pick = scores + correction
    size = n // group_count
    best = [float(pick[g * size:(g + 1) * size].max()) for g in range(group_count)]
    kept = sorted(range(group_count), key=lambda g: (-best[g], g))[:group_keep]
    allowed = [i for i in range(n) if i // size in kept]
    idx = sorted(allowed, key=lambda i: (-float(pick[i]), i))[:top]
    w = scores[idx]
    return idx, w / (w.sum() + 1e-20)


def choice_margin(scores, correction, top, group_count, group_keep, stake=1e-3):
    """How far the choice is from another one that would matter: the smaller of the
    distance between the last kept group and the first one left out and the distance
    between the last chosen output and the first one left out.  A pair whose outputs all
    have scores below ``stake`` does not count (swapping them moves next to no weight), nor
    does a side with nothing left out; then the margin is infinite."""
    n = scores.numel()
    pick = scores + correction
    size = n // group_count
    groups = sorted(range(group_count),
                    key=lambda g: (-float(pick[g * size:(g + 1) * size].max()), g))
    kept = groups[:group_keep]
    margin = math.inf
    if group_keep < group_count:
        last, first_out = groups[group_keep - 1], groups[group_keep]
        at_stake = max(float(scores[g * size:(g + 1) * size].max()) for g in (last, first_out))
        if at_stake >= stake:
            margin = float(pick[last * size:(last + 1) * size].max()
                           - pick[first_out * size:(first_out + 1) * size].max())
    allowed = sorted((i for i in range(n) if i // size in kept),
                     key=lambda i: (-float(pick[i]), i))
    if top < len(allowed):
        last, first_out = allowed[top - 1], allowed[top]
        if max(float(scores[last]), float(scores[first_out])) >= stake:
            margin = min(margin, float(pick[last] - pick[first_out]))
    return margin


def moe_ff(h, weights, p, f, store=ident, margins=None):
    r = f["router"]
    experts, identity = r["experts"], r.get("identity", 0)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    scores = torch.softmax(h @ _w(weights, f"{p}.router").T, dim=-1)
    corr = _w(weights, f"{p}.correction")
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        idx, w = choose(scores[t], corr, r["top"], groups["count"], groups["keep"])
        if margins is not None:
            margins[t] = min(margins[t], choice_margin(scores[t], corr, r["top"],
                                                       groups["count"], groups["keep"]))
        for e, we in zip(idx, w):
            if e >= experts:
                out[t] += we * h[t]
            else:
                out[t] += we * gated_silu(h[t:t + 1], weights, f"{p}.e{e}", store)[0]
    if f.get("shared"):
        out = out + gated_silu(h, weights, f"{p}.shared", store)
    return out


# -- the model -----------------------------------------------------------------------
def forward(cfg, weights, tokens, store=ident, layers_out=None, margins=None):
    """Logits [T, vocab].  ``layers_out`` (a list) receives the stream after every layer;
    ``margins`` (a list) receives, per token, the smallest ``choice_margin`` of its routers."""
    eps = cfg["norm"]["eps"]
    if margins is not None:
        margins[:] = [math.inf] * len(tokens)
    positions = list(range(len(tokens)))
    x = embed(cfg, weights, tokens)
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = store(rms_norm(x, _w(weights, f"{p}.norm1"), eps))
        mixer = {"attention": attention, "attention_2": attention_2}[layer["type"]]
        m = layer["mixer"]
        a, v = mixer(h, weights, f"{p}.mix", m, eps, positions,
                     v_first if m.get("v_mix") else None, store)
        if m.get("v_mix") and v_first is None:
            v_first = v
        x = x + store(a)
        f = layer.get("mlp")
        if f is not None:
            h = store(rms_norm(x, _w(weights, f"{p}.norm2"), eps))
            y = dense_ff(h, weights, f"{p}.mlp", store) if f["kind"] == "dense" else \
                moe_ff(h, weights, f"{p}.mlp", f, store, margins)
            x = x + store(y)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = store(rms_norm(x, _w(weights, "final.norm"), eps))
    return h @ _w(weights, "head").T
