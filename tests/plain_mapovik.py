"""The Mapovik design stated plainly, in float64, one function per mechanism.

Nothing here is shared with the engine: no part, no kernel face, no cache.  A model is a
``config`` (the parsed config.json) and ``weights`` (name -> tensor); ``forward`` runs a
whole sequence from position 0 and returns the logits of every position.  ``store`` is
applied wherever a run in a narrower element type would store an activation (the
identity by default; a rounding to bfloat16 imitates such a run, from which tests derive
their bounds).

Notation: h is a sublayer's input [T, width]; W x means x @ W.T for a stored [out, in].
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


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * w; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w


def rms_div(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(x, w, bias=None):
    """x [T, C]; w [C, taps], last column the current token's; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros(T, C, dtype=x.dtype)
    for j in range(taps):
        out = out + padded[j:j + T] * w[:, j]
    if bias is not None:
        out = out + bias
    return out


def rotate_half(x, positions, dims, base, factor):
    """x [T, heads, d]: the first ``dims`` entries of each head are turned, entry i with
    entry i + dims/2, by the angle p * base^(-2i/dims) / factor."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = torch.pow(torch.tensor(base, dtype=F64), -2.0 * i / dims) / factor
    a = positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


# -- mixers ------------------------------------------------------------------
def softmax_attention(h, weights, p, m, positions, store=ident):
    """Causal grouped-query attention with partly rotated queries and keys."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ _w(weights, f"{p}.q").T).view(T, H, dk)
    k = store(h @ _w(weights, f"{p}.k").T).view(T, G, dk)
    v = store(h @ _w(weights, f"{p}.v").T).view(T, G, dv)
    rot = m.get("rot")
    if rot is not None:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = store(rotate_half(q, positions, rot["dims"], float(rot["base"]), factor))
        k = store(rotate_half(k, positions, rot["dims"], float(rot["base"]), factor))
    out = torch.zeros(T, H, dv, dtype=F64)
    per = H // G
    mask = positions[None, :] <= positions[:, None]
    for hh in range(H):
        g = hh // per
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        s = torch.where(mask, s, torch.tensor(-math.inf, dtype=F64))
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    return store(out.reshape(T, H * dv)) @ _w(weights, f"{p}.o").T


def state_space(h, weights, p, m, eps, store=ident):
    """Selective state space with a scalar decay per head (Mamba-2)."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = store(h @ _w(weights, f"{p}.in").T)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = store(silu(causal_conv(xbc, _w(weights, f"{p}.conv"), _w(weights, f"{p}.conv.b"))))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + _w(weights, f"{p}.dt_bias"))
    a = torch.exp(-torch.exp(_w(weights, f"{p}.A_log")) * dt)        # [T, H]
    D = _w(weights, f"{p}.D")
    y = torch.zeros(T, H, P, dtype=F64)
    per = H // G
    for hh in range(H):
        g = hh // per
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = a[t, hh] * S + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S.T @ C[t, g] + D[hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms_div(y.view(T, ng, inner // ng), eps).reshape(T, inner) * _w(weights, f"{p}.norm")
    return store(y) @ _w(weights, f"{p}.o").T


def parallel_mixer(h, weights, p, m, eps, positions, store=ident):
    left = softmax_attention(h, weights, f"{p}.left", m["left"], positions, store)
    right = state_space(h, weights, f"{p}.right", m["right"], eps, store)
    return 0.5 * (rms_div(left, eps) * _w(weights, f"{p}.left.out")
                  + rms_div(right, eps) * _w(weights, f"{p}.right.out"))


def channel_delta(h, weights, p, m, eps, store=ident):
    """Gated delta rule with a decay per head and key channel."""
    T = h.shape[0]
    H, Hk, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def short(name):
        return store(silu(causal_conv(store(h @ _w(weights, f"{p}.{name}").T),
                                      _w(weights, f"{p}.{name}.conv"))))

    q, k, v = short("q").view(T, Hk, dk), short("k").view(T, Hk, dk), short("v").view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(store(h @ _w(weights, f"{p}.b").T))               # [T, H]
    za = store(store(h @ _w(weights, f"{p}.a1").T) @ _w(weights, f"{p}.a2").T)
    za = (za + _w(weights, f"{p}.dt_bias")).view(T, H, dk)
    g = torch.exp(-torch.exp(_w(weights, f"{p}.A_log"))[None, :, None] * softplus(za))
    o = torch.zeros(T, H, dv, dtype=F64)
    per = H // Hk
    for hh in range(H):
        j = hh // per
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = g[t, hh][:, None] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, j])
            S = S + torch.outer(k[t, j], u)
            o[t, hh] = S.T @ q[t, j]
    o = rms_div(o, eps) * _w(weights, f"{p}.norm")
    gate = torch.sigmoid(store(store(h @ _w(weights, f"{p}.g1").T) @ _w(weights, f"{p}.g2").T))
    o = o.reshape(T, H * dv) * gate
    return store(o) @ _w(weights, f"{p}.o").T


# -- feed-forward ------------------------------------------------------------
def dense_ff(h, weights, p, store=ident):
    a = torch.relu(store(h @ _w(weights, f"{p}.up").T))
    return store(a * a) @ _w(weights, f"{p}.down").T


def expert(h, weights, p, store=ident):
    a = silu(store(h @ _w(weights, f"{p}.gate").T)) * store(h @ _w(weights, f"{p}.up").T)
    return store(a) @ _w(weights, f"{p}.down").T


def table_experts(h, weights, p, tokens, store=ident):
    """Each token's experts are a row of a table indexed by its id; equal weights."""
    table = weights[f"{p}.table"].long()
    top = table.shape[1]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            out[t] += expert(h[t:t + 1], weights, f"{p}.e{e}", store)[0] / top
    return out


# -- the model ---------------------------------------------------------------
def run_order(config):
    """[(layer, pass or None, first of its pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    return order + [(i, None, False) for i in range(b, n)]


def layer(x, weights, config, i, tokens, positions, store=ident):
    spec = config["layers"][i]
    eps, m, p = float(config["norm"]["eps"]), float(config["residual_mult"]), f"l{i}"
    h = store(layer_norm(x, _w(weights, f"{p}.norm1"), eps))
    if spec["type"] == "parallel":
        a = parallel_mixer(h, weights, f"{p}.mix", spec["mixer"], eps, positions, store)
    elif spec["type"] == "channel_delta":
        a = channel_delta(h, weights, f"{p}.mix", spec["mixer"], eps, store)
    else:
        raise ValueError(spec["type"])
    x = x + m * a
    mlp = spec.get("mlp")
    if mlp is not None:
        h = store(layer_norm(x, _w(weights, f"{p}.norm2"), eps))
        if mlp["kind"] == "dense":
            f = dense_ff(h, weights, f"{p}.mlp", store)
        elif mlp["kind"] == "moe":
            f = table_experts(h, weights, f"{p}.mlp", tokens, store)
        else:
            raise ValueError(mlp["kind"])
        x = x + m * f
    return x


def forward(config, weights, tokens, store=ident, streams=None):
    """Logits [T, vocab] of a whole sequence from position 0.  ``streams``, a list, takes
    the residual stream after every layer run."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x0 = _w(weights, "embed")[tokens]
    x = x0
    for i, t, first in run_order(config):
        if first:
            x = store(torch.cat([x, x0], -1)) @ _w(weights, "loop.in").T
            x = x + _w(weights, "loop.step")[t]
        x = layer(x, weights, config, i, tokens, positions, store)
        if streams is not None:
            streams.append(x.clone())
    h = store(layer_norm(x, _w(weights, "final.norm"), float(config["norm"]["eps"])))
    return (h @ _w(weights, "head").T) * float(config["logit_scale"])
