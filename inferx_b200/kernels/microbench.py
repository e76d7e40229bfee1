"""Kernel-level timings with achieved bandwidth or FLOP rate.

    python -m inferx_b200.kernels.microbench attn_decode --batch 8 --context 4096 [--form tma|mma|scalar]
    python -m inferx_b200.kernels.microbench grouped --tokens 8
    python -m inferx_b200.kernels.microbench dense --rows 8 --n 6144 --k 2048
    python -m inferx_b200.kernels.microbench attn_prefill --tokens 2048 [--form tc|mma]
    python -m inferx_b200.kernels.microbench attn_prefill --tokens 512 --context 8192 [--splits N]
    python -m inferx_b200.kernels.microbench router --tokens 2048
    python -m inferx_b200.kernels.microbench qkv --rows 8 [--separate]
    python -m inferx_b200.kernels.microbench grouped --tokens 2048
    python -m inferx_b200.kernels.microbench latent_attn --tokens 2048 --rank 512 --rot-dim 64 [--form mma|general]
    python -m inferx_b200.kernels.microbench latent_attn --tokens 1 --batch 8 --context 4096
    python -m inferx_b200.kernels.microbench rowwise --tokens 4096 --hidden 2048 --inter 5632
    python -m inferx_b200.kernels.microbench recurrent --tokens 4096 --batch 1 --hidden 2048 --head-dim 64
    python -m inferx_b200.kernels.microbench recurrent --tokens 64 --batch 64 --hidden 2048 --head-dim 64
    python -m inferx_b200.kernels.microbench attn_prefill --tokens 2048 --softcap 30
    python -m inferx_b200.kernels.microbench prepared --tokens 2048 --hidden 2048 --heads 16 --kv-heads 4 --inter 4096 --experts 32 --batch 8 --window 1024

Each case runs one kernel face at Qwen1.5-MoE-A2.7B sizes (or the sizes given),
cycling through enough copies of its inputs that consecutive iterations do not
find them in the 126 MB L2, timed with CUDA events after warm-up.  One JSON line
per case: microseconds per call, bytes (or FLOP) per call by the algorithm, and the
achieved rate.  The reference's counterpart is its per-kernel bench harness
(bench/cuda_timer.h:1-40, bench/decode_step_bench.cc).
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import types

import torch

L2_BYTES = 126 << 20


EAGER = [False]   # --eager: no graph capture (for profilers that want plain launches)


def _time(fn, n_variants, iters, warmup=5):
    """Microseconds per call.  The calls are captured into one CUDA graph and the
    graph is replayed, so the host's launch cost does not hide a short kernel."""
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    if EAGER[0]:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(iters):
            fn(i % n_variants)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) * 1e3 / iters
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i % n_variants)
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / iters


def _copies(bytes_per_copy):
    return max(2, int(math.ceil(2 * L2_BYTES / max(1, bytes_per_copy))))


def attn_decode(args):
    from . import ops
    B, C, heads, kvh, hd, page = args.batch, args.context, args.heads, args.kv_heads, \
        args.head_dim, args.page
    dt = torch.bfloat16
    pages_per_seq = -(-C // page)
    per_copy = B * pages_per_seq * page * kvh * hd * 2 * 2
    n = min(_copies(per_copy), 8)
    P = B * pages_per_seq
    kcs = [torch.randn(P, kvh, page, hd, device="cuda", dtype=dt) for _ in range(n)]
    vcs = [torch.randn(P, kvh, page, hd, device="cuda", dtype=dt) for _ in range(n)]
    bt = torch.randperm(P, device="cuda").to(torch.int32).view(B, pages_per_seq)
    q = torch.randn(B, heads, hd, device="cuda", dtype=dt)
    kv_len = torch.full((B,), C, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(hd)

    def fn(i):
        ops.paged_attention_decode(q, kcs[i], vcs[i], bt, kv_len, C, args.window, scale,
                                   splits=args.splits or None, kernel=args.form or None,
                                   softcap=args.softcap)
    us = _time(fn, n, args.iters)
    span = min(C, args.window) if args.window else C
    nbytes = B * span * kvh * hd * 2 * 2
    return {"case": "attn_decode", "batch": B, "context": C, "heads": heads, "kv_heads": kvh,
            "head_dim": hd, "splits": args.splits, "form": args.form or "auto", "us": round(us, 2), "bytes": nbytes,
            "GBps": round(nbytes / us / 1e3, 1)}


def grouped(args):
    from . import ops
    T, H, I, E, k = args.tokens, args.hidden, args.inter, args.experts, args.top_k
    dt = torch.bfloat16
    per_copy = E * 3 * I * H * 2
    n = _copies(per_copy)
    wgu = [torch.randn(E, 2 * I, H, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    wd = [torch.randn(E, H, I, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    x = torch.randn(T, H, device="cuda", dtype=dt)
    g = torch.Generator(device="cuda").manual_seed(0)
    idx = torch.stack([torch.randperm(E, device="cuda", generator=g)[:k] for _ in range(T)]
                      ).to(torch.int32)
    offsets, rows, dest = ops.moe_dispatch(idx, E)
    touched = int(torch.unique(idx).numel())
    act = ops.grouped_gate_up_swiglu(x, rows, offsets, wgu[0])

    def f1(i):
        ops.grouped_gate_up_swiglu(x, rows, offsets, wgu[i])

    def f2(i):
        ops.grouped_down(act, offsets, wd[i])
    us1 = _time(f1, n, args.iters)
    us2 = _time(f2, n, args.iters)
    b1, b2 = touched * 2 * I * H * 2, touched * I * H * 2
    fl1, fl2 = 2 * T * k * 2 * I * H, 2 * T * k * I * H
    return {"case": "grouped", "tokens": T, "experts_touched": touched,
            "gate_up_us": round(us1, 2), "gate_up_GBps": round(b1 / us1 / 1e3, 1),
            "gate_up_TFLOPs": round(fl1 / us1 / 1e6, 1),
            "down_us": round(us2, 2), "down_GBps": round(b2 / us2 / 1e3, 1),
            "down_TFLOPs": round(fl2 / us2 / 1e6, 1)}


def dense(args):
    from . import ops
    M, N, K = args.rows, args.n, args.k
    dt = torch.float32 if args.dtype == "float32" else torch.bfloat16
    n = _copies(N * K * 2)
    ws = [torch.randn(N, K, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    x = torch.randn(M, K, device="cuda", dtype=dt)

    def fn(i):
        if args.swiglu:
            ops.gate_up_swiglu(x, ws[i])
        else:
            ops.linear(x, ws[i])
    us = _time(fn, n, args.iters)
    nbytes = N * K * (4 if dt == torch.float32 else 2)
    return {"case": "dense", "rows": M, "n": N, "k": K, "swiglu": bool(args.swiglu),
            "dtype": args.dtype,
            "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1),
            "TFLOPs": round(2 * M * N * K / us / 1e6, 2)}


def qkv(args):
    """The QKV projection of a few-token step with bias, rotation and cache write: the one
    fused kernel, or (--separate) the product followed by the rotation kernel."""
    from . import ops
    T, H, heads, kvh, hd, page = args.rows, args.hidden, args.heads, args.kv_heads, args.head_dim, args.page
    dt = torch.bfloat16
    width = (heads + 2 * kvh) * hd
    n = _copies(width * H * 2)
    ws = [torch.randn(width, H, device="cuda", dtype=dt) * 0.02 for _ in range(n)]
    bias = torch.randn(width, device="cuda") * 0.1
    x = torch.randn(T, H, device="cuda", dtype=dt)
    positions = torch.arange(4000, 4000 + T, dtype=torch.int32, device="cuda")
    inv = (10000.0 ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().cuda()
    kc = torch.zeros(T + 1, kvh, page, hd, device="cuda", dtype=dt)
    vc = torch.zeros_like(kc)
    slots = (torch.arange(T, dtype=torch.int32, device="cuda") * page)
    ops.set_dependent_launch(True)

    def fused(i):
        ops.qkv_project_rope_append(x, ws[i], bias, positions, inv, hd, heads, kvh, hd, kc, vc, slots)

    def separate(i):
        ops.qkv_rope_append(ops.linear(x, ws[i]), bias, positions, inv, hd, heads, kvh, hd, kc, vc,
                            slots)
    us = _time(separate if args.separate else fused, n, args.iters)
    nbytes = width * H * 2
    return {"case": "qkv", "rows": T, "width": width, "k": H, "fused": not args.separate,
            "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}


def router(args):
    from . import ops
    T, H, E, k = args.tokens, args.hidden, args.experts, args.top_k
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, H, device="cuda", dtype=torch.float32) * 0.02
    extra = torch.randn(H, device="cuda", dtype=torch.float32) * 0.02

    def fn(i):
        ops.router_topk(x, w, k, False, 1.0, extra_w=extra)
    us = _time(fn, 1, args.iters)
    idx = ops.router_topk(x, w, k, False, 1.0, extra_w=extra)[1]

    def fd(i):
        ops.moe_dispatch(idx, E)
    return {"case": "router", "tokens": T, "router_us": round(us, 2),
            "dispatch_us": round(_time(fd, 1, args.iters), 2)}


def attn_prefill(args):
    from . import ops
    T, heads, kvh, hd, page = args.tokens, args.heads, args.kv_heads, args.head_dim, args.page
    dt = torch.float32 if args.dtype == "float32" else torch.bfloat16
    C = max(args.context if args.context_given else T, T)   # keys: the portion ends the context
    pages = -(-C // page)
    kc = torch.randn(pages, kvh, page, hd, device="cuda", dtype=dt)
    vc = torch.randn(pages, kvh, page, hd, device="cuda", dtype=dt)
    bt = torch.randperm(pages, device="cuda").to(torch.int32).view(1, pages)
    q = torch.randn(T, heads, hd, device="cuda", dtype=dt)
    step = types.SimpleNamespace(
        seq_of_token=torch.zeros(T, dtype=torch.int32, device="cuda"),
        positions=torch.arange(T, dtype=torch.int32, device="cuda"),
        cu_q=torch.tensor([0, T], dtype=torch.int32, device="cuda"),
        q_pos0=torch.full((1,), C - T, dtype=torch.int32, device="cuda"),
        kv_len=torch.full((1,), C, dtype=torch.int32, device="cuda"),
        max_q_len=T, max_kv_len=C, all_decode=False, num_seqs=1, num_tokens=T)
    scale = 1.0 / math.sqrt(hd)

    def fn(i):
        if args.form == "tiled":      # the CUDA-core kernel (any element type)
            ops.paged_attention_tiled(q, kc, vc, bt, step.cu_q, step.q_pos0, args.window, scale)
        else:
            ops.paged_attention_prefill(q, kc, vc, bt, step.cu_q, step.q_pos0, args.window, scale,
                                        kernel=args.form or None, splits=args.splits or None,
                                        softcap=args.softcap)
    us = _time(fn, 1, args.iters)
    flops = 4 * heads * hd * (T * T / 2 + T * (C - T))
    return {"case": "attn_prefill", "tokens": T, "context": C, "heads": heads, "head_dim": hd,
            "splits": args.splits or "auto",
            "form": args.form or "auto",
            "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 1)}


def latent_attn(args):
    """Attention over cached latent records: ``--tokens`` > 1 is one prompt of that many
    tokens; ``--tokens 1`` is ``--batch`` sequences of ``--context`` tokens bringing one
    token each.  FLOP = 2 * (2 * rank + rot) per (query row, visible key)."""
    from . import ops
    T, H, rank, dr, page, W = args.tokens, args.heads, args.rank, args.rot_dim, args.page, \
        args.window
    dt = torch.float32 if args.dtype == "float32" else torch.bfloat16
    decode = T == 1
    S = args.batch if decode else 1
    C = args.context if decode else max(args.context if args.context_given else T, T)
    pages_per_seq = -(-C // page)
    P = S * pages_per_seq
    per_copy = P * page * (rank + dr) * 2
    n = min(_copies(per_copy), 8) if decode else 1
    caches = [torch.randn(P, 1, page, rank + dr, device="cuda", dtype=dt) * 0.3 for _ in range(n)]
    bt = torch.randperm(P, device="cuda").to(torch.int32).view(S, pages_per_seq)
    rows = S * T
    q_lat = torch.randn(H, rows, rank, device="cuda", dtype=dt) * 0.3
    q_rot = torch.randn(rows, H, dr, device="cuda", dtype=dt) * 0.3
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    step = types.SimpleNamespace(
        seq_of_token=i32([s for s in range(S) for _ in range(T)]),
        positions=i32([C - T + t for _ in range(S) for t in range(T)]),
        cu_q=i32([s * T for s in range(S + 1)]), q_pos0=i32([C - T] * S), q_lens=[T] * S)
    scale = 1.0 / math.sqrt(rank)

    def fn(i):
        ops.latent_attention(q_lat, q_rot, caches[i], bt, step, W, scale,
                             kernel=args.form or None)
    us = _time(fn, n, args.iters)
    pairs = 0
    for t in range(T):
        pos = C - T + t
        pairs += min(pos + 1, W) if W else pos + 1
    pairs *= S * H
    flops = 2 * (2 * rank + dr) * pairs
    span = min(C, W + T - 1) if W else C
    nbytes = S * span * (rank + dr) * caches[0].element_size()
    return {"case": "latent_attn", "tokens": T, "batch": S, "context": C, "heads": H,
            "rank": rank, "rot_dim": dr, "window": W, "form": args.form or "auto",
            "us": round(us, 2), "TFLOPs": round(flops / us / 1e6, 2), "cache_bytes": nbytes,
            "GBps": round(nbytes / us / 1e3, 1)}


def rowwise(args):
    """The row-wise kernels of the sublayer-norm decoders beside the like kernels of the
    pre-norm ones, ``--tokens`` rows of ``--hidden`` (feed-forward ``--inter``): achieved
    GB/s over the bytes the operation has to move."""
    from . import ops
    T, W, I = args.tokens, args.hidden, args.inter
    dt = torch.bfloat16
    n = max(2, min(8, _copies(T * W * 14)))
    resid = [torch.randn(T, W, device="cuda") for _ in range(n)]
    delta32 = [torch.randn(T, W, device="cuda") for _ in range(n)]
    delta16 = [d.to(dt) for d in delta32]
    gu = [torch.randn(T, 2 * I, device="cuda", dtype=dt) for _ in range(n)]
    gain = torch.ones(W, device="cuda")
    mix = torch.rand(W, device="cuda")
    state = torch.zeros(2, W, device="cuda")
    H, D = args.heads, args.head_dim
    o = [torch.randn(H, T, D, device="cuda", dtype=dt) for _ in range(n)]
    proj = [torch.randn(T, H * D, device="cuda", dtype=dt) for _ in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    step = types.SimpleNamespace(cu_q=i32([0, T]), seq_of_token=torch.zeros(T, dtype=torch.int32,
                                                                            device="cuda"),
                                 state_slot=i32([1]))
    cases = {
        "token_shift": (lambda i: ops.token_shift(resid[i], mix, state, step, dt), 6 * T * W),
        "group_norm_add+cast": (lambda i: ops.group_norm_add(resid[i], delta32[i], gain, 4, 1e-5,
                                                             dt), 14 * T * W),
        "add_rmsnorm": (lambda i: ops.add_rmsnorm(resid[i], delta16[i], gain, 1e-5, dt),
                        12 * T * W),
        "glu_clamped": (lambda i: ops.glu_clamped(gu[i], 7.0, 1.702, 1.0), 6 * T * I),
        "silu_mul": (lambda i: ops.silu_mul(gu[i]), 6 * T * I),
        "gate_heads": (lambda i: ops.gate_heads(o[i], proj[i], 0), 6 * T * H * D),
    }
    out = {"case": "rowwise", "tokens": T, "hidden": W, "inter": I}
    for name, (fn, nbytes) in cases.items():
        us = _time(fn, n, args.iters)
        out[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
    return out


def recurrent(args):
    """The kernels of the recurrent mixers and of the parallel arrangement: ``--tokens`` rows
    of ``--hidden`` as one prompt (``--batch`` 1) or as that many sequences of one token
    (``--batch`` = ``--tokens``); heads of ``--head-dim`` key and value entries.  Achieved
    GB/s over the bytes the operation has to move."""
    from . import ops
    T, W, B = args.tokens, args.hidden, max(1, args.batch)
    K = V = args.head_dim
    H = W // K
    R = args.rank if args.rank <= 128 else 64
    dt = torch.bfloat16
    n = max(2, min(8, _copies(T * W * 14)))
    resid = [torch.randn(T, W, device="cuda") for _ in range(n)]
    d32 = [torch.randn(T, W, device="cuda") for _ in range(n)]
    d16 = [torch.randn(T, W, device="cuda", dtype=dt) for _ in range(n)]
    x16 = [torch.randn(T, W, device="cuda", dtype=dt) for _ in range(n)]
    gain = torch.ones(W, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    per = T // B
    step = types.SimpleNamespace(
        cu_q=i32([i * per for i in range(B + 1)]), num_seqs=B,
        seq_of_token=torch.arange(T, dtype=torch.int32, device="cuda") // per,
        state_slot=torch.arange(B, dtype=torch.int32, device="cuda"),
        positions=torch.arange(T, dtype=torch.int32, device="cuda") % per)
    mu = torch.rand(5, W, device="cuda")
    prev = torch.zeros(B, W, device="cuda")
    states = [torch.zeros(B, H, K, V, device="cuda") for _ in range(n)]
    qkv = [torch.randn(3, T, H * K, device="cuda", dtype=dt) * 0.1 for _ in range(n)]
    decay = [torch.rand(T, H * K, device="cuda") * 0.1 + 0.9 for _ in range(n)]
    u = torch.randn(H, K, device="cuda")
    low = [torch.randn(T, R, device="cuda") for _ in range(n)]
    w2 = torch.randn(R, H * K, device="cuda") * 0.1
    b = torch.zeros(H * K, device="cuda")
    o = [torch.randn(T, H, V, device="cuda") for _ in range(n)]
    G = max(1, H // 4)
    qk = [torch.randn(T, (H + G) * K, device="cuda", dtype=dt) for _ in range(n)]
    pages = -(-T // 16) + 1
    kc = torch.zeros(pages, G, 16, K, device="cuda", dtype=dt)
    vc = torch.zeros_like(kc)
    slots = torch.arange(T, dtype=torch.int32, device="cuda")
    state_bytes = 2 * B * H * K * V * 4
    cases = {
        "add_rmsnorm_sum(2 terms, 2 norms)": (
            lambda i: ops.add_rmsnorm_sum(resid[i], [d32[i], d16[i]], None, (gain, gain), 1e-5, dt),
            (8 + 4 + 2 + 4) * T * W),
        "add_rmsnorm": (lambda i: ops.add_rmsnorm(resid[i], d16[i], gain, 1e-5, dt), 12 * T * W),
        "shift_mix(5)": (lambda i: ops.shift_mix(x16[i], mu, prev, step), 12 * T * W),
        "lowrank_decay": (lambda i: ops.lowrank_decay(low[i], w2, b, "exp_exp_tanh"),
                          4 * T * (R + H * K)),
        "linear_recurrence(bonus)": (
            lambda i: ops.linear_recurrence(qkv[i][0], qkv[i][1], qkv[i][2], decay[i], u,
                                            states[i], step, H, K, V, 1.0, True),
            T * H * (3 * K * 2 + K * 4 + V * 4) + state_bytes),
        "linear_recurrence(plain)": (
            lambda i: ops.linear_recurrence(qkv[i][0], qkv[i][1], qkv[i][2], decay[i], None,
                                            states[i], step, H, K, V, 0.125, False),
            T * H * (3 * K * 2 + K * 4 + V * 4) + state_bytes),
        "head_norm_gate": (lambda i: ops.head_norm_gate(o[i], gain, x16[i], 1e-5, dt),
                           (4 + 2 + 2) * T * W),
        "qk_norm_append": (
            lambda i: ops.qk_norm_append(qk[i], gain[:K], gain[:K], step.positions, H, G, K, 1e-5,
                                         0.1, 128, kc, vc, slots),
            T * K * (2 * (H + G) + 2 * H + 4 * G)),
    }
    out = {"case": "recurrent", "tokens": T, "sequences": B, "hidden": W, "heads": H,
           "head_dim": K, "rank": R}
    for name, (fn, nbytes) in cases.items():
        us = _time(fn, n, args.iters)
        out[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
    flops = 2 * 3 * T * H * K * V      # decay, outer product and read-out per state entry
    us = out["linear_recurrence(bonus)"]["us"]
    out["linear_recurrence(bonus)"]["TFLOPs_fp32"] = round(flops / us / 1e6, 2)
    return out


def delta(args):
    """The kernels of the convolution-and-state mixers and of the scaled pre-norm arrangement:
    ``--tokens`` rows of ``--hidden`` as one prompt (``--batch`` 1) or as that many sequences
    of one token (``--batch`` = ``--tokens``).  State-space heads of 64 values with 128 state
    entries in 2 groups; delta heads of 64 key and 128 value entries; convolutions of 4 taps.
    With ``--context``: single-token attention over that many keys for heads of
    ``--head-dim`` keys and twice as wide values, on the kernel of any size.  Achieved GB/s
    over the bytes the operation has to move."""
    from . import ops
    T, W, B = args.tokens, args.hidden, max(1, args.batch)
    dt = torch.bfloat16
    n = max(2, min(8, _copies(T * W * 14)))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    per = T // B
    step = types.SimpleNamespace(
        cu_q=i32([i * per for i in range(B + 1)]), num_seqs=B, max_q_len=per, num_tokens=T,
        seq_of_token=torch.arange(T, dtype=torch.int32, device="cuda") // per,
        state_slot=torch.arange(B, dtype=torch.int32, device="cuda"),
        positions=torch.arange(T, dtype=torch.int32, device="cuda") % per)
    gain = torch.ones(W, device="cuda")
    resid = [torch.randn(T, W, device="cuda") for _ in range(n)]
    d32 = [torch.randn(T, W, device="cuda") for _ in range(n)]
    x16 = [torch.randn(T, W, device="cuda", dtype=dt) for _ in range(n)]
    # state space: heads of 64 values, 128 state entries, 2 groups
    SH, SV, SN, SG = W // 64, 64, 128, 2
    cw = SH * SV + 2 * SG * SN
    xbc = [torch.randn(T, cw, device="cuda", dtype=dt) * 0.3 for _ in range(n)]
    sdt = [torch.randn(T, SH, device="cuda", dtype=dt) for _ in range(n)]
    hp = [torch.randn(SH, device="cuda") for _ in range(3)]
    s_states = [torch.zeros(B, SH, SN, SV, device="cuda") for _ in range(n)]
    conv_w, conv_b = torch.randn(cw, 4, device="cuda"), torch.randn(cw, device="cuda")
    conv_st = torch.zeros(B, 3, cw, device="cuda")
    y32 = [torch.randn(T, SH * SV, device="cuda") for _ in range(n)]
    # delta rule: heads of 64 key and 128 value entries
    DH, DK, DV = W // 128, 64, 128
    dq = [torch.randn(2, T, DH * DK, device="cuda", dtype=dt) for _ in range(n)]
    dv = [torch.randn(T, DH * DV, device="cuda", dtype=dt) for _ in range(n)]
    beta = [torch.randn(T, DH, device="cuda", dtype=dt) for _ in range(n)]
    decay = [torch.rand(T, DH * DK, device="cuda") * 0.1 + 0.9 for _ in range(n)]
    d_states = [torch.zeros(B, DH, DK, DV, device="cuda") for _ in range(n)]
    R = 64
    low = [torch.randn(T, R, device="cuda", dtype=dt) for _ in range(n)]
    w2 = torch.randn(R, DH * DK, device="cuda") * 0.1
    rate = torch.zeros(DH, device="cuda")
    o = [torch.randn(T, DH, DV, device="cuda") for _ in range(n)]
    cases = {
        "add_scaled_norm(layer norm)": (
            lambda i: ops.add_scaled_norm(resid[i], d32[i], 0.5, None, gain, 1e-5, dt),
            (8 + 4 + 2) * T * W),
        "causal_conv(4 taps, silu)": (
            lambda i: ops.causal_conv(xbc[i], conv_w, conv_b, conv_st, step), 4 * T * cw),
        "ssd_recurrence": (
            lambda i: ops.ssd_recurrence(xbc[i], sdt[i], *hp, s_states[i], step, SH, SV, SN, SG),
            T * (2 * cw + 4 * SH * SV) + 2 * B * SH * SN * SV * 4),
        "gated_group_norm": (
            lambda i: ops.gated_group_norm(y32[i], x16[i][:, :SH * SV], gain[:SH * SV], 2, 1e-5),
            (4 + 2 + 2) * T * SH * SV),
        "normed_pair_mean": (
            lambda i: ops.normed_pair_mean(d32[i], resid[i], gain, gain, 1e-5), 12 * T * W),
        "lowrank_decay(softplus rate)": (
            lambda i: ops.lowrank_decay(low[i], w2, torch.zeros_like(w2[0]), "exp_rate_softplus",
                                        head_log_rate=rate), T * (2 * R + 4 * DH * DK)),
        "delta_recurrence": (
            lambda i: ops.delta_recurrence(dq[i][0], dq[i][1], dv[i], beta[i], decay[i],
                                           d_states[i], step, DH, DH, DK, DV, 1e-6, 0.125),
            T * DH * (2 * DK * 2 + DK * 4 + DV * 2 + DV * 4) + 2 * B * DH * DK * DV * 4),
        "head_norm_gate(sigmoid)": (
            lambda i: ops.head_norm_gate(o[i], gain[:DV], x16[i][:, :DH * DV], 1e-5, dt,
                                         gate_form="sigmoid"), (4 + 2 + 2) * T * DH * DV),
    }
    out = {"case": "delta", "tokens": T, "sequences": B, "hidden": W}
    for name, (fn, nbytes) in cases.items():
        us = _time(fn, n, args.iters)
        out[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
    out["ssd_recurrence"]["TFLOPs_fp32"] = round(
        2 * 3 * T * SH * SN * SV / out["ssd_recurrence"]["us"] / 1e6, 2)
    out["delta_recurrence"]["TFLOPs_fp32"] = round(
        2 * 4 * T * DH * DK * DV / out["delta_recurrence"]["us"] / 1e6, 2)
    if args.context:
        S, C, hd, page = max(1, args.batch), args.context, args.head_dim, args.page
        heads, kvh, vd = args.heads, args.kv_heads, 2 * args.head_dim
        blocks = -(-C // page)
        m = max(2, min(8, _copies(S * kvh * C * (hd + vd) * 2)))
        kcs = [torch.randn(S * blocks, kvh, page, hd, device="cuda", dtype=dt) for _ in range(m)]
        vcs = [torch.randn(S * blocks, kvh, page, vd, device="cuda", dtype=dt) for _ in range(m)]
        bt = torch.arange(S * blocks, dtype=torch.int32, device="cuda").view(S, blocks)
        kv_len = torch.full((S,), C, dtype=torch.int32, device="cuda")
        qs = torch.randn(S, heads, hd, device="cuda", dtype=dt)
        us = _time(lambda i: ops.paged_attention_decode_any(qs, kcs[i], vcs[i], bt, kv_len, C, 0,
                                                            hd ** -0.5), m, args.iters)
        nbytes = S * kvh * C * (hd + vd) * 2
        out["paged_attention_decode_any"] = {
            "sequences": S, "context": C, "heads": heads, "kv_heads": kvh, "head_dim": hd,
            "value_dim": vd, "us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
    return out


def prepared(args):
    """The kernels of the decoders with prepared attention, each beside the like kernel of
    the Qwen2-MoE path at the same sizes: ``--tokens`` rows of ``--hidden``, ``--heads``
    over ``--kv-heads`` heads of ``--head-dim`` (keys and values), a feed-forward of
    ``--inter``, ``--experts`` router outputs of which ``--top-k`` are chosen; attention of
    one prompt of ``--tokens`` tokens, and of ``--batch`` single tokens at ``--context``,
    over a window of ``--window`` (1024 when not given).  GB/s over the bytes the operation
    has to move; attention also as GFLOP/s of its two products."""
    from . import ops
    T, W, I = args.tokens, args.hidden, args.inter
    H, G, D = args.heads, args.kv_heads, args.head_dim
    E, K = args.experts, args.top_k
    win = args.window or 1024
    dt = torch.bfloat16
    dev = "cuda"
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    n = max(2, min(8, _copies(T * W * 8)))
    vocab, buckets = 32000, 65521
    table = torch.randn(vocab, W, device=dev, dtype=dt)
    pairs = torch.randn(buckets + 1, W, device=dev, dtype=dt)
    gain = torch.ones(W, device=dev)
    ids = [torch.randint(0, vocab, (T,), device=dev, dtype=torch.int32) for _ in range(n)]
    step = types.SimpleNamespace(
        cu_q=i32([0, T]), seq_of_token=torch.zeros(T, dtype=torch.int32, device=dev),
        state_slot=i32([0]), positions=torch.arange(T, dtype=torch.int32, device=dev),
        q_pos0=i32([0]), token_ids=ids[0], num_seqs=1, num_tokens=T)
    prev = torch.zeros(2, 1, dtype=torch.int32, device=dev)

    def embed_pair(i):
        step.token_ids = ids[i]
        ops.embed_pair_norm(table, pairs, gain, step, prev, buckets, 31, 7, 1e-6)
    dq, dk = H * D, G * D
    row = dq + 2 * dk
    qkv = [torch.randn(T, row, device=dev, dtype=dt) for _ in range(n)]
    page = args.page
    P = -(-T // page) + 1
    kc = torch.zeros(P, G, page, D, device=dev, dtype=dt)
    vc = torch.zeros(P, G, page, D, device=dev, dtype=dt)
    slots = torch.arange(T, dtype=torch.int32, device=dev)
    freq = torch.rand(D // 2, device=dev)
    qg, kg = torch.ones(dq, device=dev), torch.ones(dk, device=dev)
    lam = torch.tensor([0.3], device=dev)
    earlier = [torch.randn(T, dk, device=dev, dtype=dt) for _ in range(n)]
    gu = [torch.randn(T, 2 * I, device=dev, dtype=dt) for _ in range(n)]
    bias = torch.randn(2 * I, device=dev)
    x = [torch.randn(T, W, device=dev, dtype=dt) for _ in range(n)]
    rw = torch.randn(E, W, device=dev) * 0.05
    corr = torch.randn(E, device=dev) * 0.1
    groups = 4 if E % 4 == 0 else 1
    keep = 2 if groups == 4 and 2 * (E // 4) >= K else groups
    cases = {
        "embed_pair_norm": (embed_pair, T * W * (2 + 2 + 4)),
        "embed (like)": (lambda i: ops.embed(table, ids[i]), T * W * (2 + 4)),
        "attention_prepare (projection norm, half rotation, blend)": (
            lambda i: ops.attention_prepare(qkv[i], step.positions, freq, 1.1, D, False, H, G, D,
                                            D, qg, kg, 1e-6, False, earlier[i], lam, kc, vc,
                                            slots), T * (2 * row * 2 + dk * 2)),
        "attention_prepare (pair rotation, unit heads)": (
            lambda i: ops.attention_prepare(qkv[i], step.positions, freq[:D // 4].contiguous(),
                                            1.0, D // 2, True, H, G, D, D, None, None, 1e-6, True,
                                            None, None, kc, vc, slots), T * 2 * row * 2),
        "qkv_rope_append (like)": (
            lambda i: ops.qkv_rope_append(qkv[i], None, step.positions, freq, D, H, G, D, kc, vc,
                                          slots), T * 2 * row * 2),
        "glu_bias_act (gelu_tanh, biases)": (lambda i: ops.glu_bias_act(gu[i], bias, "gelu_tanh"),
                                             6 * T * I),
        "silu_mul (like)": (lambda i: ops.silu_mul(gu[i]), 6 * T * I),
        "router_topk (correction, groups, sum + eps)": (
            lambda i: ops.router_topk(x[i], rw, K, True, 1.0, correction=corr, group_count=groups,
                                      group_keep=keep, renorm_eps=1e-20), T * W * 2),
        "router_topk (like)": (lambda i: ops.router_topk(x[i], rw, K, True, 1.0), T * W * 2),
    }
    out = {"case": "prepared", "tokens": T, "hidden": W, "inter": I, "heads": H, "kv_heads": G,
           "head_dim": D, "experts": E, "top_k": K, "window": win}
    for name, (fn, nbytes) in cases.items():
        us = _time(fn, n, args.iters)
        out[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
    # attention: one prompt of T tokens over the window; B single tokens at the context
    scale = 1.0 / math.sqrt(D)
    pages = -(-T // page)
    kp = torch.randn(pages, G, page, D, device=dev, dtype=dt) * 0.3
    vp = torch.randn(pages, G, page, D, device=dev, dtype=dt)
    bt = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    q = torch.randn(T, H, D, device=dev, dtype=dt) * 0.3
    seen = sum(min(p + 1, win) for p in range(T))
    flops = 4.0 * H * D * seen
    prompt = {
        "tiled fp32 weights, kept first keys, sink": lambda i: ops.paged_attention_tiled(
            q, kp, vp, bt, step.cu_q, step.q_pos0, win, scale, 0.0, 4, True),
        "tiled fp32 weights": lambda i: ops.paged_attention_tiled(
            q, kp, vp, bt, step.cu_q, step.q_pos0, win, scale),
        "tcgen05 16-bit weights, kept first keys, sink": lambda i:
            ops.paged_attention_prefill_exact(q, kp, vp, bt, step.cu_q, step.q_pos0, win, scale,
                                              4, True, kernel="tc"),
        "mma.sync 16-bit weights, kept first keys, sink": lambda i:
            ops.paged_attention_prefill_exact(q, kp, vp, bt, step.cu_q, step.q_pos0, win, scale,
                                              4, True, kernel="mma"),
        "mma.sync 8-bit weights (like, older form)": lambda i: ops.paged_attention_prefill(
            q, kp, vp, bt, step.cu_q, step.q_pos0, win, scale, kernel="mma"),
        "tcgen05 (like)": lambda i: ops.paged_attention_prefill(
            q, kp, vp, bt, step.cu_q, step.q_pos0, win, scale, max_kv_len=T),
    }
    for name, fn in prompt.items():
        us = _time(fn, 1, max(3, args.iters // 10))
        out[f"prompt attention: {name}"] = {"us": round(us, 1),
                                            "GFLOPs": round(flops / us / 1e3, 1)}
    B, C = args.batch, args.context
    per_seq = -(-C // page)
    nc = min(_copies(B * min(C, win) * G * D * 4), 8)
    kcs = [torch.randn(B * per_seq, G, page, D, device=dev, dtype=dt) * 0.3 for _ in range(nc)]
    vcs = [torch.randn(B * per_seq, G, page, D, device=dev, dtype=dt) for _ in range(nc)]
    btd = torch.randperm(B * per_seq, device=dev).to(torch.int32).view(B, per_seq)
    qd = torch.randn(B, H, D, device=dev, dtype=dt) * 0.3
    kv_len = torch.full((B,), C, dtype=torch.int32, device=dev)
    nbytes = B * min(C, win) * G * D * 2 * 2
    single = {
        "any-size fp32 weights, kept first keys, sink": lambda i: ops.paged_attention_decode_any(
            qd, kcs[i], vcs[i], btd, kv_len, C, win, scale, keep_first=4, sink=True),
        "any-size fp32 weights": lambda i: ops.paged_attention_decode_any(
            qd, kcs[i], vcs[i], btd, kv_len, C, win, scale),
        "mma.sync 16-bit weights, kept first keys, sink": lambda i:
            ops.paged_attention_decode_exact(qd, kcs[i], vcs[i], btd, kv_len, C, win, scale,
                                             keep_first=4, sink=True),
        "mma.sync 8-bit weights (like, older form)": lambda i: ops.paged_attention_decode(
            qd, kcs[i], vcs[i], btd, kv_len, C, win, scale, kernel="mma"),
        "TMA (like)": lambda i: ops.paged_attention_decode(qd, kcs[i], vcs[i], btd, kv_len, C,
                                                           win, scale),
    }
    for name, fn in single.items():
        us = _time(fn, nc, args.iters)
        out[f"single-token attention: {name}"] = {"us": round(us, 2),
                                                  "GBps": round(nbytes / us / 1e3, 1)}
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=["attn_decode", "grouped", "dense", "attn_prefill", "router",
                                     "qkv", "latent_attn", "rowwise", "recurrent", "delta",
                                     "prepared"])
    ap.add_argument("--softcap", type=float, default=0.0,
                    help="attn_decode, attn_prefill: squash scores to softcap * tanh(s / softcap)")
    ap.add_argument("--rank", type=int, default=512, help="latent_attn: entries of the latent")
    ap.add_argument("--rot-dim", type=int, default=64, help="latent_attn: rotated key entries")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--form", default="", help="attn_decode: tma, mma or scalar; attn_prefill: tc, mma or tiled (default: auto)")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=1408)
    ap.add_argument("--experts", type=int, default=60)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="dense, attn_prefill --form tiled: the element type")
    ap.add_argument("--separate", action="store_true",
                    help="qkv: the product and the rotation as two kernels")
    ap.add_argument("--eager", action="store_true", help="plain launches, no graph capture")
    args = ap.parse_args(argv)
    args.context_given = any(a == "--context" or a.startswith("--context=") for a in (argv or sys.argv[1:]))
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 3
    EAGER[0] = args.eager
    print(json.dumps(globals()[args.case](args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
