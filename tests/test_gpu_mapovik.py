"""The Mapovik design on the GPU: every new kernel alone against its plain statement
(tests/host_ops.py), then the engine against the plain model (tests/plain_mapovik.py):
whole prompts, prefill against token-by-token decoding, portions down to two tokens,
unequal batches with pages and slots used again, long decoding with recorded steps, and
greedy generation through the engine's own entry point."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import host_ops
import mapovik_cases as mk
import model_cases as mc
import plain_mapovik as plain
import traces
from conftest import ROOT
from inferx_b200.engine.replay import ReplaySession

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _ops():
    from inferx_b200.kernels import ops
    return ops


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


def _step(q_lens, starts, slots=None):
    """A batch description: sequence s brings q_lens[s] tokens from position starts[s]."""
    seq_of, pos, cu = [], [], [0]
    for s, (n, a) in enumerate(zip(q_lens, starts)):
        seq_of += [s] * n
        pos += list(range(a, a + n))
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return SimpleNamespace(
        seq_of_token=i32(seq_of), positions=i32(pos), cu_q=i32(cu), q_pos0=i32(list(starts)),
        q_lens=list(q_lens), num_seqs=len(q_lens), num_tokens=len(seq_of),
        kv_len=i32([a + n for n, a in zip(q_lens, starts)]),
        max_kv_len=max(a + n for n, a in zip(q_lens, starts)), max_q_len=max(q_lens),
        all_decode=all(n == 1 for n in q_lens), num_decode_seqs=0, cu_q_prompt=None,
        state_slot=i32(slots if slots is not None else list(range(len(q_lens)))))


def _cuda(ns):
    return SimpleNamespace(**{k: (v.cuda() if torch.is_tensor(v) else v)
                              for k, v in vars(ns).items()})


def _rel(a, b):
    return float((a - b).abs().max()) / max(float(b.abs().max()), 1e-30)


# -- kernels alone -------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 2048, 61, 7168])
@pytest.mark.parametrize("center", [True, False])
def test_scaled_add_and_norm(dtype, width, center):
    g = torch.Generator().manual_seed(width)
    T = 7
    resid = torch.randn(T, width, generator=g) + 3.0      # a mean that centring must remove
    gain = 1.0 + 0.3 * torch.randn(width, generator=g)
    vec = torch.randn(width, generator=g)
    for delta in (torch.randn(T, width, generator=g), torch.randn(T, width, generator=g).to(dtype),
                  None):
        for v in (None, vec):
            r_ref = resid.clone()
            ref = host_ops.add_scaled_norm(r_ref, delta, 0.35, v, gain, 1e-5, dtype, center)
            r = resid.cuda()
            out = _ops().add_scaled_norm(r, None if delta is None else delta.cuda(), 0.35,
                                         None if v is None else v.cuda(), gain.cuda(), 1e-5, dtype,
                                         center)
            torch.testing.assert_close(r.cpu(), r_ref, rtol=2e-6, atol=2e-6)
            torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    rows = torch.tensor([6, 0, 3, 3], dtype=torch.int32)
    delta = torch.randn(T, width, generator=g)
    ref = host_ops.add_scaled_norm(resid.clone(), delta, 0.5, vec, gain, 1e-5, dtype, center,
                                   rows=rows)
    r = resid.cuda()
    out = _ops().add_scaled_norm(r, delta.cuda(), 0.5, vec.cuda(), gain.cuda(), 1e-5, dtype, center,
                                 rows=rows.cuda())
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    assert torch.equal(r.cpu(), resid)            # gathered rows leave the stream alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 1024, 61])
def test_stream_concat(dtype, width):
    g = torch.Generator().manual_seed(width)
    T = 5
    resid, first, delta = (torch.randn(T, width, generator=g) for _ in range(3))
    vec = torch.randn(width, generator=g)
    for d, v in ((delta, vec), (delta.to(dtype), None), (None, vec), (None, None)):
        ref = host_ops.stream_concat(resid, d, 0.7, v, first, dtype)
        r = resid.cuda()
        out = _ops().stream_concat(r, None if d is None else d.cuda(), 0.7,
                                   None if v is None else v.cuda(), first.cuda(), dtype)
        assert out.shape == (T, 2 * width) and torch.equal(r.cpu(), resid)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,taps,bias", [(40, 4, True), (33, 2, False), (130, 5, True),
                                         (7, 1, False), (512, 3, False)])
def test_causal_conv_reads_and_moves_the_kept_inputs(dtype, C, taps, bias):
    """Sequences that bring fewer tokens than the taps reach back, exactly as many, more,
    and one token; a slot of no sequence is untouched."""
    g = torch.Generator().manual_seed(C + taps)
    q_lens = [1, taps - 1 or 1, 9, 2, taps + 3]
    step = _step(q_lens, [30, 0, 5, 11, 0], slots=[4, 0, 2, 5, 1])
    T = sum(q_lens)
    wide = torch.randn(T, C + 6, generator=g).to(dtype)
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    state = torch.randn(7, taps - 1, C, generator=g)
    st_ref = state.clone()
    ref = host_ops.causal_conv(wide[:, 3:3 + C], w, b, st_ref, step, silu=True)
    st = state.cuda()
    out = _ops().causal_conv(wide.cuda()[:, 3:3 + C], w.cuda(), None if b is None else b.cuda(),
                             st, _cuda(step), silu=True)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    torch.testing.assert_close(st.cpu(), st_ref, rtol=1e-6, atol=1e-6)
    assert torch.equal(st.cpu()[3], state[3]) and torch.equal(st.cpu()[6], state[6])


def test_causal_conv_does_not_depend_on_the_cut():
    C, taps, T = 50, 4, 23
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, C, generator=g).to(torch.bfloat16).cuda()
    w, b = torch.randn(C, taps, generator=g).cuda(), torch.randn(C, generator=g).cuda()
    st0 = torch.zeros(2, taps - 1, C, device="cuda")
    whole = _ops().causal_conv(x, w, b, st0, _cuda(_step([T], [0], [1])))
    st1 = torch.zeros(2, taps - 1, C, device="cuda")
    parts, at = [], 0
    for n in (2, 1, 1, 5, 2, 3, 1, 8):
        xx = torch.cat([x[:2], x[at:at + n]]).contiguous()        # beside another sequence
        o = _ops().causal_conv(xx, w, b, st1, _cuda(_step([2, n], [0, at], [0, 1])))
        parts.append(o[2:])
        at += n
    assert at == T and torch.equal(torch.cat(parts), whole) and torch.equal(st0[1], st1[1])
    # the first tokens see zeros before them: token 0 is act(b + w[:, -1] * x[0])
    z = b + w[:, -1] * x[0].float()
    torch.testing.assert_close(whole[0].float(), (z * torch.sigmoid(z)), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,taps,bias", [(64, 4, True), (38, 2, False), (258, 3, True)])
def test_causal_conv_of_long_steps_walks_runs_of_tokens(dtype, C, taps, bias):
    """Steps of a thousand tokens and more: sequences that begin inside a run of tokens, at
    its first and at its last token, a sequence of one token, kept inputs from earlier; the
    same bits as the same tokens in short steps."""
    g = torch.Generator().manual_seed(C * taps)
    q_lens = [16, 1000, 1, 15, 2, 331]
    starts = [0, 7, 3, 0, 1, 40]
    step = _step(q_lens, starts, slots=[5, 0, 2, 4, 1, 6])
    T = sum(q_lens)
    wide = torch.randn(T, C + 6, generator=g).to(dtype)
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g) if bias else None
    state = torch.randn(7, taps - 1, C, generator=g)
    st_ref = state.clone()
    ref = host_ops.causal_conv(wide[:, 2:2 + C], w, b, st_ref, step, silu=True)
    st = state.cuda()
    bc = None if b is None else b.cuda()
    out = _ops().causal_conv(wide.cuda()[:, 2:2 + C], w.cuda(), bc, st, _cuda(step), silu=True)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    torch.testing.assert_close(st.cpu(), st_ref, rtol=1e-6, atol=1e-6)
    # sequence by sequence in portions of at most 300 tokens (the kernel of single tokens)
    st2, at, parts = state.cuda(), 0, []
    for n_all, p0, slot in zip(q_lens, starts, [5, 0, 2, 4, 1, 6]):
        done = 0
        while done < n_all:
            n = min(300, n_all - done)
            xx = wide.cuda()[at + done:at + done + n, 2:2 + C]
            parts.append(_ops().causal_conv(xx, w.cuda(), bc, st2,
                                            _cuda(_step([n], [p0 + done], [slot])), silu=True))
            done += n
        at += n_all
    assert torch.equal(torch.cat(parts), out) and torch.equal(st2, st)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V,N,G", [(4, 24, 32, 2), (3, 8, 12, 1), (5, 3, 7, 5), (2, 64, 128, 1),
                                     (8, 40, 64, 4), (1, 100, 16, 1)])
def test_state_space_recurrence(dtype, H, V, N, G):
    g = torch.Generator().manual_seed(H * V + N)
    q_lens = [1, 37, 2, 16, 17]
    step = _step(q_lens, [9, 0, 4, 0, 3], slots=[5, 0, 2, 4, 1])
    T = sum(q_lens)
    width = H * V + 2 * G * N
    wide = (torch.randn(T, width + H + 4, generator=g) * 0.7).to(dtype)
    xbc, dt = wide[:, 2:2 + width], wide[:, 2 + width:2 + width + H]
    dt_bias, a_log, d_skip = (torch.randn(H, generator=g) for _ in range(3))
    state = torch.randn(6, H, N, V, generator=g)
    st_ref = state.clone()
    ref = host_ops.ssd_recurrence(xbc, dt, dt_bias, a_log, d_skip, st_ref, step, H, V, N, G)
    st, wd = state.cuda(), wide.cuda()
    out = _ops().ssd_recurrence(wd[:, 2:2 + width], wd[:, 2 + width:2 + width + H], dt_bias.cuda(),
                                a_log.cuda(), d_skip.cuda(), st, _cuda(step), H, V, N, G)
    assert _rel(out.cpu(), ref) <= 2e-5 and _rel(st.cpu(), st_ref) <= 2e-5
    assert torch.equal(st.cpu()[3], state[3])     # a slot of no sequence is untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V,N,G", [(2, 40, 24, 1), (4, 64, 128, 2), (3, 5, 7, 3)])
def test_state_space_recurrence_in_segments(dtype, H, V, N, G):
    """Long prompts are walked in segments side by side and joined: a long prompt beside a
    single token and a portion that continues a state, against the plain walk and against the
    same tokens in portions too short to be cut."""
    g = torch.Generator().manual_seed(H + V + N)
    q_lens = [700, 1, 131]
    step = _step(q_lens, [0, 40, 64], slots=[2, 0, 1])
    T = sum(q_lens)
    width = H * V + 2 * G * N
    xbc = (torch.randn(T, width, generator=g) * 0.7).to(dtype)
    dt = torch.randn(T, H, generator=g).to(dtype)
    dt_bias, a_log, d_skip = (torch.randn(H, generator=g) for _ in range(3))
    a_log -= 2.0                                   # decays near 1: far tokens stay in the state
    state = torch.randn(3, H, N, V, generator=g)
    st_ref = state.clone()
    ref = host_ops.ssd_recurrence(xbc, dt, dt_bias, a_log, d_skip, st_ref, step, H, V, N, G)
    hp = [t.cuda() for t in (dt_bias, a_log, d_skip)]
    st = state.cuda()
    out = _ops().ssd_recurrence(xbc.cuda(), dt.cuda(), *hp, st, _cuda(step), H, V, N, G)
    assert _rel(out.cpu(), ref) <= 3e-5 and _rel(st.cpu(), st_ref) <= 3e-5
    st2, at, outs = state.cuda(), 0, []
    while at < 700:
        n = min(100, 700 - at)
        outs.append(_ops().ssd_recurrence(xbc[at:at + n].cuda(), dt[at:at + n].cuda(), *hp, st2,
                                          _cuda(_step([n], [at], [2])), H, V, N, G))
        at += n
    assert _rel(torch.cat(outs).cpu(), out[:700].cpu()) <= 1e-5
    assert _rel(st2[2].cpu(), st[2].cpu()) <= 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,HK,K,V", [(4, 4, 32, 48), (4, 2, 12, 20), (6, 3, 5, 9), (2, 1, 128, 64),
                                      (3, 1, 7, 5), (2, 2, 64, 128), (1, 1, 24, 100)])
def test_delta_recurrence(dtype, H, HK, K, V):
    g = torch.Generator().manual_seed(H * K + V)
    q_lens = [1, 37, 2, 16, 17]
    step = _step(q_lens, [9, 0, 4, 0, 3], slots=[5, 0, 2, 4, 1])
    T = sum(q_lens)
    wide = torch.randn(T, 2 * HK * K + H * V + H + 2, generator=g).to(dtype)
    cut = [1, 1 + HK * K, 1 + 2 * HK * K, 1 + 2 * HK * K + H * V, 1 + 2 * HK * K + H * V + H]
    decay = torch.rand(T, H * K, generator=g) * 0.6 + 0.4
    state = torch.randn(6, H, K, V, generator=g)
    st_ref = state.clone()
    views = lambda t: [t[:, a:b] for a, b in zip(cut[:-1], cut[1:])]
    ref = host_ops.delta_recurrence(*views(wide), decay, st_ref, step, H, HK, K, V, 1e-6,
                                    K ** -0.5)
    st = state.cuda()
    out = _ops().delta_recurrence(*views(wide.cuda()), decay.cuda(), st, _cuda(step), H, HK, K, V,
                                  1e-6, K ** -0.5)
    assert _rel(out.cpu(), ref) <= 3e-5 and _rel(st.cpu(), st_ref) <= 3e-5
    assert torch.equal(st.cpu()[3], state[3])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,HK,K,V", [(2, 1, 24, 40), (4, 2, 64, 128), (3, 3, 5, 7), (2, 2, 128, 32),
                                      (1, 1, 40, 33)])
def test_delta_recurrence_in_segments(dtype, H, HK, K, V):
    """Long prompts are walked in segments whose start states are rebuilt from each earlier
    segment's own state and the product of its transition matrices: a long prompt beside a
    single token and a portion that continues a state, against the plain walk and against
    the same tokens in portions too short to be cut."""
    g = torch.Generator().manual_seed(H * K + V)
    q_lens = [700, 1, 131]
    step = _step(q_lens, [0, 40, 64], slots=[2, 0, 1])
    T = sum(q_lens)
    q, k = (torch.randn(T, HK * K, generator=g).to(dtype) for _ in range(2))
    v = torch.randn(T, H * V, generator=g).to(dtype)
    beta = (torch.randn(T, H, generator=g) * 2).to(dtype)
    decay = torch.rand(T, H * K, generator=g) * 0.1 + 0.9      # far tokens stay in the state
    state = torch.randn(3, H, K, V, generator=g)
    st_ref = state.clone()
    ref = host_ops.delta_recurrence(q, k, v, beta, decay, st_ref, step, H, HK, K, V, 1e-6,
                                    K ** -0.5)
    st = state.cuda()
    args = lambda sl: [t[sl].cuda() for t in (q, k, v, beta, decay)]
    out = _ops().delta_recurrence(*args(slice(0, T)), st, _cuda(step), H, HK, K, V, 1e-6,
                                  K ** -0.5)
    assert _rel(out.cpu(), ref) <= 5e-5 and _rel(st.cpu(), st_ref) <= 5e-5
    st2, at, outs = state.cuda(), 0, []
    while at < 700:
        n = min(100, 700 - at)
        outs.append(_ops().delta_recurrence(*args(slice(at, at + n)), st2,
                                            _cuda(_step([n], [at], [2])), H, HK, K, V, 1e-6,
                                            K ** -0.5))
        at += n
    assert _rel(torch.cat(outs).cpu(), out[:700].cpu()) <= 2e-5
    assert _rel(st2[2].cpu(), st[2].cpu()) <= 2e-5


def test_recurrences_do_not_depend_on_the_cut():
    """The same tokens in one step, in portions and one by one, alone and beside another
    sequence: the same bits, in the outputs and in the states."""
    ops = _ops()
    H, HK, K, V, G, T = 4, 2, 48, 40, 2, 45
    g = torch.Generator().manual_seed(1)
    q, k = (torch.randn(T, HK * K, generator=g).to(torch.bfloat16).cuda() for _ in range(2))
    v = torch.randn(T, H * V, generator=g).to(torch.bfloat16).cuda()
    beta = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    decay = (torch.rand(T, H * K, generator=g) * 0.3 + 0.7).cuda()
    xbc = torch.randn(T, H * V + 2 * G * K, generator=g).to(torch.bfloat16).cuda()
    dt = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    hp = [torch.randn(H, generator=g).cuda() for _ in range(3)]

    def run(step, sl, st_d, st_s, lead=0):
        pick = lambda t: (torch.cat([t[:lead], t[sl]]).contiguous() if lead else t[sl].contiguous())
        a = ops.delta_recurrence(pick(q), pick(k), pick(v), pick(beta), pick(decay), st_d, step, H,
                                 HK, K, V, 1e-6, K ** -0.5)
        b = ops.ssd_recurrence(pick(xbc), pick(dt), *hp, st_s, step, H, V, K, G)
        return a[lead:], b[lead:]

    d0, s0 = (torch.zeros(3, H, K, V, device="cuda") for _ in range(2))
    whole = run(_cuda(_step([T], [0], [1])), slice(0, T), d0, s0)
    d1, s1 = (torch.zeros(3, H, K, V, device="cuda") for _ in range(2))
    parts, at = [], 0
    for n in (2, 17, 1, 16, 1, 1, 7):
        parts.append(run(_cuda(_step([3, n], [0, at], [0, 1])), slice(at, at + n), d1, s1, lead=3))
        at += n
    assert at == T
    for i in range(2):
        assert torch.equal(torch.cat([p[i] for p in parts]), whole[i])
    assert torch.equal(d1[1], d0[1]) and torch.equal(s1[1], s0[1])


@pytest.mark.parametrize("far", [1, 63, 64, 65, 900])
def test_delta_state_keeps_one_write_from_far_back(far):
    """Token 0 writes the value 5 under a key that no later token touches (later keys are
    orthogonal to it, decay 1): a query with that key reads 5 back ``far`` tokens later,
    whole and after the state went through portions and single tokens."""
    ops = _ops()
    H, K, V = 2, 16, 24
    T = far + 1
    g = torch.Generator().manual_seed(far)
    k = torch.zeros(T, H * K)
    k[:, 1:K] = torch.randn(T, K - 1, generator=g)          # head 0 of the keys: entry 0 free
    k[:, K + 1:] = torch.randn(T, K - 1, generator=g)
    k[0] = 0
    k[0, 0] = k[0, K] = 3.0
    q = k.clone()
    q[T - 1] = k[0]
    v = torch.randn(T, H * V, generator=g)
    v[0] = 5.0
    beta = torch.full((T, H), 30.0)                          # sigmoid = 1: a full write
    decay = torch.ones(T, H * K)
    outs = []
    for cuts in ([T], [1] * T if T < 80 else [T - 40] + [1] * 40, [2] * (T // 2) + [1] * (T % 2)):
        st = torch.zeros(1, H, K, V, device="cuda")
        at, last = 0, None
        for n in cuts:
            sl = slice(at, at + n)
            last = ops.delta_recurrence(q[sl].cuda(), k[sl].cuda(), v[sl].cuda(), beta[sl].cuda(),
                                        decay[sl].cuda(), st, _cuda(_step([n], [at], [0])), H, H, K,
                                        V, 1e-6, 1.0)
            at += n
        outs.append(last[-1].cpu())
        torch.testing.assert_close(last[-1].cpu(), torch.full((H, V), 5.0), rtol=1e-4, atol=1e-4)
    if T < 128:
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    else:      # long portions are walked in segments: the same up to rounding
        assert _rel(outs[1], outs[0]) <= 1e-6 and _rel(outs[2], outs[0]) <= 1e-6
    # a decay of one half per token on the written channel takes the value away
    decay[:, 0] = 0.5
    st = torch.zeros(1, H, K, V, device="cuda")
    o = ops.delta_recurrence(q.cuda(), k.cuda(), v.cuda(), beta.cuda(), decay.cuda(), st,
                             _cuda(_step([T], [0], [0])), H, H, K, V, 1e-6, 1.0)
    torch.testing.assert_close(o[-1, 0].cpu(), torch.full((V,), 5.0 * 0.5 ** far), rtol=1e-4,
                               atol=1e-6)
    torch.testing.assert_close(o[-1, 1].cpu(), torch.full((V,), 5.0), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,groups", [(128, 2), (24, 3), (15, 5), (512, 1), (1024, 8)])
def test_gated_group_norm(dtype, W, groups):
    g = torch.Generator().manual_seed(W)
    T = 6
    y = torch.randn(T, W, generator=g) * 3.0
    wide = (torch.randn(T, W + 8, generator=g) * 2.0).to(dtype)
    gain = 1.0 + 0.3 * torch.randn(W, generator=g)
    ref = host_ops.gated_group_norm(y, wide[:, 8:], gain, groups, 1e-5)
    out = _ops().gated_group_norm(y.cuda(), wide.cuda()[:, 8:], gain.cuda(), groups, 1e-5)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W", [96, 61, 2048])
def test_normed_pair_mean(dtype, W):
    g = torch.Generator().manual_seed(W)
    left = (torch.randn(5, W, generator=g) * 7.0).to(dtype)
    right = (torch.randn(5, W, generator=g) * 0.1).to(dtype)
    gl, gr = (1.0 + 0.3 * torch.randn(W, generator=g) for _ in range(2))
    ref = host_ops.normed_pair_mean(left, right, gl, gr, 1e-5)
    out = _ops().normed_pair_mean(left.cuda(), right.cuda(), gl.cuda(), gr.cuda(), 1e-5)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), ref, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_kernels(dtype):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 77, generator=g).to(dtype)
    torch.testing.assert_close(_ops().relu_squared(x.cuda()).cpu().float(),
                               host_ops.relu_squared(x).float(), **_tol(dtype))
    table = torch.stack([torch.randperm(7, generator=g)[:3] for _ in range(50)]).to(torch.int32)
    ids = torch.tensor([49, 0, 7, 7, 23], dtype=torch.int32)
    wts, idx = _ops().table_route(ids.cuda(), table.cuda(), 7)
    assert torch.equal(idx.cpu(), table[ids.long()])
    assert torch.equal(wts.cpu(), torch.full((5, 3), 1.0 / 3.0))
    o = torch.randn(6, 3, 20, generator=g) * 4.0
    gain = 1.0 + 0.3 * torch.randn(20, generator=g)
    gate = (torch.randn(6, 60, generator=g) * 2.0).to(dtype)
    ref = host_ops.head_norm_gate(o, gain, gate, 1e-5, dtype, gate_form="sigmoid")
    out = _ops().head_norm_gate(o.cuda(), gain.cuda(), gate.cuda(), 1e-5, dtype,
                                gate_form="sigmoid")
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    inner = torch.randn(6, 5, generator=g).to(dtype)
    w2t, b = torch.randn(5, 4 * 12, generator=g), torch.randn(4 * 12, generator=g)
    rate = torch.randn(4, generator=g)
    ref = host_ops.lowrank_decay(inner, w2t, b, "exp_rate_softplus", head_log_rate=rate)
    out = _ops().lowrank_decay(inner.cuda(), w2t.cuda(), b.cuda(), mode="exp_rate_softplus",
                               head_log_rate=rate.cuda())
    torch.testing.assert_close(out.cpu(), ref, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,vd,rot,factor", [(4, 2, 20, 28, 10, 3.0), (8, 2, 96, 160, 32, 2.5),
                                                        (3, 1, 16, 8, 0, 1.0), (2, 2, 64, 128, 64, 1.0)])
def test_rotation_of_leading_entries_with_values_of_their_own_size(dtype, heads, kvh, hd, vd, rot,
                                                                   factor):
    ops = _ops()
    T, page, P = 11, 4, 9
    g = torch.Generator().manual_seed(hd)
    qkv = torch.randn(T, (heads + kvh) * hd + kvh * vd, generator=g).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 100, 101, 7, 8, 9, 31999, 32000], dtype=torch.int32)
    inv = (5000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))
           / factor).float()
    slots = torch.randperm(P * page, generator=g)[:T].to(torch.int32)
    kc, vc = torch.zeros(P, kvh, page, hd, dtype=dtype), torch.zeros(P, kvh, page, vd, dtype=dtype)
    kc_d, vc_d = kc.clone().cuda(), vc.clone().cuda()
    q, k, v = ops.qkv_rope_append(qkv.cuda(), None, positions.cuda(), inv.cuda() if rot else None,
                                  rot, heads, kvh, hd, kc_d, vc_d, slots.cuda(),
                                  want_dense_kv=True, value_dim=vd)
    qr, kr, vr = host_ops.qkv_rope_append(qkv, None, positions, inv if rot else None, rot, heads,
                                          kvh, hd, kc, vc, slots, want_dense_kv=True, value_dim=vd)
    for a, b in ((q, qr), (k, kr), (v, vr), (kc_d, kc), (vc_d, vc)):
        torch.testing.assert_close(a.cpu().float(), b.float(), **_tol(dtype))
    assert v.shape == (T, kvh, vd)
    # what lies beyond the rotated entries passes unchanged; position 0 turns nothing
    raw_q = qkv[:, :heads * hd].reshape(T, heads, hd)
    assert torch.equal(q.cpu()[:, :, rot:], raw_q[:, :, rot:])
    assert torch.equal(q.cpu()[0], raw_q[0])


def _kv_case(seed, H, G, D, VD, page, q_lens, starts, dtype):
    g = torch.Generator().manual_seed(seed)
    step = _step(q_lens, starts)
    S = len(q_lens)
    need = [-(-(a + n) // page) for n, a in zip(q_lens, starts)]
    total = sum(need) + 3
    perm = torch.randperm(total, generator=g).to(torch.int32)
    bt = torch.full((S, max(need)), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(need):
        bt[s, :n] = perm[at:at + n]
        at += n
    kc = (torch.randn(total, G, page, D, generator=g) * 0.3).to(dtype)
    vc = (torch.randn(total, G, page, VD, generator=g)).to(dtype)
    q = (torch.randn(sum(q_lens), H, D, generator=g) * 0.3).to(dtype)
    return step, bt, kc, vc, q


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,VD", [(20, 28), (64, 128), (128, 64), (9, 3), (96, 96), (64, 256)])
@pytest.mark.parametrize("decode", [True, False])
def test_attention_with_values_of_their_own_size_finds_one_key(dtype, D, VD, decode):
    """One key among 700 carries a score far above the rest and a value of fives: far
    back, on either side of a page border, at position 0, the query's own.  Prompts and
    single tokens, beside a second sequence; weights in 32-bit whatever the element type."""
    H, G, page, scale = 4, 2, 16, 0.5
    query_pos = 700
    for key_pos in (0, 16 * 40 - 1, 16 * 40, 333, 699, 700):
        q_lens, starts = ([1, 1], [query_pos, 5]) if decode else ([9, 3], [query_pos - 8, 0])
        step, bt, kc, vc, q = _kv_case(3, H, G, D, VD, page, q_lens, starts, dtype)
        n0 = q_lens[0]
        q[:n0] = q[n0 - 1, 0]
        qv = q[n0 - 1, 0].float()
        pg, off = bt[0, key_pos // page].long(), key_pos % page
        kc[pg, :, off] = (qv * (60.0 / scale) / (qv * qv).sum()).to(dtype)
        vc[pg, :, off] = 5.0
        ref = host_ops.paged_attention(q, kc, vc, bt, step, 0, scale)
        out = _ops().paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), _cuda(step), 0,
                                     scale, fp32_weights=True).cpu().float()
        assert out.shape == (sum(q_lens), H, VD)
        torch.testing.assert_close(out, ref.float(), **_tol(dtype))
        assert float(out[n0 - 1].mean()) > 4.9, (key_pos, float(out[n0 - 1].mean()))
        if not decode and key_pos == 700:
            # the query before it must not see that key
            assert float(out[n0 - 2].abs().mean()) < 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,VD", [(3, 1, 24, 40), (10, 2, 96, 160), (8, 8, 200, 72),
                                      (2, 1, 320, 512), (16, 2, 64, 64), (6, 2, 7, 5)])
@pytest.mark.parametrize("window,softcap", [(0, 0.0), (100, 0.0), (0, 3.0)])
def test_single_token_attention_of_any_size_in_splits(dtype, H, G, D, VD, window, softcap):
    """Steps of single tokens over contexts of 1 to 1,000 keys: every grouping of heads,
    sizes on both sides of a lane's share, the split chosen by the kernel, none and one
    that leaves blocks without keys."""
    page, scale = 8, 0.4
    q_lens, starts = [1, 1, 1, 1], [0, 129, 999, 63]
    step, bt, kc, vc, q = _kv_case(H + D, H, G, D, VD, page, q_lens, starts, dtype)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, step.seq_of_token, step.positions,
                                           window, scale, softcap).float()
    cs = _cuda(step)
    for splits in (None, 1, 40):
        out = _ops().paged_attention_decode_any(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                                cs.kv_len, cs.max_kv_len, window, scale, softcap,
                                                splits=splits).cpu().float()
        assert out.shape == (4, H, VD)
        torch.testing.assert_close(out, ref, **_tol(dtype))
    # the dispatcher takes this kernel for such a step
    via = _ops().paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cs, window, scale,
                                 softcap=softcap, fp32_weights=True).cpu().float()
    torch.testing.assert_close(via, ref, **_tol(dtype))


# -- the engine against the plain model ------------------------------------------------
CASES = [("MA", mk.MA, 0, [5, 9, 17, 40, 3, 70], 4), ("MB", mk.MB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("MC", mk.MC, 3, [21, 1, 50, 2, 37], 4), ("MD", mk.MD, 2, [130, 2, 64, 33], 16)]


def _folder_dtype(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, dtype, name, cfg, seed, lengths, page, kind):
    d = mk.make_model_dir(cfg, tmp_path / "m", seed, dtype=_folder_dtype(dtype))
    reqs = mk.make_requests(cfg, lengths, seed)
    ref = mk.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=page, max_live=4)
    rows = mc.run_trace(sess, steps)
    worst = mc.compare(rows, ref, mk.bound_for(dtype, d, reqs), f"{name}/{kind}/{dtype}")
    print(f"{name}/{kind}/{dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_recorded_steps(tmp_path, dtype):
    """250 tokens one by one after a short prompt: the states and the convolutions' kept
    inputs are carried through recorded steps, every pass of the loop in its own."""
    cfg = mk.MA
    d = mk.make_model_dir(cfg, tmp_path / "m", 3, dtype=_folder_dtype(dtype))
    reqs = mk.make_requests(cfg, [270], 3)
    ref = mk.reference_rows(d, reqs)
    steps = traces.tail_decode(reqs, 250)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, use_graphs=True)
    rows = mc.run_trace(sess, steps)
    assert len(rows) == 270 and sess.executor.graph_replays >= 200
    mc.compare(rows, ref, mk.bound_for(dtype, d, reqs), f"long decode {dtype}")


@pytest.mark.parametrize("dtype,kind", [("bfloat16", "whole"), ("bfloat16", "mixed"),
                                        ("float32", "tail")])
def test_long_prompts(tmp_path, dtype, kind):
    """Prompts of several hundred tokens at head sizes 64 and 128 with value heads of
    another size: long walks of both recurrences, attention over many pages."""
    cfg = mk.MD
    d = mk.make_model_dir(cfg, tmp_path / "m", 11, dtype=_folder_dtype(dtype))
    reqs = mk.make_requests(cfg, [600, 260], 11)
    ref = mk.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=4)
    rows = mc.run_trace(sess, steps)
    sess.executor.poll_errors()
    mc.compare(rows, ref, mk.bound_for(dtype, d, reqs), f"long/{kind}/{dtype}")


def test_prefill_equals_decoding_in_32_bit(tmp_path):
    """The same sequence whole, token by token and in portions of two: the three runs
    agree with each other far inside their distance to the plain model."""
    cfg = mk.MC
    d = mk.make_model_dir(cfg, tmp_path / "m", 6)
    reqs = mk.make_requests(cfg, [75], 6)
    runs = []
    for steps in (traces.whole(reqs), traces.tail_decode(reqs, 74),
                  traces.portions(reqs, sizes=(2,))):
        sess = ReplaySession(d, "float32", 128, page_size=8, max_live=1)
        rows = mc.run_trace(sess, steps)
        runs.append(torch.stack([rows[("r0", p)] for p in range(75)]))
    scale = float(runs[0].abs().max())
    for other in runs[1:]:
        assert float((other - runs[0]).abs().max()) / scale < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    cfg = mk.MB
    d = mk.make_model_dir(cfg, tmp_path / "m", 5, dtype="bfloat16")
    reqs = mk.make_requests(cfg, [70, 33, 20, 9, 50, 41], 5)
    ref = mk.reference_rows(d, reqs)
    steps = traces.mixed(reqs, max_live=4, seed=1)
    out = tmp_path / "out"
    p = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(traces.peak_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    outs = []
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        outs.append(None if n == 0 else torch.from_numpy(
            np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n, cfg["vocab"]).copy()))
    rows = traces.collect(steps, outs)
    mc.compare(rows, ref, mk.bound_for(dtype, d, reqs), f"trace_run/{dtype}")


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = mk.make_model_dir(mk.MA, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(mk.make_requests(mk.MA, [7, 19, 3, 30, 11], 8).values())
    eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=4, max_num_seqs=3,
                                     num_gpu_blocks_override=96, prefill_chunk=6,
                                     max_model_len=64))
    done = eng.generate([Request(p, SamplingParams(max_tokens=12, ignore_eos=True))
                         for p in prompts])
    for p, c_out in zip(prompts, done):
        seq = list(p)
        for tok in c_out.output_tokens:
            lg = plain.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            # the engine's choice is the plain model's, unless the two best are a tie in fp32
            assert tok == int(lg.argmax()) or float(top[0] - top[1]) < 1e-4 * float(lg.abs().max())
            seq.append(tok)
        assert len(c_out.output_tokens) == 12
