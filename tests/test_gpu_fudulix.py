"""The Fudulix design on the GPU: every new kernel and kernel option alone against its plain
statement (tests/host_ops.py), then the engine against the plain model
(tests/plain_fudulix.py): whole prompts, prefill against token-by-token decoding, portions
down to two tokens, unequal batches with pages and slots used again, long decoding with
recorded steps over windows and kept tokens, and greedy generation through the engine's own
entry point."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import fudulix_cases as fk
import host_ops
import model_cases as mc
import plain_fudulix as plain
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


def _step(q_lens, starts, slots=None, tokens=None):
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
        state_slot=i32(slots if slots is not None else list(range(len(q_lens)))),
        token_ids=i32(tokens if tokens is not None else [0] * len(seq_of)))


def _cuda(ns):
    return SimpleNamespace(**{k: (v.cuda() if torch.is_tensor(v) else v)
                              for k, v in vars(ns).items()})


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


# -- kernels alone -------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,buckets", [(96, 53), (61, 7), (2048, 1021)])
def test_pair_embedding_reads_and_moves_the_previous_token(dtype, width, buckets):
    """Sequences at position 0, in the middle of a prompt and with one token; the previous
    token of a portion's first token comes from the slot, and the slot takes the last."""
    g = torch.Generator().manual_seed(width)
    vocab = 200
    table = torch.randn(vocab, width, generator=g).to(dtype)
    pairs = torch.randn(buckets + 1, width, generator=g).to(dtype)
    gain = 1.0 + 0.3 * torch.randn(width, generator=g)
    q_lens, starts, slots = [3, 1, 4, 1], [0, 17, 5, 0], [2, 0, 5, 3]
    toks = torch.randint(0, vocab, (sum(q_lens),), generator=g).tolist()
    step = _step(q_lens, starts, slots, toks)
    state = torch.randint(0, vocab, (6, 1), generator=g).to(torch.int32)
    ref_state = state.clone()
    ref = host_ops.embed_pair_norm(table, pairs, gain, step, ref_state, buckets, 31, 7, 1e-5)
    dev_state = state.cuda()
    out = _ops().embed_pair_norm(table.cuda(), pairs.cuda(), gain.cuda(), _cuda(step), dev_state,
                                 buckets, 31, 7, 1e-5)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), ref, rtol=2e-5, atol=2e-5)
    assert torch.equal(dev_state.cpu(), ref_state)
    assert ref_state[2, 0] == toks[2] and ref_state[1, 0] == state[1, 0]   # slot 1: no sequence
    # the row of a first token is the table's last, whatever the slot holds
    first = (table[toks[0]].float() + pairs[buckets].float())
    first = first / torch.sqrt((first * first).mean() + 1e-5) * gain
    torch.testing.assert_close(out[0].cpu(), first, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,vd,rot,inter,proj,unit", [
    (4, 2, 24, 16, 12, False, True, False), (6, 2, 16, 16, 8, True, False, True),
    (3, 1, 10, 6, 10, True, False, True), (5, 1, 6, 7, 4, False, True, False),
    (8, 2, 128, 64, 64, True, True, True), (2, 2, 64, 64, 0, False, False, False),
    (32, 8, 128, 128, 128, False, True, False)])
def test_preparation_of_q_k_v(dtype, heads, kvh, hd, vd, rot, inter, proj, unit):
    """Projection norm, rotation in both pairings with a factor on cos and sin, unit heads,
    value blend, the dense q and the page writes, on rows that are views of a wider one."""
    g = torch.Generator().manual_seed(heads * hd + rot)
    # views that start off a 16-byte mark, and on one (the kernel's two forms)
    for lead, lead_e in ((3, 4), (8, 16)):
        _prepare_case(dtype, heads, kvh, hd, vd, rot, inter, proj, unit, g, lead, lead_e)


def _prepare_case(dtype, heads, kvh, hd, vd, rot, inter, proj, unit, g, lead, lead_e):
    T, page, pages = 11, 4, 9
    dq, dk, dv = heads * hd, kvh * hd, kvh * vd
    wide = (torch.randn(T, dq + dk + dv + 16, generator=g) * 2.0).to(dtype)
    qkv = wide[:, lead:lead + dq + dk + dv]
    earlier_wide = torch.randn(T, dv + 24, generator=g).to(dtype)
    earlier = earlier_wide[:, lead_e:lead_e + dv]
    pos = torch.tensor([0, 1, 2, 3, 900, 901, 7, 8, 9, 65, 66], dtype=torch.int32)
    freq = (torch.rand(rot // 2, generator=g) * 1.5) if rot else None
    qg = (1.0 + 0.3 * torch.randn(dq, generator=g)) if proj else None
    kg = (1.0 + 0.3 * torch.randn(dk, generator=g)) if proj else None
    lam = torch.tensor([0.3])
    slots = torch.randperm(page * pages, generator=g)[:T].to(torch.int32)
    for mix in (None, earlier):
        kc_ref = torch.zeros(pages, kvh, page, hd, dtype=dtype)
        vc_ref = torch.zeros(pages, kvh, page, vd, dtype=dtype)
        q_ref, k_ref, v_ref = host_ops.attention_prepare(
            qkv, pos, freq, 1.07, rot, inter, heads, kvh, hd, vd, qg, kg, 1e-5, unit, mix, lam,
            kc_ref, vc_ref, slots, want_dense_kv=True)
        kc, vc = torch.zeros_like(kc_ref).cuda(), torch.zeros_like(vc_ref).cuda()
        dev = lambda t: None if t is None else t.cuda()
        wide_d = wide.cuda()
        early_d = earlier_wide.cuda()
        q, k, v = _ops().attention_prepare(
            wide_d[:, lead:lead + dq + dk + dv], pos.cuda(), dev(freq), 1.07, rot, inter, heads,
            kvh, hd, vd, dev(qg), dev(kg), 1e-5, unit,
            None if mix is None else early_d[:, lead_e:lead_e + dv],
            lam.cuda(), kc, vc, slots.cuda(), want_dense_kv=True)
        for got, want in ((q, q_ref), (k, k_ref), (v, v_ref), (kc, kc_ref), (vc, vc_ref)):
            torch.testing.assert_close(got.cpu().float(), want.float(), **_tol(dtype))
    if unit:
        assert abs(float((q_ref.float() ** 2).mean(-1).mean()) - 1.0) < 2e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I,act,bias", [(5, 72, "gelu_tanh", True), (3, 33, "gelu_tanh", True),
                                          (600, 512, "gelu_tanh", True), (7, 40, "silu", False),
                                          (2, 1408, "silu", True)])
def test_gated_unit_with_biases(dtype, T, I, act, bias):
    g = torch.Generator().manual_seed(T + I)
    gu = (torch.randn(T, 2 * I, generator=g) * 3.0).to(dtype)
    b = torch.randn(2 * I, generator=g) * 2.0 if bias else None
    ref = host_ops.glu_bias_act(gu, b, act)
    out = _ops().glu_bias_act(gu.cuda(), None if b is None else b.cuda(), act)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_identity_rows(dtype):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(9, 40, generator=g).to(dtype)
    topk = torch.tensor([[0, 4], [5, 1], [2, 3], [4, 5], [1, 0], [3, 3 + 2], [0, 1], [4, 2],
                         [5, 4]], dtype=torch.int32)
    offsets, rows, dest = host_ops.moe_dispatch(topk, 6)
    y = torch.full((18, 40), 7.0).to(dtype)
    ref = host_ops.identity_rows(x, rows, offsets, 4, y.clone())
    got = _ops().identity_rows(x.cuda(), rows.cuda(), offsets.cuda(), 4, y.cuda()).cpu()
    assert torch.equal(got, ref)
    lo = int(offsets[4])
    assert torch.equal(got[:lo], y[:lo]) and torch.equal(got[lo], x[rows[lo].long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [3, 130, 1500])
@pytest.mark.parametrize("E,k,groups,keep", [(6, 2, 3, 2), (14, 2, 2, 1), (12, 3, 4, 2),
                                             (64, 6, 8, 3), (5, 5, 0, 0), (8, 1, 1, 1)])
def test_router_with_correction_groups_and_identity_outputs(dtype, T, E, k, groups, keep):
    """The few-token kernels and the fused one choose alike; corrections (some far
    negative) move the choice and leave the weights alone; only the kept groups are chosen
    from; the weights of a token sum to one."""
    g = torch.Generator().manual_seed(E * 7 + T)
    H = 96 if dtype == torch.float32 else 256
    x = torch.randn(T, H, generator=g).to(dtype)
    w = torch.randn(E, H, generator=g) * 0.15
    corr = torch.randn(E, generator=g) * 0.2 - 0.3
    ref_w, ref_i, _ = host_ops.router_topk(x, w, k, True, 1.0, correction=corr, group_count=groups,
                                           group_keep=keep, renorm_eps=1e-20)
    tw, ti, _ = _ops().router_topk(x.cuda(), w.cuda(), k, True, 1.0, correction=corr.cuda(),
                                   group_count=groups, group_keep=keep, renorm_eps=1e-20)
    tw, ti = tw.cpu(), ti.cpu()
    # a choice may differ only where two corrected scores are within rounding of each other
    same = (ti == ref_i).all(-1)
    assert float(same.float().mean()) > 0.99
    torch.testing.assert_close(tw[same], ref_w[same], rtol=2e-4, atol=2e-6)
    torch.testing.assert_close(tw.sum(-1), torch.ones(T), rtol=1e-5, atol=1e-5)
    if groups:
        size = E // groups
        assert int(torch.tensor([len({int(e) // size for e in row}) for row in ti]).max()) <= keep
    plain_w, plain_i, _ = host_ops.router_topk(x, w, k, True, 1.0)
    if k < E and T >= 130:
        assert not torch.equal(plain_i, ref_i)      # the correction and the groups matter


def _sharp_case(dtype, D, VD, decode, query_pos, key_pos, window, page=16):
    H, G, scale = 4, 2, 0.5
    q_lens, starts = ([1, 1], [query_pos, 5]) if decode else ([9, 3], [query_pos - 8, 0])
    step, bt, kc, vc, q = _kv_case(3, H, G, D, VD, page, q_lens, starts, dtype)
    n0 = q_lens[0]
    q[:n0] = q[n0 - 1, 0]
    qv = q[n0 - 1, 0].float()
    pg, off = bt[0, key_pos // page].long(), key_pos % page
    kc[pg, :, off] = (qv * (60.0 / scale) / (qv * qv).sum()).to(dtype)
    vc[pg, :, off] = 5.0
    return step, bt, kc, vc, q, n0, scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,VD", [(24, 16), (96, 48), (64, 64), (10, 6), (128, 64)])
@pytest.mark.parametrize("decode", [True, False])
def test_window_with_kept_first_keys_finds_one_key(dtype, D, VD, decode):
    """One key carries a score far above the rest and a value of fives.  It is seen just
    inside the window, not just outside it, among the kept first keys (the last kept one
    too), not directly behind them; in prompts and for single tokens."""
    window, keep, query_pos = 40, 5, 700
    for key_pos, seen in ((700, True), (661, True), (660, False), (0, True), (4, True),
                          (5, False), (333, False)):
        step, bt, kc, vc, q, n0, scale = _sharp_case(dtype, D, VD, decode, query_pos, key_pos,
                                                     window)
        ref = host_ops.paged_attention(q, kc, vc, bt, step, window, scale, keep_first=keep)
        out = _ops().paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), _cuda(step),
                                     window, scale, fp32_weights=True, keep_first=keep
                                     ).cpu().float()
        torch.testing.assert_close(out, ref.float(), **_tol(dtype))
        mean = float(out[n0 - 1].mean())
        assert (mean > 4.9) == seen, (key_pos, mean)
    # pages between the kept keys and the window may have been given back
    step, bt, kc, vc, q, n0, scale = _sharp_case(dtype, D, VD, decode, query_pos, 2, window)
    ref = host_ops.paged_attention(q, kc, vc, bt, step, window, scale, keep_first=keep)
    gone = bt.clone()
    gone[0, 1:(query_pos - 8 - window) // 16 - 1] = -1
    out = _ops().paged_attention(q.cuda(), kc.cuda(), vc.cuda(), gone.cuda(), _cuda(step), window,
                                 scale, fp32_weights=True, keep_first=keep).cpu().float()
    torch.testing.assert_close(out, ref.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [True, False])
def test_sink_takes_its_share_of_the_weights(dtype, decode):
    """With every score far below zero the sink takes nearly all the weight and the output
    nearly vanishes; with one score far above zero it takes nearly none."""
    D, VD, window = 32, 20, 50
    step, bt, kc, vc, q, n0, scale = _sharp_case(dtype, D, VD, decode, 300, 290, window)
    for flip in (False, True):
        kk = -kc.abs() * 30.0 if flip else kc
        qq = q.abs() if flip else q
        ref = host_ops.paged_attention(qq, kk, vc, bt, step, window, scale, sink=True)
        out = _ops().paged_attention(qq.cuda(), kk.cuda(), vc.cuda(), bt.cuda(), _cuda(step),
                                     window, scale, fp32_weights=True, sink=True).cpu().float()
        torch.testing.assert_close(out, ref.float(), **_tol(dtype))
        without = host_ops.paged_attention(qq, kk, vc, bt, step, window, scale)
        if flip:
            assert float(out[n0 - 1].abs().max()) < 0.05 * float(without[n0 - 1].abs().max())
        else:
            assert float(out[n0 - 1].mean()) > 4.9


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,VD", [(3, 1, 24, 40), (8, 2, 96, 48), (16, 2, 64, 64), (6, 2, 7, 5)])
@pytest.mark.parametrize("window,keep,sink", [(100, 4, False), (100, 0, True), (7, 9, True),
                                              (1, 1, False), (0, 3, True)])
def test_single_token_attention_in_splits_with_kept_keys_and_sink(dtype, H, G, D, VD, window, keep,
                                                                  sink):
    page, scale = 8, 0.4
    q_lens, starts = [1, 1, 1, 1], [0, 129, 999, 63]
    step, bt, kc, vc, q = _kv_case(H + D, H, G, D, VD, page, q_lens, starts, dtype)
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, step.seq_of_token, step.positions,
                                           window, scale, 0.0, keep if window else 0, sink).float()
    cs = _cuda(step)
    for splits in (None, 1, 40):
        out = _ops().paged_attention_decode_any(
            q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cs.kv_len, cs.max_kv_len, window, scale,
            0.0, splits=splits, keep_first=keep if window else 0, sink=sink).cpu().float()
        torch.testing.assert_close(out, ref, **_tol(dtype))
    # the block-per-token kernel and the tiled one agree with the same statement
    gen = _ops().paged_attention_generic(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                         cs.seq_of_token, cs.positions, window, scale, 0.0,
                                         keep if window else 0, sink).cpu().float()
    torch.testing.assert_close(gen, ref, **_tol(dtype))
    if D % 4 == 0 and VD % 4 == 0:
        til = _ops().paged_attention_tiled(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cs.cu_q,
                                           cs.q_pos0, window, scale, 0.0, keep if window else 0,
                                           sink).cpu().float()
        torch.testing.assert_close(til, ref, **_tol(dtype))


@pytest.mark.parametrize("H,G,D,VD", [(8, 2, 64, 64), (4, 4, 64, 128), (16, 2, 128, 64),
                                      (20, 1, 128, 128)])
@pytest.mark.parametrize("window,keep,sink", [(0, 0, False), (100, 4, False), (100, 0, True),
                                              (70, 130, True), (1, 1, False)])
def test_tensor_core_attention_with_16_bit_weights(H, G, D, VD, window, keep, sink):
    """The tensor-core kernels whose weights enter the product with the values as two bfloat16
    terms: prompts of unequal length beside each other and single tokens in splits, against
    the statement with 32-bit weights, and far closer to the CUDA-core kernel with 32-bit
    weights than one rounding of a weight to bfloat16 would leave them."""
    dtype, page, scale = torch.bfloat16, 16, 0.35
    k = keep if window else 0
    q_lens, starts = [70, 5, 130, 1], [200, 0, 63, 400]
    step, bt, kc, vc, q = _kv_case(H + VD, H, G, D, VD, page, q_lens, starts, dtype)
    vc = vc + 3.0          # values with a mean: an error of the weights does not average out
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, step.seq_of_token, step.positions,
                                           window, scale, 0.0, k, sink).float()
    cs = _cuda(step)
    exact = _ops().paged_attention_tiled(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cs.cu_q,
                                         cs.q_pos0, window, scale, 0.0, k, sink).cpu().float()
    # the tcgen05 form (keys and values of one size) and the mma.sync form (any of the four)
    for form in (("tc", "mma") if D == VD else ("mma",)):
        out = _ops().paged_attention_prefill_exact(
            q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cs.cu_q, cs.q_pos0, window, scale, k, sink,
            kernel=form).cpu().float()
        torch.testing.assert_close(out, ref, **_tol(dtype))
        # both round their result to bfloat16 once: they differ by that rounding at most
        assert float((out - exact).abs().max()) <= 2.0 ** -7 * float(exact.abs().max()), form
        assert float((out - exact).abs().mean()) <= 2.0 ** -11 * float(exact.abs().max()), form
    q_lens, starts = [1, 1, 1, 1], [0, 129, 999, 63]
    step, bt, kc, vc, q = _kv_case(H + D, H, G, D, VD, page, q_lens, starts, dtype)
    vc = vc + 3.0
    ref = host_ops.paged_attention_generic(q, kc, vc, bt, step.seq_of_token, step.positions,
                                           window, scale, 0.0, k, sink).float()
    cs = _cuda(step)
    for splits in (None, 1, 7):
        out = _ops().paged_attention_decode_exact(
            q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cs.kv_len, cs.max_kv_len, window, scale,
            splits=splits, keep_first=k, sink=sink).cpu().float()
        torch.testing.assert_close(out, ref, **_tol(dtype))
        assert float((out - ref).abs().mean()) <= 2.0 ** -10 * float(ref.abs().max())
    # the dispatcher takes these kernels for such heads
    via = _ops().paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cs, window, scale,
                                 fp32_weights=True, keep_first=k, sink=sink).cpu().float()
    torch.testing.assert_close(via, out)


def test_prompt_attention_does_not_depend_on_the_cut():
    """A sequence's queries whole and in portions that start inside a tile, with kept keys
    and the sink: the tiled kernel gives the same bits."""
    H, G, D, VD, page, scale, window, keep = 4, 2, 24, 16, 8, 0.4, 70, 6
    step, bt, kc, vc, q = _kv_case(9, H, G, D, VD, page, [300], [0], torch.float32)
    whole = _ops().paged_attention_tiled(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(),
                                         step.cu_q.cuda(), step.q_pos0.cuda(), window, scale, 0.0,
                                         keep, True).cpu()
    at = 0
    for n in (5, 2, 90, 33, 1, 169):
        part = _step([n], [at])
        out = _ops().paged_attention_tiled(q[at:at + n].contiguous().cuda(), kc.cuda(), vc.cuda(),
                                           bt.cuda(), part.cu_q.cuda(), part.q_pos0.cuda(), window,
                                           scale, 0.0, keep, True).cpu()
        assert torch.equal(out, whole[at:at + n])
        at += n


# -- the engine against the plain model ------------------------------------------------
CASES = [("FA", fk.FA, 0, [5, 9, 17, 40, 3, 70], 4), ("FB", fk.FB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("FC", fk.FC, 2, [130, 2, 64, 33], 16)]


def _folder_dtype(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, dtype, name, cfg, seed, lengths, page, kind):
    d = fk.make_model_dir(cfg, tmp_path / "m", seed, dtype=_folder_dtype(dtype))
    reqs = fk.make_requests(cfg, lengths, seed)
    ref = fk.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=page, max_live=4)
    rows = fk.rows_to_compare(dtype, d, reqs, mc.run_trace(sess, steps))
    worst = mc.compare(rows, ref, fk.bound_for(dtype, d, reqs), f"{name}/{kind}/{dtype}")
    print(f"{name}/{kind}/{dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_recorded_steps(tmp_path, dtype):
    """250 tokens one by one after a short prompt: every window passes over decoded tokens,
    pages fall behind it and are given back, the kept first tokens stay, and the previous
    token and the convolutions' kept inputs are carried through recorded steps."""
    cfg = fk.FA
    d = fk.make_model_dir(cfg, tmp_path / "m", 3, dtype=_folder_dtype(dtype))
    reqs = fk.make_requests(cfg, [270], 3)
    ref = fk.reference_rows(d, reqs)
    steps = traces.tail_decode(reqs, 250)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, use_graphs=True)
    rows = mc.run_trace(sess, steps)
    assert len(rows) == 270 and sess.executor.graph_replays >= 200
    rows = fk.rows_to_compare(dtype, d, reqs, rows, share=0.05)
    mc.compare(rows, ref, fk.bound_for(dtype, d, reqs), f"long decode {dtype}")


@pytest.mark.parametrize("dtype,kind", [("bfloat16", "whole"), ("bfloat16", "mixed"),
                                        ("float32", "tail")])
def test_long_prompts(tmp_path, dtype, kind):
    """Prompts of several hundred tokens at head sizes 32 to 128: many key tiles, windows
    and kept tokens far apart, attention over many pages."""
    cfg = fk.FC
    d = fk.make_model_dir(cfg, tmp_path / "m", 11, dtype=_folder_dtype(dtype))
    reqs = fk.make_requests(cfg, [400, 260], 11)
    ref = fk.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=4)
    rows = mc.run_trace(sess, steps)
    sess.executor.poll_errors()
    rows = fk.rows_to_compare(dtype, d, reqs, rows, share=0.05)
    mc.compare(rows, ref, fk.bound_for(dtype, d, reqs), f"long/{kind}/{dtype}")


def test_prefill_equals_decoding_in_32_bit(tmp_path):
    """The same sequence whole, token by token and in portions of two: the three runs
    agree with each other far inside their distance to the plain model."""
    cfg = fk.FB
    d = fk.make_model_dir(cfg, tmp_path / "m", 6)
    reqs = fk.make_requests(cfg, [75], 6)
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
    cfg = fk.FA
    d = fk.make_model_dir(cfg, tmp_path / "m", 5, dtype="bfloat16")
    reqs = fk.make_requests(cfg, [70, 33, 20, 9, 50, 41], 5)
    ref = fk.reference_rows(d, reqs)
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
    rows = fk.rows_to_compare(dtype, d, reqs, traces.collect(steps, outs))
    mc.compare(rows, ref, fk.bound_for(dtype, d, reqs), f"trace_run/{dtype}")


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = fk.make_model_dir(fk.FA, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(fk.make_requests(fk.FA, [7, 19, 3, 30, 11], 8).values())
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


def test_command_line_and_sampling(tmp_path):
    """The generation program takes a folder of the design like any other: greedy output is
    the plain model's, and sampling with a seed (temperature, top-k, top-p, a repetition
    penalty) gives the same tokens twice."""
    d = fk.make_model_dir(fk.FB, tmp_path / "m", 9)
    c, w = plain.read_model_folder(d)
    base = [sys.executable, os.path.join(ROOT, "bin", "inferx-generate"), d, "--dtype", "fp32",
            "--block-size", "4", "--max-model-len", "64", "--max-num-seqs", "2",
            "--num-gpu-blocks-override", "48", "--log-level", "warning"]
    p = subprocess.run(base + ["--prompt-ids", "5,17,3,90,41", "--prompt-ids", "9 8 7",
                               "--max-tokens", "6", "--ignore-eos"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [json.loads(ln) for ln in p.stdout.splitlines() if ln.startswith("{")]
    assert [l["index"] for l in lines] == [0, 1]
    for line, prompt in zip(lines, ([5, 17, 3, 90, 41], [9, 8, 7])):
        seq = list(prompt)
        for tok in line["output_ids"]:
            lg = plain.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            assert tok == int(lg.argmax()) or float(top[0] - top[1]) < 1e-4 * float(lg.abs().max())
            seq.append(tok)
        assert len(line["output_ids"]) == 6
    sampled = []
    for _ in range(2):
        p = subprocess.run(base + ["--prompt-ids", "9 8 7", "--max-tokens", "8", "--ignore-eos",
                                   "--temperature", "0.9", "--top-k", "20", "--top-p", "0.9",
                                   "--seed", "3", "--repetition-penalty", "1.2"],
                           capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        (line,) = [json.loads(ln) for ln in p.stdout.splitlines() if ln.startswith("{")]
        sampled.append(line["output_ids"])
    assert sampled[0] == sampled[1] and len(sampled[0]) == 8
