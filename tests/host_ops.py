"""Plain fp32 statements of what each kernel computes, with torch on the CPU.

Two uses: (1) the ``-m gpu`` kernel tests compare each CUDA kernel with the
function of the same name here; (2) the CPU tests put this module where the engine
expects its kernel module, so that the cache manager, the step function and the
scheduler are exercised against the plain model without a GPU.  It is a test
double, not a product path: the package itself never imports it and refuses CPU
tensors.  Everything is computed in fp32 whatever the storage type.
"""
from __future__ import annotations

import torch


def _f(t):
    return t.to(torch.float32)


def embed(table, ids, out=None, scale=1.0):
    r = _f(table)[ids.long()] * scale
    if out is not None:
        out.copy_(r)
        return out
    return r


def add_rmsnorm(resid, delta, gain, eps, out_dtype, rows=None):
    if rows is None:
        if delta is not None:
            resid += _f(delta)
        v = resid
    else:
        v = resid[rows.long()]
        if delta is not None:
            v = v + _f(delta)[rows.long()]
    ms = (v * v).sum(-1, keepdim=True) / v.shape[-1]
    return (v * (1.0 / torch.sqrt(ms + eps)) * gain).to(out_dtype)


def silu_mul(gu):
    i = gu.shape[1] // 2
    g, u = _f(gu[:, :i]), _f(gu[:, i:])
    return (g / (1.0 + torch.exp(-g)) * u).to(gu.dtype)


def linear(x, w, out_dtype=None):
    return (_f(x) @ _f(w).T).to(out_dtype or x.dtype)


def gate_up_swiglu(x, w_gate_up):
    return silu_mul(linear(x, w_gate_up))


def _rotate(x, positions, inv_freq, rot):
    # x [T, heads, hd] fp32
    if not rot:
        return x
    half = rot // 2
    a = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rot]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]], dim=-1)


def _scatter(cache, rows, slots):
    # cache [P, kvh, page, hd]; rows [T, kvh, hd]
    page = cache.shape[2]
    for t in range(rows.shape[0]):
        s = int(slots[t])
        if s >= 0:
            cache[s // page, :, s % page, :] = rows[t].to(cache.dtype)


def qkv_rope_append(qkv, bias, positions, inv_freq, rotary_dim, heads, kv_heads, head_dim,
                    k_cache, v_cache, slots, want_dense_kv=False, value_dim=0):
    T = qkv.shape[0]
    x = _f(qkv)
    if bias is not None:
        x = x + bias
    dq, dkv = heads * head_dim, kv_heads * head_dim
    q = _rotate(x[:, :dq].reshape(T, heads, head_dim), positions, inv_freq, rotary_dim)
    k = _rotate(x[:, dq:dq + dkv].reshape(T, kv_heads, head_dim), positions, inv_freq, rotary_dim)
    v = x[:, dq + dkv:].reshape(T, kv_heads, value_dim or head_dim)
    q, k, v = q.to(qkv.dtype), k.to(qkv.dtype), v.to(qkv.dtype)
    if k_cache is not None:
        _scatter(k_cache, k, slots)
        _scatter(v_cache, v, slots)
    return (q, k, v) if want_dense_kv else q


def append_kv(k, v, k_cache, v_cache, slots):
    _scatter(k_cache, k, slots)
    _scatter(v_cache, v, slots)


def paged_attention_generic(q, k_cache, v_cache, block_table, seq_of_token, positions, window,
                            scale, softcap=0.0, keep_first=0, sink=False):
    T, heads, hd = q.shape
    P, kvh, page, _ = k_cache.shape
    rep = heads // kvh
    out = torch.zeros(T, heads, v_cache.shape[3], dtype=torch.float32)
    for t in range(T):
        s, pos = int(seq_of_token[t]), int(positions[t])
        start = max(0, pos - window + 1) if window > 0 else 0
        kp = torch.arange(start, pos + 1)
        if keep_first > 0 and start > 0:      # the request's first tokens stay visible
            kp = torch.cat([torch.arange(0, min(keep_first, start)), kp])
        pages = block_table[s][(kp // page).long()].long()
        assert (pages >= 0).all(), "attention reads a page that was given back"
        offs = (kp % page).long()
        for h in range(heads):
            kh = h // rep
            keys = _f(k_cache[pages, kh, offs, :])
            vals = _f(v_cache[pages, kh, offs, :])
            sc = (keys @ _f(q[t, h])) * scale
            if softcap > 0:
                sc = softcap * torch.tanh(sc / softcap)
            top = torch.clamp(sc.max(), min=0.0) if sink else sc.max()
            p = torch.exp(sc - top)
            # the sink: a key of score 0 that has no value
            den = p.sum() + (torch.exp(-top) if sink else 0.0)
            out[t, h] = (p[:, None] * vals).sum(0) / den
    return out.to(q.dtype)


def paged_attention(q, k_cache, v_cache, block_table, step, window, scale, softcap=0.0,
                    fp32_weights=False, keep_first=0, sink=False):
    return paged_attention_generic(q, k_cache, v_cache, block_table, step.seq_of_token,
                                   step.positions, window, scale, softcap, keep_first, sink)


def router_topk(x, w, top_k, renormalize, scale, extra_w=None, correction=None, group_count=0,
                group_keep=0, renorm_eps=-1.0):
    logits = _f(x) @ w.T
    p = torch.softmax(logits, dim=-1)
    T, E = p.shape
    if correction is not None or group_count or renorm_eps >= 0:
        # the choice is by score + correction, inside the best groups; weights are the scores
        pick = p + (correction if correction is not None else 0.0)
        if group_count:
            size = E // group_count
            best = pick.view(T, group_count, size).max(-1).values
            kept = torch.zeros(T, group_count, dtype=torch.bool)
            work = best.clone()
            for _ in range(group_keep):
                top = work.max(-1).values
                g = (work == top[:, None]).to(torch.int32).argmax(-1)
                kept[torch.arange(T), g] = True
                work[torch.arange(T), g] = float("-inf")
            pick = torch.where(kept.repeat_interleave(size, dim=1), pick,
                               torch.full_like(pick, float("-inf")))
        tw = torch.zeros(T, top_k)
        ti = torch.zeros(T, top_k, dtype=torch.int32)
        for s in range(top_k):
            top = pick.max(-1).values
            idx = (pick == top[:, None]).to(torch.int32).argmax(-1)
            tw[:, s] = p[torch.arange(T), idx]
            ti[:, s] = idx.to(torch.int32)
            pick[torch.arange(T), idx] = float("-inf")
        tot = tw.sum(-1, keepdim=True)
        if renorm_eps >= 0:
            tw = tw / (tot + renorm_eps)
        elif renormalize:
            tw = torch.where(tot > 0, tw / tot, tw)
        ex = (_f(x) @ extra_w) if extra_w is not None else None
        return tw * scale, ti, ex
    tw = torch.zeros(T, top_k)
    ti = torch.zeros(T, top_k, dtype=torch.int32)
    work = p.clone()
    for s in range(top_k):
        best = work.max(dim=-1).values
        # ties to the lower index: first position equal to the max
        idx = (work == best[:, None]).to(torch.int32).argmax(dim=-1)
        tw[:, s] = best
        ti[:, s] = idx.to(torch.int32)
        work[torch.arange(T), idx] = -2.0
    if renormalize:
        tot = tw.sum(-1, keepdim=True)
        tw = torch.where(tot > 0, tw / tot, tw)
    ex = (_f(x) @ extra_w) if extra_w is not None else None
    return tw * scale, ti, ex


def moe_dispatch(topk_idx, num_experts):
    T, k = topk_idx.shape
    flat = topk_idx.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    rows = (order // k).to(torch.int32)
    dest = torch.empty(T * k, dtype=torch.int32)
    dest[order] = torch.arange(T * k, dtype=torch.int32)
    return offsets, rows, dest


def grouped_gate_up_swiglu(x, rows, offsets, w_gate_up):
    E, two_i, H = w_gate_up.shape
    i = two_i // 2
    out = torch.zeros(rows.numel(), i, dtype=torch.float32)
    for e in range(E):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi > lo:
            xe = _f(x[rows[lo:hi].long()])
            g = xe @ _f(w_gate_up[e, :i]).T
            u = xe @ _f(w_gate_up[e, i:]).T
            out[lo:hi] = g / (1.0 + torch.exp(-g)) * u
    return out.to(x.dtype)


def grouped_down(act, offsets, w_down, offsets_settled=False):
    E, H, i = w_down.shape
    out = torch.zeros(act.shape[0], H, dtype=torch.float32)
    for e in range(E):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi > lo:
            out[lo:hi] = _f(act[lo:hi]) @ _f(w_down[e]).T
    return out.to(act.dtype)


def moe_combine(y, dest, topk_w, shared, shared_logit):
    T, k = topk_w.shape
    out = torch.zeros(T, y.shape[1], dtype=torch.float32)
    for s in range(k):
        out += topk_w[:, s:s + 1] * _f(y[dest.view(T, k)[:, s].long()])
    if shared is not None:
        sh = _f(shared)
        if shared_logit is not None:
            sh = sh * (1.0 / (1.0 + torch.exp(-shared_logit)))[:, None]
        out += sh
    return out.to(y.dtype)


def _uniform(seed):
    mask = (1 << 64) - 1
    z = (int(seed) + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def apply_penalties(logits, hist_ids, hist_counts, penalties, mask_ids):
    R, V = logits.shape
    for r in range(R):
        if hist_ids is not None:
            pres, freq, rep = (float(v) for v in penalties[r])
            if pres != 0.0 or freq != 0.0 or rep != 1.0:
                for j in range(hist_ids.shape[1]):
                    t = int(hist_ids[r, j])
                    if not 0 <= t < V:
                        continue
                    v = logits[r, t]
                    if rep != 1.0:
                        v = v / rep if v > 0 else v * rep
                    logits[r, t] = v - pres - freq * float(hist_counts[r, j])
        if mask_ids is not None:
            for j in range(mask_ids.shape[1]):
                t = int(mask_ids[r, j])
                if 0 <= t < V:
                    logits[r, t] = float("-inf")


def max_top_logprobs():
    return 20


def token_logprobs(logits, chosen, want_k=None, top=0):
    R, V = logits.shape
    chosen_lp = torch.zeros(R, dtype=torch.float32)
    top_ids = torch.full((R, top), -1, dtype=torch.int32) if top else None
    top_lps = torch.zeros((R, top), dtype=torch.float32) if top else None
    for r in range(R):
        k = int(want_k[r]) if want_k is not None else 0
        if k < 0:
            continue
        row = logits[r].to(torch.float64)
        log_z = torch.log(torch.exp(row - row.max()).sum()) + row.max()
        chosen_lp[r] = float(row[int(chosen[r])] - log_z)
        order = sorted(range(V), key=lambda i: (-float(row[i]), i))[:min(k, top)]
        for j, i in enumerate(order):
            top_ids[r, j] = i
            top_lps[r, j] = float(row[i] - log_z)
    return chosen_lp, top_ids, top_lps


def sample(logits, temperature=None, seeds=None, top_p=None, top_k=None, min_p=None, out=None):
    R, V = logits.shape
    ids = torch.zeros(R, dtype=torch.int32)
    for r in range(R):
        t = float(temperature[r]) if temperature is not None else 0.0
        row = logits[r].to(torch.float64)
        if not t > 0:
            ids[r] = int((row == row.max()).to(torch.int32).argmax())
            continue
        p = torch.exp(row / t - (row / t).max())
        keep = torch.ones(V, dtype=torch.bool)
        order = torch.sort(p, descending=True, stable=True).indices
        k = int(top_k[r]) if top_k is not None else 0
        if 0 < k < V:
            keep &= p >= p[order[k - 1]]
        mp = float(min_p[r]) if min_p is not None else 0.0
        if mp > 0:
            keep &= p >= mp * p.max()
        tp = float(top_p[r]) if top_p is not None else 1.0
        if tp < 1.0:
            ps = torch.where(keep, p, torch.zeros_like(p))[order]
            c = torch.cumsum(ps, 0) / p.sum()
            n = int((c < tp).sum().item()) + 1
            cut = ps[min(n, V) - 1]
            keep &= p >= cut
        pk = torch.where(keep, p, torch.zeros_like(p))
        c = torch.cumsum(pk, 0)
        target = _uniform(int(seeds[r]) if seeds is not None else 0) * c[-1].item()
        idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64)).item())
        idx = min(idx, V - 1)
        while not keep[idx]:
            idx += 1
        ids[r] = idx
    if out is not None:
        out.copy_(ids)
        return out
    return ids


# -- parts of decoders that normalise a sublayer's output, shift tokens, gate or clamp ----
def token_shift(resid, mix, state, step, out_dtype):
    out = torch.empty_like(resid)
    cu = [int(v) for v in step.cu_q]
    for s in range(len(cu) - 1):
        a, b = cu[s], cu[s + 1]
        slot = int(step.state_slot[s])
        prev = torch.cat([state[slot][None, :], resid[a:b - 1]], dim=0)
        out[a:b] = resid[a:b] + (prev - resid[a:b]) * mix
        state[slot] = resid[b - 1]
    return out.to(out_dtype)


def _group_norm(v, gain, groups, eps):
    n, w = v.shape
    parts = v.reshape(n, groups, w // groups)
    ms = (parts * parts).sum(-1, keepdim=True) / (w // groups)
    return (parts * (1.0 / torch.sqrt(ms + eps))).reshape(n, w) * gain


def group_norm_add(resid, delta, gain, groups, eps, cast_dtype=None):
    resid += _group_norm(_f(delta), gain, groups, eps)
    return resid.to(cast_dtype) if cast_dtype is not None else None


def group_norm_rows(resid, rows, gain, groups, eps, out_dtype):
    v = resid if rows is None else resid[rows.long()]
    return _group_norm(v, gain, groups, eps).to(out_dtype)


def glu_clamped(gu, limit, alpha, up_shift):
    i = gu.shape[1] // 2
    g = torch.clamp(_f(gu[:, :i]), max=limit)
    u = torch.clamp(_f(gu[:, i:]), -limit, limit)
    return (g / (1.0 + torch.exp(-alpha * g)) * (u + up_shift)).to(gu.dtype)


def gate_up_glu_clamped(x, w_gate_up, limit, alpha, up_shift):
    return glu_clamped(linear(x, w_gate_up), limit, alpha, up_shift)


def batched_linear(x, w):
    return torch.bmm(_f(x), _f(w).transpose(1, 2)).to(x.dtype)


def _turn_pairs(v, positions, freq, mag, rot_dims):
    # v [T, ..., d]: pairs (2i, 2i+1), i < rot_dims / 2, turned by position * freq[i]
    if not rot_dims:
        return v
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [rot_dims // 2]
    a = (positions.to(torch.float32)[:, None] * freq[None, :]).reshape(shape)
    c, s = torch.cos(a) * mag, torch.sin(a) * mag
    out = v.clone()
    u, w = v[..., 0:rot_dims:2], v[..., 1:rot_dims:2]
    out[..., 0:rot_dims:2] = u * c - w * s
    out[..., 1:rot_dims:2] = w * c + u * s
    return out


def latent_prepare(proj, q_off, kv_off, positions, freq, mag, gain, eps, heads, dim, rot_dim,
                   rot_dims, rank, cache, slots):
    T = proj.shape[0]
    x = _f(proj)
    if cache is not None:
        c = x[:, kv_off:kv_off + rank]
        c = c * (1.0 / torch.sqrt((c * c).sum(-1, keepdim=True) / rank + eps)) * gain
        kr = _turn_pairs(x[:, kv_off + rank:kv_off + rank + rot_dim], positions, freq, mag,
                         rot_dims)
        _scatter(cache, torch.cat([c, kr], dim=-1)[:, None, :], slots)
    q = x[:, q_off:q_off + heads * (dim + rot_dim)].reshape(T, heads, dim + rot_dim)
    q_rot = _turn_pairs(q[..., dim:], positions, freq, mag, rot_dims).contiguous().to(proj.dtype)
    return q_rot, q[..., :dim].transpose(0, 1).contiguous().to(proj.dtype)


def latent_attention(q_lat, q_rot, cache, block_table, step, window, scale):
    H, T, rank = q_lat.shape
    page = cache.shape[2]
    out = torch.zeros(H, T, rank, dtype=torch.float32)
    for t in range(T):
        s, pos = int(step.seq_of_token[t]), int(step.positions[t])
        start = max(0, pos - window + 1) if window > 0 else 0
        kp = torch.arange(start, pos + 1)
        pages = block_table[s][(kp // page).long()].long()
        assert (pages >= 0).all(), "attention reads a page that was given back"
        rec = _f(cache[pages, 0, (kp % page).long(), :])
        q = torch.cat([_f(q_lat[:, t]), _f(q_rot[t])], dim=-1)       # [H, rank + rot]
        sc = (q @ rec.T) * scale
        p = torch.exp(sc - sc.max(dim=-1, keepdim=True).values)
        out[:, t] = (p @ rec[:, :rank]) / p.sum(-1, keepdim=True)
    return out.to(q_lat.dtype)


def gate_heads(o, proj, gate_off):
    H, T, D = o.shape
    g = _f(proj[:, gate_off:gate_off + H * D])
    return (_f(o).transpose(0, 1).reshape(T, H * D) / (1.0 + torch.exp(-g))).to(o.dtype)


# ---------------------------------------------------------------------------------------
# parts of decoders with a parallel arrangement, recurrent mixers and tied keys/values
def embed_sinusoid(table, ids, positions, freq, scale):
    x = _f(table)[ids.long()] * scale
    a = positions.to(torch.float32)[:, None] * freq[None, :]
    W = x.shape[1]
    pos = torch.stack([torch.sin(a), torch.cos(a)], dim=-1).reshape(x.shape[0], -1)[:, :W]
    return x + pos


def add_rmsnorm_sum(resid, terms, vector, gains, eps, out_dtype, rows=None):
    total = None
    for t in terms:
        if hasattr(t, "materialize"):
            t = t.materialize()
        total = _f(t) if total is None else total + _f(t)
    if vector is not None:
        total = vector[None, :].expand_as(resid) if total is None else total + vector
    if rows is None:
        if total is not None:
            resid += total
        v = resid
    else:
        v = resid[rows.long()]
        if total is not None:
            v = v + total[rows.long()]
    ms = (v * v).sum(-1, keepdim=True) / v.shape[-1]
    n = v * (1.0 / torch.sqrt(ms + eps))
    return tuple((n * g).to(out_dtype) for g in gains)


def qk_norm_append(qk, q_gain, k_gain, positions, heads, kv_heads, head_dim, eps, temp_coef,
                   temp_every, k_cache, v_cache, slots):
    T = qk.shape[0]
    x = _f(qk)
    q = x[:, :heads * head_dim].reshape(T, heads, head_dim)
    k = x[:, heads * head_dim:].reshape(T, kv_heads, head_dim)

    def unit(v):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)

    qn = unit(q) * q_gain
    if temp_every > 0:
        p = positions.to(torch.float32)
        qn = qn * (1.0 + temp_coef * torch.log(torch.floor((p + 1) / temp_every) + 1.0))[:, None, None]
    if k_cache is not None:
        _scatter(k_cache, unit(k) * k_gain, slots)
        _scatter(v_cache, k, slots)
    return qn.to(qk.dtype)


def shift_mix(x, mu, state, step):
    T, W = x.shape
    out = torch.zeros(mu.shape[0], T, W)
    for s in range(step.num_seqs):
        a, b = int(step.cu_q[s]), int(step.cu_q[s + 1])
        slot = int(step.state_slot[s])
        h = _f(x[a:b])
        prev = torch.cat([state[slot][None, :], h[:-1]], 0)
        out[:, a:b] = h[None] + (prev - h)[None] * mu[:, None, :]
        state[slot] = h[-1]
    return out.to(x.dtype)


def lowrank_decay(x, w2t, b, mode, tau=1.0, head_log_rate=None):
    x = _f(x)
    if mode == "exp_rate_softplus":
        z = x @ w2t + (b if b is not None else 0.0)
        rate = torch.exp(head_log_rate).repeat_interleave(w2t.shape[1] // head_log_rate.numel())
        return torch.exp(-rate * torch.nn.functional.softplus(z, threshold=30.0))
    if mode == "exp_exp_tanh":
        return torch.exp(-torch.exp(torch.tanh(x) @ w2t + b))
    assert mode == "sigmoid_root"
    return torch.exp(torch.nn.functional.logsigmoid(x @ w2t + b) / tau)


def linear_recurrence(q, k, v, decay, bonus, state, step, heads, dim, vdim, q_scale=1.0,
                      bonus_form=False):
    T = q.shape[0]
    qf = _f(q).reshape(T, heads, dim) * q_scale
    kf, vf = _f(k).reshape(T, heads, dim), _f(v).reshape(T, heads, vdim)
    w = decay.reshape(T, heads, dim)
    out = torch.zeros(T, heads, vdim)
    for s in range(step.num_seqs):
        slot = int(step.state_slot[s])
        S = state[slot].clone()
        for t in range(int(step.cu_q[s]), int(step.cu_q[s + 1])):
            kv = kf[t][:, :, None] * vf[t][:, None, :]
            if bonus_form:
                out[t] = torch.einsum("hkv,hk->hv", S + bonus[:, :, None] * kv, qf[t])
                S = w[t][:, :, None] * S + kv
            else:
                S = w[t][:, :, None] * S + kv
                out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
        state[slot] = S
    return out


def head_norm_gate(o, weight, gate, eps, out_dtype, gate_form="silu"):
    T, H, V = o.shape
    n = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
    n = n * (weight.reshape(H, V) if weight.numel() == H * V else weight)
    g = _f(gate).reshape(T, H, V)
    act = torch.sigmoid(g) if gate_form == "sigmoid" else g / (1.0 + torch.exp(-g))
    return (n * act).reshape(T, H * V).to(out_dtype)


# -- layers around a short convolution and a matrix of state; the scaled pre-norm ---------
def _pending_total(resid, delta, delta_scale, vector):
    if hasattr(delta, "materialize"):
        delta = delta.materialize()
    total = None
    if delta is not None:
        total = _f(delta) * delta_scale
    if vector is not None:
        total = vector[None, :].expand_as(resid) if total is None else total + vector
    return total


def add_scaled_norm(resid, delta, delta_scale, vector, gain, eps, out_dtype, center=True,
                    rows=None):
    total = _pending_total(resid, delta, delta_scale, vector)
    if rows is None:
        if total is not None:
            resid += total
        v = resid
    else:
        v = resid[rows.long()]
        if total is not None:
            v = v + total[rows.long()]
    if center:
        v = v - v.mean(-1, keepdim=True)
    ms = (v * v).mean(-1, keepdim=True)
    return (v / torch.sqrt(ms + eps) * gain).to(out_dtype)


def stream_concat(resid, delta, delta_scale, vector, first, out_dtype):
    total = _pending_total(resid, delta, delta_scale, vector)
    x = resid if total is None else resid + total
    return torch.cat([x, first], -1).to(out_dtype)


def causal_conv(x, w, bias, state, step, silu=True):
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros(T, C)
    for s in range(step.num_seqs):
        a, b = int(step.cu_q[s]), int(step.cu_q[s + 1])
        if b <= a:
            continue
        slot = int(step.state_slot[s])
        past = state[slot] if taps > 1 else torch.zeros(0, C)
        rows = torch.cat([past, _f(x[a:b])], 0)                   # [taps - 1 + n, C]
        acc = torch.zeros(b - a, C) if bias is None else bias[None, :].repeat(b - a, 1)
        for j in range(taps):
            acc = acc + rows[j:j + b - a] * w[:, j]
        out[a:b] = acc
        if taps > 1:
            state[slot] = rows[-(taps - 1):]
    if silu:
        out = out * torch.sigmoid(out)
    return out.to(x.dtype)


def ssd_recurrence(xbc, dt_raw, dt_bias, a_log, d_skip, state, step, heads, vdim, nstate,
                   groups):
    T = xbc.shape[0]
    inner = heads * vdim
    x = _f(xbc[:, :inner]).reshape(T, heads, vdim)
    B = _f(xbc[:, inner:inner + groups * nstate]).reshape(T, groups, nstate)
    C = _f(xbc[:, inner + groups * nstate:]).reshape(T, groups, nstate)
    per = heads // groups
    B, C = B.repeat_interleave(per, 1), C.repeat_interleave(per, 1)       # [T, heads, N]
    dt = torch.nn.functional.softplus(_f(dt_raw) + dt_bias, threshold=30.0)
    a = torch.exp(-torch.exp(a_log) * dt)
    out = torch.zeros(T, heads, vdim)
    for s in range(step.num_seqs):
        slot = int(step.state_slot[s])
        S = state[slot].clone()
        for t in range(int(step.cu_q[s]), int(step.cu_q[s + 1])):
            S = a[t][:, None, None] * S + (dt[t][:, None] * B[t])[:, :, None] * x[t][:, None, :]
            out[t] = torch.einsum("hnv,hn->hv", S, C[t]) + d_skip[:, None] * x[t]
        state[slot] = S
    return out.reshape(T, inner)


def delta_recurrence(q, k, v, beta_raw, decay, state, step, heads, kv_heads, dim, vdim,
                     unit_eps, q_scale):
    T = q.shape[0]
    per = heads // kv_heads

    def unit(z):
        z = _f(z).reshape(T, kv_heads, dim)
        return (z / torch.sqrt((z * z).sum(-1, keepdim=True) + unit_eps)).repeat_interleave(per, 1)

    qf, kf = unit(q) * q_scale, unit(k)
    vf = _f(v).reshape(T, heads, vdim)
    beta = torch.sigmoid(_f(beta_raw))
    g = decay.reshape(T, heads, dim)
    out = torch.zeros(T, heads, vdim)
    for s in range(step.num_seqs):
        slot = int(step.state_slot[s])
        S = state[slot].clone()
        for t in range(int(step.cu_q[s]), int(step.cu_q[s + 1])):
            S = g[t][:, :, None] * S
            u = beta[t][:, None] * (vf[t] - torch.einsum("hkv,hk->hv", S, kf[t]))
            S = S + kf[t][:, :, None] * u[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
        state[slot] = S
    return out


def gated_group_norm(y, z, gain, groups, eps):
    T, W = y.shape
    zz = _f(z)
    v = (y * (zz * torch.sigmoid(zz))).reshape(T, groups, W // groups)
    v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
    return (v.reshape(T, W) * gain).to(z.dtype)


def normed_pair_mean(left, right, gain_left, gain_right, eps):
    def unit(v):
        v = _f(v)
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
    return 0.5 * (unit(left) * gain_left + unit(right) * gain_right)


def relu_squared(x):
    v = torch.relu(_f(x))
    return (v * v).to(x.dtype)


def table_route(token_ids, table, num_experts):
    idx = table[token_ids.long()].to(torch.int32)
    return torch.full(idx.shape, 1.0 / table.shape[1], dtype=torch.float32), idx


def scale_rows(x, scale):
    x *= scale
    return x


# -- embedding from token pairs, prepared attention, biased gated unit, identity experts ----
def embed_pair_norm(table, pair_table, gain, step, prev_state, buckets, mul_prev, mul_cur, eps):
    ids = [int(v) for v in step.token_ids]
    cu = [int(v) for v in step.cu_q]
    rows = []
    for s in range(len(cu) - 1):
        slot = int(step.state_slot[s])
        pos0 = int(step.q_pos0[s])
        for t in range(cu[s], cu[s + 1]):
            if pos0 + (t - cu[s]) == 0:
                rows.append(buckets)
            else:
                prev = ids[t - 1] if t > cu[s] else int(prev_state[slot, 0])
                rows.append((prev * mul_prev + ids[t] * mul_cur) % buckets)
        prev_state[slot, 0] = ids[cu[s + 1] - 1]
    x = _f(table)[torch.tensor(ids)] + _f(pair_table)[torch.tensor(rows)]
    ms = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(ms + eps)) * gain


def _turn(v, positions, freq, magnitude, rot, interleaved):
    # v [T, heads, dim] fp32
    if not rot:
        return v
    a = positions.to(torch.float32)[:, None] * freq[None, :]
    c, s = (torch.cos(a) * magnitude)[:, None, :], (torch.sin(a) * magnitude)[:, None, :]
    out = v.clone()
    if interleaved:
        x, y = v[..., 0:rot:2], v[..., 1:rot:2]
        out[..., 0:rot:2] = x * c - y * s
        out[..., 1:rot:2] = y * c + x * s
    else:
        h = rot // 2
        x, y = v[..., :h], v[..., h:rot]
        out[..., :h] = x * c - y * s
        out[..., h:rot] = y * c + x * s
    return out


def attention_prepare(qkv, positions, freq, magnitude, rot, interleaved, heads, kv_heads,
                      head_dim, value_dim, q_gain, k_gain, eps, head_unit, earlier, lam,
                      k_cache, v_cache, slots, want_dense_kv=False):
    T = qkv.shape[0]
    dq, dk = heads * head_dim, kv_heads * head_dim
    x = _f(qkv)
    q, k, v = x[:, :dq], x[:, dq:dq + dk], x[:, dq + dk:]

    def whole(z, g):
        ms = (z * z).sum(-1, keepdim=True) / z.shape[-1]
        return z * (1.0 / torch.sqrt(ms + eps)) * g
    if q_gain is not None:
        q, k = whole(q, q_gain), whole(k, k_gain)
    q = _turn(q.reshape(T, heads, head_dim), positions, freq, magnitude, rot, interleaved)
    k = _turn(k.reshape(T, kv_heads, head_dim), positions, freq, magnitude, rot, interleaved)
    if head_unit:
        q = q * (1.0 / torch.sqrt((q * q).sum(-1, keepdim=True) / head_dim + eps))
        k = k * (1.0 / torch.sqrt((k * k).sum(-1, keepdim=True) / head_dim + eps))
    if earlier is not None:
        m = float(lam.reshape(-1)[0])
        v = (1.0 - m) * v + m * _f(earlier)
    v = v.reshape(T, kv_heads, value_dim)
    q, k, v = q.to(qkv.dtype), k.to(qkv.dtype), v.to(qkv.dtype)
    if k_cache is not None:
        _scatter(k_cache, k, slots)
        _scatter(v_cache, v, slots)
    return (q, k, v) if want_dense_kv else q


def glu_bias_act(gu, bias, activation="gelu_tanh"):
    i = gu.shape[1] // 2
    x = _f(gu)
    if bias is not None:
        x = x + bias
    g, u = x[:, :i], x[:, i:]
    if activation == "silu":
        a = g / (1.0 + torch.exp(-g))
    else:
        a = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g * g * g)))
    return (a * u).to(gu.dtype)


def identity_rows(x, rows, offsets, first_identity, y):
    lo, hi = int(offsets[first_identity]), int(offsets[-1])
    if hi > lo:
        y[lo:hi] = x[rows[lo:hi].long()].to(y.dtype)
    return y
