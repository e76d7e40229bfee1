"""Grouped-query attention over the paged cache.

The reference's layer body (src/model/qwen2.cc:912-1030): one fused QKV
projection (weights concatenated in q, k, v order, qwen2.cc:1368-1403), biases on
Q, K and V only, rotation of Q and K after the bias, rotated keys written to the
cache before attention (qwen2.cc:928-931), scores scaled by a constant given in
the spec, causal by position with an optional window, and an output projection
without bias.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import PagedKvNeed, StateNeed
from .registry import build_part, register_part


_HF_NAMES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
             "q_proj.bias", "k_proj.bias", "v_proj.bias")


class AttentionMixer:
    """Grouped-query attention.  The value heads may have a size of their own
    (``spec.value_dim``): the value pages are then that wide and the fp32-arithmetic
    kernels run; they also run when the spec asks for 32-bit softmax weights."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec = spec
        self.ctx = ctx
        self.prefix = prefix
        self.vdim = int(getattr(spec, "value_dim", 0) or spec.head_dim)
        self.exact = bool(getattr(spec, "fp32_weights", False))
        self.position = build_part("position", spec.position, ctx, prefix)
        self.qkv_w = self.qkv_b = self.o_w = None

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_attention_limits", None)
        if check is not None:
            s = self.spec
            check(s.heads, s.kv_heads, s.head_dim, self.ctx.dtype, self.prefix,
                  allow_odd=self.exact or self.vdim != s.head_dim)
            if self.vdim != s.head_dim:
                check(s.heads, s.kv_heads, self.vdim, self.ctx.dtype, self.prefix, allow_odd=True)

    def _names(self):
        names = tuple(getattr(self.spec, "names", _HF_NAMES))
        return [f"{self.prefix}.{n}" for n in names + _HF_NAMES[len(names):]]

    # -- weights -----------------------------------------------------------
    def tensors(self):
        s = self.spec
        q, k, v, o, qb, kb, vb = self._names()
        dq, dk, dv = s.heads * s.head_dim, s.kv_heads * s.head_dim, s.kv_heads * self.vdim
        decls = [
            TensorDecl(q, (dq, s.hidden)),
            TensorDecl(k, (dk, s.hidden)),
            TensorDecl(v, (dv, s.hidden)),
            TensorDecl(o, (s.hidden, s.heads * self.vdim)),
        ]
        if s.qkv_bias:
            decls += [
                TensorDecl(qb, (dq,), keep="float32", init="bias"),
                TensorDecl(kb, (dk,), keep="float32", init="bias"),
                TensorDecl(vb, (dv,), keep="float32", init="bias"),
            ]
        if self.position is not None:
            decls += self.position.tensors()
        return decls

    def bind(self, w):
        q, k, v, o, qb, kb, vb = self._names()
        self.qkv_w = torch.cat([w[q], w[k], w[v]], dim=0).contiguous()
        self.o_w = w[o]
        if self.spec.qkv_bias:
            self.qkv_b = torch.cat([w[qb], w[kb], w[vb]], dim=0).contiguous()
        if self.position is not None:
            self.position.bind(w)

    # -- cache -------------------------------------------------------------
    def cache_needs(self):
        s = self.spec
        if self.vdim != s.head_dim:
            return [PagedKvNeed(s.kv_heads, s.head_dim, s.window,
                                entry_dims=(s.head_dim, self.vdim))]
        return [PagedKvNeed(s.kv_heads, s.head_dim, s.window)]

    # -- step --------------------------------------------------------------
    def _project_out(self, attn, tokens):
        s = self.spec
        out_dtype = torch.float32 if getattr(s, "out_float32", False) else None
        return self.ctx.ops.linear(attn.view(tokens, s.heads * self.vdim), self.o_w,
                                   out_dtype=out_dtype)

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        group = step.groups[cache.group]
        inv_freq, rot = (None, 0)
        if self.position is not None:
            inv_freq, rot = self.position.rotary_table()
        custom = getattr(self.position, "apply", None)
        plain = self.vdim == s.head_dim and not self.exact
        if not plain:
            if custom is not None:
                raise ValueError(f"{self.prefix}: a position encoding that is not a rotation "
                                 "table is not combined with value heads of another size")
            qkv = ops.linear(x, self.qkv_w)
            q = ops.qkv_rope_append(
                qkv, self.qkv_b, step.positions, inv_freq, rot, s.heads, s.kv_heads, s.head_dim,
                cache.k if cache.writes else None, cache.v if cache.writes else None,
                group.slots if cache.writes else None, value_dim=self.vdim)
            attn = ops.paged_attention(q, cache.k, cache.v, group.block_table, step, s.window,
                                       s.scale, fp32_weights=True)
            return self._project_out(attn, step.num_tokens)
        fused = getattr(ops, "qkv_project_applies", None)
        if custom is None and cache.writes and fused is not None and fused(
                x, self.qkv_w, s.heads, s.kv_heads, s.head_dim, rot):
            # a few tokens: projection, bias, rotation and cache write in one kernel
            q = ops.qkv_project_rope_append(
                x, self.qkv_w, self.qkv_b, step.positions, inv_freq, rot, s.heads, s.kv_heads,
                s.head_dim, cache.k, cache.v, group.slots)
            attn = ops.paged_attention(q, cache.k, cache.v, group.block_table, step, s.window,
                                       s.scale)
            return self._project_out(attn, step.num_tokens)
        qkv = ops.linear(x, self.qkv_w)
        if custom is None:
            q = ops.qkv_rope_append(
                qkv, self.qkv_b, step.positions, inv_freq, rot, s.heads, s.kv_heads, s.head_dim,
                cache.k if cache.writes else None, cache.v if cache.writes else None,
                group.slots if cache.writes else None)
        else:
            # an encoding that is not a rotation table works on dense q and k first
            q, k, v = ops.qkv_rope_append(qkv, self.qkv_b, step.positions, None, 0, s.heads,
                                          s.kv_heads, s.head_dim, None, None, None,
                                          want_dense_kv=True)
            custom(q, k, step.positions)
            if cache.writes:
                ops.append_kv(k, v, cache.k, cache.v, group.slots)
        attn = ops.paged_attention(q, cache.k, cache.v, group.block_table, step, s.window, s.scale)
        return self._project_out(attn, step.num_tokens)


register_part("mixer", "attention", AttentionMixer)


class TiedKvAttentionMixer:
    """Grouped-query attention whose values are its keys as projected: one projection
    gives q and k, the raw k rows are stored as the values and the RMS-normed ones as the
    keys (both in pages of the same shape, so every paged attention kernel serves), the
    normed queries take the position's temperature, and the scores may be squashed by
    tanh.  Norms, temperature and the squashing are fp32."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        self.qk_w = self.o_w = self.q_gain = self.k_gain = None

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_attention_limits", None)
        if check is not None:
            s = self.spec
            check(s.heads, s.kv_heads, s.head_dim, self.ctx.dtype, self.prefix, allow_odd=True)

    def _name(self, key):
        return f"{self.prefix}.{dict(self.spec.names)[key]}"

    def tensors(self):
        s = self.spec
        return [
            TensorDecl(self._name("q"), (s.heads * s.head_dim, s.hidden)),
            TensorDecl(self._name("k"), (s.kv_heads * s.head_dim, s.hidden)),
            TensorDecl(self._name("q_norm"), (s.head_dim,), keep="float32", init="gain"),
            TensorDecl(self._name("k_norm"), (s.head_dim,), keep="float32", init="gain"),
            TensorDecl(self._name("o"), (s.hidden, s.heads * s.head_dim)),
        ]

    def bind(self, w):
        self.qk_w = torch.cat([w[self._name("q")], w[self._name("k")]], dim=0).contiguous()
        self.q_gain, self.k_gain = w[self._name("q_norm")], w[self._name("k_norm")]
        self.o_w = w[self._name("o")]

    def cache_needs(self):
        return [PagedKvNeed(self.spec.kv_heads, self.spec.head_dim, self.spec.window)]

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        group = step.groups[cache.group]
        qk = ops.linear(x, self.qk_w)
        q = ops.qk_norm_append(
            qk, self.q_gain, self.k_gain, step.positions, s.heads, s.kv_heads, s.head_dim,
            s.norm_eps, s.temp_coef, s.temp_every,
            cache.k if cache.writes else None, cache.v if cache.writes else None,
            group.slots if cache.writes else None)
        attn = ops.paged_attention(q, cache.k, cache.v, group.block_table, step, s.window,
                                   s.scale, softcap=s.softcap)
        return ops.linear(attn.view(step.num_tokens, s.heads * s.head_dim), self.o_w,
                          out_dtype=torch.float32)


register_part("mixer", "attention_tied_kv", TiedKvAttentionMixer)


CONV_INPUTS = "attention_conv_inputs"


class PreparedAttentionMixer:
    """Grouped-query attention over a window whose q, k and v pass, between the projection
    and the cache, a short causal convolution, a norm of the whole q and k rows, the
    rotation, a division of every q and k head by its root mean square and a blend of the
    values with those an earlier layer left for this step - each only where the spec asks
    for it.  The window may keep a request's first tokens visible and the softmax may have
    one added to its denominator.  Keys and values live in the framework's pages (the
    value pages as wide as the value heads); the convolutions' last inputs in the state
    slots.  Norms, angles, scores and weights are fp32 in every element type."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError(f"{prefix}: {s.heads} heads do not split over {s.kv_heads} "
                             "key/value heads")
        if s.value_mix not in ("none", "source", "mix"):
            raise ValueError(f"{prefix}: value_mix {s.value_mix!r}")
        self.vdim = int(s.value_dim or s.head_dim)
        self.dq, self.dk = s.heads * s.head_dim, s.kv_heads * s.head_dim
        self.dv = s.kv_heads * self.vdim
        self.taps = int(s.conv_taps) if s.conv_taps and s.conv_taps > 1 else 1
        self.has_conv = bool(s.conv_taps)
        self.position = build_part("position", s.position, ctx, prefix)
        if self.position is not None and not hasattr(self.position, "pair_table"):
            raise ValueError(f"{prefix}: the position encoding must give a table of pair "
                             "frequencies")
        self.names = dict(s.names)
        self.qkv_w = self.o_w = self.conv_w = self.q_gain = self.k_gain = self.lam = None

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_attention_limits", None)
        if check is not None:
            s = self.spec
            check(s.heads, s.kv_heads, s.head_dim, self.ctx.dtype, self.prefix, allow_odd=True)
            check(s.heads, s.kv_heads, self.vdim, self.ctx.dtype, self.prefix, allow_odd=True)
        check = getattr(self.ctx.ops, "check_delta_limits", None)
        if check is not None and self.taps > 1:
            check(1, self.taps, self.prefix)

    def _n(self, key):
        return f"{self.prefix}.{self.names[key]}"

    def tensors(self):
        s = self.spec
        decls = [TensorDecl(self._n("q"), (self.dq, s.hidden)),
                 TensorDecl(self._n("k"), (self.dk, s.hidden)),
                 TensorDecl(self._n("v"), (self.dv, s.hidden)),
                 TensorDecl(self._n("o"), (s.hidden, s.heads * self.vdim))]
        if self.has_conv:
            decls += [TensorDecl(self._n("q_conv"), (self.dq, s.conv_taps), keep="float32"),
                      TensorDecl(self._n("k_conv"), (self.dk, s.conv_taps), keep="float32"),
                      TensorDecl(self._n("v_conv"), (self.dv, s.conv_taps), keep="float32")]
        if s.projection_norm:
            decls += [TensorDecl(self._n("q_norm"), (self.dq,), keep="float32", init="gain"),
                      TensorDecl(self._n("k_norm"), (self.dk,), keep="float32", init="gain")]
        # the layer that leaves its values has the scalar too (it is not used there); a layer
        # that mixes nothing may have it in its checkpoint all the same
        decls.append(TensorDecl(self._n("mix"), (), keep="float32", init="bias",
                                optional=s.value_mix == "none"))
        return decls

    def bind(self, w):
        s = self.spec
        self.qkv_w = torch.cat([w[self._n("q")], w[self._n("k")], w[self._n("v")]],
                               dim=0).contiguous()
        self.o_w = w[self._n("o")]
        if self.has_conv:
            self.conv_w = torch.cat([w[self._n("q_conv")], w[self._n("k_conv")],
                                     w[self._n("v_conv")]], dim=0).contiguous()
        if s.projection_norm:
            self.q_gain, self.k_gain = w[self._n("q_norm")], w[self._n("k_norm")]
        if s.value_mix == "mix":
            self.lam = w[self._n("mix")].reshape(1).contiguous()

    def cache_needs(self):
        s = self.spec
        needs = [PagedKvNeed(s.kv_heads, s.head_dim, s.window,
                             entry_dims=(s.head_dim, self.vdim),
                             keep_first=s.keep_first if s.window > 0 else 0)]
        if self.taps > 1:
            needs.append(StateNeed(CONV_INPUTS, (self.taps - 1, self.dq + self.dk + self.dv),
                                   torch.float32))
        return needs

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        group = step.groups[cache.group]
        qkv = ops.linear(x, self.qkv_w)                     # [T, q | k | v]
        if self.has_conv:
            qkv = ops.causal_conv(qkv, self.conv_w, None, cache.state.get(CONV_INPUTS), step,
                                  silu=False)
        key = f"value_mix:{s.value_mix_key}"
        earlier = None
        if s.value_mix == "mix":
            if key not in step.shared:
                raise ValueError(f"{self.prefix}: no earlier layer left values to mix with")
            earlier = step.shared[key]
        freq, magnitude, rot, interleaved = (None, 1.0, 0, False)
        if self.position is not None:
            freq, magnitude, rot, interleaved = self.position.pair_table()
        q = ops.attention_prepare(
            qkv, step.positions, freq, magnitude, rot, interleaved, s.heads, s.kv_heads,
            s.head_dim, self.vdim, self.q_gain, self.k_gain, s.norm_eps, s.head_unit_norm,
            earlier, self.lam, cache.k if cache.writes else None,
            cache.v if cache.writes else None, group.slots if cache.writes else None)
        if s.value_mix == "source":
            # this layer's values as projected (and convolved): a view of its own rows
            step.shared[key] = qkv[:, self.dq + self.dk:]
        attn = ops.paged_attention(q, cache.k, cache.v, group.block_table, step, s.window,
                                   s.scale, fp32_weights=True,
                                   keep_first=s.keep_first if s.window > 0 else 0, sink=s.sink)
        return ops.linear(attn.view(step.num_tokens, s.heads * self.vdim), self.o_w)


register_part("mixer", "attention_prepared", PreparedAttentionMixer)
