"""Mixers built around a short causal convolution and a matrix of state per head.

* ``StateSpaceMixer`` (kind "state_space"): selective state space with a scalar decay per
  head.  One input projection laid out [z | x | B | C | dt]; x, B, C pass a causal
  convolution with bias and silu; dt = softplus(dt + dt_bias);
  S_t = exp(-exp(A_h) dt_t) S_(t-1) + dt_t B_t x_t^T,  y_t = S_t^T C_t + D_h x_t;
  y * silu(z) is RMS-normed in equal parts, multiplied by a gain and projected.
* ``GatedDeltaMixer`` (kind "gated_delta"): delta rule with a decay per head and key
  channel.  q, k, v pass convolutions (no bias) and silu; q and k become unit vectors per
  head; S <- diag(g_t) S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t; o is
  RMS-normed per head, multiplied by a gain and a sigmoid gate from a low-rank product, and
  projected.

Both keep, per request, S in fp32 and the last taps - 1 inputs of their convolutions in
the cache manager's state slots (zeroed when a slot is handed out: the zeros before
position 0 and the empty state).  The recurrences, step sizes, decays, unit norms and
output norms are fp32; the projections and convolutions are in the run's element type.
A sequence's state column is owned by one thread from its first token of a step to its
last and every sum has an order fixed by the sizes alone, so a position's result does
not depend on how the sequence was cut into steps or on what else is in the batch.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import StateNeed
from .registry import register_part

SSD_STATE, SSD_CONV = "ssd_state", "ssd_conv_inputs"
DELTA_STATE, DELTA_CONV = "delta_state", "delta_conv_inputs"


def _rank(spec_rank: int) -> int:
    return spec_rank if spec_rank > 0 else -1


class StateSpaceMixer:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.p = spec, ctx, prefix
        s = spec
        if s.heads % s.groups:
            raise ValueError(f"{prefix}: {s.heads} heads do not split over {s.groups} groups")
        self.inner = s.heads * s.vdim
        if self.inner % s.norm_groups:
            raise ValueError(f"{prefix}: {self.inner} channels do not split into "
                             f"{s.norm_groups} norm groups")
        self.conv_width = self.inner + 2 * s.groups * s.state
        self.names = dict(s.names)

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_delta_limits", None)
        if check is not None:
            check(self.spec.state, self.spec.conv, self.p)

    def _n(self, key):
        return f"{self.p}.{self.names[key]}"

    def tensors(self):
        s = self.spec
        return [
            TensorDecl(self._n("in"), (2 * self.inner + 2 * s.groups * s.state + s.heads,
                                       s.hidden)),
            TensorDecl(self._n("conv"), (self.conv_width, s.conv), keep="float32"),
            TensorDecl(self._n("conv_bias"), (self.conv_width,), keep="float32", init="bias"),
            TensorDecl(self._n("dt_bias"), (s.heads,), keep="float32", init="bias"),
            TensorDecl(self._n("a_log"), (s.heads,), keep="float32", init="bias"),
            TensorDecl(self._n("d"), (s.heads,), keep="float32", init="gain"),
            TensorDecl(self._n("norm"), (self.inner,), keep="float32", init="gain"),
            TensorDecl(self._n("o"), (s.hidden, self.inner)),
        ]

    def bind(self, w):
        self.in_w = w[self._n("in")]
        self.conv_w, self.conv_b = w[self._n("conv")].contiguous(), w[self._n("conv_bias")]
        self.dt_bias, self.a_log, self.d = (w[self._n(k)] for k in ("dt_bias", "a_log", "d"))
        self.norm_w, self.o_w = w[self._n("norm")], w[self._n("o")]

    def cache_needs(self):
        s = self.spec
        needs = [StateNeed(SSD_STATE, (s.heads, s.state, s.vdim), torch.float32)]
        if s.conv > 1:
            needs.append(StateNeed(SSD_CONV, (s.conv - 1, self.conv_width), torch.float32))
        return needs

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        proj = ops.linear(x, self.in_w)            # [T, z | x | B | C | dt]
        z = proj[:, :self.inner]
        xbc = ops.causal_conv(proj[:, self.inner:self.inner + self.conv_width], self.conv_w,
                              self.conv_b, cache.state.get(SSD_CONV), step, silu=True)
        y = ops.ssd_recurrence(xbc, proj[:, self.inner + self.conv_width:], self.dt_bias,
                               self.a_log, self.d, cache.state[SSD_STATE], step, s.heads,
                               s.vdim, s.state, s.groups)              # fp32 [T, inner]
        y = ops.gated_group_norm(y, z, self.norm_w, s.norm_groups, s.norm_eps)
        return ops.linear(y, self.o_w, out_dtype=torch.float32)


class GatedDeltaMixer:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.p = spec, ctx, prefix
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError(f"{prefix}: {s.heads} heads do not split over {s.kv_heads} "
                             "query/key heads")
        self.qk = s.kv_heads * s.dim
        self.hv = s.heads * s.vdim
        self.conv_width = 2 * self.qk + self.hv

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_delta_limits", None)
        if check is not None:
            check(self.spec.dim, self.spec.conv, self.p)

    def tensors(self):
        s, p = self.spec, self.p
        hk = s.heads * s.dim
        ra, rg = _rank(s.decay_rank), _rank(s.gate_rank)
        return [
            TensorDecl(f"{p}.q", (self.qk, s.hidden)), TensorDecl(f"{p}.k", (self.qk, s.hidden)),
            TensorDecl(f"{p}.v", (self.hv, s.hidden)),
            TensorDecl(f"{p}.q.conv", (self.qk, s.conv), keep="float32"),
            TensorDecl(f"{p}.k.conv", (self.qk, s.conv), keep="float32"),
            TensorDecl(f"{p}.v.conv", (self.hv, s.conv), keep="float32"),
            TensorDecl(f"{p}.b", (s.heads, s.hidden)),
            TensorDecl(f"{p}.A_log", (s.heads,), keep="float32", init="bias"),
            TensorDecl(f"{p}.norm", (s.vdim,), keep="float32", init="gain"),
            TensorDecl(f"{p}.a1", (ra, s.hidden)),
            TensorDecl(f"{p}.a2", (hk, ra), keep="float32"),
            TensorDecl(f"{p}.dt_bias", (hk,), keep="float32", init="bias"),
            TensorDecl(f"{p}.g1", (rg, s.hidden)),
            TensorDecl(f"{p}.g2", (self.hv, rg)),
            TensorDecl(f"{p}.o", (s.hidden, self.hv)),
        ]

    def bind(self, w):
        p = self.p
        for a, b in (("a1", "a2"), ("g1", "g2")):
            if w[f"{p}.{a}"].shape[0] != w[f"{p}.{b}"].shape[1]:
                raise ValueError(f"{p}: {a} has {w[f'{p}.{a}'].shape[0]} rows, {b} "
                                 f"{w[f'{p}.{b}'].shape[1]} columns")
        # one product for everything that reads the mixer's input: q | k | v | b | a1
        self.front_w = torch.cat([w[f"{p}.q"], w[f"{p}.k"], w[f"{p}.v"], w[f"{p}.b"],
                                  w[f"{p}.a1"]], dim=0).contiguous()
        self.decay_rank = w[f"{p}.a1"].shape[0]
        self.conv_w = torch.cat([w[f"{p}.q.conv"], w[f"{p}.k.conv"], w[f"{p}.v.conv"]],
                                dim=0).contiguous()
        self.a2_t, self.dt_bias = w[f"{p}.a2"].t().contiguous(), w[f"{p}.dt_bias"]
        self.a_log = w[f"{p}.A_log"]
        self.g1_w, self.g2_w = w[f"{p}.g1"], w[f"{p}.g2"]
        self.norm_w, self.o_w = w[f"{p}.norm"], w[f"{p}.o"]

    def cache_needs(self):
        s = self.spec
        needs = [StateNeed(DELTA_STATE, (s.heads, s.dim, s.vdim), torch.float32)]
        if s.conv > 1:
            needs.append(StateNeed(DELTA_CONV, (s.conv - 1, self.conv_width), torch.float32))
        return needs

    def forward(self, x, step, cache):
        s, ops = self.spec, self.ctx.ops
        cw = self.conv_width
        front = ops.linear(x, self.front_w)         # [T, q | k | v | b | a1]
        qkv = ops.causal_conv(front[:, :cw], self.conv_w, None, cache.state.get(DELTA_CONV),
                              step, silu=True)
        decay = ops.lowrank_decay(front[:, cw + s.heads:], self.a2_t, self.dt_bias,
                                  mode="exp_rate_softplus", head_log_rate=self.a_log)
        o = ops.delta_recurrence(qkv[:, :self.qk], qkv[:, self.qk:2 * self.qk],
                                 qkv[:, 2 * self.qk:], front[:, cw:cw + s.heads], decay,
                                 cache.state[DELTA_STATE], step, s.heads, s.kv_heads, s.dim,
                                 s.vdim, s.unit_eps, float(s.dim) ** -0.5)
        gate = ops.linear(ops.linear(x, self.g1_w), self.g2_w)            # [T, heads * vdim]
        y = ops.head_norm_gate(o, self.norm_w, gate, s.norm_eps, self.ctx.dtype,
                               gate_form="sigmoid")
        return ops.linear(y, self.o_w, out_dtype=torch.float32)


class NormedPairMixer:
    """Two mixers side by side on the same input; the result is the mean of their outputs,
    each first RMS-normed over the model width with a gain of its own.  Each keeps what it
    needs in the layer's cache: records per token for one, state slots for the other."""

    def __init__(self, spec, ctx, prefix: str):
        from .registry import build_part
        self.spec, self.ctx, self.p = spec, ctx, prefix
        self.left = build_part("mixer", spec.left, ctx, f"{prefix}.{spec.left_name}")
        self.right = build_part("mixer", spec.right, ctx, f"{prefix}.{spec.right_name}")
        self.gain_names = (f"{prefix}.{spec.left_name}{spec.gain_suffix}",
                           f"{prefix}.{spec.right_name}{spec.gain_suffix}")

    def check_limits(self):
        for m in (self.left, self.right):
            if hasattr(m, "check_limits"):
                m.check_limits()

    def tensors(self):
        own = [TensorDecl(n, (self.spec.hidden,), keep="float32", init="gain")
               for n in self.gain_names]
        return self.left.tensors() + self.right.tensors() + own

    def bind(self, w):
        self.left.bind({d.name: w[d.name] for d in self.left.tensors()})
        self.right.bind({d.name: w[d.name] for d in self.right.tensors()})
        self.gain_left, self.gain_right = (w[n] for n in self.gain_names)

    def cache_needs(self):
        return list(self.left.cache_needs()) + list(self.right.cache_needs())

    def forward(self, x, step, cache):
        a = self.left.forward(x, step, cache)
        b = self.right.forward(x, step, cache)
        if a.dtype != b.dtype:
            a, b = a.to(torch.float32), b.to(torch.float32)
        return self.ctx.ops.normed_pair_mean(a, b, self.gain_left, self.gain_right,
                                             self.spec.norm_eps)


register_part("mixer", "state_space", StateSpaceMixer)
register_part("mixer", "gated_delta", GatedDeltaMixer)
register_part("mixer", "normed_pair", NormedPairMixer)
