"""Feed-forward parts: the dense SwiGLU and the routed mixture of experts.

Dense (src/model/qwen2.cc:1042-1048, 1413-1434): gate and up fused along the
output dimension, ``silu(gate) * up``, down projection, no biases.

Mixture of experts (src/model/moe_ffn.cc:158-367): router logits -> softmax over
all experts -> top-k (ties to the lower index) -> optional renormalisation ->
routed scale; stable dispatch by expert; per expert ``down(silu(gate(x)) *
up(x))``; combine in slot order with fp32 weights; a shared expert over every
token whose output is scaled by ``sigmoid(x . w_gate)`` when gated
(moe_ffn.cc:308-355).  Expert weights are stacked per layer as
``[E, 2I, H]`` (gate rows then up rows per expert) and ``[E, H, I]``
(src/model/deepseek_v2.cc:519-556).
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .registry import build_part, register_part


class SwiGluFeedForward:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        self.gate_up_w = self.down_w = None

    def _names(self):
        return getattr(self.spec, "names", ("gate_proj.weight", "up_proj.weight",
                                            "down_proj.weight"))

    def tensors(self):
        s, p = self.spec, self.prefix
        g, u, d = self._names()
        return [
            TensorDecl(f"{p}.{g}", (s.intermediate, s.hidden)),
            TensorDecl(f"{p}.{u}", (s.intermediate, s.hidden)),
            TensorDecl(f"{p}.{d}", (s.hidden, s.intermediate)),
        ]

    def bind(self, w):
        p = self.prefix
        g, u, d = self._names()
        self.gate_up_w = torch.cat([w[f"{p}.{g}"], w[f"{p}.{u}"]], dim=0).contiguous()
        self.down_w = w[f"{p}.{d}"]

    def forward(self, x, step=None):
        ops = self.ctx.ops
        return ops.linear(ops.gate_up_swiglu(x, self.gate_up_w), self.down_w)


class ClampedGluFeedForward:
    """``down(min(g, L) * sigmoid(alpha * min(g, L)) * (clamp(u, -L, L) + up_shift))``: a
    gated unit whose gate is cut off above and whose linear branch is cut off on both
    sides before one is added to it.  Gate and up are one product over concatenated
    weights; the result leaves in fp32 for the norm that follows."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        self.gate_up_w = self.down_w = None

    def tensors(self):
        s, p = self.spec, self.prefix
        g, u, d = s.names
        return [
            TensorDecl(f"{p}.{g}", (s.intermediate, s.hidden)),
            TensorDecl(f"{p}.{u}", (s.intermediate, s.hidden)),
            TensorDecl(f"{p}.{d}", (s.hidden, s.intermediate)),
        ]

    def bind(self, w):
        p = self.prefix
        g, u, d = self.spec.names
        self.gate_up_w = torch.cat([w[f"{p}.{g}"], w[f"{p}.{u}"]], dim=0).contiguous()
        self.down_w = w[f"{p}.{d}"]

    def forward(self, x, step=None):
        s, ops = self.spec, self.ctx.ops
        act = ops.gate_up_glu_clamped(x, self.gate_up_w, s.limit, s.alpha, s.up_shift)
        return ops.linear(act, self.down_w, out_dtype=torch.float32)


class BiasedGluFeedForward:
    """``down(act(gate h + b_g) * (up h + b_u)) + b_d``: a gated unit with a bias on each of
    its three projections and the tanh form of gelu (or silu) on the gate.  Gate and up
    are one product over concatenated weights; their biases and the activation are one
    pass over its result; the last bias travels with the output as the vector of a pending
    sum, so the norm that adds the output to the stream adds it in the same pass."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        if spec.activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"{prefix}: activation {spec.activation!r}")
        self.gate_up_w = self.down_w = self.gate_up_b = self.down_b = None

    def _bias_names(self):
        return [f"{self.prefix}.{n}{self.spec.bias_suffix}" for n in self.spec.names]

    def tensors(self):
        s, p = self.spec, self.prefix
        g, u, d = s.names
        decls = [TensorDecl(f"{p}.{g}", (s.intermediate, s.hidden)),
                 TensorDecl(f"{p}.{u}", (s.intermediate, s.hidden)),
                 TensorDecl(f"{p}.{d}", (s.hidden, s.intermediate))]
        if s.bias:
            gb, ub, db = self._bias_names()
            decls += [TensorDecl(gb, (s.intermediate,), keep="float32", init="bias"),
                      TensorDecl(ub, (s.intermediate,), keep="float32", init="bias"),
                      TensorDecl(db, (s.hidden,), keep="float32", init="bias")]
        return decls

    def bind(self, w):
        p = self.prefix
        g, u, d = self.spec.names
        self.gate_up_w = torch.cat([w[f"{p}.{g}"], w[f"{p}.{u}"]], dim=0).contiguous()
        self.down_w = w[f"{p}.{d}"]
        if self.spec.bias:
            gb, ub, db = self._bias_names()
            self.gate_up_b = torch.cat([w[gb], w[ub]], dim=0).contiguous()
            self.down_b = w[db]

    def forward(self, x, step=None):
        from .base import PendingSum
        ops = self.ctx.ops
        act = ops.glu_bias_act(ops.linear(x, self.gate_up_w), self.gate_up_b,
                               self.spec.activation)
        y = ops.linear(act, self.down_w)
        if self.down_b is None:
            return y
        return PendingSum(terms=[y], vector=self.down_b, dtype=self.ctx.dtype)


_SIDE_STREAMS: dict = {}


class MoeFeedForward:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        self.identity = int(getattr(spec, "identity_experts", 0) or 0)
        self.outputs = spec.num_experts + self.identity      # what the router scores
        self.group_count = int(getattr(spec, "group_count", 0) or 0)
        self.group_keep = int(getattr(spec, "group_keep", 0) or 0)
        self.renorm_eps = float(getattr(spec, "renorm_eps", -1.0))
        self.correction_name = getattr(spec, "correction_name", None)
        self.correction = None
        self.ruled = bool(self.identity or self.group_count or self.correction_name
                          or self.renorm_eps >= 0)
        if spec.top_k > self.outputs:
            raise ValueError("top_k exceeds the number of experts")
        if self.group_count and (self.outputs % self.group_count
                                 or not 0 < self.group_keep <= self.group_count
                                 or self.group_keep * (self.outputs // self.group_count)
                                 < spec.top_k):
            raise ValueError(f"{prefix}: {self.group_keep} of {self.group_count} groups over "
                             f"{self.outputs} router outputs, {spec.top_k} chosen")
        self.router_w = self.expert_gate_up = self.expert_down = None
        self.shared = None
        self._shared_bytes = 0
        self.shared_gate_w = None
        self._side = None
        if spec.shared is not None:
            # any registered feed-forward may serve as the shared expert
            self.shared = build_part("feed_forward", spec.shared, ctx,
                                     f"{prefix}.{spec.shared_name}")

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_router_limits", None)
        if check is not None:
            check(self.spec.hidden, self.outputs, self.spec.top_k, self.prefix)
        check = getattr(self.ctx.ops, "check_router_group_limits", None)
        if check is not None and self.group_count:
            check(self.group_count, self.prefix)
        if self.shared is not None and hasattr(self.shared, "check_limits"):
            self.shared.check_limits()

    def _router_name(self):
        return f"{self.prefix}.{getattr(self.spec, 'router_name', 'gate.weight')}"

    def _expert_names(self, e: int):
        names = getattr(self.spec, "expert_names", (
            "experts.{e}.gate_proj.weight", "experts.{e}.up_proj.weight",
            "experts.{e}.down_proj.weight"))
        return tuple(f"{self.prefix}.{n.format(e=e)}" for n in names)

    def tensors(self):
        s, p = self.spec, self.prefix
        decls = [TensorDecl(self._router_name(), (self.outputs, s.hidden), keep="float32")]
        if self.correction_name:
            decls.append(TensorDecl(f"{p}.{self.correction_name}", (self.outputs,),
                                    keep="float32", init="bias"))
        for e in range(s.num_experts):
            g, u, d = self._expert_names(e)
            decls += [
                TensorDecl(g, (s.expert_intermediate, s.hidden)),
                TensorDecl(u, (s.expert_intermediate, s.hidden)),
                TensorDecl(d, (s.hidden, s.expert_intermediate)),
            ]
        if self.shared is not None:
            decls += self.shared.tensors()
            if s.shared_gated:
                decls.append(TensorDecl(f"{p}.{s.shared_gate_name}.weight", (1, s.hidden),
                                        keep="float32"))
        return decls

    def bind(self, w):
        s, p = self.spec, self.prefix
        self.router_w = w[self._router_name()]
        if self.correction_name:
            self.correction = w[f"{p}.{self.correction_name}"]
        gu = torch.empty((s.num_experts, 2 * s.expert_intermediate, s.hidden),
                         dtype=self.ctx.dtype, device=self.ctx.device)
        dn = torch.empty((s.num_experts, s.hidden, s.expert_intermediate),
                         dtype=self.ctx.dtype, device=self.ctx.device)
        for e in range(s.num_experts):
            g, u, d = self._expert_names(e)
            gu[e, :s.expert_intermediate] = w[g]
            gu[e, s.expert_intermediate:] = w[u]
            dn[e] = w[d]
        self.expert_gate_up, self.expert_down = gu, dn
        if self.shared is not None:
            self.shared.bind({d.name: w[d.name] for d in self.shared.tensors()})
            self._shared_bytes = sum(w[d.name].numel() * w[d.name].element_size()
                                     for d in self.shared.tensors())
            if s.shared_gated:
                self.shared_gate_w = w[f"{p}.{s.shared_gate_name}.weight"].reshape(-1).contiguous()

    # In a step of few tokens the kernels leave the GPU partly idle; the shared
    # expert (which needs nothing from the router) then runs beside the routed experts,
    # on a stream of its own: its products cover the router's short kernels and the
    # boundaries between them (69 MB of shared weights a layer: a decode step of 3.94
    # against 4.27 ms at batch 8, 13.4 against 13.5 ms at batch 64).  One case is left
    # out: a large shared expert in a step of a few tokens, where its products and the
    # routed ones are the same kind of weight-streaming kernel, each able to keep the
    # memory busy alone, and beside each other they only take each other's places on the
    # multiprocessors (440 MB of shared weights a layer at batch 8: 19.3 ms beside, 16.1 ms
    # after; at batch 1, where the routed products are short, 6.1 beside against 6.6 ms,
    # and at batch 32, where the routed products are persistent tensor-core kernels, 24.7
    # against 25.4 ms).  Swapping the roles there - the shared expert on the main stream,
    # the router's short kernels and the dispatch beside it - measured worse still (20.1 ms).
    #
    # In larger steps the shared expert still runs on the stream of its own, but it
    # is handed over later, after the dispatch and just before the routed gate/up product:
    # at prompt sizes the routed products are bound by reading the experts' weights and
    # leave the tensor pipe idle, the shared expert's products are bound by the tensor
    # pipe, and the routed kernels, launched first, keep their places (a prompt portion of
    # 512 tokens 5.0 against 5.6 ms, 1,024 tokens 7.1 against 7.6 ms, 2,048 tokens 12.26
    # against 12.55 ms, 8,192 tokens 44.6 against 45.0 ms; handed over first, as below the
    # bound, 5.5 / 7.2 / 12.1 / 45.5 ms).  Not for a large shared expert: at the sizes that
    # have one (64 experts of 2560 x 3584, eight chosen) an expert sees 256 rows of a
    # 2,048-token portion and the routed products keep the tensor pipe busy themselves
    # (62.5 against 62.7 ms), while what the shared expert allocates on its own stream (a
    # gigabyte at 8,192 tokens and 20,480 columns) comes on top of what the main stream
    # holds, since the allocator keeps a pool per stream.
    # Between the two the later hand-over already pays (128 tokens 3.84 against 4.18 ms,
    # 256 tokens 4.19 against 4.55 ms; 32 tokens and decode steps of 32 and 64 sequences the
    # same either way), so the early one is kept for steps of at most 16 tokens, and, for a
    # large shared expert, which is never handed over late, up to 256.
    OVERLAP_MAX_TOKENS = 256
    EARLY_MAX_TOKENS = 16
    OVERLAP_LARGE_WEIGHT_BYTES = 160 << 20
    OVERLAP_LARGE_NOT_FOR_TOKENS = (3, 16)

    def _overlap_shared(self, tokens: int) -> bool:
        """Whether the shared expert is handed to its stream before the router."""
        large = self._shared_bytes > self.OVERLAP_LARGE_WEIGHT_BYTES
        if tokens > (self.OVERLAP_MAX_TOKENS if large else self.EARLY_MAX_TOKENS):
            return False
        lo, hi = self.OVERLAP_LARGE_NOT_FOR_TOKENS
        return not (large and lo <= tokens <= hi)

    def _side_stream(self):
        # One stream per device for all layers: the allocator keeps a pool of memory per
        # stream, and a stream per layer kept every layer's copy of the shared expert's
        # activations for itself (7 GB at 8,192 tokens and 24 layers); the layers run one
        # after the other anyway.
        if self._side is None:
            dev = torch.device(self.ctx.device)
            if dev not in _SIDE_STREAMS:
                _SIDE_STREAMS[dev] = torch.cuda.Stream(device=dev)
            self._side = _SIDE_STREAMS[dev]
        return self._side

    def forward(self, x, step=None):
        s, ops = self.spec, self.ctx.ops
        shared, side, ready = None, None, None
        beside = self.shared is not None and x.is_cuda
        if beside and self._overlap_shared(x.shape[0]):
            side = self._side_stream()
            main = torch.cuda.current_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                shared = self.shared.forward(x, step)
        elif (beside and x.shape[0] > self.EARLY_MAX_TOKENS
              and self._shared_bytes <= self.OVERLAP_LARGE_WEIGHT_BYTES):
            side = self._side_stream()
            main = torch.cuda.current_stream(x.device)
            ready = main.record_event()        # x is there; what follows is not waited for
        if self.ruled:
            topk_w, topk_idx, shared_logit = ops.router_topk(
                x, self.router_w, s.top_k, s.renormalize, s.routed_scale,
                extra_w=self.shared_gate_w, correction=self.correction,
                group_count=self.group_count, group_keep=self.group_keep,
                renorm_eps=self.renorm_eps)
        else:
            topk_w, topk_idx, shared_logit = ops.router_topk(
                x, self.router_w, s.top_k, s.renormalize, s.routed_scale,
                extra_w=self.shared_gate_w)
        # identity experts are the router's last outputs: the stable dispatch puts their
        # rows behind every expert's, where no product writes
        all_offsets, rows, dest = ops.moe_dispatch(topk_idx, self.outputs)
        offsets = all_offsets[:s.num_experts + 1] if self.identity else all_offsets
        if ready is not None:
            side.wait_event(ready)
            with torch.cuda.stream(side):
                shared = self.shared.forward(x, step)
        act = ops.grouped_gate_up_swiglu(x, rows, offsets, self.expert_gate_up)
        # `offsets` was written by the dispatch, two launches back: the down product may
        # start on its weights while the gate/up product drains
        y = ops.grouped_down(act, offsets, self.expert_down, offsets_settled=True)
        if self.identity:
            # a token's row for an identity expert is its own input
            ops.identity_rows(x, rows, all_offsets, s.num_experts, y)
        if side is not None:
            main.wait_stream(side)
        elif self.shared is not None:
            shared = self.shared.forward(x, step)
        combine = getattr(ops, "moe_combine_pending", ops.moe_combine)
        return combine(y, dest, topk_w, shared, shared_logit)


class ReluSquaredFeedForward:
    """``down(relu(up h)^2)``, no biases; the result leaves in fp32 for the norm that adds
    it."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        self.up_w = self.down_w = None

    def tensors(self):
        s, p = self.spec, self.prefix
        u, d = s.names
        return [TensorDecl(f"{p}.{u}", (s.intermediate, s.hidden)),
                TensorDecl(f"{p}.{d}", (s.hidden, s.intermediate))]

    def bind(self, w):
        u, d = self.spec.names
        self.up_w, self.down_w = w[f"{self.prefix}.{u}"], w[f"{self.prefix}.{d}"]

    def forward(self, x, step=None):
        ops = self.ctx.ops
        act = ops.relu_squared(ops.linear(x, self.up_w))
        return ops.linear(act, self.down_w, out_dtype=torch.float32)


class TableMoeFeedForward:
    """Mixture of gated experts whose choice is a table look-up: row ``token id`` of an
    integer table [vocab, top] names the token's experts, each with weight 1 / top.  After
    the look-up it is the routed mixture's own path: stable dispatch by expert, grouped
    gate/up product with silu(gate) * up, grouped down product, combine in slot order with
    fp32 weights."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx, self.prefix = spec, ctx, prefix
        if not 0 < spec.top_k <= spec.num_experts:
            raise ValueError(f"{prefix}: {spec.top_k} of {spec.num_experts} experts")
        self.table = self.expert_gate_up = self.expert_down = None

    def check_limits(self):
        check = getattr(self.ctx.ops, "check_router_limits", None)
        if check is not None:
            check(self.spec.hidden, self.spec.num_experts, self.spec.top_k, self.prefix)

    def _expert_names(self, e: int):
        return tuple(f"{self.prefix}.{n.format(e=e)}" for n in self.spec.expert_names)

    def tensors(self):
        s, p = self.spec, self.prefix
        decls = [TensorDecl(f"{p}.{s.table_name}", (s.vocab, s.top_k), keep="int32",
                            init="distinct", high=s.num_experts)]
        for e in range(s.num_experts):
            g, u, d = self._expert_names(e)
            decls += [TensorDecl(g, (s.expert_intermediate, s.hidden)),
                      TensorDecl(u, (s.expert_intermediate, s.hidden)),
                      TensorDecl(d, (s.hidden, s.expert_intermediate))]
        return decls

    def bind(self, w):
        s, p = self.spec, self.prefix
        self.table = w[f"{p}.{s.table_name}"].contiguous()
        lo, hi = int(self.table.min()), int(self.table.max())
        if lo < 0 or hi >= s.num_experts:
            raise ValueError(f"{p}.{s.table_name}: entries {lo}..{hi} name experts outside "
                             f"0..{s.num_experts - 1}")
        gu = torch.empty((s.num_experts, 2 * s.expert_intermediate, s.hidden),
                         dtype=self.ctx.dtype, device=self.ctx.device)
        dn = torch.empty((s.num_experts, s.hidden, s.expert_intermediate),
                         dtype=self.ctx.dtype, device=self.ctx.device)
        for e in range(s.num_experts):
            g, u, d = self._expert_names(e)
            gu[e, :s.expert_intermediate] = w[g]
            gu[e, s.expert_intermediate:] = w[u]
            dn[e] = w[d]
        self.expert_gate_up, self.expert_down = gu, dn

    def forward(self, x, step=None):
        s, ops = self.spec, self.ctx.ops
        topk_w, topk_idx = ops.table_route(step.token_ids, self.table, s.num_experts)
        offsets, rows, dest = ops.moe_dispatch(topk_idx, s.num_experts)
        act = ops.grouped_gate_up_swiglu(x, rows, offsets, self.expert_gate_up)
        y = ops.grouped_down(act, offsets, self.expert_down, offsets_settled=True)
        combine = getattr(ops, "moe_combine_pending", ops.moe_combine)
        return combine(y, dest, topk_w, None, None)


register_part("feed_forward", "swiglu", SwiGluFeedForward)
register_part("feed_forward", "moe", MoeFeedForward)
register_part("feed_forward", "clamped_glu", ClampedGluFeedForward)
register_part("feed_forward", "relu_squared", ReluSquaredFeedForward)
register_part("feed_forward", "glu_biased", BiasedGluFeedForward)
register_part("feed_forward", "moe_table", TableMoeFeedForward)
