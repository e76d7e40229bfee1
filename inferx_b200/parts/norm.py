"""RMSNorm with the residual add folded in.

``out = x * (1 / sqrt(mean(x^2) + eps)) * gain`` with the sum in fp32, no mean
subtraction, no bias, the gain used as stored (not 1 + gain): the reference's
RmsNormKernel (src/backends/cuda/ops/layers.cu:50-76).  A spec with ``gain_offset`` 1
describes weights stored around zero; the offset is added once, in fp32, when the
weights are bound.  The residual add that the
reference does in a kernel of its own (layers.cu:542-548) happens in the same
pass, on an fp32 residual stream.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .registry import register_part


class RmsNorm:
    # the contribution to add may arrive unwritten (``ops.CombinePending``); the kernel
    # behind ``add_rmsnorm`` folds it in
    accepts_pending = True

    def __init__(self, spec, ctx, prefix: str):
        self.spec = spec
        self.ctx = ctx
        self.name = f"{prefix}{getattr(spec, 'suffix', '.weight')}"
        self.offset = float(getattr(spec, "gain_offset", 0.0))
        self.gain = None

    def tensors(self):
        # a weight stored around zero (the gain is offset + w) is drawn like a bias
        return [TensorDecl(self.name, (self.spec.size,), keep="float32",
                           init="bias" if self.offset else "gain")]

    def bind(self, weights):
        self.gain = weights[self.name]
        if self.offset:
            self.gain = (self.gain + self.offset).contiguous()    # fp32, once

    def forward(self, resid, delta, rows=None):
        if hasattr(delta, "terms"):      # several contributions and a vector, one pass
            return self.ctx.ops.add_rmsnorm_sum(resid, delta.terms, delta.vector, (self.gain,),
                                                self.spec.eps, self.ctx.dtype, rows=rows)[0]
        return self.ctx.ops.add_rmsnorm(resid, delta, self.gain, self.spec.eps, self.ctx.dtype,
                                        rows=rows)

    def forward_pair(self, resid, delta, other: "RmsNorm"):
        """This norm's and ``other``'s view of the same rows (``resid`` after ``delta`` was
        added), from one pass over the stream."""
        terms = delta.terms if hasattr(delta, "terms") else ([] if delta is None else [delta])
        vector = getattr(delta, "vector", None)
        return self.ctx.ops.add_rmsnorm_sum(resid, terms, vector, (self.gain, other.gain),
                                            self.spec.eps, self.ctx.dtype)


register_part("norm", "rmsnorm", RmsNorm)


class LayerNorm:
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * gain, no bias, all in fp32, with the
    residual add folded in: what is pending (one tensor times a scale, and a vector) is
    added to the stream in the pass that normalises it."""
    accepts_pending = True
    accepts_scaled = True

    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx = spec, ctx
        self.name = f"{prefix}{getattr(spec, 'suffix', '.weight')}"
        self.gain = None

    def tensors(self):
        return [TensorDecl(self.name, (self.spec.size,), keep="float32", init="gain")]

    def bind(self, weights):
        self.gain = weights[self.name]

    def forward(self, resid, delta, rows=None):
        scale, vector = 1.0, None
        if hasattr(delta, "terms"):
            scale, vector = float(getattr(delta, "scale", 1.0)), delta.vector
            if len(delta.terms) == 1:
                delta = delta.terms[0]
            elif not delta.terms:
                delta = None
            else:                       # several tensors: their scaled sum, written once
                vector_free = type(delta)(terms=delta.terms, dtype=torch.float32,
                                          scale=delta.scale)
                delta, scale = vector_free.materialize(), 1.0
        return self.ctx.ops.add_scaled_norm(resid, delta, scale, vector, self.gain,
                                            self.spec.eps, self.ctx.dtype, center=True, rows=rows)


register_part("norm", "layernorm", LayerNorm)


class GroupedRmsNorm:
    """RMS norm in groups: a row is cut into ``groups`` equal consecutive parts, each is
    divided by its own sqrt(mean(part^2) + eps), and the whole row is multiplied by the
    gain; all in fp32.  Two uses: ``add_normed`` normalises a sublayer's output and adds
    it into the residual stream (x += norm(f(x))); ``forward`` normalises rows of the
    residual stream itself (the model's last norm)."""

    def __init__(self, spec, ctx, prefix: str):
        self.spec = spec
        self.ctx = ctx
        self.name = prefix
        self.gain = None
        if spec.groups <= 0 or spec.size % spec.groups:
            raise ValueError(f"{prefix}: {spec.size} entries do not split into {spec.groups} "
                             "equal groups")

    def tensors(self):
        return [TensorDecl(self.name, (self.spec.size,), keep="float32", init="gain")]

    def bind(self, weights):
        self.gain = weights[self.name]

    def add_normed(self, resid, delta, cast_dtype=None):
        """resid += norm(delta) * gain; the new residual in ``cast_dtype`` if asked."""
        return self.ctx.ops.group_norm_add(resid, delta, self.gain, self.spec.groups,
                                           self.spec.eps, cast_dtype)

    def forward(self, resid, delta, rows=None):
        if delta is not None:
            raise ValueError("a grouped norm of the residual stream takes no pending "
                             "contribution; add it first")
        return self.ctx.ops.group_norm_rows(resid, rows, self.gain, self.spec.groups,
                                            self.spec.eps, self.ctx.dtype)


register_part("norm", "grouped_rmsnorm", GroupedRmsNorm)
