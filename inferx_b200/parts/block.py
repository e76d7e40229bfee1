"""The decoder: blocks built from specs, run in the order a schedule gives.

A block is the pre-norm residual arrangement of the reference's layer body
(src/model/qwen2.cc:908-1051): ``x += mixer(norm(x)); x += ffn(norm(x))``.  The
residual stream ``x`` is fp32; each sub-part returns its contribution in the
run's element type and the following norm adds it in (one pass over the row
instead of the reference's copy + add + norm).  The decoder embeds, runs the
schedule's entries in order (a layer may appear twice, or read another layer's
cache), gathers the rows whose logits are wanted *before* the final norm, and
multiplies those rows by the head (the reference multiplies all rows,
src/model/qwen2.cc:1066).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..weights import loader as wl
from ..weights.loader import TensorDecl
from .base import BuildContext, LayerCache, PendingSum, StepContext
from .registry import build_part, register_part


class PreNormBlock:
    """``x += m * mixer(norm(x)); x += m * ffn(norm(x))`` on the fp32 residual stream, with
    ``m`` the spec's ``residual_scale`` (1 unless the design scales its sublayers); a layer
    may have no feed-forward."""

    def __init__(self, spec, ctx: BuildContext, prefix: str):
        p = prefix
        self.spec, self.ctx = spec, ctx
        self.scale = float(getattr(spec, "residual_scale", 1.0))
        self.input_norm = build_part("norm", spec.input_norm, ctx, f"{p}.{spec.input_norm_name}")
        self.mixer = build_part("mixer", spec.mixer, ctx, f"{p}.{spec.mixer_name}")
        self.ffn = build_part("feed_forward", spec.ffn, ctx, f"{p}.{spec.ffn_name}")
        self.post_norm = (build_part("norm", spec.post_norm, ctx, f"{p}.{spec.post_norm_name}")
                          if self.ffn is not None else None)

    def parts(self):
        return [x for x in (self.input_norm, self.mixer, self.post_norm, self.ffn)
                if x is not None]

    def cache_needs(self):
        return list(self.mixer.cache_needs())

    def _scaled(self, term, norm):
        """A sublayer's output as the next norm takes it: times the residual scale."""
        if self.scale == 1.0:
            return term
        pending = PendingSum(terms=[term], dtype=self.ctx.dtype, scale=self.scale)
        if norm is None or getattr(norm, "accepts_scaled", False):
            return pending
        return pending.materialize()

    def forward(self, resid, pending, step: StepContext, cache: LayerCache):
        """``pending`` is the previous block's contribution not yet added to
        ``resid``; returns this block's own pending contribution."""
        if hasattr(pending, "materialize") and not getattr(self.input_norm, "accepts_pending",
                                                            False):
            pending = pending.materialize()
        n = self.input_norm.forward(resid, pending)
        a = self.mixer.forward(n, step, cache)
        if self.ffn is None:
            return self._scaled(a, None)
        n = self.post_norm.forward(resid, self._scaled(a, self.post_norm))
        return self._scaled(self.ffn.forward(n, step), None)


class SublayerNormBlock:
    """``x += norm(mixer(shift(x))); x += norm(ffn(x))`` on the fp32 residual stream: the
    sublayers read the stream itself and their OUTPUT is normalised before it is added.
    ``spec.input_norm`` follows the mixer, ``spec.post_norm`` the feed-forward;
    ``spec.mixer_input`` transforms what the mixer reads and may keep state per request.
    A layer may have no feed-forward."""

    def __init__(self, spec, ctx: BuildContext, prefix: str):
        p = prefix
        self.spec, self.ctx = spec, ctx
        self.mixer_input = build_part("mixer_input", spec.mixer_input, ctx,
                                      f"{p}.{spec.mixer_input_name}")
        self.mixer = build_part("mixer", spec.mixer, ctx, f"{p}.{spec.mixer_name}")
        self.mixer_norm = build_part("norm", spec.input_norm, ctx, f"{p}.{spec.input_norm_name}")
        self.ffn = build_part("feed_forward", spec.ffn, ctx, f"{p}.{spec.ffn_name}")
        self.ffn_norm = (build_part("norm", spec.post_norm, ctx, f"{p}.{spec.post_norm_name}")
                         if self.ffn is not None else None)

    def parts(self):
        return [x for x in (self.mixer_input, self.mixer, self.mixer_norm, self.ffn,
                            self.ffn_norm) if x is not None]

    def cache_needs(self):
        needs = list(self.mixer.cache_needs())
        if self.mixer_input is not None:
            needs += list(self.mixer_input.cache_needs())
        return needs

    def forward(self, resid, pending, step: StepContext, cache: LayerCache):
        if pending is not None:     # a block of another arrangement ran before this one
            if hasattr(pending, "materialize"):
                pending = pending.materialize()
            resid.add_(pending.to(resid.dtype))
        dt = self.ctx.dtype
        h = (self.mixer_input.forward(resid, step, cache) if self.mixer_input is not None
             else resid.to(dt))
        a = self.mixer.forward(h, step, cache)
        if self.ffn is None:
            self.mixer_norm.add_normed(resid, a)
            return None
        n = self.mixer_norm.add_normed(resid, a, cast_dtype=dt)
        self.ffn_norm.add_normed(resid, self.ffn.forward(n, step))
        return None


class ParallelBlock:
    """``x += mixer(input_norm(x)) + ffn(post_norm(x))``: both sublayers read the same x,
    each through a norm of its own, and their outputs are added to the stream together.
    The sum is left pending, so the next norm adds it in the pass in which it normalises;
    two RMS norms with the same eps are computed in one pass.  A layer may have no
    feed-forward."""

    def __init__(self, spec, ctx: BuildContext, prefix: str):
        p = prefix
        self.spec, self.ctx = spec, ctx
        self.input_norm = build_part("norm", spec.input_norm, ctx, f"{p}.{spec.input_norm_name}")
        self.mixer = build_part("mixer", spec.mixer, ctx, f"{p}.{spec.mixer_name}")
        self.ffn = build_part("feed_forward", spec.ffn, ctx, f"{p}.{spec.ffn_name}")
        self.post_norm = (build_part("norm", spec.post_norm, ctx, f"{p}.{spec.post_norm_name}")
                          if self.ffn is not None else None)

    def parts(self):
        return [x for x in (self.input_norm, self.mixer, self.post_norm, self.ffn)
                if x is not None]

    def cache_needs(self):
        return list(self.mixer.cache_needs())

    def forward(self, resid, pending, step: StepContext, cache: LayerCache):
        a_norm, f_norm = self.input_norm, self.post_norm
        if f_norm is None:
            if hasattr(pending, "materialize") and not getattr(a_norm, "accepts_pending", False):
                pending = pending.materialize()
            a = self.mixer.forward(a_norm.forward(resid, pending), step, cache)
            return PendingSum(terms=[a], dtype=self.ctx.dtype)
        if hasattr(a_norm, "forward_pair") and hasattr(f_norm, "gain") and \
                a_norm.spec.eps == f_norm.spec.eps:
            na, nf = a_norm.forward_pair(resid, pending, f_norm)
        else:
            if hasattr(pending, "materialize") and not getattr(a_norm, "accepts_pending", False):
                pending = pending.materialize()
            na = a_norm.forward(resid, pending)
            nf = f_norm.forward(resid, None)
        a = self.mixer.forward(na, step, cache)
        f = self.ffn.forward(nf, step)
        return PendingSum(terms=[a, f], dtype=self.ctx.dtype)


class DecoderModel:
    """Embedding, scheduled blocks, final norm and head, from a ``ModelSpec``."""

    def __init__(self, spec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        self.blocks = [build_part("block", ls, ctx, ls.prefix) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, ctx, spec.final_norm_name)
        self.embed_position = build_part("position", getattr(spec, "embed_position", None), ctx,
                                         spec.embed_name)
        # a part that forms the stream from the tokens in a way of its own (it gets the
        # embedding table and may keep state per request), or None: the table's rows
        self.embedding = build_part("embedding", getattr(spec, "embedding", None), ctx,
                                    spec.embed_name)
        self.embed = None
        self.head = None
        self.stream_tables = {}      # checkpoint name -> fp32 [rows, hidden]
        for e in spec.schedule:
            if not (0 <= e.layer < len(self.blocks)) or not (0 <= e.cache_layer < len(self.blocks)):
                raise ValueError(f"schedule entry {e} names a layer that does not exist")
            b = getattr(e, "before", None)
            if b is not None and b.table is not None and not (0 <= b.row < b.rows):
                raise ValueError(f"schedule entry {e} adds row {b.row} of {b.rows}")
        # A cache unit is one layer's cache and state; a layer whose runs keep caches of
        # their own has one unit per copy.  Units 0..L-1 are the layers' first copies.
        extra = sorted({(e.cache_layer, e.cache_copy) for e in spec.schedule
                        if getattr(e, "cache_copy", 0)})
        self.cache_units = [(i, 0) for i in range(len(self.blocks))] + extra
        self._unit_index = {u: i for i, u in enumerate(self.cache_units)}
        # cache units of parts outside the schedule come after the layers' (their caches
        # follow the schedule's in the list ``forward`` gets)
        self.extra_cache_units = []
        if self.embedding is not None and self.embedding.cache_needs():
            self.extra_cache_units.append(len(self.cache_units))
        self._keeps_embedding = any(
            getattr(e, "before", None) is not None
            and (e.before.embedding or getattr(e.before, "project", None))
            for e in spec.schedule)
        if ctx.ops is not None:
            # sizes beyond what the kernels take are refused now, not at the first launch
            for b in self.blocks:
                for part in b.parts():
                    if hasattr(part, "check_limits"):
                        part.check_limits()

    # -- weights -----------------------------------------------------------
    def _own_tensors(self) -> List[TensorDecl]:
        s = self.spec
        decls = [TensorDecl(s.embed_name, (s.vocab_size, s.hidden))]
        if not s.tied_head:
            decls.append(TensorDecl(s.head_name, (s.vocab_size, s.hidden)))
        tables = {}
        for e in s.schedule:
            b = getattr(e, "before", None)
            if b is not None and b.table is not None:
                if tables.setdefault(b.table, b.rows) != b.rows:
                    raise ValueError(f"table {b.table!r} is given two sizes in the schedule")
        decls += [TensorDecl(name, (rows, s.hidden), keep="float32", init="bias")
                  for name, rows in tables.items()]
        projections = sorted({e.before.project for e in s.schedule
                              if getattr(e, "before", None) is not None
                              and getattr(e.before, "project", None)})
        decls += [TensorDecl(name, (s.hidden, 2 * s.hidden)) for name in projections]
        return decls

    def tensors(self) -> List[TensorDecl]:
        decls = self._own_tensors()
        for b in self.blocks:
            for part in b.parts():
                decls += part.tensors()
        decls += self.final_norm.tensors()
        if self.embedding is not None:
            decls += self.embedding.tensors()
        return decls

    def load(self, source: wl.WeightSource, where: str = "weights") -> None:
        """Check every declared tensor against the source, then bind part by part."""
        wl.check(self.tensors(), source, where)
        dt, dev = self.ctx.dtype, self.ctx.device

        held = source.names()

        def fetch(decls):
            # (a tensor declared optional is fetched only if the source has it)
            return {d.name: wl.materialize(d, source, dt, dev) for d in decls
                    if not getattr(d, "optional", False) or held is None or d.name in held}

        own = fetch(self._own_tensors())
        self.embed = own[self.spec.embed_name]
        self.head = self.embed if self.spec.tied_head else own[self.spec.head_name]
        self.stream_tables = {n: t for n, t in own.items()
                              if n not in (self.spec.embed_name, self.spec.head_name)}
        # (the matrices of stream projections live in the same table, by name)
        for b in self.blocks:
            for part in b.parts():
                part.bind(fetch(part.tensors()))
        self.final_norm.bind(fetch(self.final_norm.tensors()))
        if self.embedding is not None:
            self.embedding.bind(fetch(self.embedding.tensors()))

    # -- cache needs -------------------------------------------------------
    def cache_needs(self) -> List[list]:
        """Per cache unit (a layer, or one of several copies of a layer's cache), what the
        layer's mixer wants kept between steps."""
        needs = [list(self.blocks[layer].cache_needs()) for layer, _ in self.cache_units]
        if self.extra_cache_units:
            needs.append(list(self.embedding.cache_needs()))
        return needs

    def cache_unit(self, entry) -> int:
        """The cache unit a schedule entry reads and writes."""
        return self._unit_index[(entry.cache_layer, getattr(entry, "cache_copy", 0))]

    def _project_stream(self, resid, pending, before, embedded):
        """The stream becomes W [x; x0]: what is pending is added while the two halves are
        laid side by side in the run's element type, and the product leaves in fp32."""
        ops = self.ctx.ops
        scale, vector, delta = 1.0, None, pending
        if hasattr(pending, "terms"):
            scale, vector = float(getattr(pending, "scale", 1.0)), pending.vector
            if len(pending.terms) == 1:
                delta = pending.terms[0]
            elif not pending.terms:
                delta = None
            else:
                delta, scale = PendingSum(terms=pending.terms, dtype=torch.float32,
                                          scale=scale).materialize(), 1.0
        both = ops.stream_concat(resid, delta, scale, vector, embedded, self.ctx.dtype)
        return ops.linear(both, self.stream_tables[before.project], out_dtype=torch.float32)

    def _add_before(self, pending, before, embedded):
        """What a run's ``before`` names joins what is still to be added to the stream."""
        terms, scale, vector = [], 1.0, None
        if pending is not None:
            if hasattr(pending, "terms"):
                scale = float(getattr(pending, "scale", 1.0))
                if scale != 1.0 and before.embedding:
                    # the embedding output joins unscaled: the scaled sum is written first
                    terms, scale = [pending.materialize()], 1.0
                else:
                    terms, vector = list(pending.terms), pending.vector
            else:
                terms = [pending]
        if before.embedding:
            terms.append(embedded)
        if before.table is not None:
            row = self.stream_tables[before.table][before.row]
            vector = row if vector is None else vector + row
        return PendingSum(terms=terms, vector=vector, dtype=self.ctx.dtype, scale=scale)

    # -- step --------------------------------------------------------------
    def forward(self, step: StepContext, caches: List[LayerCache],
                logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs the batch; returns fp32 logits [R, vocab] for ``logit_rows`` (token
        indices into the batch), or None when no logits are wanted."""
        ops = self.ctx.ops
        if hasattr(ops, "set_dependent_launch"):
            ops.set_dependent_launch(step.num_tokens <= ops.DEPENDENT_LAUNCH_MAX_TOKENS)
        if self.embedding is not None:
            own = caches[len(self.spec.schedule)] if self.extra_cache_units else None
            resid = self.embedding.forward(self.embed, step, own)
        elif self.embed_position is not None:
            resid = self.embed_position.embed(self.embed, step.token_ids, step.positions,
                                              self.spec.embed_scale)
        elif self.spec.embed_scale != 1.0:
            resid = ops.embed(self.embed, step.token_ids, scale=self.spec.embed_scale)
        else:
            resid = ops.embed(self.embed, step.token_ids)
        embedded = resid.clone() if self._keeps_embedding else None
        pending = None
        for entry, cache in zip(self.spec.schedule, caches):
            if getattr(entry, "before", None) is not None:
                if getattr(entry.before, "project", None):
                    resid = self._project_stream(resid, pending, entry.before, embedded)
                    pending = None
                pending = self._add_before(pending, entry.before, embedded)
            pending = self.blocks[entry.layer].forward(resid, pending, step, cache)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        if hasattr(pending, "materialize") and not getattr(self.final_norm, "accepts_pending",
                                                            False):
            pending = pending.materialize()
        n = self.final_norm.forward(resid, pending, rows=logit_rows)
        logits = ops.linear(n, self.head, out_dtype=torch.float32)
        scale = float(getattr(self.spec, "logit_scale", 1.0))
        return logits if scale == 1.0 else ops.scale_rows(logits, scale)


Block = PreNormBlock
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sublayer_norm", SublayerNormBlock)
register_part("block", "parallel", ParallelBlock)
