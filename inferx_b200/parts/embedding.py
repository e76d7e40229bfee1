"""Parts that form the residual stream from the token ids.

``PairEmbedding`` (kind "pair_embedding"): the stream starts as the RMS norm of
embed[token] + pair[row], where the row of the pair table is a hash of the previous and
the current token, (previous * mul_prev + token * mul_cur) mod buckets, and the table's
last row (number ``buckets``) for a sequence's first token.  The previous token of a
sequence is state per request, kept in the cache manager's state slots like any other:
the first token of a step reads it, the step's last token of the sequence replaces it,
and a slot that is handed out anew needs none, because position 0 has no previous token.
The sum, the mean of squares and the stream itself are fp32.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorDecl
from .base import StateNeed
from .registry import register_part

PREVIOUS_TOKEN = "previous_token"


class PairEmbedding:
    def __init__(self, spec, ctx, prefix: str):
        self.spec, self.ctx = spec, ctx
        if spec.buckets <= 0 or spec.mul_prev < 0 or spec.mul_cur < 0:
            raise ValueError(f"pair embedding: {spec.buckets} buckets, factors "
                             f"{spec.mul_prev} and {spec.mul_cur}")
        self.width = int(spec.norm.size)
        self.table = self.gain = None

    def tensors(self):
        s = self.spec
        return [TensorDecl(s.table_name, (s.buckets + 1, self.width)),
                TensorDecl(s.norm_name, (self.width,), keep="float32", init="gain")]

    def bind(self, w):
        self.table, self.gain = w[self.spec.table_name], w[self.spec.norm_name]

    def cache_needs(self):
        return [StateNeed(PREVIOUS_TOKEN, (1,), torch.int32)]

    def forward(self, embed_table, step, cache):
        s = self.spec
        return self.ctx.ops.embed_pair_norm(
            embed_table, self.table, self.gain, step, cache.state[PREVIOUS_TOKEN], s.buckets,
            s.mul_prev, s.mul_cur, s.norm.eps)


register_part("embedding", "pair_embedding", PairEmbedding)
