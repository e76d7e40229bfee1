"""Mapovik: from the typed config to a ``ModelSpec``.

The only file that knows how this design chooses its parts.  Every layer is the
pre-norm arrangement with a scaled residual, x += m * mixer(norm1(x)); x += m *
ffn(norm2(x)), with layer norms that have a gain and no bias.  A "parallel" layer's mixer
is softmax attention (grouped key/value heads, value heads of a size of their own, the
leading entries of each head rotated with linearly scaled frequencies) and a state-space
mixer side by side, their outputs RMS-normed and averaged; a "channel_delta" layer's mixer
is the delta rule with a decay per key channel.  The feed-forward is down(relu(up h)^2),
a mixture of gated experts chosen by a table indexed with the token id, or none.  The
stream starts as embed[token]; the head is a matrix of its own and its products are
multiplied by ``logit_scale``.  Layers loop.start .. loop.stop-1 run loop.times times in a
row with the same weights, every pass with caches and state of its own; ahead of every
pass the stream x becomes ``loop.in`` [x; x0] (x0 the embedding output) and row t of
``loop.step`` is added.  Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.in``,
``loop.step``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``.

Scores, maxima, sums and softmax weights are 32-bit in every attention kernel.  Heads whose
values have the keys' size and an even one run on the kernels the other models use (in
bfloat16 the tensor-core kernels, where the weights enter their product with the values as
bfloat16 operands of a matrix product with 32-bit accumulation); every other shape, and
every 32-bit run, on the fp32-arithmetic kernels.
"""
from __future__ import annotations

from ..config.mapovik_config import DENSE, PARALLEL, MapovikConfig
from ..parts.specs import (AttentionSpec, GatedDeltaSpec, LayerNormSpec, LayerSpec, ModelSpec,
                           NormedPairSpec, ReluSquaredSpec, RopeSpec, RunEntry, StateSpaceSpec,
                           StreamAddSpec, TableMoeSpec)

LOOP_TABLE = "loop.step"
LOOP_PROJECTION = "loop.in"
UNIT_EPS = 1e-6               # fixed by the design: q and k are x / sqrt(sum x^2 + 1e-6)


def _mixer(cfg: MapovikConfig, layer):
    if layer.type == PARALLEL:
        a, s = layer.left, layer.right
        position = (RopeSpec(head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base,
                             scaling_factor=a.rot_factor) if a.rot_dims else None)
        general = a.vdim != a.dim or a.dim % 2 == 1
        left = AttentionSpec(
            hidden=cfg.width, heads=a.heads, kv_heads=a.kv_heads, head_dim=a.dim,
            qkv_bias=False, scale=a.scale, window=0, position=position,
            value_dim=a.vdim if a.vdim != a.dim else 0, fp32_weights=general, out_float32=True,
            names=("q", "k", "v", "o"))
        right = StateSpaceSpec(hidden=cfg.width, heads=s.heads, vdim=s.vdim, state=s.state,
                               groups=s.groups, conv=s.conv, norm_groups=s.norm_groups,
                               norm_eps=cfg.norm_eps)
        return NormedPairSpec(hidden=cfg.width, left=left, right=right, norm_eps=cfg.norm_eps)
    d = layer.delta
    return GatedDeltaSpec(hidden=cfg.width, heads=d.heads, kv_heads=d.kv_heads, dim=d.dim,
                          vdim=d.vdim, conv=d.conv, norm_eps=cfg.norm_eps, unit_eps=UNIT_EPS,
                          decay_rank=d.rank, gate_rank=d.gate_rank)


def _ffn(cfg: MapovikConfig, f):
    if f is None:
        return None
    if f.kind == DENSE:
        return ReluSquaredSpec(hidden=cfg.width, intermediate=f.ff)
    return TableMoeSpec(hidden=cfg.width, vocab=cfg.vocab, num_experts=f.experts, top_k=f.top,
                        expert_intermediate=f.ff)


def build_spec(cfg: MapovikConfig) -> ModelSpec:
    norm = LayerNormSpec(size=cfg.width, eps=cfg.norm_eps, suffix="")
    layers = []
    for i, layer in enumerate(cfg.layers):
        ffn = _ffn(cfg, layer.mlp)
        layers.append(LayerSpec(
            prefix=f"l{i}", input_norm=norm, mixer=_mixer(cfg, layer),
            post_norm=norm if ffn is not None else None, ffn=ffn, input_norm_name="norm1",
            mixer_name="mix", post_norm_name="norm2", ffn_name="mlp", kind="pre_norm",
            residual_scale=cfg.residual_mult))
    n, a, b = len(layers), cfg.loop_start, cfg.loop_stop
    if not cfg.has_loop:
        schedule = [RunEntry(i) for i in range(n)]
    else:
        schedule = [RunEntry(i) for i in range(a)]
        for t in range(cfg.loop_times):
            for i in range(a, b):
                before = (StreamAddSpec(table=LOOP_TABLE, rows=cfg.loop_times, row=t,
                                        project=LOOP_PROJECTION) if i == a else None)
                schedule.append(RunEntry(i, cache_copy=t, before=before))
        schedule += [RunEntry(i) for i in range(b, n)]
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=cfg.width,
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, tied_head=False,
        embed_name="embed", final_norm_name="final.norm", head_name="head",
        logit_scale=cfg.logit_scale)
