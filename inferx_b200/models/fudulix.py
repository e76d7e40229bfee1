"""Fudulix: from the typed config to a ``ModelSpec``.

The only file that knows how this design chooses its parts.  The stream starts as the RMS
norm of embed[token] plus a row of a hashed table of token pairs.  Every layer is the
pre-norm arrangement, x += mixer(norm1(x)); x += ffn(norm2(x)), with RMS norms whose gains
are used as stored.  Both kinds of layer are grouped-query attention over a window with
value heads of a size of their own, and differ in how q, k and v are prepared and masked:
"attention" rotates neighbouring pairs with wavelength-stretched frequencies, then divides
every q and k head by its root mean square, and its softmax has one added to the
denominator; "attention_2" passes q, k and v through short causal convolutions, norms the
whole q and k rows with gains, rotates in the half-split layout with ramp-stretched
frequencies and a factor on cos and sin, and its window also keeps the sequence's first
tokens.  Layers that mix values blend theirs with those of the first such layer.  The
feed-forward is a gated unit with biases and the tanh form of gelu, or a mixture of silu
gated experts whose router knows groups, a correction used for the choice alone and
identity experts, with a shared expert beside it; or none.  Tensor names: ``embed``,
``bigram``, ``embed.norm``, ``final.norm``, ``head`` and per layer i ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.fudulix_config import ATTENTION, DENSE, FudulixConfig
from ..parts.specs import (BiasedGluSpec, LayerSpec, ModelSpec, MoeSpec, PairEmbeddingSpec,
                           PreparedAttentionSpec, RmsNormSpec, RunEntry, ScaledRopeSpec,
                           SwiGluSpec)

RENORM_EPS = 1e-20            # fixed by the design: chosen weights over (their sum + 1e-20)


def _position(kind, m):
    if m.rot is None or m.rot.dims == 0:
        return None
    first = kind == ATTENTION
    scaling = None
    if m.rot.scaling is not None:
        scaling = (("wavelength" if first else "ramp"),) + tuple(m.rot.scaling)
    return ScaledRopeSpec(head_dim=m.dim, rotary_dim=m.rot.dims, theta=m.rot.base,
                          layout="interleaved" if first else "half", scaling=scaling)


def _mixer(cfg: FudulixConfig, layer, mix_role: str):
    m = layer.mixer
    first = layer.type == ATTENTION
    return PreparedAttentionSpec(
        hidden=cfg.width, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
        scale=m.scale, window=m.window, position=_position(layer.type, m), norm_eps=cfg.norm_eps,
        keep_first=m.keep_first, sink=first, conv_taps=0 if first else m.conv,
        projection_norm=not first, head_unit_norm=first, value_mix=mix_role)


def _ffn(cfg: FudulixConfig, f):
    if f is None:
        return None
    if f.kind == DENSE:
        return BiasedGluSpec(hidden=cfg.width, intermediate=f.ff, activation="gelu_tanh")
    shared = (SwiGluSpec(hidden=cfg.width, intermediate=f.shared_ff, names=("gate", "up", "down"))
              if f.shared_ff else None)
    return MoeSpec(
        hidden=cfg.width, num_experts=f.experts, top_k=f.top, expert_intermediate=f.ff,
        renormalize=True, routed_scale=1.0, shared=shared, shared_gated=False,
        shared_name="shared", router_name="router",
        expert_names=("e{e}.gate", "e{e}.up", "e{e}.down"), identity_experts=f.identity,
        correction_name="correction", group_count=f.group_count, group_keep=f.group_keep,
        renorm_eps=RENORM_EPS)


def build_spec(cfg: FudulixConfig) -> ModelSpec:
    norm = RmsNormSpec(size=cfg.width, eps=cfg.norm_eps, suffix="")
    layers = []
    mixing = False
    for i, layer in enumerate(cfg.layers):
        role = "none"
        if layer.mixer.v_mix:
            role = "mix" if mixing else "source"
            mixing = True
        ffn = _ffn(cfg, layer.mlp)
        layers.append(LayerSpec(
            prefix=f"l{i}", input_norm=norm, mixer=_mixer(cfg, layer, role),
            post_norm=norm if ffn is not None else None, ffn=ffn, input_norm_name="norm1",
            mixer_name="mix", post_norm_name="norm2", ffn_name="mlp", kind="pre_norm"))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=cfg.width,
        layers=tuple(layers), schedule=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm, tied_head=False, embed_name="embed", final_norm_name="final.norm",
        head_name="head",
        embedding=PairEmbeddingSpec(buckets=cfg.buckets, mul_prev=cfg.mul_prev,
                                    mul_cur=cfg.mul_cur, norm=norm))
