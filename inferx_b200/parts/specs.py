"""Plain-data descriptions of the parts a decoder is put together from.

A model is described by a ``ModelSpec``: a list of ``LayerSpec`` (each naming its
mixer, feed-forward and norms by ``kind`` with every size and constant as a
field) and a ``schedule`` that says in which order layers run and whose cache
each run reads.  Nothing in this file knows an architecture; an architecture's
spec builder (``inferx_b200/models``) fills these in from its typed config, the
way the reference hands every number to ``MoeFfn::Config`` explicitly
(include/inferx/model/moe_ffn.h:108-132) and passes eps/theta/scale/window as
arguments to its ops (include/inferx/ops/layers.h:32,57,176,206).

A spec is any dataclass with a ``kind`` attribute; new kinds need no change
here, only a registration of the class that runs them (``parts/registry.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional


@dataclass(frozen=True)
class RmsNormSpec:
    """x / sqrt(mean(x^2) + eps) * (gain_offset + w).  ``gain_offset`` is 1 for weights
    stored around zero; ``suffix`` is what the tensor's name adds to the part's prefix."""
    size: int
    eps: float
    gain_offset: float = 0.0
    suffix: str = ".weight"
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class SinusoidSpec:
    """A position vector added to the embedding: entry 2i is sin(p * base^(-2i/size)),
    entry 2i+1 the cosine of the same angle."""
    size: int
    base: float = 10000.0
    kind: str = "sinusoid_added"


@dataclass(frozen=True)
class LayerNormSpec:
    """(x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w: a layer norm with a gain and
    no bias.  ``suffix`` is what the tensor's name adds to the part's prefix."""
    size: int
    eps: float
    suffix: str = ".weight"
    kind: str = "layernorm"


@dataclass(frozen=True)
class RopeSpec:
    """Half-split (NeoX) rotary encoding of the first ``rotary_dim`` of each head.  Every
    frequency is divided by ``scaling_factor`` (linear position scaling; 1: none)."""
    head_dim: int
    rotary_dim: int
    theta: float
    scaling_factor: float = 1.0
    kind: str = "rope"


@dataclass(frozen=True)
class GroupedRmsNormSpec:
    """RMS norm of ``groups`` equal consecutive parts of a row, each over its own root
    mean square, then the whole row times the gain."""
    size: int
    eps: float
    groups: int = 1
    kind: str = "grouped_rmsnorm"


@dataclass(frozen=True)
class InterleavedRopeSpec:
    """Rotary encoding of neighbouring pairs (2i, 2i+1) of the first ``rotary_dim``
    entries of a vector of ``head_dim``, frequency ``theta^(-2i/rotary_dim)``.  With
    ``scaling_factor`` > 0 the frequencies are stretched YaRN-wise: pair i keeps its
    frequency below ``lo``, has it divided by the factor above ``hi`` and is blended
    linearly in between, where lo and hi are the pair indices at which the original
    context ``original_context`` holds ``fast_turns`` and ``slow_turns`` full turns;
    cos and sin are multiplied by ``0.1 ln(factor) + 1``."""
    head_dim: int
    rotary_dim: int
    theta: float
    scaling_factor: float = 0.0
    original_context: float = 0.0
    fast_turns: float = 32.0
    slow_turns: float = 1.0
    kind: str = "rope_interleaved"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are widened from one cached latent per token.
    Per head: ``dim`` plain and ``rot_dim`` rotated query/key entries, ``vdim`` value
    entries; the latent has ``kv_rank`` entries and is RMS-normed with ``latent_eps``;
    one rotated key part of ``rot_dim`` is shared by all heads.  ``output_gate``: the
    heads' outputs are multiplied by sigmoid(W_g h) before the output projection."""
    hidden: int
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int        # keys visible to a query including itself; 0 = all
    position: Any      # encoding of the rotated part, or None
    latent_eps: float
    output_gate: bool = True
    # tensor names inside the mixer's prefix
    names: tuple = (("q", "q"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"), ("uk", "uk"),
                    ("uv", "uv"), ("g", "g"), ("o", "o"))
    kind: str = "latent_attention"


@dataclass(frozen=True)
class TokenShiftSpec:
    """h_t + (h_{t-1} - h_t) * mix per channel, with zeros before a sequence's first
    token; the previous token's h is per-request state."""
    size: int
    kind: str = "token_shift"


@dataclass(frozen=True)
class ClampedGluSpec:
    """down(min(g, L) * sigmoid(alpha * min(g, L)) * (clamp(u, -L, L) + up_shift)) with
    g and u the gate and up projections."""
    hidden: int
    intermediate: int
    limit: float
    alpha: float = 1.702
    up_shift: float = 1.0
    names: tuple = ("gate", "up", "down")
    kind: str = "clamped_glu"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention.  ``value_dim`` is the size of a value head when it
    differs from the query/key size ``head_dim`` (0: the same).  ``fp32_weights``: scores,
    softmax weights and their products with the values stay in 32-bit arithmetic whatever
    the element type (the tensor-core kernels round the weights to the values' type).
    ``names`` are the tensors of q, k, v, o (and their biases) inside the prefix;
    ``out_float32``: the output projection leaves in fp32."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    qkv_bias: bool
    scale: float
    window: int  # keys visible to a query including itself; 0 = all
    position: Any  # a position-encoding spec, or None
    value_dim: int = 0
    fp32_weights: bool = False
    out_float32: bool = False
    names: tuple = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
                    "q_proj.bias", "k_proj.bias", "v_proj.bias")
    kind: str = "attention"


@dataclass(frozen=True)
class TiedKvAttentionSpec:
    """Grouped-query softmax attention whose values are its keys as projected.  Queries
    and keys are RMS-normed per head (gains ``q.norm`` / ``k.norm`` shared by the heads)
    after the values were taken; no rotation.  The query at position p is multiplied by
    1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (``temp_every`` 0: not at all);
    scores are (q . k) * scale and, with ``softcap`` > 0, softcap * tanh(score / softcap)."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    scale: float
    norm_eps: float
    softcap: float = 0.0
    temp_coef: float = 0.0
    temp_every: int = 0
    window: int = 0
    names: tuple = (("q", "q"), ("k", "k"), ("q_norm", "q.norm"), ("k_norm", "k.norm"),
                    ("o", "o"))
    kind: str = "attention_tied_kv"


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a decay per key channel and a state [heads, dim, vdim] per
    request: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q scaled by
    ``q_scale``; a_t = sigmoid(z_t)^(1 / tau), z_t = W_a2 (W_a1 h) + b, a low-rank product
    whose inner size ``decay_rank`` is the checkpoint's when 0.  Each head's output is
    RMS-normed over vdim (gain shared by the heads), multiplied by silu(W_g h), projected."""
    hidden: int
    heads: int
    dim: int
    vdim: int
    tau: float
    q_scale: float
    norm_eps: float
    decay_rank: int = 0
    kind: str = "gated_linear_attention"


@dataclass(frozen=True)
class WkvSpec:
    """Time mixing with state [heads, dim, dim] per request and the previous token's input
    as further state.  Each of r, k, v, g, w reads h + (h_prev - h) * mu of its own;
    decay w_t = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)) per key channel (inner size
    ``decay_rank``, the checkpoint's when 0); o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,
    then S_t = diag(w_t) S_(t-1) + k_t v_t^T.  Each head's output is divided by its root
    mean square, multiplied by a gain over all heads and by silu(W_g mix_g), projected."""
    hidden: int
    heads: int
    dim: int
    norm_eps: float
    decay_rank: int = 0
    kind: str = "wkv"


@dataclass(frozen=True)
class StateSpaceSpec:
    """Selective state space with a scalar decay per head (state-space duality): one input
    projection laid out [z: inner | x: inner | B: groups * state | C: groups * state | dt:
    heads] with inner = heads * vdim; x, B and C pass a causal convolution of ``conv`` taps
    per channel (with bias) and silu; dt = softplus(dt + dt_bias);
    S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D x_t per head (head
    h reads group h // (heads / groups)); y * silu(z) is RMS-normed in ``norm_groups`` equal
    parts, multiplied by a gain and projected.  State per request: S [heads, state, vdim]
    fp32 and the last conv - 1 inputs of the convolution."""
    hidden: int
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int
    norm_eps: float
    names: tuple = (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"),
                    ("dt_bias", "dt_bias"), ("a_log", "A_log"), ("d", "D"), ("norm", "norm"),
                    ("o", "o"))
    kind: str = "state_space"


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Delta rule with a decay per head and key channel.  q, k ([kv_heads, dim]) and v
    ([heads, vdim]) each pass a causal convolution of ``conv`` taps per channel (no bias)
    and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times
    dim^(-1/2); beta = sigmoid(W_b h); decay g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) +
    dt_bias)) [heads, dim].  Per head: S <- g * S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  o is RMS-normed per head (gain over vdim shared by the heads), multiplied by
    sigmoid(W_g2 (W_g1 h)) and projected.  The inner sizes of the two low-rank products
    are the checkpoint's when 0.  State per request: S [heads, dim, vdim] fp32 and the last
    conv - 1 inputs of the convolutions."""
    hidden: int
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    norm_eps: float
    unit_eps: float = 1e-6
    decay_rank: int = 0
    gate_rank: int = 0
    kind: str = "gated_delta"


@dataclass(frozen=True)
class NormedPairSpec:
    """Two mixers side by side reading the same input; the result is the mean of their
    outputs, each first RMS-normed over the model width with a gain of its own
    (``<name>.out`` inside the prefix)."""
    hidden: int
    left: Any
    right: Any
    norm_eps: float
    left_name: str = "left"
    right_name: str = "right"
    gain_suffix: str = ".out"
    kind: str = "normed_pair"


@dataclass(frozen=True)
class ReluSquaredSpec:
    """down(relu(up h)^2), no biases."""
    hidden: int
    intermediate: int
    names: tuple = ("up", "down")
    kind: str = "relu_squared"


@dataclass(frozen=True)
class TableMoeSpec:
    """Mixture of gated experts without a router: row ``token id`` of an integer table
    [vocab, top] names the token's experts (the entries of a row differ); each has weight
    1 / top.  Expert: down(silu(gate h) * (up h))."""
    hidden: int
    vocab: int
    num_experts: int
    top_k: int
    expert_intermediate: int
    table_name: str = "table"
    expert_names: tuple = ("e{e}.gate", "e{e}.up", "e{e}.down")
    kind: str = "moe_table"


@dataclass(frozen=True)
class ScaledRopeSpec:
    """Rotary encoding of the first ``rotary_dim`` entries of each head with a choice of
    pairing and of frequency stretching.  ``layout`` "half" pairs entry i with entry
    i + rotary_dim / 2, "interleaved" pairs 2i with 2i + 1; pair i turns by position *
    f_i with f_i = theta^(-2i / rotary_dim).  ``scaling`` is None or a tuple:
    ("wavelength", factor, low, high, original): with l = 2 pi / f, f stays where
    l < original / high, becomes f / factor where l > original / low, and in between
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low);
    ("ramp", factor, original, fast, slow): with pair(t) = rotary_dim ln(original /
    (2 pi t)) / (2 ln theta), lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)),
    rotary_dim - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is
    f_i / factor * r_i + f_i (1 - r_i), and cos and sin are multiplied by
    0.1 ln(factor) + 1."""
    head_dim: int
    rotary_dim: int
    theta: float
    layout: str = "half"
    scaling: Any = None
    kind: str = "rope_scaled"


@dataclass(frozen=True)
class PreparedAttentionSpec:
    """Grouped-query softmax attention whose queries, keys and values are prepared between
    the projection and the cache: in this order, a causal convolution over time of
    ``conv_taps`` taps per channel of q, k and v (no bias, no activation; 0 or 1: none;
    the last taps - 1 projected rows are state per request), an RMS norm of the whole q
    row and of the whole k row with gains (``projection_norm``), the rotation
    (``position``), a division of every q and k head by its own root mean square
    (``head_unit_norm``), and the value mixing: with ``value_mix`` "mix" the values become
    (1 - lambda) v + lambda v0, v0 being the values of the same token left by the layer
    whose ``value_mix`` is "source" (the first of the model that mixes) and lambda a
    scalar of the checkpoint; what is mixed is what the cache holds.  A query at position
    i sees key j <= i when i - j < ``window`` (0: all) or j < ``keep_first``.  With
    ``sink`` one is added to the softmax's denominator (a key of score 0 without a
    value).  Scores are (q . k) * scale; scores, weights and their products with the values
    are 32-bit arithmetic in every element type."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    window: int
    position: Any
    norm_eps: float
    keep_first: int = 0
    sink: bool = False
    conv_taps: int = 0
    projection_norm: bool = False
    head_unit_norm: bool = False
    value_mix: str = "none"          # "none" | "source" | "mix"
    value_mix_key: str = "values"    # layers that mix with one another share the key
    names: tuple = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_norm", "q.norm"),
                    ("k_norm", "k.norm"), ("q_conv", "q.conv"), ("k_conv", "k.conv"),
                    ("v_conv", "v.conv"), ("mix", "vmix"))
    kind: str = "attention_prepared"


@dataclass(frozen=True)
class BiasedGluSpec:
    """down(act(gate h + b_g) * (up h + b_u)) + b_d with ``activation`` "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))) or "silu"; ``bias`` off: no b."""
    hidden: int
    intermediate: int
    activation: str = "gelu_tanh"
    bias: bool = True
    names: tuple = ("gate", "up", "down")
    bias_suffix: str = ".b"
    kind: str = "glu_biased"


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """The stream starts as norm(embed[token] + pair[row]) with row = (previous token *
    mul_prev + token * mul_cur) mod buckets, row ``buckets`` (the table's last) for a
    sequence's first token, and ``norm`` an RMS norm spec whose gain is ``norm_name``.
    The previous token is state per request."""
    buckets: int
    mul_prev: int
    mul_cur: int
    norm: Any
    table_name: str = "bigram"
    norm_name: str = "embed.norm"
    kind: str = "pair_embedding"


@dataclass(frozen=True)
class SwiGluSpec:
    hidden: int
    intermediate: int
    # tensor names inside the part's prefix: gate, up, down
    names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
    kind: str = "swiglu"


@dataclass(frozen=True)
class MoeSpec:
    hidden: int
    num_experts: int
    top_k: int
    expert_intermediate: int
    renormalize: bool
    routed_scale: float
    shared: Any               # a feed-forward spec run over every token, or None
    shared_gated: bool        # its output scaled by sigmoid(x . w_gate)
    shared_name: str = "shared_expert"
    shared_gate_name: str = "shared_expert_gate"
    # tensor names inside the part's prefix: the router's matrix, and one expert's
    # prefix with {e} for its number followed by its gate, up and down matrices
    router_name: str = "gate.weight"
    expert_names: tuple = ("experts.{e}.gate_proj.weight", "experts.{e}.up_proj.weight",
                           "experts.{e}.down_proj.weight")
    # The router may have more outputs than there are experts: its last
    # ``identity_experts`` outputs stand for experts that return their input.  With
    # ``correction_name`` a vector of the checkpoint is added to the scores for the choice
    # alone (the weights stay the plain scores).  With ``group_count`` > 0 the router's
    # outputs form that many equal groups of neighbours, a group's value is its largest
    # score (with the correction), and only outputs of the ``group_keep`` best groups can
    # be chosen.  ``renorm_eps`` >= 0: the chosen weights are divided by (their sum +
    # renorm_eps) instead of the guarded division ``renormalize`` does.
    identity_experts: int = 0
    correction_name: Optional[str] = None
    group_count: int = 0
    group_keep: int = 0
    renorm_eps: float = -1.0
    kind: str = "moe"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its parts, and ``kind``, the arrangement they run in.  "pre_norm" is
    x += mixer(norm(x)); x += ffn(norm(x)); "sublayer_norm" is x += norm(mixer(x));
    x += norm(ffn(x)), where ``input_norm`` follows the mixer and ``post_norm`` the
    feed-forward (``ffn`` and ``post_norm`` may be None: a layer without feed-forward);
    "parallel" is x += mixer(input_norm(x)) + ffn(post_norm(x)), both of the same x."""
    prefix: str  # tensor-name prefix, e.g. "model.layers.3"
    input_norm: Any
    mixer: Any
    post_norm: Any
    ffn: Any
    # names of the sub-parts inside the prefix (checkpoint naming)
    input_norm_name: str = "input_layernorm"
    mixer_name: str = "self_attn"
    post_norm_name: str = "post_attention_layernorm"
    ffn_name: str = "mlp"
    kind: str = "pre_norm"
    # a transform of what the mixer reads (a token shift, for instance), or None
    mixer_input: Any = None
    mixer_input_name: str = "shift"
    # "pre_norm" only: each sublayer's output is multiplied by this before it is added
    residual_scale: float = 1.0


@dataclass(frozen=True)
class StreamAddSpec:
    """Something done to the residual stream ahead of a run.  With ``project`` (a matrix
    [width, 2 width] by its checkpoint name) the stream x first becomes W [x; x0], x0 being
    the stream as it was before the first run (the embedding output).  Then row ``row`` of
    the tensor ``table`` ([rows, width], by its checkpoint name) is added and, with
    ``embedding``, the embedding output once more."""
    table: Optional[str] = None
    rows: int = 0
    row: int = 0
    embedding: bool = False
    project: Optional[str] = None


@dataclass(frozen=True)
class RunEntry:
    """One execution of a layer.  By default the run keeps its own cache (it writes
    this step's keys and values, then reads).  ``cache_of`` names a layer whose
    cache this run only reads: another layer's, or its own when the layer is run a
    second time in the schedule and must see what its first run stored.
    ``cache_copy`` numbers caches of the same layer: a layer that runs several times
    with the same weights, each run with a cache and state of its own, gives its runs
    different numbers.  ``before`` is added to the stream ahead of the run."""
    layer: int
    cache_of: Optional[int] = None
    cache_copy: int = 0
    before: Optional[StreamAddSpec] = None

    @property
    def cache_layer(self) -> int:
        return self.layer if self.cache_of is None else self.cache_of

    @property
    def writes_cache(self) -> bool:
        return self.cache_of is None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    layers: tuple
    schedule: tuple  # of RunEntry
    final_norm: Any
    tied_head: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"
    embed_scale: float = 1.0     # the residual stream starts as embed[token] * embed_scale
    logit_scale: float = 1.0     # the head's products are multiplied by this
    embed_position: Any = None   # a position spec whose vector is added to the embedding
    embedding: Any = None        # a spec of what forms the stream from the tokens (None: the table's rows)
