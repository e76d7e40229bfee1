"""Typed configuration of the Fudulix design, read from its own ``config.json``.

Top level: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.bigram``
(``buckets``, ``mul_prev``, ``mul_cur``: the hashed table of token pairs added to the
embedding) and ``layers``: one object per layer with ``type`` ("attention": interleaved
rotation, unit heads, a window, a sink in the softmax; "attention_2": short convolutions,
a norm over the whole projection, rotate-half, a window that keeps the first tokens),
``mixer`` (its sizes and constants) and ``mlp`` (``kind`` "dense" or "moe", or null for
none).  Every size and constant a model of the design can vary is read from there; what
has a natural "off" may be absent (no rotation, no stretching of its frequencies, no
convolution, no kept first tokens, no value mixing, no identity experts, no groups, no
shared expert, no feed-forward).  A key of the wrong JSON type, an unknown layer type or
feed-forward kind, or sizes that do not fit are refused with the place named.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .mapovik_config import _object
from .model_config import ConfigError, _Reader

ARCHITECTURE = "Fudulix"
ATTENTION, ATTENTION_2 = "attention", "attention_2"
DENSE, MOE = "dense", "moe"


@dataclass(frozen=True)
class FudulixRotation:
    dims: int
    base: float
    # None, or the stretching's constants in the order the spec of the rotation takes them:
    # attention: (factor, low, high, original); attention_2: (factor, original, fast, slow)
    scaling: Optional[Tuple[float, ...]] = None


@dataclass(frozen=True)
class FudulixMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int               # mask.size: a query sees itself and the window - 1 before it; 0: all
    keep_first: int = 0       # attention_2: the first tokens stay visible
    conv: int = 0             # attention_2: taps of the convolutions after the projections
    v_mix: bool = False
    rot: Optional[FudulixRotation] = None


@dataclass(frozen=True)
class FudulixMlp:
    kind: str
    ff: int                   # dense: inner width; moe: an expert's inner width
    experts: int = 0
    top: int = 0
    identity: int = 0         # router outputs beyond the experts that return their input
    group_count: int = 0      # 0: no groups
    group_keep: int = 0
    shared_ff: int = 0        # 0: no shared expert


@dataclass(frozen=True)
class FudulixLayer:
    type: str
    mixer: FudulixMixer
    mlp: Optional[FudulixMlp] = None


@dataclass(frozen=True)
class FudulixConfig:
    vocab: int
    width: int
    norm_eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: Tuple[FudulixLayer, ...]
    torch_dtype: str = "bfloat16"
    architecture: str = ARCHITECTURE
    eos_token_ids: tuple = ()

    ARCHITECTURE = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_json(cls, obj: Mapping[str, Any], where: str = "config.json") -> "FudulixConfig":
        r = _Reader(obj, where)
        name = r.string("architecture")
        if name != ARCHITECTURE:
            raise ConfigError(f"{where}: architecture {name!r} is not {ARCHITECTURE!r}")
        norm = _Reader(_object(obj, "norm", where), f"{where}: norm")
        emb = _object(obj, "embedding", where)
        big = _Reader(_object(emb, "bigram", f"{where}: embedding"), f"{where}: embedding.bigram")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = tuple(_layer(lo, f"{where}: layers[{i}]") for i, lo in enumerate(raw_layers))
        cfg = cls(vocab=r.integer("vocab"), width=r.integer("width"), norm_eps=norm.number("eps"),
                  buckets=big.integer("buckets"), mul_prev=big.integer("mul_prev"),
                  mul_cur=big.integer("mul_cur"), layers=layers,
                  torch_dtype=r.string("torch_dtype", "bfloat16"))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        def need(ok, msg):
            if not ok:
                raise ConfigError(f"{where}: {msg}")

        need(self.vocab > 0 and self.width > 0, "'vocab' and 'width' must be positive")
        need(self.norm_eps > 0, "'norm.eps' must be positive")
        need(self.buckets > 0 and self.mul_prev >= 0 and self.mul_cur >= 0,
             f"embedding.bigram: {self.buckets} buckets, factors {self.mul_prev} and "
             f"{self.mul_cur}")
        # the hash is formed in 64-bit integers
        need(max(self.mul_prev, self.mul_cur) * max(self.vocab, 1) < (1 << 61),
             "embedding.bigram: the factors times the vocabulary overflow the hash")
        mixed = None
        for i, layer in enumerate(self.layers):
            m, at = layer.mixer, f"layers[{i}].mixer"
            need(min(m.heads, m.kv_heads, m.dim, m.vdim) > 0 and m.heads % m.kv_heads == 0,
                 f"{at}: {m.heads} heads of {m.dim} / {m.vdim} over {m.kv_heads} key/value heads")
            need(m.window >= 0, f"{at}.mask: size {m.window} must not be negative")
            need(m.keep_first >= 0 and m.conv >= 0, f"{at}: keep_first {m.keep_first}, conv {m.conv}")
            if m.rot is not None:
                need(0 <= m.rot.dims <= m.dim and m.rot.dims % 2 == 0 and m.rot.base > 0,
                     f"{at}.rot: {m.rot.dims} rotated entries of {m.dim}, base {m.rot.base}")
                if m.rot.scaling is not None:
                    need(m.rot.scaling[0] > 0, f"{at}.rot.scaling: factor {m.rot.scaling[0]}")
                    if layer.type == ATTENTION:
                        need(m.rot.scaling[2] != m.rot.scaling[1],
                             f"{at}.rot.scaling: 'high' equals 'low'")
                    else:
                        need(m.rot.base != 1.0 and min(m.rot.scaling[1:]) > 0,
                             f"{at}.rot.scaling: original, fast and slow must be positive")
            if m.v_mix:
                if mixed is None:
                    mixed = (i, m.kv_heads * m.vdim)
                else:
                    need(m.kv_heads * m.vdim == mixed[1],
                         f"{at}: {m.kv_heads * m.vdim} value entries a token cannot be mixed "
                         f"with the {mixed[1]} of layer {mixed[0]}")
            f = layer.mlp
            if f is not None:
                need(f.ff > 0, f"layers[{i}].mlp: inner width {f.ff}")
                if f.kind == MOE:
                    outs = f.experts + f.identity
                    need(f.experts >= 0 and f.identity >= 0 and 0 < f.top <= outs,
                         f"layers[{i}].mlp.router: {f.top} of {f.experts} experts and "
                         f"{f.identity} identity experts")
                    if f.group_count:
                        need(f.group_count > 0 and outs % f.group_count == 0
                             and 0 < f.group_keep <= f.group_count
                             and f.group_keep * (outs // f.group_count) >= f.top,
                             f"layers[{i}].mlp.router.groups: {f.group_keep} of "
                             f"{f.group_count} groups over {outs} outputs, {f.top} chosen")
                    need(f.shared_ff >= 0, f"layers[{i}].mlp.shared: inner width {f.shared_ff}")

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps},
               "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev,
                                        "mul_cur": self.mul_cur}},
               "layers": [], "torch_dtype": self.torch_dtype}
        for layer in self.layers:
            m = layer.mixer
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                     "scale": m.scale, "mask": {"size": m.window} if m.window else {},
                     "v_mix": m.v_mix}
            if layer.type == ATTENTION_2:
                if m.window:
                    mixer["mask"]["keep_first"] = m.keep_first
                mixer["conv"] = m.conv
            if m.rot is not None:
                rot = {"dims": m.rot.dims, "base": m.rot.base}
                if m.rot.scaling is not None:
                    keys = (("factor", "low", "high", "original") if layer.type == ATTENTION
                            else ("factor", "original", "fast", "slow"))
                    rot["scaling"] = dict(zip(keys, m.rot.scaling))
                mixer["rot"] = rot
            mlp = None
            if layer.mlp is not None:
                f = layer.mlp
                if f.kind == DENSE:
                    mlp = {"kind": DENSE, "ff": f.ff}
                else:
                    router = {"experts": f.experts, "top": f.top, "identity": f.identity}
                    if f.group_count:
                        router["groups"] = {"count": f.group_count, "keep": f.group_keep}
                    mlp = {"kind": MOE, "expert": {"ff": f.ff}, "router": router}
                    if f.shared_ff:
                        mlp["shared"] = {"ff": f.shared_ff}
            out["layers"].append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        return out


def _rotation(obj, kind, where) -> Optional[FudulixRotation]:
    if obj.get("rot") is None:
        return None
    rot = _Reader(_object(obj, "rot", where), f"{where}.rot")
    scaling = None
    if rot.obj.get("scaling") is not None:
        sc = _Reader(_object(rot.obj, "scaling", f"{where}.rot"), f"{where}.rot.scaling")
        keys = (("factor", "low", "high", "original") if kind == ATTENTION
                else ("factor", "original", "fast", "slow"))
        scaling = tuple(sc.number(k) for k in keys)
    return FudulixRotation(dims=rot.integer("dims"), base=rot.number("base"), scaling=scaling)


def _layer(obj, where) -> FudulixLayer:
    if not isinstance(obj, Mapping):
        raise ConfigError(f"{where}: must be an object")
    kind = _Reader(obj, where).string("type")
    if kind not in (ATTENTION, ATTENTION_2):
        # an unknown kind of layer is refused, never run as another
        raise ConfigError(f"{where}: unknown layer type {kind!r} "
                          f"(known: {ATTENTION!r}, {ATTENTION_2!r})")
    at = f"{where}.mixer"
    m = _Reader(_object(obj, "mixer", where), at)
    mask = _Reader(_object(m.obj, "mask", at, default={}), f"{at}.mask")
    heads, dim = m.integer("heads"), m.integer("dim")
    second = kind == ATTENTION_2
    mixer = FudulixMixer(
        heads=heads, kv_heads=m.integer("kv_heads", heads), dim=dim, vdim=m.integer("vdim", dim),
        scale=m.number("scale"), window=mask.integer("size", 0),
        keep_first=mask.integer("keep_first", 0) if second else 0,
        conv=m.integer("conv", 0) if second else 0, v_mix=m.boolean("v_mix", False),
        rot=_rotation(m.obj, kind, at))
    mlp = None
    if obj.get("mlp") is not None:
        f = _Reader(_object(obj, "mlp", where), f"{where}.mlp")
        fk = f.string("kind")
        if fk == DENSE:
            mlp = FudulixMlp(kind=DENSE, ff=f.integer("ff"))
        elif fk == MOE:
            ex = _Reader(_object(f.obj, "expert", f"{where}.mlp"), f"{where}.mlp.expert")
            ro = _Reader(_object(f.obj, "router", f"{where}.mlp"), f"{where}.mlp.router")
            count = keep = 0
            if ro.obj.get("groups") is not None:
                gr = _Reader(_object(ro.obj, "groups", f"{where}.mlp.router"),
                             f"{where}.mlp.router.groups")
                count, keep = gr.integer("count"), gr.integer("keep")
            shared = 0
            if f.obj.get("shared") is not None:
                shared = _Reader(_object(f.obj, "shared", f"{where}.mlp"),
                                 f"{where}.mlp.shared").integer("ff")
            mlp = FudulixMlp(kind=MOE, ff=ex.integer("ff"), experts=ro.integer("experts"),
                             top=ro.integer("top"), identity=ro.integer("identity", 0),
                             group_count=count, group_keep=keep, shared_ff=shared)
        else:
            raise ConfigError(f"{where}.mlp: unknown kind {fk!r} (known: {DENSE!r}, {MOE!r})")
    return FudulixLayer(type=kind, mixer=mixer, mlp=mlp)
