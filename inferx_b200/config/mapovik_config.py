"""Typed configuration of the Mapovik design, read from its own ``config.json``.

Top level: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (the
factor on every sublayer's output), ``logit_scale``, ``layers`` (one object per layer:
``type`` is "parallel" - softmax attention and a state-space mixer side by side - or
"channel_delta" - a delta rule with a decay per key channel -, ``mixer`` holds the sizes and
constants, ``mlp`` the feed-forward: ``kind`` "dense", "moe", or null for none) and
``loop`` (``start``, ``stop``, ``times``: layers start..stop-1 run ``times`` times in a row).
Every size and constant a model of the design can vary is read from there; what has a
natural "off" may be absent (no loop, no rotation, no scaling of the rotation's
frequencies, no feed-forward).  The inner sizes of the delta rule's two low-rank products
are not keys of the design: the checkpoint's tensors give them; ``mixer.rank`` and
``mixer.gate_rank`` are read only so that a folder of random weights can be written from a
configuration alone.  A key of the wrong JSON type, an unknown layer type or feed-forward
kind, or sizes that do not fit are refused with the place named.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, _Reader

ARCHITECTURE = "Mapovik"
PARALLEL, CHANNEL_DELTA = "parallel", "channel_delta"
DENSE, MOE = "dense", "moe"


@dataclass(frozen=True)
class MapovikAttention:
    heads: int
    kv_heads: int
    dim: int                  # query / key entries per head
    vdim: int                 # value entries per head
    scale: float              # factor on q . k
    rot_dims: int = 0         # leading entries of each head that are rotated; 0: none
    rot_base: float = 10000.0
    rot_factor: float = 1.0   # every frequency is divided by this


@dataclass(frozen=True)
class MapovikStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class MapovikDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    rank: int = 0             # inner size of the decay's low-rank product; 0: the checkpoint's
    gate_rank: int = 0        # inner size of the gate's low-rank product; 0: the checkpoint's


@dataclass(frozen=True)
class MapovikMlp:
    kind: str
    ff: int                   # dense: inner width; moe: an expert's inner width
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class MapovikLayer:
    type: str
    left: Optional[MapovikAttention] = None      # parallel
    right: Optional[MapovikStateSpace] = None    # parallel
    delta: Optional[MapovikDelta] = None         # channel_delta
    mlp: Optional[MapovikMlp] = None


@dataclass(frozen=True)
class MapovikConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    layers: Tuple[MapovikLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1       # 1 with start == stop: no loop
    torch_dtype: str = "bfloat16"
    architecture: str = ARCHITECTURE
    eos_token_ids: tuple = ()

    ARCHITECTURE = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    @classmethod
    def from_json(cls, obj: Mapping[str, Any], where: str = "config.json") -> "MapovikConfig":
        r = _Reader(obj, where)
        name = r.string("architecture")
        if name != ARCHITECTURE:
            raise ConfigError(f"{where}: architecture {name!r} is not {ARCHITECTURE!r}")
        norm = _Reader(_object(obj, "norm", where), f"{where}: norm")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = tuple(_layer(lo, f"{where}: layers[{i}]") for i, lo in enumerate(raw_layers))
        start = stop = 0
        times = 1
        if obj.get("loop") is not None:
            lp = _Reader(_object(obj, "loop", where), f"{where}: loop")
            start, stop, times = lp.integer("start"), lp.integer("stop"), lp.integer("times")
        cfg = cls(vocab=r.integer("vocab"), width=r.integer("width"), norm_eps=norm.number("eps"),
                  residual_mult=r.number("residual_mult", 1.0),
                  logit_scale=r.number("logit_scale", 1.0), layers=layers, loop_start=start,
                  loop_stop=stop, loop_times=times,
                  torch_dtype=r.string("torch_dtype", "bfloat16"))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        def need(ok, msg):
            if not ok:
                raise ConfigError(f"{where}: {msg}")

        need(self.vocab > 0 and self.width > 0, "'vocab' and 'width' must be positive")
        need(self.norm_eps > 0, "'norm.eps' must be positive")
        need(0 <= self.loop_start <= self.loop_stop <= len(self.layers) and self.loop_times >= 1,
             f"'loop' {self.loop_start}..{self.loop_stop} x {self.loop_times} does not fit "
             f"{len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            at = f"layers[{i}].mixer"
            if layer.type == PARALLEL:
                a, s = layer.left, layer.right
                need(min(a.heads, a.kv_heads, a.dim, a.vdim) > 0 and a.heads % a.kv_heads == 0,
                     f"{at}.left: {a.heads} heads of {a.dim} / {a.vdim} over {a.kv_heads} "
                     "key/value heads")
                need(0 <= a.rot_dims <= a.dim and a.rot_dims % 2 == 0 and a.rot_factor > 0
                     and a.rot_base > 0,
                     f"{at}.left.rot: {a.rot_dims} rotated entries of {a.dim}, base "
                     f"{a.rot_base}, factor {a.rot_factor}")
                need(min(s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups) > 0
                     and s.heads % s.groups == 0 and (s.heads * s.vdim) % s.norm_groups == 0,
                     f"{at}.right: {s.heads} heads of {s.vdim} in {s.groups} groups and "
                     f"{s.norm_groups} norm groups")
            else:
                d = layer.delta
                need(min(d.heads, d.kv_heads, d.dim, d.vdim, d.conv) > 0
                     and d.heads % d.kv_heads == 0 and d.rank >= 0 and d.gate_rank >= 0,
                     f"{at}: {d.heads} heads of {d.dim} / {d.vdim} over {d.kv_heads} "
                     "query/key heads")
            f = layer.mlp
            if f is not None:
                need(f.ff > 0, f"layers[{i}].mlp: inner width {f.ff}")
                if f.kind == MOE:
                    need(0 < f.top <= f.experts,
                         f"layers[{i}].mlp: {f.top} of {f.experts} experts")

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "logit_scale": self.logit_scale, "layers": [], "torch_dtype": self.torch_dtype}
        if self.has_loop:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop,
                           "times": self.loop_times}
        for layer in self.layers:
            if layer.type == PARALLEL:
                a, s = layer.left, layer.right
                left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
                        "scale": a.scale}
                if a.rot_dims:
                    left["rot"] = {"dims": a.rot_dims, "base": a.rot_base}
                    if a.rot_factor != 1.0:
                        left["rot"]["scaling"] = {"factor": a.rot_factor}
                mixer = {"left": left,
                         "right": {"heads": s.heads, "vdim": s.vdim, "state": s.state,
                                   "groups": s.groups, "conv": s.conv,
                                   "norm_groups": s.norm_groups}}
            else:
                d = layer.delta
                mixer = {"heads": d.heads, "kv_heads": d.kv_heads, "dim": d.dim, "vdim": d.vdim,
                         "conv": d.conv}
                if d.rank:
                    mixer["rank"] = d.rank
                if d.gate_rank:
                    mixer["gate_rank"] = d.gate_rank
            mlp = None
            if layer.mlp is not None:
                f = layer.mlp
                if f.kind == DENSE:
                    mlp = {"kind": DENSE, "ff": f.ff}
                else:
                    mlp = {"kind": MOE, "expert": {"ff": f.ff},
                           "router": {"experts": f.experts, "top": f.top}}
            out["layers"].append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        return out


def _object(obj, key, where, default=None):
    v = obj.get(key) if isinstance(obj, Mapping) else None
    if v is None:
        if default is None:
            raise ConfigError(f"{where}: required object '{key}' is missing")
        return default
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: '{key}' must be an object, got {v!r}")
    return v


def _attention(obj, where) -> MapovikAttention:
    m = _Reader(obj, where)
    heads = m.integer("heads")
    dim = m.integer("dim")
    dims, base, factor = 0, 10000.0, 1.0
    if obj.get("rot") is not None:
        rot = _Reader(_object(obj, "rot", where), f"{where}.rot")
        dims, base = rot.integer("dims"), rot.number("base")
        if rot.obj.get("scaling") is not None:
            factor = _Reader(_object(rot.obj, "scaling", f"{where}.rot"),
                             f"{where}.rot.scaling").number("factor", 1.0)
    return MapovikAttention(heads=heads, kv_heads=m.integer("kv_heads", heads), dim=dim,
                            vdim=m.integer("vdim", dim), scale=m.number("scale"),
                            rot_dims=dims, rot_base=base, rot_factor=factor)


def _layer(obj, where) -> MapovikLayer:
    if not isinstance(obj, Mapping):
        raise ConfigError(f"{where}: must be an object")
    kind = _Reader(obj, where).string("type")
    mixer = _object(obj, "mixer", where)
    left = right = delta = None
    if kind == PARALLEL:
        left = _attention(_object(mixer, "left", f"{where}.mixer"), f"{where}.mixer.left")
        s = _Reader(_object(mixer, "right", f"{where}.mixer"), f"{where}.mixer.right")
        right = MapovikStateSpace(heads=s.integer("heads"), vdim=s.integer("vdim"),
                                  state=s.integer("state"), groups=s.integer("groups", 1),
                                  conv=s.integer("conv"), norm_groups=s.integer("norm_groups", 1))
    elif kind == CHANNEL_DELTA:
        m = _Reader(mixer, f"{where}.mixer")
        heads, dim = m.integer("heads"), m.integer("dim")
        delta = MapovikDelta(heads=heads, kv_heads=m.integer("kv_heads", heads), dim=dim,
                             vdim=m.integer("vdim", dim), conv=m.integer("conv"),
                             rank=m.integer("rank", 0), gate_rank=m.integer("gate_rank", 0))
    else:
        # an unknown kind of layer is refused, never run as another
        raise ConfigError(f"{where}: unknown layer type {kind!r} "
                          f"(known: {PARALLEL!r}, {CHANNEL_DELTA!r})")
    mlp = None
    if obj.get("mlp") is not None:
        f = _Reader(_object(obj, "mlp", where), f"{where}.mlp")
        fk = f.string("kind")
        if fk == DENSE:
            mlp = MapovikMlp(kind=DENSE, ff=f.integer("ff"))
        elif fk == MOE:
            ex = _Reader(_object(f.obj, "expert", f"{where}.mlp"), f"{where}.mlp.expert")
            ro = _Reader(_object(f.obj, "router", f"{where}.mlp"), f"{where}.mlp.router")
            mlp = MapovikMlp(kind=MOE, ff=ex.integer("ff"), experts=ro.integer("experts"),
                             top=ro.integer("top"))
        else:
            raise ConfigError(f"{where}.mlp: unknown kind {fk!r} (known: {DENSE!r}, {MOE!r})")
    return MapovikLayer(type=kind, left=left, right=right, delta=delta, mlp=mlp)
