"""The Bugapel configuration: config.json -> BugapelConfig.

A Bugapel config.json lists its layers one by one. A layer's mixer is softmax attention of one of two makes or a
gated linear attention, followed by a mixture-of-experts feed-forward or none; the residual stream may be several
streams that every sublayer reads a weighted sum of and writes back through a small mixing matrix:

    {"architecture": "Bugapel", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "streams": n, "logit_softcap": c,
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                                                 "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}}},
                 "mlp": {"kind": "moe", "expert": {"ff"},
                         "router": {"experts", "top", "scale", "groups": {"count", "keep"}}} or null},
                {"type": "attention_2", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                                                   "mask": {"size", "keep_first"}, "rot": {"base", "dims"}}, ...},
                {"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, ...}]}

"attention": no biases, rotation in the rotate-half layout, queries and keys made unit-RMS per head after the
rotation, a softmax whose denominator holds one more term of score 0. "attention_2": biases on all four projections,
rotation in the interleaved layout, a sliding window that also keeps the first tokens, an ordinary softmax.
Where a key may be left out its mechanism is switched off (no rotation without `rot`, no stretching of wavelengths
without `scaling`, no window without `mask`, one plain residual stream without `streams`, no cap without
`logit_softcap`, no groups of experts without `groups`); no default stands for a model's value.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import InvalidArgument, NotFound, Unsupported
from .reader import KeyReader

DEFAULT_CONTEXT = 131072      # the design has no positional limit; block tables are sized for this unless told otherwise


@dataclass(frozen=True)
class BugapelWavelengths:
    """Frequencies keep their value below a wavelength of original / high, are divided by `factor` above original /
    low, and pass from one to the other in between."""
    factor: float
    low: float
    high: float
    original: float

    def divisor(self, frequency: float) -> float:
        """What a frequency is divided by."""
        wavelength = 2.0 * math.pi / frequency
        if wavelength < self.original / self.high:
            return 1.0
        if wavelength > self.original / self.low:
            return self.factor
        s = (self.original / wavelength - self.low) / (self.high - self.low)
        return 1.0 / ((1.0 - s) / self.factor + s)


@dataclass(frozen=True)
class BugapelAttention:
    make: int                    # 1: "attention", 2: "attention_2"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int                # how many of a head's first numbers are turned (0: none)
    rot_base: float
    wavelengths: Optional[BugapelWavelengths]
    window: int                  # 0: all earlier keys
    keep_first: int              # keys at positions below this stay visible behind the window


@dataclass(frozen=True)
class BugapelGLA:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 0                # inner size of the decay's two-step projection; 0: read from the tensor's shape


@dataclass(frozen=True)
class BugapelMoE:
    ff: int
    experts: int
    top: int
    scale: float
    groups: int                  # 1: no groups
    keep_groups: int


@dataclass(frozen=True)
class BugapelLayer:
    type: str
    mixer: Union[BugapelAttention, BugapelGLA]
    mlp: Optional[BugapelMoE]


def _positive(where: str, **sizes) -> None:
    for name, value in sizes.items():
        if not value > 0:
            raise InvalidArgument(f"{where}: '{name}' must be positive")


def _read_attention(mr: KeyReader, make: int) -> BugapelAttention:
    heads, dim = mr.int("heads"), mr.int("dim")
    rot = mr.object_or_none("rot")
    mask = mr.object_or_none("mask") if make == 2 else None
    wavelengths = None
    if rot is not None:
        sc = rot.object_or_none("scaling")
        if sc is not None:
            wavelengths = BugapelWavelengths(sc.float_or("factor", 1.0), sc.float_or("low", 1.0), sc.float_or("high", 4.0),
                                             sc.float_or("original", 8192.0))
            _positive(sc.where, factor=wavelengths.factor, low=wavelengths.low, high=wavelengths.high,
                      original=wavelengths.original)
            if wavelengths.high <= wavelengths.low:
                raise InvalidArgument(f"{sc.where}: 'high' must exceed 'low'")
    m = BugapelAttention(make, heads, mr.int_or("kv_heads", heads), dim, mr.int_or("vdim", dim),
                         mr.float_or("scale", dim ** -0.5),
                         rot.int_or("dims", dim) if rot is not None else 0,
                         rot.float_or("base", 10000.0) if rot is not None else 10000.0, wavelengths,
                         mask.int_or("size", 0) if mask is not None else 0,
                         mask.int_or("keep_first", 0) if mask is not None else 0)
    _positive(mr.where, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, rot_base=m.rot_base)
    if m.heads % m.kv_heads:
        raise InvalidArgument(f"{mr.where}: {m.heads} heads do not divide into {m.kv_heads} key/value heads")
    if m.rot_dims < 0 or m.rot_dims > m.dim or m.rot_dims % 2:
        raise InvalidArgument(f"{mr.where}: rot.dims {m.rot_dims} must be even and at most dim {m.dim}")
    if m.window < 0 or m.keep_first < 0:
        raise InvalidArgument(f"{mr.where}: mask.size and mask.keep_first must not be negative")
    return m


def _read_gla(mr: KeyReader) -> BugapelGLA:
    heads, dim = mr.int("heads"), mr.int("dim")
    m = BugapelGLA(heads, dim, mr.int_or("vdim", dim), mr.float_or("tau", 1.0), mr.int_or("rank", 0))
    _positive(mr.where, heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau)
    return m


def _read_moe(pr: KeyReader) -> BugapelMoE:
    kind = pr.str_or("kind", "moe")
    if kind != "moe":
        raise Unsupported(f"{pr.where}: a feed-forward of kind '{kind}'; this design has 'moe'")
    expert, router = pr.object_or_none("expert"), pr.object_or_none("router")
    if expert is None or router is None:
        raise NotFound(f"{pr.where}: needs 'expert' and 'router'")
    groups = router.object_or_none("groups")
    m = BugapelMoE(expert.int("ff"), router.int("experts"), router.int("top"), router.float_or("scale", 1.0),
                   groups.int_or("count", 1) if groups is not None else 1,
                   groups.int_or("keep", 1) if groups is not None else 1)
    _positive(pr.where, ff=m.ff, experts=m.experts, top=m.top, groups=m.groups, keep=m.keep_groups)
    if m.experts % m.groups:
        raise InvalidArgument(f"{pr.where}: {m.experts} experts do not divide into {m.groups} groups")
    if m.keep_groups > m.groups:
        raise InvalidArgument(f"{pr.where}: keeps {m.keep_groups} of {m.groups} groups")
    if m.top > m.keep_groups * (m.experts // m.groups):
        raise InvalidArgument(f"{pr.where}: {m.top} experts a token cannot come from {m.keep_groups} groups of "
                              f"{m.experts // m.groups}")
    return m


@dataclass(frozen=True)
class BugapelConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    streams: int                 # 0: one plain residual stream; n > 0: n streams with mixing weights per sublayer
    logit_softcap: float         # 0: no cap
    layers: Tuple[BugapelLayer, ...]
    context: int = DEFAULT_CONTEXT

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.context

    @classmethod
    def from_dict(cls, obj: Mapping[str, Any]) -> "BugapelConfig":
        top = KeyReader(obj)
        vocab, width = top.int("vocab"), top.int("width")
        _positive("config.json", vocab=vocab, width=width)
        norm = top.object_or_none("norm")
        emb = top.object_or_none("embedding")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise NotFound("config.json: missing 'layers' (a list with one entry per layer)")
        layers = []
        for i, raw in enumerate(raw_layers):
            lr = KeyReader(raw, f"config.json: layers[{i}]")
            kind = lr.str_or("type", None)
            mr = lr.object_or_none("mixer")
            if mr is None:
                raise NotFound(f"config.json: layers[{i}] has no 'mixer'")
            if kind == "attention":
                mixer = _read_attention(mr, 1)
            elif kind == "attention_2":
                mixer = _read_attention(mr, 2)
            elif kind == "gla":
                mixer = _read_gla(mr)
            else:
                raise Unsupported(f"config.json: layers[{i}] has a mixer of type '{kind}'; this design has 'attention', "
                                  f"'attention_2' and 'gla'")
            pr = lr.object_or_none("mlp")
            layers.append(BugapelLayer(kind, mixer, _read_moe(pr) if pr is not None else None))
        softcap = top.float_or("logit_softcap", 0.0)
        streams = top.int_or("streams", 0)
        if softcap < 0 or streams < 0:
            raise InvalidArgument("config.json: logit_softcap and streams must not be negative")
        return cls(vocab, width, norm.float_or("eps", 1e-5) if norm is not None else 1e-5,
                   emb.float_or("scale", 1.0) if emb is not None else 1.0, streams, softcap, tuple(layers),
                   top.int_or("context", DEFAULT_CONTEXT))
