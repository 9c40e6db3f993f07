"""The Rodelorn configuration: config.json -> RodelornConfig.

A Rodelorn config.json lists its layers one by one. A layer's mixer is a gated delta rule (`type` "delta"; further
instances of it with sizes of their own are numbered, "delta_2") or two mixers side by side that read the same input
("parallel": windowed attention on the left, a gated linear recurrence on the right), followed by a gated dense
feed-forward or none:

    {"architecture": "Rodelorn", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "logit_scale": c, "logit_softcap": t,
     "layers": [{"type": "delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"},
                 "mlp": {"kind": "dense", "ff": F} or null},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                                    "rot": {"base", "dims", "scaling": {"factor"}}},
                           "right": {"width", "blocks", "conv"}, "left_scale", "right_scale"}, ...}]}

Where a key may be left out its mechanism is switched off (no window without `mask`, no rotation without `rot`, no
stretching of the positions without `scaling`, no cap without `logit_softcap`, scales of 1); no default stands for a
model's value.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import InvalidArgument, NotFound, Unsupported
from .reader import KeyReader

DEFAULT_CONTEXT = 131072      # the design has no positional limit; block tables are sized for this unless told otherwise


@dataclass(frozen=True)
class RodelornDelta:
    heads: int                   # value heads, each with a matrix state dim x vdim
    kv_heads: int                # query/key heads, each shared by heads / kv_heads value heads
    dim: int
    vdim: int
    conv: int                    # taps of the short convolutions


@dataclass(frozen=True)
class RodelornAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                  # 0: all earlier keys
    rot_dims: int                # how many of a head's first numbers are turned (0: none)
    rot_base: float
    rot_factor: float            # every frequency is divided by it


@dataclass(frozen=True)
class RodelornRecurrence:
    width: int
    blocks: int                  # equal parts of the channels, each with square gate matrices of its own
    conv: int


@dataclass(frozen=True)
class RodelornPair:
    left: Union[RodelornAttention, RodelornRecurrence]
    right: Union[RodelornAttention, RodelornRecurrence]
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class RodelornMLP:
    kind: str
    ff: int


@dataclass(frozen=True)
class RodelornLayer:
    type: str
    mixer: Union[RodelornDelta, RodelornPair]
    mlp: Optional[RodelornMLP]


def _positive(where: str, **sizes: int) -> None:
    for name, value in sizes.items():
        if value <= 0:
            raise InvalidArgument(f"{where}: '{name}' must be positive")


def _read_delta(mr: KeyReader) -> RodelornDelta:
    heads, dim = mr.int("heads"), mr.int("dim")
    m = RodelornDelta(heads, mr.int_or("kv_heads", heads), dim, mr.int_or("vdim", dim), mr.int("conv"))
    _positive(mr.where, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, conv=m.conv)
    if m.heads % m.kv_heads:
        raise InvalidArgument(f"{mr.where}: {m.heads} heads do not divide into {m.kv_heads} query/key heads")
    return m


def _read_attention(mr: KeyReader) -> RodelornAttention:
    heads, dim = mr.int("heads"), mr.int("dim")
    mask, rot = mr.object_or_none("mask"), mr.object_or_none("rot")
    scaling = rot.object_or_none("scaling") if rot is not None else None
    m = RodelornAttention(heads, mr.int_or("kv_heads", heads), dim, mr.int_or("vdim", dim),
                          mr.float_or("scale", dim ** -0.5), mask.int_or("size", 0) if mask is not None else 0,
                          rot.int_or("dims", dim) if rot is not None else 0,
                          rot.float_or("base", 10000.0) if rot is not None else 10000.0,
                          scaling.float_or("factor", 1.0) if scaling is not None else 1.0)
    _positive(mr.where, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim)
    if m.heads % m.kv_heads:
        raise InvalidArgument(f"{mr.where}: {m.heads} heads do not divide into {m.kv_heads} key/value heads")
    if m.window < 0:
        raise InvalidArgument(f"{mr.where}: mask.size must not be negative")
    if m.rot_dims < 0 or m.rot_dims > m.dim or m.rot_dims % 2:
        raise InvalidArgument(f"{mr.where}: rot.dims {m.rot_dims} must be even and at most dim {m.dim}")
    if not m.rot_factor > 0 or not m.rot_base > 0:
        raise InvalidArgument(f"{mr.where}: rot.base and rot.scaling.factor must be positive")
    return m


def _read_recurrence(mr: KeyReader) -> RodelornRecurrence:
    m = RodelornRecurrence(mr.int("width"), mr.int_or("blocks", 1), mr.int("conv"))
    _positive(mr.where, width=m.width, blocks=m.blocks, conv=m.conv)
    if m.width % m.blocks:
        raise InvalidArgument(f"{mr.where}: {m.width} channels do not divide into {m.blocks} blocks")
    return m


def _read_side(mr: Optional[KeyReader], where: str):
    """One side of a pair: a gated linear recurrence when it gives `blocks` or `width`, else attention."""
    if mr is None:
        raise NotFound(f"{where} is missing")
    if mr.has("width") or mr.has("blocks"):
        return _read_recurrence(mr)
    return _read_attention(mr)


@dataclass(frozen=True)
class RodelornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float         # 0: no cap
    layers: Tuple[RodelornLayer, ...]
    context: int = DEFAULT_CONTEXT

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.context

    @classmethod
    def from_dict(cls, obj: Mapping[str, Any]) -> "RodelornConfig":
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
            base = re.sub(r"_\d+$", "", kind or "")          # "delta_2": another instance of "delta"
            if base == "delta":
                mixer = _read_delta(mr)
            elif base == "parallel":
                mixer = RodelornPair(_read_side(mr.object_or_none("left"), f"{mr.where}: left"),
                                     _read_side(mr.object_or_none("right"), f"{mr.where}: right"),
                                     mr.float_or("left_scale", 1.0), mr.float_or("right_scale", 1.0))
            else:
                raise Unsupported(f"config.json: layers[{i}] has a mixer of type '{kind}'; this design has 'delta' "
                                  f"and 'parallel' (and numbered instances of them)")
            mlp = None
            pr = lr.object_or_none("mlp")
            if pr is not None:
                mlp = RodelornMLP(pr.str_or("kind", "dense"), pr.int("ff"))
                if mlp.kind != "dense":
                    raise Unsupported(f"config.json: layers[{i}] has a feed-forward of kind '{mlp.kind}'; this design has 'dense'")
                _positive(f"config.json: layers[{i}]: mlp", ff=mlp.ff)
            layers.append(RodelornLayer(base, mixer, mlp))
        softcap = top.float_or("logit_softcap", 0.0)
        if softcap < 0:
            raise InvalidArgument("config.json: logit_softcap must not be negative")
        return cls(vocab, width, norm.float_or("eps", 1e-6) if norm is not None else 1e-6,
                   emb.float_or("scale", 1.0) if emb is not None else 1.0, top.float_or("logit_scale", 1.0), softcap,
                   tuple(layers), top.int_or("context", DEFAULT_CONTEXT))
