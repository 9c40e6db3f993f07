"""How a layer arranges its parts around the residual stream.

"pre_norm" (Llama): x += s * mixer(norm1(x)); x += s * ffn(norm2(x)), s the residual scale
(dynalm/src/model/transformer.cpp:602-697). "parallel": x += mixer(norm1(x)) + ffn(norm2(x)), both
parts fed from the same x. The residual stream is float32; the sum of a part's output into it is
fused into the norm that follows, so a block leaves its last output (the parallel one: both) pending.
"post_norm": x <- norm1(a x + mixer(x)); x <- norm2(a x + ffn(x)): the sublayers read the stream itself and each
norm closes its own sum, so nothing is left pending and the stream is always a normed row.
"hyper_connections": the stream has several parts; a sublayer reads a weighted sum of them and every part becomes a
mix of all parts plus its own share of the sublayer's result.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..kernels import ops
from .base import TensorDecl, build_part, register_block, register_connection


@dataclass
class ResidualStream:
    """x: float32 [rows, width]. `pending` (compute dtype) times `pending_scale` is still to be added, and so is
    `pending2` (unscaled), the second output of an arrangement that leaves two."""

    x: torch.Tensor
    pending: Optional[torch.Tensor] = None
    pending_scale: float = 1.0
    pending2: Optional[torch.Tensor] = None
    as_input: Optional[torch.Tensor] = None      # x in the compute dtype, when the part that wrote x last also left that
    # A stream of several parts: float32 [rows, parts * width], a row's parts one after the other; x is then stale until
    # `flush` has summed them. `link` is the stream connection of the sublayer whose result is `pending`.
    streams: Optional[torch.Tensor] = None
    parts: int = 1
    link: Optional[object] = None

    def flush(self) -> torch.Tensor:
        if self.streams is not None:
            link = self.link if self.pending is not None else None
            ops.stream_sum(self.streams, self.parts, self.x, delta=self.pending, delta_scale=self.pending_scale,
                           mix=link.mix if link is not None else None, write=link.write if link is not None else None)
            self.streams, self.parts, self.link, self.pending = None, 1, None, None
            self.flush_second()
            return self.x
        if self.pending is not None:
            ops.residual_add(self.x, self.pending, self.pending_scale)
            self.pending = None
        self.flush_second()
        return self.x

    def flush_second(self) -> None:
        """Adds the second pending output now; for a consumer that takes one delta only."""
        if self.pending2 is not None:
            ops.residual_add(self.x, self.pending2, 1.0)
            self.pending2 = None


class Block:
    """What every arrangement shares: it builds the parts its spec lists (each from the registry its spec names,
    kept as attributes under the spec's names), and answers for them where the engine asks a layer as a whole:
    which cache it keeps, whether its launches may be captured in a CUDA graph or re-issued by address."""

    cache_part = "mixer"        # the name of the part whose cache_spec() is the layer's

    def __init__(self, spec, store, runtime):
        self.spec = spec
        self.rt = runtime
        self.part_names = list(spec.parts)
        for name, part_spec in spec.parts.items():
            setattr(self, name, build_part(part_spec, store, runtime))
        parts = self.parts()
        # only if every part says so of itself (a position encoding that a mixer holds included)
        inner = [getattr(p, "position", None) for p in parts]
        self.replay_safe = all(getattr(p, "replay_safe", False) for p in parts + [p for p in inner if p is not None])
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in parts)

    def parts(self):
        return [getattr(self, n) for n in self.part_names]

    def cache_spec(self):
        part = getattr(self, self.cache_part, None)
        return part.cache_spec() if part is not None and hasattr(part, "cache_spec") else None

    def step_plans(self) -> list:
        return [plan for p in self.parts() for plan in (p.step_plans() if hasattr(p, "step_plans") else [])]

    def graph_key(self, ctx) -> tuple:
        key = ()
        for p in self.parts():
            f = getattr(p, "graph_key", None)
            if f is not None:
                key += tuple(f(ctx))
        return key


@register_block("pre_norm")
class PreNormBlock(Block):
    """parts: mixer_norm, mixer, and optionally ffn_norm + ffn; parameter: residual_scale (default 1). Without a
    feed-forward the layer is x += s * mixer(norm1(x))."""

    def __init__(self, spec, store, runtime):
        super().__init__(spec, store, runtime)
        self.scale = float(spec.get("residual_scale", 1.0))
        self.has_ffn = "ffn" in spec.parts

    def forward(self, stream: ResidualStream, ctx, cache, owns_cache: bool) -> ResidualStream:
        rows, width = stream.x.shape
        stream.flush_second()                      # (an arrangement that leaves two outputs may stand in front)
        few = rows <= ops.SKINNY_FAST_ROWS         # a step bound by the stream of weights: say early what comes next
        h = self.rt.buffer("normed", (rows, width))
        if few:
            ops.stream_ahead(getattr(self.mixer, "first_weights", lambda: None)())
        self.mixer_norm.forward(stream.x, h, delta=stream.pending, delta_scale=stream.pending_scale)
        a = self.mixer.forward(h, ctx, cache, owns_cache)
        if not self.has_ffn:
            stream.pending, stream.pending_scale = a, self.scale
            stream.as_input = None
            return stream
        h = self.rt.buffer("normed", (rows, width))
        if few:
            ops.stream_ahead(getattr(self.ffn, "first_weights", lambda: None)())
        self.ffn_norm.forward(stream.x, h, delta=a, delta_scale=self.scale)
        f = self.ffn.forward(h, ctx)
        stream.pending, stream.pending_scale = f, self.scale
        stream.as_input = None
        return stream


@register_block("parallel")
class ParallelBlock(Block):
    """parts: mixer_norm, mixer, and optionally ffn_norm + ffn; x <- x + (mixer(norm1(x)) + ffn(norm2(x))), both
    norms of the same x. The two norms share their statistic (one mean of squares per row) and differ in their
    weights only, so one kernel reads the row once, adds what the layer before left pending, and writes both
    normalised rows (ops.rmsnorm_pair). Without a feed-forward the layer is x <- x + mixer(norm1(x))."""

    def __init__(self, spec, store, runtime):
        super().__init__(spec, store, runtime)
        self.has_ffn = "ffn" in spec.parts
        if self.has_ffn and float(spec.ffn_norm.eps) != float(spec.mixer_norm.eps):
            from ..errors import Unsupported
            raise Unsupported("parallel block: the two norms share one statistic and so one eps")

    def forward(self, stream: ResidualStream, ctx, cache, owns_cache: bool) -> ResidualStream:
        rows, width = stream.x.shape
        if stream.pending is not None and stream.pending_scale != 1.0:
            stream.flush()
        h1 = self.rt.buffer("normed", (rows, width))
        h2 = self.rt.buffer("normed_ffn", (rows, width)) if self.has_ffn else None
        self.mixer_norm.forward_pair(stream.x, h1, self.ffn_norm if self.has_ffn else None, h2,
                                     delta_a=stream.pending, delta_b=stream.pending2)
        a = self.mixer.forward(h1, ctx, cache, owns_cache)
        f = self.ffn.forward(h2, ctx) if self.has_ffn else None
        stream.pending, stream.pending_scale, stream.pending2 = a, 1.0, f
        stream.as_input = None
        return stream


@register_block("post_norm")
class PostNormBlock(Block):
    """parts: mixer, mixer_norm, and optionally ffn + ffn_norm, the norms of a kind that closes a sum ("rms_after_sum":
    they carry the weight alpha of the stream and the per-channel scale of the sublayer's result). x <-
    mixer_norm(alpha x + mixer(x)), then x <- ffn_norm(alpha x + ffn(x)). A sublayer's matrix products read x in the
    compute dtype; the norm kernel writes that copy beside the float32 stream (on the 32-bit path the stream itself is
    read), and the first layer of a model makes it from the embedding."""

    def __init__(self, spec, store, runtime):
        super().__init__(spec, store, runtime)
        self.has_ffn = "ffn" in spec.parts

    def forward(self, stream: ResidualStream, ctx, cache, owns_cache: bool) -> ResidualStream:
        rows, width = stream.x.shape
        stream.flush()                             # (an arrangement that leaves its outputs pending may stand in front)
        narrow = self.rt.dtype != torch.float32
        h = stream.as_input
        if not narrow:
            h = stream.x
        elif h is None:
            h = self.rt.buffer("stream_copy", (rows, width))
            ops.cast_rows(stream.x, h)
        a = self.mixer.forward(h, ctx, cache, owns_cache)
        if narrow:
            h = self.rt.buffer("stream_copy", (rows, width))
        self.mixer_norm.forward(stream.x, h if narrow else None, a)
        if self.has_ffn:
            f = self.ffn.forward(h, ctx)
            self.ffn_norm.forward(stream.x, h if narrow else None, f)
        stream.as_input = h if narrow else None
        return stream


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """parts: mixer_norm, mixer, mixer_post_norm, and optionally ffn_norm, ffn, ffn_post_norm: a norm in front of
    every sublayer and one behind it, before its result joins the stream: x <- x + post1(mixer(pre1(x))), then x <- x +
    post2(ffn(pre2(x))). The norm behind the mixer, the sum and the norm in front of the feed-forward are one kernel
    (ops.norm_add_norm), which keeps the row in shared memory between the two; the stream is float32 and nothing is
    left pending."""

    def __init__(self, spec, store, runtime):
        super().__init__(spec, store, runtime)
        self.has_ffn = "ffn" in spec.parts

    def forward(self, stream: ResidualStream, ctx, cache, owns_cache: bool) -> ResidualStream:
        rows, width = stream.x.shape
        stream.flush_second()                      # (an arrangement that leaves its outputs pending may stand in front)
        h = self.rt.buffer("normed", (rows, width))
        self.mixer_norm.forward(stream.x, h, delta=stream.pending, delta_scale=stream.pending_scale)
        stream.pending = None
        a = self.mixer.forward(h, ctx, cache, owns_cache)
        post = self.mixer_post_norm
        if self.has_ffn:
            h = self.rt.buffer("normed", (rows, width))
            ops.norm_add_norm(stream.x, a, post.weight, post.eps, self.ffn_norm.weight, self.ffn_norm.eps, h)
            f = self.ffn.forward(h, ctx)
            post = self.ffn_post_norm
            ops.norm_add_norm(stream.x, f, post.weight, post.eps)
        else:
            ops.norm_add_norm(stream.x, a, post.weight, post.eps)
        stream.pending_scale = 1.0
        stream.as_input = None
        return stream


@register_connection("hyper")
class HyperConnection:
    """The weights with which one sublayer sits on a stream of n parts: it reads sum_s read[s] x_s, and its result y
    changes every part at once, x_t <- sum_s mix[s, t] x_s + write[t] * y (mix is indexed [from, to]). Tensors: in [n],
    out [n], mix [n, n]; float32."""

    replay_safe = True     # it launches nothing itself
    graph_safe = True

    @staticmethod
    def declare(spec):
        n = spec.streams
        return {"in": TensorDecl((n,), role="vector", init="around_one"),
                "out": TensorDecl((n,), role="vector", init="around_one"),
                "mix": TensorDecl((n, n), role="vector", init="near_identity")}

    def __init__(self, spec, tensors, runtime):
        self.spec = spec
        self.read = tensors["in"].contiguous()
        self.write = tensors["out"].contiguous()
        self.mix = tensors["mix"].contiguous()


@register_block("hyper_connections")
class HyperConnectionBlock(Block):
    """parts: mixer_norm, mixer, mixer_link, and optionally ffn_norm, ffn, ffn_link; parameter: streams (n). The stream
    is n parts, all equal to the embedding at the start; for each sublayer u = sum_s read[s] x_s, y = sublayer(norm(u)),
    x_t <- sum_s mix[s, t] x_s + write[t] y. The update a sublayer leaves is applied by the norm kernel of the sublayer
    that follows (in this layer or the next), which reads a row's parts once, writes them back and norms their weighted
    sum; the model's final norm reads the plain sum of the parts the same way. The norms are of a kind that reads such a
    stream (`forward_stream`; "layer")."""

    def __init__(self, spec, store, runtime):
        super().__init__(spec, store, runtime)
        self.has_ffn = "ffn" in spec.parts
        self.n = int(spec.streams)
        if not 0 < self.n <= ops.STREAM_MAX_PARTS:
            from ..errors import Unsupported
            raise Unsupported(f"hyper_connections: {self.n} streams ({ops.STREAM_MAX_PARTS} at most)")

    def last_link(self):
        """The stream connection of the sublayer whose result this layer leaves pending."""
        return self.ffn_link if self.has_ffn else self.mixer_link

    def entry_tensors(self, stream: ResidualStream) -> list:
        """The tensors of the layer in front that this layer's first norm reads (engine/launch_memo.py)."""
        link = stream.link if stream.streams is not None and stream.pending is not None else None
        return [link.mix, link.write] if link is not None else []

    def forward(self, stream: ResidualStream, ctx, cache, owns_cache: bool) -> ResidualStream:
        rows, width = stream.x.shape
        rt, n = self.rt, self.n
        init = None
        if stream.streams is None:                 # the first layer of its kind: every part starts as the stream so far
            init = stream.flush()
            stream.streams = rt.buffer("residual_parts", (rows, n * width), torch.float32)
            stream.parts = n
        elif stream.parts != n:
            from ..errors import Unsupported
            raise Unsupported("hyper_connections: layers of one model share the number of streams")
        h = rt.buffer("normed", (rows, width))
        self.mixer_norm.forward_stream(stream.streams, n, h, init=init, delta=stream.pending, link=stream.link,
                                       read=self.mixer_link.read)
        a = self.mixer.forward(h, ctx, cache, owns_cache)
        stream.pending, stream.pending_scale, stream.link = a, 1.0, self.mixer_link
        if self.has_ffn:
            h = rt.buffer("normed", (rows, width))
            self.ffn_norm.forward_stream(stream.streams, n, h, delta=a, link=self.mixer_link, read=self.ffn_link.read)
            f = self.ffn.forward(h, ctx)
            stream.pending, stream.link = f, self.ffn_link
        stream.as_input = None
        return stream
