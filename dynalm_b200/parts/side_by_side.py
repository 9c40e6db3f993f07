"""Two mixers side by side: the "side_by_side" mixer.

Both read the same input; the result is left_scale * left(h) + right_scale * right(h), summed in float32. The two are
mixers in their own right, given as MixerSpecs in the parameters `left` and `right`; their tensors are declared under
"left.<name>" and "right.<name>". One of them may keep pages and the other a state row (attention beside a
recurrence): the pair then asks for pages that carry a state row (CacheSpec.state_shape on a spec of kind "pages"), and
hands each side its own share.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import ops
from .base import MIXERS, CacheSpec, TensorDecl, register_mixer

SIDES = ("left", "right")


@register_mixer("side_by_side")
class SideBySideMixer:
    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        out = {}
        for side in SIDES:
            sub = getattr(spec, side)
            for local, decl in MIXERS.get(sub.kind).declare(sub).items():
                out[f"{side}.{local}"] = decl
        return out

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        self.spec = spec
        self.rt = runtime
        for side in SIDES:
            sub = getattr(spec, side)
            own = {k[len(side) + 1:]: v for k, v in tensors.items() if k.startswith(side + ".")}
            part = MIXERS.get(sub.kind)(sub, own, runtime)
            if not hasattr(part, "out_name"):
                raise Unsupported(f"side_by_side: a mixer of kind '{sub.kind}' cannot name the buffer of its result")
            part.out_name = f"mixer_out_{side}"             # the two results live side by side until they are summed
            setattr(self, side, part)
        self.left_scale = float(spec.get("left_scale", 1.0))
        self.right_scale = float(spec.get("right_scale", 1.0))
        self.replay_safe = all(getattr(getattr(self, s), "replay_safe", False) for s in SIDES)
        self.graph_safe = all(getattr(getattr(self, s), "graph_safe", False) for s in SIDES)
        specs = [getattr(self, s).cache_spec() for s in SIDES]
        kinds = [c.kind for c in specs if c is not None]
        if len(kinds) != len(set(kinds)):
            raise Unsupported("side_by_side: two mixers that both keep pages, or both a state row, have no cache to share")
        self._kinds = [c.kind if c is not None else None for c in specs]

    def first_weights(self):
        f = getattr(self.left, "first_weights", None)
        return f() if f is not None else None

    def step_plans(self) -> list:
        return [p for s in SIDES for p in (getattr(self, s).step_plans() if hasattr(getattr(self, s), "step_plans") else [])]

    def graph_key(self, ctx) -> tuple:
        key = ()
        for s in SIDES:
            f = getattr(getattr(self, s), "graph_key", None)
            if f is not None:
                key += tuple(f(ctx))
        return key

    def cache_spec(self) -> Optional[CacheSpec]:
        specs = {c.kind: c for c in (getattr(self, s).cache_spec() for s in SIDES) if c is not None}
        pages, state = specs.get("pages"), specs.get("state")
        if pages is None or state is None:
            return pages or state
        return CacheSpec(kind="pages", entry_shape=pages.entry_shape, tensors=pages.tensors, window=pages.window,
                         state_shape=state.state_shape, dtype=pages.dtype, state_dtype=state.dtype)

    @staticmethod
    def _share(cache, kind: Optional[str]):
        """The part of the pair's cache that a side of this kind owns."""
        if kind is None or cache is None:
            return None
        if kind == "state" and cache.kind == "pages":
            return cache.state                              # the state row that the pair's pages carry
        return cache

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        a = self.left.forward(x, ctx, self._share(cache, self._kinds[0]), owns_cache)
        b = self.right.forward(x, ctx, self._share(cache, self._kinds[1]), owns_cache)
        out = self.rt.buffer("pair_out", (x.shape[0], self.spec.width), torch.float32)
        ops.scaled_sum(a, self.left_scale, b, self.right_scale, out)
        return out
