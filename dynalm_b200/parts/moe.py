"""Mixture-of-experts feed-forward: the "routed_mlp" kind.

Every token uses `top` of `experts` small ungated feed-forward layers, expert j being down_j(act(up_j x)) without
biases. The router's logits z = W_router x are float32; scores are their softmax over ALL experts. Experts form `groups`
equal groups of neighbours, a group's score is its largest score, and only experts of the `keep_groups` best groups can
be chosen; of those the `top` with the largest scores are. Their weights are their scores divided by their sum (+ 1e-20),
times `weight_scale`, and the result is the weighted sum of the chosen experts' outputs.

On the device: the router product, `moe_route` (one thread a token), `moe_group` (the step's (token, expert) pairs put
in the order of their experts, with the list of row tiles), the two products over those tiles with the matrix of each
tile's expert (`moe_linear`: the activation sits in the first one's epilogue, the second leaves float32), and
`moe_combine`. Nothing comes back to the host, so the launches depend on the number of rows alone.

Parameters: inner, experts, top, groups, keep_groups, weight_scale, activation ("relu2"). Tensors: router [experts,
width], up<j> [inner, width], down<j> [width, inner].
"""

from __future__ import annotations

from typing import Dict

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from .base import TensorDecl, register_feed_forward


@register_feed_forward("routed_mlp")
class RoutedMLP:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        out = {"router": TensorDecl((spec.experts, spec.width))}
        for j in range(spec.experts):
            out[f"up{j}"] = TensorDecl((spec.inner, spec.width))
            out[f"down{j}"] = TensorDecl((spec.width, spec.inner))
        return out

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        E, top = int(spec.experts), int(spec.top)
        groups, keep = int(spec.get("groups", 1)), int(spec.get("keep_groups", 1))
        if spec.get("activation", "relu2") != "relu2":
            raise Unsupported(f"routed_mlp: activation '{spec.activation}' has no kernel (relu2 does)")
        if E > ops.MOE_MAX_EXPERTS or E % groups or not 0 < keep <= groups or not 0 < top <= keep * (E // groups):
            raise Unsupported(f"routed_mlp: {E} experts in {groups} groups, {keep} kept, {top} a token")
        self.spec = spec
        self.rt = runtime
        self.E, self.top, self.groups, self.keep = E, top, groups, keep
        self.scale = float(spec.get("weight_scale", 1.0))
        self.w_router = tensors["router"]
        self.w_up = torch.stack([tensors[f"up{j}"] for j in range(E)]).contiguous()         # [E, inner, width]
        self.w_down = torch.stack([tensors[f"down{j}"] for j in range(E)]).contiguous()     # [E, width, inner]

    def first_weights(self) -> torch.Tensor:
        return self.w_router

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        s, rt = self.spec, self.rt
        rows = x.shape[0]
        E, top = self.E, self.top
        pairs = rows * top
        logits = rt.buffer("moe_logits", (rows, E), torch.float32)
        linear(x, self.w_router, logits)                                  # float32 accumulation and result
        ids = rt.buffer("moe_ids", (rows, top), torch.int32)
        weights = rt.buffer("moe_weights", (rows, top), torch.float32)
        ops.moe_route(logits, top, self.groups, self.keep, self.scale, ids, weights)
        most = rt.max_tokens * top
        place_of = rt.flat(f"moe_place_of_{top}", most, torch.int32)
        pair_at = rt.flat(f"moe_pair_at_{top}", most, torch.int32)
        tiles = rt.flat(f"moe_tiles_{top}_{E}", 3 * ops.moe_max_tiles(most, E), torch.int32)
        n_tiles = rt.flat("moe_n_tiles", 1, torch.int32)
        tile_rows = ops.moe_tile_rows(pairs, E, x, (s.width, s.inner))
        ops.moe_group(ids, pairs, E, place_of, pair_at, tiles, n_tiles, tile_rows)
        max_tiles = ops.moe_max_tiles(pairs, E, tile_rows)
        act = rt.flat(f"moe_act_{top}_{s.inner}", most * s.inner, x.dtype)[:pairs * s.inner].view(pairs, s.inner)
        per_pair = rt.flat(f"moe_out_{top}_{s.width}", most * s.width, torch.float32)[:pairs * s.width].view(pairs, s.width)
        if tile_rows == ops.MOE_WIDE_TILE_ROWS and ops.moe_linear_tcgen05_applies(x, self.w_up, act) \
                and ops.moe_linear_tcgen05_applies(act, self.w_down, per_pair):
            # a long step: the rows once in the order of their experts, then both products on the tcgen05 tensor cores
            sorted_rows = rt.flat(f"moe_rows_{top}_{s.width}", most * s.width, x.dtype)[:pairs * s.width].view(pairs, s.width)
            ops.moe_gather(x, pair_at, top, sorted_rows)
            ops.moe_linear_tcgen05(sorted_rows, self.w_up, act, tiles, n_tiles, max_tiles, "relu2")
            ops.moe_linear_tcgen05(act, self.w_down, per_pair, tiles, n_tiles, max_tiles, "none")
        else:
            ops.moe_linear(x, pair_at, top, self.w_up, act, tiles, n_tiles, max_tiles, "relu2", tile_rows)
            ops.moe_linear(act, None, 1, self.w_down, per_pair, tiles, n_tiles, max_tiles, "none", tile_rows)
        y = rt.buffer("ffn_out", (rows, s.width))
        ops.moe_combine(per_pair, place_of, weights, top, y)
        return y
