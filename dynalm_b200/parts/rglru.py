"""A recurrent block around a real-gated linear recurrent unit: the "rglru" mixer.

Two branches of `inner` channels leave the layer's input: a gate branch y = gelu_tanh(W_y h + b_y) and a recurrent
branch u = conv(W_x h + b_x), a causal convolution over the last `taps` tokens per channel with a bias and no
activation. The channels are cut into `blocks` equal parts, each with two square matrices of its own:

    r = sigmoid(Wa[b] u_b + ba[b]),   i = sigmoid(Wi[b] u_b + bi[b])
    a = exp(-c r softplus(lam)),      S <- a S + sqrt(1 - a^2) (i * u)        (c = decay_scale, S starts at zero)

and the mixer's output is W_o (S * y). (The unit is the one of "Griffin: Mixing Gated Linear Recurrences with Local
Attention for Efficient Language Models", De et al.) Nothing is cached per token: a request keeps one row of a
float32 state array, [S | the last taps - 1 inputs of the convolution], which the cache manager hands out zeroed.
Gates, decays and the state are float32 whatever the compute dtype.

All sizes come from the spec: inner, blocks, taps, decay_scale (default 8).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import CacheSpec, TensorDecl, register_mixer


@register_mixer("rglru")
class GatedLinearRecurrence:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row and request counts only
    out_name = "mixer_out"     # the workspace buffer of the result; a mixer that holds this one may name another

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        R, B = spec.inner, spec.blocks
        nb = R // B
        return {
            "y": TensorDecl((R, spec.width)), "y_bias": TensorDecl((R,), role="vector", init="bias"),
            "x": TensorDecl((R, spec.width)), "x_bias": TensorDecl((R,), role="vector", init="bias"),
            "conv": TensorDecl((R, spec.taps), role="vector", init="bias"),
            "conv_bias": TensorDecl((R,), role="vector", init="bias"),
            "ra": TensorDecl((B, nb, nb), role="vector", init="bias"), "ra_bias": TensorDecl((B, nb), role="vector", init="bias"),
            "ri": TensorDecl((B, nb, nb), role="vector", init="bias"), "ri_bias": TensorDecl((B, nb), role="vector", init="bias"),
            "lam": TensorDecl((R,), role="vector", init="bias"),
            "o": TensorDecl((spec.width, R)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        if spec.inner % spec.blocks:
            raise Unsupported(f"rglru: {spec.inner} channels do not divide into {spec.blocks} blocks")
        self.spec = spec
        self.rt = runtime
        self.inner = spec.inner
        self.w_in = torch.cat([tensors["y"], tensors["x"]], dim=0).contiguous()        # one product: [y | x]
        self.y_bias, self.x_bias = tensors["y_bias"], tensors["x_bias"]
        self.taps = tensors["conv"].t().contiguous()                                   # [taps, channels]
        self.conv_bias = tensors["conv_bias"]
        self.wa_t = tensors["ra"].transpose(1, 2).contiguous()                          # [blocks, in, out]
        self.wi_t = tensors["ri"].transpose(1, 2).contiguous()
        self.ba, self.bi = tensors["ra_bias"].reshape(-1).contiguous(), tensors["ri_bias"].reshape(-1).contiguous()
        self.lam = tensors["lam"]
        self.w_o = tensors["o"]
        self.decay_scale = float(spec.get("decay_scale", 8.0))
        self.keep_off = self.inner                          # where a slot's kept convolution inputs begin

    def first_weights(self) -> torch.Tensor:
        return self.w_in

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(kind="state", state_shape=(self.inner * self.spec.taps,), dtype="float32")

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] in the compute dtype -> [rows, width] (or split-K partial sums of it)."""
        s, rt, R = self.spec, self.rt, self.inner
        if not owns_cache or cache is None or cache.kind != "state":
            raise Unsupported("rglru: every run of the layer keeps a state of its own")
        (state,) = cache.arrays
        rows = x.shape[0]
        proj = rt.buffer("rglru_proj", (rows, 2 * R))
        linear(x, self.w_in, proj)
        u = rt.buffer("rglru_conv", (rows, R))
        ops.short_conv(proj, R, R, self.taps, self.conv_bias, state, self.keep_off, ctx.positions, ctx.row_request,
                       ctx.row_slot, ctx.pos_start, u, act="none", in_bias=self.x_bias)
        ops.ssm_conv_keep(proj, R, R, s.taps, state, self.keep_off, ctx.q_start, ctx.state_slots, ctx.num_requests)
        a = rt.buffer("rglru_a", (rows, R), torch.float32)
        m = rt.buffer("rglru_m", (rows, R), torch.float32)
        ops.rglru_gates(u, self.wa_t, self.ba, self.wi_t, self.bi, self.lam, self.decay_scale, a, m)
        g = rt.buffer("rglru_out", (rows, R))
        ops.rglru_scan(a, m, proj, 0, self.y_bias, state, ctx.q_start, ctx.state_slots, g, ctx.num_requests)
        return linear_partial(g, self.w_o, rt, self.out_name)
