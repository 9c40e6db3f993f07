"""The gated delta rule: the "gated_delta" mixer.

One projection of the layer's input gives, per token, q and k of G heads of d numbers, v of H heads of e numbers, the
output gate (H x e), and per head a raw write strength b and a raw step size a. q, k and v pass a short causal
convolution over the last `taps` tokens (per channel, no bias) and silu; q and k are then made unit vectors per head
(q also times d^(-1/2)). Per head h (query/key head h / (H / G)), with a matrix state S (d x e) that starts at zero:

    g = exp(-exp(a_log_h) softplus(a + dt_bias_h)),   beta = sigmoid(b)
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

and the mixer's output is o_proj(o / rms(o) * norm * silu(gate)), each head normed by itself over its e numbers with
one weight vector shared by the heads. Nothing is cached per token: a request keeps one row of a float32 state array,
[S of every head | the last taps - 1 inputs of the convolutions], which the cache manager hands out zeroed.

All sizes come from the spec: num_heads (H), num_kv_heads (G), head_dim (d), value_dim (e), taps, eps.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import CacheSpec, TensorDecl, register_mixer


@register_mixer("gated_delta")
class GatedDeltaMixer:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row and request counts only
    out_name = "mixer_out"     # the workspace buffer of the result; a mixer that holds this one may name another

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        H, G, d, e, K = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim, spec.taps
        return {
            "q": TensorDecl((G * d, spec.width)), "k": TensorDecl((G * d, spec.width)), "v": TensorDecl((H * e, spec.width)),
            "q_conv": TensorDecl((G * d, K), role="vector", init="bias"),
            "k_conv": TensorDecl((G * d, K), role="vector", init="bias"),
            "v_conv": TensorDecl((H * e, K), role="vector", init="bias"),
            "b": TensorDecl((H, spec.width)), "a": TensorDecl((H, spec.width)),
            "a_log": TensorDecl((H,), role="vector", init="bias"),
            "dt_bias": TensorDecl((H,), role="vector", init="bias"),
            "norm": TensorDecl((e,), role="vector", init="around_one"),
            "gate": TensorDecl((H * e, spec.width)),
            "o": TensorDecl((spec.width, H * e)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        H, G, d, e = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        if H % G:
            raise Unsupported(f"gated_delta: {H} heads do not divide into {G} query/key heads")
        if d > 512:
            raise Unsupported(f"gated_delta: a state of {d} rows has no kernel (512 at most)")
        self.spec = spec
        self.rt = runtime
        self.qk, self.inner = G * d, H * e
        self.channels = 2 * self.qk + self.inner
        # one product: [q | k | v | gate | b | a]; the convolution runs over the first three
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "gate", "b", "a")], dim=0).contiguous()
        self.taps = torch.cat([tensors[n] for n in ("q_conv", "k_conv", "v_conv")], dim=0).t().contiguous()   # [taps, channels]
        self.a_log, self.dt_bias, self.norm = tensors["a_log"], tensors["dt_bias"], tensors["norm"]
        self.w_o = tensors["o"]
        self.eps = float(spec.eps)
        self.keep_off = H * d * e                          # where a slot's kept convolution inputs begin

    def first_weights(self) -> torch.Tensor:
        return self.w_in

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(kind="state", state_shape=(self.keep_off + (self.spec.taps - 1) * self.channels,), dtype="float32")

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] in the compute dtype -> [rows, width] (or split-K partial sums of it)."""
        s, rt = self.spec, self.rt
        if not owns_cache or cache is None or cache.kind != "state":
            raise Unsupported("gated_delta: every run of the layer keeps a state of its own")
        (state,) = cache.arrays
        rows = x.shape[0]
        H, G, d, e = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        proj = rt.buffer("delta_proj", (rows, self.w_in.shape[0]))
        linear(x, self.w_in, proj)
        u = rt.buffer("delta_conv", (rows, self.channels))
        ops.short_conv(proj, 0, self.channels, self.taps, None, state, self.keep_off, ctx.positions, ctx.row_request,
                       ctx.row_slot, ctx.pos_start, u, act="silu")
        ops.ssm_conv_keep(proj, 0, self.channels, s.taps, state, self.keep_off, ctx.q_start, ctx.state_slots,
                          ctx.num_requests)
        o = rt.buffer("delta_o", (rows, self.inner), torch.float32)
        gate_col = self.channels
        ops.delta_rule(u, 0, self.qk, 2 * self.qk, proj, gate_col + self.inner, gate_col + self.inner + H, self.a_log,
                       self.dt_bias, state, ctx.q_start, ctx.state_slots, o, ctx.num_requests, H, G, d, e)
        g = rt.buffer("delta_gated", (rows, self.inner))
        ops.head_norm_gate(o, proj, gate_col, self.norm, self.eps, g, H, e)
        return linear_partial(g, self.w_o, rt, self.out_name)
