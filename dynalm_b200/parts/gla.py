"""Gated linear attention: the "gla" mixer.

One projection of the layer's input gives, per token, q and k of H heads of d numbers, v of H heads of e numbers, the
output gate (H x e) and the inner vector of the decay (r numbers); a second, small product takes that inner vector to
one raw decay per head and key channel, z (H x d, with a bias, float32). Per head, with a matrix state S (d x e) that
starts at zero and is carried from token to token in float32:

    alpha = sigmoid(z)^(1 / tau);   S <- diag(alpha) S + k v^T;   o = S^T (q d^(-1/2))

(the decay acts on the rows of S, which belong to key channels; the read-out comes after the write). The mixer's output
is o_proj(o / rms(o) * norm * silu(gate)), each head normed by itself over its e numbers with one weight vector shared
by the heads. Nothing is cached per token: a request keeps one row of a float32 state array, S of every head, which the
cache manager hands out zeroed.

All sizes come from the spec: num_heads (H), head_dim (d), value_dim (e), rank (r), tau, eps.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import CacheSpec, TensorDecl, register_mixer


@register_mixer("gla")
class GatedLinearAttention:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row and request counts only
    out_name = "mixer_out"     # the workspace buffer of the result; a mixer that holds this one may name another

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        H, d, e, r = spec.num_heads, spec.head_dim, spec.value_dim, spec.rank
        return {
            "q": TensorDecl((H * d, spec.width)), "k": TensorDecl((H * d, spec.width)), "v": TensorDecl((H * e, spec.width)),
            "gate": TensorDecl((H * e, spec.width)),
            "decay_in": TensorDecl((r, spec.width)),
            "decay_out": TensorDecl((H * d, r)),
            "decay_bias": TensorDecl((H * d,), role="vector", init="bias"),
            "norm": TensorDecl((e,), role="vector", init="around_one"),
            "o": TensorDecl((spec.width, H * e)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        H, d, e = spec.num_heads, spec.head_dim, spec.value_dim
        if d > 512:
            raise Unsupported(f"gla: a state of {d} rows has no kernel (512 at most)")
        if not float(spec.tau) > 0:
            raise Unsupported("gla: tau must be positive")
        self.spec = spec
        self.rt = runtime
        self.qk, self.inner = H * d, H * e
        # one product: [q | k | v | gate | inner vector of the decay]
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "gate", "decay_in")], dim=0).contiguous()
        self.w_decay, self.b_decay = tensors["decay_out"], tensors["decay_bias"]
        self.norm = tensors["norm"]
        self.w_o = tensors["o"]
        self.eps = float(spec.eps)
        self.tau = float(spec.tau)
        self.q_scale = float(d) ** -0.5

    def first_weights(self) -> torch.Tensor:
        return self.w_in

    def cache_spec(self) -> Optional[CacheSpec]:
        s = self.spec
        return CacheSpec(kind="state", state_shape=(s.num_heads * s.head_dim * s.value_dim,), dtype="float32")

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] in the compute dtype -> [rows, width] (or split-K partial sums of it)."""
        s, rt = self.spec, self.rt
        if not owns_cache or cache is None or cache.kind != "state":
            raise Unsupported("gla: every run of the layer keeps a state of its own")
        (state,) = cache.arrays
        rows = x.shape[0]
        H, d, e = s.num_heads, s.head_dim, s.value_dim
        proj = rt.buffer("gla_proj", (rows, self.w_in.shape[0]))
        linear(x, self.w_in, proj)
        gate_col = 2 * self.qk + self.inner
        z = rt.buffer("gla_decay", (rows, self.qk), torch.float32)
        inner_vec = proj[:, gate_col + self.inner:]
        if x.dtype == torch.float32:
            ops.gemm_simt(inner_vec, self.w_decay, z, self.b_decay, 1.0)
            z_bias = None
        else:
            linear(inner_vec, self.w_decay, z)         # float32 sums; the bias joins where the decays are formed
            z_bias = self.b_decay
        o = rt.buffer("gla_o", (rows, self.inner), torch.float32)
        ops.gla_scan(proj, 0, self.qk, 2 * self.qk, z, self.tau, self.q_scale, state, ctx.q_start, ctx.state_slots, o,
                     ctx.num_requests, H, d, e, z_bias=z_bias)
        g = rt.buffer("gla_gated", (rows, self.inner))
        ops.head_norm_gate(o, proj, gate_col, self.norm, self.eps, g, H, e)
        return linear_partial(g, self.w_o, rt, self.out_name)
