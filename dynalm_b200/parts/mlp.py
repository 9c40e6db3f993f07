"""Gated feed-forward: down(act(gate x) * up x), the "gated_mlp" kind
(dynalm/src/model/transformer.cpp:671-693), act silu or the tanh form of GELU (parameter `activation`). Gate and up
run as one product against [Wg; Wu].
Ungated feed-forward: down(act(up x)), the "mlp" kind, act the squared ReLU or the tanh form of GELU."""

from __future__ import annotations

from typing import Dict

import torch

from ..errors import Unsupported
from ..kernels import ops
from ..kernels.gemm import linear_act, linear_geglu, linear_partial, linear_swiglu
from .base import TensorDecl, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts (and graph_key) only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        return {
            "gate": TensorDecl((spec.inner, spec.width)),
            "up": TensorDecl((spec.inner, spec.width)),
            "down": TensorDecl((spec.width, spec.inner)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        self.activation = spec.get("activation", "silu")
        if self.activation not in ("silu", "gelu_tanh"):
            raise Unsupported(f"gated_mlp: activation '{self.activation}' has no kernel (silu and gelu_tanh do)")
        self.spec = spec
        self.rt = runtime
        self.w_gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.w_down = tensors["down"]

    def first_weights(self) -> torch.Tensor:
        """The weights this part streams first (a block may say so to the kernel in front, kernels/ops.stream_ahead)."""
        return self.w_gate_up

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if x.shape[0] <= ops.SKINNY_FAST_ROWS:
            ops.stream_ahead(self.w_down)              # taken by the gate | up product, read by the product after it
        if self.activation == "gelu_tanh":
            act = linear_geglu(x, self.w_gate_up, rt, s.inner)
        else:
            act = linear_swiglu(x, self.w_gate_up, rt, s.inner)
        return linear_partial(act, self.w_down, rt, "ffn_out")


@register_feed_forward("mlp")
class DenseMLP:
    """down(act(up x)) without a gate (parameters inner, activation: "relu2" = max(z, 0)^2, "gelu_tanh" =
    0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))))."""

    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        return {
            "up": TensorDecl((spec.inner, spec.width)),
            "down": TensorDecl((spec.width, spec.inner)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        self.activation = spec.get("activation", "relu2")
        if self.activation not in ("relu2", "gelu_tanh"):
            raise Unsupported(f"mlp: activation '{self.activation}' has no kernel (relu2 and gelu_tanh do)")
        self.spec = spec
        self.rt = runtime
        self.w_up = tensors["up"]
        self.w_down = tensors["down"]

    def first_weights(self) -> torch.Tensor:
        return self.w_up

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if x.shape[0] <= ops.SKINNY_FAST_ROWS:
            ops.stream_ahead(self.w_down)              # taken by the up product, read by the product after it
        act = linear_act(x, self.w_up, rt, s.inner, self.activation)
        return linear_partial(act, self.w_down, rt, "ffn_out")
