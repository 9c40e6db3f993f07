"""RMSNorm over the float32 residual stream (CpuDevice::rms_norm, dynacore/cpu/cpu_device.cpp:1179-1205), in front of a
sublayer ("rms") or after the sum that a sublayer's result enters ("rms_after_sum"); layer norm with weight and bias
("layer") over a stream of one part or of several."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import TensorDecl, register_norm


@register_norm("rms")
class RMSNorm:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.width,), role="vector", init="around_one")}

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        self.spec = spec
        self.weight = tensors["weight"]
        self.eps = float(spec.eps)

    def forward(self, residual: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
                delta_scale: float = 1.0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out = norm(residual + delta_scale * delta); the sum is written back to `residual` unless
        `rows` picks a subset. Everything is computed in float32; `out` has the compute dtype."""
        ops.rmsnorm(residual, self.weight, self.eps, out, delta=delta, delta_scale=delta_scale, rows=rows)
        return out

    def forward_pair(self, residual: torch.Tensor, out: torch.Tensor, other: Optional["RMSNorm"],
                     other_out: Optional[torch.Tensor], delta_a: Optional[torch.Tensor] = None,
                     delta_b: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
        """This norm and `other` (same width and eps, its own weight; may be None) of the same row, in one kernel:
        residual += delta_a + delta_b (written back unless `rows` selects), out = norm * weight, other_out = norm *
        other's weight."""
        ops.rmsnorm_pair(residual, self.weight, out, other.weight if other is not None else None, other_out, self.eps,
                         delta_a=delta_a, delta_b=delta_b, rows=rows)


@register_norm("rms_after_sum")
class RMSNormAfterSum:
    """x <- rmsnorm(alpha * x + delta_scale * delta) * weight: the norm of a layer that norms what it has just summed.
    `alpha` (a parameter, default 1) weighs the stream against the sublayer's result; `delta_scale` is a per-channel
    scale of that result, there when the model has its tensor. The stream itself becomes the normed row."""

    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.width,), role="vector", init="around_one"),
                "delta_scale": TensorDecl((spec.width,), role="vector", required=False, init="around_one")}

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        self.spec = spec
        self.weight = tensors["weight"]
        self.delta_scale = tensors.get("delta_scale")
        self.eps = float(spec.eps)
        self.alpha = float(spec.get("alpha", 1.0))

    def forward(self, residual: torch.Tensor, out: Optional[torch.Tensor], delta: torch.Tensor) -> None:
        """residual (float32, in place) <- the normed sum; out (compute dtype, or None) <- a copy for the products of
        the next sublayer. delta: the sublayer's result, [n, width] or split-K partial sums [parts, n, width]."""
        ops.norm_after_sum(residual, delta, self.weight, self.eps, self.alpha, self.delta_scale, out)


@register_norm("layer")
class LayerNorm:
    """y = (x - mean) / sqrt(mean of squared deviations + eps) * weight + bias, in float32, two passes over the row.
    The stream it reads may have several parts (parts/block.py, "hyper_connections"): `forward_stream` norms a weighted
    sum of them after applying the update that the sublayer in front left pending; `forward` is the same for a stream of
    one part, with the interface of the other norms."""

    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.width,), role="vector", init="around_one"),
                "bias": TensorDecl((spec.width,), role="vector", required=False, init="bias")}

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        self.spec = spec
        self.weight = tensors["weight"]
        self.bias = tensors.get("bias")
        self.eps = float(spec.eps)

    def forward(self, residual: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
                delta_scale: float = 1.0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out = norm(residual + delta_scale * delta); the sum is written back to `residual` unless `rows` picks a
        subset."""
        ops.stream_layer_norm(residual, 1, self.weight, self.bias, self.eps, out, delta=delta, delta_scale=delta_scale,
                              rows=rows)
        return out

    def forward_stream(self, streams: torch.Tensor, parts: int, out: torch.Tensor, init: Optional[torch.Tensor] = None,
                       delta: Optional[torch.Tensor] = None, link=None, read: Optional[torch.Tensor] = None,
                       rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out = norm(sum_t read[t] x_t) over a stream of `parts` parts [n, parts * width], after x_t <- sum_s
        link.mix[s, t] x_s + link.write[t] * delta when the sublayer in front left `delta` pending (`link`: its stream
        connection); `init`: every part starts as this row; `read` None: the plain sum of the parts."""
        ops.stream_layer_norm(streams, parts, self.weight, self.bias, self.eps, out, init=init, delta=delta,
                              mix=link.mix if link is not None else None, write=link.write if link is not None else None,
                              read=read, rows=rows)
        return out
