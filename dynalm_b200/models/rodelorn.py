"""The Rodelorn architecture: config.json -> RodelornConfig -> ModelPlan.

A decoder whose layers norm in front of AND behind every sublayer: x <- x + norm1b(mixer(norm1(x))), x <- x +
norm2b(ffn(norm2(x))) (block kind "sandwich_norm"). The mixer of a layer is a gated delta rule (parts/delta_rule.py,
kind "gated_delta") or two mixers side by side that read the same input (parts/side_by_side.py): windowed attention
with queries and keys normed over their whole projection, a partial rotation and an output gate (parts/attention.py,
kind "gated_attention") beside a gated linear recurrence (parts/rglru.py, kind "rglru"). The feed-forward is gated with
the tanh form of GELU (parts/mlp.py, kind "gated_mlp"), or absent. The logits are scaled and then capped by a tanh.
Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`,
`l<i>.mix.{q,q.conv,k,k.conv,v,v.conv,b,a,A_log,dt_bias,norm,g,o}` or
`l<i>.mix.left.{q,k,v,q.norm,k.norm,g,o}` with `l<i>.mix.right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}`,
`l<i>.mlp.{gate,up,down}`, `final.norm`, `head`.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

from ..config.plan import (BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec, ModelPlan, NormSpec,
                           PositionSpec)
from ..config.rodelorn import RodelornAttention, RodelornConfig, RodelornDelta, RodelornPair, RodelornRecurrence
from ..registry import register_architecture

_DELTA = (("q", "q"), ("q_conv", "q.conv"), ("k", "k"), ("k_conv", "k.conv"), ("v", "v"), ("v_conv", "v.conv"), ("b", "b"),
          ("a", "a"), ("a_log", "A_log"), ("dt_bias", "dt_bias"), ("norm", "norm"), ("gate", "g"), ("o", "o"))
_ATTENTION = (("q", "q"), ("k", "k"), ("v", "v"), ("q_norm", "q.norm"), ("k_norm", "k.norm"), ("gate", "g"), ("o", "o"))
_RECURRENCE = (("y", "y"), ("y_bias", "y.b"), ("x", "x"), ("x_bias", "x.b"), ("conv", "conv"), ("conv_bias", "conv.b"),
               ("ra", "ra"), ("ra_bias", "ra.b"), ("ri", "ri"), ("ri_bias", "ri.b"), ("lam", "lam"), ("o", "o"))


def _side(m, width: int, eps: float):
    """(spec without tensor names, local name -> name under the side's prefix) of one side of a pair."""
    if isinstance(m, RodelornAttention):
        position = None
        if m.rot_dims > 0:
            # every frequency base^(-2i / dims) is divided by the factor before it meets the position
            position = PositionSpec("rotary", head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                                    factors=(m.rot_factor,) * (m.rot_dims // 2) if m.rot_factor != 1.0 else None)
        params = dict(num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale,
                      window=m.window, eps=eps, qk_norm="projection", gated=True, position=position)
        return "gated_attention", params, _ATTENTION
    assert isinstance(m, RodelornRecurrence)
    return "rglru", dict(inner=m.width, blocks=m.blocks, taps=m.conv, decay_scale=8.0), _RECURRENCE


class RodelornArchitecture:
    name = "Rodelorn"
    model_types = ("rodelorn",)

    def read_config(self, obj: Mapping[str, Any]) -> RodelornConfig:
        return RodelornConfig.from_dict(obj)

    def plan(self, cfg: RodelornConfig, present: Optional[set] = None) -> ModelPlan:
        layers, order, ignorable = [], [], []
        W, eps = cfg.width, cfg.norm_eps
        for i, layer in enumerate(cfg.layers):
            p, m = f"l{i}.", layer.mixer
            if isinstance(m, RodelornDelta):
                names = {k: p + "mix." + f for k, f in _DELTA}
                mixer = MixerSpec("gated_delta", W, names, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                  value_dim=m.vdim, taps=m.conv, eps=eps)
            else:
                assert isinstance(m, RodelornPair)
                names: Dict[str, str] = {}
                subs = {}
                for side, sub in (("left", m.left), ("right", m.right)):
                    kind, params, locals_ = _side(sub, W, eps)
                    subs[side] = MixerSpec(kind, W, None, **params)
                    names.update({f"{side}.{k}": f"{p}mix.{side}.{f}" for k, f in locals_})
                mixer = MixerSpec("side_by_side", W, names, left=subs["left"], right=subs["right"],
                                  left_scale=m.left_scale, right_scale=m.right_scale)

            def norm(name: str) -> NormSpec:
                return NormSpec("rms", W, eps, {"weight": p + name})

            parts = dict(mixer_norm=norm("norm1"), mixer=mixer, mixer_post_norm=norm("norm1b"))
            if layer.mlp is not None:
                parts["ffn_norm"] = norm("norm2")
                parts["ffn"] = FeedForwardSpec("gated_mlp", W, {"gate": p + "mlp.gate", "up": p + "mlp.up",
                                                                "down": p + "mlp.down"},
                                               inner=layer.mlp.ff, activation="gelu_tanh")
                parts["ffn_post_norm"] = norm("norm2b")
            else:
                ignorable += [p + "norm2", p + "norm2b"]      # a layer without a feed-forward may still carry them
            layers.append(BlockSpec("sandwich_norm", **parts))
            order.append(LayerRun(i))
        plan = ModelPlan(
            embedding=EmbeddingSpec(cfg.vocab, W, cfg.embedding_scale, {"weight": "embed"}),
            layers=layers, order=order,
            final_norm=NormSpec("rms", W, eps, {"weight": "final.norm"}),
            head=HeadSpec(cfg.vocab, W, False, 1.0, {"weight": "head"}, logit_scale=cfg.logit_scale,
                          softcap=cfg.logit_softcap),
            context_length=cfg.context, ignorable=tuple(ignorable))
        plan.validate()
        return plan


register_architecture(RodelornArchitecture())
