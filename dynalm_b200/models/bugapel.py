"""The Bugapel architecture: config.json -> BugapelConfig -> ModelPlan.

A pre-norm decoder with layer norms (weight and bias) whose residual stream may be several streams
("hyper_connections", parts/block.py: every sublayer reads a weighted sum of the streams and writes its result back
through a small mixing matrix; the model's output is the sum of the streams). The mixer of a layer is softmax attention
of one of two makes (parts/attention.py, kind "gated_attention" with its parameters set either way: per-head unit
queries and keys and a denominator with one more term of score 0, or biases, an interleaved rotation and a window that
keeps the first tokens) or gated linear attention (parts/gla.py, kind "gla"). The feed-forward is a mixture of experts
with a squared ReLU (parts/moe.py, kind "routed_mlp"), or absent. The head is the embedding table; logits are capped by
a tanh.
Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm1.b`, `l<i>.norm2`, `l<i>.norm2.b`, `l<i>.hc{1,2}.{in,out,mix}`,
`l<i>.mix.{q,k,v,o}` (+ `.b` each for the second make), `l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b}`,
`l<i>.mlp.router`, `l<i>.mlp.e<j>.{up,down}`, `final.norm`, `final.norm.b`.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

from ..config.bugapel import BugapelAttention, BugapelConfig, BugapelGLA
from ..config.plan import (BlockSpec, ConnectionSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec, ModelPlan, NormSpec,
                           PositionSpec)
from ..errors import NotFound
from ..registry import register_architecture


def _attention(m: BugapelAttention, width: int, eps: float, p: str) -> MixerSpec:
    position = None
    if m.rot_dims > 0:
        half = m.rot_dims // 2
        factors = None
        if m.wavelengths is not None:
            factors = tuple(m.wavelengths.divisor(m.rot_base ** (-2.0 * i / m.rot_dims)) for i in range(half))
        position = PositionSpec("rotary" if m.make == 1 else "rotary_interleaved", head_dim=m.dim, rotary_dim=m.rot_dims,
                                theta=m.rot_base, factors=factors)
    names = {k: p + "mix." + k for k in ("q", "k", "v", "o")}
    if m.make == 2:
        names.update({k + "_bias": p + "mix." + k + ".b" for k in ("q", "k", "v", "o")})
    return MixerSpec("gated_attention", width, names, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                     value_dim=m.vdim, scale=m.scale, window=m.window, keep_first=m.keep_first if m.window > 0 else 0,
                     eps=eps, qk_norm="head" if m.make == 1 else "none", sink="zero" if m.make == 1 else "none",
                     gated=False, position=position)


class BugapelArchitecture:
    name = "Bugapel"
    model_types = ("bugapel",)

    def read_config(self, obj: Mapping[str, Any]) -> BugapelConfig:
        return BugapelConfig.from_dict(obj)

    def plan(self, cfg: BugapelConfig, present: Optional[Any] = None) -> ModelPlan:
        """`present`: the tensors of the model folder, when known; where it also gives their shapes (a mapping), the
        inner size of a gated-linear-attention layer's decay projection is read from there."""
        layers, order = [], []
        W, eps, S = cfg.width, cfg.norm_eps, cfg.streams
        for i, layer in enumerate(cfg.layers):
            p, m = f"l{i}.", layer.mixer
            if isinstance(m, BugapelAttention):
                mixer = _attention(m, W, eps, p)
            else:
                assert isinstance(m, BugapelGLA)
                rank = m.rank
                if isinstance(present, Mapping) and p + "mix.a1" in present:
                    rank = int(present[p + "mix.a1"][0])
                if rank <= 0:
                    raise NotFound(f"config.json: layers[{i}]: the inner size of the decay projection is given neither by a "
                                   f"tensor '{p}mix.a1' nor by 'rank'")
                names = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm", "decay_in": "a1",
                         "decay_out": "a2", "decay_bias": "a2.b"}
                mixer = MixerSpec("gla", W, {k: p + "mix." + f for k, f in names.items()}, num_heads=m.heads,
                                  head_dim=m.dim, value_dim=m.vdim, tau=m.tau, rank=rank, eps=eps)

            def norm(name: str) -> NormSpec:
                return NormSpec("layer", W, eps, {"weight": p + name, "bias": p + name + ".b"})

            parts: Dict[str, Any] = dict(mixer_norm=norm("norm1"), mixer=mixer)
            if layer.mlp is not None:
                f = layer.mlp
                names = {"router": p + "mlp.router"}
                for j in range(f.experts):
                    names[f"up{j}"] = f"{p}mlp.e{j}.up"
                    names[f"down{j}"] = f"{p}mlp.e{j}.down"
                parts["ffn_norm"] = norm("norm2")
                parts["ffn"] = FeedForwardSpec("routed_mlp", W, names, inner=f.ff, experts=f.experts, top=f.top,
                                               groups=f.groups, keep_groups=f.keep_groups, weight_scale=f.scale,
                                               activation="relu2")
            if S > 0:
                # the weights of the streams around each sublayer are parts of their own (parts/block.py)
                parts["mixer_link"] = ConnectionSpec("hyper", W, {k: f"{p}hc1.{k}" for k in ("in", "out", "mix")}, streams=S)
                if layer.mlp is not None:
                    parts["ffn_link"] = ConnectionSpec("hyper", W, {k: f"{p}hc2.{k}" for k in ("in", "out", "mix")}, streams=S)
                layers.append(BlockSpec("hyper_connections", **parts, streams=S))
            else:
                layers.append(BlockSpec("pre_norm", **parts))
            order.append(LayerRun(i))
        ignorable = []
        for i, layer in enumerate(cfg.layers):
            if layer.mlp is None:          # a layer without a feed-forward may still carry its norm and its stream weights
                ignorable += [f"l{i}.norm2", f"l{i}.norm2.b"] + [f"l{i}.hc2.{k}" for k in ("in", "out", "mix")]
        plan = ModelPlan(
            embedding=EmbeddingSpec(cfg.vocab, W, cfg.embedding_scale, {"weight": "embed"}),
            layers=layers, order=order,
            final_norm=NormSpec("layer", W, eps, {"weight": "final.norm", "bias": "final.norm.b"}),
            head=HeadSpec(cfg.vocab, W, True, 1.0, {}, softcap=cfg.logit_softcap),
            context_length=cfg.context, ignorable=tuple(ignorable))
        plan.validate()
        return plan


register_architecture(BugapelArchitecture())
