"""Bugapel without a GPU: reading config.json, the plan it turns into, which tensors each layer declares, the caches its
mixers ask for, and the plain implementation against its own reading token by token and by hand."""

import copy

import numpy as np
import pytest
import torch

import plain_bugapel as plain
from bugapel_configs import B_A, B_B, B_C, BUGAPEL, ONLY_GLA

from dynalm_b200.errors import InvalidArgument, NotFound, Unsupported
from dynalm_b200.parts import CONNECTIONS, FEED_FORWARDS, MIXERS, NORMS
from dynalm_b200.registry import find_architecture
from dynalm_b200.weights import write_model_folder
from dynalm_b200.weights.loader import WeightMismatch, expected_tensors, open_model_folder


def _plan(cfg, present=None):
    arch = find_architecture(cfg)
    return arch.read_config(cfg), arch.plan(arch.read_config(cfg), present)


def test_config_reads_every_size_per_layer():
    cfg, plan = _plan(B_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale, cfg.streams, cfg.logit_softcap) == (300, 96, 1e-5, 2.5, 3, 12.0)
    assert [l.type for l in cfg.layers] == ["attention", "gla", "attention_2", "attention", "gla"]
    a = cfg.layers[0].mixer
    assert (a.make, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.rot_dims, a.rot_base) == (1, 4, 2, 32, 16, 0.9, 16, 900.0)
    assert (a.wavelengths.factor, a.wavelengths.low, a.wavelengths.high, a.wavelengths.original) == (4.0, 1.0, 4.0, 64)
    b = cfg.layers[2].mixer
    assert (b.make, b.window, b.keep_first, b.rot_dims, b.wavelengths) == (2, 20, 3, 8, None)
    g = cfg.layers[1].mixer
    assert (g.heads, g.dim, g.vdim, g.tau, g.rank) == (3, 24, 40, 8.0, 12)
    f = cfg.layers[0].mlp
    assert (f.ff, f.experts, f.top, f.scale, f.groups, f.keep_groups) == (40, 6, 2, 1.3, 3, 2)
    assert cfg.layers[1].mlp is None
    m = plan.layers[0].mixer
    assert (m.kind, m.qk_norm, m.sink, m.window, m.keep_first, m.position.kind) == ("gated_attention", "head", "zero", 0, 0, "rotary")
    m2 = plan.layers[2].mixer
    assert (m2.qk_norm, m2.sink, m2.window, m2.keep_first, m2.position.kind) == ("none", "none", 20, 3, "rotary_interleaved")
    assert set(m2.tensors) == {"q", "k", "v", "o", "q_bias", "k_bias", "v_bias", "o_bias"} and m2.tensors["o_bias"] == "l2.mix.o.b"
    assert plan.layers[0].kind == "hyper_connections" and plan.layers[0].streams == 3
    assert plan.layers[0].mixer_link.tensors == {"in": "l0.hc1.in", "out": "l0.hc1.out", "mix": "l0.hc1.mix"}
    assert "ffn" not in plan.layers[1].parts and "ffn_link" not in plan.layers[1].parts
    assert {"l1.norm2", "l1.norm2.b", "l1.hc2.mix"} <= set(plan.ignorable)
    r = plan.layers[0].ffn
    assert (r.kind, r.inner, r.experts, r.top, r.groups, r.keep_groups, r.weight_scale) == ("routed_mlp", 40, 6, 2, 3, 2, 1.3)
    assert plan.head.tied and plan.head.softcap == 12.0 and plan.embedding.scale == 2.5
    assert plan.final_norm.kind == "layer" and plan.final_norm.tensors == {"weight": "final.norm", "bias": "final.norm.b"}


def test_the_stretching_rule_has_three_ranges():
    cfg, plan = _plan(B_A)
    w = cfg.layers[0].mixer.wavelengths
    factors = plan.layers[0].mixer.position.factors
    want = plain.frequencies(900.0, 16, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64})
    plainf = plain.frequencies(900.0, 16)
    assert np.allclose(plainf / np.array(factors), want, rtol=1e-12)
    kinds = {1.0 if f == 1.0 else (4.0 if f == 4.0 else 0.0) for f in factors}
    assert kinds == {1.0, 4.0, 0.0}, "the test model has frequencies that are kept, divided and blended"
    assert w.divisor(1.0) == 1.0 and w.divisor(1e-6) == 4.0


def test_keys_left_out_switch_a_mechanism_off():
    cfg, plan = _plan(B_C)
    assert (cfg.embedding_scale, cfg.streams, cfg.logit_softcap) == (1.0, 0, 0.0)
    assert plan.layers[0].kind == "pre_norm" and "mixer_link" not in plan.layers[0].parts
    cfg, plan = _plan(B_B)
    assert plan.layers[1].mixer.position is None and plan.layers[3].mixer.position is None
    assert plan.layers[4].mixer.window == 0 and plan.layers[4].mixer.keep_first == 0
    assert plan.layers[0].ffn.groups == 1 and plan.layers[0].streams == 1


def test_refusals():
    def broken(change):
        cfg = copy.deepcopy(B_A)
        change(cfg)
        return cfg
    with pytest.raises(Unsupported):
        _plan(broken(lambda c: c["layers"][0].update(type="conv")))
    with pytest.raises(InvalidArgument):
        _plan(broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3)))
    with pytest.raises(InvalidArgument):
        _plan(broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=15)))
    with pytest.raises(InvalidArgument):
        _plan(broken(lambda c: c["layers"][0]["mlp"]["router"].update(experts=7)))
    with pytest.raises(InvalidArgument):
        _plan(broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=5)))
    with pytest.raises(Unsupported):
        _plan(broken(lambda c: c["layers"][0]["mlp"].update(kind="dense")))
    with pytest.raises(NotFound):
        _plan(broken(lambda c: c["layers"][1]["mixer"].pop("rank")))
    with pytest.raises(NotFound):
        _plan(broken(lambda c: c.pop("layers")))


def test_the_decay_projection_takes_its_inner_size_from_the_file(tmp_path):
    """A folder whose config.json does not give `rank`: the plan reads it from the tensor's shape."""
    write_model_folder(str(tmp_path), ONLY_GLA, 3, dtype=torch.float32)
    import json
    import os
    cfg = copy.deepcopy(ONLY_GLA)
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank")
    with open(os.path.join(str(tmp_path), "config.json"), "w") as f:
        json.dump(cfg, f)
    folder = open_model_folder(str(tmp_path))
    assert [l.mixer.rank for l in folder.plan.layers] == [8, 4]
    folder.close()


def test_declared_tensors_and_the_loaders_one_error(tmp_path):
    cfg, plan = _plan(B_A)
    want = expected_tensors(plan)
    assert want["l0.hc1.mix"].shape == (3, 3) and want["l0.hc2.in"].shape == (3,)
    assert want["l1.mix.a1"].shape == (12, 96) and want["l1.mix.a2"].shape == (72, 12) and want["l1.mix.a2.b"].shape == (72,)
    assert want["l1.mix.norm"].shape == (40,) and want["l1.mix.g"].shape == (120, 96)
    assert want["l2.mix.k.b"].shape == (72,) and want["l2.mix.v"].shape == (72, 96)
    assert want["l0.mlp.e5.down"].shape == (96, 40) and want["l0.mlp.router"].shape == (6, 96)
    assert "l1.hc2.in" not in want and "l0.mix.q.b" not in want and "head" not in want
    write_model_folder(str(tmp_path), B_A, 1, dtype=torch.float32)
    import json
    import os
    bad = copy.deepcopy(B_A)
    bad["layers"][0]["mixer"]["heads"] = 8
    bad["layers"][2]["mlp"]["router"]["experts"] = 5
    with open(os.path.join(str(tmp_path), "config.json"), "w") as f:
        json.dump(bad, f)
    with pytest.raises(WeightMismatch) as e:
        open_model_folder(str(tmp_path))
    assert "l2.mlp.e4.up" in e.value.missing and any(n == "l0.mix.q" for n, _, _ in e.value.wrong_shape)


def test_registries_hold_the_new_kinds():
    assert "gla" in MIXERS.kinds() and "routed_mlp" in FEED_FORWARDS.kinds() and "layer" in NORMS.kinds()
    assert "hyper" in CONNECTIONS.kinds()


@pytest.mark.parametrize("name", sorted(BUGAPEL))
def test_plain_whole_equals_plain_token_by_token(name, tmp_path):
    cfg, seed = BUGAPEL[name]
    write_model_folder(str(tmp_path), cfg, seed, dtype=torch.float32)
    model = plain.PlainBugapel(str(tmp_path))
    toks = [int(t) for t in np.random.RandomState(3).randint(0, cfg["vocab"], 75)]
    whole = model.logits(toks)
    assert np.abs(model.logits_stepwise(toks) - whole).max() < 1e-11
    assert np.abs(model.logits(toks, cuts=[2, 31, 3, 20]) - whole).max() < 1e-11


def test_plain_mechanisms_by_hand():
    # the mask: a window of 3 that keeps the first 2
    see = [[j for j in range(8) if plain.visible(i, j, 3, 2)] for i in range(8)]
    assert see[0] == [0] and see[4] == [0, 1, 2, 3, 4] and see[5] == [0, 1, 3, 4, 5] and see[7] == [0, 1, 5, 6, 7]
    # the sink: one key of score 0 -> half of its value
    q, k, v = np.zeros((1, 1, 4)), np.ones((1, 1, 4)), np.full((1, 1, 2), 6.0)
    assert np.allclose(plain.attend(q, k, v, [0], [0], 1.0, sink=True), 3.0)
    assert np.allclose(plain.attend(q, k, v, [0], [0], 1.0, sink=False), 6.0)
    # rotation: a quarter turn of the pair (1, 0) in either layout
    f = np.array([np.pi / 2])
    x = np.array([[[1.0, 0.0, 5.0]]])
    assert np.allclose(plain.rotate(x, [1], f, "pairs"), [[[0.0, 1.0, 5.0]]]) and np.allclose(plain.rotate(x, [1], f, "halves"), [[[0.0, 1.0, 5.0]]])
    y = np.array([[[1.0, 2.0, 0.0, 0.0]]])
    f2 = np.array([np.pi / 2, np.pi])
    assert np.allclose(plain.rotate(y, [1], f2, "halves"), [[[0.0, -2.0, 1.0, 0.0]]])
    assert np.allclose(plain.rotate(y, [1], f2, "pairs"), [[[-2.0, 1.0, 0.0, 0.0]]])
    # routing: the best expert of all lies in a group that loses to a group with a larger maximum? no: its group wins
    chosen, w = plain.route(np.array([4.0, -5.0, 3.0, 3.0]), 1, 2, 1, 2.0)
    assert chosen == [0] and np.isclose(w.sum(), 2.0)
    chosen, _ = plain.route(np.array([1.0, 0.9, 5.0, -9.0]), 2, 2, 1, 1.0)
    assert chosen == [2, 3], "both experts come from the one kept group, however weak the second"
    # layer norm: mean and variance of the deviations
    out = plain.layer_norm(np.array([1.0, 3.0]), np.array([2.0, 2.0]), np.array([1.0, 1.0]), 0.0)
    assert np.allclose(out, [-1.0, 3.0])
