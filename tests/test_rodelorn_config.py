"""Rodelorn without a GPU: reading config.json, the plan it turns into, which tensors each layer declares, the cache
a pair of mixers asks for, and the plain implementation against its own reading token by token and by hand."""

import copy
import json

import numpy as np
import pytest
import torch

import plain_rodelorn as plain
from rodelorn_configs import O_A, O_B, O_C, RODELORN

from dynalm_b200.cache import CacheManager
from dynalm_b200.errors import InvalidArgument, NotFound, Unsupported
from dynalm_b200.parts.base import CacheSpec
from dynalm_b200.registry import find_architecture
from dynalm_b200.weights import write_model_folder
from dynalm_b200.weights.loader import WeightMismatch, expected_tensors, open_model_folder


def _plan(cfg, present=None):
    arch = find_architecture(cfg)
    return arch.read_config(cfg), arch.plan(arch.read_config(cfg), present)


def test_config_reads_every_size_per_layer():
    cfg, plan = _plan(O_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale, cfg.logit_scale, cfg.logit_softcap) == \
        (300, 96, 1e-5, 2.5, 0.5, 9.0)
    assert [l.type for l in cfg.layers] == ["parallel", "delta", "delta", "parallel"]       # "delta_2" is a delta layer
    a, r = cfg.layers[0].mixer.left, cfg.layers[0].mixer.right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.rot_dims, a.rot_base, a.rot_factor) == \
        (4, 2, 32, 16, 0.21, 20, 8, 10000.0, 4.0)
    assert (r.width, r.blocks, r.conv) == (48, 3, 3)
    assert (cfg.layers[0].mixer.left_scale, cfg.layers[0].mixer.right_scale) == (0.7, 1.3)
    d = cfg.layers[2].mixer
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (3, 3, 32, 8, 2)
    m = plan.layers[0].mixer
    assert m.kind == "side_by_side" and (m.left_scale, m.right_scale) == (0.7, 1.3)
    assert (m.left.kind, m.left.num_heads, m.left.num_kv_heads, m.left.head_dim, m.left.value_dim, m.left.window) == \
        ("gated_attention", 4, 2, 32, 16, 20)
    assert (m.left.position.kind, m.left.position.rotary_dim, m.left.position.factors) == ("rotary", 8, (4.0,) * 4)
    assert (m.right.kind, m.right.inner, m.right.blocks, m.right.taps, m.right.decay_scale) == ("rglru", 48, 3, 3, 8.0)
    assert plan.layers[1].mixer.kind == "gated_delta" and plan.layers[1].mixer.taps == 3
    assert plan.layers[0].kind == "sandwich_norm" and plan.layers[0].ffn.activation == "gelu_tanh"
    assert (plan.head.logit_scale, plan.head.softcap, plan.embedding.scale) == (0.5, 9.0, 2.5)


def test_keys_left_out_switch_a_mechanism_off():
    cfg, plan = _plan(O_B)
    assert (cfg.embedding_scale, cfg.logit_scale, cfg.logit_softcap) == (1.0, 1.0, 0.0)
    a = cfg.layers[1].mixer.left
    assert a.window == 0 and a.rot_dims == 0 and plan.layers[1].mixer.left.position is None
    assert (cfg.layers[1].mixer.left_scale, cfg.layers[1].mixer.right_scale) == (1.0, 1.0)
    assert cfg.layers[2].mixer.left.rot_factor == 1.0 and plan.layers[2].mixer.left.position.factors is None
    assert cfg.layers[1].mlp is None and "ffn" not in plan.layers[1].parts and "ffn_post_norm" not in plan.layers[1].parts
    assert {"l1.norm2", "l1.norm2b"} <= set(plan.ignorable)
    assert plan.head.softcap == 0.0


def test_declared_tensors_and_their_shapes():
    _, plan = _plan(O_A)
    shapes = {n: d.shape for n, d in expected_tensors(plan).items()}
    assert shapes["l0.mix.left.q"] == (128, 96) and shapes["l0.mix.left.k"] == (64, 96) and shapes["l0.mix.left.v"] == (32, 96)
    assert shapes["l0.mix.left.q.norm"] == (128,) and shapes["l0.mix.left.k.norm"] == (64,)
    assert shapes["l0.mix.left.g"] == (64, 96) and shapes["l0.mix.left.o"] == (96, 64)
    assert shapes["l0.mix.right.ra"] == (3, 16, 16) and shapes["l0.mix.right.ri.b"] == (3, 16)
    assert shapes["l0.mix.right.conv"] == (48, 3) and shapes["l0.mix.right.lam"] == (48,) and shapes["l0.mix.right.o"] == (96, 48)
    assert shapes["l1.mix.q"] == (32, 96) and shapes["l1.mix.v"] == (96, 96) and shapes["l1.mix.v.conv"] == (96, 3)
    assert shapes["l1.mix.b"] == (4, 96) and shapes["l1.mix.A_log"] == (4,) and shapes["l1.mix.norm"] == (24,)
    assert shapes["l2.mix.q.conv"] == (96, 2) and shapes["l2.mix.g"] == (24, 96)
    assert {"embed", "head", "final.norm", "l0.norm1b", "l3.norm2b", "l0.mlp.gate", "l1.mlp.down"} <= set(shapes)


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="attention"), Unsupported),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), Unsupported),
    (lambda c: c["layers"][1]["mixer"].pop("heads"), NotFound),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), InvalidArgument),            # 4 heads on 3 query/key heads
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), InvalidArgument),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=34), InvalidArgument),     # more than the head
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=3), InvalidArgument),      # pairs
    (lambda c: c["layers"][0]["mixer"]["right"].update(blocks=5), InvalidArgument),          # 48 channels in 5 blocks
    (lambda c: c["layers"][0]["mixer"].pop("right"), NotFound),
    (lambda c: c.update(logit_softcap=-1.0), InvalidArgument),
    (lambda c: c.pop("layers"), NotFound),
])
def test_config_refusals(change, error):
    cfg = copy.deepcopy(O_A)
    change(cfg)
    with pytest.raises(error):
        _plan(cfg)


def test_a_folder_is_written_read_and_checked(tmp_path):
    write_model_folder(str(tmp_path), O_A, 3, dtype=torch.bfloat16)
    folder = open_model_folder(str(tmp_path))
    assert folder.architecture.name == "Rodelorn" and len(folder.plan.layers) == 4
    folder.close()
    other = copy.deepcopy(O_A)
    other["layers"][1]["mixer"]["vdim"] = 32                     # another value size: shapes disagree, one error lists them
    (tmp_path / "config.json").write_text(json.dumps(other))
    with pytest.raises(WeightMismatch) as e:
        open_model_folder(str(tmp_path))
    assert "l1.mix.v" in str(e.value) and "l1.mix.norm" in str(e.value)


def test_a_pair_asks_for_pages_that_carry_a_state_row():
    """The cache of a pair: the attention's pages with the recurrence's state row beside them, both handed out,
    cleared and given back with the request."""
    from dynalm_b200.parts.side_by_side import SideBySideMixer

    class Side:
        out_name = "x"
        def __init__(self, spec): self._spec = spec
        def cache_spec(self): return self._spec
    pair = SideBySideMixer.__new__(SideBySideMixer)
    pair.left = Side(CacheSpec(kind="pages", entry_shape=(2, 16), tensors=2, window=20))
    pair.right = Side(CacheSpec(kind="state", state_shape=(144,), dtype="float32"))
    spec = pair.cache_spec()
    assert (spec.kind, spec.entry_shape, spec.tensors, spec.window, spec.state_shape) == ("pages", (2, 16), 2, 20, (144,))
    lone = CacheSpec(kind="state", state_shape=(7,), dtype="float32")
    mgr = CacheManager([spec, lone, spec], page_size=16, max_tokens=64, max_requests=2, context=64, device=None,
                       dtype=torch.float32)
    assert len(mgr.groups) == 1 and set(mgr.state_specs) == {0, 1, 2}
    mgr.add_request("a")
    mgr.reserve("a", 40)
    assert mgr.free_pages == 1
    with pytest.raises(Unsupported):
        mgr.truncate("a", 10)                       # a state row cannot be rewound
    mgr.free_request("a")
    assert mgr.free_pages == 4 and mgr.free_slots == 2
    mgr.check()


@pytest.mark.parametrize("name", sorted(RODELORN))
def test_plain_whole_sequence_equals_plain_greedy_and_keeps_layers(name, tmp_path):
    cfg, seed = RODELORN[name]
    write_model_folder(str(tmp_path), cfg, seed, dtype=torch.float32)
    model = plain.PlainRodelorn(str(tmp_path))
    tokens = [int(t) for t in np.random.RandomState(2).randint(0, cfg["vocab"], size=30)]
    z, layers = model.logits(tokens, layers=True)
    assert z.shape == (30, cfg["vocab"]) and layers.shape == (len(cfg["layers"]), 30, cfg["width"])
    assert np.isfinite(z).all()
    cap = cfg.get("logit_softcap")
    if cap:
        assert np.abs(z).max() < cap
    g = model.greedy(tokens[:10], 3)
    assert g[0] == int(np.argmax(z[9]))
    assert g[1] == int(np.argmax(model.logits(tokens[:10] + g[:1])[-1]))


def test_plain_mechanisms_by_hand():
    assert np.allclose(plain.rms_norm(np.array([3.0, 4.0]), 0.0), np.array([3.0, 4.0]) / np.sqrt(12.5))
    assert plain.gelu_tanh(np.array([1.0]))[0] == pytest.approx(0.841192, abs=1e-6)
    # the last tap is the current token's; zeros stand before the start
    conv = plain.ShortConv(np.array([[100.0, 10.0, 1.0]]), np.array([0.5]))
    assert [float(conv.step(np.array([v]))[0]) for v in (1.0, 2.0, 4.0)] == [1.5, 12.5, 124.5]
    # pair (i, i + dims / 2) turns by position * base^(-2i / dims) / factor; what lies behind `dims` passes
    v = np.array([[1.0, 1.0, 0.0, 0.0, 9.0]])
    r = plain.rotate_half(v, 2, 4, 100.0, 2.0)
    assert np.allclose(r[0], [np.cos(1.0), np.cos(0.1), np.sin(1.0), np.sin(0.1), 9.0])
    # one delta head with d = e = 1, no decay (a very negative step size), beta = 1 (a large b): the state holds the
    # newest value per unit key, so the read-out of a token is its own value times k q
    t = {"p.q": np.array([[1.0]]), "p.k": np.array([[1.0]]), "p.v": np.array([[2.0]]), "p.q.conv": np.array([[1.0]]),
         "p.k.conv": np.array([[1.0]]), "p.v.conv": np.array([[1.0]]), "p.b": np.array([[50.0]]), "p.a": np.array([[0.0]]),
         "p.A_log": np.array([0.0]), "p.dt_bias": np.array([-50.0]), "p.norm": np.array([1.0]), "p.g": np.array([[1.0]]),
         "p.o": np.array([[1.0]])}
    mix = plain.DeltaMixer({"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 1}, t, "p.", 0.0)
    out = mix.step(np.array([3.0]), 0)
    v3 = plain.silu(np.array([6.0]))[0]
    assert mix.S[0, 0, 0] == pytest.approx(v3, rel=1e-5)                   # k is a unit vector: S = k v
    assert out[0] == pytest.approx(plain.silu(np.array([3.0]))[0], rel=1e-5)      # o / rms(o) = 1, times silu(gate)
    mix.step(np.array([-3.0]), 1)                                          # k = -1 (unit): S k = -v3, u = v' + v3 ...
    assert np.isfinite(mix.S).all()
    # the gated linear recurrence from S = 0: the first token is scaled by sqrt(1 - a^2) like every other
    R = {"p.y": np.array([[0.0]]), "p.y.b": np.array([10.0]), "p.x": np.array([[1.0]]), "p.x.b": np.array([0.0]),
         "p.conv": np.array([[1.0]]), "p.conv.b": np.array([0.0]), "p.ra": np.array([[[0.0]]]), "p.ra.b": np.array([[0.0]]),
         "p.ri": np.array([[[0.0]]]), "p.ri.b": np.array([[50.0]]), "p.lam": np.array([0.0]), "p.o": np.array([[1.0]])}
    lru = plain.GatedLinearRecurrence({"width": 1, "blocks": 1, "conv": 1}, R, "p.")
    a = np.exp(-8.0 * 0.5 * np.log(2.0))
    first = lru.step(np.array([2.0]), 0)
    assert first[0] == pytest.approx(np.sqrt(1 - a * a) * 2.0 * plain.gelu_tanh(np.array([10.0]))[0], rel=1e-9)
    second = lru.step(np.array([0.0]), 1)
    assert second[0] == pytest.approx(a * first[0], rel=1e-9)
    # a window of 2 sees itself and one token back
    A = {"p.q": np.eye(2), "p.k": np.eye(2), "p.v": np.eye(2), "p.q.norm": np.ones(2), "p.k.norm": np.ones(2), "p.o": np.eye(2)}
    att = plain.WindowAttention({"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.0, "mask": {"size": 2}}, A, "p.", 0.0)
    outs = [att.step(np.array(h), i) for i, h in enumerate(([1.0, 0.0], [0.0, 1.0], [4.0, 4.0]))]
    assert np.allclose(outs[1], [0.5, 0.5]) and np.allclose(outs[2], [2.0, 2.5])      # the first token has left the window
