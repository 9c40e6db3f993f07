"""Rodelorn on the GPU against the plain implementation (tests/plain_rodelorn.py): every mechanism alone with inputs
made so that a fault shows, then whole models through the step function in every cut (whole, a long tail decoded
token by token, portions down to two tokens, mixed batches over a pool so small that pages and slots are used
again), in 32-bit and in bfloat16, and greedy generation through the engine's entry point and scheduler."""

import os
import subprocess

import numpy as np
import pytest
import torch

import plain_rodelorn as plain
from replay_util import (ROOT, compare, plan_chunks, plan_many_rows, plan_mixed, plan_tail, plan_whole, random_requests,
                         run_plan_in_process, run_plan_trace_run)
from rodelorn_configs import ONE_KIND, RODELORN

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# float32: (absolute, relative to the row's largest logit) on every logit. bfloat16: the spread of a row's difference
# against the spread of its logits, (bound of the median row, bound of every row); rounding alone gives 0.015 to 0.02 at
# the median row and up to 0.15 at the worst row of the worst-conditioned of the three models.
TOL = {"float32": (2e-5, 2e-5), "bfloat16": (0.04, 0.3)}
SPREAD = {"float32": False, "bfloat16": True}
LENGTHS = {"oa": [5, 70, 150, 33, 260, 129], "ob": [1, 7, 64, 100, 129, 40], "oc": [3, 48, 95, 200, 16, 131]}
SIZES = [16, 7, 2, 5, 3, 2, 11, 32, 2, 9, 64, 2]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """dtype -> name -> model folder whose file holds that dtype."""
    from dynalm_b200.weights import write_model_folder
    out = {"float32": {}, "bfloat16": {}}
    for name, (cfg, seed) in RODELORN.items():
        for dtype, t in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            d = tmp_path_factory.mktemp(f"rodelorn_{name}_{dtype}")
            write_model_folder(str(d), cfg, seed, dtype=t)
            out[dtype][name] = str(d)
    return out


@pytest.fixture(scope="module")
def plain_logits(folders):
    made = {}

    class Lookup:
        def __getitem__(self, key):
            name, dtype = key
            if key not in made:
                reqs = random_requests(RODELORN[name][0]["vocab"], LENGTHS[name], seed=71 + len(made))
                model = plain.PlainRodelorn(folders[dtype][name])
                made[key] = (reqs, {r: model.logits(t) for r, t in reqs.items()})
            return made[key]
    return Lookup()


def _built(folder, dtype, kv_tokens, max_batch, max_requests=8):
    from dynalm_b200.engine import build
    return build(folder, dtype=dtype, kv_tokens=kv_tokens, max_batch_tokens=max_batch, max_requests=max_requests,
                 context=max(kv_tokens, 256))


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV, dtype)


def _np(t):
    return t.double().cpu().numpy()


def _ints(v):
    return torch.tensor(list(v), dtype=torch.int32, device=DEV)


def _step_arrays(portions, slots):
    """The step's index arrays for requests that bring (first position, tokens) each, in state slots `slots`."""
    positions, row_request, row_slot, q_start, pos_start = [], [], [], [0], []
    for r, ((first, n), slot) in enumerate(zip(portions, slots)):
        positions += list(range(first, first + n))
        row_request += [r] * n
        row_slot += [slot] * n
        q_start.append(q_start[-1] + n)
        pos_start.append(first)
    return _ints(positions), _ints(row_request), _ints(row_slot), _ints(q_start), _ints(pos_start), _ints(slots)


def _close(got, want, tol, what=""):
    err = np.abs(got - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), f"{what}: {err:.3g}"


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,channels,col0,act,biased", [(4, 40, 3, "silu", False), (3, 64, 16, "none", True),
                                                           (1, 16, 8, "none", True), (2, 7, 3, "silu", False),
                                                           (5, 300, 3, "none", True)])
def test_short_convolution_in_portions(dtype, taps, channels, col0, act, biased):
    """Two requests cut differently (portions shorter than, equal to and longer than the taps) in one batch, with and
    without an activation, a bias on the result and a bias on every real input; a slot that is used again."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(taps * 100 + channels)
    extra = 2 if col0 % 8 else 8
    w = _t(rng.randn(channels, taps))
    b = _t(rng.randn(channels)) if biased else None
    ib = _t(rng.randn(channels)) if biased else None
    keep_off = 11
    state = torch.zeros(4, keep_off + (taps - 1) * channels + 5, device=DEV)
    state[:, :keep_off] = 7.0
    seqs = {2: rng.randn(23, channels), 0: rng.randn(17, channels)}
    cuts = {2: [1, 1, 2, 3, 4, 5, 1, 6], 0: [5, 1, 1, 1, 2, 7]}

    def ref(u):
        y = plain.causal_conv(_np(_t(u, dtype)), _np(w), _np(b) if biased else None, _np(ib) if biased else None)
        return plain.silu(y) if act == "silu" else y

    def run(batch):
        rows = sum(n for _, _, n in batch)
        proj = torch.zeros(rows, col0 + channels + extra, dtype=dtype, device=DEV)
        r0 = 0
        for s, first, n in batch:
            proj[r0:r0 + n, col0:col0 + channels] = _t(seqs[s][first:first + n], dtype)
            r0 += n
        pos, rreq, rslot, q_start, pos_start, slots = _step_arrays([(f, n) for _, f, n in batch], [s for s, _, _ in batch])
        out = torch.zeros(rows, channels, dtype=dtype, device=DEV)
        ops.short_conv(proj, col0, channels, w.t().contiguous(), b, state, keep_off, pos, rreq, rslot, pos_start, out,
                       act=act, in_bias=ib)
        ops.ssm_conv_keep(proj, col0, channels, taps, state, keep_off, q_start, slots, len(batch))
        return out

    want = {s: ref(u) for s, u in seqs.items()}
    at = {2: 0, 0: 0}
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for k in range(8):
        batch = [(s, at[s], cuts[s][k]) for s in (2, 0) if k < len(cuts[s])]
        out = run(batch)
        r0 = 0
        for s, first, n in batch:
            _close(_np(out[r0:r0 + n]), want[s][first:first + n], tol, f"slot {s} at {first}")
            r0 += n
            at[s] += n
    assert (state[:, :keep_off] == 7.0).all() and (state[1][keep_off:] == 0).all() and (state[3][keep_off:] == 0).all()
    if taps > 1:                                      # what is kept are the raw inputs, oldest first, without the bias
        last = _np(_t(seqs[2][-(taps - 1):], dtype)).reshape(-1)
        assert np.array_equal(_np(state[2, keep_off:keep_off + (taps - 1) * channels]), last)
    state[2, keep_off:] = 0                           # the slot is handed out again
    seqs[2] = rng.randn(3, channels)
    _close(_np(run([(2, 0, 3)])), ref(seqs[2]), tol, "a slot used again")


def _delta_inputs(rng, n, H, G, d, e, dtype):
    """(u rows [q | k | v], raw b and a) of one sequence, rounded to the dtype."""
    u = rng.randn(n, 2 * G * d + H * e) * 0.8
    u[0] *= 5.0                                        # what the first token writes is seen by every later one
    ba = rng.randn(n, 2 * H)
    return _np(_t(u, dtype)), _np(_t(ba, dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e", [(4, 2, 16, 24), (5, 1, 20, 12), (3, 3, 32, 8), (2, 2, 128, 64), (2, 1, 200, 40),
                                     (1, 1, 3, 5), (4, 4, 64, 64), (2, 1, 300, 16)])
def test_delta_rule_in_portions_keeps_its_state(dtype, H, G, d, e):
    """Two requests cut differently in one batch against the plain rule over each whole sequence. The first head
    forgets almost nothing, so a state that is lost, or started anew at a portion's first token, shows at every
    later token; the last head forgets quickly. Then a slot is used again."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H * 1000 + d + e)
    qk, inner = G * d, H * e
    lengths = {1: 45, 3: 21}
    cuts = {1: [1, 2, 9, 8, 1, 1, 17, 6], 3: [7, 1, 1, 2, 10]}
    a_log = rng.randn(H) * 0.3
    a_log[0] = -7.0
    a_log[-1] = 1.0 if H > 1 else -7.0
    dt_bias = rng.randn(H) * 0.3
    seqs, want = {}, {}
    for s, n in lengths.items():
        u, ba = _delta_inputs(rng, n, H, G, d, e, dtype)
        seqs[s] = (u, ba)
        want[s], _ = plain.delta_rule_scan(u[:, :qk].reshape(n, G, d), u[:, qk:2 * qk].reshape(n, G, d),
                                           u[:, 2 * qk:].reshape(n, H, e), ba[:, :H], ba[:, H:], a_log, dt_bias)
    tail = 9
    state = torch.zeros(5, H * d * e + tail, device=DEV)
    state[:, H * d * e:] = 3.0
    b_col = 3
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    at = {1: 0, 3: 0}
    for k in range(8):
        batch = [(s, at[s], cuts[s][k]) for s in (3, 1) if k < len(cuts[s])]
        rows = sum(n for _, _, n in batch)
        u = torch.cat([_t(seqs[s][0][f:f + n], dtype) for s, f, n in batch])
        proj = torch.zeros(rows, b_col + 2 * H + 2, dtype=dtype, device=DEV)
        proj[:, b_col:b_col + 2 * H] = torch.cat([_t(seqs[s][1][f:f + n], dtype) for s, f, n in batch])
        _, _, _, q_start, _, slots = _step_arrays([(f, n) for _, f, n in batch], [s for s, _, _ in batch])
        o = torch.zeros(rows, inner, device=DEV)
        ops.delta_rule(u, 0, qk, 2 * qk, proj, b_col, b_col + H, _t(a_log), _t(dt_bias), state, q_start, slots, o,
                       len(batch), H, G, d, e)
        r0 = 0
        for s, first, n in batch:
            _close(_np(o[r0:r0 + n]), want[s][first:first + n].reshape(n, inner), tol, f"slot {s}, tokens {first}..{first + n - 1}")
            r0 += n
            at[s] += n
    assert (state[:, H * d * e:] == 3.0).all() and (state[0][:H * d * e] == 0).all() and (state[2][:H * d * e] == 0).all()
    state[1, :H * d * e] = 0                           # the slot is handed out again
    u, ba = _delta_inputs(rng, 6, H, G, d, e, dtype)
    ref, S = plain.delta_rule_scan(u[:, :qk].reshape(6, G, d), u[:, qk:2 * qk].reshape(6, G, d), u[:, 2 * qk:].reshape(6, H, e),
                                   ba[:, :H], ba[:, H:], a_log, dt_bias)
    proj = torch.zeros(6, b_col + 2 * H + 2, dtype=dtype, device=DEV)
    proj[:, b_col:b_col + 2 * H] = _t(ba, dtype)
    o = torch.zeros(6, inner, device=DEV)
    ops.delta_rule(_t(u, dtype), 0, qk, 2 * qk, proj, b_col, b_col + H, _t(a_log), _t(dt_bias), state, _ints([0, 6]),
                   _ints([1]), o, 1, H, G, d, e)
    _close(_np(o), ref.reshape(6, inner), tol, "a slot used again")
    _close(_np(state[1, :H * d * e]), S.reshape(-1), tol, "the state that is left")


def test_delta_rule_reads_what_the_token_wrote():
    """One token from an empty state with beta = 1 and no decay: S = k v^T with k a unit vector, so the read-out with
    q = k is v / sqrt(d). A read-out before the write would give zero."""
    from dynalm_b200.kernels import ops
    H, G, d, e = 2, 1, 8, 4
    u = torch.zeros(1, 2 * G * d + H * e, device=DEV)
    u[0, 2] = 3.0                                      # q
    u[0, G * d + 2] = 5.0                              # k, the same direction
    v = torch.arange(1, H * e + 1, device=DEV, dtype=torch.float32)
    u[0, 2 * G * d:] = v
    proj = torch.zeros(1, 2 * H, device=DEV)
    proj[0, :H] = 40.0                                 # sigmoid -> 1
    proj[0, H:] = -40.0                                # softplus -> 0: nothing is forgotten
    state = torch.zeros(1, H * d * e, device=DEV)
    o = torch.zeros(1, H * e, device=DEV)
    ops.delta_rule(u, 0, G * d, 2 * G * d, proj, 0, H, torch.zeros(H, device=DEV), torch.zeros(H, device=DEV), state,
                   _ints([0, 1]), _ints([0]), o, 1, H, G, d, e)
    _close(_np(o[0]), _np(v) / np.sqrt(d), 1e-5, "read-out after the write")


@pytest.mark.parametrize("H,G,d,e", [(3, 1, 20, 12), (2, 2, 128, 40), (4, 2, 48, 70)])
def test_delta_rule_steps_of_single_tokens(H, G, d, e):
    """Steps with no more rows than requests take the kernel for single tokens: three requests decode side by side
    from states that a prompt left, then a step in which one request brings nothing and another brings two tokens
    (as many rows as requests all the same), against the plain rule over each whole sequence."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(d + e)
    qk, inner = G * d, H * e
    a_log, dt_bias = rng.randn(H) * 0.3, rng.randn(H) * 0.3
    a_log[0] = -7.0
    n, prompt = 14, 5
    seqs, want = {}, {}
    for s in (0, 2, 3):
        seqs[s] = _delta_inputs(rng, n, H, G, d, e, torch.float32)
        u, ba = seqs[s]
        want[s], _ = plain.delta_rule_scan(u[:, :qk].reshape(n, G, d), u[:, qk:2 * qk].reshape(n, G, d),
                                           u[:, 2 * qk:].reshape(n, H, e), ba[:, :H], ba[:, H:], a_log, dt_bias)
    state = torch.zeros(4, H * d * e, device=DEV)

    def step(batch):                                   # [(slot, first, count)]
        rows = sum(c for _, _, c in batch)
        u = torch.cat([_t(seqs[s][0][f:f + c]) for s, f, c in batch if c] or [torch.zeros(0, 2 * qk + inner, device=DEV)])
        proj = torch.cat([_t(seqs[s][1][f:f + c]) for s, f, c in batch if c])
        starts = np.cumsum([0] + [c for _, _, c in batch])
        o = torch.zeros(rows, inner, device=DEV)
        ops.delta_rule(u, 0, qk, 2 * qk, proj, 0, H, _t(a_log), _t(dt_bias), state, _ints(starts), _ints([s for s, _, _ in batch]),
                       o, len(batch), H, G, d, e)
        for (s, f, c), r0 in zip(batch, starts):
            if c:
                _close(_np(o[r0:r0 + c]), want[s][f:f + c].reshape(c, inner), 3e-5, f"slot {s}, tokens {f}..{f + c - 1}")

    step([(s, 0, prompt) for s in (3, 0, 2)])
    for t in range(prompt, 10):
        step([(s, t, 1) for s in (2, 3, 0)])
    step([(0, 10, 1), (3, 10, 0), (2, 10, 2)])         # three rows, three requests
    step([(3, 10, 1), (0, 11, 1)])
    assert (state[1] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,e", [(4, 24), (3, 8), (2, 64), (5, 12), (1, 100)])
def test_head_norm_with_gate(dtype, H, e):
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H + e)
    rows, col = 9, 5
    o = _t(rng.randn(rows, H * e) * rng.uniform(0.01, 30.0, size=(rows, 1)))
    gate = torch.zeros(rows, col + H * e + 3, dtype=dtype, device=DEV)
    gate[:, col:col + H * e] = _t(rng.randn(rows, H * e) * 2.0, dtype)
    w = _t(1.0 + 0.3 * rng.randn(e))
    out = torch.zeros(rows, H * e, dtype=dtype, device=DEV)
    ops.head_norm_gate(o, gate, col, w, 1e-5, out, H, e)
    want = plain.head_norm_gate(_np(o).reshape(rows, H, e), _np(gate[:, col:col + H * e]).reshape(rows, H, e), _np(w), 1e-5)
    _close(_np(out), want.reshape(rows, H * e), 1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,blocks", [(48, 3), (40, 1), (36, 4), (128, 2), (6, 6), (300, 5)])
def test_gated_linear_recurrence_in_portions(dtype, width, blocks):
    """Gates by blocks of square matrices, then the scan of two requests cut differently in one batch. The first
    channel forgets almost nothing (a lost state shows at every later token), the last forgets at once; the first
    token of a sequence is scaled like every other (from a state of zeros)."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(width + blocks)
    nb = width // blocks
    ra, ri = rng.randn(blocks, nb, nb) * 0.5, rng.randn(blocks, nb, nb) * 0.5
    ra_b, ri_b = rng.randn(blocks, nb) * 0.5, rng.randn(blocks, nb) * 0.5
    lam = rng.randn(width)
    lam[0], lam[-1] = -9.0, 6.0
    y_bias = rng.randn(width)
    lengths = {2: 37, 0: 19}
    cuts = {2: [1, 2, 9, 8, 1, 1, 15], 0: [7, 1, 1, 2, 8]}
    y_col, keep = 3, 4
    state = torch.zeros(4, width + keep, device=DEV)
    state[:, width:] = 5.0
    seqs, want = {}, {}
    for s, n in lengths.items():
        u = _np(_t(rng.randn(n, width) * 1.5, dtype))
        y = _np(_t(rng.randn(n, width), dtype))
        a, m = plain.rglru_gates(u, ra, ra_b, ri, ri_b, lam)
        seqs[s] = (u, y)
        want[s] = plain.linear_scan(a, m) * plain.gelu_tanh(y + y_bias)
        assert abs(plain.linear_scan(a, m)[0] - m[0]).max() == 0.0
    args = (_t(np.transpose(ra, (0, 2, 1))), _t(ra_b.reshape(-1)), _t(np.transpose(ri, (0, 2, 1))), _t(ri_b.reshape(-1)), _t(lam))
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    at = {2: 0, 0: 0}
    for k in range(7):
        batch = [(s, at[s], cuts[s][k]) for s in (0, 2) if k < len(cuts[s])]
        rows = sum(n for _, _, n in batch)
        u = torch.cat([_t(seqs[s][0][f:f + n], dtype) for s, f, n in batch]).contiguous()
        y = torch.zeros(rows, y_col + width + 1, dtype=dtype, device=DEV)
        y[:, y_col:y_col + width] = torch.cat([_t(seqs[s][1][f:f + n], dtype) for s, f, n in batch])
        a = torch.zeros(rows, width, device=DEV)
        m = torch.zeros(rows, width, device=DEV)
        ops.rglru_gates(u, *args, 8.0, a, m)
        _, _, _, q_start, _, slots = _step_arrays([(f, n) for _, f, n in batch], [s for s, _, _ in batch])
        out = torch.zeros(rows, width, dtype=dtype, device=DEV)
        ops.rglru_scan(a, m, y, y_col, _t(y_bias), state, q_start, slots, out, len(batch))
        r0 = 0
        for s, first, n in batch:
            _close(_np(out[r0:r0 + n]), want[s][first:first + n], tol, f"slot {s}, tokens {first}..{first + n - 1}")
            r0 += n
            at[s] += n
    assert (state[:, width:] == 5.0).all() and (state[1][:width] == 0).all() and (state[3][:width] == 0).all()


def _paged(n_tokens, page, record, dtype, seed, slots=3, slot=1):
    """An empty cache [pages, page, record] with a shuffled block table whose row `slot` covers n_tokens."""
    blocks = -(-n_tokens // page)
    rng = np.random.RandomState(seed)
    pages = rng.permutation(blocks + 5)[:blocks].astype(np.int32)
    table = np.full((slots, blocks + 2), -1, dtype=np.int32)
    table[slot, :blocks] = pages
    cache = torch.zeros(blocks + 5, page, record, dtype=dtype, device=DEV)
    return cache, torch.from_numpy(table).to(DEV), pages


def _records(cache, pages, page, n):
    """The first n tokens' records of a paged cache, in order of position."""
    return torch.cat([cache[int(pg)] for pg in pages])[:n]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e,rot,base,factor,normed", [(4, 2, 32, 16, 8, 1e4, 4.0, True), (6, 2, 16, 16, 6, 500.0, 1.0, True),
                                                            (3, 3, 16, 16, 0, 1.0, 1.0, True), (4, 1, 64, 64, 64, 1e6, 1.0, True),
                                                            (2, 2, 16, 48, 16, 1e4, 2.0, False), (1, 1, 48, 8, 2, 7.0, 3.0, True),
                                                            (3, 1, 24, 24, 10, 1e4, 1.0, True), (2, 2, 7, 5, 6, 100.0, 1.0, True)])
def test_whole_projection_norm_rotation_and_records(dtype, H, G, d, e, rot, base, factor, normed):
    """One statistic over all of q and one over all of k (heads of very unequal size, so that a statistic per head
    shows), plain weights, the first `rot` numbers of every head turned in pairs (i, i + rot / 2) by position over
    the factor, the rest untouched; keys and values land at their position's place in shuffled pages."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H * 100 + d + rot)
    page, n, first, slot = 16, 41, 23, 1
    qw, kw, vw = H * d, G * d, G * e
    x = rng.randn(n, qw + kw + vw + 5)
    x[:, :d] *= 20.0                                                   # the first heads of q and k are far larger
    x[:, qw:qw + d] *= 20.0
    proj = _t(x, dtype)
    x = _np(proj)
    wq, wk = 1.0 + 0.3 * rng.randn(qw), 1.0 + 0.3 * rng.randn(kw)
    positions = list(range(first, first + n))
    inv_freq = _t(base ** (-2.0 * np.arange(rot // 2) / rot)) if rot else None
    cache, table, pages = _paged(first + n, page, kw + vw, dtype, seed=3)
    ops.qk_proj_norm_cache(proj, _t(wq) if normed else None, _t(wk) if normed else None, 1e-5, normed, inv_freq, rot,
                           1.0 / factor, _ints(positions), _ints([slot] * n), table, cache, kw + vw,
                           cache.view(-1)[kw:], kw + vw, H, G, d, e, page)
    want_q = plain.projection_norm_rotate(x[:, :qw], wq if normed else None, 1e-5, H, positions, rot, base, factor)
    want_k = plain.projection_norm_rotate(x[:, qw:qw + kw], wk if normed else None, 1e-5, G, positions, rot, base, factor)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    _close(_np(proj[:, :qw]), want_q.reshape(n, qw), tol, "q")
    rec = _np(_records(cache, pages, page, first + n))
    _close(rec[first:, :kw], want_k.reshape(n, kw), tol, "k in the cache")
    assert np.array_equal(rec[first:, kw:], x[:, qw + kw:qw + kw + vw]), "v in the cache"
    assert not rec[:first].any() and np.array_equal(_np(proj[:, qw:]), x[:, qw:]), "nothing else is written"
    if rot < d and not normed:
        assert np.array_equal(_np(proj[:, :qw]).reshape(n, H, d)[:, :, rot:], x[:, :qw].reshape(n, H, d)[:, :, rot:]), \
            "numbers behind the rotated ones pass unchanged"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e,window", [(4, 2, 32, 16, 20), (6, 2, 16, 16, 7), (3, 3, 16, 16, 0), (4, 1, 64, 64, 64),
                                            (2, 2, 16, 48, 33), (2, 1, 48, 8, 1), (8, 2, 128, 128, 130), (3, 1, 24, 24, 9),
                                            (2, 2, 40, 20, 0), (2, 1, 7, 5, 4)])
def test_windowed_attention_with_a_key_made_to_stand_out(dtype, H, G, d, e, window):
    """Every query gets one key at a distance of its own whose score is made to stand out: the newest key, the oldest
    key that the window still holds, the one just outside it (which must NOT be seen), a page's last and first
    token, the sequence's first token and one hundreds of tokens back. Queries are a portion of a prompt and a single
    decoded token; values of that key are made large, so that seeing it or not decides the output."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H + d + window)
    page, T, slot = 16, 437, 1
    kw, vw = G * d, G * e
    keys = rng.randn(T, G, d) * 0.3
    values = rng.randn(T, G, e)
    scale = 0.37
    cases = []                                                       # (query position, distance to its marked key)
    w = window if window else T
    for p in (T - 1, T - 2, 300, 255, 256, 64, 40, 17):
        for dist in (0, 1, w - 1, w, w + 1, p, p - p % page, p - p % page + 1, p % page, p % page + 1):
            if 0 <= dist <= p:
                cases.append((p, dist))
    cases = sorted(set(cases))
    marked = {}
    for i, (p, dist) in enumerate(cases):                            # one mark per key position; later cases yield
        marked.setdefault(p - dist, i)
    q = rng.randn(len(cases), H, d) * 0.3
    for j, i in marked.items():                                       # a direction of its own for every marked pair
        direction = rng.randn(d)
        direction *= 6.0 / np.linalg.norm(direction)
        keys[j] += direction
        q[i] += direction
        values[j] *= 9.0
    keys_t, values_t, q_t = _t(keys, dtype), _t(values, dtype), _t(q, dtype)
    same = d == e
    if same:
        k_cache, table, pages = _paged(T, page, kw, dtype, seed=9)
        v_cache = torch.zeros_like(k_cache)
        args = (k_cache, kw, v_cache, vw)
        for b, pg in enumerate(pages):
            nn = min(page, T - b * page)
            k_cache[int(pg), :nn] = keys_t[b * page:b * page + nn].reshape(nn, kw)
            v_cache[int(pg), :nn] = values_t[b * page:b * page + nn].reshape(nn, vw)
    else:
        cache, table, pages = _paged(T, page, kw + vw, dtype, seed=9)
        args = (cache, kw + vw, cache.view(-1)[kw:], kw + vw)
        for b, pg in enumerate(pages):
            nn = min(page, T - b * page)
            cache[int(pg), :nn, :kw] = keys_t[b * page:b * page + nn].reshape(nn, kw)
            cache[int(pg), :nn, kw:] = values_t[b * page:b * page + nn].reshape(nn, vw)
    positions = [p for p, _ in cases]
    out = torch.zeros(len(cases), H * e, dtype=dtype, device=DEV)
    ops.paged_attention_generic_kv(q_t.reshape(len(cases), H * d).contiguous(), *args, table, _ints(positions),
                                   _ints([slot] * len(cases)), out, H, G, d, e, page, scale, window)
    want = plain.window_attention(_np(q_t), _np(keys_t), _np(values_t), positions, scale, window)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for i, (p, dist) in enumerate(cases):
        _close(_np(out[i]), want[i].reshape(-1), tol, f"query at {p}, marked key {dist} back")
    one = torch.zeros(1, H * e, dtype=dtype, device=DEV)              # a decoded token alone gives the same row
    ops.paged_attention_generic_kv(q_t[-1:].reshape(1, H * d).contiguous(), *args, table, _ints(positions[-1:]), _ints([slot]),
                                   one, H, G, d, e, page, scale, window)
    _close(_np(one[0]), want[-1].reshape(-1), tol, "alone")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,parts", [(1, 96, 1), (7, 100, 3), (40, 128, 2), (3, 2048, 1), (5, 6, 1)])
def test_norm_behind_a_sublayer_joins_the_sum_and_the_next_norm(dtype, rows, width, parts):
    """x <- x + norm(delta) * w_post with the sum in 32-bit, then the next sublayer's input norm(x) * w_pre from the
    same pass; delta may come as partial sums of a split product. Rows of very unequal size share nothing."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(rows + width)
    x = rng.randn(rows, width) * rng.uniform(0.01, 50.0, size=(rows, 1))
    delta = rng.randn(parts, rows, width) * rng.uniform(0.01, 50.0, size=(1, rows, 1))
    w_post, w_pre = 1.0 + 0.3 * rng.randn(width), 1.0 + 0.3 * rng.randn(width)
    xt = _t(x)
    dt = _t(delta, dtype if parts == 1 else torch.float32)
    out = torch.zeros(rows, width, dtype=dtype, device=DEV)
    ops.norm_add_norm(xt, dt if parts > 1 else dt[0], _t(w_post), 1e-5, _t(w_pre), 2e-6, out)
    want_x = _np(_t(x)) + plain.rms_norm(_np(dt).sum(0), 1e-5, w_post)
    _close(_np(xt), want_x, 1e-5, "the sum")
    assert xt.dtype == torch.float32
    _close(_np(out), plain.rms_norm(want_x, 2e-6, w_pre), 1e-5 if dtype == torch.float32 else 2e-2, "the next norm")
    xt2 = _t(x)
    ops.norm_add_norm(xt2, dt if parts > 1 else dt[0], _t(w_post), 1e-5)        # the last sublayer: no norm follows
    assert torch.equal(xt2, xt)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_gates(dtype):
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(4)
    rows, inner = 7, 52
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    gu = _t(rng.randn(rows, 2 * inner) * 3.0, dtype)
    out = torch.zeros(rows, inner, dtype=dtype, device=DEV)
    ops.gelu_mul(gu, out)
    _close(_np(out), plain.gelu_tanh(_np(gu[:, :inner])) * _np(gu[:, inner:]), tol, "gelu(gate) * up")
    wide = _t(rng.randn(rows, 3 + inner + 2) * 3.0, dtype)
    x = _t(rng.randn(rows, inner), dtype)
    x0 = _np(x)
    ops.sigmoid_gate(x, wide[:, 3:])
    _close(_np(x), x0 * plain.sigmoid(_np(wide[:, 3:3 + inner])), tol, "output gate")
    a, b = _t(rng.randn(3, rows, inner)), _t(rng.randn(rows, inner), dtype)
    s = torch.zeros(rows, inner, device=DEV)
    ops.scaled_sum(a, 0.7, b, 1.3, s)
    _close(_np(s), 0.7 * _np(a).sum(0) + 1.3 * _np(b), 1e-5, "the two sides' sum")
    z = _t(rng.randn(rows, inner) * 40.0)
    z0 = _np(z)
    ops.softcap(z, 9.0)
    _close(_np(z), 9.0 * np.tanh(z0 / 9.0), 1e-5, "capped logits")
    assert np.abs(_np(z)).max() <= 9.0 and np.abs(_np(z)).max() > 8.9


# ---------------------------------------------------------------------------------------------
# whole models through the step function
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(RODELORN))
def test_replay_all_cuts(name, dtype, folders, plain_logits):
    reqs, logits = plain_logits[name, dtype]
    tol = TOL[dtype]
    plans = {
        "whole": plan_whole(reqs),
        "tail48": plan_tail(reqs, 48),
        "chunks": plan_chunks(reqs, SIZES),
        "mixed": plan_mixed(reqs, seed=5),
        "mixed2": plan_mixed(reqs, seed=6, max_live=3, decode_tail=20),
    }
    for what, plan in plans.items():
        need = plan.max_live_tokens(64)          # just what the plan needs: pages of finished requests are used again
        built = _built(folders[dtype][name], dtype, need, max(need, 64), max_requests=4)
        got = run_plan_in_process(built.step_fn, plan)
        compare(plan, got, logits, tol[0], tol[1], f"{name}/{dtype}/{what}", spread=SPREAD[dtype])
        assert built.cache.free_pages == built.cache.num_pages, "pages were lost"


def test_layers_follow_the_plain_implementation(folders, monkeypatch):
    """The residual stream behind every layer of a short prompt in 32-bit."""
    from dynalm_b200.engine import launch_memo
    monkeypatch.setattr(launch_memo, "ENABLED", False)
    name = "oa"
    reqs = random_requests(RODELORN[name][0]["vocab"], [29], seed=2)
    model = plain.PlainRodelorn(folders["float32"][name])
    toks = reqs["r0"]
    _, layers = model.logits(toks, layers=True)
    built = _built(folders["float32"][name], "float32", 64, 64, max_requests=1)
    seen = []
    for blk in built.model.blocks:
        def fwd(stream, ctx, cache, owns, orig=blk.forward):
            s = orig(stream, ctx, cache, owns)
            s.flush()
            seen.append(_np(s.x[:len(toks)]))
            return s
        blk.forward = fwd
    run_plan_in_process(built.step_fn, plan_whole(reqs))
    assert len(seen) == len(layers)
    for i, (g, w) in enumerate(zip(seen, layers)):
        _close(g, w, 2e-5, f"layer {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_single_token_rows_beside_a_portion(dtype, folders):
    """A couple of dozen live requests decoding beside portions of long prompts: unequal requests in one batch
    against each alone, with more state slots than the pairs of the other tests use."""
    name = "oa"
    vocab = RODELORN[name][0]["vocab"]
    short = {f"s{k}": v for k, v in random_requests(vocab, [12 + (5 * i) % 29 for i in range(20)], seed=8).items()}
    long = {f"l{k}": v for k, v in random_requests(vocab, [150, 90], seed=9).items()}
    model = plain.PlainRodelorn(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in {**short, **long}.items()}
    plan = plan_many_rows(short, long, seed=3, tail_lo=4, tail_hi=10)
    need = plan.max_live_tokens(64)
    built = _built(folders[dtype][name], dtype, need, 256, max_requests=24)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], f"{name}/{dtype}/many rows", spread=SPREAD[dtype])


@pytest.mark.parametrize("name", sorted(ONE_KIND))
def test_models_of_one_kind_of_layer(name, tmp_path):
    """Delta layers alone (no pages in the cache manager) and pairs alone, whole prompts and a mixed schedule, float32."""
    from dynalm_b200.weights import write_model_folder
    cfg, seed = ONE_KIND[name]
    write_model_folder(str(tmp_path), cfg, seed, dtype=torch.float32)
    reqs = random_requests(cfg["vocab"], [5, 300, 77, 130, 64], seed=3)
    model = plain.PlainRodelorn(str(tmp_path))
    logits = {r: model.logits(t) for r, t in reqs.items()}
    for what, plan in (("whole", plan_whole(reqs)), ("mixed", plan_mixed(reqs, seed=4))):
        need = plan.max_live_tokens(64)
        built = _built(str(tmp_path), "float32", need, max(need, 64), max_requests=4)
        got = run_plan_in_process(built.step_fn, plan)
        compare(plan, got, logits, *TOL["float32"], f"{name}/{what}")
        assert built.cache.free_pages == built.cache.num_pages


@pytest.mark.parametrize("name", ["oa", "oc"])
def test_long_decoding_keeps_its_place(name, folders):
    """300 tokens decoded one by one after a 3-token prompt: every window passes over decoded tokens many times, pages
    behind it are given back while the request lives, and the states of the delta rule, of the linear recurrence and
    of every convolution are carried through every step (also through steps replayed from a captured graph)."""
    dtype = "float32"
    reqs = random_requests(RODELORN[name][0]["vocab"], [303], seed=12)
    model = plain.PlainRodelorn(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_tail(reqs, 300)
    built = _built(folders[dtype][name], dtype, 320, 64, max_requests=2)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], "long decoding")
    assert built.cache.free_pages == built.cache.num_pages


def test_trace_run_replays_a_plan(folders, tmp_path):
    name = "ob"
    reqs = random_requests(RODELORN[name][0]["vocab"], [40, 7, 90], seed=13)
    model = plain.PlainRodelorn(folders["float32"][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_mixed(reqs, seed=2)
    got = run_plan_trace_run(folders["float32"][name], "float32", plan, str(tmp_path), plan.max_live_tokens(64),
                             RODELORN[name][0]["vocab"])
    compare(plan, got, logits, *TOL["float32"], "trace_run")


# ---------------------------------------------------------------------------------------------
# generation through the entry point
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(RODELORN))
def test_greedy_generation_through_the_engine(name, folders):
    from dynalm_b200 import Engine
    folder = folders["float32"][name]
    model = plain.PlainRodelorn(folder)
    reqs = random_requests(RODELORN[name][0]["vocab"], [5, 17, 33, 70], seed=14)
    eng = Engine(folder, dtype="float32", ctx=512, batch=64, max_running=4)
    outs = eng.generate(list(reqs.values()), max_tokens=12)
    for prompt, g in zip(reqs.values(), outs):
        assert g.status == "finished" and len(g.tokens) == 12
        seq = list(prompt) + list(g.tokens)
        rows = model.logits(seq[:-1])
        for i, tok in enumerate(g.tokens):
            row = rows[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - 2e-5, f"token {i}: chose {tok} at {row[tok]:.6f}, best {row.max():.6f}"
    alone = [eng.generate(p, max_tokens=12).tokens for p in reqs.values()]
    assert alone == [g.tokens for g in outs]


def test_few_pages_give_the_same_tokens(folders):
    """An engine whose pool is too small for its requests preempts and recomputes (a state cannot be rewound, so a
    preempted request starts again from its first token), and gives the tokens of a roomy one."""
    from dynalm_b200 import Engine, SchedulerConfig
    name = "ob"                                      # one of its pairs has no window: its pages are never given back
    reqs = list(random_requests(RODELORN[name][0]["vocab"], [40, 90, 17, 100, 64, 33], seed=15).values())

    def run(ctx):
        eng = Engine(folders["float32"][name], dtype="float32", ctx=ctx, batch=128, max_running=8,
                     scheduler=SchedulerConfig(max_running=6, decode_token_budget=8, prefill_token_budget=64,
                                               max_prefill_chunk=32, max_batch_tokens=128))
        out = eng.generate(reqs, max_tokens=40)
        assert eng.built.cache.free_pages == eng.built.cache.num_pages
        return [g.tokens for g in out], eng.scheduler.stats.preemptions

    roomy, p0 = run(4096)
    tight, p1 = run(320)
    assert p0 == 0 and p1 > 0
    assert tight == roomy


def test_command_line_generates(folders):
    proc = subprocess.run([os.path.join(ROOT, "bin", "dynalm"), "run", folders["bfloat16"]["oa"], "--tokens", "5,9,200,31",
                           "-n", "8", "--ctx", "256", "--batch", "64", "--no-stream"], capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(t) for t in proc.stdout.split()]
    assert len(ids) == 8 and all(0 <= t < RODELORN["oa"][0]["vocab"] for t in ids)
    from dynalm_b200 import Engine
    assert Engine(folders["bfloat16"]["oa"], ctx=256, batch=64).generate([5, 9, 200, 31], max_tokens=8).tokens == ids
