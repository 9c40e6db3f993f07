"""Bugapel on the GPU against the plain implementation (tests/plain_bugapel.py): every mechanism alone with inputs made
so that a fault shows, then whole models through the step function in every cut (whole, a long tail decoded token by
token, portions down to two tokens, mixed batches over a pool so small that pages and slots are used again), in 32-bit
and in bfloat16, and greedy generation through the engine's entry point and scheduler."""

import os
import subprocess

import numpy as np
import pytest
import torch

import plain_bugapel as plain
from bugapel_configs import BUGAPEL, ONE_KIND
from replay_util import (ROOT, compare, plan_chunks, plan_many_rows, plan_mixed, plan_tail, plan_whole, random_requests,
                         run_plan_in_process, run_plan_trace_run)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# float32: (absolute, relative to the row's largest logit) on every logit. bfloat16: the spread of a row's difference
# against the spread of its logits, (bound of the median row, bound of every row).
TOL = {"float32": (2e-5, 2e-5), "bfloat16": (0.04, 0.3)}
SPREAD = {"float32": False, "bfloat16": True}
LENGTHS = {"ba": [5, 70, 150, 33, 260, 129], "bb": [1, 7, 64, 100, 129, 40], "bc": [3, 48, 95, 200, 16, 331]}
SIZES = [16, 7, 2, 5, 3, 2, 11, 32, 2, 9, 64, 2]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """dtype -> name -> model folder whose file holds that dtype."""
    from dynalm_b200.weights import write_model_folder
    out = {"float32": {}, "bfloat16": {}}
    for name, (cfg, seed) in BUGAPEL.items():
        for dtype, t in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            d = tmp_path_factory.mktemp(f"bugapel_{name}_{dtype}")
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
                reqs = random_requests(BUGAPEL[name][0]["vocab"], LENGTHS[name], seed=171 + len(made))
                model = plain.PlainBugapel(folders[dtype][name])
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


def _close(got, want, tol, what=""):
    err = np.abs(got - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), f"{what}: {err:.3g}"


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("parts,width", [(1, 72), (3, 96), (4, 256), (8, 40), (2, 1001), (13, 64), (16, 30), (5, 9)])
def test_layer_norm_over_a_stream_of_parts(dtype, parts, width):
    """The first layer's copy of the embedding into every part, the update that a sublayer leaves (plain and as
    partial sums), the weighted read, the gather of wanted rows without a write, and a row with a large mean (the
    variance is taken from the deviations, not from a difference of means)."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(parts * 7 + width)
    rows = 13
    x0 = rng.randn(rows, width)
    x0[3] += 30.0
    w, b = 1.0 + 0.2 * rng.randn(width), 0.3 * rng.randn(width)
    mix, write, read = np.eye(parts) + 0.2 * rng.randn(parts, parts), 1.0 + 0.3 * rng.randn(parts), rng.randn(parts)
    eps = 1e-5
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    streams = torch.zeros(rows, parts * width, device=DEV)
    out = torch.zeros(rows, width, dtype=dtype, device=DEV)
    # every part starts as the embedding
    ops.stream_layer_norm(streams, parts, _t(w), _t(b), eps, out, init=_t(x0), read=_t(read))
    xs = np.stack([x0] * parts, axis=1)                                       # [rows, parts, width]
    _close(_np(streams).reshape(rows, parts, width), xs, 1e-6, "the parts after the copy")
    _close(_np(out), plain.layer_norm(np.einsum("s,rsw->rw", read, xs), w, b, eps), tol, "the first norm")
    # a sublayer's result, as three partial sums, enters through mix and write
    delta = rng.randn(3, rows, width)
    ops.stream_layer_norm(streams, parts, _t(w), None, eps, out, delta=_t(delta), mix=_t(mix), write=_t(write), read=_t(read))
    y = delta.sum(0)
    xs = np.einsum("st,rsw->rtw", mix, xs) + write[None, :, None] * y[:, None, :]
    _close(_np(streams).reshape(rows, parts, width), xs, 2e-5, "the parts after an update")
    _close(_np(out), plain.layer_norm(np.einsum("s,rsw->rw", read, xs), w, None, eps), tol, "the norm after an update")
    # the wanted rows only: nothing is written back, the read is the plain sum
    d2 = _np(_t(rng.randn(rows, width), dtype))
    pick = [11, 0, 3]
    out2 = torch.zeros(3, width, dtype=dtype, device=DEV)
    before = streams.clone()
    ops.stream_layer_norm(streams, parts, _t(w), _t(b), eps, out2, delta=_t(d2, dtype), mix=_t(mix), write=_t(write),
                          rows=_ints(pick))
    assert torch.equal(streams, before)
    xs2 = np.einsum("st,rsw->rtw", mix, xs) + write[None, :, None] * d2[:, None, :]
    _close(_np(out2), plain.layer_norm(xs2.sum(1), w, b, eps)[pick], tol, "the gathered rows")
    total = torch.zeros(rows, width, device=DEV)
    ops.stream_sum(streams, parts, total, delta=_t(d2, dtype), mix=_t(mix), write=_t(write))
    _close(_np(total), xs2.sum(1), 2e-5, "the sum of the parts")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e,rot,interleaved,unit", [(4, 2, 32, 16, 16, False, True), (6, 3, 24, 24, 8, True, False),
                                                          (5, 1, 12, 28, 0, False, True), (3, 3, 20, 12, 20, True, False),
                                                          (2, 1, 128, 64, 128, False, True), (2, 2, 200, 8, 100, True, True)])
def test_rotation_then_norm_per_head_into_shuffled_pages(dtype, H, G, d, e, rot, interleaved, unit):
    """q in place, k and v into the token's place of pages in a shuffled order, at positions up to 100,000; both layouts
    of the pairs, a rotation of part of a head, and the norm of every head by itself after the rotation."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H * 100 + d)
    page, n_pages = 8, 12
    positions = [0, 1, 7, 8, 9, 63, 64, 65, 40, 41]
    offset = 99_990
    rows = len(positions)
    proj0 = _np(_t(rng.randn(rows, H * d + G * (d + e) + 3) * 2.0, dtype))
    proj = _t(proj0, dtype)
    freq = plain.frequencies(777.0, rot, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}) if rot else np.zeros(0)
    # the request sits in slot 1; its block table maps blocks 0..8 and those of the far positions to shuffled pages
    blocks = 99_990 // page + 12
    table = torch.full((3, blocks), -1, dtype=torch.int32, device=DEV)
    order = rng.permutation(n_pages)
    pos_far = [p + (offset if i % 2 else 0) for i, p in enumerate(positions)]
    used = sorted({p // page for p in pos_far})
    assert len(used) <= n_pages
    for j, blk in enumerate(used):
        table[1, blk] = int(order[j])
    record = G * (d + e)
    cache = torch.zeros(n_pages, page, record, dtype=dtype, device=DEV)
    flat = cache.view(-1)
    ops.qk_rot_head_norm_cache(proj, _t(freq.astype(np.float32)) if rot else None, rot, interleaved, unit, 1e-5,
                               _ints(pos_far), _ints([1] * rows), table, cache, record, flat[G * d:], record, H, G, d, e, page)
    f32 = freq.astype(np.float32).astype(np.float64)
    layout = "pairs" if interleaved else "halves"
    q = plain.rotate(proj0[:, :H * d].reshape(rows, H, d), pos_far, f32, layout)
    k = plain.rotate(proj0[:, H * d:H * d + G * d].reshape(rows, G, d), pos_far, f32, layout)
    if unit:
        q, k = plain.unit_rms(q, 1e-5), plain.unit_rms(k, 1e-5)
    # float32 angles at positions of 100,000 carry an error of 100,000 * 2^-24 radians
    tol = 2e-2 if dtype == torch.float32 else 4e-2
    _close(_np(proj[:, :H * d]).reshape(rows, H, d), q, tol, "queries")
    assert np.array_equal(_np(proj[:, H * d:]), proj0[:, H * d:]), "only q is written back"
    for i, p in enumerate(pos_far):
        rec = _np(cache[int(table[1, p // page]), p % page])
        _close(rec[:G * d].reshape(G, d), k[i], tol, f"keys of position {p}")
        assert np.array_equal(rec[G * d:], proj0[i, H * d + G * d:H * d + G * (d + e)]), f"values of position {p}"
    near = [i for i, p in enumerate(pos_far) if p < 1000]
    _close(_np(proj[near, :H * d]).reshape(len(near), H, d), q[near], 2e-5 if dtype == torch.float32 else 3e-2, "near queries")


def _attention_case(rng, n, H, G, d, e, dtype, page, shuffle=True):
    """Random queries, keys and values of one request of n tokens in shuffled pages: (q [n, H*d], records, table)."""
    blocks = -(-n // page)
    order = rng.permutation(blocks + 3) if shuffle else np.arange(blocks + 3)
    table = torch.full((2, blocks + 2), -1, dtype=torch.int32, device=DEV)
    table[1, :blocks] = _ints(order[:blocks])
    q = _np(_t(rng.randn(n, H * d), dtype))
    k = _np(_t(rng.randn(n, G, d), dtype))
    v = _np(_t(rng.randn(n, G, e), dtype))
    cache = torch.zeros(blocks + 3, page, G * (d + e), dtype=dtype, device=DEV)
    for t in range(n):
        cache[int(order[t // page]), t % page] = _t(np.concatenate([k[t].reshape(-1), v[t].reshape(-1)]), dtype)
    return q, k, v, cache, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,e,window,keep,sink", [(4, 2, 32, 16, 20, 3, False), (3, 3, 20, 12, 64, 1, False),
                                                      (8, 2, 48, 32, 0, 0, True), (2, 1, 40, 8, 700, 5, True),
                                                      (2, 2, 128, 128, 160, 64, False), (5, 5, 24, 24, 600, 2, True)])
def test_attention_with_kept_first_tokens_and_a_sink(dtype, H, G, d, e, window, keep, sink):
    """Every query is pointed at one key by a large score: the key just inside the window and the one just outside, the
    last kept token and the first that is not kept, position 0, the query itself, a chunk's first and last place. A key
    that should be hidden changes nothing; one that should be seen takes the whole output. With the sink and small
    scores the extra term of the denominator is a large part of it."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(d * 10 + window)
    n, page = 1100, 16
    q, k, v, cache, table = _attention_case(rng, n, H, G, d, e, dtype, page)
    rows, targets = [], []
    w = window if window > 0 else 10 ** 9
    for i in (0, 1, keep, keep + 1, 511, 512, 513, w - 1, w, w + keep, 1023, 1024, 1099):
        if not 0 <= i < n:
            continue
        for j in (0, keep - 1, keep, i - w, i - w + 1, i, 511, 512, i - 1):
            if 0 <= j <= i:
                rows.append(i)
                targets.append(j)
    qs = q[rows].reshape(len(rows), H, d).copy()
    for r, j in enumerate(targets):
        for h in range(H):
            # a score of 30 (6 with the sink, 1 for its first queries, where the sink is a large part of the denominator)
            score = 30.0 if not sink else (6.0 if rows[r] >= 8 else 1.0)
            qs[r, h] = k[j, h // (H // G)] * (score / max(1e-6, (k[j, h // (H // G)] ** 2).sum()))
    qs = _np(_t(qs, dtype))
    out = torch.zeros(len(rows), H * e, dtype=dtype, device=DEV)
    rec = G * (d + e)
    ops.paged_attention_generic_kv(_t(qs.reshape(len(rows), H * d), dtype), cache, rec, cache.view(-1)[G * d:], rec, table,
                                   _ints(rows), _ints([1] * len(rows)), out, H, G, d, e, page, 1.0, window, keep, sink)
    flash = None
    if dtype == torch.bfloat16 and (d, e) in ops.MASKED_FLASH_SIZES:          # the tensor-core kernel, a tile of one row each
        flash = torch.zeros(len(rows), H * e, dtype=dtype, device=DEV)
        tiles = _ints([x for r, i in enumerate(rows) for x in (1, r, 1, i)])
        ops.masked_flash_attention(_t(qs.reshape(len(rows), H * d), dtype), cache, rec, cache.view(-1)[G * d:], rec, table,
                                   tiles, len(rows), flash, H, G, d, e, page, 1.0, window, keep, sink)
        grouped = torch.zeros(len(rows), H * e, dtype=dtype, device=DEV)      # the heads of a KV head as the rows of a tile
        ops.masked_flash_attention(_t(qs.reshape(len(rows), H * d), dtype), cache, rec, cache.view(-1)[G * d:], rec, table,
                                   tiles, len(rows), grouped, H, G, d, e, page, 1.0, window, keep, sink, one_token_tiles=True)
        _close(_np(grouped), _np(flash), 1e-6, "heads of a group in one block")
        for parts in (2, 5, 8):                                              # a row's key tiles dealt over blocks, then merged
            scratch = torch.zeros(ops.masked_flash_partial_floats(len(rows), H, e, parts), device=DEV)
            dealt = torch.zeros(len(rows), H * e, dtype=dtype, device=DEV)
            ops.masked_flash_attention(_t(qs.reshape(len(rows), H * d), dtype), cache, rec, cache.view(-1)[G * d:], rec, table,
                                       tiles, len(rows), dealt, H, G, d, e, page, 1.0, window, keep, sink, one_token_tiles=True,
                                       parts=parts, partial=scratch)
            for r, (i, j) in enumerate(zip(rows, targets)):
                want = plain.attend(qs[r:r + 1], k[:i + 1], v[:i + 1], [i], list(range(i + 1)), 1.0, window, keep, sink)
                _close(_np(dealt[r]).reshape(1, H, e), want, 2e-2, f"{parts} parts, query {i} pointed at key {j}")
    for r, (i, j) in enumerate(zip(rows, targets)):
        want = plain.attend(qs[r:r + 1], k[:i + 1], v[:i + 1], [i], list(range(i + 1)), 1.0, window, keep, sink)
        _close(_np(out[r]).reshape(1, H, e), want, 2e-5 if dtype == torch.float32 else 2e-2, f"query {i} pointed at key {j}")
        if flash is not None:
            _close(_np(flash[r]).reshape(1, H, e), want, 2e-2, f"flash kernel, query {i} pointed at key {j}")


@pytest.mark.parametrize("H,G,d,e,window,keep,sink", [(4, 2, 32, 16, 20, 3, False), (8, 2, 48, 32, 0, 0, True),
                                                      (2, 2, 128, 128, 160, 64, False), (3, 3, 64, 64, 70, 2, True),
                                                      (2, 1, 96, 48, 64, 65, False), (4, 4, 16, 16, 129, 1, True)])
def test_masked_flash_attention_on_portions(H, G, d, e, window, keep, sink):
    """A prompt in query tiles of up to 128 rows beside a tile that continues another request in the middle of a key
    tile; every query points at a key at one of its edges in turn (the window's first key, the one before it, the last
    kept token, the first that is not kept, position 0, itself)."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(d + window + keep)
    n, page = 333, 16
    q, k, v, cache, table = _attention_case(rng, n, H, G, d, e, torch.bfloat16, page)
    w = window if window > 0 else 10 ** 9
    qs = q.reshape(n, H, d).copy()
    for i in range(n):
        j = [i - w + 1, i - w, keep - 1, keep, 0, i][i % 6]
        if 0 <= j <= i:
            for h in range(H):
                kk = k[j, h // (H // G)]
                qs[i, h] = kk * ((4.0 if sink else 25.0) / max(1e-6, (kk ** 2).sum()))
    qs = _np(_t(qs, torch.bfloat16))
    # the rows of the step: positions 200..332 of the request first (a portion that starts inside a key tile), then 0..199
    order = list(range(200, n)) + list(range(200))
    tiles = [(1, 0, 128, 200), (1, 128, 5, 328), (1, 133, 128, 0), (1, 261, 72, 128)]
    out = torch.zeros(n, H * e, dtype=torch.bfloat16, device=DEV)
    rec = G * (d + e)
    ops.masked_flash_attention(_t(qs[order].reshape(n, H * d), torch.bfloat16), cache, rec, cache.view(-1)[G * d:], rec, table,
                               _ints([x for t in tiles for x in t]), len(tiles), out, H, G, d, e, page, 0.5, window, keep, sink)
    want = plain.attend(qs, k, v, list(range(n)), list(range(n)), 0.5, window, keep, sink)
    _close(_np(out).reshape(n, H, e), want[order], 2e-2, "portions")


def test_a_bias_joins_before_the_rotation():
    """The bias of q | k | v added inside the kernel that turns and norms: equal to a projection that carried it."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(5)
    H, G, d, e, rot, page = 3, 1, 24, 16, 12, 8
    rows = 6
    width = H * d + G * (d + e)
    proj0, bias = rng.randn(rows, width), rng.randn(width)
    freq = _t(plain.frequencies(100.0, rot).astype(np.float32))
    table = _ints(range(4)).view(1, 4)
    outs = []
    for fused in (True, False):
        proj = _t(proj0 if fused else proj0 + bias)
        cache = torch.zeros(4, page, G * (d + e), device=DEV)
        ops.qk_rot_head_norm_cache(proj, freq, rot, True, True, 1e-5, _ints(range(rows)), _ints([0] * rows), table, cache,
                                   G * (d + e), cache.view(-1)[G * d:], G * (d + e), H, G, d, e, page, bias=_t(bias) if fused else None)
        outs.append((_np(proj[:, :H * d]), _np(cache)))
    _close(outs[0][0], outs[1][0], 1e-5, "queries")
    _close(outs[0][1], outs[1][1], 1e-5, "keys and values")


def _gla_inputs(rng, n, H, d, e, dtype):
    u = rng.randn(n, 2 * H * d + H * e) * 0.7
    u[0] *= 4.0                                        # what the first token writes is seen by every later one
    z = rng.randn(n, H * d) * 2.0
    z[:, :d] = 12.0                                    # the first head forgets almost nothing
    z[:, -1] = -12.0                                   # the last channel forgets at once
    return _np(_t(u, dtype)), _np(_t(z))


def _gla_plain(u, z, H, d, e, tau):
    n = u.shape[0]
    S = np.zeros((H, d, e))
    o = np.zeros((n, H, e))
    for t in range(n):
        S, o[t] = plain.linear_attention_step(S, u[t, :H * d].reshape(H, d), u[t, H * d:2 * H * d].reshape(H, d),
                                              u[t, 2 * H * d:].reshape(H, e), z[t].reshape(H, d), tau)
    return o.reshape(n, H * e), S


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,e,tau", [(3, 24, 40, 8.0), (2, 64, 16, 3.0), (5, 7, 5, 1.0), (2, 128, 64, 16.0), (1, 200, 33, 2.0),
                                       (2, 32, 32, 4.0), (1, 300, 8, 5.0), (4, 16, 130, 1.5)])
def test_linear_attention_in_portions_keeps_its_state(dtype, H, d, e, tau):
    """Two requests cut differently in one batch (single tokens, portions longer than a tile) against the plain rule
    over each whole sequence; a state that is lost or started anew shows at every later token of the first head. Then
    the state that is left, the neighbours' rows, and a slot that is used again."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H * 1000 + d + e)
    lengths = {1: 61, 3: 23}
    cuts = {1: [1, 2, 9, 8, 1, 1, 33, 6], 3: [7, 1, 1, 2, 12]}
    seqs = {s: _gla_inputs(rng, n, H, d, e, dtype) for s, n in lengths.items()}
    want = {s: _gla_plain(u, z, H, d, e, tau) for s, (u, z) in seqs.items()}
    tail = 5
    state = torch.zeros(5, H * d * e + tail, device=DEV)
    state[:, H * d * e:] = 3.0
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    at = {1: 0, 3: 0}
    for step in range(8):
        batch = [(s, at[s], cuts[s][step]) for s in (3, 1) if step < len(cuts[s])]
        rows = sum(c for _, _, c in batch)
        proj = torch.zeros(rows, 2 + 2 * H * d + H * e + 1, dtype=dtype, device=DEV)
        proj[:, 2:-1] = torch.cat([_t(seqs[s][0][f:f + c], dtype) for s, f, c in batch])
        z = torch.cat([_t(seqs[s][1][f:f + c]) for s, f, c in batch]).contiguous()
        starts = np.cumsum([0] + [c for _, _, c in batch])
        o = torch.zeros(rows, H * e, device=DEV)
        ops.gla_scan(proj, 2, 2 + H * d, 2 + 2 * H * d, z, tau, d ** -0.5, state, _ints(starts), _ints([s for s, _, _ in batch]), o,
                     len(batch), H, d, e)
        for (s, f, c), r0 in zip(batch, starts):
            _close(_np(o[r0:r0 + c]), want[s][0][f:f + c], tol, f"slot {s}, tokens {f}..{f + c - 1}")
            at[s] += c
    assert (state[:, H * d * e:] == 3.0).all() and (state[0] [:H * d * e] == 0).all() and (state[2][:H * d * e] == 0).all()
    S = _np(state[1, :H * d * e]).reshape(H, e, d).transpose(0, 2, 1)          # kept transposed
    _close(S, want[1][1], tol, "the state that is left")
    state[1, :H * d * e] = 0                           # the slot is handed out again
    u, z = _gla_inputs(rng, 6, H, d, e, dtype)
    proj = torch.zeros(6, 2 + 2 * H * d + H * e + 1, dtype=dtype, device=DEV)
    proj[:, 2:-1] = _t(u, dtype)
    o = torch.zeros(6, H * e, device=DEV)
    ops.gla_scan(proj, 2, 2 + H * d, 2 + 2 * H * d, _t(z), tau, d ** -0.5, state, _ints([0, 6]), _ints([1]), o, 1, H, d, e)
    _close(_np(o), _gla_plain(u, z, H, d, e, tau)[0], tol, "a slot used again")


@pytest.mark.parametrize("H,d,e", [(8, 64, 128), (4, 128, 96)])
def test_linear_attention_of_many_requests_side_by_side(H, d, e):
    """A dozen requests in one step (single tokens, then two or three tokens each): with that many columns in flight the
    kernel lays a column over the fewest lanes, the layout a large decode batch runs with."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(d + e)
    n_req, tau = 24, 4.0
    seqs = [_gla_inputs(rng, 7, H, d, e, torch.float32) for _ in range(n_req)]
    want = [_gla_plain(u, z, H, d, e, tau)[0] for u, z in seqs]
    state = torch.zeros(n_req + 1, H * d * e, device=DEV)
    slots = [(5 * r) % n_req for r in range(n_req)]
    at = 0
    for take in (1, 1, 3, 2):
        proj = torch.cat([_t(u[at:at + take]) for u, _ in seqs])
        z = torch.cat([_t(zz[at:at + take]) for _, zz in seqs]).contiguous()
        o = torch.zeros(n_req * take, H * e, device=DEV)
        ops.gla_scan(proj, 0, H * d, 2 * H * d, z, tau, d ** -0.5, state, _ints(range(0, n_req * take + 1, take)), _ints(slots), o,
                     n_req, H, d, e)
        for r in range(n_req):
            _close(_np(o[r * take:(r + 1) * take]), want[r][at:at + take], 3e-5, f"request {r}, tokens from {at}")
        at += take
    assert (state[n_req] == 0).all()


def test_linear_attention_reads_after_the_write_and_decays_rows():
    """One token from an empty state: o = (q . k) d^(-1/2) v, which a read before the write would leave at zero. A
    second token with k = 0: the state's row of key channel i has decayed by sigmoid(z_i)^(1/tau), whatever the value
    column."""
    from dynalm_b200.kernels import ops
    H, d, e, tau = 1, 8, 4, 2.0
    proj = torch.zeros(2, 2 * d + e, device=DEV)
    proj[0, 2], proj[0, d + 2] = 3.0, 5.0              # q and k along channel 2
    proj[0, d + 5] = 1.0                               # k also along channel 5
    proj[0, 2 * d:] = torch.arange(1, e + 1, device=DEV)
    proj[1, 2], proj[1, 5] = 1.0, 1.0                  # the second token reads channels 2 and 5, writes nothing
    z = torch.zeros(2, d, device=DEV)
    z[1, 2], z[1, 5] = 0.0, 40.0                       # channel 2 halves^(1/tau), channel 5 stays
    state = torch.zeros(1, d * e, device=DEV)
    o = torch.zeros(2, e, device=DEV)
    ops.gla_scan(proj, 0, d, 2 * d, z, tau, d ** -0.5, state, _ints([0, 2]), _ints([0]), o, 1, H, d, e)
    v = np.arange(1, e + 1, dtype=np.float64)
    _close(_np(o[0]), 15.0 * d ** -0.5 * v, 1e-5, "read-out after the write")
    _close(_np(o[1]), (5.0 * 0.5 ** (1 / tau) + 1.0) * d ** -0.5 * v, 1e-5, "decay by key channel")


@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (8, 3, 2, 1), (5, 5, 1, 1), (8, 2, 4, 2), (1, 1, 1, 1), (12, 3, 3, 3),
                                               (64, 6, 8, 3)])
def test_router_picks_experts_of_the_best_groups(E, top, groups, keep):
    """Random logits, and rows made so that the best expert of all sits in a group that loses: a group's score is its
    LARGEST score, so one strong expert keeps its group, and two middling ones do not beat it."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(E * 10 + top)
    rows = 40
    z = rng.randn(rows, E) * 2.0
    per = E // groups
    if groups > keep and per > 1:
        z[0] = -5.0
        z[0, 0] = 4.0                                  # group 0: one strong expert
        z[0, per:2 * per] = 3.0                        # group 1: all middling, a larger sum, a smaller maximum
    logits = _t(z)
    ids = torch.zeros(rows, top, dtype=torch.int32, device=DEV)
    w = torch.zeros(rows, top, device=DEV)
    ops.moe_route(logits, top, groups, keep, 1.7, ids, w)
    for r in range(rows):
        chosen, weights = plain.route(_np(logits[r]), top, groups, keep, 1.7)
        assert [int(i) for i in ids[r]] == chosen, f"row {r}"
        _close(_np(w[r]), weights, 2e-6, f"weights of row {r}")
        assert abs(float(w[r].sum()) - 1.7) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,width,inner,rows", [(6, 2, 96, 40, 50), (4, 1, 64, 32, 7), (5, 5, 72, 17, 33), (8, 3, 256, 128, 300),
                                                    (3, 2, 128, 64, 1), (16, 2, 160, 224, 130), (4, 2, 192, 320, 700)])
def test_experts_over_grouped_pairs(dtype, E, top, width, inner, rows):
    """The whole feed-forward after the router: pairs grouped by expert (some experts get none, one gets more than a
    tile), both products with the squared ReLU between them, the weighted sum in the order of a token's experts."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(E + width)
    x = _np(_t(rng.randn(rows, width), dtype))
    up = _np(_t(rng.randn(E, inner, width) * 0.2, dtype))
    down = _np(_t(rng.randn(E, width, inner) * 0.2, dtype))
    ids = np.stack([rng.permutation(E)[:top] for _ in range(rows)])
    if top == 1 and E > 2:
        ids[ids == E - 1] = 0                          # the last expert idles
    weights = rng.rand(rows, top) + 0.1
    pairs = rows * top
    want = np.zeros((rows, width))
    for r in range(rows):
        for k in range(top):
            want[r] += weights[r, k] * plain.expert(x[r], up[ids[r, k]], down[ids[r, k]])
    wide = dtype == torch.bfloat16 and width % 64 == 0 and inner % 64 == 0
    for tile_rows in ((ops.MOE_TILE_ROWS, ops.MOE_WIDE_TILE_ROWS) if wide else (ops.MOE_TILE_ROWS,)):
        place_of = torch.zeros(pairs, dtype=torch.int32, device=DEV)
        pair_at = torch.zeros(pairs, dtype=torch.int32, device=DEV)
        max_tiles = ops.moe_max_tiles(pairs, E, tile_rows)
        tiles = torch.zeros(3 * max_tiles, dtype=torch.int32, device=DEV)
        n_tiles = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.moe_group(_ints(ids.reshape(-1)), pairs, E, place_of, pair_at, tiles, n_tiles, tile_rows)
        po, pa = place_of.cpu().numpy(), pair_at.cpu().numpy()
        assert sorted(po) == list(range(pairs)) and all(pa[po[p]] == p for p in range(pairs))
        by_place = ids.reshape(-1)[pa]
        assert all(by_place[i] <= by_place[i + 1] for i in range(pairs - 1)), "places run expert by expert"
        nt = int(n_tiles[0])
        assert nt <= max_tiles
        covered = []
        for ex, first, count in tiles[:3 * nt].view(nt, 3).cpu().numpy():
            assert 0 < count <= tile_rows and all(by_place[first:first + count] == ex)
            covered += list(range(first, first + count))
        assert sorted(covered) == list(range(pairs))
        act = torch.zeros(pairs, inner, dtype=dtype, device=DEV)
        ops.moe_linear(_t(x, dtype), pair_at, top, _t(up, dtype), act, tiles, n_tiles, max_tiles, "relu2", tile_rows)
        out = torch.zeros(pairs, width, device=DEV)
        ops.moe_linear(act, None, 1, _t(down, dtype), out, tiles, n_tiles, max_tiles, "none", tile_rows)
        y = torch.zeros(rows, width, dtype=dtype, device=DEV)
        ops.moe_combine(out, place_of, _t(weights), top, y)
        _close(_np(y), want, 3e-5 if dtype == torch.float32 else 3e-2, f"the experts' weighted sum, tiles of {tile_rows}")
        if tile_rows == ops.MOE_WIDE_TILE_ROWS and ops.moe_linear_tcgen05_applies(_t(x, dtype), _t(up, dtype), act):
            # the same on the tcgen05 tensor cores, from rows gathered into the order of their experts
            rows_sorted = torch.zeros(pairs, width, dtype=dtype, device=DEV)
            ops.moe_gather(_t(x, dtype), pair_at, top, rows_sorted)
            assert torch.equal(rows_sorted, _t(x, dtype)[(pair_at // top).long()])
            act2 = torch.zeros(pairs, inner, dtype=dtype, device=DEV)
            ops.moe_linear_tcgen05(rows_sorted, _t(up, dtype), act2, tiles, n_tiles, max_tiles, "relu2")
            out2 = torch.zeros(pairs, width, device=DEV)
            ops.moe_linear_tcgen05(act2, _t(down, dtype), out2, tiles, n_tiles, max_tiles, "none")
            assert ops.gemm_tcgen05_status() == 0
            y2 = torch.zeros(rows, width, dtype=dtype, device=DEV)
            ops.moe_combine(out2, place_of, _t(weights), top, y2)
            _close(_np(y2), want, 3e-2, "the experts' weighted sum on tcgen05")


# ---------------------------------------------------------------------------------------------
# whole models through the step function
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(BUGAPEL))
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


@pytest.mark.parametrize("name", ["ba", "bc"])
def test_layers_follow_the_plain_implementation(name, folders, monkeypatch):
    """The residual stream (the sum of its parts) behind every layer of a short prompt in 32-bit."""
    from dynalm_b200.engine import launch_memo
    monkeypatch.setattr(launch_memo, "ENABLED", False)
    reqs = random_requests(BUGAPEL[name][0]["vocab"], [29], seed=2)
    model = plain.PlainBugapel(folders["float32"][name])
    toks = reqs["r0"]
    _, layers = model.logits(toks, layers=True)
    built = _built(folders["float32"][name], "float32", 64, 64, max_requests=1)
    seen = []
    for blk in built.model.blocks:
        def fwd(stream, ctx, cache, owns, orig=blk.forward):
            import copy
            s = orig(stream, ctx, cache, owns)
            total = torch.zeros_like(s.x)
            if s.streams is not None:
                from dynalm_b200.kernels import ops
                ops.stream_sum(s.streams, s.parts, total, delta=s.pending, mix=s.link.mix, write=s.link.write)
            else:
                c = copy.copy(s)
                total.copy_(s.x)
                c.x = total
                c.flush()
            seen.append(_np(total[:len(toks)]))
            return s
        blk.forward = fwd
    run_plan_in_process(built.step_fn, plan_whole(reqs))
    assert len(seen) == len(layers)
    for i, (g, w) in enumerate(zip(seen, layers)):
        _close(g, w, 2e-5, f"layer {i}")


def test_layers_issued_by_address_equal_layers_run_through_their_parts(folders, monkeypatch):
    """A model whose layers repeat: with the layers after the first of a kind re-issued by address (each with the
    stream weights of the layer in front of it) the logits are bit for bit those of every layer run through its parts."""
    from dynalm_b200.engine import launch_memo
    from dynalm_b200.weights import write_model_folder
    import tempfile
    cfg = dict(BUGAPEL["ba"][0])
    cfg["layers"] = [cfg["layers"][0], cfg["layers"][1]] * 3
    reqs = random_requests(cfg["vocab"], [40, 9], seed=4)
    outs = []
    with tempfile.TemporaryDirectory() as d:
        write_model_folder(d, cfg, 5, dtype=torch.float32)
        for enabled in (True, False):
            monkeypatch.setattr(launch_memo, "ENABLED", enabled)
            before = launch_memo.REPLAYED_LAYERS
            built = _built(d, "float32", 128, 64, max_requests=2)
            outs.append(run_plan_in_process(built.step_fn, plan_chunks(reqs, [16, 3, 2])))
            assert (launch_memo.REPLAYED_LAYERS > before) == enabled
        model = plain.PlainBugapel(d)
        compare(plan_chunks(reqs, [16, 3, 2]), outs[0], {r: model.logits(t) for r, t in reqs.items()}, *TOL["float32"], "repeated layers")
    assert all(np.array_equal(outs[0][k], outs[1][k]) for k in outs[0])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_single_token_rows_beside_a_portion(dtype, folders):
    """A couple of dozen live requests decoding beside portions of long prompts: unequal requests in one batch
    against each alone, with more state slots than the other tests use."""
    name = "ba"
    vocab = BUGAPEL[name][0]["vocab"]
    short = {f"s{k}": v for k, v in random_requests(vocab, [12 + (5 * i) % 29 for i in range(20)], seed=8).items()}
    long = {f"l{k}": v for k, v in random_requests(vocab, [150, 90], seed=9).items()}
    model = plain.PlainBugapel(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in {**short, **long}.items()}
    plan = plan_many_rows(short, long, seed=3, tail_lo=4, tail_hi=10)
    need = plan.max_live_tokens(64)
    built = _built(folders[dtype][name], dtype, need, 256, max_requests=24)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], f"{name}/{dtype}/many rows", spread=SPREAD[dtype])


@pytest.mark.parametrize("name", sorted(ONE_KIND))
def test_models_of_one_kind_of_layer(name, tmp_path):
    """Linear attention alone (no pages in the cache manager) and attention alone, whole prompts and a mixed schedule."""
    from dynalm_b200.weights import write_model_folder
    cfg, seed = ONE_KIND[name]
    write_model_folder(str(tmp_path), cfg, seed, dtype=torch.float32)
    reqs = random_requests(cfg["vocab"], [5, 300, 77, 130, 64], seed=3)
    model = plain.PlainBugapel(str(tmp_path))
    logits = {r: model.logits(t) for r, t in reqs.items()}
    for what, plan in (("whole", plan_whole(reqs)), ("mixed", plan_mixed(reqs, seed=4))):
        need = plan.max_live_tokens(64)
        built = _built(str(tmp_path), "float32", need, max(need, 64), max_requests=4)
        got = run_plan_in_process(built.step_fn, plan)
        compare(plan, got, logits, *TOL["float32"], f"{name}/{what}")
        assert built.cache.free_pages == built.cache.num_pages


@pytest.mark.parametrize("name", ["ba", "bc"])
def test_long_decoding_keeps_its_place(name, folders):
    """300 tokens decoded one by one after a 3-token prompt: every window passes over decoded tokens many times while
    the first tokens stay visible, and the state of every linear-attention head is carried through every step (also
    through steps replayed from a captured graph)."""
    dtype = "float32"
    reqs = random_requests(BUGAPEL[name][0]["vocab"], [303], seed=12)
    model = plain.PlainBugapel(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_tail(reqs, 300)
    built = _built(folders[dtype][name], dtype, 320, 64, max_requests=2)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], "long decoding")
    assert built.cache.free_pages == built.cache.num_pages


def test_trace_run_replays_a_plan(folders, tmp_path):
    name = "bb"
    reqs = random_requests(BUGAPEL[name][0]["vocab"], [40, 7, 90], seed=13)
    model = plain.PlainBugapel(folders["float32"][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_mixed(reqs, seed=2)
    got = run_plan_trace_run(folders["float32"][name], "float32", plan, str(tmp_path), plan.max_live_tokens(64),
                             BUGAPEL[name][0]["vocab"])
    compare(plan, got, logits, *TOL["float32"], "trace_run")


# ---------------------------------------------------------------------------------------------
# generation through the entry point
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(BUGAPEL))
def test_greedy_generation_through_the_engine(name, folders):
    from dynalm_b200 import Engine
    folder = folders["float32"][name]
    model = plain.PlainBugapel(folder)
    reqs = random_requests(BUGAPEL[name][0]["vocab"], [5, 17, 33, 70], seed=14)
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
    name = "ba"
    reqs = list(random_requests(BUGAPEL[name][0]["vocab"], [40, 90, 17, 100, 64, 33], seed=15).values())

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
    proc = subprocess.run([os.path.join(ROOT, "bin", "dynalm"), "run", folders["bfloat16"]["ba"], "--tokens", "5,9,200,31",
                           "-n", "8", "--ctx", "256", "--batch", "64", "--no-stream"], capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(t) for t in proc.stdout.split()]
    assert len(ids) == 8 and all(0 <= t < BUGAPEL["ba"][0]["vocab"] for t in ids)
    from dynalm_b200 import Engine
    assert Engine(folders["bfloat16"]["ba"], ctx=256, batch=64).generate([5, 9, 200, 31], max_tokens=8).tokens == ids
