"""Tiny Rodelorn configurations for tests: config.json dicts that differ in every size, constant and layer order."""


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def attention(heads, kv_heads, dim, vdim, scale, window=None, dims=None, base=10000.0, factor=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def recurrence(width, blocks, conv):
    return {"width": width, "blocks": blocks, "conv": conv}


def pair(left, right, left_scale=None, right_scale=None):
    m = {"left": left, "right": right}
    if left_scale is not None:
        m["left_scale"] = left_scale
    if right_scale is not None:
        m["right_scale"] = right_scale
    return m


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# A pair first, then two delta layers of different sizes, then a pair again. Values narrower than keys (the cache
# holds records [k | v]), a window a little longer than a page, a rotation of a quarter of a head with stretched
# positions, three blocks of gate matrices, unequal scales of the two sides.
_PA = pair(attention(4, 2, 32, 16, 0.21, window=20, dims=8, factor=4.0), recurrence(48, 3, 3), 0.7, 1.3)
O_A = {"architecture": "Rodelorn", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
       "logit_scale": 0.5, "logit_softcap": 9.0, "layers": [
           layer("parallel", _PA, 160),
           layer("delta", delta(4, 2, 16, 24, 3), 160),
           layer("delta_2", delta(3, 3, 32, 8, 2), 160),
           layer("parallel", _PA, 160),
       ]}

# Sizes that defeat every vector path (a width that is no multiple of 8, an odd vocabulary), a delta layer first with
# one query/key head for five heads and a single tap (nothing of the convolution is kept), attention without a window
# and without a rotation whose keys and values have one size that is no multiple of 16, one block of gate matrices, a window shorter than a
# page with a rotation that is no multiple of four numbers, a layer without a feed-forward, no embedding scale, no
# scale and no cap of the logits, no scales of the sides.
O_B = {"architecture": "Rodelorn", "vocab": 257, "width": 100, "norm": {"eps": 3e-5}, "layers": [
    layer("delta", delta(5, 1, 20, 12, 1), 172),
    layer("parallel", pair(attention(3, 3, 24, 24, 0.4), recurrence(40, 1, 2)), None),
    layer("parallel_2", pair(attention(6, 2, 16, 16, 0.3, window=7, dims=6, base=500.0), recurrence(36, 4, 1)), 172),
]}

# Wide pieces: a delta state of 128 rows (a column over several lanes), five taps, attention with one key/value head
# for four heads of 64 whose whole head is rotated, a window of exactly four pages, a large base, values wider than keys
# in a second pair.
O_C = {"architecture": "Rodelorn", "vocab": 272, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
       "logit_scale": 2.0, "logit_softcap": 30.0, "layers": [
           layer("delta", delta(2, 2, 128, 64, 4), 96),
           layer("parallel", pair(attention(4, 1, 64, 64, 0.11, window=64, dims=64, base=1e6), recurrence(96, 4, 5),
                                  1.0, 0.25), 96),
           layer("parallel", pair(attention(2, 2, 40, 48, 0.5, window=33, dims=16, factor=2.0), recurrence(64, 2, 2),
                                  2.0, 1.0), None),
           layer("delta_3", delta(4, 1, 40, 40, 5), 96),
       ]}

RODELORN = {"oa": (O_A, 61), "ob": (O_B, 62), "oc": (O_C, 63)}

# Models of one kind of layer. Delta layers alone keep no pages at all (six taps, values wider than keys in one layer);
# pairs alone keep no state rows of their own (five heads with five key/value heads of 72 numbers of which 36 turn,
# values of 40, a window of three tokens in the second pair, seven taps, no embedding scale and no cap).
_PB = pair(attention(5, 5, 72, 40, 0.2, window=70, dims=36, factor=3.0), recurrence(200, 5, 6), 0.3, 1.7)
ONE_KIND = {
    "only_delta": ({"architecture": "Rodelorn", "vocab": 301, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
                    "logit_softcap": 5.0, "layers": [
                        layer("delta", delta(6, 3, 48, 20, 6), 100),
                        layer("delta_2", delta(2, 1, 24, 56, 2), None),
                        layer("delta", delta(6, 3, 48, 20, 6), 100)]}, 64),
    "only_pairs": ({"architecture": "Rodelorn", "vocab": 333, "width": 120, "norm": {"eps": 1e-5}, "logit_scale": 0.7, "layers": [
        layer("parallel", _PB, 64),
        layer("parallel_2", pair(attention(2, 1, 8, 8, 0.6, window=3, dims=2), recurrence(24, 3, 7)), 64),
        layer("parallel", _PB, None)]}, 65),
}
