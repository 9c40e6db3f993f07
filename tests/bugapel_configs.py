"""Tiny Bugapel configurations for tests: config.json dicts that differ in every size, constant and layer order."""


def attention(heads, kv_heads, dim, vdim, scale, dims=None, base=10000.0, stretch=None):
    """The first make: unit queries and keys per head, one more term of score 0 in the softmax's denominator."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
        if stretch is not None:
            factor, low, high, original = stretch
            m["rot"]["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return m


def attention_2(heads, kv_heads, dim, vdim, scale, window=None, keep_first=0, dims=None, base=10000.0):
    """The second make: biases, interleaved rotation, a window that keeps the first tokens."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
    return m


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def moe(ff, experts, top, scale=1.0, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# Three streams. Values narrower than keys, a rotation of half a head whose frequencies fall into all three ranges of the
# stretching rule, a window a little longer than a page's third with three kept tokens, experts in three groups of which
# two are kept, a linear-attention layer without a feed-forward.
B_A = {"architecture": "Bugapel", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
       "streams": 3, "logit_softcap": 12.0,
       "layers": [
           layer("attention", attention(4, 2, 32, 16, 0.9, dims=16, base=900.0, stretch=(4.0, 1.0, 4.0, 64)),
                 moe(40, 6, 2, 1.3, groups=(3, 2))),
           layer("gla", gla(3, 24, 40, 8.0, 12)),
           layer("attention_2", attention_2(6, 3, 24, 24, 0.2, window=20, keep_first=3, dims=8, base=500.0),
                 moe(24, 4, 1)),
           layer("attention", attention(2, 2, 48, 48, 1.7, dims=48, base=50000.0), moe(40, 6, 3, 0.8, groups=(2, 1))),
           layer("gla", gla(2, 64, 16, 3.0, 5), moe(56, 3, 3, 2.0)),
       ]}

# One stream with weights of its own (a 1 x 1 mix). Odd sizes that defeat every vector path; a window of exactly a page
# with one kept token, one longer than any request, an attention without a rotation, every head with keys of its own,
# all experts chosen, a single expert.
B_B = {"architecture": "Bugapel", "vocab": 257, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
       "streams": 1,
       "layers": [
           layer("attention_2", attention_2(3, 3, 20, 12, 0.3, window=64, keep_first=1, dims=20, base=10000.0),
                 moe(17, 5, 5, 1.0)),
           layer("attention", attention(5, 1, 12, 28, 2.2), moe(33, 1, 1, 0.7)),
           layer("gla", gla(5, 7, 5, 1.0, 3), moe(16, 8, 2, 1.0, groups=(4, 2))),
           layer("attention_2", attention_2(2, 1, 40, 8, 0.15, window=1000, keep_first=5), None),
           layer("attention_2", attention_2(4, 2, 16, 16, 0.25, dims=4, base=77.0), moe(8, 2, 2, 1.1, groups=(2, 2))),
       ]}

# A plain residual stream (no `streams`), no cap, no embedding scale. Heads of 64 and 128 as a served model has them, a
# window of two pages and a half with a page's worth of kept tokens, a wide linear-attention state, and a last layer
# without a feed-forward whose window keeps no first tokens (its pages go back as the window passes).
B_C = {"architecture": "Bugapel", "vocab": 512, "width": 128, "norm": {"eps": 1e-5},
       "layers": [
           layer("gla", gla(2, 128, 64, 16.0, 16), moe(64, 4, 2, 1.0, groups=(2, 1))),
           layer("attention", attention(4, 1, 64, 64, 1.0, dims=32, base=2e5, stretch=(6.0, 1.0, 3.0, 256)),
                 moe(64, 4, 2, 1.5)),
           layer("attention_2", attention_2(2, 2, 128, 128, 0.09, window=160, keep_first=64, dims=128, base=3e5),
                 moe(32, 8, 4, 1.0, groups=(4, 3))),
           layer("attention_2", attention_2(2, 2, 64, 64, 0.12, window=100, dims=32, base=1e4)),
       ]}

BUGAPEL = {"ba": (B_A, 21), "bb": (B_B, 22), "bc": (B_C, 23)}

# models of one kind of layer alone: linear attention keeps no pages at all
ONLY_GLA = {"architecture": "Bugapel", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "streams": 2,
            "layers": [layer("gla", gla(2, 32, 32, 4.0, 8), moe(32, 4, 2, 1.0)), layer("gla", gla(4, 16, 8, 2.0, 4))]}
ONLY_ATTENTION = {"architecture": "Bugapel", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "streams": 2,
                  "layers": [layer("attention", attention(2, 1, 32, 32, 1.0, dims=32)),
                             layer("attention_2", attention_2(2, 2, 32, 16, 0.2, window=7, keep_first=2, dims=16),
                                   moe(32, 2, 1, 1.0))]}
ONE_KIND = {"gla": (ONLY_GLA, 31), "attention": (ONLY_ATTENTION, 32)}
