"""A plain, slow Rodelorn for tests: float64 NumPy, one function per mechanism.

It shares no code with `dynalm_b200`: it reads config.json and model.safetensors by itself. Every mechanism is
written token by token from explicit state (the matrix of a delta-rule head, the vector of a gated linear
recurrence, the last inputs of a short convolution, the keys and values of an attention layer), so a prompt may be
fed in any portions: `PlainRodelorn.logits(tokens)` feeds it whole, `logits(tokens, cuts=[...])` in pieces, and the
two agree to rounding of float64.

Notation. W the stream's width. Delta rule: H heads, G query/key heads of size d, values of size e, K taps.
Attention: H query heads, G key/value heads, key size d, value size e, window w, the first r numbers of a head
rotated. Gated linear recurrence: width R in B blocks, K taps.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


def read_tensors(path: str) -> Dict[str, np.ndarray]:
    """A safetensors file: 8-byte little-endian header length, JSON header, data. Floats come back as float64."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = raw[8 + hlen:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        buf = data[lo:hi]
        if e["dtype"] == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif e["dtype"] == "I32":
            a = np.frombuffer(buf, dtype="<i4").copy()
        else:
            raise ValueError(f"dtype {e['dtype']} of {name}")
        out[name] = a.reshape(e["shape"])
    return out


# --------------------------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------------------------

def rms_norm(x, eps, weight=None):
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y * weight if weight is not None else y


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gated_mlp(h, gate, up, down):
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


class ShortConv:
    """y_t[c] = bias[c] + sum_j taps[c, j] x_(t - (K - 1 - j))[c], zeros before the start. The state is the last
    K - 1 inputs."""

    def __init__(self, taps, bias=None):
        self.taps, self.bias = taps, bias
        self.past = np.zeros((taps.shape[1] - 1, taps.shape[0]))

    def step(self, x):
        rows = np.concatenate([self.past, x[None]], axis=0)          # oldest first, the current token's last
        y = np.einsum("kc,ck->c", rows, self.taps)
        if self.bias is not None:
            y = y + self.bias
        self.past = rows[1:]
        return y


def rotate_half(x, pos, dims, base, factor):
    """The first `dims` numbers of every head (last axis): number i pairs with number i + dims / 2 and the pair
    turns by pos * base^(-2 i / dims) / factor."""
    half = dims // 2
    a = pos * base ** (-2.0 * np.arange(half) / dims) / factor
    c, s = np.cos(a), np.sin(a)
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


class DeltaMixer:
    """The gated delta rule with short convolutions, unit-length queries and keys and a gated norm per head."""

    def __init__(self, m, t, p, eps):
        self.H, self.d = m["heads"], m["dim"]
        self.G, self.e = m.get("kv_heads", self.H), m.get("vdim", self.d)
        self.eps = eps
        self.t = {k[len(p):]: v for k, v in t.items() if k.startswith(p)}
        self.cq, self.ck, self.cv = (ShortConv(self.t[n + ".conv"]) for n in "qkv")
        self.S = np.zeros((self.H, self.d, self.e))

    def step(self, h, pos):
        t, H, G, d, e = self.t, self.H, self.G, self.d, self.e
        q = silu(self.cq.step(t["q"] @ h)).reshape(G, d)
        k = silu(self.ck.step(t["k"] @ h)).reshape(G, d)
        v = silu(self.cv.step(t["v"] @ h)).reshape(H, e)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        beta = sigmoid(t["b"] @ h)
        g = np.exp(-np.exp(t["A_log"]) * softplus(t["a"] @ h + t["dt_bias"]))
        gate = silu(t["g"] @ h).reshape(H, e)
        out = np.zeros((H, e))
        for i in range(H):
            j = i // (H // G)
            S = self.S[i] * g[i]
            u = beta[i] * (v[i] - S.T @ k[j])
            S = S + np.outer(k[j], u)
            self.S[i] = S
            out[i] = rms_norm(S.T @ q[j], self.eps, t["norm"]) * gate[i]
        return t["o"] @ out.reshape(-1)


class WindowAttention:
    """Grouped-query attention over a sliding window: a norm over the whole query and key projections, a partial
    rotation, softmax, and a sigmoid gate on the concatenated heads."""

    def __init__(self, m, t, p, eps):
        self.m, self.eps = m, eps
        self.t = {k[len(p):]: v for k, v in t.items() if k.startswith(p)}
        self.keys: List[np.ndarray] = []
        self.values: List[np.ndarray] = []

    def step(self, h, pos):
        m, t = self.m, self.t
        H, d = m["heads"], m["dim"]
        G, e, scale = m.get("kv_heads", H), m.get("vdim", d), m.get("scale", d ** -0.5)
        q = rms_norm(t["q"] @ h, self.eps, t["q.norm"]).reshape(H, d)
        k = rms_norm(t["k"] @ h, self.eps, t["k.norm"]).reshape(G, d)
        v = (t["v"] @ h).reshape(G, e)
        rot = m.get("rot")
        if rot is not None:
            factor = (rot.get("scaling") or {}).get("factor", 1.0)
            q = rotate_half(q, pos, rot["dims"], rot["base"], factor)
            k = rotate_half(k, pos, rot["dims"], rot["base"], factor)
        self.keys.append(k)
        self.values.append(v)
        w = (m.get("mask") or {}).get("size", 0)
        lo = max(0, pos - w + 1) if w > 0 else 0
        K = np.stack(self.keys[lo:pos + 1])          # [keys, G, d]
        V = np.stack(self.values[lo:pos + 1])
        out = np.zeros((H, e))
        for i in range(H):
            j = i // (H // G)
            s = K[:, j] @ q[i] * scale
            p = np.exp(s - s.max())
            out[i] = (p / p.sum()) @ V[:, j]
        out = out.reshape(-1)
        if "g" in t:
            out = out * sigmoid(t["g"] @ h)
        return t["o"] @ out


class GatedLinearRecurrence:
    """Two branches: y = gelu(Wy h + by); u = conv(Wx h + bx); block-diagonal gates r, i of u; a = exp(-8 r
    softplus(lam)); S <- a S + sqrt(1 - a^2) i u; out = Wo (S y)."""

    def __init__(self, m, t, p):
        self.B, self.R = m.get("blocks", 1), m["width"]
        self.t = {k[len(p):]: v for k, v in t.items() if k.startswith(p)}
        self.conv = ShortConv(self.t["conv"], self.t["conv.b"])
        self.S = np.zeros(self.R)

    def step(self, h, pos):
        t, B, R = self.t, self.B, self.R
        y = gelu_tanh(t["y"] @ h + t["y.b"])
        u = self.conv.step(t["x"] @ h + t["x.b"])
        ub = u.reshape(B, R // B)
        r = sigmoid(np.einsum("boi,bi->bo", t["ra"], ub) + t["ra.b"]).reshape(-1)
        i = sigmoid(np.einsum("boi,bi->bo", t["ri"], ub) + t["ri.b"]).reshape(-1)
        a = np.exp(-8.0 * r * softplus(t["lam"]))
        self.S = a * self.S + np.sqrt(1.0 - a * a) * i * u
        return t["o"] @ (self.S * y)


class SideBySide:
    def __init__(self, m, t, p, eps):
        self.left = WindowAttention(m["left"], t, p + "left.", eps)
        self.right = GatedLinearRecurrence(m["right"], t, p + "right.")
        self.ls, self.rs = m.get("left_scale", 1.0), m.get("right_scale", 1.0)

    def step(self, h, pos):
        return self.ls * self.left.step(h, pos) + self.rs * self.right.step(h, pos)


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------

class PlainRodelorn:
    def __init__(self, folder: Optional[str] = None, config: Optional[dict] = None, tensors: Optional[dict] = None):
        if folder is not None:
            with open(os.path.join(folder, "config.json")) as f:
                config = json.load(f)
            tensors = read_tensors(os.path.join(folder, "model.safetensors"))
        self.cfg, self.t = config, {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = (config.get("norm") or {}).get("eps", 1e-6)

    def new_state(self):
        mixers = []
        for i, layer in enumerate(self.cfg["layers"]):
            p = f"l{i}.mix."
            kind = layer["type"].rstrip("0123456789").rstrip("_")      # "delta_2": another instance of "delta"
            if kind == "delta":
                mixers.append(DeltaMixer(layer["mixer"], self.t, p, self.eps))
            elif kind == "parallel":
                mixers.append(SideBySide(layer["mixer"], self.t, p, self.eps))
            else:
                raise ValueError(layer["type"])
        return mixers

    def token(self, state, token: int, pos: int, layers_out: Optional[list] = None):
        """One token through every layer; returns the stream after the last layer."""
        t, eps = self.t, self.eps
        x = t["embed"][token] * (self.cfg.get("embedding") or {}).get("scale", 1.0)
        for i, layer in enumerate(self.cfg["layers"]):
            p = f"l{i}."
            x = x + rms_norm(state[i].step(rms_norm(x, eps, t[p + "norm1"]), pos), eps, t[p + "norm1b"])
            if layer.get("mlp") is not None:
                f = gated_mlp(rms_norm(x, eps, t[p + "norm2"]), t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"])
                x = x + rms_norm(f, eps, t[p + "norm2b"])
            if layers_out is not None:
                layers_out.append(x.copy())
        return x

    def head(self, x):
        z = (self.t["head"] @ rms_norm(x, self.eps, self.t["final.norm"])) * self.cfg.get("logit_scale", 1.0)
        cap = self.cfg.get("logit_softcap")
        return cap * np.tanh(z / cap) if cap else z

    def logits(self, tokens: Sequence[int], layers: bool = False):
        """[tokens, vocab]; with `layers` also the stream after every layer, [layers, tokens, W]."""
        state = self.new_state()
        out, per = [], []
        for pos, tok in enumerate(tokens):
            lo: list = []
            out.append(self.head(self.token(state, int(tok), pos, lo)))
            per.append(lo)
        z = np.stack(out)
        return (z, np.stack(per).transpose(1, 0, 2)) if layers else z

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        state = self.new_state()
        x = None
        for pos, tok in enumerate(prompt):
            x = self.token(state, int(tok), pos)
        out = []
        for j in range(n):
            nxt = int(np.argmax(self.head(x)))
            out.append(nxt)
            if j + 1 < n:
                x = self.token(state, nxt, len(prompt) + j)
        return out


# --------------------------------------------------------------------------------------------
# the same mechanisms over arrays of a whole sequence (for tests of one mechanism alone)
# --------------------------------------------------------------------------------------------

def causal_conv(x, taps, bias=None, in_bias=None):
    """x: [n, C]; taps: [C, K], the last column the current token's; zeros before the start. in_bias joins every real
    input before the taps (not the zeros in front)."""
    conv = ShortConv(np.asarray(taps, dtype=np.float64), bias)
    return np.stack([conv.step(row + in_bias if in_bias is not None else row) for row in np.asarray(x, dtype=np.float64)])


def delta_rule_scan(q, k, v, b_raw, a_raw, a_log, dt_bias, S=None):
    """q, k: [n, G, d] (after convolution and silu, not yet unit vectors); v: [n, H, e]; b_raw, a_raw: [n, H].
    Returns o [n, H, e] and the last state [H, d, e]."""
    n, G, d = q.shape
    H, e = v.shape[1], v.shape[2]
    S = np.zeros((H, d, e)) if S is None else S.copy()
    out = np.zeros((n, H, e))
    for t in range(n):
        qt = q[t] / np.sqrt((q[t] * q[t]).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
        kt = k[t] / np.sqrt((k[t] * k[t]).sum(-1, keepdims=True) + 1e-6)
        beta = sigmoid(b_raw[t])
        g = np.exp(-np.exp(a_log) * softplus(a_raw[t] + dt_bias))
        for h in range(H):
            j = h // (H // G)
            M = S[h] * g[h]
            u = beta[h] * (v[t, h] - M.T @ kt[j])
            S[h] = M + np.outer(kt[j], u)
            out[t, h] = S[h].T @ qt[j]
    return out, S


def head_norm_gate(o, gate, weight, eps):
    """o, gate: [n, H, e]; weight: [e]."""
    return rms_norm(o, eps, weight) * silu(gate)


def rglru_gates(u, ra, ra_b, ri, ri_b, lam, c=8.0):
    """u: [n, R]; ra, ri: [B, out, in]; biases [B, R / B]. Returns the decay a and the gated input sqrt(1 - a^2) i u."""
    n, R = u.shape
    B = ra.shape[0]
    ub = u.reshape(n, B, R // B)
    r = sigmoid(np.einsum("boi,nbi->nbo", ra, ub) + ra_b).reshape(n, R)
    i = sigmoid(np.einsum("boi,nbi->nbo", ri, ub) + ri_b).reshape(n, R)
    a = np.exp(-c * r * softplus(lam))
    return a, np.sqrt(1.0 - a * a) * i * u


def linear_scan(a, m, S=None):
    """S_t = a_t S_(t-1) + m_t from S (zeros when None), also for the first token. Returns every S_t."""
    S = np.zeros(a.shape[1]) if S is None else S.copy()
    out = np.zeros_like(a)
    for t in range(a.shape[0]):
        S = a[t] * S + m[t]
        out[t] = S
    return out


def projection_norm_rotate(x, weight, eps, heads, positions, dims, base, factor):
    """x: [n, heads * d]: one statistic over the whole row, plain weight, then the partial rotation per head."""
    n = x.shape[0]
    y = rms_norm(x, eps, weight).reshape(n, heads, -1) if weight is not None else x.reshape(n, heads, -1).copy()
    if dims:
        for t in range(n):
            y[t] = rotate_half(y[t], positions[t], dims, base, factor)
    return y


def window_attention(q, keys, values, q_positions, scale, window):
    """q: [n, H, d] at q_positions; keys [T, G, d], values [T, G, e] of positions 0..T-1. Position p sees
    max(0, p - window + 1)..p (all of 0..p when window is 0)."""
    n, H, _ = q.shape
    G, e = keys.shape[1], values.shape[2]
    out = np.zeros((n, H, e))
    for t, p in enumerate(q_positions):
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(H):
            j = h // (H // G)
            s = keys[lo:p + 1, j] @ q[t, h] * scale
            w = np.exp(s - s.max())
            out[t, h] = (w / w.sum()) @ values[lo:p + 1, j]
    return out
