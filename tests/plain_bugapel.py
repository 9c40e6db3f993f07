"""A plain, slow Bugapel for tests: float64 NumPy, one function per mechanism.

It shares no code with `dynalm_b200`: it reads config.json and model.safetensors by itself. Two readings of the same
equations stand side by side: `PlainBugapel.logits(tokens)` runs a whole sequence at once (attention as a masked matrix,
the linear attention as a loop over tokens), `logits_stepwise(tokens)` feeds one token at a time from explicit state (the
keys and values seen so far, the matrix of every linear-attention head); they agree to rounding of float64.

Notation. W the stream's width, n streams. Attention: H query heads, G key/value heads, key size d, value size e, the
first r numbers of a head rotated, window w with the first f keys kept. Linear attention: H heads, key size d, value
size e, temperature tau.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

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

def layer_norm(x, weight, bias, eps):
    mu = x.mean(axis=-1, keepdims=True)
    dev = x - mu
    y = dev / np.sqrt((dev * dev).mean(axis=-1, keepdims=True) + eps) * weight
    return y + bias if bias is not None else y


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def frequencies(base: float, r: int, stretch: Optional[dict] = None):
    """base^(-2i/r) for i < r/2; with `stretch` {factor, low, high, original}: kept where the wavelength is below
    original / high, divided by factor where it is above original / low, and blended in between."""
    f = np.array([base ** (-2.0 * i / r) for i in range(r // 2)])
    if not stretch:
        return f
    out = []
    for fi in f:
        wave = 2.0 * math.pi / fi
        if wave < stretch["original"] / stretch["high"]:
            out.append(fi)
        elif wave > stretch["original"] / stretch["low"]:
            out.append(fi / stretch["factor"])
        else:
            s = (stretch["original"] / wave - stretch["low"]) / (stretch["high"] - stretch["low"])
            out.append((1.0 - s) * fi / stretch["factor"] + s * fi)
    return np.array(out)


def rotate(x, positions, freq, layout: str):
    """x [T, heads, d]; the first 2 * len(freq) numbers of every head turn by position * freq. layout "halves": number
    i pairs with i + r/2; "pairs": number 2i pairs with 2i + 1."""
    r = 2 * len(freq)
    if r == 0:
        return x
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    y = x.copy()
    if layout == "halves":
        a, b = x[..., :r // 2], x[..., r // 2:r]
        y[..., :r // 2], y[..., r // 2:r] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., 0:r:2], x[..., 1:r:2]
        y[..., 0:r:2], y[..., 1:r:2] = a * c - b * s, b * c + a * s
    return y


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    return j <= i and (window <= 0 or i - j < window or j < keep_first)


def attend(q, k, v, q_pos, k_pos, scale, window=0, keep_first=0, sink=False):
    """q [Tq, H, d], k [Tk, G, d], v [Tk, G, e] -> [Tq, H, e]. With `sink` the denominator holds one more exp(0)."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((Tq, H, v.shape[2]))
    for a in range(Tq):
        js = [b for b in range(len(k_pos)) if visible(q_pos[a], k_pos[b], window, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = (k[js, g] @ q[a, h]) * scale
            m = max(s.max(), 0.0) if sink else s.max()
            w = np.exp(s - m)
            den = w.sum() + (math.exp(-m) if sink else 0.0)
            out[a, h] = (w[:, None] * v[js, g]).sum(0) / den
    return out


def linear_attention_step(S, q, k, v, z, tau):
    """One token of gated linear attention. S [H, d, e] -> (S', o [H, e]): the decay sigmoid(z)^(1/tau) acts on the rows of
    S (key channels), then k v^T is written, then q * d^(-1/2) reads."""
    alpha = np.exp(-np.logaddexp(0.0, -z) / tau)                  # [H, d]
    S = alpha[:, :, None] * S + k[:, :, None] * v[:, None, :]
    o = np.einsum("hde,hd->he", S, q * q.shape[-1] ** -0.5)
    return S, o


def head_norm_gate(o, gate, weight, eps):
    """o, gate [..., H, e]: every head normed by itself, times the shared weight, times silu(gate)."""
    return unit_rms(o, eps) * weight * silu(gate)


def route(z, top: int, groups: int, keep: int, scale: float):
    """Router logits z [E] -> (chosen experts, their weights)."""
    s = np.exp(z - z.max())
    s = s / s.sum()
    E = len(s)
    allowed = np.ones(E, dtype=bool)
    if groups > 1:
        per = E // groups
        best = np.argsort(-s.reshape(groups, per).max(axis=1), kind="stable")[:keep]
        allowed[:] = False
        for g in best:
            allowed[g * per:(g + 1) * per] = True
    order = [int(i) for i in np.argsort(-np.where(allowed, s, -1.0), kind="stable")[:top]]
    w = s[order]
    return order, w / (w.sum() + 1e-20) * scale


def expert(x, up, down):
    return down @ (np.maximum(up @ x, 0.0) ** 2)


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------

class PlainBugapel:
    def __init__(self, folder: Optional[str] = None, config: Optional[dict] = None, tensors: Optional[dict] = None):
        if folder is not None:
            with open(os.path.join(folder, "config.json")) as f:
                config = json.load(f)
            tensors = read_tensors(os.path.join(folder, "model.safetensors"))
        self.cfg, self.t = config, {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = (config.get("norm") or {}).get("eps", 1e-5)
        self.n = config.get("streams", 0)

    # mixers over a run of tokens [T, W] at the given positions, from and into `state`
    def _attention(self, i, h, positions, state):
        m, t, p = self.cfg["layers"][i]["mixer"], self.t, f"l{i}.mix."
        second = self.cfg["layers"][i]["type"] == "attention_2"
        T = h.shape[0]
        H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
        q, k, v = h @ t[p + "q"].T, h @ t[p + "k"].T, h @ t[p + "v"].T
        if second:
            q, k, v = q + t[p + "q.b"], k + t[p + "k.b"], v + t[p + "v.b"]
        q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, e)
        rot = m.get("rot")
        if rot:
            f = frequencies(rot["base"], rot["dims"], rot.get("scaling"))
            layout = "pairs" if second else "halves"
            q, k = rotate(q, positions, f, layout), rotate(k, positions, f, layout)
        if not second:
            q, k = unit_rms(q, self.eps), unit_rms(k, self.eps)
        state.setdefault("k", []).extend(k)
        state.setdefault("v", []).extend(v)
        state.setdefault("pos", []).extend(positions)
        mask = m.get("mask") if second else None
        o = attend(q, np.array(state["k"]), np.array(state["v"]), positions, state["pos"], m["scale"],
                   mask["size"] if mask else 0, mask.get("keep_first", 0) if mask else 0, sink=not second)
        y = o.reshape(T, H * e) @ t[p + "o"].T
        return y + t[p + "o.b"] if second else y

    def _linear_attention(self, i, h, state):
        m, t, p = self.cfg["layers"][i]["mixer"], self.t, f"l{i}.mix."
        T = h.shape[0]
        H, d, e = m["heads"], m["dim"], m.get("vdim", m["dim"])
        q, k = (h @ t[p + "q"].T).reshape(T, H, d), (h @ t[p + "k"].T).reshape(T, H, d)
        v = (h @ t[p + "v"].T).reshape(T, H, e)
        z = ((h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "a2.b"]).reshape(T, H, d)
        S = state.get("S", np.zeros((H, d, e)))
        o = np.zeros((T, H, e))
        for a in range(T):
            S, o[a] = linear_attention_step(S, q[a], k[a], v[a], z[a], m["tau"])
        state["S"] = S
        g = head_norm_gate(o, (h @ t[p + "g"].T).reshape(T, H, e), t[p + "norm"], self.eps)
        return g.reshape(T, H * e) @ t[p + "o"].T

    def _moe(self, i, h):
        f, t, p = self.cfg["layers"][i]["mlp"], self.t, f"l{i}.mlp."
        r = f["router"]
        groups = r.get("groups") or {}
        out = np.zeros_like(h)
        for a in range(h.shape[0]):
            chosen, w = route(t[p + "router"] @ h[a], r["top"], groups.get("count", 1), groups.get("keep", 1), r.get("scale", 1.0))
            for j, wj in zip(chosen, w):
                out[a] += wj * expert(h[a], t[f"{p}e{j}.up"], t[f"{p}e{j}.down"])
        return out

    def run(self, tokens, positions, states, layers_out: Optional[list] = None):
        """A run of tokens through every layer from and into `states` (one dict per layer); returns the stream [T, W]
        (the sum of the streams when there are several)."""
        t, cfg, n = self.t, self.cfg, self.n
        x = t["embed"][np.asarray(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
        xs = [x.copy() for _ in range(n)] if n else None
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            for q in (1, 2):
                if q == 2 and layer.get("mlp") is None:
                    continue
                u = sum(t[f"{p}hc{q}.in"][s] * xs[s] for s in range(n)) if n else x
                hn = layer_norm(u, t[f"{p}norm{q}"], t.get(f"{p}norm{q}.b"), self.eps)
                if q == 2:
                    y = self._moe(i, hn)
                elif layer["type"] == "gla":
                    y = self._linear_attention(i, hn, states[i])
                else:
                    y = self._attention(i, hn, list(positions), states[i])
                if n:
                    mix, w = t[f"{p}hc{q}.mix"], t[f"{p}hc{q}.out"]
                    xs = [sum(mix[s, b] * xs[s] for s in range(n)) + w[b] * y for b in range(n)]
                else:
                    x = x + y
            if layers_out is not None:
                layers_out.append(sum(xs) if n else x.copy())
        return sum(xs) if n else x

    def head(self, x):
        z = layer_norm(x, self.t["final.norm"], self.t.get("final.norm.b"), self.eps) @ self.t["embed"].T
        cap = self.cfg.get("logit_softcap")
        return cap * np.tanh(z / cap) if cap else z

    def logits(self, tokens, layers: bool = False, cuts: Optional[List[int]] = None):
        """Logits [T, vocab] of a sequence fed whole, or in portions of the sizes `cuts` (the rest in one piece)."""
        states = [dict() for _ in self.cfg["layers"]]
        seen = [] if layers else None
        sizes = list(cuts or []) + [len(tokens)]
        at, rows, per_layer = 0, [], []
        for size in sizes:
            size = min(size, len(tokens) - at)
            if size <= 0:
                continue
            part = [] if layers else None
            rows.append(self.head(self.run(tokens[at:at + size], range(at, at + size), states, part)))
            if layers:
                per_layer.append(part)
            at += size
        out = np.concatenate(rows)
        if layers:
            return out, [np.concatenate([part[i] for part in per_layer]) for i in range(len(self.cfg["layers"]))]
        return out

    def logits_stepwise(self, tokens):
        return self.logits(tokens, cuts=[1] * len(tokens))
