"""Plain, slow Gunirax: whole sequences, no cache, one function per mechanism, NumPy only, float64.

A decoder whose ``config.json`` lists its layers.  The stream starts as the embedded token times a constant.  Layers
are pre-norm,  x <- x + mixer(N1(x));  x <- x + ff(N2(x)),  and every norm (the layers', the final one) is a dynamic
tanh:  N(x) = tanh(alpha x) * w + b  with a learned scalar alpha; no mean, no variance.  ``loop`` runs the layers
start .. stop-1 ``times`` times in a row with the same weights; before every pass but the first the embedded rows
(the stream as it was before the first layer) are added to the stream.

* mixer ``parallel``: two mixers read the same input; the result is half the sum of their outputs, each RMS-normed
  over the width with a weight of its own.
  left: grouped-query attention whose values are its keys as projected.  Queries and keys have biases, are rotated
  (pairs (2i, 2i+1), the first ``rot.dims`` columns, frequencies rescaled by wavelength) and then divided by their
  root mean square per head.  Position i sees j <= i of its own chunk of ``mask.size`` positions.  The weight of a
  visible key is sigmoid(scale q.k + pb_h), not normalised; the heads' weights are mixed by a matrix T [H, H] before
  they meet the values; every head's output is multiplied by sigmoid((W_g h)_h).
  right: a matrix memory with a fixed decay per head on silu'd queries, keys and values; the concatenated heads are
  RMS-normed together, multiplied by sigmoid(W_g h) and projected.
* mixer ``hgrn2``: a matrix memory whose forget gate f = l + (1 - l) sigmoid(W_f h + b) decays the rows of the state
  and whose complement 1 - f is the key; the read-out is RMS-normed per head.
* feed-forward ``dense``: W_down (silu(W_gate h) * W_up h).  ``moe``: sigmoid router scores; the choice adds a
  correction per expert and is limited to the best groups of neighbouring experts (a group's score: the sum of its
  two largest corrected scores); weights are the chosen scores over their sum, times a constant; experts and the
  shared expert are W_down relu(W_up h)^2.

It shares no code with the library: its own safetensors reader, its own reading of ``config.json``.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np

F = np.float64


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n).decode("utf-8"))
        data = fh.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        elif info["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"plain reader: dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"]).astype(F)
    return out


# ---- small pieces --------------------------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def dynamic_tanh(x: np.ndarray, w: Dict[str, np.ndarray], name: str) -> np.ndarray:
    return np.tanh(float(w[name + ".alpha"]) * x) * w[name] + w[name + ".b"]


# ---- the left branch: chunked sigmoid attention with mixed heads ---------------------------------------------

def rotary_frequencies(rot: dict) -> np.ndarray:
    dims = int(rot["dims"])
    i = np.arange(dims // 2, dtype=F)
    f = float(rot["base"]) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
        wave = 2.0 * math.pi / f
        s = (original / wave - low) / (high - low)
        mid = (1.0 - s) * f / factor + s * f
        f = np.where(wave < original / high, f, np.where(wave > original / low, f / factor, mid))
    return f


def rotate(x: np.ndarray, rot: dict, first_position: int = 0) -> np.ndarray:
    """x: [tokens, heads, dim]; the pair (2i, 2i+1) of the first rot.dims columns turns by position * f_i."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    f = rotary_frequencies(rot)
    pos = np.arange(first_position, first_position + x.shape[0], dtype=F)
    a = pos[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def chunk_visible(n: int, size: int, first_position: int = 0) -> np.ndarray:
    """[n, n] booleans: row i sees column j when j <= i and both lie in the same chunk of ``size`` positions."""
    p = np.arange(first_position, first_position + n)
    return (p[None, :] <= p[:, None]) & ((p[None, :] // size) == (p[:, None] // size))


def window_visible(n: int, size: int) -> np.ndarray:
    """[n, n] booleans: row i sees the last ``size`` positions up to itself (a mask the design does not use; the
    library's attention part offers it beside the chunks)."""
    p = np.arange(n)
    return (p[None, :] <= p[:, None]) & (p[:, None] - p[None, :] < size)


def sigmoid_attention(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, m: dict, eps: float, see=None) -> np.ndarray:
    n = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).reshape(n, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).reshape(n, G, D)
    v = k                                                    # the values are the keys as projected
    q = rms_unit(rotate(q, m["rot"]), eps)
    kk = rms_unit(rotate(k, m["rot"]), eps)
    if see is None:
        see = chunk_visible(n, int(m["mask"]["size"]) if m.get("mask") else n)   # no mask: one chunk holds everything
    per = H // G
    weights = np.zeros((H, n, n), dtype=F)
    for g in range(H):
        score = (q[:, g, :] @ kk[:, g // per, :].T) * float(m["scale"])
        weights[g] = np.where(see, sigmoid(score + w[pre + "pb"][g]), 0.0)
    mixed = np.einsum("hg,gij->hij", w[pre + "talk"], weights)
    gate = sigmoid(h @ w[pre + "g"].T)                       # [n, H]
    heads = [(mixed[hh] @ v[:, hh // per, :]) * gate[:, hh:hh + 1] for hh in range(H)]
    return np.concatenate(heads, axis=1) @ w[pre + "o"].T


# ---- matrix memories ----------------------------------------------------------------------------------------

def lightning(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, m: dict, eps: float) -> np.ndarray:
    n = h.shape[0]
    H, d, vd = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[pre + "q"].T).reshape(n, H, d)
    k = silu(h @ w[pre + "k"].T).reshape(n, H, d)
    v = silu(h @ w[pre + "v"].T).reshape(n, H, vd)
    out = np.zeros((n, H, vd), dtype=F)
    for hh in range(H):
        S = np.zeros((d, vd), dtype=F)
        decay = float(m["decay"][hh])
        for t in range(n):
            S = decay * S + np.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    o = rms_unit(out.reshape(n, H * vd), eps) * w[pre + "norm"]
    return (o * sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def hgrn2(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, m: dict, eps: float) -> np.ndarray:
    n = h.shape[0]
    H, d, vd = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w[pre + "q"].T).reshape(n, H, d)
    v = (h @ w[pre + "v"].T).reshape(n, H, vd)
    low = w[pre + "lower"]
    f = (low + (1.0 - low) * sigmoid(h @ w[pre + "f"].T + w[pre + "f.b"])).reshape(n, H, d)
    out = np.zeros((n, H, vd), dtype=F)
    for hh in range(H):
        S = np.zeros((d, vd), dtype=F)
        for t in range(n):
            S = f[t, hh][:, None] * S + np.outer(1.0 - f[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    o = rms_unit(out, eps) * w[pre + "norm"]
    return o.reshape(n, H * vd) @ w[pre + "o"].T


def parallel(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, m: dict, eps: float) -> np.ndarray:
    left = sigmoid_attention(h, w, pre + "left.", m["left"], eps)
    right = lightning(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * w[pre + "left.out"] + rms_unit(right, eps) * w[pre + "right.out"])


# ---- feed-forwards ------------------------------------------------------------------------------------------

def dense(h: np.ndarray, w: Dict[str, np.ndarray], pre: str) -> np.ndarray:
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def relu2_expert(h: np.ndarray, w: Dict[str, np.ndarray], pre: str) -> np.ndarray:
    return (np.maximum(h @ w[pre + "up"].T, 0.0) ** 2) @ w[pre + "down"].T


def route(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, r: dict):
    """(chosen experts [n, top], their weights [n, top])."""
    E, top = int(r["experts"]), int(r["top"])
    count, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
    s = sigmoid(h @ w[pre + "router"].T)
    choice = s + w[pre + "correction"]
    per = E // count
    chosen = np.zeros((h.shape[0], top), dtype=np.int64)
    weights = np.zeros((h.shape[0], top), dtype=F)
    for t in range(h.shape[0]):
        c = choice[t].reshape(count, per)
        group_score = np.sort(c, axis=1)[:, ::-1][:, :2].sum(axis=1)
        kept = np.argsort(-group_score, kind="stable")[:keep]
        allowed = np.full(E, -np.inf)
        for g in kept:
            allowed[g * per:(g + 1) * per] = choice[t, g * per:(g + 1) * per]
        idx = np.argsort(-allowed, kind="stable")[:top]
        chosen[t] = idx
        weights[t] = s[t, idx] / (s[t, idx].sum() + 1e-20) * float(r["scale"])
    return chosen, weights


def routed(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, mlp: dict) -> np.ndarray:
    chosen, weights = route(h, w, pre, mlp["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weights[t]):
            out[t] += g * relu2_expert(h[t:t + 1], w, f"{pre}e{int(e)}.")[0]
    if mlp.get("shared") is not None:
        out = out + relu2_expert(h, w, pre + "shared.")
    return out


def feed_forward(h: np.ndarray, w: Dict[str, np.ndarray], pre: str, mlp: Optional[dict]):
    if mlp is None:
        return None
    return dense(h, w, pre) if mlp["kind"] == "dense" else routed(h, w, pre, mlp)


# ---- the model ------------------------------------------------------------------------------------------------

def layer_runs(cfg: dict) -> List[dict]:
    """The executed layers in order: {"layer": i, "restart": whether the embedded rows are added first}."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [{"layer": i, "restart": False} for i in range(start)]
    for p in range(times if stop > start else 0):
        runs += [{"layer": i, "restart": p > 0 and i == start} for i in range(start, stop)]
    runs += [{"layer": i, "restart": False} for i in range(max(stop, start), n)]
    return runs


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, return_layers: bool = False):
    """Logits [tokens, vocab] of one whole sequence; with ``return_layers`` also the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"][np.asarray(tokens, dtype=np.int64)] * float(cfg["embedding"]["scale"])
    x = x0.copy()
    streams = []
    for run in layer_runs(cfg):
        i = run["layer"]
        layer, pre = cfg["layers"][i], f"l{i}."
        if run["restart"]:
            x = x + x0
        h = dynamic_tanh(x, w, pre + "norm1")
        if layer["type"] == "parallel":
            x = x + parallel(h, w, pre + "mix.", layer["mixer"], eps)
        elif layer["type"] == "hgrn2":
            x = x + hgrn2(h, w, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            x = x + feed_forward(dynamic_tanh(x, w, pre + "norm2"), w, pre + "mlp.", layer["mlp"])
        streams.append(x.copy())
    logits = dynamic_tanh(x, w, "final.norm") @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits


def load_folder(path: str):
    with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    return cfg, read_safetensors(os.path.join(path, "model.safetensors"))


class PlainGunirax:
    """A model folder read once; whole sequences through ``forward``."""

    def __init__(self, folder: str):
        self.cfg, self.w = load_folder(folder)

    def logits(self, tokens) -> np.ndarray:
        return forward(self.cfg, self.w, tokens)

    def layers(self, tokens) -> np.ndarray:
        return forward(self.cfg, self.w, tokens, return_layers=True)[1]

    def greedy(self, prompt, n: int) -> List[int]:
        seq, out = list(prompt), []
        for _ in range(n):
            t = int(np.argmax(self.logits(seq)[-1]))
            out.append(t)
            seq.append(t)
        return out
