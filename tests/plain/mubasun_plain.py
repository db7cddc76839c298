"""Plain, slow Mubasun: whole sequences, no cache, one function per mechanism, NumPy only, float64.

A decoder whose ``config.json`` lists its layers.  The stream starts as the embedded token plus a learned vector
of its position.  A layer norms the stream once and adds the sum of its two sublayers, which both read the normed row:

    h = N(x);   x <- x + (mixer(h) + ff(h))            N: an RMS norm taken in groups, times a weight

* mixer ``attention``: grouped-query softmax attention.  Queries and keys pass an RMS norm over their whole
  projection (all heads at once).  Nothing is rotated: score(i, j) = scale q_i . k_j - m_h (i - j) with
  ``m_h = 2^(-8 (h + 1) / heads)``, over the keys with ``0 <= i - j < mask.size`` (all earlier keys without a mask).  The concatenated heads are multiplied by ``sigmoid(W_g h)`` before the output matrix.
  ``kv_from`` = j: queries of its own against the normed keys and the values that layer j made.
* feed-forward ``dense``: ``W_down xielu(W_up h)`` with two learned numbers per layer.
* feed-forward ``moe``: a softmax router over experts and identity experts; the ``top`` largest of score + correction
  are chosen; an expert's weight is its score times ``router.scale``; experts are ``W_down (silu(W_gate h) * W_up h)``,
  an identity expert gives ``h`` itself; a shared expert of the same form is added times ``sigmoid(w_sg . h)``.

It shares no code with the library: its own safetensors reader, its own reading of ``config.json``.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence, Tuple

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
        else:
            raise ValueError(f"plain reader: dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"]).astype(F)
    return out


# ---- small pieces --------------------------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def silu(z):
    return z * sigmoid(z)


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def group_norm(x: np.ndarray, w: np.ndarray, groups: int, eps: float) -> np.ndarray:
    """Rows cut into ``groups`` equal consecutive pieces, each piece divided by its own root mean square."""
    rows, width = x.shape
    pieces = x.reshape(rows, groups, width // groups)
    return rms_unit(pieces, eps).reshape(rows, width) * w


def xielu(z: np.ndarray, p: float, q: float) -> np.ndarray:
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - z) + z / 2
    return np.where(z > 0, pos, neg)


def slopes(heads: int) -> np.ndarray:
    return 2.0 ** (-8.0 * (np.arange(heads) + 1) / heads)


# ---- the mixer ---------------------------------------------------------------------------------------------------

def keys_and_values(h: np.ndarray, w: Dict[str, np.ndarray], eps: float) -> Tuple[np.ndarray, np.ndarray]:
    """What a layer with projections of its own keeps: keys after their norm over the whole projection, and values."""
    return rms_unit(h @ w["k"].T, eps) * w["k.norm"], h @ w["v"].T


def attention(h: np.ndarray, w: Dict[str, np.ndarray], m: dict, eps: float,
              kv: Optional[Tuple[np.ndarray, np.ndarray]] = None, first_position: int = 0):
    """Returns (output rows, (keys, values)).  ``kv``: another layer's keys and values instead of this one's."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (rms_unit(h @ w["q"].T, eps) * w["q.norm"]).reshape(T, H, d)
    if kv is None:
        kv = keys_and_values(h, w, eps)
    k, v = kv[0].reshape(T, G, d), kv[1].reshape(T, G, dv)
    size = (m.get("mask") or {}).get("size")
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    seen = j <= i
    if size is not None:
        seen &= (i - j) < int(size)
    out = np.zeros((T, H, dv), dtype=F)
    for head, slope in enumerate(slopes(H)):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"]) - slope * (i - j)
        s = np.where(seen, s, -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, head] = (p / p.sum(axis=-1, keepdims=True)) @ v[:, g]
    gated = out.reshape(T, H * dv) * sigmoid(h @ w["g"].T)
    return gated @ w["o"].T, kv


# ---- the feed-forwards ----------------------------------------------------------------------------------------------

def dense(h: np.ndarray, w: Dict[str, np.ndarray]) -> np.ndarray:
    p, q = (float(v) for v in w["act"])
    return xielu(h @ w["up"].T, p, q) @ w["down"].T


def gated_expert(h: np.ndarray, w: Dict[str, np.ndarray], prefix: str) -> np.ndarray:
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h: np.ndarray, w: Dict[str, np.ndarray], r: dict):
    """(chosen [rows, top] experts, their weights): softmax scores over experts and identity experts; the choice adds
    the correction, the weights do not; ties go to the lower index."""
    z = h @ w["router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    chosen = np.argsort(-(s + w["correction"]), axis=-1, kind="stable")[:, :int(r["top"])]
    return chosen, np.take_along_axis(s, chosen, axis=-1) * float(r["scale"])


def routed(h: np.ndarray, w: Dict[str, np.ndarray], mlp: dict) -> np.ndarray:
    r = mlp["router"]
    E = int(r["experts"])
    chosen, weights = route(h, w, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], weights[t]):
            if e >= E:                                   # an identity expert: the row itself
                out[t] += a * h[t]
            else:
                out[t] += a * gated_expert(h[t:t + 1], w, f"e{e}.")[0]
    if mlp.get("shared"):
        out += gated_expert(h, w, "shared.") * sigmoid(h @ w["shared.sg"].T)
    return out


def feed_forward(h: np.ndarray, w: Dict[str, np.ndarray], mlp: Optional[dict]):
    if not mlp:
        return 0.0
    if mlp["kind"] == "dense":
        return dense(h, w)
    if mlp["kind"] == "moe":
        return routed(h, w, mlp)
    raise ValueError(f"plain: mlp.kind {mlp['kind']!r}")


# ---- the model -------------------------------------------------------------------------------------------------------

class PlainMubasun:
    def __init__(self, model_dir: str):
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
            self.cfg = json.load(fh)
        self.w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
        self.eps = float(self.cfg["norm"]["eps"])
        self.groups = int(self.cfg["norm"].get("groups", 1))

    def sub(self, prefix: str) -> Dict[str, np.ndarray]:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def residual_stream(self, ids: Sequence[int]) -> List[np.ndarray]:
        """The stream after the embedding and after every layer."""
        cfg, w, eps = self.cfg, self.w, self.eps
        ids = np.asarray(ids, dtype=np.int64)
        x = w["embed"][ids] + w["pos"][:len(ids)]
        streams, kept = [x], {}
        for i, layer in enumerate(cfg["layers"]):
            if layer["type"] != "attention":
                raise ValueError(f"plain: mixer {layer['type']!r}")
            h = group_norm(x, w[f"l{i}.norm1"], self.groups, eps)
            m = layer["mixer"]
            src = m.get("kv_from")
            y, kept[i] = attention(h, self.sub(f"l{i}.mix."), m, eps, kv=None if src is None else kept[int(src)])
            x = x + (y + feed_forward(h, self.sub(f"l{i}.mlp."), layer.get("mlp")))
            streams.append(x)
        return streams

    def logits(self, ids: Sequence[int]) -> np.ndarray:
        x = self.residual_stream(ids)[-1]
        return group_norm(x, self.w["final.norm"], self.groups, self.eps) @ self.w["head"].T

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        seq, out = list(prompt), []
        for _ in range(n):
            t = int(np.argmax(self.logits(seq)[-1]))
            out.append(t)
            seq.append(t)
        return out
