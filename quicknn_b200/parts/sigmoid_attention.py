"""Attention with sigmoid weights: no softmax, nothing normalised over the keys, and heads that mix their weights.

    q = W_q x (+ b_q),  k = W_k x (+ b_k)                       H query heads, G key/value heads of ``head_dim``
    v = k as projected (``values_from_keys``), or W_v x (+ b_v)
    q, k <- rotated (the position part), then divided by their root mean square per head (``qk_norm``, no weight)
    w_g(i, j) = sigmoid(scale q_g(i) . k(j) + pb_g)             for the keys j that position i sees (``mask``)
    m_h(i, j) = sum_g talk[h, g] w_g(i, j)                       (``talk``: a learned matrix [H, H])
    o_h(i) = sigmoid((W_g x)_h) * sum_j m_h(i, j) v(j)           (``out_gate``: one number per token and head)
    y = W_o concat_h o_h

``mask`` = {"kind": "chunk" | "window" | "causal", "size": n}: position i sees j <= i of its own chunk of n positions
(chunks counted from position 0 of the sequence), the last n positions, or every earlier position.  Everything but the
mask's kind and size, the scale and the sizes is optional: ``bias``, ``qk_norm`` = {"eps": e}, ``head_bias`` (pb),
``talk``, ``out_gate``, ``values_from_keys``.

q, k (, v) and the gate's logits are one product against the stacked matrix.  One kernel (``ops.head_prep``) adds the
biases, copies the keys as values, rotates, norms and appends keys and values to the cache line; one kernel
(``ops.sigmoid_attention``) does the rest for whole prompts (keys from the step's rows; bfloat16 prompts at head
sizes 32 to 256 on the tensor cores), for steps that continue
sequences (cached keys, then the step's rows; the append comes after it, so that a ring as short as the mask is never
overwritten under a row that still needs it) and for single tokens (keys from the line, in several ranges per
sequence where the context is long).  The cache line keeps ``mask.size`` positions as a ring (all of them for "causal").
Scores, sigmoids, the mix over heads and the weighted sums are float32 in both precisions.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheNeed, Mixer
from .linear import project, stack_rows
from .spec import PartSpec

TILES_PER_RANGE = 2          # key tiles of 32 that a block of a decode step walks at least, where the context is long


@MIXERS.register("sigmoid_attention")
class SigmoidAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        if self.n_kv < 1 or self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_kv} kv heads do not divide {self.n_heads} heads")
        mask = p.get("mask") or {"kind": "causal", "size": 0}
        self.mask_kind = str(mask["kind"])
        self.mask_size = int(mask.get("size") or 0)
        if self.mask_kind not in ops.MASKS or (self.mask_kind != "causal" and self.mask_size < 1):
            raise ValueError(f"sigmoid attention: mask {dict(mask)!r} (kinds: {sorted(ops.MASKS)}; a size of at least 1)")
        self.has_bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        self.has_head_bias = bool(p.get("head_bias", False))
        self.has_talk = bool(p.get("talk", False))
        self.out_gate = bool(p.get("out_gate", False))
        self.values_from_keys = bool(p.get("values_from_keys", False))
        pos: PartSpec = p["position"]
        self.position = POSITIONS.get(pos.kind)(pos)
        self.rot_dim = int(getattr(self.position, "rotary_dim", 0))
        self.w_in: Optional[torch.Tensor] = None         # q | k | (v) | gate logits | zero rows up to a multiple of 8
        self.w_o: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.pb: Optional[torch.Tensor] = None
        self.talk: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        W, H, G, D = int(p["hidden_size"]), int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        M, B = cls.PARAM_ROLE_MATRIX, cls.PARAM_ROLE_NORM
        own_v = not p.get("values_from_keys", False)
        out = {"q_proj": ((H * D, W), M), "k_proj": ((G * D, W), M), "o_proj": ((W, H * D), M)}
        if own_v:
            out["v_proj"] = ((G * D, W), M)
        if p.get("bias", False):
            out.update({"q_bias": ((H * D,), B), "k_bias": ((G * D,), B)})
            if own_v:
                out["v_bias"] = ((G * D,), B)
        if p.get("head_bias", False):
            out["head_bias"] = ((H,), B)
        if p.get("talk", False):
            out["talk"] = ((H, H), M)
        if p.get("out_gate", False):
            out["g_proj"] = ((H, W), M)
        return out

    def load(self, tensors, compute_dtype, device) -> None:
        H, G, D = self.n_heads, self.n_kv, self.head_dim
        own_v = not self.values_from_keys
        parts = [tensors["q_proj"], tensors["k_proj"]] + ([tensors["v_proj"]] if own_v else [])
        if self.out_gate:
            parts.append(tensors["g_proj"])
        rows = sum(t.shape[0] for t in parts)
        if rows % 8:                                         # rows of the product in whole 16-byte pieces
            parts.append(torch.zeros((8 - rows % 8, self.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = stack_rows(parts)
        self.w_o = tensors["o_proj"].contiguous()
        if self.has_bias:
            bs = [tensors["q_bias"], tensors["k_bias"]] + ([tensors["v_bias"]] if own_v else [])
            self.bias = torch.cat([b.to(torch.float32) for b in bs]).contiguous()
        if self.has_head_bias:
            self.pb = tensors["head_bias"].to(torch.float32).contiguous()
        if self.has_talk:
            self.talk = tensors["talk"].to(torch.float32).contiguous()
        self.position.prepare(device)
        why = (ops.sigmoid_attention_refusal(compute_dtype, H, G, D) or ops.linear_refusal(self.w_in.dtype, self.hidden)
               or ops.linear_refusal(self.w_o.dtype, H * D))
        if why:
            raise ValueError(f"sigmoid attention: {why}")

    def weight_bytes(self) -> int:
        ws = (self.w_in, self.w_o, self.bias, self.pb, self.talk)
        return sum(w.numel() * w.element_size() for w in ws if w is not None)

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(self.n_kv, self.head_dim, None if self.mask_kind == "causal" else self.mask_size)

    def decode_splits(self, step) -> int:
        """Key ranges per sequence in a decode step: one while a sequence sees few tiles of keys; with a long context
        as many as keep every block at ``TILES_PER_RANGE`` tiles, and no more blocks than two rounds of the device."""
        fixed = step.tuning.get("decode_splits")
        if fixed:
            return int(fixed)
        longest = step.longest or step.max_seq or 0
        if self.mask_kind != "causal":
            longest = min(longest, self.mask_size) if longest else self.mask_size
        tiles = -(-max(1, longest) // 32)
        return max(1, min(tiles // TILES_PER_RANGE, 296 // max(1, step.n_seqs), 64))

    def schedule(self, step) -> tuple:
        return (self.decode_splits(step),) if step.mode == "decode" else ()

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        H, G, D = self.n_heads, self.n_kv, self.head_dim
        extend = step.mode == "extend"
        decode = step.mode == "decode"
        p = project(x, self.w_in)                            # q | k | (v) | gate logits
        gate_col = (H + G) * D + (0 if self.values_from_keys else G * D)
        norm_dim = D if self.qk_norm else 0
        eps = float(self.qk_norm["eps"]) if self.qk_norm else 0.0
        rot = dict(rot_dim=self.rot_dim, inv_freq=self.position.inv_freq if self.rot_dim else None,
                   interleaved=getattr(self.position, "layout", "half") == "interleaved", tok_pos=step.tok_pos,
                   tok_slot=step.tok_slot, line=line, append=bool(not extend and line is not None and line.writes))
        if self.values_from_keys:
            packed = torch.empty((p.shape[0], (H + 2 * G) * D), dtype=p.dtype, device=p.device)
            ops.head_prep(p, 0, H, G, G * D, D, dst=packed, bias=self.bias, norm_dim=norm_dim, eps=eps, norm_last=True,
                          plain_norm=bool(self.qk_norm), values_are_keys=True, **rot)
        else:
            packed = ops.head_prep(p, 0, H, G, G * D, D, bias=self.bias, norm_dim=norm_dim, eps=eps, norm_last=True,
                                   plain_norm=bool(self.qk_norm), **rot)
        a = ops.sigmoid_attention(packed, H, G, D, step.tok_pos, step.tok_row0, step.tok_slot, line, own_rows=not decode,
                                  mask=self.mask_kind, mask_size=self.mask_size, scale=self.scale, pb=self.pb,
                                  talk=self.talk, gate=p if self.out_gate else None, gate_col=gate_col,
                                  splits=self.decode_splits(step) if decode else 1,
                                  seq_row0=step.seq_row0 if step.mode == "prefill" else None,
                                  seq_len=step.seq_len if step.mode == "prefill" else None,
                                  longest=step.max_q_len if step.mode == "prefill" else 0)
        if extend and line is not None and line.writes:
            ops.cache_append(packed, H, G, D, step.tok_pos, step.tok_slot, line)
        return project(a, self.w_o)
