"""Position encodings.  A position part places a step's tokens: it changes the queries and keys
of the packed q|k|v rows according to their positions and appends keys and values to the cache
(one kernel does both, so the two belong to one call).

Reference: GO_LLM_ROPE, angle = position * exp(-ln(theta) * 2j / head_dim), half-split
rotation of the whole head (src/backends/vulkan/shaders/tensor.comp:318-327).  The
frequencies are computed once on the host in float64 and rounded to float32; the
angle itself is formed in float32 on the device.

Options of ``rotary``: ``rotary_dim`` (the first columns of a head that rotate; the rest pass), ``layout`` ("half":
column j pairs with j + rotary_dim/2; "interleaved": column 2j with 2j + 1) and ``scaling``
({"factor", "low", "high", "original"}): frequencies rescaled by wavelength l = 2 pi / f, kept where
l < original/high, divided by factor where l > original/low, and blended linearly in original/l between the two.
A mixer may hand ``place`` a ``HeadPrep``: a bias over the packed row and an RMS norm per head of queries and keys
that come before the rotation; the position part then does all of it in one kernel.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import POSITIONS, HeadPrep, HeadShape, Positions
from .spec import PartSpec


def scaled_frequencies(f: torch.Tensor, scaling) -> torch.Tensor:
    """The frequencies ``f`` (float64) rescaled by wavelength: see the module's header."""
    factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
    original = float(scaling["original"])
    wave = 2.0 * math.pi / f
    s = ((original / wave - low) / (high - low)).clamp(0.0, 1.0)
    blended = (1.0 - s) * f / factor + s * f
    return torch.where(wave < original / high, f, torch.where(wave > original / low, f / factor, blended))


def _prepare_and_place(prep, qkv, heads: HeadShape, step, line, append, rot_dim, inv_freq, interleaved) -> None:
    """Bias, head norms, rotation and append in the one kernel that does them all."""
    ops.head_prep(qkv, 0, heads.n_heads, heads.n_kv_heads, heads.n_kv_heads * heads.head_dim, heads.head_dim,
                  bias=prep.bias if prep else None, q_norm=prep.q_norm if prep else None,
                  k_norm=prep.k_norm if prep else None, norm_dim=prep.norm_dim if prep else 0,
                  eps=prep.eps if prep else 0.0, rot_dim=rot_dim, inv_freq=inv_freq, interleaved=interleaved,
                  tok_pos=step.tok_pos, tok_slot=step.tok_slot, line=line,
                  append=bool(append and line is not None and line.writes and heads.n_kv_heads > 0),
                  norm_whole=bool(prep.whole) if prep else False)


@POSITIONS.register("rotary")
class Rotary(Positions):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not (0 <= self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.layout = str(spec.get("layout", "half"))
        if self.layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout {self.layout!r} is neither 'half' nor 'interleaved'")
        self.scaling = spec.get("scaling")
        self.inv_freq: Optional[torch.Tensor] = None

    def frequencies(self) -> torch.Tensor:
        """float64, one per rotated pair."""
        j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        f = torch.exp(-math.log(self.theta) * 2.0 * j / max(1, self.rotary_dim))
        return scaled_frequencies(f, self.scaling) if self.scaling else f

    def prepare(self, device) -> None:
        self.inv_freq = self.frequencies().to(torch.float32).to(device)

    def place(self, qkv, heads: HeadShape, step, line, append: bool = True, prep: Optional[HeadPrep] = None) -> None:
        if prep is not None or self.layout != "half" or heads.n_kv_heads == 0:
            _prepare_and_place(prep, qkv, heads, step, line, append, self.rotary_dim, self.inv_freq,
                               self.layout == "interleaved")
            return
        ops.rope_cache_write(qkv, heads.n_heads, heads.n_kv_heads, heads.head_dim, self.rotary_dim, self.inv_freq,
                             step.tok_pos, step.tok_slot, line.k, line.v, line.page_table, line.page_size, line.ring,
                             line.slot_len, bool(append and line.writes))

    def project_and_place(self, x, w_qkv, heads: HeadShape, step, line):
        """For the few rows of a decode step, rotation and append ride in the product's epilogue."""
        if step.mode != "decode" or self.layout != "half" or heads.n_kv_heads == 0:
            return None
        if not ops.qkv_rope_cache_fusable(x, w_qkv, heads.head_dim, self.rotary_dim):
            return None
        return ops.qkv_rope_cache(x, w_qkv, heads.n_heads, heads.n_kv_heads, heads.head_dim, self.inv_freq,
                                  step.tok_pos, step.tok_slot, line.k, line.v, line.page_table, line.page_size,
                                  line.ring, line.slot_len, line.writes)


@POSITIONS.register("none")
class NoPositions(Positions):
    """Keys and queries are used as projected (rotated width 0)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.get("head_dim", 0))
        self.rotary_dim = 0
        self.inv_freq: Optional[torch.Tensor] = None

    def prepare(self, device) -> None:
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)

    def place(self, qkv, heads: HeadShape, step, line, append: bool = True, prep: Optional[HeadPrep] = None) -> None:
        if prep is not None:
            _prepare_and_place(prep, qkv, heads, step, line, append, 0, None, False)
        elif append and line.writes and heads.n_kv_heads > 0:
            ops.cache_append(qkv, heads.n_heads, heads.n_kv_heads, heads.head_dim, step.tok_pos, step.tok_slot, line)
