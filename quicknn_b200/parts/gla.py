"""Gated linear attention: a recurrent mixer whose state is a matrix per head (``gla``), and its sibling whose forget
gate also decides what is written (``hgrn2``, below).

    q = W_q x * dim^(-1/2),  k = W_k x  (heads x dim),   v = W_v x  (heads x vdim)
    a = sigmoid(W_a2 (W_a1 x) + b)^(1/tau)               a decay per key channel, float32
    S_t = diag(a_t) S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t                 S: [dim, vdim] float32 per head
    y = W_o ( rmsnorm_per_head(o) * silu(W_g x) )

The state lives in the cache's fixed-size state region, one [heads, dim, vdim] float32 block per slot, zeroed
when the slot is handed out; the mixer needs no keys or values.  A step walks each sequence's rows in order from
the slot's state and leaves the new state there, so whole prompts, portions and single tokens are one kernel.
q, k, v and the gate are one stacked product; the decay's logits are formed in float32 from the low-rank
projection's output, and the decay itself (log-sigmoid, division by tau, exponential) in the same kernel's epilogue.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, CacheNeed, Mixer, StateNeed
from .linear import project, stack_rows
from .spec import PartSpec


@MIXERS.register("gla")
class GatedLinearAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.decay_rank = int(p["decay_rank"])
        self.tau = float(p["tau"])
        self.eps = float(p["eps"])
        if not self.tau > 0:
            raise ValueError(f"gla: tau must be positive (got {self.tau})")
        if self.dim > 256:
            raise ValueError(f"gla: at most 256 key channels per head (got {self.dim})")
        self.w_in: Optional[torch.Tensor] = None         # q | k | v | gate rows
        self.w_a1: Optional[torch.Tensor] = None
        self.w_a2: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        W, H, d, vd, ra = int(p["hidden_size"]), int(p["n_heads"]), int(p["dim"]), int(p["vdim"]), int(p["decay_rank"])
        M, N = cls.PARAM_ROLE_MATRIX, cls.PARAM_ROLE_SCALE
        return {"q": ((H * d, W), M), "k": ((H * d, W), M), "v": ((H * vd, W), M), "gate": ((H * vd, W), M),
                "o": ((W, H * vd), M), "norm": ((vd,), N), "a1": ((ra, W), M), "a2": ((H * d, ra), M),
                "a2_bias": ((H * d,), cls.PARAM_ROLE_NORM)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_in = stack_rows([tensors["q"], tensors["k"], tensors["v"], tensors["gate"]])
        self.w_a1 = tensors["a1"].contiguous()
        self.w_a2 = tensors["a2"].contiguous()
        self.bias = tensors["a2_bias"].contiguous()
        self.norm = tensors["norm"].contiguous()
        self.w_o = tensors["o"].contiguous()

    def weight_bytes(self) -> int:
        ws = (self.w_in, self.w_a1, self.w_a2, self.bias, self.norm, self.w_o)
        return sum(w.numel() * w.element_size() for w in ws)

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.n_heads, self.dim, self.vdim), "float32")

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        H, d, vd = self.n_heads, self.dim, self.vdim
        p = project(x, self.w_in)                                         # q | k | v | gate
        a = ops.small_linear_f32(project(x, self.w_a1), self.w_a2, self.bias, self.tau)     # the decays, float32
        o = ops.gla_scan(p, 0, H * d, 2 * H * d, a, float(d) ** -0.5,
                         None if step.mode == "decode" else step.seq_row0,
                         None if step.mode == "decode" else step.seq_len,
                         step.slots, line.state, step.n_seqs, H, d, vd,
                         longest=0 if step.mode == "decode" else step.max_q_len)
        g = ops.gla_norm_gate(o, self.norm, self.eps, p, 2 * H * d + H * vd, H, vd)
        return project(g, self.w_o)


@MIXERS.register("hgrn2")
class HGRN2(Mixer):
    """A matrix memory without keys: the forget gate decays the rows of the state and its complement is written
    (Qin et al., "HGRN2: Gated Linear RNNs with State Expansion").

        q = silu(W_q x)  (heads x dim),   v = W_v x  (heads x vdim)
        f = l + (1 - l) * sigmoid(W_f x + b)          per head and key channel, l a learned lower bound; float32
        S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,   o_t = S_t^T q_t
        y = W_o concat_h( o_h / rms(o_h) * w_norm )   w_norm: [vdim], shared by the heads

    q, the gate's pre-activations and v are one stacked product; one kernel applies the silu to q and forms f in
    float32; the scan is the ``gla`` scan with the key read as 1 - f (float32, inside the kernel).  State as ``gla``."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.eps = float(p["eps"])
        if self.dim > 256:
            raise ValueError(f"hgrn2: at most 256 key channels per head (got {self.dim})")
        self.w_in: Optional[torch.Tensor] = None         # q | f | v rows
        self.f_bias: Optional[torch.Tensor] = None
        self.lower: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        W, H, d, vd = int(p["hidden_size"]), int(p["n_heads"]), int(p["dim"]), int(p["vdim"])
        M, B = cls.PARAM_ROLE_MATRIX, cls.PARAM_ROLE_NORM
        return {"q": ((H * d, W), M), "f": ((H * d, W), M), "f_bias": ((H * d,), B), "lower": ((H * d,), B),
                "v": ((H * vd, W), M), "norm": ((vd,), cls.PARAM_ROLE_SCALE), "o": ((W, H * vd), M)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_in = stack_rows([tensors["q"], tensors["f"], tensors["v"]])
        self.f_bias = tensors["f_bias"].contiguous()
        self.lower = tensors["lower"].contiguous()
        self.norm = tensors["norm"].contiguous()
        self.w_o = tensors["o"].contiguous()

    def weight_bytes(self) -> int:
        ws = (self.w_in, self.f_bias, self.lower, self.norm, self.w_o)
        return sum(w.numel() * w.element_size() for w in ws)

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.n_heads, self.dim, self.vdim), "float32")

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        H, d, vd = self.n_heads, self.dim, self.vdim
        p = project(x, self.w_in)                                         # q | f's pre-activations | v
        f = ops.bounded_gates(p, 0, H * d, H * d, H * d, self.f_bias, self.lower)       # silu(q) in place; f, float32
        decode = step.mode == "decode"
        o = ops.gla_scan(p, 0, 0, 2 * H * d, f, 1.0, None if decode else step.seq_row0,
                         None if decode else step.seq_len, step.slots, line.state, step.n_seqs, H, d, vd,
                         longest=0 if decode else step.max_q_len, key_from_decay=True)
        n = ops.head_norm_gate(o, vd, H, vd, self.eps, None, 0, "none", weight=self.norm, out_dtype=p.dtype)
        return project(n, self.w_o)
