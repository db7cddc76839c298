"""Matrix memories with one decay per head: a state S [dim, vdim] per head that every token decays and adds an outer
product to, read with the query.  Two mixers share one scan (``ops.memory_scan``):

``retention``: a fixed decay per head, no denominator, rotated queries and keys.

    q = rot(W_q x),  k = rot(W_k x) dim^(-1/2),  v = W_v x
    S_t = decay_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t
    y = W_o ( o / rms(o) per head  *  silu(W_g x) )

``mlstm``: exponential input gate and sigmoid forget gate per head, both soft-capped, kept bounded by a running maximum
m, with a normaliser vector n beside S (Beck et al., "xLSTM: Extended Long Short-Term Memory", the matrix memory).

    q = W_q x dim^(-1/2),  k = W_k x,  v = W_v x
    i = cap tanh((W_i x + b_i) / cap),   f = log sigmoid(cap tanh((W_f x + b_f) / cap))
    m_t = max(f + m_{t-1}, i)            (m_0 = 0)
    S_t = e^(f + m_{t-1} - m_t) S_{t-1} + e^(i - m_t) k v^T,    n_t likewise with k alone
    o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6)
    y = W_o ( o / rms(o) per head * w_norm * sigmoid(W_g x) )

``lightning``: a fixed decay per head on queries, keys and values that pass silu; no rotation and no other scale;
the read-out of all heads together is RMS-normed with a weight per column and multiplied by a sigmoid gate.

    q = silu(W_q x),  k = silu(W_k x),  v = silu(W_v x)
    S_t = decay_h S_{t-1} + k_t v_t^T,   o_t = S_t^T q_t
    y = W_o ( o / rms(o over all heads) * w_norm * sigmoid(W_g x) )

The state lives in the cache's fixed-size state region, float32, zeroed when the slot is handed out: for ``mlstm`` a
slot keeps [heads, dim, vdim + 1] (the last column is n: the normaliser is the state column of a value that is 1 in
every row) and then m per head.  One scan walks every sequence's rows in order from the slot's state and back, so
prompts, portions and single tokens are the same launches.  Gates, decays, rotation angles, the state and the norms
are float32 in both precisions; the rotated queries and keys of ``retention`` go into the scan as float32 rows (they are
not rounded to bfloat16 again).  The scale of the keys (retention) is applied on the query's side of o = S^T q, which is
linear in both.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheNeed, Mixer, StateNeed
from .linear import project, stack_rows
from .spec import PartSpec


class _MatrixMemory(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.eps = float(p["eps"])
        if self.dim > 256:
            raise ValueError(f"{spec.kind}: at most 256 key channels per head (got {self.dim})")
        self.w_in: Optional[torch.Tensor] = None         # q | k | v | gate rows
        self.w_o: Optional[torch.Tensor] = None

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def _rows(self, step):
        """(first rows, row counts, longest) of the step's sequences; a decode step is a row each."""
        if step.mode == "decode":
            return None, None, 0
        return step.seq_row0, step.seq_len, step.max_q_len


@MIXERS.register("retention")
class Retention(_MatrixMemory):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.decay = tuple(float(d) for d in p["decay"])
        if len(self.decay) != self.n_heads:
            raise ValueError(f"retention: {len(self.decay)} decays for {self.n_heads} heads")
        pos: PartSpec = p["position"]
        self.position = POSITIONS.get(pos.kind)(pos)
        self.rot_dim = int(getattr(self.position, "rotary_dim", 0))
        self.decay_dev: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        W, H, d, vd = int(p["hidden_size"]), int(p["n_heads"]), int(p["dim"]), int(p["vdim"])
        M = cls.PARAM_ROLE_MATRIX
        return {"q": ((H * d, W), M), "k": ((H * d, W), M), "v": ((H * vd, W), M), "gate": ((H * vd, W), M),
                "o": ((W, H * vd), M)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_in = stack_rows([tensors["q"], tensors["k"], tensors["v"], tensors["gate"]])
        self.w_o = tensors["o"].contiguous()
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)
        self.position.prepare(device)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.n_heads * self.dim * self.vdim,), "float32")

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        H, d, vd = self.n_heads, self.dim, self.vdim
        p = project(x, self.w_in)                                         # q | k | v | gate
        # rotated q and k, and v beside them, as float32 rows for the scan
        rows = torch.empty((p.shape[0], H * (2 * d + vd)), dtype=torch.float32, device=p.device)
        ops.head_prep(p, 0, H, H, H * vd, d, dst=rows, rot_dim=self.rot_dim, inv_freq=self.position.inv_freq,
                      interleaved=getattr(self.position, "layout", "half") == "interleaved", tok_pos=step.tok_pos)
        row0, lens, longest = self._rows(step)
        o = ops.memory_scan(rows, 0, H * d, 2 * H * d, self.decay_dev, 0, None, 0, float(d) ** -0.5, False, row0, lens,
                            step.slots, line.state, step.n_seqs, H, d, vd, longest=longest)
        g = ops.head_norm_gate(o, vd, H, vd, self.eps, p, 2 * H * d + H * vd, "silu")
        return project(g, self.w_o)


@MIXERS.register("lightning")
class LightningAttention(_MatrixMemory):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.decay = tuple(float(d) for d in spec.params["decay"])
        if len(self.decay) != self.n_heads:
            raise ValueError(f"lightning: {len(self.decay)} decays for {self.n_heads} heads")
        self.decay_dev: Optional[torch.Tensor] = None
        self.w_gate: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        W, H, d, vd = int(p["hidden_size"]), int(p["n_heads"]), int(p["dim"]), int(p["vdim"])
        M = cls.PARAM_ROLE_MATRIX
        return {"q": ((H * d, W), M), "k": ((H * d, W), M), "v": ((H * vd, W), M), "gate": ((H * vd, W), M),
                "o": ((W, H * vd), M), "norm": ((H * vd,), cls.PARAM_ROLE_SCALE)}

    def load(self, tensors, compute_dtype, device) -> None:
        # q | k | v are one product whose epilogue is the silu; the gate's logits are a product of their own
        self.w_in = stack_rows([tensors["q"], tensors["k"], tensors["v"]])
        self.w_gate = tensors["gate"].contiguous()
        self.w_o = tensors["o"].contiguous()
        self.norm = tensors["norm"].contiguous()
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_gate, self.w_o, self.norm))

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.n_heads * self.dim * self.vdim,), "float32")

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        H, d, vd = self.n_heads, self.dim, self.vdim
        p = project(x, self.w_in, epilogue=ops.EPI_ACT, activation="silu")          # silu(q | k | v)
        g = project(x, self.w_gate)
        row0, lens, longest = self._rows(step)
        o = ops.memory_scan(p, 0, H * d, 2 * H * d, self.decay_dev, 0, None, 0, 1.0, False, row0, lens, step.slots,
                            line.state, step.n_seqs, H, d, vd, longest=longest)
        # one norm over all heads together: a single "head" as wide as the row, a weight per column
        n = ops.head_norm_gate(o, H * vd, 1, H * vd, self.eps, g, 0, "sigmoid", weight=self.norm)
        return project(n, self.w_o)


@MIXERS.register("mlstm")
class MatrixLSTM(_MatrixMemory):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.cap = float(spec.params["gate_cap"])
        if not self.cap > 0:
            raise ValueError(f"mlstm: gate_cap must be positive (got {self.cap})")
        self.w_gates: Optional[torch.Tensor] = None      # input gates' rows, then forget gates'
        self.b_gates: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        W, H, d, vd = int(p["hidden_size"]), int(p["n_heads"]), int(p["dim"]), int(p["vdim"])
        M, B, S = cls.PARAM_ROLE_MATRIX, cls.PARAM_ROLE_NORM, cls.PARAM_ROLE_SCALE
        return {"q": ((H * d, W), M), "k": ((H * d, W), M), "v": ((H * vd, W), M), "gate": ((H * vd, W), M),
                "o": ((W, H * vd), M), "norm": ((H * vd,), S), "i": ((H, W), M), "i_bias": ((H,), B),
                "f": ((H, W), M), "f_bias": ((H,), B)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_in = stack_rows([tensors["q"], tensors["k"], tensors["v"], tensors["gate"]])
        self.w_o = tensors["o"].contiguous()
        self.w_gates = stack_rows([tensors["i"], tensors["f"]])
        self.b_gates = torch.cat([tensors["i_bias"].to(torch.float32), tensors["f_bias"].to(torch.float32)]).contiguous()
        self.norm = tensors["norm"].contiguous()

    def weight_bytes(self) -> int:
        ws = (self.w_in, self.w_o, self.w_gates, self.b_gates, self.norm)
        return sum(w.numel() * w.element_size() for w in ws)

    @property
    def _m_offset(self) -> int:
        return self.n_heads * self.dim * (self.vdim + 1)

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self._m_offset + self.n_heads,), "float32")

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        H, d, vd = self.n_heads, self.dim, self.vdim
        p = project(x, self.w_in)                                         # q | k | v | gate
        row0, lens, longest = self._rows(step)
        pre = ops.small_linear_f32(x, self.w_gates)                       # the gates' pre-activations, float32
        gates = ops.mlstm_gates(pre, self.b_gates, self.cap, row0, lens, step.slots, line.state, self._m_offset,
                                step.n_seqs, H)                           # decay | key weight | e^-m
        o = ops.memory_scan(p, 0, H * d, 2 * H * d, gates, 3 * H, gates, H, float(d) ** -0.5, True, row0, lens,
                            step.slots, line.state, step.n_seqs, H, d, vd, longest=longest)
        g = ops.head_norm_gate(o, vd + 1, H, vd, self.eps, p, 2 * H * d + H * vd, "sigmoid", weight=self.norm,
                               den=gates, den_col=2 * H)
        return project(g, self.w_o)
