"""Feed-forward parts.  ``gated_mlp``: down(act(gate(x)) * up(x)).  ``mlp``: down(act(up(x))), without a gate.
``mlp`` also takes the activation ``xielu`` with two learned numbers p, q per layer (the parameter ``act_params``):
z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.

Reference: two products and a GO_GEGLU dispatch, then the down product
(src/models/QuickNN.Models.Gemma2.pas:184-187; gelu_tanh at shaders/tensor.comp:23).
Gate and up are one product against the stacked matrix; for up to 64 rows the
activation is the product's epilogue.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import math

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward
from .linear import project, stack_rows
from .spec import PartSpec


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.get("activation", "gelu_tanh"))
        if self.activation not in ops.ACT_CODES:
            raise ValueError(f"activation {self.activation!r} is not one of {sorted(ops.ACT_CODES)}")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        H, I = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        M = cls.PARAM_ROLE_MATRIX
        return {"gate_proj": ((I, H), M), "up_proj": ((I, H), M), "down_proj": ((H, I), M)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_gate_up = stack_rows([tensors["gate_proj"], tensors["up_proj"]])
        self.w_down = tensors["down_proj"].contiguous()
        why = ops.linear_refusal(self.w_gate_up.dtype, self.hidden) or ops.linear_refusal(self.w_down.dtype, self.inter)
        if why:
            raise ValueError(f"gated feed-forward: {why}")

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        h = project(x, self.w_gate_up, epilogue=ops.EPI_GATED, activation=self.activation)
        return project(h, self.w_down)


@FEED_FORWARDS.register("mlp")
class MLP(FeedForward):
    """down(act(up(x))) with ``activation`` one of ``ops.ACT_CODES`` (``relu2``: the square of relu) or ``xielu``."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.params["activation"])
        if self.activation != "xielu" and self.activation not in ops.ACT_CODES:
            raise ValueError(f"activation {self.activation!r} is not one of {sorted(ops.ACT_CODES) + ['xielu']}")
        self.xielu = (0.0, 0.0)           # softplus(p), 1/2 + softplus(q)
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        H, I = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        M = cls.PARAM_ROLE_MATRIX
        out = {"up_proj": ((I, H), M), "down_proj": ((H, I), M)}
        if str(spec.params["activation"]) == "xielu":
            out["act_params"] = ((2,), cls.PARAM_ROLE_NORM)
        return out

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_up = tensors["up_proj"].contiguous()
        self.w_down = tensors["down_proj"].contiguous()
        if self.activation == "xielu":
            # the two constants once, when the model is built (float64 on the host, rounded to float32 by the kernel's
            # arguments)
            p, q = (float(v) for v in tensors["act_params"].detach().to("cpu", torch.float64).tolist())
            softplus = lambda z: max(z, 0.0) + math.log1p(math.exp(-abs(z)))          # noqa: E731
            self.xielu = (softplus(p), 0.5 + softplus(q))

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down))

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        if self.activation == "xielu":
            # the product kernels for whole prompts apply it in their epilogue, with its two constants
            return project(project(x, self.w_up, epilogue=ops.EPI_ACT, activation="xielu", act_consts=self.xielu),
                           self.w_down)
        return project(project(x, self.w_up, epilogue=ops.EPI_ACT, activation=self.activation), self.w_down)
