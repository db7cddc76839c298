"""Norms.  ``layernorm``: y = (x - mean) / sqrt(var + eps) * w, var the mean of the squared deviations, no bias.
``none``: the rows as they are, in the element type asked for (what a sublayer reads when it reads the stream itself).
``rmsnorm``: y = x / sqrt(mean(x^2) + eps) * (w + offset), offset 1 for the
"(1 + w)" flavour.  Reference: GO_NORM without centring and bias
(src/backends/vulkan/shaders/tensor.comp:63-72; Operations.pas:129-149); the
reference's files hold 1 + w already (src/models/QuickNN.Models.Gemma2.pas:58), the
checkpoints read here hold w.
``group_rmsnorm``: the row is cut into ``groups`` equal consecutive pieces, each is divided by its own
sqrt(mean(piece^2) + eps), and the whole is multiplied by w (one group: an RMS norm with a plain weight).
``dynamic_tanh``: y = tanh(alpha x) * w + b with one learned number alpha, a weight and a bias per column; no mean and
no variance are formed (Zhu et al., "Transformers without Normalization").  Parameters ``weight``, ``alpha`` (a
scalar) and ``b``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import NORMS, Norm
from .spec import PartSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.unit_offset = bool(spec.get("unit_offset", False))
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        role = cls.PARAM_ROLE_NORM if spec.get("unit_offset", False) else cls.PARAM_ROLE_SCALE
        return {"weight": ((int(spec.params["size"]),), role)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.weight = tensors["weight"].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.unit_offset, out_dtype)

    def of_embedding(self, tokens: torch.Tensor, table: torch.Tensor, scale: float, out_dtype: torch.dtype):
        """(embedded rows, self(embedded rows)) in one kernel: the first norm of a model's first layer."""
        return ops.embed_rmsnorm(tokens, table, scale, self.weight, self.eps, self.unit_offset, out_dtype)

    def add_to(self, resid: torch.Tensor, y: torch.Tensor, then: Optional["RMSNorm"] = None,
               out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """resid += self(y); returns then(resid) when ``then`` is given, in one kernel."""
        if then is None:
            return ops.add_rmsnorm(resid, y, self.weight, self.eps, self.unit_offset)
        return ops.add_rmsnorm(resid, y, self.weight, self.eps, self.unit_offset,
                               then.weight, then.eps, then.unit_offset, out_dtype)


@NORMS.register("group_rmsnorm")
class GroupRMSNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.groups = int(spec.get("groups", 1))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"group_rmsnorm: {self.groups} groups do not divide the width {self.size}")
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {"weight": ((int(spec.params["size"]),), cls.PARAM_ROLE_SCALE)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.weight = tensors["weight"].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.group_rmsnorm(x, self.weight, self.eps, self.groups, out_dtype)

    def of_embedding_rows(self, tokens, table, scale: float, pos_table, tok_pos, out_dtype: torch.dtype):
        """(embedded rows with their position vectors, self(those rows)) in one kernel."""
        return ops.embed_pos(tokens, table, scale, pos_table, tok_pos, self.weight, self.eps, self.groups, out_dtype)

    def after_add(self, resid: torch.Tensor, a, b, out_dtype: torch.dtype) -> torch.Tensor:
        """resid += a + b, then self(resid), in one kernel."""
        return ops.add2_group_rmsnorm(resid, a, b, self.weight, self.eps, self.groups, out_dtype)


@NORMS.register("layernorm")
class LayerNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {"weight": ((int(spec.params["size"]),), cls.PARAM_ROLE_SCALE)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.weight = tensors["weight"].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.layernorm(x, self.weight, self.eps, out_dtype)

    def add_to(self, resid: torch.Tensor, y: torch.Tensor, bias: Optional[torch.Tensor] = None,
               copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """resid += self(y + bias); with ``copy_dtype`` returns the new stream in that element type, in one kernel."""
        return ops.add_layernorm(resid, y, self.weight, self.eps, bias, copy_dtype)


@NORMS.register("none")
class NoNorm(Norm):
    """No norm at all: the rows in the element type asked for."""

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.cast(x, out_dtype)


@NORMS.register("dynamic_tanh")
class DynamicTanh(Norm):
    """tanh(alpha x) * w + b.  alpha is read once, when the model is built, and travels as a kernel argument."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.alpha = 1.0
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        n = int(spec.params["size"])
        return {"weight": ((n,), cls.PARAM_ROLE_SCALE), "alpha": ((), cls.PARAM_ROLE_SCALE), "b": ((n,), cls.PARAM_ROLE_NORM)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.weight = tensors["weight"].contiguous()
        self.bias = tensors["b"].contiguous()
        self.alpha = float(tensors["alpha"].detach().to("cpu", torch.float32).reshape(()).item())

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.weight, self.bias))

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.dyt(x, self.alpha, self.weight, self.bias, out_dtype)

    def of_embedding(self, tokens: torch.Tensor, table: torch.Tensor, scale: float, out_dtype: torch.dtype):
        """(embedded rows, self(embedded rows)) in one kernel: the first norm of a model's first layer."""
        return ops.embed_dyt(tokens, table, scale, self.alpha, self.weight, self.bias, out_dtype)

    def add_then(self, resid: torch.Tensor, y, out_dtype: torch.dtype, extra=None) -> torch.Tensor:
        """resid += y (+ extra, float32 rows), then self(resid), in one kernel."""
        return ops.add_dyt(resid, y, extra, self.alpha, self.weight, self.bias, out_dtype)
