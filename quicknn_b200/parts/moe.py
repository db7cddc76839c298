"""Feed-forwards with a clamped gated activation, dense and routed.

``clamped_mlp``: down(act(gate(x), up(x))) with  g = min(gate, limit),  u = clamp(up, -limit, limit),
act = g * sigmoid(alpha * g) * (u + 1)  (alpha 1.702 unless given).

``routed_experts``: ``experts`` such feed-forwards, of which every token uses the ``top`` with the largest router
scores.  Router logits and scores are float32; scores are sigmoid(logit) (or a softmax over the experts), optionally
renormalised over the chosen ones; the score multiplies the expert's *input* (``weight_on`` = "input": the
sum over the chosen experts of expert(score * x)) or its output.  A shared expert of the same form, with sizes and
limit of its own, may run for every token beside them.  Options: ``activation`` "silu" (the plain gate
silu(gate) * up instead of the clamped one; no ``limit``); ``correction`` (a learned number per expert that is
added to the scores for the choice only; the weights are the scores without it); ``route_scale`` (multiplies the
weights); ``identity`` = n (the router has n more outputs than there are experts; those stand for identity
experts: such an entry contributes weight * x and owns no parameters); ``shared_gate`` (the shared
expert's output is multiplied by sigmoid(w . x), one number per token); ``gated`` False (experts without a gate:
down(act(up(x))) with ``activation`` one of ``ops.ACT_CODES``, e.g. "relu2"; each expert then owns ``up_proj`` and
``down_proj`` only); ``groups`` = (count, keep) (the experts form ``count`` equal groups of neighbours, a group's score is
the sum of its two largest ranking values, and only experts of the ``keep`` best groups can be chosen).  Everything from the router to the sum stays on the
device (no count is read back), so a decode step with routed layers is captured in a CUDA graph like any other.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward
from .linear import project, stack_rows
from .spec import PartSpec


@FEED_FORWARDS.register("clamped_mlp")
class ClampedMLP(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.limit = float(spec.params["limit"])
        self.alpha = float(spec.get("alpha", 1.702))
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

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        h = ops.gated_act_clamped(project(x, self.w_gate_up), self.limit, self.alpha)
        return project(h, self.w_down)


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_experts = int(p["experts"])
        self.top = int(p["top"])
        self.inter = int(p["intermediate_size"])
        self.activation = str(p.get("activation", "clamped"))
        self.gated = bool(p.get("gated", True))
        if self.gated and self.activation not in ("clamped", "silu"):
            raise ValueError(f"routed experts: activation {self.activation!r} is neither 'clamped' nor 'silu'")
        if not self.gated and self.activation not in ops.ACT_CODES:
            raise ValueError(f"routed experts without a gate: activation {self.activation!r} is not one of {sorted(ops.ACT_CODES)}")
        groups = p.get("groups")
        self.groups = None if groups is None else (int(groups[0]), int(groups[1]))
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or int(p["experts"]) % count or not (1 <= keep <= count) or keep * (int(p["experts"]) // count) < int(p["top"]):
                raise ValueError(f"routed experts: {count} groups of which {keep} are kept do not fit "
                                 f"{p['experts']} experts and top {p['top']}")
            if int(p.get("identity", 0)):
                raise ValueError("routed experts: groups of experts and identity experts do not go together")
        self.limit = float(p["limit"]) if self.activation == "clamped" else 0.0
        self.alpha = float(p.get("alpha", 1.702))
        self.identity = int(p.get("identity", 0))
        self.has_correction = bool(p.get("correction", False))
        self.route_scale = float(p.get("route_scale", 1.0))
        self.has_shared_gate = bool(p.get("shared_gate", False))
        self.score = str(p.get("score", "sigmoid"))
        self.renormalize = bool(p.get("renormalize", False))
        self.weight_on_input = str(p.get("weight_on", "input")) == "input"
        if self.identity < 0 or not (1 <= self.top <= self.n_experts + self.identity) or self.top > 16:
            raise ValueError(f"routed experts: top {self.top} of {self.n_experts} experts and {self.identity} identity "
                             f"experts (at most 16)")
        if self.score not in ops.MOE_SCORES:
            raise ValueError(f"routed experts: score {self.score!r} is not one of {sorted(ops.MOE_SCORES)}")
        shared: Optional[PartSpec] = p.get("shared")
        self.shared = None if shared is None else FEED_FORWARDS.get(shared.kind)(shared)
        if self.has_shared_gate and self.shared is None:
            raise ValueError("routed experts: a gate for a shared expert that is not there")
        self.correction: Optional[torch.Tensor] = None
        self.w_shared_gate: Optional[torch.Tensor] = None
        self.w_router_and_gate: Optional[torch.Tensor] = None
        self.w_router: Optional[torch.Tensor] = None
        self.w_gate_up: Optional[torch.Tensor] = None      # [experts, 2 * ff, width]
        self.w_down: Optional[torch.Tensor] = None         # [experts, width, ff]

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        H, I, E = int(p["hidden_size"]), int(p["intermediate_size"]), int(p["experts"])
        M = cls.PARAM_ROLE_MATRIX
        out: Dict[str, Tuple[Tuple[int, ...], str]] = {"router": ((E + int(p.get("identity", 0)), H), M)}
        if p.get("correction", False):
            out["correction"] = ((E + int(p.get("identity", 0)),), cls.PARAM_ROLE_NORM)
        if p.get("shared_gate", False):
            out["shared_gate"] = ((1, H), M)
        for e in range(E):
            if p.get("gated", True):
                out[f"experts.{e}.gate_proj"] = ((I, H), M)
            out[f"experts.{e}.up_proj"] = ((I, H), M)
            out[f"experts.{e}.down_proj"] = ((H, I), M)
        shared: Optional[PartSpec] = p.get("shared")
        if shared is not None:
            for k, v in FEED_FORWARDS.get(shared.kind).param_shapes(shared).items():
                out["shared." + k] = v
        return out

    def load(self, tensors, compute_dtype, device) -> None:
        E = self.n_experts
        self.w_router = tensors["router"].contiguous()
        if self.gated:
            self.w_gate_up = torch.stack([stack_rows([tensors[f"experts.{e}.gate_proj"], tensors[f"experts.{e}.up_proj"]])
                                          for e in range(E)]).contiguous()
        else:                                               # up rows alone: [experts, ff, width]
            self.w_gate_up = torch.stack([tensors[f"experts.{e}.up_proj"] for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"experts.{e}.down_proj"] for e in range(E)]).contiguous()
        if self.w_gate_up.dtype != self.w_down.dtype:
            wide = torch.float32
            self.w_gate_up, self.w_down = self.w_gate_up.to(wide), self.w_down.to(wide)
        if self.has_correction:
            self.correction = tensors["correction"].to(torch.float32).contiguous()
        if self.has_shared_gate:
            self.w_shared_gate = tensors["shared_gate"].contiguous()
            if self.w_shared_gate.dtype == self.w_router.dtype:
                # the gate's row behind the router's: the router's kernel forms its logit in the same pass
                both = stack_rows([self.w_router, self.w_shared_gate])
                n = self.w_router.shape[0]
                self.w_router_and_gate, self.w_router, self.w_shared_gate = both, both[:n], both[n:]
        if self.shared is not None:
            self.shared.load({k[len("shared."):]: v for k, v in tensors.items() if k.startswith("shared.")},
                             compute_dtype, device)

    def weight_bytes(self) -> int:
        n = sum(w.numel() * w.element_size() for w in (self.w_router, self.w_gate_up, self.w_down, self.correction,
                                                       self.w_shared_gate) if w is not None)
        return n + (self.shared.weight_bytes() if self.shared is not None else 0)

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        if self.w_router_and_gate is not None:
            sel_e, sel_w, gate = ops.moe_route(x, self.w_router_and_gate, self.top, self.score, self.renormalize,
                                               self.correction, self.route_scale, extra=1, groups=self.groups)
        else:
            sel_e, sel_w = ops.moe_route(x, self.w_router, self.top, self.score, self.renormalize, self.correction,
                                         self.route_scale, groups=self.groups)
            gate = ops.small_linear_f32(x, self.w_shared_gate) if self.has_shared_gate else None
        shared = self.shared.forward(x, step) if self.shared is not None else None
        xe = x if x.dtype == self.w_gate_up.dtype else ops.cast(x, self.w_gate_up.dtype)
        act = ops.GATED_CLAMPED if self.activation == "clamped" else ops.ACT_CODES[self.activation]
        return ops.moe_experts(xe, sel_e, sel_w, self.top, self.w_gate_up, self.w_down, act, self.limit,
                               self.alpha, self.weight_on_input, shared, shared_gate=gate, identity=self.identity > 0,
                               gated=self.gated)
