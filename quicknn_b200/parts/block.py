"""Blocks: how norms, mixer and feed-forward sit around the residual stream.

``sandwich`` (Gemma 2, src/models/QuickNN.Models.Gemma2.pas:166-189): a norm before
and after each sublayer, the post-norm applied to the sublayer's output before it
is added:  x += post(mixer(pre(x)));  x += post(ff(pre(x))).
``prenorm``: x += m mixer(pre(x));  x += m ff(pre(x)), with a constant m (``residual_mult``, 1 unless given) and a
feed-forward that a layer may lack.  The add and the norm that follows are one kernel for an RMSNorm and for every norm
that offers ``add_then`` (the dynamic tanh).

``postnorm``: x += norm(mixer(x));  x += norm(ff(x)): the sublayers read the stream itself and only what they give
is normed (a layer norm here; any norm unfused).  A mixer's ``out_bias`` and the mean of a ``parallel`` mixer's
branches are formed inside the kernel that norms and adds.

``parallel``: h = norm(x);  x += mixer(h) + ff(h): a single norm feeds the mixer and the feed-forward alike, and their sum is
added to the stream (a layer may lack the feed-forward).  With a ``group_rmsnorm`` the add and the next layer's
norm are one kernel.

The residual stream is float32 in both precisions.  When the norms are RMSNorm the
post-norm, the add and the next pre-norm run as one kernel; that also holds across the
border of two layers: ``forward`` may be handed its input already normed (``normed``) and
may be asked to apply the first norm of the layer that runs next (``next_norm``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block
from .norm import GroupRMSNorm, LayerNorm, NoNorm, RMSNorm
from .parallel import ParallelMixer
from .spec import LayerSpec, PartSpec


class _LayerParts(Block):
    NORM_NAMES: Tuple[str, ...] = ()

    def __init__(self, layer: LayerSpec):
        super().__init__(layer.block)
        self.layer = layer
        self.mixer = MIXERS.get(layer.mixer.kind)(layer.mixer)
        self.ff = None if layer.feed_forward is None else FEED_FORWARDS.get(layer.feed_forward.kind)(layer.feed_forward)
        names = self.norm_names(layer)
        missing = [n for n in names if n not in layer.norms]
        if missing:
            raise ValueError(f"block '{layer.block.kind}' needs the norms {missing}")
        self.norms = {n: NORMS.get(layer.norms[n].kind)(layer.norms[n]) for n in names}

    @classmethod
    def norm_names(cls, layer: LayerSpec) -> Tuple[str, ...]:
        """The norms that this arrangement has for this layer (a layer without a feed-forward has none around it)."""
        if layer.feed_forward is None:
            return tuple(n for n in cls.NORM_NAMES if not n.endswith("_ff"))
        return cls.NORM_NAMES

    @classmethod
    def layer_param_shapes(cls, layer: LayerSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        out: Dict[str, Tuple[Tuple[int, ...], str]] = {}
        for k, v in MIXERS.get(layer.mixer.kind).param_shapes(layer.mixer).items():
            out["mixer." + k] = v
        if layer.feed_forward is not None:
            for k, v in FEED_FORWARDS.get(layer.feed_forward.kind).param_shapes(layer.feed_forward).items():
                out["ff." + k] = v
        for n in cls.norm_names(layer):
            for k, v in NORMS.get(layer.norms[n].kind).param_shapes(layer.norms[n]).items():
                out[f"norms.{n}.{k}"] = v
        return out

    def load(self, tensors, compute_dtype, device) -> None:
        def sub(prefix):
            return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
        self.mixer.load(sub("mixer."), compute_dtype, device)
        if self.ff is not None:
            self.ff.load(sub("ff."), compute_dtype, device)
        for n, part in self.norms.items():
            part.load(sub(f"norms.{n}."), compute_dtype, device)

    def weight_bytes(self) -> int:
        return (self.mixer.weight_bytes() + (self.ff.weight_bytes() if self.ff is not None else 0)
                + sum(n.weight_bytes() for n in self.norms.values()))

    def scratch_need(self, step) -> int:
        return max(self.mixer.scratch_need(step), self.ff.scratch_need(step) if self.ff is not None else 0)

    def schedule(self, step) -> tuple:
        return self.mixer.schedule(step) + (self.ff.schedule(step) if self.ff is not None else ())


@BLOCKS.register("sandwich")
class SandwichBlock(_LayerParts):
    NORM_NAMES = ("pre_mixer", "post_mixer", "pre_ff", "post_ff")

    def first_norm(self):
        return self.norms["pre_mixer"]

    def forward(self, resid: torch.Tensor, step, line, normed=None, next_norm=None):
        """Returns the residual stream, or (residual stream, next_norm(residual stream)) when
        ``next_norm`` (an RMSNorm) is given."""
        nm = self.norms
        act = step.act_dtype
        n = normed if normed is not None else nm["pre_mixer"](resid, act)
        y = self.mixer.forward(n, step, line)
        if isinstance(nm["post_mixer"], RMSNorm) and isinstance(nm["pre_ff"], RMSNorm):
            n = nm["post_mixer"].add_to(resid, y, then=nm["pre_ff"], out_dtype=act)
        else:
            ops.add_(resid, nm["post_mixer"](y, act))
            n = nm["pre_ff"](resid, act)
        y = self.ff.forward(n, step)
        if isinstance(nm["post_ff"], RMSNorm):
            if isinstance(next_norm, RMSNorm):
                return resid, nm["post_ff"].add_to(resid, y, then=next_norm, out_dtype=act)
            nm["post_ff"].add_to(resid, y)
        else:
            ops.add_(resid, nm["post_ff"](y, act))
        if next_norm is not None:
            return resid, next_norm(resid, act)
        return resid


@BLOCKS.register("prenorm")
class PreNormBlock(_LayerParts):
    NORM_NAMES = ("pre_mixer", "pre_ff")

    def first_norm(self):
        return self.norms["pre_mixer"]

    def __init__(self, layer: LayerSpec):
        super().__init__(layer)
        # what a sublayer gives is multiplied by this constant before it is added (1: the usual pre-norm block)
        self.mult = float(layer.block.get("residual_mult", 1.0))

    def _add(self, resid: torch.Tensor, y: torch.Tensor, then, act):
        """resid += mult * y, and then(resid) in the same kernel when ``then`` is an RMSNorm."""
        if isinstance(then, RMSNorm):
            return ops.add_scaled_rmsnorm(resid, y, self.mult, then.weight, then.eps, then.unit_offset, act)
        if self.mult == 1.0 and hasattr(then, "add_then"):       # a norm that has the add in its own kernel
            return then.add_then(resid, y, act)
        if self.mult == 1.0:
            ops.add_(resid, y)
        else:
            ops.add_scaled_rmsnorm(resid, y, self.mult)
        return None if then is None else then(resid, act)

    def forward(self, resid: torch.Tensor, step, line, normed=None, next_norm=None):
        act = step.act_dtype
        n = normed if normed is not None else self.norms["pre_mixer"](resid, act)
        y = self.mixer.forward(n, step, line)
        if self.ff is not None:
            n = self._add(resid, y, self.norms["pre_ff"], act)
            y = self.ff.forward(n, step)
        n = self._add(resid, y, next_norm, act)
        if next_norm is not None:
            return resid, n
        return resid


@BLOCKS.register("postnorm")
class PostNormBlock(_LayerParts):
    """x += norm(mixer(x)); x += norm(ff(x)).  What a sublayer reads is the stream in the activations' element type:
    the kernel that adds a sublayer's normed output writes that copy too (and hands it to the next layer when that
    one also reads the stream as it is)."""

    NORM_NAMES = ("post_mixer", "post_ff")

    def __init__(self, layer: LayerSpec):
        super().__init__(layer)
        self._reads = NoNorm(PartSpec("none", {}))
        if hasattr(self.mixer, "defer_out_bias"):           # the output's bias rides in the kernel that norms and adds
            self.mixer.defer_out_bias = True

    def first_norm(self):
        return self._reads

    def _add(self, resid: torch.Tensor, y, norm, act, want_copy: bool, bias=None, branches=None):
        """resid += norm(y); returns the new stream as activations when ``want_copy``."""
        copy = act if want_copy else None
        if isinstance(norm, LayerNorm):
            if branches is not None:
                mixer, outs = branches
                return ops.add_mean_layernorm(resid, outs, mixer.out_weights, mixer.eps, norm.weight, norm.eps, copy)
            return norm.add_to(resid, y, bias=bias, copy_dtype=copy)
        if branches is not None:
            mixer, outs = branches
            y = ops.mean_rmsnorm(outs, mixer.out_weights, mixer.eps, act)
        if bias is not None:
            y = ops.add_bias_(y, bias)
        ops.add_(resid, norm(y, act))
        return ops.cast(resid, act) if want_copy else None

    def forward(self, resid: torch.Tensor, step, line, normed=None, next_norm=None):
        act = step.act_dtype
        nm = self.norms
        n = normed if normed is not None else ops.cast(resid, act)
        handed = isinstance(next_norm, NoNorm)
        last_is_mixer = self.ff is None
        want = (not last_is_mixer) or handed
        if isinstance(self.mixer, ParallelMixer) and isinstance(nm["post_mixer"], LayerNorm):
            outs = self.mixer.forward_branches(n, step, line)
            n = self._add(resid, None, nm["post_mixer"], act, want, branches=(self.mixer, outs))
        else:
            y = self.mixer.forward(n, step, line)
            bias = self.mixer.out_bias if getattr(self.mixer, "defer_out_bias", False) else None
            n = self._add(resid, y, nm["post_mixer"], act, want, bias=bias)
        if self.ff is not None:
            y = self.ff.forward(n, step)
            n = self._add(resid, y, nm["post_ff"], act, handed)
        if next_norm is None:
            return resid
        return resid, (n if handed else next_norm(resid, act))


@BLOCKS.register("parallel")
class ParallelBlock(_LayerParts):
    """h = norm(x); x += mixer(h) + ff(h)."""

    NORM_NAMES = ("pre",)

    @classmethod
    def norm_names(cls, layer: LayerSpec) -> Tuple[str, ...]:
        return cls.NORM_NAMES

    def first_norm(self):
        return self.norms["pre"]

    def forward(self, resid: torch.Tensor, step, line, normed=None, next_norm=None):
        act = step.act_dtype
        h = normed if normed is not None else self.norms["pre"](resid, act)
        a = self.mixer.forward(h, step, line)
        f = self.ff.forward(h, step) if self.ff is not None else None
        if isinstance(next_norm, GroupRMSNorm):
            return resid, next_norm.after_add(resid, a, f, act)
        ops.add2_group_rmsnorm(resid, a, f)
        if next_norm is not None:
            return resid, next_norm(resid, act)
        return resid
