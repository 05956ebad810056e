"""RMSNorm: width and eps are parameters of the part (mini_hisparse/model.py:43-51)."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Norm, Product, StepContext
from .registry import register_norm
from .spec import ParamSpec, PartSpec


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * weight, computed in float32 from the float32 residual.

    The weight is a plain multiplier (not 1 + w) and there is no bias, as in the reference.  With
    ``offset`` (a number, usually 1) the stored tensor is a deviation around zero and the multiplier is
    offset + w: the sum is formed once at load, in float32, and the kernels see a plain weight.
    With ``gain`` (a number) the multiplier is gain * w, formed once at load in float32: a block that adds a
    fixed multiple of a normalised branch to the stream.
    With ``delta`` the kernel first adds it to the residual (and writes the sum back when all
    rows are processed), so the residual add costs no extra pass over memory.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])
        self.weight_name = spec.get("weight_name", "weight")     # "" if the tensor is named by the prefix alone
        self.offset = float(spec.get("offset", 0.0))
        self.gain = float(spec.get("gain", 1.0))
        self.weight = None

    def parameters(self):
        return {self.weight_name: ParamSpec((self.width,), role="vector", init=("normal", 1.0 - self.offset, 0.1))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name]
        if self.offset:
            self.weight = self.weight.float() + self.offset
        if self.gain != 1.0:
            self.weight = self.weight.float() * self.gain

    def forward_post(self, x, ctx: StepContext, delta: Product | None, alpha: float = 1.0, keep: float = 0.0,
                     name="x_copy"):
        """Post-norm, in place: x <- keep * x + rms(alpha * x + delta) * weight (float32).
        Returns the new rows in the compute dtype (x itself when that is float32): what the next
        product reads, since nothing normalises the stream again before it."""
        copy = None if ctx.rt.dtype == torch.float32 else ctx.ws.get(name, tuple(x.shape), ctx.rt.dtype)
        if delta is not None:
            delta = delta.settle_also(x)
        if delta is None:
            K.norm_mix(x, self.weight, self.eps, alpha=alpha, keep=keep, copy=copy)
        else:
            K.norm_mix(x, self.weight, self.eps, delta=delta.tensor, nsplit=delta.nsplit,
                       split_stride=delta.split_stride, alpha=alpha, keep=keep, copy=copy)
        return x if copy is None else copy

    def forward(self, x, ctx: StepContext, delta: Product | None = None, rows=None, name="h"):
        R = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get(name, (R, self.width), ctx.rt.dtype)
        if delta is not None:
            delta = delta.settle_also(x)
        if delta is None:
            K.add_rmsnorm(x, self.weight, self.eps, out, rows=rows)
        else:
            K.add_rmsnorm(x, self.weight, self.eps, out, delta=delta.tensor, nsplit=delta.nsplit,
                          split_stride=delta.split_stride, rows=rows)
        return out


@register_norm("layernorm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * weight with var the mean of the squared deviations, no bias,
    in float32 from the float32 residual.  With ``delta`` the kernel adds it (and the product that
    rides along as ``delta.also``: the two sublayers of a parallel block) to the residual first and
    writes the sum back when all rows are processed."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])
        self.weight_name = spec.get("weight_name", "weight")
        self.weight = None

    def kernel_modules(self):
        return ("mixparts",)

    def parameters(self):
        return {self.weight_name: ParamSpec((self.width,), role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name]

    def forward(self, x, ctx: StepContext, delta: Product | None = None, rows=None, name="h"):
        R = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get(name, (R, self.width), ctx.rt.dtype)
        second = delta.also if delta is not None else None
        if second is not None and second.also is not None:
            second = second.settle_also(x)
        K.add_layernorm(x, self.weight, self.eps, out, delta=delta, delta2=second, rows=rows)
        return out
