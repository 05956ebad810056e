"""Gates: parts that turn a block's input into logits whose sigmoid multiplies something else."""
from __future__ import annotations

import torch

from .base import Part, Product, StepContext
from .registry import register_gate
from .spec import ParamSpec, PartSpec


@register_gate("linear_gate")
class LinearGate(Part):
    """z = W h + b, ``width`` numbers per token from an input ``hidden_size`` wide; the consumer takes the sigmoid
    (in float32, inside the kernel that applies it).  Tensors: the matrix under ``weight_name`` ("" if the prefix
    alone names it) and the bias under ``bias_name`` (None: no bias)."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.width = int(spec["width"])
        self.weight_name = spec.get("weight_name", "weight")
        self.bias_name = spec.get("bias_name", "bias")
        self.weight = self.bias = None

    def parameters(self):
        p = {self.weight_name: ParamSpec((self.width, self.hidden))}
        if self.bias_name is not None:
            p[self.bias_name] = ParamSpec((self.width,), role="vector", init=("normal", 0.0, 0.5))
        return p

    def load(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()
        self.bias = tensors.get(self.bias_name) if self.bias_name is not None else None

    def logits(self, h, ctx: StepContext, name: str) -> Product:
        """The logits WITHOUT the bias as a float32 product (possibly split-K parts); the consumer adds ``bias``."""
        return ctx.rt.linear(h, self.weight, ctx.ws, name, out_dtype=torch.float32)
