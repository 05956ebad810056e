"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import FeedForward, Product, StepContext
from .registry import register_feed_forward
from .spec import ParamSpec, PartSpec


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)), no biases (mini_hisparse/model.py:63-71).

    gate_proj and up_proj are stacked into one [2 I, H] weight at load, in the layout the
    runtime's product wants (interleaved in blocks when the gate is fused into the product's
    epilogue); the checkpoint names stay gate_proj / up_proj / down_proj.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.gate_up = None
        self.gate_block = self.inter
        self.down = None

    def parameters(self):
        return {
            "gate_proj.weight": ParamSpec((self.inter, self.hidden)),
            "up_proj.weight": ParamSpec((self.inter, self.hidden)),
            "down_proj.weight": ParamSpec((self.hidden, self.inter)),
        }

    def load(self, tensors):
        self.gate_up, self.gate_block = self.rt.swiglu_layout(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, h, ctx: StepContext) -> Product:
        rt, ws = ctx.rt, ctx.ws
        act = rt.linear_swiglu(h, self.gate_up, self.gate_block, ws, "ff_act")
        return rt.linear(act, self.down, ws, "ff_out")


@register_feed_forward("mlp_act")
class ActivatedMLP(FeedForward):
    """down(act(up(x))), no gate, no biases; ``activation``: "relu2" (the square of relu), "silu" or
    "gelu_tanh", computed in float32 on the product's float32 output, or "polynorm":
    act(z) = a rms(z) + b rms(z^2) + c rms(z^3) + e with the powers taken element by element, each divided by its
    own root mean square over the token's ``intermediate_size`` values (``eps`` inside the root), and the four numbers
    (a, b, c, e) stored as the tensor ``coef_name`` (default "act").  Tensor names: ``up_name`` and
    ``down_name`` (default "up" and "down")."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "relu2")
        self.polynorm = self.activation == "polynorm"
        if not self.polynorm and (self.activation not in K.ACTIVATIONS or self.activation == "copy"):
            raise ValueError(f"unknown activation {self.activation!r}")
        self.up_name, self.down_name = spec.get("up_name", "up"), spec.get("down_name", "down")
        self.coef_name = spec.get("coef_name", "act")
        self.eps = float(spec["eps"]) if self.polynorm else 0.0
        self.up = self.down = self.coef = None

    def kernel_modules(self):
        return ("gateparts",) if self.polynorm else ("postnorm",)

    def parameters(self):
        p = {self.up_name: ParamSpec((self.inter, self.hidden)),
             self.down_name: ParamSpec((self.hidden, self.inter))}
        if self.polynorm:
            p[self.coef_name] = ParamSpec((4,), role="vector", init=("normal", 0.3, 0.3))
        return p

    def load(self, tensors):
        self.up = tensors[self.up_name].contiguous()
        self.down = tensors[self.down_name].contiguous()
        if self.polynorm:
            self.coef = tensors[self.coef_name].contiguous()

    def forward(self, h, ctx: StepContext) -> Product:
        rt, ws = ctx.rt, ctx.ws
        z = rt.linear(h, self.up, ws, "ff_up", out_dtype=torch.float32)
        act = ws.get("ff_act", (h.shape[0], self.inter), rt.dtype)
        if self.polynorm:
            K.polynorm_rows(z.tensor, self.coef, self.eps, act, nsplit=z.nsplit, split_stride=z.split_stride)
        else:
            K.act_rows(z.tensor, act, self.activation, nsplit=z.nsplit, split_stride=z.split_stride)
        return rt.linear(act, self.down, ws, "ff_out", out_dtype=torch.float32)       # it joins a float32 sum


@register_feed_forward("token_side")
class TokenSide(FeedForward):
    """A per-layer input from the token itself, added to the stream as a normalised branch:

        e = table[token, column0 : column0 + dim];  g = gelu_tanh(W_gate x) * e;  y = W_proj g;
        x <- x + rms(y) * w

    The table is a part of the model (ModelSpec.shared, key ``table``) of which every layer reads its
    own ``dim`` columns from ``column0``.  Tensors: gate [dim, hidden], proj [hidden, dim], norm [hidden].
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.dim = int(spec["dim"])
        self.column0 = int(spec["column0"])
        self.eps = float(spec["eps"])
        self.table_key = spec.get("table", "side")
        self.table = None
        self.gate = self.proj = self.norm = None

    def kernel_modules(self):
        return ("postnorm",)

    def parameters(self):
        return {"gate": ParamSpec((self.dim, self.hidden)), "proj": ParamSpec((self.hidden, self.dim)),
                "norm": ParamSpec((self.hidden,), role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        self.gate, self.proj, self.norm = tensors["gate"].contiguous(), tensors["proj"].contiguous(), tensors["norm"]

    def bind(self, shared):
        self.table = shared[self.table_key]
        if self.column0 + self.dim > self.table.width:
            raise ValueError(f"columns {self.column0}..{self.column0 + self.dim} are outside a table {self.table.width} wide")

    def forward_into(self, x, h, ctx: StepContext, keep_copy: bool = True):
        """Add the branch into the float32 stream ``x`` (``h``: its rows in the compute dtype); returns
        the new rows in the compute dtype (``keep_copy`` False: nobody reads them, None is returned)."""
        rt, ws = ctx.rt, ctx.ws
        z = rt.linear(h, self.gate, ws, "side_gate", out_dtype=torch.float32)
        g = ws.get("side_g", (h.shape[0], self.dim), rt.dtype)
        K.table_gate(z.tensor, self.table.weight, self.column0, ctx.tokens, g, nsplit=z.nsplit,
                     split_stride=z.split_stride, status=ctx.status)
        y = rt.linear(g, self.proj, ws, "side_out", out_dtype=torch.float32)
        copy = None if rt.dtype == torch.float32 or not keep_copy else ws.get("x_copy", tuple(x.shape), rt.dtype)
        K.norm_mix(x, self.norm, self.eps, delta=y.tensor, nsplit=y.nsplit, split_stride=y.split_stride,
                   alpha=0.0, keep=1.0, copy=copy)
        if not keep_copy:
            return None
        return x if copy is None else copy

    def forward(self, h, ctx):
        raise NotImplementedError("a token_side part adds into the stream: call forward_into")


@register_feed_forward("glu")
class GatedMLP(FeedForward):
    """down(act(gate(x)) * up(x)), no biases; ``activation``: "silu" or "gelu_tanh", computed in float32 on
    the stacked product's float32 output.  Tensor names: ``gate_name``, ``up_name``, ``down_name`` (default
    "gate", "up", "down").  The output is float32: it joins a float32 sum."""

    ACTS = {"silu": 0, "gelu_tanh": 1}

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.activation = spec.get("activation", "silu")
        if self.activation not in self.ACTS:
            raise ValueError(f"unknown activation {self.activation!r} of a gated feed-forward")
        self.names = (spec.get("gate_name", "gate"), spec.get("up_name", "up"), spec.get("down_name", "down"))
        self.gate_up = self.down = None
        self.gate_block = self.inter

    def kernel_modules(self):
        return ("mixparts",)

    def parameters(self):
        g, u, d = self.names
        return {g: ParamSpec((self.inter, self.hidden)), u: ParamSpec((self.inter, self.hidden)),
                d: ParamSpec((self.hidden, self.inter))}

    def load(self, tensors):
        g, u, d = self.names
        self.gate_up, self.gate_block = self.rt.glu_layout(tensors[g], tensors[u])
        self.down = tensors[d].contiguous()

    def forward(self, h, ctx: StepContext) -> Product:
        rt, ws = ctx.rt, ctx.ws
        act = rt.linear_glu(h, self.gate_up, self.gate_block, self.activation, ws, "ff_act")
        return rt.linear(act, self.down, ws, "ff_out", out_dtype=torch.float32)
