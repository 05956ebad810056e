"""A routed feed-forward: a router chooses a few small gated feed-forwards (experts) per token."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import FeedForward, Product, StepContext
from .multimap_attention import _pad_rows
from .registry import register_feed_forward
from .spec import ParamSpec, PartSpec


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """Router logits z = W_r h in float32 over ``experts + identity`` outputs; s = softmax(z).

    * Choice: the ``top`` largest of s + correction (a stored vector), looked for only inside the best ``group_keep``
      of ``group_count`` equal groups of neighbouring outputs (a group's score is its largest choice score; outputs
      of the other groups cannot be chosen).  The weights are the chosen outputs' s, without the correction, divided
      by their sum (+ 1e-20).
    * The first ``experts`` outputs are experts W_down (silu(W_gate h) * (W_up h)) of width ``expert_ff``; the last
      ``identity`` outputs are identity experts that return h itself and store nothing.
    * ``shared_ff`` (None: none): an expert of that width that every token uses, added times sigmoid(w_sg . h).

    * ``correction`` False: no correction tensor (the choice is by s alone, which is the choice of the largest z, and
      the weights are the softmax over the chosen z); ``router_bias`` True: z = W_r h + b with a stored bias
      ``router.b``.

    Tensors: router, router.b, correction, e<i>.{gate, up, down}, shared.{gate, up, down, sg}.  The experts' weights are
    stacked at load ([experts, 2 ff, hidden] with gate above up, and [experts, hidden, ff]); the shared gate's row
    rides below the router's in one product.  Nothing between the router and the weighted sum goes through the host.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.experts, self.identity = int(spec["experts"]), int(spec.get("identity", 0))
        self.top = int(spec["top"])
        self.groups, self.keep = int(spec.get("group_count") or 1), int(spec.get("group_keep") or 1)
        self.ff = int(spec["expert_ff"])
        self.shared_ff = spec.get("shared_ff")
        self.outputs = self.experts + self.identity
        self.has_correction = bool(spec.get("correction", True))
        self.has_bias = bool(spec.get("router_bias", False))
        self.router_bias = None
        if self.outputs % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.outputs} router outputs in {self.groups} groups of which {self.keep} are kept")
        if not 1 <= self.top <= self.outputs // self.groups * self.keep:
            raise ValueError(f"{self.top} experts a token out of {self.outputs // self.groups * self.keep} that can be chosen")
        self.router = self.correction = self.gate_up = self.down = None
        self.shared_gate_up = self.shared_down = None
        self.shared_block = 0

    def kernel_modules(self):
        return ("moe", "mixparts")

    def parameters(self):
        p = {"router": ParamSpec((self.outputs, self.hidden), init=("normal", 0.0, 0.3))}
        if self.has_correction:
            p["correction"] = ParamSpec((self.outputs,), role="vector", init=("normal", 0.0, 0.02))
        if self.has_bias:
            p["router.b"] = ParamSpec((self.outputs,), role="vector", init=("normal", 0.0, 0.5))
        for e in range(self.experts):
            p[f"e{e}.gate"] = ParamSpec((self.ff, self.hidden))
            p[f"e{e}.up"] = ParamSpec((self.ff, self.hidden))
            p[f"e{e}.down"] = ParamSpec((self.hidden, self.ff))
        if self.shared_ff is not None:
            f = int(self.shared_ff)
            p.update({"shared.gate": ParamSpec((f, self.hidden)), "shared.up": ParamSpec((f, self.hidden)),
                      "shared.down": ParamSpec((self.hidden, f)), "shared.sg": ParamSpec((1, self.hidden))})
        return p

    def load(self, tensors):
        rows = [tensors["router"]] + ([tensors["shared.sg"]] if self.shared_ff is not None else [])
        self.router = _pad_rows(torch.cat(rows, 0))             # [router outputs | shared gate | zeros]
        self.correction = tensors.get("correction")
        self.router_bias = tensors.get("router.b")
        E = self.experts
        self.gate_up = torch.stack([torch.cat((tensors[f"e{e}.gate"], tensors[f"e{e}.up"]), 0) for e in range(E)]).contiguous()
        self.down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        if self.shared_ff is not None:
            self.shared_gate_up, self.shared_block = self.rt.glu_layout(tensors["shared.gate"], tensors["shared.up"])
            self.shared_down = tensors["shared.down"].contiguous()

    def forward(self, h, ctx: StepContext) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        E, top, pairs = self.experts, self.top, h.shape[0] * self.top
        logits = rt.linear(h, self.router, ws, "moe_logits", out_dtype=torch.float32)
        chosen = ws.get("moe_chosen", (T, top), torch.int32)
        weights = ws.get("moe_weights", (T, top), torch.float32)
        K.moe_route(logits, self.correction, chosen, weights, outputs=self.outputs, top=top, groups=self.groups,
                    keep=self.keep, bias=self.router_bias)
        plan = ws.get("moe_plan", (K.moe_plan_words(pairs, E),), torch.int32)
        K.moe_plan(chosen, plan, experts=E)
        act = ws.get("moe_act", (pairs, self.ff), rt.dtype)
        K.moe_linear(h, plan, self.gate_up, act, pairs=pairs, experts=E, gather=True, glu=True)
        y = ws.get("moe_y", (pairs, self.hidden), torch.float32)
        K.moe_linear(act, plan, self.down, y, pairs=pairs, experts=E, gather=False, glu=False)
        shared = gate = None
        if self.shared_ff is not None:
            a = rt.linear_glu(h, self.shared_gate_up, self.shared_block, "silu", ws, "moe_shared_act")
            shared = rt.linear(a, self.shared_down, ws, "moe_shared", out_dtype=torch.float32)
            gate = _Columns(logits.tensor[..., self.outputs:self.outputs + 1], logits.nsplit, logits.split_stride)
        out = ws.get("ff_out", (T, self.hidden), torch.float32)
        K.moe_combine(y, plan, chosen, weights, h, out, experts=E, shared=shared, shared_gate=gate)
        return Product(out)


class _Columns:
    """A run of columns of a split product, with the parts' stride of the whole product."""

    def __init__(self, tensor, nsplit, split_stride):
        self.tensor, self.nsplit, self.split_stride = tensor, nsplit, split_stride
