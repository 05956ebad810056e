"""Token embedding and output head."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Part, Product, StepContext
from .registry import EMBEDDINGS, HEADS
from .spec import ParamSpec, PartSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """x = table[tokens] (mini_hisparse/model.py:86,166), times ``scale`` if the spec gives one (the
    reference has none); output is the float32 residual.  ``weight_name``: the tensor's local name
    ("" if the prefix alone names it).  With ``copy`` the rows are also left in the compute dtype as
    ctx.extras["x_copy"], for a first block that reads the stream without normalising it.  With
    ``keep`` = (name, row width, first column) the rows are also left, in the compute dtype, in those
    columns of a matrix ctx.extras[name] [T, row width], for a later part that reads the embedding
    output again (the input of a pass over repeated layers)."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.vocab = int(spec["vocab_size"])
        self.width = int(spec["hidden_size"])
        self.scale = float(spec.get("scale", 1.0))
        self.copy = bool(spec.get("copy", False))
        self.keep = spec.get("keep")
        self.weight_name = spec.get("weight_name", "weight")
        self.weight = None

    def kernel_modules(self):
        return ("mixparts",) if self.keep else ()

    def parameters(self):
        return {self.weight_name: ParamSpec((self.vocab, self.width))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = self._forward(ctx)
        if self.keep:
            name, ld, col0 = self.keep
            kept = ctx.ws.get(name, (ctx.T, int(ld)), ctx.rt.dtype)
            K.stream_pack(x, kept, int(col0))
            ctx.extras[name] = kept
        return x

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.ws.get("residual", (ctx.T, self.width), torch.float32)
        copy = None
        if self.copy and ctx.rt.dtype != torch.float32:
            copy = ctx.ws.get("x_copy", (ctx.T, self.width), ctx.rt.dtype)
        K.embed(self.weight, ctx.tokens, x, status=ctx.status, scale=self.scale, copy=copy)
        if self.copy:
            ctx.extras["x_copy"] = x if copy is None else copy
        return x


@EMBEDDINGS.register("stream_input")
class StreamInput(Part):
    """A part of the model as a whole that replaces the residual stream by a product of itself and the
    embedding output:  x <- W [x ; x0]  with W [width, 2 width] (x's columns first).  It runs where the
    run order says (RunEntry.before), e.g. at the start of every pass over repeated layers.

    The embedding leaves x0 in the right half of ctx.extras[``buffer``] [T, 2 width] (TokenEmbedding's
    ``keep``); this part writes the stream, with everything still pending added, into the left half,
    leaves the stream at ZERO and returns the product as pending, so that the next norm's pass over the
    stream adds it (0 + W [x ; x0]) like any other product, split-K parts included."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.width = int(spec["width"])
        self.buffer = spec.get("buffer", "stream_cat")
        self.weight_name = spec.get("weight_name", "in")
        self.weight = None

    def kernel_modules(self):
        return ("mixparts",)

    def parameters(self):
        return {self.weight_name: ParamSpec((self.width, 2 * self.width))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()

    def forward_stream(self, x, pending: Product | None, ctx: StepContext):
        cat = ctx.extras.get(self.buffer)
        if cat is None:
            raise RuntimeError(f"the embedding did not keep its output in {self.buffer!r}")
        K.stream_pack(x, cat, 0, delta=pending, delta2=pending.also if pending is not None else None, zero=True)
        return x, ctx.rt.linear(cat, self.weight, ctx.ws, "stream_in", out_dtype=torch.float32)


@EMBEDDINGS.register("token_table")
class TokenTable(Part):
    """A table [vocab, width] that other parts index by token id (a model-level part: ModelSpec.shared)."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.vocab = int(spec["vocab_size"])
        self.width = int(spec["width"])
        self.weight_name = spec.get("weight_name", "weight")
        self.weight = None

    def parameters(self):
        return {self.weight_name: ParamSpec((self.vocab, self.width))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()


@HEADS.register("lm_head")
class LMHead(Part):
    """logits = h W^T in float32, no bias (mini_hisparse/model.py:96,181).  With ``tied`` the
    embedding table is the weight and the checkpoint holds no lm_head tensor.  With ``softcap`` c the logits
    are capped smoothly: logits <- c tanh(logits / c), in float32."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.vocab = int(spec["vocab_size"])
        self.width = int(spec["hidden_size"])
        self.tied = bool(spec["tied"])
        self.softcap = float(spec.get("softcap") or 0.0)
        self.weight_name = spec.get("weight_name", "weight")
        self.weight = None

    def parameters(self):
        if self.tied:
            return {self.weight_name: ParamSpec((self.vocab, self.width), optional=True)}
        return {self.weight_name: ParamSpec((self.vocab, self.width))}

    def load(self, tensors):
        if not self.tied:
            self.weight = tensors[self.weight_name].contiguous()

    def tie(self, embedding: TokenEmbedding):
        self.weight = embedding.weight

    def kernel_modules(self):
        return ("gateparts",) if self.softcap else ()

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = ctx.rt.linear(h, self.weight, ctx.ws, "logits", out_dtype=torch.float32, allow_split=False).matrix
        if self.softcap:
            K.softcap_rows(logits, self.softcap)
        return logits
