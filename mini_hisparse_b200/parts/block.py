"""Block arrangements: how a layer's norms, mixer and feed-forward are wired to the residual."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Block, CacheView, Product, StepContext
from .registry import FEED_FORWARDS, GATES, MIXERS, NORMS, register_block
from .spec import LayerSpec


@register_block("pre_norm")
class PreNormBlock(Block):
    """x = x + mixer(norm1(x)); x = x + ff(norm2(x))   (mini_hisparse/model.py:137,155-158).

    The residual adds are folded into the norms that follow them: the block receives the
    previous block's still-unadded output as ``pending`` and returns its own.
    """

    def __init__(self, spec: LayerSpec, rt):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.part("mixer_norm"), rt=rt)
        self.mixer = MIXERS.build(spec.part("mixer"), rt=rt)
        self.ff_norm = NORMS.build(spec.part("ff_norm"), rt=rt)
        self.feed_forward = FEED_FORWARDS.build(spec.part("feed_forward"), rt=rt)

    def parts(self):
        return {
            "mixer_norm": self.mixer_norm,
            "mixer": self.mixer,
            "ff_norm": self.ff_norm,
            "feed_forward": self.feed_forward,
        }

    def forward(self, x, pending: Product | None, ctx: StepContext, cache: CacheView | None) -> Product:
        h = self.mixer_norm.forward(x, ctx, delta=pending)
        a = self.mixer.forward(h, ctx, cache)
        h = self.ff_norm.forward(x, ctx, delta=a)
        return self.feed_forward.forward(h, ctx)


@register_block("post_norm")
class PostNormBlock(Block):
    """Post-norm with a scaled stream (the norm comes behind the residual addition):

        x <- norm1(alpha x + mixer(x));   x <- norm2(alpha x + ff(x))  (if the layer has a feed-forward);
        x <- x + side(x)                  (if the layer has a "side" part: a normalised branch of its own)

    Mixer and feed-forward take the un-normalised stream as input, so every kernel that writes the stream also leaves its rows
    in the compute dtype (ctx.extras["x_copy"]; the float32 path reads the stream directly).  Roles:
    "mixer", "mixer_norm", and optionally "feed_forward" with "ff_norm", and "side".  Options: alpha, and
    ``keep`` (default 0): the stream's own share beside the norm, x <- keep x + norm(alpha x + sublayer(x)); alpha = 0
    with keep = 1 is a block whose norms sit on the sublayers' outputs alone, x <- x + norm(sublayer(x)).
    Nothing is left pending: the block returns None.
    """

    keeps_copy = True

    def __init__(self, spec: LayerSpec, rt):
        self.spec = spec
        self.alpha = float(spec.option("alpha", 1.0))
        self.keep = float(spec.option("keep", 0.0))
        self.mixer = MIXERS.build(spec.part("mixer"), rt=rt)
        self.mixer_norm = NORMS.build(spec.part("mixer_norm"), rt=rt)
        self.feed_forward = self.ff_norm = self.side = None
        if spec.has("feed_forward"):
            self.feed_forward = FEED_FORWARDS.build(spec.part("feed_forward"), rt=rt)
            self.ff_norm = NORMS.build(spec.part("ff_norm"), rt=rt)
        if spec.has("side"):
            self.side = FEED_FORWARDS.build(spec.part("side"), rt=rt)

    def parts(self):
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.feed_forward is not None:
            out.update(ff_norm=self.ff_norm, feed_forward=self.feed_forward)
        if self.side is not None:
            out["side"] = self.side
        return out

    def bind(self, shared):
        for part in self.parts().values():
            if hasattr(part, "bind"):
                part.bind(shared)

    def forward(self, x, pending: Product | None, ctx: StepContext, cache: CacheView | None):
        if pending is not None:          # the block before this one was of another arrangement
            pending.add_into(x)
            ctx.extras.pop("x_copy", None)
        h = ctx.extras.get("x_copy")
        if h is None:
            h = x
            if ctx.rt.dtype != x.dtype:
                h = ctx.ws.get("x_copy", tuple(x.shape), ctx.rt.dtype)
                K.act_rows(x, h, "copy")
        a = self.mixer.forward(h, ctx, cache)
        h = self.mixer_norm.forward_post(x, ctx, a, alpha=self.alpha, keep=self.keep)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, ctx)
            h = self.ff_norm.forward_post(x, ctx, f, alpha=self.alpha, keep=self.keep)
        if self.side is not None:
            h = self.side.forward_into(x, h, ctx)
        ctx.extras["x_copy"] = h
        return None


@register_block("parallel")
class ParallelBlock(Block):
    """One norm, both sublayers read its output:  h = norm(x);  x <- x + mixer(h) + ff(h).

    Roles: "norm", "mixer", and optionally "feed_forward" (a layer without one adds the mixer alone).
    Both outputs are left pending together (Product.also); the next norm adds them into the stream in
    the same pass in which it normalises.
    """

    def __init__(self, spec: LayerSpec, rt):
        self.spec = spec
        self.norm = NORMS.build(spec.part("norm"), rt=rt)
        self.mixer = MIXERS.build(spec.part("mixer"), rt=rt)
        self.feed_forward = FEED_FORWARDS.build(spec.part("feed_forward"), rt=rt) if spec.has("feed_forward") else None

    def parts(self):
        out = {"norm": self.norm, "mixer": self.mixer}
        if self.feed_forward is not None:
            out["feed_forward"] = self.feed_forward
        return out

    #: up to this many tokens the two sublayers run side by side on two streams (see forward)
    BRANCH_MAX_TOKENS = 64

    def forward(self, x, pending: Product | None, ctx: StepContext, cache: CacheView | None) -> Product:
        h = self.norm.forward(x, ctx, delta=pending)
        if self.feed_forward is None:
            return self.mixer.forward(h, ctx, cache)
        branch = ctx.extras.get("branch_stream") if h.shape[0] <= self.BRANCH_MAX_TOKENS else None
        if branch is None:
            a = self.mixer.forward(h, ctx, cache)
            f = self.feed_forward.forward(h, ctx)
            return Product(a.tensor, a.nsplit, also=f)
        # A step of few tokens (decoding): the feed-forward streams most of the layer's weights while the
        # mixer is a chain of small kernels that wait for one another; the two read the same h and write
        # buffers of their own, so the feed-forward runs on a second stream beside the mixer (in a captured
        # graph: two branches of the graph) and the next norm waits for both.  Only for few tokens: their
        # products are the ones that need no scratch shared between launches.
        main = torch.cuda.current_stream()
        fork, join = ctx.extras["branch_events"]
        fork.record(main)
        branch.wait_event(fork)
        with torch.cuda.stream(branch), K.stream_scope():
            f = self.feed_forward.forward(h, ctx)
            join.record(branch)
        a = self.mixer.forward(h, ctx, cache)
        main.wait_event(join)
        return Product(a.tensor, a.nsplit, also=f)


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm before AND behind each sublayer, the behind one on the sublayer's result alone:

        h = norm1(x);  x <- x + norm1b(mixer(h) * sigmoid(gate1(h)))
        h = norm2(x);  x <- x + norm2b(ff(h) * sigmoid(gate2(h)))      (if the layer has a feed-forward)
        x <- x + side(x)                                              (if the layer has a "side" part)

    Roles: "mixer_norm", "mixer", "mixer_post_norm"; optionally "mixer_gate"; optionally "ff_norm",
    "feed_forward", "ff_post_norm" and "ff_gate"; optionally "side".  A gate is a part of the gates' registry that
    gives logits (and a bias) as wide as the stream; without one the sublayer's result is normalised as it is.
    One kernel multiplies by the gate, normalises, adds into the stream and already applies the norm that the
    next sublayer opens with; the side branch reads the stream's rows in the compute dtype from the same kernel.
    """

    keeps_copy = False

    def __init__(self, spec: LayerSpec, rt):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.part("mixer_norm"), rt=rt)
        self.mixer = MIXERS.build(spec.part("mixer"), rt=rt)
        self.mixer_post_norm = NORMS.build(spec.part("mixer_post_norm"), rt=rt)
        self.mixer_gate = GATES.build(spec.part("mixer_gate"), rt=rt) if spec.has("mixer_gate") else None
        self.feed_forward = self.ff_norm = self.ff_post_norm = self.ff_gate = self.side = None
        if spec.has("feed_forward"):
            self.ff_norm = NORMS.build(spec.part("ff_norm"), rt=rt)
            self.feed_forward = FEED_FORWARDS.build(spec.part("feed_forward"), rt=rt)
            self.ff_post_norm = NORMS.build(spec.part("ff_post_norm"), rt=rt)
            self.ff_gate = GATES.build(spec.part("ff_gate"), rt=rt) if spec.has("ff_gate") else None
        if spec.has("side"):
            self.side = FEED_FORWARDS.build(spec.part("side"), rt=rt)

    def parts(self):
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.mixer_gate is not None:
            out["mixer_gate"] = self.mixer_gate
        if self.feed_forward is not None:
            out.update(ff_norm=self.ff_norm, feed_forward=self.feed_forward, ff_post_norm=self.ff_post_norm)
            if self.ff_gate is not None:
                out["ff_gate"] = self.ff_gate
        if self.side is not None:
            out["side"] = self.side
        return out

    def kernel_modules(self):
        return ("gateparts",)

    def bind(self, shared):
        for part in self.parts().values():
            if hasattr(part, "bind"):
                part.bind(shared)

    def _join(self, x, result: Product, gate, h, post, ctx, *, copy=None, then=None, name="gate"):
        """x <- x + post(result * sigmoid(gate(h))); ``then``: the norm whose output of the new x is wanted too."""
        if result.also is not None:
            raise ValueError("a sandwich block normalises one product per sublayer")
        z = gate.logits(h, ctx, name) if gate is not None else None
        nxt = ctx.ws.get("h2", tuple(x.shape), ctx.rt.dtype) if then is not None else None
        K.gated_norm_add(x, result, post.weight, post.eps, gate=z, bias=gate.bias if gate is not None else None,
                         copy=copy, next_weight=then.weight if then is not None else None,
                         next_eps=then.eps if then is not None else None, next_out=nxt)
        return nxt

    def forward(self, x, pending: Product | None, ctx: StepContext, cache: CacheView | None):
        rt, ws = ctx.rt, ctx.ws
        h = self.mixer_norm.forward(x, ctx, delta=pending)
        a = self.mixer.forward(h, ctx, cache)
        want_copy = self.side is not None and rt.dtype != torch.float32
        last = self.feed_forward is None
        copy = ws.get("x_copy", tuple(x.shape), rt.dtype) if want_copy and last else None
        h2 = self._join(x, a, self.mixer_gate, h, self.mixer_post_norm, ctx, copy=copy,
                        then=None if last else self.ff_norm, name="gate1")
        if not last:
            f = self.feed_forward.forward(h2, ctx)
            copy = ws.get("x_copy", tuple(x.shape), rt.dtype) if want_copy else None
            self._join(x, f, self.ff_gate, h2, self.ff_post_norm, ctx, copy=copy, name="gate2")
        if self.side is not None:
            self.side.forward_into(x, x if copy is None else copy, ctx, keep_copy=False)
        return None
