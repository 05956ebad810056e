"""Linear attention whose decay is computed from the input, per key channel and token, over a float32 state
that is carried from step to step: gated linear attention ("gla") and HGRN2 ("hgrn2")."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import CacheView, Mixer, Product, StepContext
from .lightning import SCAN_MAX_TOKENS, ChunkPlanner
from .multimap_attention import _pad_rows
from .registry import register_mixer
from .spec import ParamSpec, PartSpec, StateNeed

SMEM_LIMIT = 200 * 1024


class DecayedStateMixer(Mixer):
    """What the two mixers share: the recurrence

        S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t      per head, S [dim, vdim] float32, zero at admission

    and what follows it: every head's o_t divided by its own root mean square over vdim and multiplied by a plain
    weight ``norm`` [vdim] that the heads share, the heads side by side, an optional multiplier, then W_o.
    Decoded tokens and portions of up to 16 tokens are walked token by token; longer portions go in chunks whose
    states are built in parallel (csrc/gatedlinear.cu).  q, k, v and log a enter the recurrence as float32.
    Parameters: hidden_size, heads, dim, vdim, eps.
    """

    mode = ""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.dk, self.dv = int(spec["dim"]), int(spec["vdim"])
        self.eps = float(spec["eps"])
        self.qw, self.vw = self.heads * self.dk, self.heads * self.dv
        self.weight = self.o_weight = self.norm = None
        self.chunk = 0

    def kernel_modules(self):
        return ("gatedlinear",)

    def cache_need(self):
        return StateNeed(shape=(self.heads, self.dk, self.dv), dtype="float32")

    def plan_key(self):
        return ("decayed_state", self._chunk())

    def planner(self, page_size: int, sm_count: int):
        return ChunkPlanner(self._chunk())

    def _chunk(self) -> int:
        """Tokens per chunk of the chunked route: 64 where two CTAs' tiles fit an SM side by side, else 32 (shorter
        chunks cost fewer products inside them and more states), else 16."""
        if not self.chunk:
            lk, dvp = (self.dk + 3) // 4 * 4 + 4, (self.dv + 3) // 4 * 4    # rows padded to whole float4s
            need = lambda c: 4 * (c * lk + c * dvp + c * (c + 4) + max(2 * c * lk, 4 * dvp))
            self.chunk = 64 if 2 * need(64) <= SMEM_LIMIT else 32 if need(32) <= SMEM_LIMIT else 16
        return self.chunk

    def _prepare(self, h, ctx: StepContext, q, k, v, g) -> tuple[Product | None, int]:
        """Fill the recurrence's inputs; returns the product whose columns (from the returned column on) multiply
        the normalised output through silu, or None."""
        raise NotImplementedError

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        q = ws.get("gl_q", (T, self.qw), torch.float32)
        k = ws.get("gl_k", (T, self.qw), torch.float32)
        g = ws.get("gl_g", (T, self.qw), torch.float32)
        v = ws.get("gl_v", (T, self.vw), torch.float32)
        gate, gate0 = self._prepare(h, ctx, q, k, v, g)
        o = ws.get("gl_o", (T, self.vw), torch.float32)
        args = (q, k, g, v, cache.storage, o, ctx.tok_seg, ctx.seg_slot, ctx.positions)
        common = dict(heads=self.heads, dk=self.dk, dv=self.dv, writable=cache.writable)
        meta = cache.meta
        n_chunks = meta.get("num_chunks", 0)
        short = any(s.count <= SCAN_MAX_TOKENS for s in ctx.segments) if n_chunks else True
        if short:
            K.gated_linear_scan(*args, **common, max_tokens=SCAN_MAX_TOKENS if n_chunks else 0)
        if n_chunks:
            scratch = ws.get("gl_chunk_states", (n_chunks * self.heads * (self.dk * self.dv + self.dk),), torch.float32)
            K.gated_linear_chunked(*args, meta["chunks"], n_chunks, meta["seg_chunks"], meta["num_long"], scratch,
                                   self._chunk(), **common)
        out = ws.get("gl_normed", (T, self.vw), rt.dtype)
        K.gated_linear_head_norm(o, self.norm, self.eps, out, heads=self.heads, dv=self.dv, gate=gate, gate0=gate0)
        return rt.linear(out, self.o_weight, ws, "mix_out", out_dtype=torch.float32)      # it joins a float32 sum


@register_mixer("gla")
class GatedLinearAttention(DecayedStateMixer):
    """q = W_q h * dim^(-1/2), k = W_k h, v = W_v h; the decay of key channel c of a head at token t is
    a = sigmoid(z)^(1/tau) with z = W_a2 (W_a1 h) + b (a low-rank product); the normalised heads are multiplied
    by silu(W_g h).  Further parameters: tau, decay_rank (None: whatever the stored a1 and a2 have).  Tensors: q, k, v, g, a1, a2, a2.b, norm, o."""

    mode = "gla"

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.tau = float(spec["tau"])
        rank = spec.get("decay_rank")            # None: read off the stored matrices' shapes
        self.rank = -1 if rank is None else int(rank)
        if not self.tau > 0:
            raise ValueError("the decay's temperature tau must be positive")
        self.a2 = self.a2_bias = None

    def parameters(self):
        return {"q": ParamSpec((self.qw, self.hidden)), "k": ParamSpec((self.qw, self.hidden)),
                "v": ParamSpec((self.vw, self.hidden)), "g": ParamSpec((self.vw, self.hidden)),
                "a1": ParamSpec((self.rank, self.hidden)), "a2": ParamSpec((self.qw, self.rank), init=("normal", 0.0, 0.3)),
                "a2.b": ParamSpec((self.qw,), role="vector", init=("normal", 2.0, 1.0)),
                "o": ParamSpec((self.hidden, self.vw)),
                "norm": ParamSpec((self.dv,), role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        # one product for [q | k | v | g | a1]; the low-rank decay's second matrix takes a1's columns from it
        self.weight = _pad_rows(torch.cat((tensors["q"], tensors["k"], tensors["v"], tensors["g"], tensors["a1"]), 0))
        self.a2 = tensors["a2"].contiguous()
        if tensors["a1"].shape[0] != self.a2.shape[1]:
            raise ValueError(f"the decay's two matrices do not meet: {list(tensors['a1'].shape)} and {list(self.a2.shape)}")
        self.rank = self.a2.shape[1]
        self.a2_bias = tensors["a2.b"]
        self.o_weight = tensors["o"].contiguous()
        self.norm = tensors["norm"]

    def _prepare(self, h, ctx, q, k, v, g):
        proj = ctx.rt.linear(h, self.weight, ctx.ws, "gl_proj", out_dtype=torch.float32)
        K.gated_linear_prep("gla", proj, 0, self.qw, 2 * self.qw, 2 * self.qw + 2 * self.vw, self.a2_bias, q, k, v, g,
                            a2=self.a2, qscale=self.dk ** -0.5, tau=self.tau)
        return proj, 2 * self.qw + self.vw


@register_mixer("hgrn2")
class HGRN2(DecayedStateMixer):
    """Linear attention in which the forget gate also decides what is written: q = silu(W_q h), v = W_v h,
    f = low + (1 - low) sigmoid(W_f h + b) per head and channel with a stored lower bound ``lower``; the decay is f
    and the key is 1 - f; no other scale and no output gate.  Tensors: q, f, f.b, lower, v, norm, o."""

    mode = "hgrn2"

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.f_bias = self.lower = None

    def parameters(self):
        return {"q": ParamSpec((self.qw, self.hidden)), "f": ParamSpec((self.qw, self.hidden)),
                "f.b": ParamSpec((self.qw,), role="vector", init=("normal", 1.0, 1.0)),
                "lower": ParamSpec((self.qw,), role="vector", init=("normal", 0.5, 0.15)),
                "v": ParamSpec((self.vw, self.hidden)), "o": ParamSpec((self.hidden, self.vw)),
                "norm": ParamSpec((self.dv,), role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        self.weight = _pad_rows(torch.cat((tensors["q"], tensors["f"], tensors["v"]), 0))
        self.f_bias, self.lower = tensors["f.b"], tensors["lower"]
        self.o_weight = tensors["o"].contiguous()
        self.norm = tensors["norm"]

    def _prepare(self, h, ctx, q, k, v, g):
        proj = ctx.rt.linear(h, self.weight, ctx.ws, "gl_proj", out_dtype=torch.float32)
        K.gated_linear_prep("hgrn2", proj, 0, 0, 2 * self.qw, self.qw, self.f_bias, q, k, v, g, low=self.lower)
        return None, 0
