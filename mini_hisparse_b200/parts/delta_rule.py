"""The gated delta rule: a linear recurrence over a float32 state whose write corrects what the state already
returns for the key."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import CacheView, Mixer, Product, StepContext
from .multimap_attention import _pad_rows
from .registry import register_mixer
from .spec import ParamSpec, PartSpec, StateNeed


@register_mixer("gated_delta")
class GatedDeltaRule(Mixer):
    """q = W_q h, k = W_k h [kv_heads x dim], v = W_v h [heads x vdim], no biases; head h reads q/k head
    h / (heads / kv_heads).

    * q, k and v each pass a short causal convolution over time, one filter of ``conv`` taps per channel (the last tap
      is the current token's, zeros before the start of the sequence, no bias), and silu.
    * q and k become unit vectors per head, x / sqrt(sum x^2 + 1e-6); q is also multiplied by dim^(-1/2).
    * beta = sigmoid(W_b h) and g = exp(-exp(A_log) softplus(W_a h + dt_bias)), one of each per head and token.
    * Per head, over a state S [dim, vdim] that starts at zero:
          S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q      (o sees the token's own write)
    * Every head's o is divided by its root mean square over vdim, times a plain weight ``norm`` [vdim] shared by
      the heads, times silu(W_g h); then W_o.

    Per request the part keeps the state and the last conv - 1 inputs of the convolutions, both float32, in ONE
    slot: [heads x dim x vdim | (conv - 1) x channels].  Everything between the input projection and the output
    projection is float32.  Parameters: hidden_size, heads, kv_heads, dim, vdim, conv, eps.
    Tensors: q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, g, norm, o.
    """

    UNIT_EPS = 1e-6

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.heads, self.kv_heads = int(spec["heads"]), int(spec["kv_heads"])
        self.dk, self.dv = int(spec["dim"]), int(spec["vdim"])
        self.taps = int(spec["conv"])
        self.eps = float(spec["eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads cannot share {self.kv_heads} q/k heads")
        if not 1 <= self.taps <= 16:
            raise ValueError("the short convolution has 1 to 16 taps")
        if self.dk > 256:
            raise ValueError("the recurrence kernel takes keys up to 256 wide")
        self.qk, self.vw = self.kv_heads * self.dk, self.heads * self.dv
        self.channels = 2 * self.qk + self.vw
        self.state_elems = self.heads * self.dk * self.dv
        self.weight = self.o_weight = self.norm = self.filters = self.A_log = self.dt_bias = None

    def kernel_modules(self):
        return ("deltarule", "gatedlinear")

    def cache_need(self):
        return StateNeed(shape=(self.state_elems + (self.taps - 1) * self.channels,), dtype="float32")

    def parameters(self):
        vec = dict(role="vector")
        return {"q": ParamSpec((self.qk, self.hidden)), "k": ParamSpec((self.qk, self.hidden)),
                "v": ParamSpec((self.vw, self.hidden)), "g": ParamSpec((self.vw, self.hidden)),
                "b": ParamSpec((self.heads, self.hidden), init=("normal", 0.0, 0.1)),
                "a": ParamSpec((self.heads, self.hidden), init=("normal", 0.0, 0.1)),
                "q.conv": ParamSpec((self.qk, self.taps), init=("normal", 0.0, 0.5), **vec),
                "k.conv": ParamSpec((self.qk, self.taps), init=("normal", 0.0, 0.5), **vec),
                "v.conv": ParamSpec((self.vw, self.taps), init=("normal", 0.0, 0.5), **vec),
                "A_log": ParamSpec((self.heads,), init=("normal", -1.0, 0.5), **vec),
                "dt_bias": ParamSpec((self.heads,), init=("normal", 0.0, 0.5), **vec),
                "norm": ParamSpec((self.dv,), init=("normal", 1.0, 0.1), **vec),
                "o": ParamSpec((self.hidden, self.vw))}

    def load(self, tensors):
        # one product for [q | k | v | b | a | g]
        self.weight = _pad_rows(torch.cat([tensors[n] for n in ("q", "k", "v", "b", "a", "g")], 0))
        self.filters = torch.cat([tensors[n + ".conv"].float() for n in ("q", "k", "v")], 0).contiguous()
        self.A_log, self.dt_bias = tensors["A_log"].float(), tensors["dt_bias"].float()
        self.norm = tensors["norm"]
        self.o_weight = tensors["o"].contiguous()

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        proj = rt.linear(h, self.weight, ws, "dr_proj", out_dtype=torch.float32)
        b0 = self.channels
        a0, g0 = b0 + self.heads, b0 + 2 * self.heads
        q = ws.get("dr_q", (T, self.qk), torch.float32)
        k = ws.get("dr_k", (T, self.qk), torch.float32)
        v = ws.get("dr_v", (T, self.vw), torch.float32)
        beta = ws.get("dr_beta", (T, self.heads), torch.float32)
        decay = ws.get("dr_decay", (T, self.heads), torch.float32)
        slots = cache.storage                                   # [slots, state | kept inputs]
        kept = slots[:, self.state_elems:]
        K.delta_prep(proj, 0, b0, a0, self.filters, self.A_log, self.dt_bias, kept, ctx.tok_seg, ctx.seg_slot,
                     ctx.positions, q, k, v, beta, decay, heads=self.heads, kv_heads=self.kv_heads, dk=self.dk,
                     dv=self.dv, qscale=self.dk ** -0.5, unit_eps=self.UNIT_EPS)
        if cache.writable and self.taps > 1:
            K.delta_conv_keep(proj, 0, kept, ctx.tok_seg, ctx.seg_slot, ctx.positions, channels=self.channels,
                              taps=self.taps)
        o = ws.get("dr_o", (T, self.vw), torch.float32)
        K.delta_scan(q, k, v, beta, decay, slots, o, ctx.tok_seg, ctx.seg_slot, ctx.positions, heads=self.heads,
                     kv_heads=self.kv_heads, dk=self.dk, dv=self.dv, writable=cache.writable)
        out = ws.get("dr_normed", (T, self.vw), rt.dtype)
        K.gated_linear_head_norm(o, self.norm, self.eps, out, heads=self.heads, dv=self.dv, gate=proj, gate0=g0)
        return rt.linear(out, self.o_weight, ws, "mix_out", out_dtype=torch.float32)
