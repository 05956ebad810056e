"""Sliding-window attention whose far keys are not simply lost: the window's past is seen as block means
("pooled_window_attention"), or the first positions of the sequence stay visible and the heads' softmax weights
are mixed before they meet the values ("kept_first_attention")."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .attention import ITEM_INTS, ROW_TILE, AttentionPlanner, AttentionShape
from .base import CacheView, Mixer, Product, StepContext
from .multimap_attention import _pad_rows
from .registry import POSITIONS, register_mixer
from .spec import PagedKVNeed, ParamSpec, PartSpec


class WindowAttentionBase(Mixer):
    """What the two mixers share: q = W_q h [q_heads x dim], k = W_k h [kv_heads x dim], v = W_v h
    [kv_heads x vdim] without biases, RMS norms on q and k before the rotation of the first ``rotary_dim``
    elements of every head (half-split pairs), score = (q . k) * scale, a window of ``window`` positions
    (query i sees j with 0 <= i - j < window), one softmax over everything a query sees, W_o at the end.
    The cache keeps every position (what lies behind the window is still read, as itself or as a mean).
    Scores, softmax, norms and angles are float32; q and the cached rows have the compute dtype.
    Parameters: hidden_size, q_heads, kv_heads, dim, vdim, scale, window, eps, position (a PartSpec).
    """

    per_head_norm = False

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.nq, self.nkv = int(spec["q_heads"]), int(spec["kv_heads"])
        self.dk, self.dv = int(spec["dim"]), int(spec["vdim"])
        self.scale = float(spec["scale"])
        self.window = int(spec["window"])
        self.eps = float(spec["eps"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot be grouped over {self.nkv} KV heads")
        if self.window < 1:
            raise ValueError("the window must hold at least the query's own position")
        self.position = POSITIONS.build(spec["position"], rt=rt)
        if getattr(self.position, "interleaved", False):
            raise ValueError(f"{spec.kind} rotates half-split pairs only")
        self.qw, self.kw, self.vw, self.ow = self.nq * self.dk, self.nkv * self.dk, self.nkv * self.dv, self.nq * self.dv
        self.weight = self.o_weight = self.q_norm = self.k_norm = None

    def kernel_family(self) -> str:
        """"mma": mma.sync tiles of 64 rows for long portions and of 16 rows for decoded tokens and short portions
        (bfloat16, widths that are multiples of 8 up to 128); "simt": the CUDA cores (float32, and every other width)."""
        if self.rt is None or self.rt.dtype != torch.bfloat16 or not K.attention_mma_ext_supports(self.dk, self.dv):
            return "simt"
        if not self.scale > 0.0:        # the tensor-core kernels take the running maximum of the raw products
            return "simt"
        return "mma"

    def kernel_modules(self):
        if self.kernel_family() == "simt":
            return ("attention_simt", "postnorm", "maskparts")
        return ("attention_simt", "attention_mma_ext", "postnorm", "maskparts")

    def plan_key(self):
        return (self.spec.kind, self.nq, self.nkv, self.window)

    def planner(self, page_size: int, sm_count: int):
        rows = 64 if self.kernel_family() == "mma" else ROW_TILE
        return AttentionPlanner(AttentionShape(self.nq, self.nkv, self.window, rows), sm_count)

    def _norm_shapes(self):
        return ((self.dk,), (self.dk,)) if self.per_head_norm else ((self.qw,), (self.kw,))

    def _project(self, h, ctx: StepContext, cache: CacheView, *, v_eps=0.0, page_extra=0):
        """The stacked product, both norms, the rotation and the append; returns (the product, q)."""
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        if not cache.writable:
            raise ValueError(f"a {self.spec.kind} layer owns its cache")
        proj = rt.linear(h, self.weight, ws, "wa_proj", out_dtype=torch.float32)
        q = ws.get("wa_q", (T, self.qw), rt.dtype)
        rdim = int(getattr(self.position, "rotary_dim", 0) or 0)
        K.qknorm_rope_append(proj.tensor, self.q_norm, self.k_norm, self.eps, ctx.positions, ctx.tok_seg,
                             cache.meta["block_table"], self.position.inv_freq, rdim, q, cache.storage, nq=self.nq,
                             nkv=self.nkv, dk=self.dk, dv=self.dv, page_size=cache.page_size, nsplit=proj.nsplit,
                             split_stride=proj.split_stride, status=ctx.status, per_head=self.per_head_norm,
                             v_eps=v_eps, page_extra=page_extra)
        return proj, q

    def _attend_mma(self, q, out, ctx: StepContext, cache: CacheView, **options):
        """The plan's items on the tensor cores: 16-row tiles whose key splits the last CTA merges, 64-row tiles.
        With value_head="all" everything the kernel writes has a plane per KV head."""
        ws, meta, T = ctx.ws, cache.meta, q.shape[0]
        part_rows = max(1, meta["part_rows_cap"])
        planes = (self.nkv,) if options.get("value_head") == "all" else ()
        part_acc = ws.get("attn_part_acc", planes + (part_rows, self.nq, self.dv), torch.float32)
        part_ml = ws.get("attn_part_ml", planes + (part_rows, self.nq, 2), torch.float32)
        n_small, n_big = meta["n_small"], meta["n_big"]
        args = (q, cache.storage, out, part_acc, part_ml)
        tail = (ctx.positions, meta["block_table"], meta["tok_part_row"])
        common = dict(nq=self.nq, nkv=self.nkv, d=self.dk, dv=self.dv, page_size=cache.page_size, window=self.window,
                      scale=self.scale, **options)
        if n_small:
            chunks = -(-(self.nq // self.nkv) // ROW_TILE)
            counters = ws.get_zeroed("attn_counters", planes + (T * self.nkv * chunks,), torch.int32)
            K.attention_mma_ext(*args, meta["items"], n_small, 16, *tail, **common, tok_nsplit=meta["tok_nsplit"],
                                counters=counters)
        if n_big:
            K.attention_mma_ext(*args, meta["items"][n_small * ITEM_INTS:], n_big, 64, *tail, **common)

    def _attend(self, q, out, width, ctx: StepContext, cache: CacheView, **options):
        """The plan's items on the CUDA cores and the merge of split tokens; ``width`` is an output row's."""
        ws, meta = ctx.ws, cache.meta
        gate = {k: options[k] for k in ("gate", "gate_nsplit", "gate_split_stride") if k in options}
        part_rows = max(1, meta["part_rows_cap"])
        part_acc = ws.get("attn_part_acc", (part_rows, self.nq, width), torch.float32)
        part_ml = ws.get("attn_part_ml", (part_rows, self.nq, 2), torch.float32)
        n = meta["n_small"] + meta["n_big"]
        if n:
            K.attention_simt(q, cache.storage, out, part_acc, part_ml, meta["items"], n, n, ctx.positions,
                             meta["block_table"], meta["tok_part_row"], nq=self.nq, nkv=self.nkv, d=self.dk,
                             dv=self.dv, page_size=cache.page_size, window=self.window, scale=self.scale, **options)
        if meta["any_split"]:
            K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], out, nq=self.nq,
                                d=width, **gate)


@register_mixer("pooled_window_attention")
class PooledWindowAttention(WindowAttentionBase):
    """Beside the window's own positions a query at position i sees ONE key and value for every block of ``pool``
    positions that lies wholly before the window (block b = positions b pool .. b pool + pool - 1, seen when
    b pool + pool - 1 <= i - window): the mean of the block's keys and the mean of its values as the cache holds
    them.  Positions that have left the window while their block is not complete behind it are not seen at all.

    * q and k are each RMS-normalised as ONE vector spanning every head (plain weights as long as the projection).
    * Every head's value is divided by its root mean square over vdim (no weight) and cached so.
    * The heads' outputs are multiplied by sigmoid(W_g h) before W_o.

    The block means live in the tail of the pages (PagedKVNeed.pool): the token that completes a block writes them.
    Further parameter: pool.  Tensors: q, k, v, q.norm, k.norm, g, o.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.pool = int(spec["pool"])
        if self.pool < 1:
            raise ValueError("pooled blocks hold at least one position")

    def cache_need(self):
        return PagedKVNeed(kv_heads=self.nkv, head_dim=self.dk, window=None, v_dim=self.dv, pool=self.pool)

    def plan_key(self):
        return super().plan_key() + (self.pool,)

    def parameters(self):
        qn, kn = self._norm_shapes()
        return {"q": ParamSpec((self.qw, self.hidden)), "k": ParamSpec((self.kw, self.hidden)),
                "v": ParamSpec((self.vw, self.hidden)), "g": ParamSpec((self.ow, self.hidden)),
                "o": ParamSpec((self.hidden, self.ow)),
                "q.norm": ParamSpec(qn, role="vector", init=("normal", 1.0, 0.1)),
                "k.norm": ParamSpec(kn, role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        self.weight = _pad_rows(torch.cat((tensors["q"], tensors["k"], tensors["v"], tensors["g"]), 0))   # [q | k | v | g]
        self.o_weight = tensors["o"].contiguous()
        self.q_norm, self.k_norm = tensors["q.norm"], tensors["k.norm"]

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        extra = self.nkv * K.pool_slots(cache.page_size, self.pool) * (self.dk + self.dv)
        proj, q = self._project(h, ctx, cache, v_eps=self.eps, page_extra=extra)
        K.pool_means(cache.storage, ctx.positions, ctx.tok_seg, cache.meta["block_table"], nkv=self.nkv, d=self.dk,
                     dv=self.dv, page_size=cache.page_size, pool=self.pool, status=ctx.status)
        p = proj.tensor
        g0 = self.qw + self.kw + self.vw
        attn = ws.get("wa_attn", (T, self.ow), rt.dtype)
        gate = dict(gate=(p[0] if proj.nsplit > 1 else p)[:, g0:g0 + self.ow], gate_nsplit=proj.nsplit,
                    gate_split_stride=proj.split_stride)
        if self.kernel_family() == "mma":
            self._attend_mma(q, attn, ctx, cache, pool=self.pool, **gate)
        else:
            self._attend(q, attn, self.dv, ctx, cache, pool=self.pool, **gate)
        return rt.linear(attn, self.o_weight, ws, "mix_out", out_dtype=torch.float32)


@register_mixer("kept_first_attention")
class KeptFirstAttention(WindowAttentionBase):
    """Beside the window's positions a query sees the first ``keep_first`` positions of its sequence, at their true
    positions (for the rotation as for the distances).

    * q and k are RMS-normalised head by head, with one weight [dim] each that all heads share.
    * After the softmax the heads' weights are mixed, w'_h(i, j) = sum_g talk[h, g] w_g(i, j), and head h applies
      w'_h to the values of its own KV head.  Since the mix is linear it is taken on outputs: every head's weights
      are applied to the values of every KV head (an output row [kv_heads x vdim]), and
      o_h = sum_g talk[h, g] a_g[kv(h)].

    Further parameter: keep_first.  Tensors: q, k, v, q.norm, k.norm, talk, o.
    """

    per_head_norm = True

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.keep_first = int(spec["keep_first"])
        if self.keep_first < 0:
            raise ValueError("keep_first cannot be negative")
        if self.dv > 512:
            raise ValueError(f"values {self.dv} wide: the attention kernels take up to 512")
        self.talk = None

    def cache_need(self):
        return PagedKVNeed(kv_heads=self.nkv, head_dim=self.dk, window=None, v_dim=self.dv)

    def plan_key(self):
        return super().plan_key() + (self.keep_first,)

    def parameters(self):
        qn, kn = self._norm_shapes()
        return {"q": ParamSpec((self.qw, self.hidden)), "k": ParamSpec((self.kw, self.hidden)),
                "v": ParamSpec((self.vw, self.hidden)), "o": ParamSpec((self.hidden, self.ow)),
                "q.norm": ParamSpec(qn, role="vector", init=("normal", 1.0, 0.1)),
                "k.norm": ParamSpec(kn, role="vector", init=("normal", 1.0, 0.1)),
                "talk": ParamSpec((self.nq, self.nq), role="vector", init=("normal", 0.0, 0.5))}

    def load(self, tensors):
        self.weight = _pad_rows(torch.cat((tensors["q"], tensors["k"], tensors["v"]), 0))      # [q | k | v]
        self.o_weight = tensors["o"].contiguous()
        self.q_norm, self.k_norm = tensors["q.norm"], tensors["k.norm"]
        self.talk = tensors["talk"].float().contiguous()

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        _, q = self._project(h, ctx, cache)
        wide = self.nkv * self.dv
        attn = ws.get("wa_attn", (T, self.ow), rt.dtype)
        if self.kernel_family() == "mma":
            # every query head's weights over the values of each KV head in turn (gridDim.z), a plane of outputs each
            planes = ws.get("wa_every", (self.nkv, T, self.nq, self.dv), torch.float32)
            self._attend_mma(q, planes, ctx, cache, keep_first=self.keep_first, value_head="all")
            K.talk_mix(planes, self.talk, attn, nq=self.nq, nkv=self.nkv, dv=self.dv, planes=True)
        elif wide <= 512:
            every = ws.get("wa_every", (T, self.nq, wide), torch.float32)
            self._attend(q, every, wide, ctx, cache, keep_first=self.keep_first, all_values=True)
            K.talk_mix(every, self.talk, attn, nq=self.nq, nkv=self.nkv, dv=self.dv)
        else:       # rows too wide for one pass on the CUDA cores: a pass and a plane per KV head
            planes = ws.get("wa_every", (self.nkv, T, self.nq, self.dv), torch.float32)
            for c in range(self.nkv):
                self._attend(q, planes[c], self.dv, ctx, cache, keep_first=self.keep_first, value_head=c)
            K.talk_mix(planes, self.talk, attn, nq=self.nq, nkv=self.nkv, dv=self.dv, planes=True)
        return rt.linear(attn, self.o_weight, ws, "mix_out", out_dtype=torch.float32)
