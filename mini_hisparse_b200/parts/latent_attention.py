"""Attention over a latent cache: per position one low-rank row from which every head's keys and values
are expanded, plus one rotated key part shared by all heads."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .attention import ITEM_INTS, ROW_TILE, AttentionPlanner, AttentionShape
from .base import CacheView, Mixer, Product, StepContext
from .multimap_attention import _pad_rows
from .registry import POSITIONS, register_mixer
from .spec import PagedRowsNeed, ParamSpec, PartSpec


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """q = W_q h, per head [dim unrotated | rot_dim rotated];  [c | kr] = W_dkv h with c ``kv_rank`` wide.

    * c <- c / sqrt(mean(c^2) + eps) * w_c; kr (rot_dim wide, not normalised) is rotated by the position part
      and is the rotated key part of EVERY head; the rotated part of each q head is rotated the same way.
    * Head i: k_i = [W_uk,i c | kr], v_i = W_uv,i c; s = (q_i . k_i) * scale; causal softmax over the last
      ``window`` keys (None: all of them); the head's output times sigmoid(W_g h)_i (``gate``, default True);
      then W_o.  With ``sink`` the softmax's denominator has one more term, exp(sink_i): a stored logit per head
      that stands for no position, brings no value and is not scaled.
    * ``own_kv`` False: the layer has no W_dkv and no norm weight; it reads the cache rows of another run entry
      (RunEntry.cache_of), rotated as that entry wrote them, with its own queries, expansions, sink and gate.
    * Only [c | kr] is cached (PagedRowsNeed(kv_rank + rot_dim)).  The expansions are never formed per key:
      q_i . (W_uk,i c) = (W_uk,i^T q_i) . c, so the query is carried into the latent space (one small matrix
      per head), attention runs with the cached row as key AND, in its first kv_rank elements, as value, and
      the output sum_j p_j c_j is expanded once per query by W_uv,i.

    Parameters: hidden_size, heads, dim, rot_dim, vdim, kv_rank, scale, window, eps, position (a PartSpec
    over rot_dim elements), gate, sink, own_kv.  Tensors: q, dkv, dkv.norm, uk, uv, g, sink, o.  Scores, softmax, the latent's norm,
    angles and the gate are float32.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.d, self.dr, self.dv = int(spec["dim"]), int(spec["rot_dim"]), int(spec["vdim"])
        self.rank = int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.eps = float(spec["eps"])
        self.has_gate = bool(spec.get("gate", True))
        self.has_sink = bool(spec.get("sink", False))
        self.own_kv = bool(spec.get("own_kv", True))
        self.position = POSITIONS.build(spec["position"], rt=rt)
        if int(getattr(self.position, "rotary_dim", 0) or 0) != self.dr:
            raise ValueError(f"the position part must rotate all {self.dr} elements of the rotated key part")
        self.width = self.rank + self.dr                    # a cache row, and a query in the latent space
        if self.rank > 512:
            raise ValueError(f"a latent {self.rank} wide: the attention kernels take values up to 512 wide")
        self.qw, self.ow = self.heads * (self.d + self.dr), self.heads * self.dv
        self.weight = self.o_weight = self.c_norm = self.uk_t = self.uv = self.sink = None

    def kernel_family(self, page_size: int | None = None) -> str:
        """"tc": tcgen05 128-row tiles for long portions (bfloat16, a cache row 64 or 128 wide, pages that divide
        64) and TMA-fed 16-row tiles for the rest; "mma": mma.sync tiles of 64 and 16 rows (bfloat16, a cache
        row of at most 128 elements, a multiple of 8 like the latent); "simt": the CUDA cores (float32, and every
        other width)."""
        if (self.rt is None or self.rt.dtype != torch.bfloat16 or not self.scale > 0.0
                or not K.attention_mma_ext_supports(self.width, self.rank)):
            return "simt"
        if page_size is not None and self.width in (64, 128) and K.attention_tma_supports(self.width, page_size):
            return "tc"
        return "mma"

    def value_width(self, page_size: int | None) -> int:
        """How much of a cache row the attention kernels take as the value: the latent; in the "tc" family the
        whole row (its tiles have keys and values of one width; the columns behind the latent are not read
        afterwards)."""
        return self.width if self.kernel_family(page_size) == "tc" else self.rank

    def kernel_modules(self):
        if self.kernel_family() == "simt":
            return ("attention_simt", "mixparts")
        if self.width in (64, 128):
            return ("attention_simt", "attention_mma_ext", "attention_tma", "attention_tc", "mixparts")
        return ("attention_simt", "attention_mma_ext", "mixparts")

    def cache_need(self):
        return PagedRowsNeed(width=self.width, window=self.window)

    def plan_key(self):
        return ("latent_attention", self.heads, self.window, self.width, self.rt is not None and self.rt.dtype)

    def planner(self, page_size: int, sm_count: int):
        rows = {"tc": 128, "mma": 64, "simt": ROW_TILE}[self.kernel_family(page_size)]
        return AttentionPlanner(AttentionShape(self.heads, 1, self.window, rows), sm_count)

    def parameters(self):
        p = {"q": ParamSpec((self.qw, self.hidden)),
             "uk": ParamSpec((self.heads * self.d, self.rank)), "uv": ParamSpec((self.heads * self.dv, self.rank)),
             "o": ParamSpec((self.hidden, self.ow))}
        if self.own_kv:
            p.update({"dkv": ParamSpec((self.width, self.hidden)),
                      "dkv.norm": ParamSpec((self.rank,), role="vector", init=("normal", 1.0, 0.1))})
        if self.has_gate:
            p["g"] = ParamSpec((self.heads, self.hidden))
        if self.has_sink:
            p["sink"] = ParamSpec((self.heads,), role="vector", init=("normal", 0.0, 1.0))
        return p

    def load(self, tensors):
        rows = [tensors["q"]] + ([tensors["dkv"]] if self.own_kv else []) + ([tensors["g"]] if self.has_gate else [])
        self.weight = _pad_rows(torch.cat(rows, 0))                                               # [q | c | kr | g]
        self.o_weight = tensors["o"].contiguous()
        self.c_norm = tensors.get("dkv.norm")
        self.sink = tensors.get("sink")
        # per head: the key expansion transposed [rank, dim] (it carries q into the latent space) and the
        # value expansion as stored [vdim, rank]
        self.uk_t = tensors["uk"].view(self.heads, self.d, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].view(self.heads, self.dv, self.rank).contiguous()

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        meta = cache.meta
        if cache.writable != self.own_kv:
            raise ValueError("a latent_attention layer with a W_dkv of its own owns its cache, one without reads another's")
        proj = rt.linear(h, self.weight, ws, "la_proj", out_dtype=torch.float32)
        p = proj.tensor
        q_plain = ws.get("la_q_plain", (T, self.heads, self.d), rt.dtype)
        q_full = ws.get("la_q", (T, self.heads, self.width), rt.dtype)
        K.latent_prep(p, self.c_norm, self.eps, ctx.positions, ctx.tok_seg, meta["block_table"],
                      self.position.inv_freq, bool(getattr(self.position, "interleaved", False)), q_plain, q_full,
                      cache.storage, heads=self.heads, d=self.d, dr=self.dr, rank=self.rank,
                      page_size=cache.page_size, write_kv=cache.writable, nsplit=proj.nsplit,
                      split_stride=proj.split_stride, status=ctx.status)
        K.head_linear(q_plain, self.uk_t, q_full[:, :, :self.rank])
        g0 = self.qw + (self.width if self.own_kv else 0)
        gate = {}
        if self.has_gate:
            gate = dict(gate=(p[0] if proj.nsplit > 1 else p)[:, g0:g0 + self.heads], gate_nsplit=proj.nsplit,
                        gate_split_stride=proj.split_stride, gate_per_head=True)
        opts = dict(gate)                 # what the attention kernels get; the merge of key splits gets the gate only
        if self.has_sink:
            opts["sink"] = self.sink
        family = self.kernel_family(cache.page_size)
        vw = self.value_width(cache.page_size)
        lat = ws.get("la_out", (T, self.heads, vw), rt.dtype)                     # sum_j p_j c_j, gated
        part_rows = max(1, meta["part_rows_cap"])
        part_acc = ws.get("attn_part_acc", (part_rows, self.heads, vw), torch.float32)
        part_ml = ws.get("attn_part_ml", (part_rows, self.heads, 2), torch.float32)
        n_small, n_big = meta["n_small"], meta["n_big"]
        common = dict(nq=self.heads, nkv=1, d=self.width, dv=vw, page_size=cache.page_size,
                      window=self.window or 0, scale=self.scale, shared_kv=True, **opts)
        args = (q_full, cache.storage, lat, part_acc, part_ml)
        tail = (ctx.positions, meta["block_table"], meta["tok_part_row"])
        if family != "simt":
            if n_small:          # decoded tokens and short portions: 16-row tiles, key splits merged by the last CTA
                chunks = -(-self.heads // ROW_TILE)
                counters = ws.get_zeroed("attn_counters", (T * chunks,), torch.int32)
                if family == "tc":      # TMA-fed tiles
                    K.attention_tma_ext(*args, meta["items"], n_small, 16, *tail, nq=self.heads, nkv=1, d=self.width,
                                        page_size=cache.page_size, window=self.window or 0, scale=self.scale,
                                        shared_kv=True, **opts, tok_nsplit=meta["tok_nsplit"], counters=counters,
                                        status=ctx.status)
                else:
                    K.attention_mma_ext(*args, meta["items"], n_small, 16, *tail, **common,
                                        tok_nsplit=meta["tok_nsplit"], counters=counters)
            big_items = meta["items"][n_small * ITEM_INTS:]
            if n_big and family == "tc":      # long portions: tcgen05 128-row tiles, split along the keys when few
                K.attention_tc_ext(q_full, cache.storage, lat, big_items, n_big, ctx.positions, meta["block_table"],
                                   nq=self.heads, nkv=1, d=self.width, page_size=cache.page_size,
                                   window=self.window or 0, scale=self.scale, status=ctx.status, part_acc=part_acc,
                                   part_ml=part_ml, tok_part_row=meta["tok_part_row"], shared_kv=True, **opts)
                if meta.get("big_split"):
                    K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], lat,
                                        nq=self.heads, d=vw, **gate)
            elif n_big:          # long portions: 64-row tiles
                K.attention_mma_ext(*args, big_items, n_big, 64, *tail, **common)
        else:
            n = n_small + n_big
            if n:
                K.attention_simt(*args, meta["items"], n, n, *tail, **common)
            if meta["any_split"]:
                K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], lat, nq=self.heads,
                                    d=vw, **gate)
        attn = ws.get("la_attn", (T, self.heads, self.dv), rt.dtype)
        K.head_linear(lat[:, :, :self.rank], self.uv, attn)
        return rt.linear(attn.view(T, self.ow), self.o_weight, ws, "mix_out", out_dtype=torch.float32)
