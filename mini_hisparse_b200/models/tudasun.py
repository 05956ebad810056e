"""Tudasun as data: the ModelSpec of a TudasunConfig and its registry entry.

Every layer is a sandwich block: a norm (RMS, weight stored around zero: 1 + w) before and behind each sublayer,
the sublayer's result multiplied by a sigmoid gate computed from the sublayer's input before the behind norm.  The
mixer is gated linear attention or HGRN2 (a decay per key channel computed from the input, a float32 state per request)
or latent attention (a cached low-rank row and one rotated key part shared by the heads, a softmax sink per head);
a latent layer with ``kv_from`` has no rows of its own: its run entry reads the cache of the layer it names.  The
feed-forward is dense with the PolyNorm activation, or routed (experts and identity experts in groups, a shared
expert).  Every layer ends with an input from the token itself (a slice of a table shared by all layers).  The
logits are capped by tanh.  Tensor names: embed, side.embed, l<i>.{norm1, norm1b, norm2, norm2b, rg1, rg1.b, rg2,
rg2.b, mix.*, mlp.*, side.*}, final.norm, head.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tudasun import DenseFF, TudasunConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def tudasun_spec(cfg: TudasunConfig) -> ModelSpec:
    W = cfg.width
    norm = PartSpec.make("rmsnorm", width=W, eps=cfg.eps, weight_name="", offset=1.0)
    gate = PartSpec.make("linear_gate", hidden_size=W, width=W, weight_name="", bias_name="b")
    layers, order, entry_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        entry = RunEntry(i)
        if layer.type == "gla":
            mixer = PartSpec.make("gla", hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau,
                                  decay_rank=m.decay_rank, eps=cfg.eps)
        elif layer.type == "hgrn2":
            mixer = PartSpec.make("hgrn2", hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, eps=cfg.eps)
        else:
            position = (PartSpec.make("rotary", head_dim=m.rot_dim, theta=m.rot_base, rotary_dim=m.rot_dim,
                                      style="interleaved") if m.rot_dim else PartSpec.make("none"))
            mixer = PartSpec.make("latent_attention", hidden_size=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim,
                                  vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale, window=None, eps=cfg.eps,
                                  position=position, gate=False, sink=True, own_kv=m.kv_from is None)
            if m.kv_from is not None:
                entry = RunEntry(i, cache_of=entry_of[m.kv_from])
        entry_of[i] = len(order)
        order.append(entry)
        parts = {"mixer_norm": norm, "mixer": mixer, "mixer_gate": gate, "mixer_post_norm": norm}
        if layer.mlp is not None:
            if isinstance(layer.mlp, DenseFF):
                ff = PartSpec.make("mlp_act", hidden_size=W, intermediate_size=layer.mlp.ff, activation="polynorm",
                                   eps=cfg.eps, coef_name="act")
            else:
                r = layer.mlp
                ff = PartSpec.make("routed_experts", hidden_size=W, experts=r.experts, identity=r.identity, top=r.top,
                                   group_count=r.group_count, group_keep=r.group_keep, expert_ff=r.expert_ff,
                                   shared_ff=r.shared_ff)
            parts.update({"ff_norm": norm, "feed_forward": ff, "ff_gate": gate, "ff_post_norm": norm})
        if cfg.side_dim is not None:
            parts["side"] = PartSpec.make("token_side", hidden_size=W, dim=cfg.side_dim, column0=i * cfg.side_dim,
                                          eps=cfg.eps, table="side")
        layers.append(LayerSpec.make(f"l{i}", "sandwich", parts,
                                     {"mixer_norm": "norm1", "mixer": "mix", "mixer_gate": "rg1", "mixer_post_norm": "norm1b",
                                      "ff_norm": "norm2", "feed_forward": "mlp", "ff_gate": "rg2", "ff_post_norm": "norm2b",
                                      "side": "side"}))
    shared = ()
    if cfg.side_dim is not None:
        shared = (("side", PartSpec.make("token_table", vocab_size=cfg.vocab, width=len(cfg.layers) * cfg.side_dim,
                                         weight_name="embed"), "side"),)
    return ModelSpec(
        architecture="Tudasun", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec.make("token_embedding", vocab_size=cfg.vocab, hidden_size=W, weight_name=""),
        embedding_name="embed", layers=tuple(layers), order=tuple(order),
        final_norm=norm, final_norm_name="final.norm",
        head=PartSpec.make("lm_head", vocab_size=cfg.vocab, hidden_size=W, tied=False, weight_name="",
                           softcap=cfg.softcap),
        head_name="head", shared=shared,
    )


register_architecture("Tudasun", TudasunConfig, tudasun_spec, replace=True)
