"""Rizovik as data: the ModelSpec of a RizovikConfig and its registry entry.

Every layer normalises its sublayers' OUTPUTS only: x <- x + m n1(mixer(x)), x <- x + m n2(ff(x)) with a fixed
multiplier m; mixer and feed-forward read the stream itself.  That is the post-norm arrangement with the stream kept
beside the norm (alpha = 0, keep = 1) and m folded into the norms' weights.  The mixer is sliding-window attention that
sees the window's past as block means ("attention"), sliding-window attention that keeps the first positions and mixes
the heads' softmax weights ("attention_2"), or the gated delta rule ("delta"); the feed-forward is routed (the largest
router logits, a softmax over the chosen ones).  A layer with ``weights_of`` is a second run entry of the layer it names:
the same parts, a cache or state of its own.  The head is the embedding table.  Tensor names: embed,
l<i>.{norm1, norm2, mix.*, mlp.*}, final.norm.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.rizovik import DeltaMixer, RizovikConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def rizovik_spec(cfg: RizovikConfig) -> ModelSpec:
    W = cfg.width
    add_norm = PartSpec.make("rmsnorm", width=W, eps=cfg.eps, weight_name="", gain=cfg.residual_mult)
    layers, order, spec_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        m = layer.mixer
        if isinstance(m, DeltaMixer):
            mixer = PartSpec.make("gated_delta", hidden_size=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim,
                                  vdim=m.vdim, conv=m.conv, eps=cfg.eps)
        else:
            position = (PartSpec.make("rotary", head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims,
                                      scaling_factor=m.rot_factor, float64_table=True)
                        if m.rot_dims else PartSpec.make("none"))
            common = dict(hidden_size=W, q_heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale,
                          window=m.window, eps=cfg.eps, position=position)
            if layer.type == "attention":
                mixer = PartSpec.make("pooled_window_attention", pool=m.pool, **common)
            else:
                mixer = PartSpec.make("kept_first_attention", keep_first=m.keep_first, **common)
        parts = {"mixer": mixer, "mixer_norm": add_norm}
        if layer.mlp is not None:
            r = layer.mlp
            parts.update({"feed_forward": PartSpec.make("routed_experts", hidden_size=W, experts=r.experts, top=r.top,
                                                        expert_ff=r.expert_ff, correction=False, router_bias=True),
                          "ff_norm": add_norm})
        spec_of[i] = len(layers)
        layers.append(LayerSpec.make(f"l{i}", "post_norm", parts,
                                     {"mixer": "mix", "mixer_norm": "norm1", "feed_forward": "mlp", "ff_norm": "norm2"},
                                     options={"alpha": 0.0, "keep": 1.0}))
    for i, layer in enumerate(cfg.layers):
        order.append(RunEntry(spec_of[i if layer.weights_of is None else layer.weights_of]))
    return ModelSpec(
        architecture="Rizovik", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec.make("token_embedding", vocab_size=cfg.vocab, hidden_size=W, weight_name=""),
        embedding_name="embed", layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec.make("rmsnorm", width=W, eps=cfg.eps, weight_name=""), final_norm_name="final.norm",
        head=PartSpec.make("lm_head", vocab_size=cfg.vocab, hidden_size=W, tied=True, weight_name="weight"),
        head_name="head",
    )


register_architecture("Rizovik", RizovikConfig, rizovik_spec, replace=True)
