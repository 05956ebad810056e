"""Tudasun on the host: the configuration reader, the spec it makes (a latent layer that reads another layer's
rows, layers without a feed-forward, the per-layer token input), the tensors it expects, the caches it asks for
and the plain router beside a hand-made case.  No GPU."""
import copy

import pytest
import torch

from mini_hisparse_b200.config.qwen2 import ConfigError
from mini_hisparse_b200.config.registry import resolve
from mini_hisparse_b200.config.tudasun import TudasunConfig
from mini_hisparse_b200.parts.registry import MIXERS
from mini_hisparse_b200.parts.spec import PagedRowsNeed, StateNeed
from mini_hisparse_b200.weights.expected import expected_tensors_of_spec
from plain import tudasun_plain as P


def config():
    lat = dict(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, scale=0.2, rot=dict(dims=4, base=50.0))
    moe = dict(kind="moe", expert=dict(ff=24), shared=dict(ff=40),
               router=dict(experts=6, identity=2, top=2, groups=dict(count=4, keep=2)))
    return dict(architecture="Tudasun", vocab=50, width=40, norm=dict(eps=1e-5), logit_softcap=20.0,
                token_side=dict(dim=6), layers=[
                    dict(type="hgrn2", mixer=dict(heads=2, dim=8, vdim=12), mlp=dict(kind="dense", ff=48)),
                    dict(type="latent_attention", mixer=dict(lat), mlp=moe),
                    dict(type="gla", mixer=dict(heads=5, dim=4, vdim=8, tau=8.0, decay_rank=3), mlp=None),
                    dict(type="latent_attention", mixer=dict(lat, heads=2, kv_from=1), mlp=dict(kind="dense", ff=56))])


def test_run_order_names_and_cache_needs():
    cfg, spec = resolve(config())
    assert isinstance(cfg, TudasunConfig) and cfg.softcap == 20.0 and cfg.side_dim == 6
    # the fourth layer owns no rows: its entry reads the cache of the second layer's entry
    assert [(e.layer, e.cache_of) for e in spec.order] == [(0, None), (1, None), (2, None), (3, 1)]
    names = expected_tensors_of_spec(spec)
    assert {"embed", "side.embed", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.rg1",
            "l0.rg1.b", "l0.rg2", "l0.rg2.b", "l0.mix.q", "l0.mix.f", "l0.mix.f.b", "l0.mix.lower", "l0.mix.v", "l0.mix.norm",
            "l0.mix.o", "l0.mlp.up", "l0.mlp.down", "l0.mlp.act", "l0.side.gate", "l0.side.proj", "l0.side.norm",
            "l1.mix.q", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv", "l1.mix.sink", "l1.mix.o",
            "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e0.gate", "l1.mlp.e5.down", "l1.mlp.shared.gate",
            "l1.mlp.shared.up", "l1.mlp.shared.down", "l1.mlp.shared.sg", "l2.mix.a1", "l2.mix.a2", "l2.mix.a2.b",
            "l2.mix.g", "l2.mix.k", "l3.mix.uk", "l3.mix.sink"} <= set(names)
    # identity experts store nothing; a layer without a feed-forward has no second pair of norms and no second gate;
    # a layer that reads another's rows has no down-projection; latent attention here has no gate per head
    assert not any(n.startswith(("l1.mlp.e6", "l1.mlp.e7", "l2.mlp", "l2.norm2", "l2.rg2", "l3.mix.dkv")) for n in names)
    assert "l1.mix.g" not in names and "l3.mix.g" not in names
    assert names["side.embed"].shape == (50, 4 * 6) and names["l1.mlp.router"].shape == (8, 40)
    assert names["l1.mlp.correction"].shape == (8,) and names["l1.mlp.shared.sg"].shape == (1, 40)
    assert names["l0.mix.q"].shape == (16, 40) and names["l0.mix.v"].shape == (24, 40) and names["l0.mix.norm"].shape == (12,)
    assert names["l2.mix.a1"].shape == (3, 40) and names["l2.mix.a2"].shape == (20, 3) and names["l2.mix.g"].shape == (40, 40)
    assert names["l1.mix.q"].shape == (3 * 12, 40) and names["l1.mix.dkv"].shape == (24, 40)
    assert names["l3.mix.q"].shape == (2 * 12, 40) and names["l3.mix.uv"].shape == (2 * 12, 20) and names["l3.mix.sink"].shape == (2,)
    assert names["l0.mlp.act"].shape == (4,) and names["l0.rg1"].shape == (40, 40)
    mixers = [MIXERS.build(layer.part("mixer")) for layer in spec.layers]
    assert mixers[0].cache_need() == StateNeed(shape=(2, 8, 12), dtype="float32")
    assert mixers[2].cache_need() == StateNeed(shape=(5, 4, 8), dtype="float32")
    assert mixers[1].cache_need() == PagedRowsNeed(width=24, window=None) == mixers[3].cache_need()
    assert mixers[1].cache_need().page_shape(8) == (8, 24)
    assert mixers[1].own_kv and not mixers[3].own_kv


def test_what_may_be_left_out():
    c = config()
    c.pop("token_side")
    c.pop("logit_softcap")
    c["layers"][1]["mlp"].pop("shared")
    c["layers"][1]["mlp"]["router"].pop("groups")
    c["layers"][1]["mlp"]["router"]["identity"] = 0
    c["layers"][2]["mixer"].pop("decay_rank")          # then the stored matrices say it
    cfg, spec = resolve(c)
    names = expected_tensors_of_spec(spec)
    assert cfg.softcap is None and cfg.side_dim is None and not spec.shared
    assert not any("side" in n or "shared" in n for n in names)
    assert names["l1.mlp.router"].shape == (6, 40) and names["l2.mix.a1"].shape == (-1, 40)


def test_what_the_reader_refuses():
    for change in (lambda c: c.update(extra=1), lambda c: c.pop("width"), lambda c: c["norm"].update(kind="rms"),
                   lambda c: c["layers"][0].update(type="conv"), lambda c: c["layers"][0]["mixer"].update(tau=2.0),
                   lambda c: c["layers"][0]["mlp"].update(kind="routed"), lambda c: c["layers"][2]["mixer"].pop("tau"),
                   lambda c: c["layers"][2]["mixer"].update(tau=0.0), lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
                   lambda c: c["layers"][1]["mixer"]["rot"].update(dims=2), lambda c: c["layers"][1]["mixer"].update(window=8),
                   lambda c: c["layers"][3]["mixer"].update(kv_from=3), lambda c: c["layers"][3]["mixer"].update(kv_from=0),
                   lambda c: c["layers"][3]["mixer"].update(kv_rank=16), lambda c: c["layers"][1]["mixer"].update(kv_from=3),
                   lambda c: c["layers"][1]["mlp"]["router"].update(top=5),                     # two kept groups hold four
                   lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3),         # eight outputs in three groups
                   lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=5),
                   lambda c: c["layers"][1]["mlp"]["expert"].update(bias=True), lambda c: c.update(logit_softcap=-1.0)):
        c = copy.deepcopy(config())
        change(c)
        with pytest.raises(ConfigError):
            TudasunConfig.from_dict(c)


def test_the_plain_router_on_a_case_made_by_hand():
    """Six outputs in three groups of which two are kept, two chosen.  The softmax favours output 4; the correction
    lifts output 0 above everything and pushes 4's group out; weights are the chosen outputs' softmax values
    without the correction, divided by their sum."""
    logits = torch.tensor([[0.0, 1.0, 2.0, 0.5, 3.0, 0.2]], dtype=torch.float64)
    w = {"router": torch.eye(6, dtype=torch.float64), "correction": torch.tensor([2.0, 0.0, 0.0, 0.0, -1.0, 0.0], dtype=torch.float64)}
    r = dict(experts=4, identity=2, top=2, groups=dict(count=3, keep=2))
    s = torch.softmax(logits, -1)[0]
    chosen, weights = P.route(logits, w, "", r)
    # groups (0,1), (2,3), (4,5): group scores s0 + 2, s2, max(s4 - 1, s5) -> the first two are kept
    assert chosen[0].tolist() == [0, 2]
    torch.testing.assert_close(weights[0], torch.stack((s[0], s[2])) / (s[0] + s[2]))
    # without groups output 1 (0.08) still loses to output 2 (0.21) and output 4 (0.57 - 1) is negative
    chosen, _ = P.route(logits, w, "", dict(r, groups=None))
    assert chosen[0].tolist() == [0, 2]
    # every choice score negative: the dropped groups must not win by counting as zero
    w["correction"] = torch.tensor([-5.0, -5.0, -5.0, -5.0, -9.0, -9.0], dtype=torch.float64)
    chosen, _ = P.route(logits, w, "", dict(r, groups=dict(count=3, keep=1)))
    assert sorted(chosen[0].tolist()) == [2, 3]
