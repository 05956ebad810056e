"""Rizovik on the host: the configuration reader, the spec it makes (layers that run another layer's tensors over
caches of their own, layers without a feed-forward), the tensors it expects, the caches it asks for (a page with a
tail for block means, one slot for state and kept inputs) and the plain functions beside hand-made cases.  No GPU."""
import copy

import pytest
import torch

from mini_hisparse_b200.config.qwen2 import ConfigError
from mini_hisparse_b200.config.registry import resolve
from mini_hisparse_b200.config.rizovik import RizovikConfig
from mini_hisparse_b200.parts.registry import MIXERS
from mini_hisparse_b200.parts.spec import PagedKVNeed, StateNeed
from mini_hisparse_b200.weights.expected import expected_tensors_of_spec
from plain import rizovik_plain as P


def config():
    pooled = dict(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.3, mask=dict(size=6, pool=3), rot=dict(dims=4, base=50.0))
    kept = dict(heads=6, kv_heads=3, dim=8, vdim=4, scale=0.25, mask=dict(size=5, keep_first=2),
                rot=dict(dims=8, base=70.0, scaling=dict(factor=4.0)))
    delta = dict(heads=4, kv_heads=2, dim=4, vdim=6, conv=3)
    moe = dict(kind="moe", expert=dict(ff=24), router=dict(experts=5, top=2))
    return dict(architecture="Rizovik", vocab=50, width=40, norm=dict(eps=1e-5), residual_mult=0.7, layers=[
        dict(type="attention", mixer=pooled, mlp=moe), dict(type="attention_2", mixer=kept, mlp=copy.deepcopy(moe)),
        dict(type="delta", mixer=delta, mlp=None),
        dict(type="attention", mixer=copy.deepcopy(pooled), mlp=copy.deepcopy(moe), weights_of=0),
        dict(type="delta", mixer=dict(delta), mlp=None, weights_of=2)])


def test_run_order_names_and_cache_needs():
    cfg, spec = resolve(config())
    assert isinstance(cfg, RizovikConfig) and cfg.residual_mult == 0.7 and len(cfg.layers) == 5
    # three layers store tensors; the fourth and fifth entries run the first and third once more, each over its own cache
    assert [layer.prefix for layer in spec.layers] == ["l0", "l1", "l2"]
    assert [(e.layer, e.cache_of) for e in spec.order] == [(0, None), (1, None), (2, None), (0, None), (2, None)]
    assert all(layer.block == "post_norm" and layer.option("alpha") == 0.0 and layer.option("keep") == 1.0 for layer in spec.layers)
    names = expected_tensors_of_spec(spec)
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g", "l0.mix.o",
            "l0.mix.q.norm", "l0.mix.k.norm", "l0.mlp.router", "l0.mlp.router.b", "l0.mlp.e0.gate", "l0.mlp.e4.down",
            "l1.mix.talk", "l1.mix.q.norm", "l2.norm1", "l2.mix.q.conv", "l2.mix.k.conv", "l2.mix.v.conv", "l2.mix.b",
            "l2.mix.a", "l2.mix.A_log", "l2.mix.dt_bias", "l2.mix.g", "l2.mix.norm", "l2.mix.o"} <= set(names)
    assert not any(n.startswith(("l3.", "l4.", "l2.mlp", "l2.norm2", "l0.mlp.e5", "l0.mlp.correction", "l1.mix.g")) for n in names)
    assert names["l0.mix.q.norm"].shape == (32,) and names["l0.mix.k.norm"].shape == (16,)        # over the whole projection
    assert names["l1.mix.q.norm"].shape == (8,) and names["l1.mix.k.norm"].shape == (8,)         # one weight for all heads
    assert names["l1.mix.talk"].shape == (6, 6) and names["l0.mix.g"].shape == (48, 40) and names["l0.mix.o"].shape == (40, 48)
    assert names["l2.mix.q"].shape == (8, 40) and names["l2.mix.v"].shape == (24, 40) and names["l2.mix.v.conv"].shape == (24, 3)
    assert names["l2.mix.b"].shape == (4, 40) and names["l2.mix.A_log"].shape == (4,) and names["l2.mix.norm"].shape == (6,)
    assert names["l0.mlp.router"].shape == (5, 40) and names["l0.mlp.router.b"].shape == (5,)
    mixers = [MIXERS.build(layer.part("mixer")) for layer in spec.layers]
    need = mixers[0].cache_need()
    assert need == PagedKVNeed(kv_heads=2, head_dim=8, window=None, v_dim=12, pool=3)
    assert need.page_shape(16) == (2 * (16 + 6) * 20,) and need.page_shape(4) == (2 * (4 + 2) * 20,)     # ceil(P / pool) means
    assert mixers[1].cache_need() == PagedKVNeed(kv_heads=3, head_dim=8, window=None, v_dim=4)
    assert mixers[2].cache_need() == StateNeed(shape=(4 * 4 * 6 + 2 * (2 * 2 * 4 + 4 * 6),), dtype="float32")
    assert mixers[1].position.scaling_factor == 4.0
    torch.testing.assert_close(mixers[1].position.inv_freq.double(), 70.0 ** (-torch.arange(0, 8, 2).double() / 8) / 4.0,
                               rtol=1e-7, atol=0)
    # the multiplier rides in the norms' weights
    assert spec.layers[0].part("mixer_norm")["gain"] == 0.7 and spec.final_norm.get("gain") is None


def test_a_layer_may_run_a_later_layers_tensors():
    c = config()
    c["layers"][0]["weights_of"] = 3
    del c["layers"][3]["weights_of"]
    cfg, spec = resolve(c)
    assert [layer.prefix for layer in spec.layers] == ["l1", "l2", "l3"]
    assert [e.layer for e in spec.order] == [2, 0, 1, 2, 1]
    assert "l3.mix.q" in expected_tensors_of_spec(spec) and "l0.mix.q" not in expected_tensors_of_spec(spec)


def test_optional_pieces():
    c = config()
    del c["layers"][1]["mixer"]["rot"]["scaling"]
    del c["layers"][1]["mixer"]["mask"]["keep_first"]
    del c["layers"][0]["mixer"]["rot"]
    c["layers"][3]["mixer"] = dict(c["layers"][0]["mixer"])
    cfg, spec = resolve(c)
    assert cfg.layers[1].mixer.rot_factor == 1.0 and cfg.layers[1].mixer.keep_first == 0
    assert spec.layers[0].part("mixer")["position"].kind == "none"


@pytest.mark.parametrize("change,text", [
    (lambda c: c.update(extra=1), "unknown key"),
    (lambda c: c["layers"][0]["mixer"].update(sink=True), "unknown key"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=1), "unknown key"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(pool=2), "unknown key"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not a feed-forward"),
    (lambda c: c["layers"][0].update(type="lstm"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "lacks"),
    (lambda c: c.pop("residual_mult"), "lacks"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "divisor"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "even"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "make no sense"),
    (lambda c: c["layers"][3].update(weights_of=3), "another layer"),
    (lambda c: c["layers"][3].update(weights_of=4), "tensors of its own"),
    (lambda c: c["layers"][3]["mixer"]["mask"].update(size=7), "entries differ"),
])
def test_what_the_reader_refuses(change, text):
    c = copy.deepcopy(config())
    change(c)
    with pytest.raises(ConfigError, match=text):
        RizovikConfig.from_dict(c)


def test_plain_masks_by_hand():
    """Window 3, blocks of 2: query 6 sees positions 4, 5, 6 and the blocks {0, 1} and {2, 3}; query 4 sees 2, 3, 4 and
    block {0, 1}; query 3 sees 1, 2, 3 and no block (block {0, 1} ends at 1 > 3 - 3).  With all scores equal the output
    is the plain mean of what is seen."""
    L = 7
    k = torch.zeros(L, 1, 2, dtype=torch.float64)
    v = torch.arange(L, dtype=torch.float64).view(L, 1, 1)
    q = torch.zeros(L, 1, 2, dtype=torch.float64)
    out = P.pooled_window_softmax(q, k, v, 1.0, 3, 2)[:, 0, 0]
    assert out[6] == pytest.approx((4 + 5 + 6 + 0.5 + 2.5) / 5)
    assert out[4] == pytest.approx((2 + 3 + 4 + 0.5) / 4)
    assert out[3] == pytest.approx((1 + 2 + 3) / 3)
    assert out[0] == 0 and out[2] == pytest.approx(1.0)
    # kept first 2, window 3: query 6 sees 0, 1, 4, 5, 6; with the identity as mix the heads stay apart
    out = P.kept_first_mixed(q, k, v, torch.eye(1, dtype=torch.float64), 1.0, 3, 2)[:, 0, 0]
    assert out[6] == pytest.approx((0 + 1 + 4 + 5 + 6) / 5) and out[3] == pytest.approx((0 + 1 + 2 + 3) / 4)
    # two heads over one KV head, mixed: head 0 takes twice head 1's weights
    q2 = torch.zeros(L, 2, 2, dtype=torch.float64)
    q2[:, 1, 0] = 1.0
    k2 = k.clone()
    k2[5, 0, 0] = 30.0                                   # head 1 looks at position 5 only (when it sees it)
    talk = torch.tensor([[0.0, 2.0], [1.0, 0.0]], dtype=torch.float64)
    out = P.kept_first_mixed(q2, k2, v, talk, 1.0, 3, 0)
    assert out[6, 0, 0] == pytest.approx(2 * 5.0, abs=1e-6) and out[6, 1, 0] == pytest.approx(5.0)


def test_plain_router_and_convolution_by_hand():
    w = {"router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=torch.float64),
         "router.b": torch.tensor([0.0, 0.5, -3.0], dtype=torch.float64)}
    h = torch.tensor([[1.0, 1.0], [2.0, 0.0]], dtype=torch.float64)
    chosen, weights = P.route(h, w, "", dict(experts=3, top=2))
    assert chosen.tolist() == [[1, 0], [0, 1]]            # logits [1, 1.5, -1] and [2, 0.5, -1]
    assert weights[0].tolist() == pytest.approx(torch.softmax(torch.tensor([1.5, 1.0]), 0).tolist())
    z = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=torch.float64)
    y = P.short_convolution(z, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))      # the last tap is the current token's
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0]
