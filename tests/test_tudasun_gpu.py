"""Tudasun through the engine against the plain implementation of tests/plain/tudasun_plain.py.

Small configurations made here (none is anyone's model), random weights from a seed.  Covered: the kernels of each
mechanism alone (the gated, normalised residual addition with the next norm; PolyNorm; the cap on the logits; the
inputs of the two recurrences; the recurrence token by token and in chunks over slots that hold another request's
state, with one early token made to stand out; the norm per head with its multiplier; the router with groups,
negative choice scores and identity experts; the grouped products and the weighted sum; latent attention with a sink
over rows that stand out far back and at page borders); whole prompts; prefill against token-by-token decoding
(through captured graphs); portions down to two tokens; mixed batches over a tight pool whose freed pages are
poisoned; slots used again; long decoding; sizes that are equal or 1; generation through Engine and its scheduler;
the command line; bin/trace_run.
"""
import copy
import json
import math

import pytest
import torch

import schedules as S
from conftest import TraceRun, random_tokens, row_rms_error
from plain import tudasun_plain as P
from test_dotivik_gpu import Parts, attend, dev_i, run_steps

pytestmark = pytest.mark.gpu


def decay_mixer(kind, heads, dim, vdim, tau=None, rank=None):
    m = dict(heads=heads, dim=dim, vdim=vdim)
    if kind == "gla":
        m.update(tau=tau, decay_rank=rank)
    return m


def latent(heads, dim, rot_dim, vdim, rank, base=3000.0, scale=0.3, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=scale, rot=dict(dims=rot_dim, base=base))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return dict(kind="dense", ff=ff)


def routed(experts, identity, top, ff, groups=None, shared=None):
    router = dict(experts=experts, identity=identity, top=top)
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    m = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared is not None:
        m["shared"] = dict(ff=shared)
    return m


def layer(kind, mixer, mlp=None):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def model(vocab, width, layers, side=None, cap=None, eps=1e-5):
    cfg = dict(architecture="Tudasun", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if side is not None:
        cfg["token_side"] = dict(dim=side)
    if cap is not None:
        cfg["logit_softcap"] = cap
    return cfg


# A: every branch at once: both recurrences with heads of unequal key and value widths, latent attention whose rows
# a later layer reads with other heads, dense and routed feed-forwards (groups, identity experts, a shared expert),
# a layer without a feed-forward, the per-layer token input, capped logits; widths that are multiples of 8.
CFG_A = model(211, 96, [
    layer("hgrn2", decay_mixer("hgrn2", 3, 16, 24), dense(160)),
    layer("latent_attention", latent(6, 24, 8, 40, 48), routed(6, 2, 3, 32, groups=(4, 2), shared=64)),
    layer("gla", decay_mixer("gla", 4, 8, 24, tau=8.0, rank=5)),
    layer("latent_attention", latent(3, 24, 8, 16, 48, scale=0.5, kv_from=1), routed(5, 0, 2, 40, shared=24)),
    layer("gla", decay_mixer("gla", 2, 24, 16, tau=2.0, rank=12), dense(72))], side=12, cap=12.0)
# B: values that the usual model makes different are equal or 1 here: one head, keys as wide as values, a decay of
# rank 1 with tau 1, one expert a token out of one group with no identity and no shared expert, an identity expert
# as the only other choice, a latent as wide as a head, no token input, no cap, a width that no tensor-core product
# takes (not a multiple of 8).
CFG_B = model(97, 100, [
    layer("gla", decay_mixer("gla", 1, 20, 20, tau=1.0, rank=1), routed(3, 0, 1, 20, groups=(1, 1))),
    layer("latent_attention", latent(1, 20, 2, 20, 20, scale=1.0), routed(1, 1, 1, 12)),
    layer("hgrn2", decay_mixer("hgrn2", 1, 12, 12)),
    layer("latent_attention", latent(3, 12, 2, 12, 20, scale=0.7, kv_from=1), dense(50)),
    layer("hgrn2", decay_mixer("hgrn2", 5, 4, 20), routed(4, 4, 8, 16, groups=(2, 2), shared=100))])
# C: sizes of a real model's order: recurrent heads of 128 x 128, a cache row of 128 under many heads (tcgen05
# attention in bfloat16), experts in tiles of many rows.
CFG_C = model(300, 256, [
    layer("latent_attention", latent(16, 64, 32, 64, 96, base=1e6, scale=0.1), routed(8, 0, 2, 128, groups=(2, 1), shared=256)),
    layer("gla", decay_mixer("gla", 2, 128, 128, tau=16.0, rank=16), dense(512)),
    layer("hgrn2", decay_mixer("hgrn2", 2, 128, 128), routed(16, 4, 4, 64, groups=(5, 3))),
    layer("latent_attention", latent(4, 128, 32, 128, 96, base=1e6, scale=0.08, kv_from=0), dense(384))], side=16, cap=30.0)
# D: widths beyond the usual tiles: a cache row of 160 (the CUDA-core attention serves bfloat16 too), heads of 40 x 72
# and 200 x 8, thirteen experts of which one token uses five.
CFG_D = model(150, 128, [
    layer("gla", decay_mixer("gla", 3, 40, 72, tau=4.0, rank=7), routed(10, 3, 5, 24, shared=40)),
    layer("latent_attention", latent(4, 32, 32, 48, 128, scale=0.2), dense(256)),
    layer("hgrn2", decay_mixer("hgrn2", 1, 200, 8), dense(128))], side=8, cap=50.0)
CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}
# A row's error: the root mean square of (got - plain) as a share of the row's root mean square.  float32: the plain
# model is computed in float64; the design itself, computed in float32 in any order, differs from that by up to 4e-5
# at single positions (a sublayer's result that nearly cancels is normalised right after), and by 2e-6 on average:
# the mean is held tightly, the worst row loosely.  bfloat16: the router sees the bfloat16 rounding of its input, so
# that at a few tokens another expert wins a close call than in the plain model; again the mean over all rows is held
# tightly and the worst row loosely; every schedule is compared with the WHOLE prompt in the same dtype as well.
BF16_MEAN, BF16_WORST = 0.04, 0.8
F32_MEAN, F32_ROW = 1.5e-5, 1.5e-4
BF16_CUT_MEAN, BF16_CUT = 0.02, 0.5
SENSITIVE = 1e-3                   # what a fault of the kinds the tests are for moves the plain model's logits by, at least


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    from mini_hisparse_b200 import write_random_model

    out = {}
    for name, cfg in CONFIGS.items():
        folder = tmp_path_factory.mktemp(f"tudasun{name}")
        write_random_model(cfg, 37, folder, dtype=torch.bfloat16, matrix_std=0.15)
        out[name] = (folder, *P.load_folder(folder))
    return out


def requests_for(cfg, lengths, seed=0):
    return {f"r{i}": random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


def row_errors(got, ref):
    return (got.double() - ref.double()).pow(2).mean(-1).sqrt() / ref.double().pow(2).mean(-1).sqrt()


def check_against_plain(got, refs, dtype):
    for rid, ref in refs.items():
        assert got[rid].shape == ref.shape
    err = torch.cat([row_errors(got[rid], ref) for rid, ref in refs.items()])
    mean, worst = (F32_MEAN, F32_ROW) if dtype == "float32" else (BF16_MEAN, BF16_WORST)
    assert float(err.mean()) < mean and float(err.max()) < worst, \
        f"mean row error {float(err.mean()):.3g}, worst {float(err.max()):.3g} at {int(err.argmax())} of all rows"


def close(got, ref, tol, what=""):
    scale = float(ref.abs().max())
    err = float((got.double().cpu() - ref.double()).abs().max())
    assert err < tol * scale, f"{what}: {err:.3g} beside values up to {scale:.3g}"


# ---- the mechanisms alone ---------------------------------------------------------------------------------
@pytest.mark.parametrize("R,H,nsplit,gated", [(37, 96, 1, True), (5, 100, 3, True), (130, 1000, 2, False), (1, 8, 1, True),
                                              (3, 18, 2, True), (2, 8200, 3, True), (4, 4097, 1, False), (6, 96, 2, True)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gated_normalised_addition_with_the_next_norm(R, H, nsplit, gated, out_dtype):
    """x <- x + rms(d * sigmoid(g + b)) * w over split products, the gate a run of columns of a wider product; the
    new rows' copy and their next norm come from the same kernel."""
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(R + H)
    x = torch.randn(R, H, generator=g)
    d = torch.randn(nsplit, R, H, generator=g) * 3
    pad, off = (8, 4) if R % 2 == 0 else (7, 3)        # even R: rows that start on 16 bytes (four neighbours a thread)
    wide = torch.randn(nsplit, R, H + pad, generator=g)
    bias, w, w2 = torch.randn(H, generator=g), 1 + 0.1 * torch.randn(H, generator=g), 1 + 0.1 * torch.randn(H, generator=g)
    eps, eps2 = 1e-5, 1e-3
    y = d.double().sum(0)
    if gated:
        y = y * torch.sigmoid(wide.double().sum(0)[:, off:off + H] + bias.double())
    ref = x.double() + P.unit_rms(y, eps) * w.double()
    ref_next = P.unit_rms(ref, eps2) * w2.double()
    xd, dd, wd = x.cuda(), d.cuda(), wide.cuda()
    delta = Parts(dd if nsplit > 1 else dd[0], nsplit)
    gate = None
    if gated:
        gate = Parts((wd if nsplit > 1 else wd[0])[..., off:off + H], nsplit)
        gate.split_stride = wd.stride(0) if nsplit > 1 else 0
    copy, nxt = torch.empty(R, H, dtype=out_dtype, device="cuda"), torch.empty(R, H, dtype=out_dtype, device="cuda")
    K.gated_norm_add(xd, delta, w.cuda(), eps, gate=gate, bias=bias.cuda() if gated else None, copy=copy,
                     next_weight=w2.cuda(), next_eps=eps2, next_out=nxt)
    close(xd, ref, 2e-6, "stream")
    tol = 2e-6 if out_dtype == torch.float32 else 0.005
    close(copy.float(), ref, tol, "copy")
    close(nxt.float(), ref_next, tol, "next norm")
    x2 = x.cuda()
    K.gated_norm_add(x2, delta, w.cuda(), eps, gate=gate, bias=bias.cuda() if gated else None)     # nothing else wanted
    close(x2, ref, 2e-6, "stream alone")


@pytest.mark.parametrize("R,F,nsplit", [(9, 160, 1), (70, 50, 2), (3, 4096, 1), (2, 1, 1)])
def test_polynorm_and_the_cap(R, F, nsplit):
    """a rms(z) + b rms(z^2) + c rms(z^3) + e, every power by its own root mean square; cap * tanh(z / cap)."""
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(F)
    z = torch.randn(nsplit, R, F, generator=g) * 2
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    ref = P.polynorm(z.double().sum(0), coef.double(), 1e-5)
    for dt, tol in ((torch.float32, 3e-6), (torch.bfloat16, 0.005)):
        out = torch.empty(R, F, dtype=dt, device="cuda")
        zd = z.cuda()
        K.polynorm_rows(zd if nsplit > 1 else zd[0], coef.cuda(), 1e-5, out, nsplit=nsplit,
                        split_stride=zd.stride(0) if nsplit > 1 else 0)
        close(out.float(), ref, tol, f"polynorm {dt}")
    # the three terms are told apart: a wrong pairing of coefficient and power moves the result
    assert float((P.polynorm(z.double().sum(0), coef.double()[[1, 0, 2, 3]], 1e-5) - ref).abs().max()) > 0.1 or F == 1
    t = torch.randn(R, F, generator=g) * 40
    td = t.cuda()
    K.softcap_rows(td, 12.0)
    close(td, 12.0 * torch.tanh(t.double() / 12.0), 2e-6, "cap")


@pytest.mark.parametrize("heads,dk,dv,rank,tau", [(3, 16, 24, 5, 8.0), (1, 20, 20, 1, 1.0), (2, 128, 128, 16, 16.0),
                                                  (5, 64, 96, 4, 2.0), (7, 96, 40, 3, 4.0)])
@pytest.mark.parametrize("nsplit,T", [(1, 45), (2, 45), (2, 70)])
def test_inputs_of_the_two_recurrences(heads, dk, dv, rank, tau, nsplit, T):
    """gla: q scaled, k, v, log decay = logsigmoid(A2 (a1 columns) + b) / tau.  hgrn2: q through silu, forget gate
    above its lower bound, key = 1 - gate, log decay = log gate.  Logits from -60 to 60: nothing overflows.  Few
    tokens spread a row over several CTAs (rows wider than 256, keys wider or narrower than values); many do not."""
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(heads * dk)
    qw, vw = heads * dk, heads * dv
    ld = 2 * qw + 2 * vw + rank + 3
    proj = torch.randn(nsplit, T, ld, generator=g)
    proj[:, 0] *= 30
    pd = proj.cuda()
    prod = Parts(pd if nsplit > 1 else pd[0], nsplit)
    z = proj.double().sum(0)
    a2, bias = torch.randn(qw, rank, generator=g) * 0.5, torch.randn(qw, generator=g) * 2
    low = torch.rand(qw, generator=g) * 0.9
    outs = lambda: [torch.empty(T, n, device="cuda") for n in (qw, qw, vw, qw)]
    q, k, v, lg = outs()
    K.gated_linear_prep("gla", prod, 0, qw, 2 * qw, 2 * qw + 2 * vw, bias.cuda(), q, k, v, lg, a2=a2.cuda(),
                        qscale=dk ** -0.5, tau=tau)
    za = z[:, 2 * qw + 2 * vw: 2 * qw + 2 * vw + rank] @ a2.double().T + bias.double()
    close(q, z[:, :qw] * dk ** -0.5, 2e-6, "gla q")
    close(k, z[:, qw:2 * qw], 2e-6, "gla k")
    close(v, z[:, 2 * qw:2 * qw + vw], 2e-6, "gla v")
    close(lg, (torch.nn.functional.logsigmoid(za) / tau).clamp_min(-80.0), 5e-6, "gla log decay")
    q, k, v, lg = outs()
    K.gated_linear_prep("hgrn2", prod, 0, 0, 2 * qw, qw, bias.cuda(), q, k, v, lg, low=low.cuda())
    f = low.double() + (1 - low.double()) * torch.sigmoid(z[:, qw:2 * qw] + bias.double())
    close(q, P.silu(z[:, :qw]), 2e-6, "hgrn2 q")
    close(k, 1 - f, 2e-6, "hgrn2 key")
    close(v, z[:, 2 * qw:2 * qw + vw], 2e-6, "hgrn2 v")
    close(lg, torch.log(f).clamp_min(-80.0), 5e-6, "hgrn2 log gate")


def plain_decayed(q, k, v, decay, S0):
    """One head from the state S0 [dk, dv]: outputs [n, dv] and the state after the last token."""
    S, out = S0.clone(), []
    for t in range(q.shape[0]):
        S = decay[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out), S


@pytest.mark.parametrize("heads,dk,dv,chunk", [(3, 16, 24, 32), (2, 128, 128, 16), (1, 20, 20, 64), (1, 200, 8, 16), (5, 4, 20, 64),
                                                  (2, 128, 128, 32), (1, 4, 72, 16), (2, 64, 64, 64), (1, 6, 10, 32)])
def test_the_recurrence_token_by_token_in_chunks_and_plain_agree(heads, dk, dv, chunk):
    """Four segments (a long one from position 0 in a slot that holds another request's state, which must not be
    seen; one that goes on from its slot's state; a single token; a portion of two) through the scan and through
    the chunked route.  Decays from nearly 0 to 1.  The first token of the long segment is made to stand out for the
    last one's query (its channels barely decay), so that a state that is lost on the way shows."""
    from mini_hisparse_b200.kernels import api as K
    from mini_hisparse_b200.parts.base import Segment
    from mini_hisparse_b200.parts.lightning import ChunkPlanner

    g = torch.Generator().manual_seed(dk + dv)
    counts, starts, slots = [150, 67, 1, 2], [0, 9, 40, 5], [2, 0, 1, 3]
    T, qw, vw = sum(counts), heads * dk, heads * dv
    q, k = torch.randn(T, qw, generator=g), torch.randn(T, qw, generator=g)
    v = torch.randn(T, vw, generator=g)
    lg = -torch.rand(T, qw, generator=g).pow(3) * 3
    lg[torch.rand(T, qw, generator=g) < 0.05] = -60.0          # a channel that is wiped now and then
    lg[torch.rand(T, qw, generator=g) < 0.2] = 0.0             # and one that keeps everything
    lg[:150, :2] = -1e-4                                        # two channels of head 0 that remember the first token
    k[0, :2], v[0, :dv] = 25.0, 4.0
    q[149, :2] = 3.0
    state0 = torch.randn(4, heads, dk, dv, generator=g)
    segs, tok_seg, pos, off = [], [], [], 0
    for i, (n, st, sl) in enumerate(zip(counts, starts, slots)):
        segs.append(Segment(i, sl, st, n, off))
        tok_seg += [i] * n
        pos += list(range(st, st + n))
        off += n
    refs, ref_state = torch.zeros(T, vw, dtype=torch.float64), state0.double().clone()
    for sg in segs:
        rows = slice(sg.offset, sg.offset + sg.count)
        for h in range(heads):
            S0 = torch.zeros(dk, dv, dtype=torch.float64) if sg.start == 0 else state0[sg.slot, h].double()
            kk, vv = slice(h * dk, (h + 1) * dk), slice(h * dv, (h + 1) * dv)
            o, Sn = plain_decayed(q[rows, kk].double(), k[rows, kk].double(), v[rows, vv].double(),
                                  torch.exp(lg[rows, kk].double()), S0)
            refs[rows, vv] = o
            ref_state[sg.slot, h] = Sn
    # the oracle agrees with the plain model's own scan on the segment that starts at 0
    mine = P.decayed_outer_scan(q[:150].double().view(150, heads, dk), k[:150].double().view(150, heads, dk),
                                v[:150].double().view(150, heads, dv), torch.exp(lg[:150].double()).view(150, heads, dk))
    assert float((mine.reshape(150, vw) - refs[:150]).abs().max()) < 1e-9 * float(refs.abs().max())
    assert float(refs[149, :dv].abs().max()) > 100         # the first token dominates the last output of head 0
    args = lambda st, out: (q.cuda(), k.cuda(), lg.cuda(), v.cuda(), st, out, dev_i(tok_seg), dev_i(slots), dev_i(pos))
    common = dict(heads=heads, dk=dk, dv=dv)
    st1, o1 = state0.cuda().clone(), torch.zeros(T, vw, device="cuda")
    K.gated_linear_scan(*args(st1, o1), **common)
    st2, o2 = state0.cuda().clone(), torch.zeros(T, vw, device="cuda")
    arrays, facts = ChunkPlanner(chunk).plan(segs, T)
    assert facts["num_long"] == 2
    K.gated_linear_scan(*args(st2, o2), **common, max_tokens=16)
    scratch = torch.empty(facts["num_chunks"] * heads * (dk * dv + dk), device="cuda")
    K.gated_linear_chunked(*args(st2, o2), torch.from_numpy(arrays["chunks"]).cuda(), facts["num_chunks"],
                           torch.from_numpy(arrays["seg_chunks"]).cuda(), facts["num_long"], scratch, chunk, **common)
    # a reader that may not write (another layer's state): outputs as before, the slots untouched
    st3, o3 = state0.cuda().clone(), torch.zeros(T, vw, device="cuda")
    K.gated_linear_scan(*args(st3, o3), **common, writable=False)
    assert torch.equal(st3.cpu(), state0)
    for name, o, st in (("scan", o1, st1), ("chunked", o2, st2)):
        for sg in segs:           # every segment against its own scale
            rows = slice(sg.offset, sg.offset + sg.count)
            close(o[rows], refs[rows], 2e-5, f"{name} outputs of segment {sg.request}")
        close(st, ref_state, 1e-5, f"{name} state")
    close(o3, refs, 2e-5, "read-only outputs")


@pytest.mark.parametrize("heads,dv,gated,nsplit", [(3, 24, True, 2), (1, 20, False, 1), (2, 128, True, 1), (5, 8, True, 3)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_per_head_with_its_multiplier(heads, dv, gated, nsplit, out_dtype):
    """Every head by its OWN root mean square, one weight for all heads, times silu of a product's columns."""
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(dv)
    T, vw = 33, heads * dv
    o = torch.randn(T, vw, generator=g) * torch.logspace(-2, 2, heads).repeat_interleave(dv)     # heads of unequal size
    w = 1 + 0.2 * torch.randn(dv, generator=g)
    wide = torch.randn(nsplit, T, vw + 11, generator=g)
    ref = (P.unit_rms(o.double().view(T, heads, dv), 1e-5) * w.double()).reshape(T, vw)
    gate = None
    if gated:
        ref = ref * P.silu(wide.double().sum(0)[:, 6:6 + vw])
        wd = wide.cuda()
        gate = Parts(wd if nsplit > 1 else wd[0], nsplit)
    out = torch.empty(T, vw, dtype=out_dtype, device="cuda")
    K.gated_linear_head_norm(o.cuda(), w.cuda(), 1e-5, out, heads=heads, dv=dv, gate=gate, gate0=6)
    close(out.float(), ref, 3e-6 if out_dtype == torch.float32 else 0.005, "head norm")
    together = P.unit_rms(o.double(), 1e-5) * w.double().repeat(heads)          # one norm over all heads is another thing
    assert heads == 1 or float((together - (ref if not gated else ref / P.silu(wide.double().sum(0)[:, 6:6 + vw]))).abs().max()) > 0.5


@pytest.mark.parametrize("experts,identity,top,groups", [(6, 2, 3, (4, 2)), (16, 4, 3, (2, 1)), (3, 0, 1, None), (1, 1, 1, None),
                                                         (4, 4, 8, (2, 2)), (10, 3, 5, None), (9, 3, 2, (6, 1)), (60, 4, 6, (8, 3))])
@pytest.mark.parametrize("corrections", ["small", "negative"])
def test_router_with_groups_negative_choice_scores_and_identity_experts(experts, identity, top, groups, corrections):
    """Choice by softmax + correction inside the best groups, weights from the softmax alone.  With corrections
    far below zero every choice score is negative: an output of a dropped group (minus infinity, not zero) must still
    lose to them.  The logits are two split parts with the shared expert's gate column behind them."""
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(experts * 7 + top)
    n, T = experts + identity, 257
    z = torch.randn(2, T, n + 3, generator=g) * 1.5
    corr = torch.randn(n, generator=g) * (0.05 if corrections == "small" else 0.3) - (0.0 if corrections == "small" else 2.0)
    r = dict(experts=experts, identity=identity, top=top)
    if groups is not None:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    logits = z.sum(0)[:, :n]          # the plain router gets them through an identity matrix
    chosen_ref, w_ref = P.route(logits.double(), {"router": torch.eye(n, dtype=torch.float64), "correction": corr.double()}, "", r)
    zd = z.cuda()
    chosen = torch.empty(T, top, dtype=torch.int32, device="cuda")
    weights = torch.empty(T, top, device="cuda")
    K.moe_route(Parts(zd, 2), corr.cuda(), chosen, weights, outputs=n, top=top,
                groups=groups[0] if groups else 1, keep=groups[1] if groups else 1)
    dense_ref = torch.zeros(T, n, dtype=torch.float64).scatter(1, chosen_ref, w_ref)
    got_idx = chosen.cpu().long()
    assert int(got_idx.min()) >= 0 and int(got_idx.max()) < n
    assert all(len(set(row)) == top for row in got_idx.tolist())
    dense_got = torch.zeros(T, n, dtype=torch.float64).scatter(1, got_idx, weights.cpu().double())
    assert float((dense_got - dense_ref).abs().max()) < 3e-6
    assert float((weights.sum(-1).cpu() - 1).abs().max()) < 1e-5
    if groups is not None and corrections == "negative" and groups[1] < groups[0]:
        per = n // groups[0]
        assert all(len({i // per for i in row}) <= groups[1] for row in got_idx.tolist())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,identity,top,ff,W,shared", [(5, 2, 2, 40, 96, 64), (1, 1, 1, 12, 100, None), (16, 0, 4, 64, 256, 128),
                                                        (3, 0, 3, 24, 40, None)])
def test_grouped_products_and_the_weighted_sum(dtype, E, identity, top, ff, W, shared):
    """300 tokens of which most choose expert 0 (tiles of many rows) and some experts get few or none: the grouped
    gate/up product with silu, the grouped down product, the weighted sum with identity experts (the input itself)
    and the shared expert under its own sigmoid gate."""
    from mini_hisparse_b200.kernels import api as K

    g = torch.Generator().manual_seed(E + W)
    T, n = 300, E + identity
    h = torch.randn(T, W, generator=g).to(dtype)
    gate_up = (torch.randn(E, 2 * ff, W, generator=g) / math.sqrt(W)).to(dtype)
    down = (torch.randn(E, W, ff, generator=g) / math.sqrt(ff)).to(dtype)
    scores = torch.rand(T, n, generator=g)
    scores[:200, 0] += 2.0                              # a crowded expert
    if n > 2:
        scores[:, n // 2] -= 2.0                        # and a nearly empty one
    chosen = scores.topk(top, -1).indices.to(torch.int32)
    weights = torch.rand(T, top, generator=g) + 0.1
    hd_, w64 = h.double(), lambda t: t.double()
    ref = torch.zeros(T, W, dtype=torch.float64)
    for t in range(T):
        for e, wt in zip(chosen[t].tolist(), weights[t].tolist()):
            if e >= E:
                ref[t] += wt * hd_[t]
            else:
                a = P.silu(w64(gate_up[e, :ff]) @ hd_[t]) * (w64(gate_up[e, ff:]) @ hd_[t])
                if dtype == torch.bfloat16:
                    a = a.to(dtype).double()            # the activation is stored in the compute dtype
                ref[t] += wt * (w64(down[e]) @ a)
    sh = sg = None
    if shared is not None:
        sh_t = torch.randn(2, T, W, generator=g)
        sg_t = torch.randn(2, T, n + 1, generator=g)
        ref += torch.sigmoid(sg_t.double().sum(0)[:, n:n + 1]) * sh_t.double().sum(0)
        shd, sgd = sh_t.cuda(), sg_t.cuda()
        sh, sg = Parts(shd, 2), Parts(sgd[..., n:n + 1], 2)
    pairs = T * top
    hc, cd, wd = h.cuda(), chosen.cuda(), weights.cuda()
    plan = torch.empty(K.moe_plan_words(pairs, E), dtype=torch.int32, device="cuda")
    K.moe_plan(cd, plan, experts=E)
    act = torch.full((pairs, ff), float("nan"), dtype=dtype, device="cuda")
    K.moe_linear(hc, plan, gate_up.cuda(), act, pairs=pairs, experts=E, gather=True, glu=True)
    y = torch.full((pairs, W), float("nan"), device="cuda")
    K.moe_linear(act, plan, down.cuda(), y, pairs=pairs, experts=E, gather=False, glu=False)
    out = torch.empty(T, W, device="cuda")
    K.moe_combine(y, plan, cd, wd, hc, out, experts=E, shared=sh, shared_gate=sg)
    close(out, ref, 1e-5 if dtype == torch.float32 else 0.01, "routed sum")


@pytest.mark.parametrize("dtype,kernel", [(torch.float32, "simt"), (torch.bfloat16, "simt"), (torch.bfloat16, "mma"),
                                          (torch.bfloat16, "tc")])
@pytest.mark.parametrize("page_size,H,rank,dr,L", [(16, 6, 48, 16, 330), (8, 3, 20, 4, 150), (32, 16, 96, 32, 1300), (16, 1, 128, 32, 200),
                                                   (16, 4, 48, 16, 3)])
def test_latent_rows_far_back_at_page_borders_and_the_sink(dtype, kernel, page_size, H, rank, dr, L):
    """Causal latent attention with a sink per head over shuffled pages.  For the probing query the very first row,
    the last row of a page and the first row of the next stand out among hundreds, so that a lost far key or a page
    read one row off shows; one head's sink is large (it takes most of the weight and gives nothing), one's is far
    below every score.  A prompt portion, short portions, single decoded tokens and the first tokens of a sequence
    (where the sink weighs most)."""
    from mini_hisparse_b200.kernels import api as K
    from mini_hisparse_b200.parts.attention import AttentionShape
    from mini_hisparse_b200.parts.base import Segment

    width = rank + dr
    if kernel == "mma" and not K.attention_mma_ext_supports(width, rank):
        pytest.skip("widths the tensor-core attention does not take")
    if kernel == "tc" and not (width in (64, 128) and K.attention_tma_supports(width, page_size)):
        pytest.skip("the tcgen05 kernel takes rows 64 or 128 wide over pages that divide 64")
    vw = width if kernel == "tc" else rank
    g = torch.Generator().manual_seed(L + H)
    scale = 1.7 / math.sqrt(width)
    pages = -(-L // page_size)
    table = torch.randperm(pages + 3, generator=g)[:pages].to(torch.int32)
    rows = torch.randn(L, width, generator=g).to(dtype).double()
    q = torch.randn(L, H, width, generator=g).to(dtype).double()
    probe = L - 2 if L > 3 else L - 1
    marked = [p for p in (0, page_size - 1, page_size, 5 * page_size - 1, 5 * page_size) if p < probe]
    for i, p_ in enumerate(marked):
        qd = q[probe, 0]
        row = qd * ((6.0 + max(0.0, math.log(L / 50)) + 0.5 * i) / (scale * float(qd @ qd)))
        ones = torch.ones(rank, dtype=torch.float64)
        row[:rank] += (2.0 + i) * (ones - qd[:rank] * (float(ones @ qd[:rank]) / float(qd[:rank] @ qd[:rank])))
        rows[p_] = row.to(dtype).double()
    sink = torch.randn(H, generator=g)
    sink[0] = 8.0 + max(0.0, math.log(L / 50))
    if H > 1:
        sink[1] = -30.0
    if H > 2:
        sink[2] = 9.0
    pool = torch.full((pages + 3, page_size, width), 1e30).to(dtype).cuda()
    for p_ in range(L):
        pool[int(table[p_ // page_size]), p_ % page_size] = rows[p_].to(dtype).cuda()

    def plain(sinks, shift=0):
        diff = torch.arange(L)[:, None] - torch.arange(L)[None, :]
        s = torch.einsum("thw,lw->thl", q, rows) * scale
        s = s.masked_fill(~(diff >= shift)[:, None, :], -math.inf)
        if sinks is not None:
            s = torch.cat((s, sinks.double()[None, :, None].expand(L, H, 1)), -1)
        return torch.softmax(s, -1)[..., :L] @ rows[:, :rank]

    right = plain(sink)
    assert float((plain(None)[probe, 0] - right[probe, 0]).abs().max()) > 0.01            # the sink is felt
    assert float((plain(None)[0] - right[0]).abs().max()) > 0.05                          # most of all at the first token
    if len(marked) > 1:
        first = rows[0].clone()
        rows[0] = 0.0
        assert float((plain(sink)[probe, 0] - right[probe, 0]).abs().max()) > 0.05        # and so is the far row
        rows[0] = first
    shape = AttentionShape(H, 1, None, {"tc": 128, "mma": 64, "simt": 16}[kernel])
    bound = 4e-6 if dtype == torch.float32 else 0.02
    portion = min(30, L - 1)
    cuts = [(0, L), (L - portion, portion), (max(0, L - 9), min(9, L)), (probe, 1), (L - 1, 1), (0, min(20, L)), (0, 1), (0, 2)]
    for start, count in cuts:
        seg, r = Segment("a", 0, start, count, 0), torch.arange(start, start + count)
        opts = dict(nq=H, nkv=1, d=width, dv=vw, page_size=page_size, window=0, scale=scale, shared_kv=True, sink=sink.cuda())
        got, plan = attend(K, kernel, dtype, shape, [seg], q[r].to(dtype).cuda().contiguous(), pool, table, (H, vw), dtype, **opts)
        err = float((got[..., :rank] - right[r]).abs().max())
        assert err < bound * float(right.abs().max()), f"tokens {start}..{start + count}: {err:.3g}"


# ---- the model through the step function -----------------------------------------------------------------
PAGES = {"A": 16, "B": 8, "C": 32, "D": 16}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_schedule_agrees_with_the_plain_model(models, name, dtype):
    """Whole prompts; most of a prompt and then its tail token by token, three requests side by side (captured
    graphs); portions of changing size down to two tokens; mixed batches with up to four live requests over a pool
    that holds no more than they need, so that pages and state slots are used again (freed pages are poisoned, a
    slot keeps the last request's state until a new one starts at position 0).  Every position is compared."""
    folder, cfg, w = models[name]
    reqs = requests_for(cfg, [150, 1, 23, 97, 64, 2, 131])
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    whole = None
    for steps in (S.whole(reqs), S.tail_one_by_one(reqs, tail=45), S.changing_portions(reqs), S.mixed(reqs, seed=3)):
        got, runner, cache = run_steps(folder, dtype, steps, page_size=PAGES[name])
        check_against_plain(got, refs, dtype)
        whole = whole or got
        errs = torch.cat([row_errors(got[rid], whole[rid]) for rid in reqs])
        print(f"{name} {dtype}: rows against the whole prompt: mean {float(errs.mean()):.3g}, worst {float(errs.max()):.3g}")
        if dtype == "float32":
            assert float(errs.max()) < F32_ROW
        else:
            assert float(errs.mean()) < BF16_CUT_MEAN and float(errs.max()) < BF16_CUT
    assert all(g["pages_reused"] > 0 for g in cache["page_groups"])


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_stream_after_every_layer_agrees_with_the_plain_model(models, name):
    """float32, a prompt in two portions: the residual stream after each layer (what the runner's observer sees
    once nothing is pending) equals the plain model's, so that a layer's fault is not hidden by the ones behind it;
    and every layer moves the stream."""
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    folder, cfg, w = models[name]
    toks = random_tokens(cfg["vocab"], 70, 3)
    _, after = P.forward(cfg, w, toks, return_layers=True)
    model_ = load_model(folder, dtype="float32")
    cache = CacheManager(model_.cache_needs, CacheConfig(num_pages=8, page_size=16, max_requests=2, dtype=model_.rt.dtype))
    runner = ModelRunner(model_, cache, use_graphs=False)
    seen = {}

    def observer(i, x, pending):
        if pending is None:
            seen.setdefault(i, []).append(x.detach().double().cpu())

    runner.observer = observer
    cache.open("a")
    runner.step([StepEntry("a", toks[:41], [])])
    runner.step([StepEntry("a", toks[41:], [])])
    runner.check_status()
    prev = w["embed"][torch.as_tensor(toks)]
    for i in range(len(cfg["layers"])):
        got = torch.cat(seen[i])
        err = float((got - after[i]).abs().max())
        assert err < 2e-5 * float(after[i].abs().max()), f"layer {i} ({cfg['layers'][i]['type']}): {err:.3g}"
        assert float((after[i] - prev).pow(2).mean().sqrt()) > 0.05
        prev = after[i]
    del runner, model_


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_tokens_stay_in_the_state_and_in_the_cache(tmp_path, dtype):
    """A request of 700 tokens: decoded tokens and short portions far into it read latent rows back to the first
    (keys split over several CTAs, merged with the sink counted once) and a state that has seen every token."""
    from mini_hisparse_b200 import write_random_model

    cfg = model(120, 128, [layer("gla", decay_mixer("gla", 2, 32, 48, tau=32.0, rank=8), dense(192)),
                           layer("latent_attention", latent(4, 32, 16, 32, 48, scale=0.2)),
                           layer("hgrn2", decay_mixer("hgrn2", 2, 16, 64), routed(4, 1, 2, 48, shared=64)),
                           layer("latent_attention", latent(8, 16, 16, 24, 48, scale=0.3, kv_from=1), dense(128))], side=8, cap=20.0)
    write_random_model(cfg, 41, tmp_path, dtype=torch.bfloat16, matrix_std=0.15)
    cfg, w = P.load_folder(tmp_path)
    reqs = requests_for(cfg, [700], seed=70)
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    whole = None
    for steps in (S.whole(reqs), S.tail_one_by_one(reqs, tail=40), S.changing_portions(reqs, sizes=(530, 2, 7, 64, 3, 2))):
        got, stats, pages = run_steps(tmp_path, dtype, steps)
        check_against_plain(got, refs, dtype)
        whole = whole or got
        errs = row_errors(got["r0"], whole["r0"])
        assert float(errs.max()) < (F32_ROW if dtype == "float32" else BF16_CUT)
    # the far past matters to the plain model: another first token moves the last logits
    other = list(reqs["r0"])
    other[0] = (other[0] + 1) % cfg["vocab"]
    moved = row_errors(P.forward(cfg, w, other)[-1:].float(), refs["r0"][-1:])
    assert float(moved) > SENSITIVE


def test_the_plain_model_is_sensitive_to_what_the_tests_are_for(models):
    """A sink left out, a decay's temperature or lower bound ignored, a group rule dropped, the correction used in
    the weights, identity experts that return nothing, a shared latent taken from the wrong layer, the gate on the
    residual or the token input left out, pairs rotated in the other layout: each moves the plain model's logits
    by far more than the float32 tolerance, so the comparisons above would show them."""
    folder, cfg, w = models["A"]
    toks = random_tokens(cfg["vocab"], 90, 5)
    right = P.forward(cfg, w, toks)
    rms = float(right.pow(2).mean().sqrt())

    def moved(cfg2=None, w2=None):
        return float((P.forward(cfg2 or cfg, w2 or w, toks) - right).pow(2).mean().sqrt()) / rms

    def with_(**changes):
        w2 = dict(w)
        w2.update(changes)
        return w2

    changes_cfg = (lambda c: c["layers"][2]["mixer"].update(tau=4.0),
                   lambda c: c["layers"][1]["mlp"]["router"].pop("groups"),
                   lambda c: c["layers"][1]["mlp"]["router"].update(top=2),
                   lambda c: c["layers"][1]["mixer"]["rot"].update(base=100.0),
                   lambda c: c["layers"][1]["mixer"].update(scale=0.31),
                   lambda c: c.pop("logit_softcap"),
                   lambda c: c.pop("token_side"))
    for change in changes_cfg:
        c = copy.deepcopy(cfg)
        change(c)
        assert moved(c) > SENSITIVE
    changes_w = (with_(**{"l1.mix.sink": w["l1.mix.sink"] - 30.0}),                       # no sink to speak of
                 with_(**{"l3.mix.sink": w["l3.mix.sink"] - 30.0}),
                 with_(**{"l0.mix.lower": torch.zeros_like(w["l0.mix.lower"])}),
                 with_(**{"l1.mlp.correction": torch.zeros_like(w["l1.mlp.correction"])}),
                 with_(**{"l0.rg1.b": w["l0.rg1.b"] + 30.0, "l0.rg1": torch.zeros_like(w["l0.rg1"])}),       # gate wide open
                 with_(**{"l2.mix.norm": torch.ones_like(w["l2.mix.norm"])}),
                 with_(**{"l0.mlp.act": w["l0.mlp.act"][[1, 0, 2, 3]]}),
                 with_(**{"l3.mlp.shared.sg": torch.zeros_like(w["l3.mlp.shared.sg"])}))
    for w2 in changes_w:
        assert moved(w2=w2) > SENSITIVE


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_a_slot_used_again(models, dtype):
    """A short prompt, then 260 tokens one by one (many pages long; the float32 state goes through 260 updates), two
    requests side by side; then their slots, which still hold their states, and their pages serve new requests."""
    folder, cfg, w = models["A"]
    reqs = requests_for(cfg, [270, 265], seed=40)
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    steps = S.tail_one_by_one(reqs, tail=260, together=2)
    again = requests_for(cfg, [50, 31], seed=60)
    again = {f"again_{k}": v for k, v in again.items()}
    refs.update({rid: P.forward(cfg, w, toks).float() for rid, toks in again.items()})
    steps += S.changing_portions(again, sizes=(2, 29, 1, 7))
    got, runner, cache = run_steps(folder, dtype, steps, max_requests=2)
    check_against_plain(got, refs, dtype)
    assert runner["graph_steps"] > 200


@pytest.mark.parametrize("name", ["A", "C"])
def test_batches_of_unequal_requests_equal_each_alone(models, name):
    """float32: a request's logits in a mixed batch equal those it gets alone, to rounding."""
    folder, cfg, w = models[name]
    reqs = requests_for(cfg, [140, 3, 77, 30], seed=9)
    alone, _, _ = run_steps(folder, "float32", S.whole(reqs), page_size=16)
    mixed, _, _ = run_steps(folder, "float32", S.mixed(reqs, seed=11, tail=20), page_size=16)
    for rid in reqs:
        assert row_rms_error(mixed[rid], alone[rid]) < F32_ROW


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(models, dtype):
    """Engine.add_request / run: admission, portions under a token budget, decoding, finishing.  float32 tokens
    equal the plain model's; in bfloat16 every token is the plain model's choice for the engine's own history,
    or loses to it by less than rounding."""
    from mini_hisparse_b200 import Engine, load_model

    folder, cfg, w = models["A"]
    model_ = load_model(folder, dtype=dtype)
    engine = Engine(model_, num_pages=40, page_size=16, max_requests=3, max_tokens_per_step=48, graph_after=2)
    prompts = requests_for(cfg, [70, 9, 33], seed=80)
    for rid, p in prompts.items():
        engine.add_request(rid, p, max_new_tokens=12)
    out = engine.run()
    engine.cache.assert_invariants()
    for rid, p in prompts.items():
        assert len(out[rid]) == 12
        if dtype == "float32":
            assert out[rid] == P.generate(cfg, w, p, 12)
        else:
            seq = list(p)
            for tok in out[rid]:
                logits = P.forward(cfg, w, seq)[-1]
                assert float(logits.max() - logits[tok]) < 0.05 * float(logits.abs().max())
                seq.append(tok)


def test_command_line_demo_with_a_tudasun_config(capsys):
    """`demo --config configs/tudasun-demo.json`: random weights, three requests through Engine and scheduler."""
    from pathlib import Path

    import mini_hisparse_b200
    from mini_hisparse_b200 import cli

    config = Path(mini_hisparse_b200.__file__).parent / "configs" / "tudasun-demo.json"
    assert cli.main(["demo", "--config", str(config), "--dtype", "bfloat16", "--requests", "3", "--prompt-tokens", "70",
                     "--max-new-tokens", "6"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert [r["generated_tokens"] for r in report["requests"].values()] == [6, 6, 6]


def test_trace_run_picks_the_model_by_its_config(models, tmp_path):
    """bin/trace_run on a Tudasun folder: the same program, cache and step function as for every model."""
    folder, cfg, w = models["B"]
    reqs = requests_for(cfg, [60, 21], seed=90)
    refs = {rid: P.forward(cfg, w, toks).float() for rid, toks in reqs.items()}
    steps = S.mixed(reqs, seed=1, tail=10)
    run = TraceRun(folder, "float32", tmp_path / "out", S.peak_tokens(steps), page_size=16, extra=("--poison",))
    got = {}
    for entries, end in steps:
        logits = run.step(entries, end)
        row = 0
        for e in entries:
            got.setdefault(e["id"], []).append(logits[row: row + len(e["want"])])
            row += len(e["want"])
    assert run.close() == 0
    check_against_plain({k: torch.cat(v) for k, v in got.items()}, refs, "float32")
