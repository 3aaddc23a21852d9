"""Livovik on the GPU against the plain implementation (tests/plain_livovik.py): each mechanism alone, then
whole models through the step function, the scheduler and the trace program; prompts whole, in portions down
to two tokens, decoded token by token, and in mixed batches with pages and slots used again. Inputs are made
so that a fault shows where random ones would hide it: the input at one position is scaled up so that its key
wins every score it takes part in (a block edge that is one off, a far key that is lost, the first tokens),
and sinks are large enough to take a visible share of every softmax."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import livovik_tiny as L
import plain_livovik as P
import replay
from test_gpu_zukotar import SCHEDULES, Harness, bind, check, cut, rel, rnd

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def as_stored(weights, dtype):
    return {k: (v.to(DT[dtype]) if v.is_floating_point() else v).to(P.F64) for k, v in weights.items()}


# ------------------------------------------------------------------ small kernels

@pytest.mark.parametrize("H", [40, 96, 100, 1024, 2500])
def test_postnorm_adds_parts_and_a_gated_summand_in_float(H):
    from rllm_b200.kernels import sink
    T = 9
    h, y, y2, zg, w = rnd(T, H, seed=1), rnd(T, 3, H, seed=2), rnd(T, H, seed=3), rnd(T, 1, seed=4), rnd(H, seed=5) + 1
    s = 1.75 * h.double() + y.double().sum(1) + torch.sigmoid(zg.double()) * y2.double()
    want = P.rms_norm(s, w.double(), 1e-5)
    hd = h.to(DEV)
    copy = torch.empty((T, H), dtype=torch.bfloat16, device=DEV)
    sink.postnorm(hd, y.to(DEV), 1.75, w.to(DEV), 1e-5, y2.to(DEV), zg.to(DEV), copy)
    assert rel(hd, want) < 2e-6 and torch.equal(copy, hd.bfloat16())
    # one part, nothing else; and no sublayer output at all
    hd = h.to(DEV)
    sink.postnorm(hd, y[:, 0].contiguous().to(DEV), 1.0, w.to(DEV), 1e-5)
    assert rel(hd, P.rms_norm(h.double() + y[:, 0].double(), w.double(), 1e-5)) < 2e-6
    assert torch.equal(sink.cast_rows(hd), hd.bfloat16())


@pytest.mark.parametrize("dtype", list(DT))
def test_activations(dtype):
    from rllm_b200.kernels import sink
    gu, f = rnd(37, 2 * 24, seed=1, scale=2.0), rnd(37, seed=2).abs() + 0.1
    g, u = f[:, None].double() * gu[:, :24].double(), f[:, None].double() * gu[:, 24:].double()
    want = g * torch.sigmoid(g) * u
    got = sink.gated_act(gu.to(DEV), DT[dtype], f.to(DEV))
    assert got.dtype == DT[dtype] and rel(got, want) < (2e-6 if dtype == "float32" else 8e-3)
    if dtype == "bfloat16":
        gb = gu.bfloat16()
        want = gb[:, :24].double() * torch.sigmoid(gb[:, :24].double()) * gb[:, 24:].double()
        assert rel(sink.gated_act(gb.to(DEV), torch.bfloat16), want) < 8e-3
    x = rnd(50, 33, seed=3).to(DT[dtype])
    assert rel(sink.relu2_(x.to(DEV).clone()), torch.relu(x.double()) ** 2) < (1e-6 if dtype == "float32" else 8e-3)
    from rllm_b200.kernels import ops
    w = rnd(21, 33, seed=4).to(DT[dtype])            # the CUDA-core product squares in float and rounds once
    got = ops.gemm_simt(x.to(DEV), w.to(DEV), ops.EPI_RELU2)
    assert got.dtype == DT[dtype] and rel(got, torch.relu(x.double() @ w.double().T) ** 2) < (2e-6 if dtype == "float32" else 6e-3)


@pytest.mark.parametrize("E,top", [(8, 1), (6, 2), (7, 3), (64, 8), (4, 4)])
def test_router_scores_by_sigmoid(E, top):
    from rllm_b200.kernels import mix
    z = rnd(41, E, seed=E + top, scale=2.0)
    idx, wt = P.route(z.double(), torch.eye(E, dtype=P.F64), top)
    gi, gw = mix.moe_topk(z.to(DEV), top, score="sigmoid")
    assert torch.equal(gi.cpu().long(), idx) and rel(gw, wt) < 1e-6
    if top > 1:
        assert float(gw.sum(1).max()) > 1.0          # scores by themselves: not a distribution over the experts


# ------------------------------------------------------------------ the mixer alone, over steps

def mixer_weights(W, m, seed):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    shapes = {"q": (H * D, W), "k": (G * D, W), "v": (G * V, W), "q.norm": (D,), "k.norm": (D,), "sink": (H,), "g": (H, W),
              "o": (W, H * V)}
    w = {"x." + k: rnd(*s, seed=seed + i, scale=0.25) for i, (k, s) in enumerate(shapes.items())}
    w["x.q.norm"], w["x.k.norm"] = w["x.q.norm"] + 1, w["x.k.norm"] + 1
    w["x.sink"] = w["x.sink"] * 8          # a sink that is left out, scaled or counted twice moves every row
    return w


def make_mixer(W, m, eps=1e-6):
    from rllm_b200.config.livovik import SinkAttentionConfig
    from rllm_b200.parts import RotaryEmbedding, SinkGQAttention
    c = SinkAttentionConfig.from_dict(m, "mixer")
    rope = RotaryEmbedding(c.dim, c.rot_base, c.rot_scaling, rot_dim=c.rot_dims) if c.rot_dims else None
    return SinkGQAttention(W, c.heads, c.kv_heads, c.dim, c.vdim, position=rope, scale=c.scale, chunk=c.chunk, qk_norm=True,
                           sink=True, gate=True, eps=eps)


MIXERS = [
    (L.attn(4, 2, 32, 16, 0.2, L.rot(10000.0, 16, (8.0, 1.0, 4.0, 64)), 21), 4),     # blocks over several pages, half rotated
    (L.attn(4, 4, 16, 32, 0.3, L.rot(500.0, 16), 16), 16),                            # block = page, as many kv heads as heads
    (L.attn(6, 1, 24, 40, 0.17, L.rot(1e6, 8), 3), 8),                                # blocks shorter than a page, one kv head
    (L.attn(2, 2, 48, 48, 0.125, None, None), 8),                                     # no rotation, no mask
    (L.attn(3, 1, 20, 12, 0.25, L.rot(10000.0, 20, (4.0, 1.0, 2.0, 32)), 33), 16),    # nothing a multiple of 8
    (L.attn(16, 1, 64, 32, 0.11, L.rot(300000.0, 32, (6.0, 1.0, 3.0, 128)), 64), 16),  # a token's heads fill a row tile
    (L.attn(2, 2, 128, 128, 0.09, L.rot(10000.0, 128), 50), 16),                      # the largest head size
    (L.attn(8, 4, 16, 16, 0.25, L.rot(10000.0, 8), 1), 4),                            # a block of one position: the query alone
]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("m,page", MIXERS)
def test_attention_mixer_over_steps(dtype, m, page):
    """Inputs at the first positions, at page borders, far back and just inside and just outside the blocks of
    queries 70 and 96 are scaled up: their keys then win the scores of the queries that see them."""
    W, n = 40, 97
    w = mixer_weights(W, m, seed=m["heads"])
    h = rnd(n, W, seed=9)
    size = (m.get("mask") or {"size": 30})["size"]
    special = {0, 1, page - 1, page, 2 * page + 1, 50}
    for qpos in (96, 70):
        start = qpos // size * size
        special |= {max(0, start - 1), start, min(qpos, start + 1)}
    for p in special:
        h[p] *= 6.0
    want = P.attention_mixer(h.to(DT[dtype]).double(), as_stored({k[2:]: v for k, v in w.items()}, dtype), m, 1e-6)
    part = make_mixer(W, m)
    bind(part, w, dtype, "x.")
    hd = h.to(DT[dtype]).to(DEV)
    tol = 2e-5 if dtype == "float32" else 4e-2
    outs = {}
    for name, sched in SCHEDULES.items():
        hs = Harness(dtype, [part.cache_spec()], page_size=page, pages=2 + (n + page - 1) // page)
        got, i = [], 0
        for q in cut(n, sched(n)):
            got.append(hs.run([("a", q)], lambda ctx, cache: part.forward(hd[i: i + q], ctx, cache)))
            i += q
            hs.cache.check()
        outs[name] = torch.cat(got)
        assert outs[name].dtype == torch.float32 and rel(outs[name], want) < tol, name
    if dtype == "float32":       # the same bits however the tokens were cut
        assert all(torch.equal(outs["whole"], o) for o in outs.values())
    # two requests in one step, unequal portions beside single tokens; then a third on pages that were used
    hb = rnd(47, W, seed=10)
    hb[3] *= 6.0
    want_b = P.attention_mixer(hb.to(DT[dtype]).double(), as_stored({k[2:]: v for k, v in w.items()}, dtype), m, 1e-6)
    hbd = hb.to(DT[dtype]).to(DEV)
    hs = Harness(dtype, [part.cache_spec()], page_size=page, pages=4 + (n + 47 + 2 * page - 1) // page)
    got_a, got_b, ia, ib = [], [], 0, 0
    for qa, qb in ((30, 5), (1, 40), (66, 2)):
        y = hs.run([("a", qa), ("b", qb)], lambda ctx, cache: part.forward(
            torch.cat([hd[ia: ia + qa], hbd[ib: ib + qb]]), ctx, cache))
        got_a.append(y[:qa]); got_b.append(y[qa:])
        ia += qa; ib += qb
        hs.cache.check()
    assert rel(torch.cat(got_a), want) < tol and rel(torch.cat(got_b), want_b) < tol
    hs.engine.end(["a", "b"])
    again = hs.run([("c", 47)], lambda ctx, cache: part.forward(hbd, ctx, cache))
    assert rel(again, want_b) < tol


def test_pages_before_the_current_block_go_back_to_the_pool():
    """A request of 100 positions under a block rule of 21 positions and pages of 4 holds, after every step,
    only the pages from its current block on; a second layer group without the rule keeps all of its pages."""
    from rllm_b200.cache import CacheManager
    from rllm_b200.parts import KVCacheSpec
    specs = [KVCacheSpec(1, 16, None, 21, 8), KVCacheSpec(2, 16)]
    cm = CacheManager(specs, 4, 40, 2, torch.float32, DEV)
    assert cm.groups[0].tensors[0]["v"].shape[-1] == 8 and cm.groups[0].tensors[0]["k"].shape[-1] == 16
    rc = cm.open("a")
    total = 0
    for q in (5, 17, 1, 1, 30, 2, 44):
        cm.reserve(rc, total + q)
        total += q
        cm.commit(rc, total)
        cm.check()
        first = (total // 21 * 21) // 4
        pages = rc.pages_array(0)
        assert (pages[:first] == -1).all() and (pages[first:] >= 0).all()
        assert (rc.pages_array(1) >= 0).all()
    cm.close("a")
    cm.check()
    assert cm.free_pages() == [40, 40]


@pytest.mark.parametrize("chunk,window", [(None, None), (200, None), (None, 77), (64, 40), (1000, None)])
def test_decoding_deals_the_keys_out_to_several_ctas(chunk, window):
    """Long contexts, one query token per request: the keys of a request are cut into ranges for several CTAs
    and merged; one far key is made to win so that a lost range shows. Against the float kernel on the same cache."""
    from rllm_b200.kernels import sink
    g = torch.Generator().manual_seed(5)
    nh, nkv, kd, vd, page, n_pages = 8, 2, 64, 48, 16, 140
    lens = [1500, 333, 2048, 1]
    S = len(lens)
    kc = (torch.randn(n_pages * S, nkv, page, kd, generator=g) * 0.5).bfloat16().to(DEV)
    vc = torch.randn(n_pages * S, nkv, page, vd, generator=g).bfloat16().to(DEV)
    q = torch.randn(S, nh * kd, generator=g).bfloat16().to(DEV)
    bt = torch.arange(n_pages * S, dtype=torch.int32).view(S, n_pages).flip(0).contiguous().to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(S, dtype=torch.int32, device=DEV)
    cu = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    far = 1500 - 1 - (30 if window or (chunk and chunk < 1500) else 1400)
    kc[bt[0, far // page].item(), :, far % page] = q[0].view(nh, kd)[::4] * 2     # key `far` of request 0 wins
    sinks = torch.randn(nh, generator=g).to(DEV)
    gate = torch.randn(S, nh, generator=g).to(DEV)
    want = sink.sink_attention_simt(q, kc, vc, seq, pos, bt, nh, 0.125, window, chunk, sinks, gate)
    for splits in (1, 3, 16):
        got = sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, S, 1, nh, 0.125, window, chunk, sinks, gate, splits, 2048)
        assert rel(got, want) < 2e-2, splits


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("chunk,window", [(None, None), (200, None), (1024, 300), (64, None)])
def test_the_kernels_of_plain_attention_take_mask_sink_and_gate(hd, chunk, window):
    """Equal key and value sizes of 64 or 128: the cluster kernel for single tokens and the tcgen05 kernel for long
    portions, with a block mask, a sink and a gate, against the float kernel on the same cache. Keys just inside
    and just outside the last query's block are made to win."""
    from rllm_b200.kernels import sink, sm100
    g = torch.Generator().manual_seed(hd)
    nh, nkv, page, n_pages = 8, 2, 16, 100
    lens, qlens = [1500, 700, 1024], [600, 700, 130]
    S = len(lens)
    kc = (torch.randn(n_pages * S, nkv, page, hd, generator=g) * 0.5).bfloat16().to(DEV)
    vc = torch.randn(n_pages * S, nkv, page, hd, generator=g).bfloat16().to(DEV)
    bt = torch.arange(n_pages * S, dtype=torch.int32).view(S, n_pages).flip(0).contiguous().to(DEV)
    sinks = (torch.randn(nh, generator=g) * 3).to(DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    # single tokens
    q = torch.randn(S, nh * hd, generator=g).bfloat16().to(DEV)
    start = 1499 // chunk * chunk if chunk else 0
    for far in (max(start - 1, 0), start, 1499 - 250):
        kc[bt[0, far // page].item(), :, far % page] = q[0].view(nh, hd)[::4] * 2
    pos = kv - 1
    seq = torch.arange(S, dtype=torch.int32, device=DEV)
    gate = torch.randn(S, nh, generator=g).to(DEV)
    want = sink.sink_attention_simt(q, kc, vc, seq, pos, bt, nh, 0.11, window, chunk, sinks, gate)
    for splits in (1, 4, 8):
        got = sm100.attention_decode(q, kc, vc, kv, bt, nh, 0.11, window, 1500, splits=splits, chunk=chunk, sinks=sinks, gate=gate)
        assert rel(got, want) < 2e-2, splits
    # long portions
    T = sum(qlens)
    q = torch.randn(T, nh * hd, generator=g).bfloat16().to(DEV)
    cu = torch.tensor([0, 600, 1300, 1430], dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(n - ql, n) for n, ql in zip(lens, qlens)]).int().to(DEV)
    seq = torch.cat([torch.full((ql,), i) for i, ql in enumerate(qlens)]).int().to(DEV)
    gate = torch.randn(T, nh, generator=g).to(DEV)
    want = sink.sink_attention_simt(q, kc, vc, seq, pos, bt, nh, 0.11, window, chunk, sinks, gate)
    got = sm100.attention_prefill_tc(q, kc, vc, cu, kv, bt, max(qlens), nh, 0.11, window, chunk=chunk, sinks=sinks, gate=gate)
    assert rel(got, want) < 2e-2
    got = sink.sink_attention_mma(q, kc, vc, seq, pos, bt, cu, S, max(qlens), nh, 0.11, window, chunk, sinks, gate)
    assert rel(got, want) < 2e-2


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("N,K", [(1, 40), (6, 256), (8, 1000), (3, 7)])
def test_product_with_a_few_weight_rows(dtype, N, K):
    from rllm_b200.kernels import ops
    x, w = rnd(21, K, seed=1).to(DT[dtype]), rnd(N, K, seed=2).to(DT[dtype])
    got = ops.gemm_skinny(x.to(DEV), w.to(DEV))
    assert got.dtype == torch.float32 and rel(got, x.double() @ w.double().T) < 3e-6


@pytest.mark.parametrize("T", [1, 8, 9, 40, 64, 130, 300, 2048])
@pytest.mark.parametrize("N,K", [(512, 256), (1536, 512)])
def test_relu_squared_in_the_store_epilogue_of_the_products(T, N, K):
    """Every kernel a step's size selects (weight streaming up to 8 tokens, tcgen05 small tiles with ranges of K
    merged in a cluster, the persistent kernel) stores max(., 0)^2 of the float result."""
    from rllm_b200.kernels import ops, sm100
    x, w = rnd(T, K, seed=T).bfloat16(), rnd(N, K, seed=N, scale=0.1).bfloat16()
    want = torch.relu(x.double() @ w.double().T) ** 2
    got = sm100.gemm(x.to(DEV), w.to(DEV), ops.EPI_STORE, relu2=True)
    assert got.dtype == torch.bfloat16 and rel(got, want) < 1e-2
    plain = sm100.gemm(x.to(DEV), w.to(DEV), ops.EPI_STORE)          # the switch leaves nothing behind
    assert rel(plain, x.double() @ w.double().T) < 1e-2 and float(plain.min()) < 0
    sm100.check_error(DEV)


def test_long_row_lists_of_gated_experts_run_on_tcgen05():
    """1,400 (token, expert) rows: the grouped products take the tcgen05 kernel, the gate/up product activates in
    its epilogue on weights kept in blocks of 16 + 16 rows. Against the plain implementation."""
    from rllm_b200.parts import GatedRoutedExperts
    W, F, E, top, T = 64, 64, 5, 2, 700
    w = {"router": rnd(E, W, seed=1, scale=0.5)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rnd(F, W, seed=10 + e, scale=0.3), rnd(F, W, seed=40 + e, scale=0.3), rnd(W, F, seed=70 + e, scale=0.3)
    ffn = GatedRoutedExperts(W, F, E, top, score="sigmoid")
    ffn.set_prefix("x.mlp.")
    bind_tree(ffn, {"x.mlp." + k: v for k, v in w.items()}, "bfloat16")
    x = rnd(T, W, seed=2).bfloat16()
    want = P.moe_ffn(x.double(), as_stored(w, "bfloat16"), {"router": {"experts": E, "top": top}})

    class Ctx:
        backend = Harness("bfloat16", []).backend
    seen = []
    be = Ctx.backend
    orig = be._mix.grouped_gemm_tc
    be._mix.grouped_gemm_tc = lambda *a, **k: (seen.append(a[4]), orig(*a, **k))[1]
    try:
        out = ffn.forward(x.to(DEV), Ctx)
    finally:
        be._mix.grouped_gemm_tc = orig
    assert seen == [be._mix.GEPI_SILU_GATED, be._mix.GEPI_STORE_F32]
    assert rel(out.parts.sum(1), want) < 2e-2


# ------------------------------------------------------------------ feed-forwards in a post-norm block

@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("top,shared", [(1, 24), (3, None), (2, 16)])
def test_feed_forwards_in_a_post_norm_block(dtype, top, shared):
    from rllm_b200.parts import ActFFN, GatedRoutedExperts, SwiGLU
    W, F, E, T = 40, 24, 6, 45
    w = {"router": rnd(E, W, seed=1, scale=0.5), "shared.sg": rnd(1, W, seed=3, scale=0.5)}
    for i, e in enumerate([f"e{e}." for e in range(E)] + ["shared."]):
        n = shared if e == "shared." else F
        if n:
            w[e + "gate"], w[e + "up"], w[e + "down"] = (rnd(n, W, seed=10 + i, scale=0.3), rnd(n, W, seed=40 + i, scale=0.3),
                                                         rnd(W, n, seed=70 + i, scale=0.3))
    if not shared:
        del w["shared.sg"]
    ffn = GatedRoutedExperts(W, F, E, top, score="sigmoid", shared=SwiGLU(W, shared, names=("gate", "up", "down")) if shared else None,
                             shared_gate=True)
    ffn.set_prefix("x.mlp.")
    bind_tree(ffn, {"x.mlp." + k: v for k, v in w.items()}, dtype)
    x = rnd(T, W, seed=2).to(DT[dtype])
    mlp = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    want = P.moe_ffn(x.double(), as_stored(w, dtype), mlp)

    class Ctx:
        backend = Harness(dtype, []).backend
    out = ffn.forward(x.to(DEV), Ctx)
    assert out.parts.shape == (T, top, W) and out.parts.dtype == torch.float32
    got = out.parts.sum(1)
    if shared:
        got = got + torch.sigmoid(out.extra_gate[:, :1]) * out.extra
    assert rel(got, want) < (3e-6 if dtype == "float32" else 2e-2)
    # the block's kernel adds the same summands
    h = rnd(T, W, seed=5)
    hd = h.to(DEV)
    wn = rnd(W, seed=6) + 1
    xn = Ctx.backend.postnorm(hd, out, 2.0, wn.to(DEV), 1e-6)
    assert rel(hd, P.rms_norm(2.0 * h.double() + want, wn.double(), 1e-6)) < (3e-6 if dtype == "float32" else 2e-2)
    assert xn.dtype == DT[dtype] and torch.equal(xn.float(), hd.to(DT[dtype]).float())
    # the dense one
    wd = {"x.up": rnd(56, W, seed=7, scale=0.3), "x.down": rnd(W, 56, seed=8, scale=0.3)}
    dense = ActFFN(W, 56, "relu2")
    bind(dense, wd, dtype, "x.")
    got = dense.forward(x.to(DEV), Ctx, None)
    assert got.dtype == torch.float32
    assert rel(got, P.dense_ffn(x.double(), as_stored({k[2:]: v for k, v in wd.items()}, dtype))) < (3e-6 if dtype == "float32" else 2e-2)


def bind_tree(part, weights, dtype):
    """Like `bind`, for a part whose children have prefixes of their own."""
    from rllm_b200.weights.loader import storage_dtype
    for p_ in part.walk():
        for p in p_.params():
            t = torch.cat([weights[p_.prefix + s.name] for s in p.sources], 0)
            setattr(p_, p.attr, t.to(storage_dtype(p.role, torch.bfloat16, DT[dtype])).to(DEV).contiguous())
    for p_ in part.walk():
        p_.finalize(torch.device(DEV), DT[dtype])


# ------------------------------------------------------------------ whole models

def requests_for(name, lens=(9, 61, 23, 150, 37, 2)):
    vocab = L.TINY[name][0]["vocab"]
    return {f"r{i}": L.random_prompt(n, vocab, 100 * len(name) + i) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("livovik")
    return {n: L.make_model_dir(root, n) for n in L.TINY}


@pytest.fixture(scope="module")
def plain(dirs):
    out = {}
    for name, d in dirs.items():
        cfg, w = P.read_model_dir(d)
        out[name] = {}
        for rid, toks in requests_for(name).items():
            lg = P.forward(cfg, w, toks).numpy()
            out[name].update({(rid, i): lg[i] for i in range(len(toks))})
    return out


FAMILIES = {"whole": replay.whole, "decode": lambda r: replay.prefill_then_decode(r, tail=40), "portions": replay.portions,
            "mixed": lambda r: replay.mixed(r, max_live=3)}


@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(L.TINY))
def test_family_matches_plain(dirs, plain, name, dtype, family):
    """The pool holds just what the live requests need and there are three slots for six requests: pages and
    slots are used again."""
    from rllm_b200.engine import load_engine
    reqs = requests_for(name)
    steps = FAMILIES[family](reqs)
    eng = load_engine(dirs[name], dtype=dtype, page_size=L.TINY[name][4],
                      max_tokens=replay.max_live_tokens(steps, reqs), max_requests=3)
    got = replay.run_in_process(eng, steps)
    eng.check()
    if dtype == "float32":
        check(got, plain[name], 3e-5, f"{name} float32 {family}")
    else:
        check(got, plain[name], 6e-2, f"{name} bfloat16 {family}", allow=0.25)


@pytest.mark.parametrize("name", list(L.TINY))
def test_float32_is_the_same_however_it_is_cut(dirs, name):
    from rllm_b200.engine import load_engine
    reqs = requests_for(name)
    ref = None
    for family, make in FAMILIES.items():
        steps = make(reqs)
        eng = load_engine(dirs[name], dtype="float32", page_size=L.TINY[name][4],
                          max_tokens=replay.max_live_tokens(steps, reqs), max_requests=3)
        got = replay.run_in_process(eng, steps)
        if ref is None:
            ref = got
        else:
            worst = max(float(np.abs(got[k] - ref[k]).max()) for k in ref)
            assert worst <= 2e-6, f"{name} {family}: differs from whole prompts by {worst}"


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 6e-2)])
def test_long_decoding_through_graphs(dirs, dtype, tol):
    """Two requests decoded side by side for 120 steps from prompts of 3 and 30 tokens: blocks begin and end among
    decoded tokens, pages are given back on the way, every step replays a graph."""
    from rllm_b200.engine import Entry, load_engine
    name = "LA"
    cfg, w = P.read_model_dir(dirs[name])
    toks = {"x": L.random_prompt(123, 160, 5), "y": L.random_prompt(150, 160, 6)}
    want = {k: P.forward(cfg, w, t).numpy() for k, t in toks.items()}
    eng = load_engine(dirs[name], dtype=dtype, page_size=4, max_tokens=320, max_requests=2)
    eng.step([Entry("x", toks["x"][:3], []), Entry("y", toks["y"][:30], [])])
    got = {}
    for i in range(120):
        lg = eng.step([Entry("x", [toks["x"][3 + i]], [0]), Entry("y", [toks["y"][30 + i]], [0])]).float().cpu().numpy()
        got[("x", 3 + i)], got[("y", 30 + i)] = lg[0], lg[1]
        eng.cache.check()
    eng.check()
    assert eng.graphs is not None and eng.graph_steps == 120
    held = eng.cache.held_pages(eng.cache.live["x"])
    assert held[0] < 123 // 4          # the pages of the blocks that have passed went back to the pool
    check(got, {(k, i): want[k][i] for (k, i) in got}, tol, f"long decoding {dtype}", allow=0.0 if dtype == "float32" else 0.25)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 6e-2)])
def test_long_portions_over_pages_that_went_back(dirs, plain_long, dtype, tol):
    """A prompt of 700 tokens in portions of 150: from the fourth portion on the layer with equal head sizes of
    128 runs its long portions on the tcgen05 kernel over a block table whose pages before the current block of
    100 positions have gone back to the pool; then 20 single tokens through graphs on the cluster kernel."""
    from rllm_b200.engine import Entry, load_engine
    from rllm_b200.kernels import sm100
    toks, want = plain_long
    eng = load_engine(dirs["LD"], dtype=dtype, page_size=16, max_tokens=768, max_requests=2)
    got, at, calls = {}, 0, []
    orig = sm100.attention_prefill_tc
    sm100.attention_prefill_tc = lambda *a, **k: (calls.append(k.get("chunk")), orig(*a, **k))[1]
    try:
        for n in (150, 150, 150, 150, 80):
            lg = eng.step([Entry("x", toks[at: at + n], list(range(n)))]).float().cpu().numpy()
            got.update({("x", at + i): lg[i] for i in range(n)})
            at += n
            eng.cache.check()
    finally:
        sm100.attention_prefill_tc = orig
    assert calls == ([100] if dtype == "bfloat16" else [])        # the fourth portion: 150 rows over 600 keys
    for i in range(20):
        got[("x", at)] = eng.step([Entry("x", [toks[at]], [0])]).float().cpu().numpy()[0]
        at += 1
    eng.check()
    assert at == len(toks) and eng.graph_steps == 20
    assert min(eng.cache.held_pages(eng.cache.live["x"])) <= (100 + 16) // 16 + 1
    check(got, {("x", i): want[i] for i in range(len(toks))}, tol, f"long portions {dtype}", allow=0.0 if dtype == "float32" else 0.25)


@pytest.fixture(scope="module")
def plain_long(dirs):
    cfg, w = P.read_model_dir(dirs["LD"])
    toks = L.random_prompt(700, cfg["vocab"], 77)
    return toks, P.forward(cfg, w, toks).numpy()


@pytest.mark.parametrize("name", ["LB", "LC"])
def test_greedy_generation_through_the_entry_point(dirs, name):
    """LLM.generate (scheduler, sampler, run-ahead decoding) against greedy decoding with the plain model."""
    from rllm_b200.api import LLM
    from rllm_b200.sampling import SamplingParams
    cfg, w = P.read_model_dir(dirs[name])
    prompts = [L.random_prompt(n, cfg["vocab"], 70 + n) for n in (4, 19, 33)]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(12):
            lg = P.forward(cfg, w, toks)[-1]
            top2 = lg.topk(2).values
            toks.append(int(lg.argmax()))
            if float(top2[0] - top2[1]) < 1e-4:      # a close call: the rest of this prompt proves nothing
                break
        want.append(toks[len(p):])
    llm = LLM(dirs[name], dtype="float32", page_size=L.TINY[name][4], num_pages=40, max_active=2, max_chunk=16)
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for g, w_ in zip(got, want):
        assert g[: len(w_)] == w_
    llm.engine.cache.check()


def test_ten_requests_decode_in_a_padded_graph(dirs):
    from rllm_b200.engine import Entry, load_engine
    name = "LC"
    cfg, w = P.read_model_dir(dirs[name])
    toks = {i: L.random_prompt(5 + 3 * i + 9, cfg["vocab"], 300 + i) for i in range(10)}
    want = {i: P.forward(cfg, w, t).numpy() for i, t in toks.items()}
    eng = load_engine(dirs[name], dtype="float32", page_size=16, max_tokens=10 * 64, max_requests=10)
    eng.step([Entry(i, t[:-9], []) for i, t in toks.items()])
    got = {}
    for k in range(9):
        lg = eng.step([Entry(i, [t[len(t) - 9 + k]], [0]) for i, t in toks.items()]).float().cpu().numpy()
        for row, (i, t) in enumerate(toks.items()):
            got[(i, len(t) - 9 + k)] = lg[row]
    eng.check()
    assert eng.graph_steps == 9
    check(got, {(i, p): want[i][p] for (i, p) in got}, 3e-5, "padded graph")


def test_command_line_runs_the_design(dirs):
    name = "LA"
    cfg, w = P.read_model_dir(dirs[name])
    prompt = L.random_prompt(11, cfg["vocab"], 3)
    toks = list(prompt)
    for _ in range(5):
        toks.append(int(P.forward(cfg, w, toks)[-1].argmax()))
    r = subprocess.run([sys.executable, os.path.join(replay.ROOT, "bin", "rllm"), "run", "--model", dirs[name],
                        "--prompt-ids", " ".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0",
                        "--dtype", "float32", "--kv-pages", "32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.split()] == toks[len(prompt):]


def test_trace_program_runs_the_design(dirs, plain, tmp_path):
    name = "LC"
    reqs = requests_for(name)
    steps = replay.mixed(reqs, max_live=4)
    got = replay.run_program(dirs[name], "float32", steps, str(tmp_path / "out"), replay.max_live_tokens(steps, reqs),
                             L.TINY[name][0]["vocab"], extra_args=["--page-size", "16"])
    check(got, plain[name], 3e-5, "trace program")
