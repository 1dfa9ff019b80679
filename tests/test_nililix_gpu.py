"""The Nililix design (windowed grouped-query attention with short convolutions, a softmax sink and output gates; squared
ReLU and routed-expert feed-forwards; sandwich norms; a looped block) on the GPU against the plain float64 oracle
(oracle/nililix_plain.py): every mechanism alone, prefill against token-by-token decoding, portions down to two tokens,
unequal batches against each request alone, pages and slots used again, keys far away, at page borders and just inside
and outside the window (in prompts and decoded), the first tokens of a sequence, long decoding, other sizes, and greedy
generation through the scheduler."""
import json
import math
import os

import pytest
import torch

from oracle import nililix_plain as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-4, torch.bfloat16: 4e-2}      # relative to the largest magnitude of the compared tensor


def _close(got, want, dtype, what, scale=1.0):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    err = (got - want).abs().max().item()
    ref = max(want.abs().max().item(), 1e-6)
    assert err <= TOL[dtype] * scale * ref, f"{what}: max error {err:.3e} against magnitude {ref:.3e}"


SC = (4.0, 1.0, 4.0, 64)          # frequency scaling that puts pairs of a small head in all three bands
A_ODD = dict(heads=6, kv_heads=2, dim=10, vdim=6, conv=3, window=7, rot_dims=6, rot_base=300.0, scaling=SC)
A_MQ = dict(heads=5, kv_heads=1, dim=8, vdim=40, conv=4, window=20, rot_dims=8, rot_base=1e4)          # group of 5 > 4 warps
A_MH = dict(heads=3, kv_heads=3, dim=16, vdim=16, conv=1, window=0, rot_dims=0, sink=False, gate=False)  # plain causal
A_TC = dict(heads=8, kv_heads=2, dim=32, vdim=16, conv=2, window=33, rot_dims=16, rot_base=5e5, scaling=(8.0, 1.0, 4.0, 128))
STACKS = {
    "odd": dict(layers=[dict(A_ODD, mlp=("dense", 50)), dict(A_MQ, mlp=("moe", 20, 6, 2, 3, 2)), dict(A_MH, mlp=None),
                        dict(A_ODD, window=1, mlp=("moe", 12, 4, 1, 1, 1))], width=40, vocab=61, loop=(1, 3, 3)),
    "tc": dict(layers=[dict(A_TC, mlp=("moe", 32, 8, 3, 4, 2)), dict(A_TC, window=64, mlp=("dense", 96)),
                       dict(A_TC, kv_heads=8, conv=5, mlp=("moe", 16, 5, 5, 1, 1))], width=64, vocab=130, loop=(0, 1, 2),
               residual_mult=1.3, logit_softcap=7.0),
    # the same attention layers without routing
    "tc-dense": dict(layers=[dict(A_TC, mlp=("dense", 96)), dict(A_TC, window=64, vdim=32, mlp=None),
                             dict(A_TC, kv_heads=8, conv=5, mlp=("dense", 40))], width=64, vocab=130, loop=(1, 3, 2), residual_mult=0.6),
    "plain": dict(layers=[dict(A_MH, mlp=("dense", 30)), dict(A_MQ, sink=False, mlp=None)], width=32, vocab=40, loop=None,
                  logit_softcap=None, residual_mult=1.0, eps=1e-6),
}

_ORACLE = {}


def _weights(name, dtype, seed):
    """Whole stacks run in bf16 get routers whose choice cannot hang on a score (``spaced_corrections``): with random
    corrections some token's choice scores lie within bf16 rounding of each other, another expert runs for it, and
    everything that attends to that token differs — which is no kernel's error.  The fp32 runs keep random corrections,
    so there the choice differs from token to token."""
    return O.random_nililix(seed=seed, spaced_corrections=dtype == torch.bfloat16, **STACKS[name])


def _oracle(name, dtype, seed, toks, layers=False):
    key = (name, dtype == torch.bfloat16, seed, tuple(toks))
    if key not in _ORACLE:
        cfg, t = _weights(name, dtype, seed)
        _ORACLE[key] = O.nililix_forward(cfg, t, toks, return_layers=True)
    return _ORACLE[key] if layers else _ORACLE[key][0]


def _model(name, dtype, seed=0):
    from trtllm_llama_b200.models.nililix import build_nililix
    cfg, t = _weights(name, dtype, seed)
    return cfg, t, build_nililix(cfg, t, dtype, "cuda")


def _session(model, max_tokens=512, max_seqs=4, page=64):
    from trtllm_llama_b200.inflight import InflightSession
    return InflightSession(model, max_tokens, max_seqs, page)


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ---------------------------------------------------------------------------------------------------------------
# operators alone
# ---------------------------------------------------------------------------------------------------------------
def test_small_row_operators():
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(2)
    x, w, res = torch.randn(11, 72, generator=g) * 3, torch.randn(72, generator=g) * 0.2 + 1, torch.randn(11, 72, generator=g)
    out = res.clone().cuda()
    ops.rmsnorm_rows(x.cuda(), w.cuda(), 1e-5, 0.0, out=out, accumulate=True, out_scale=0.6)
    _close(out, res.double() + 0.6 * O.rms_norm(x.double(), w.double(), 1e-5), torch.float32, "scaled post-norm residual update")
    vec = torch.randn(72, generator=g).to(torch.bfloat16)
    y = x.clone().cuda()
    ops.add_row_vector(y, vec.cuda())
    _close(y, x.double() + vec.double(), torch.float32, "row vector added")
    z = (torch.randn(5, 33, generator=g) * 30).cuda()
    want = 9.0 * torch.tanh(z.double() / 9.0)
    _close(ops.tanh_cap(z, 9.0), want, torch.float32, "capped logits")


@pytest.mark.parametrize("dtype", DTYPES)
def test_squared_relu_projection(dtype):
    from trtllm_llama_b200 import ops
    for M in (3, 12, 70):                        # streaming kernel, warp tiles, tcgen05 tiles
        g = torch.Generator().manual_seed(M)
        a, w = torch.randn(M, 48, generator=g).to(dtype), (torch.randn(72, 48, generator=g) / 7).to(dtype)
        got = ops.linear(a.cuda(), w.cuda(), out_dtype=torch.float32, act=ops.ACT_RELU_SQUARED)
        _close(got, torch.relu(a.double() @ w.double().T) ** 2, dtype, f"squared ReLU epilogue, {M} rows")


@pytest.mark.parametrize("scaling", [None, SC, (8.0, 1.0, 4.0, 2048), (2.0, 0.5, 3.0, 16)])
def test_rotary_table_with_scaled_frequencies(scaling):
    from trtllm_llama_b200 import ops
    pos = torch.tensor([0, 1, 7, 130, 4097], dtype=torch.int32)
    for dims, base in ((6, 300.0), (32, 250000.0)):
        tab = ops.rope_table(pos.cuda(), dims, base, scaling).cpu().double()
        fr = O.rotary_frequencies(dims, base, dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None)
        want = torch.tensor([[[math.cos(p * f), math.sin(p * f)] for f in fr] for p in pos.tolist()], dtype=torch.float64)
        assert (tab - want).abs().max() < 2e-6, f"rotary table, dims {dims}, scaling {scaling}"


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (6, 2, 3, 2), (12, 4, 4, 2), (5, 5, 1, 1), (4, 1, 4, 3), (64, 6, 8, 3)])
def test_router_choice(E, top, groups, keep):
    """Sigmoid scores, corrections that reorder the choice (some choices negative), group restriction by the two best of
    each group, weights without the correction; against the plain routine, token by token."""
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    n, W = 57, 24
    h = torch.randn(n, W, generator=g)
    P = {"router": torch.randn(E, W, generator=g) * 0.6, "correction": torch.randn(E, generator=g) * 0.5 - 0.3}
    logits = ops.linear(h.cuda(), P["router"].cuda(), out_dtype=torch.float32, compute=ops.COMPUTE_FMA32)
    ids, wts = ops.moe_route(logits, P["correction"].cuda(), top, groups, keep)
    want = O.route(h.double(), {k: v.double() for k, v in P.items()}, "", {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
    ids, wts = ids.cpu().tolist(), wts.cpu()
    for t, (wi, ww) in enumerate(want):
        assert sorted(ids[t]) == sorted(wi), f"token {t}: experts {ids[t]} against {wi}"
        for k, e in enumerate(ids[t]):
            assert abs(float(wts[t, k]) - ww[wi.index(e)]) < 1e-5, f"token {t}: weight of expert {e}"


def test_router_masks_with_minus_infinity_not_zero():
    """All choices negative: a masked group must not win because its experts would count as 0."""
    from trtllm_llama_b200 import ops
    logits = torch.tensor([[-3.0, -2.5, -2.0, -2.2, -9.0, -9.5]])
    corr = torch.tensor([-1.0, -1.0, -1.0, -1.0, -1.0, -1.0])
    ids, w = ops.moe_route(logits.cuda(), corr.cuda(), 2, 3, 1)
    assert sorted(ids.cpu().tolist()[0]) == [2, 3]
    assert torch.allclose(w.cpu().sort().values, torch.sigmoid(torch.tensor([-2.2, -2.0])), atol=1e-6)


@pytest.mark.parametrize("dtype,tiles", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)],
                         ids=["fp32-fma-tiles", "bf16-streaming-or-tcgen05", "bf16-warp-mma-tiles"])
@pytest.mark.parametrize("n", [1, 5, 40, 150, 700])
def test_routed_experts_alone(dtype, n, tiles, monkeypatch):
    """Every form of the expert products: fp32 FMA tiles, bf16 warp-MMA tiles, one streaming product per pair (few
    tokens), tcgen05 tiles over a plan of 128-row tiles (many)."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.layers import RoutedExpertsMLP
    monkeypatch.setattr(ops, "FORCE_TILE_LINEAR", tiles)
    g = torch.Generator().manual_seed(n)
    W, ff, E = 40, 24, 6
    r = lambda *s, std: (torch.randn(*s, generator=g) * std).to(dtype)
    P = {"router": r(E, W, std=0.5), "correction": r(E, std=0.5)}
    for e in range(E):
        P.update({f"e{e}.gate": r(ff, W, std=0.3), f"e{e}.up": r(ff, W, std=0.3), f"e{e}.down": r(W, ff, std=0.2)})
    mlp = RoutedExpertsMLP(w_router=P["router"].cuda(), correction=P["correction"].cuda(),
                           w_gate=torch.stack([P[f"e{e}.gate"] for e in range(E)]).cuda(),
                           w_up=torch.stack([P[f"e{e}.up"] for e in range(E)]).cuda(),
                           w_down=torch.stack([P[f"e{e}.down"] for e in range(E)]).cuda(), top=2, groups=3, keep=2)
    h = torch.randn(n, W, generator=g).to(dtype)
    got = mlp.forward(h.cuda(), None)
    fc = {"router": {"experts": E, "top": 2, "groups": {"count": 3, "keep": 2}}}
    _close(got, O.moe_mlp(h.double(), {k: v.double() for k, v in P.items()}, "", fc), dtype, f"routed experts, {n} tokens")


# ---------------------------------------------------------------------------------------------------------------
# the attention mixer alone, driven through the session's batch description
# ---------------------------------------------------------------------------------------------------------------
def _mixer_ctx(model, lens, page=16, max_seqs=4):
    """A step context for whole sequences of the given lengths: pages dealt in shuffled order, state slots poisoned."""
    from trtllm_llama_b200.inflight import RaggedBatch, StepContext
    sess = _session(model, max_tokens=page * sum(-(-n // page) for n in lens), max_seqs=max_seqs, page=page)
    for conv_state, _ in sess.states.values():
        conv_state.fill_(1e3)                   # whatever a slot held before must not matter at a sequence's start
    for pool in sess.pools.values():
        pool.fill_(float("nan"))
    perm = torch.randperm(sess.kv_cache_manager.blocks, generator=torch.Generator().manual_seed(5)).tolist()
    rows, used = [], 0
    for i, n in enumerate(lens):
        nb = -(-n // page)
        rows.append(([0] * n, 0, max_seqs - 1 - i, perm[used:used + nb]))
        used += nb
    return sess, StepContext(RaggedBatch(rows, [], "cuda"), sess.pools, sess.states, page)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [A_ODD, A_MQ, A_MH, A_TC, dict(A_TC, window=16, kv_heads=4, vdim=64, dim=64, rot_dims=64),
                                  dict(A_ODD, conv=6, window=2, sink=False), dict(A_MQ, rot_dims=2, gate=False, vdim=70)],
                         ids=["odd", "one-kv-head", "plain-causal", "tc", "tc-wide", "window2", "vdim70"])
def test_attention_mixer_alone(dtype, spec):
    from trtllm_llama_b200.models.nililix import build_nililix
    cfg, t = O.random_nililix([dict(spec, mlp=None)], width=40, seed=3)
    model = build_nililix(cfg, t, dtype, "cuda")
    lens = [45, 5, 1]
    sess, ctx = _mixer_ctx(model, lens)
    h = torch.randn(sum(lens), 40, generator=torch.Generator().manual_seed(4))
    got = model.layers[0]["mixer"].forward(h.cuda(), ctx)
    P, at = {k: v.double() for k, v in t.items()}, 0
    for n in lens:
        want = O.attention_mixer(h[at:at + n].double(), P, "l0.mix.", cfg["layers"][0]["mixer"])
        _close(got[at:at + n], want, dtype, f"attention mixer, sequence of {n}")
        at += n


def _standout_case(window, where, dist, page=16, P=70):
    """Operator-level case in which ONE key decides the answer: queries and that key are large along one direction, all
    other keys are small, and the key's value is far from the others.  ``dist`` = query position - key position."""
    g = torch.Generator().manual_seed(window * 131 + dist)
    H, G, d, dv = 4, 2, 8, 8
    q = torch.randn(P, H, d, generator=g) * 0.1
    k = torch.randn(P, G, d, generator=g) * 0.1
    v = torch.randn(P, G, dv, generator=g)
    qi = P - 1 if where == "decoded" else P - 3
    kj = qi - dist
    q[qi, :, 0] = 6.0
    k[kj, :, 0] = 6.0
    v[kj] = 50.0
    return H, G, d, dv, q, k, v, qi, kj


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("window,dist", [(9, 8), (9, 9), (33, 32), (33, 33), (64, 63), (64, 64), (0, 66), (16, 15), (16, 16), (1, 0), (1, 1)])
def test_one_key_stands_out(dtype, where, window, dist):
    """A key whose score dominates, placed just inside / just outside the window, at a page border or far back: the
    output follows its value exactly when it is visible.  Queries, keys and values go through the cache as the layer
    writes them (identity convolution, no rotation), as a prompt or with the last tokens decoded one by one."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    page, P = 16, 70
    H, G, d, dv, q, k, v, qi, kj = _standout_case(window, where, dist, page, P)
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0])
    want = O.windowed_sink_attention(q.double(), k.double(), v.double(), 0.7, window, sink.double())
    visible = window == 0 or dist < window
    assert (want[qi].abs().max() > 25.0) == visible, "the case does not separate inside from outside"
    proj = torch.cat([q.reshape(P, -1), k.reshape(P, -1), v.reshape(P, -1)], dim=1).cuda()
    C = proj.shape[1]
    conv_w = torch.ones(C, 1, dtype=dtype, device="cuda")
    blocks = [4, 0, 3, 1, 2]
    pool = torch.full((5 * page, G * (d + dv)), float("nan"), dtype=dtype, device="cuda")
    cuts = [P] if where == "prompt" else [P - 5, 1, 1, 1, 1, 1]
    at, outs = 0, []
    for n in cuts:
        b = RaggedBatch([([0] * n, at, 0, blocks)], [], "cuda")
        qq = ops.qkv_conv_rope_append(proj[at:at + n], conv_w, None, None, 0, pool, b, page, H, G, d, dv)
        outs.append(ops.window_attention(qq, pool, b, page, G, dv, 0.7, window, sink=sink.to(dtype).cuda()))
        at += n
    _close(torch.cat(outs), want, dtype, f"window {window}, key {dist} back ({where})")


@pytest.mark.parametrize("window", [0, 200, 64])
@pytest.mark.parametrize("d,dv,H,G", [(32, 16, 4, 2), (32, 32, 3, 3), (64, 32, 6, 1), (64, 64, 8, 2), (96, 96, 2, 1), (128, 64, 10, 2),
                                      (128, 128, 8, 2), (48, 24, 4, 2)])
def test_attention_operator_head_sizes(d, dv, H, G, window):
    """Every head size the tensor-core kernel is built for (and one it is not): a prompt of 300 positions over shuffled
    pages, then three tokens decoded one by one — few rows over a long context, so their key tiles are dealt to several
    CTAs and merged — against the plain formula and against the SIMT kernel."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    page, P, dt = 16, 303, torch.bfloat16
    g = torch.Generator().manual_seed(d * 7 + dv + window)
    q, k, v = torch.randn(P, H, d, generator=g).to(dt), torch.randn(P, G, d, generator=g).to(dt), torch.randn(P, G, dv, generator=g).to(dt)
    sink, gate = torch.randn(H, generator=g).to(dt), torch.randn(P, H, generator=g)
    want = O.windowed_sink_attention(q.double(), k.double(), v.double(), d ** -0.5, window, sink.double()) * torch.sigmoid(gate.double())[:, :, None]
    proj = torch.cat([q.reshape(P, -1), k.reshape(P, -1), v.reshape(P, -1)], dim=1).float().cuda()
    conv_w = torch.ones(proj.shape[1], 1, dtype=dt, device="cuda")
    nblk = -(-P // page)
    blocks = torch.randperm(nblk, generator=g).tolist()
    outs = {}
    for simt in (False, True):
        ops.FORCE_SIMT_ATTENTION = simt
        try:
            pool = torch.full((nblk * page, G * (d + dv)), float("nan"), dtype=dt, device="cuda")
            at, rows = 0, []
            for n in [P - 3, 1, 1, 1]:
                b = RaggedBatch([([0] * n, at, 0, blocks)], [], "cuda")
                qq = ops.qkv_conv_rope_append(proj[at:at + n], conv_w, None, None, 0, pool, b, page, H, G, d, dv)
                rows.append(ops.window_attention(qq, pool, b, page, G, dv, d ** -0.5, window, sink=sink.cuda(), gate=gate[at:at + n].cuda()))
                at += n
            outs[simt] = torch.cat(rows)
        finally:
            ops.FORCE_SIMT_ATTENTION = False
    _close(outs[True], want, dt, f"SIMT attention {d}/{dv}", scale=0.5)
    _close(outs[False], want, dt, f"attention {d}/{dv}, window {window}", scale=0.5)
    assert bool(ops._rl.tb_window_attention_tensor_cores(ops.DT_BF16, H, G, d, dv)) == ((d, dv) != (48, 24))


# ---------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(STACKS))
def test_prefill_matches_oracle_and_decode(dtype, name):
    cfg, t, model = _model(name, dtype)
    toks = _tokens(83, cfg["vocab"], 9)
    want, want_layers = _oracle(name, dtype, 0, toks, layers=True)
    sess = _session(model, max_tokens=256, page=16)
    layers = []
    got = sess.step([("a", toks, list(range(len(toks))))], on_layer=lambda i, x: layers.append(x.clone()))
    assert len(layers) == len(want_layers)
    for i, (g_, w_) in enumerate(zip(layers, want_layers)):
        _close(g_, w_, dtype, f"{name}: residual stream after layer run {i}", scale=2.0)
    _close(got, want, dtype, f"{name}: whole prompt", scale=2.0)
    rows = [sess.step([("b", [tok], [0])])[0] for tok in toks]          # token by token from position 0
    _close(torch.stack(rows), want, dtype, f"{name}: token-by-token", scale=2.0)
    _close(torch.stack(rows), got, dtype, f"{name}: prefill against decoding", scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "tc-dense"])
@pytest.mark.parametrize("cuts", [[2, 2, 2, 77], [1, 15, 1, 16, 17, 33], [31, 2, 50], [64, 19], [3] * 27 + [2]])
def test_portions(dtype, cuts, name):
    cfg, t, model = _model(name, dtype)
    toks = _tokens(sum(cuts), cfg["vocab"], 10)
    want = _oracle(name, dtype, 0, toks)
    sess = _session(model, max_tokens=128, page=16)
    at, rows = 0, []
    for n in cuts:
        rows.append(sess.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    _close(torch.cat(rows), want, dtype, f"{name}: portions {cuts[:6]}", scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "tc", "tc-dense"])
def test_mixed_batches_and_reuse(dtype, name):
    """Five requests of unequal length through FOUR slots and a pool that cannot hold them all at once: portions beside
    single tokens, requests that sit a step out, pages and slots handed on — every logit equals the request run alone."""
    cfg, t, model = _model(name, dtype)
    lens = {"a": 70, "b": 33, "c": 5, "d": 90, "e": 41}
    toks = {k: _tokens(n, cfg["vocab"], 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: _oracle(name, dtype, 0, v) for k, v in toks.items()}
    sess = _session(model, max_tokens=16 * 16, max_seqs=4, page=16)      # 16 pages; the five need 5 + 3 + 1 + 6 + 3 = 18
    plan = [  # (request, tokens it brings) per step
        [("a", 3), ("b", 2)], [("a", 30), ("b", 1), ("c", 2)], [("a", 1), ("c", 3), ("d", 17)], [("b", 29), ("d", 2)],
        [("a", 36), ("b", 1), ("d", 40)], [("d", 1), ("e", 16)], [("d", 30), ("e", 1)], [("e", 24)],
    ]
    at, got = {k: 0 for k in lens}, {k: [] for k in lens}
    for step in plan:
        entries = [(k, toks[k][at[k]:at[k] + n], list(range(n))) for k, n in step]
        out, row = sess.step(entries), 0
        for k, n in step:
            got[k].append(out[row:row + n])
            row, at[k] = row + n, at[k] + n
            if at[k] == lens[k]:
                sess.end(k)
    assert at == lens and not sess.live
    assert len(sess.kv_cache_manager.free_blocks) == 16 and sorted(sess.slot_manager.free) == [0, 1, 2, 3]
    for k in lens:
        _close(torch.cat(got[k]), want[k], dtype, f"{name}: request {k} in mixed batches", scale=2.0)


@pytest.mark.parametrize("graph", [True, False], ids=["replayed-graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tc", "tc-dense"])
def test_long_decoding_across_pages_and_windows(dtype, graph, name):
    """180 generated tokens: the windows (33 and 64) pass wholly over decoded tokens and the block table outgrows its
    captured width; replayed graphs and eager launches of the same step give the same answer."""
    cfg, t, model = _model(name, dtype, seed=2)
    toks = _tokens(20 + 180, cfg["vocab"], 30)
    want = _oracle(name, dtype, 2, toks)
    sess = _session(model, max_tokens=208, page=16)
    sess.use_cuda_graph = graph
    rows = [sess.step([("a", toks[:20], [19])])[0]]
    rows += [sess.step([("a", [tok], [0])])[0] for tok in toks[20:]]
    _close(torch.stack(rows), want[19:], dtype, f"{name}: 180 decoded tokens", scale=2.0)
    assert bool(sess._graphs) == graph


@pytest.mark.parametrize("dtype,name", [(torch.float32, "odd"), (torch.float32, "tc"), (torch.bfloat16, "tc"), (torch.bfloat16, "tc-dense")])
def test_greedy_generation_through_the_scheduler(dtype, name):
    """Six prompts through four slots with a small per-step budget (chunked prefill beside decodes); every generated
    id is the oracle's arg-max on the same history unless the oracle's two best logits are closer than the tolerance."""
    from trtllm_llama_b200.runtime import SamplingConfig
    cfg, t, model = _model(name, dtype, seed=4)
    prompts = [_tokens(n, cfg["vocab"], 40 + n) for n in (1, 9, 40, 17, 3, 26)]
    sess = _session(model, max_tokens=16 * 12, max_seqs=4, page=16)
    new = 12
    outs = sess.generate(prompts, new, SamplingConfig(end_id=None), max_step_tokens=24)
    assert not sess.live and len(sess.kv_cache_manager.free_blocks) == 12
    for p, o in zip(prompts, outs):
        assert len(o) == new
        lg = O.nililix_forward(cfg, t, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            best = lg[i].topk(2)
            if int(best.indices[0]) != tok:
                assert float(best.values[0] - lg[i][tok]) <= 2 * TOL[dtype] * float(lg.abs().max()), f"step {i}: id {tok} is not the arg-max"


def test_registry_and_trace_tool_end_to_end(tmp_path):
    """A checkpoint folder is recognised by its config.json, and bin/trace_run replays steps on it as a user runs it."""
    import subprocess
    import sys
    import numpy as np
    from trtllm_llama_b200 import models
    from trtllm_llama_b200.checkpoint import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, t = O.random_nililix(**STACKS["odd"])
    os.makedirs(tmp_path / "m")
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    assert "nililix" in models.registered_models()
    toks = {"a": _tokens(40, cfg["vocab"], 1), "b": _tokens(9, cfg["vocab"], 2)}
    want = {k: O.nililix_forward(cfg, t, v) for k, v in toks.items()}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": toks["a"][:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": toks["a"][30:31], "want": [0]}, {"id": "b", "tokens": toks["b"], "want": [8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": toks["a"][31:], "want": []}], "end": []},
        {"step": 3, "entries": [], "end": ["a"]},
    ]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 2", "done 3"]
    got0 = torch.from_numpy(np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(tmp_path / "o" / "1.f32", dtype="<f4").reshape(2, -1))
    _close(got0, want["a"][[0, 29]], torch.float32, "trace step 0", scale=2.0)
    _close(got1, torch.stack([want["a"][30], want["b"][8]]), torch.float32, "trace step 1", scale=2.0)
    assert not os.path.exists(tmp_path / "o" / "2.f32")


def test_generation_example_from_the_command_line(tmp_path):
    """examples/inflight/run.py on a Nililix folder: the registry picks the class, the scheduler runs the prompts, and the
    ids are the oracle's greedy continuation."""
    import csv
    import subprocess
    import sys
    from trtllm_llama_b200.checkpoint import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, t = O.random_nililix(**STACKS["tc-dense"])
    os.makedirs(tmp_path / "m")
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    prompts = [_tokens(n, cfg["vocab"], 70 + n) for n in (5, 31)]
    with open(tmp_path / "in.csv", "w") as f:
        csv.writer(f).writerows(prompts)
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "inflight", "run.py"), "--model_dir", str(tmp_path / "m"),
                        "--input_tokens", str(tmp_path / "in.csv"), "--max_output_len", "6", "--dtype", "float32",
                        "--output_csv", str(tmp_path / "out.csv"), "--max_step_tokens", "16"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    with open(tmp_path / "out.csv") as f:
        outs = [[int(x) for x in row] for row in csv.reader(f) if row]
    assert len(outs) == 2
    for p, o in zip(prompts, outs):
        o = o[-6:]
        lg = O.nililix_forward(cfg, t, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            best = lg[i].topk(2)
            if int(best.indices[0]) != tok:
                assert float(best.values[0] - lg[i][tok]) <= 2 * TOL[torch.float32] * float(lg.abs().max()), f"step {i}: id {tok}"
