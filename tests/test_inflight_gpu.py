"""In-flight served models (latent attention + gated linear recurrence) on the GPU against the plain float64 oracle
(oracle/seq_mixers.py): every mechanism alone, prefill against token-by-token decoding, portions down to two tokens,
unequal batches against each request alone, pages and state slots used again, keys far away and at page borders, the
first tokens of a sequence, long decoding, odd sizes, and greedy generation through the scheduler."""
import json
import os

import pytest
import torch

from oracle import seq_mixers as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
# relative to the largest magnitude of the compared tensor
TOL = {torch.float32: 2e-4, torch.bfloat16: 4e-2}


def _close(got, want, dtype, what, scale=1.0):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item()
    ref = max(want.abs().max().item(), 1e-6)
    assert err <= TOL[dtype] * scale * ref, f"{what}: max error {err:.3e} against magnitude {ref:.3e}"


ATT = dict(type="latent_attention", heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=40, q_rank=24, mlp=None)
ATT_MLP = dict(ATT, mlp=(50, 1.5))
REC = dict(type="rglru", width=36, blocks=3, conv=3, mlp=None)
# tensor-core friendly sizes (16 | lat + rot_dim, 32 | lat) beside the odd ones
ATT_TC = dict(type="latent_attention", heads=5, dim=16, rot_dim=16, vdim=24, kv_rank=64, q_rank=32, mlp=(64, 2.5))
STACKS = {
    "odd": dict(layers=[ATT, dict(REC, mlp=(50, 1.5)), dict(ATT, kv_from=0, mlp=(50, 1.5)), REC], width=40, vocab=61),
    "tc": dict(layers=[dict(REC, width=64, blocks=1, conv=2, mlp=(64, 3.0)), ATT_TC, dict(ATT_TC, kv_from=1), ATT_TC,
                       dict(ATT_TC, kv_from=1, mlp=None)], width=64, vocab=130, embed_scale=1.0),
    # 64 | latent and 32 | latent + rot: the eight-warp form of the tensor-core attention
    "tc8": dict(layers=[dict(ATT_TC, rot_dim=32, mlp=None), dict(type="rglru", width=32, blocks=2, conv=3, mlp=(48, 4.0)),
                        dict(ATT_TC, rot_dim=32, kv_from=0)], width=48, vocab=77, embed_scale=2.0),
    "wide": dict(layers=[dict(type="latent_attention", heads=18, dim=8, rot_dim=8, vdim=8, kv_rank=96, q_rank=16, mlp=None),
                         dict(type="rglru", width=80, blocks=5, conv=5, mlp=None)], width=32, vocab=40, eps=1e-6),
}


_ORACLE = {}


def _oracle(name, seed, toks, layers=False):
    """The oracle's answer does not depend on the product's dtype: computed once per (stack, weights, tokens)."""
    key = (name, seed, tuple(toks))
    if key not in _ORACLE:
        cfg, t = O.random_zobasun(seed=seed, **STACKS[name])
        _ORACLE[key] = O.zobasun_forward(cfg, t, toks, return_layers=True)
    return _ORACLE[key] if layers else _ORACLE[key][0]


def _model(name, dtype, seed=0):
    from trtllm_llama_b200.models.zobasun import build_zobasun
    cfg, t = O.random_zobasun(seed=seed, **STACKS[name])
    return cfg, t, build_zobasun(cfg, t, dtype, "cuda")


def _session(model, max_tokens=512, max_seqs=4, page=64):
    from trtllm_llama_b200.inflight import InflightSession
    return InflightSession(model, max_tokens, max_seqs, page)


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ---------------------------------------------------------------------------------------------------------------
# operators alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 61, 40), (7, 70, 96), (130, 256, 264), (300, 33, 17), (64, 128, 512)])
def test_linear(dtype, shape):
    from trtllm_llama_b200 import ops
    M, N, K = shape
    g = torch.Generator().manual_seed(M)
    a, w, b = torch.randn(M, K, generator=g), (torch.randn(N, K, generator=g) / K ** 0.5).to(dtype), torch.randn(N, generator=g).to(dtype)
    for a_dt in {torch.float32, dtype}:
        av = a.to(a_dt)
        want = av.double() @ w.double().T + b.double()
        for act, fn in ((ops.ACT_NONE, lambda z: z), (ops.ACT_GELU_TANH, O.gelu_tanh)):
            for compute in (ops.COMPUTE_AUTO, ops.COMPUTE_FMA32):
                got = ops.linear(av.cuda(), w.cuda(), b.cuda(), out_dtype=torch.float32, act=act, compute=compute)
                exact = compute == ops.COMPUTE_FMA32 and a_dt == torch.float32
                _close(got, fn(want), torch.float32 if exact or dtype == torch.float32 else dtype, f"linear {shape} act {act}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_batched_strided(dtype):
    from trtllm_llama_b200 import ops
    n, H, dn, dr, R = 9, 3, 20, 6, 24
    g = torch.Generator().manual_seed(1)
    q, w = torch.randn(n, H * (dn + dr), generator=g), torch.randn(H, R, dn, generator=g).to(dtype)
    out = torch.full((n, H, R + dr), 7.0, dtype=dtype, device="cuda")
    ops.linear(q.cuda().view(n, H, dn + dr)[:, :, :dn], w.cuda(), out=out[:, :, :R])
    want = torch.einsum("nhd,hrd->nhr", q.view(n, H, dn + dr)[:, :, :dn].double(), w.double())
    _close(out[:, :, :R], want, dtype, "batched linear")
    assert (out[:, :, R:] == 7.0).all(), "the batched product wrote outside its columns"


def test_rmsnorm_and_activation():
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(2)
    x, w = torch.randn(11, 72, generator=g) * 3, torch.randn(72, generator=g) * 0.2
    res = torch.randn(11, 72, generator=g)
    out = res.clone().cuda()
    ops.rmsnorm_rows(x.cuda(), w.cuda(), 1e-5, 1.0, out=out, accumulate=True)
    _close(out, res.double() + O.rms_norm(x.double(), w.double(), 1e-5, 1.0), torch.float32, "post-norm residual update")
    idx = torch.tensor([10, 0, 3], dtype=torch.int32)
    got = ops.rmsnorm_rows(x.cuda(), w.cuda(), 1e-5, 0.0, out_dtype=torch.float32, rows_idx=idx.cuda())
    _close(got, O.rms_norm(x.double()[idx.long()], w.double(), 1e-5), torch.float32, "gathered norm")
    gu = torch.randn(5, 2 * 30, generator=g) * 3
    got = ops.gated_act(gu.cuda(), torch.float32, 1.702, 1.5, 1.0)
    gg, uu = gu[:, :30].double().clamp(max=1.5), gu[:, 30:].double().clamp(-1.5, 1.5)
    _close(got, gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), torch.float32, "clamped gated activation")


@pytest.mark.parametrize("rows", [1, 3, 8, 9])
def test_gated_projection_fused_for_few_rows(rows):
    """Up to 8 rows the gate / up projection and the clamped gated activation run as one streaming kernel; it must
    equal the two-kernel form (which larger steps use) and the plain formula."""
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(rows)
    K, ff = 72, 50
    x = torch.randn(rows, K, generator=g)
    w = (torch.randn(2 * ff, K, generator=g) * 0.4).to(torch.bfloat16)
    fused = ops.linear_gated(x.cuda(), w.cuda(), torch.float32, 1.702, 1.5, 1.0)
    two = ops.gated_act(ops.linear(x.cuda(), w.cuda(), out_dtype=torch.float32), torch.float32, 1.702, 1.5, 1.0)
    xb = x.to(torch.bfloat16).double()
    gg, uu = (xb @ w[:ff].double().T).clamp(max=1.5), (xb @ w[ff:].double().T).clamp(-1.5, 1.5)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)
    _close(two, want, torch.float32, "projection + activation")
    if rows <= 8:
        _close(fused, want, torch.float32, "fused gated projection")
    else:
        assert fused is None


# ---------------------------------------------------------------------------------------------------------------
# mixers alone, driven through the session's batch description
# ---------------------------------------------------------------------------------------------------------------
def _mixer_ctx(model, lens, page=16, max_seqs=4):
    """A step context for whole sequences of the given lengths, with the pool's pages dealt in shuffled order."""
    from trtllm_llama_b200.inflight import RaggedBatch, StepContext
    sess = _session(model, max_tokens=page * sum(-(-n // page) for n in lens), max_seqs=max_seqs, page=page)
    perm = torch.randperm(sess.kv_cache_manager.blocks, generator=torch.Generator().manual_seed(5)).tolist()
    rows, used = [], 0
    for i, n in enumerate(lens):
        nb = -(-n // page)
        rows.append(([0] * n, 0, max_seqs - 1 - i, perm[used:used + nb]))
        used += nb
    return sess, StepContext(RaggedBatch(rows, [], "cuda"), sess.pools, sess.states, page)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [ATT, ATT_TC], ids=["odd", "tc"])
def test_latent_attention_alone(dtype, spec):
    from trtllm_llama_b200.models.zobasun import build_zobasun
    cfg, t = O.random_zobasun([dict(spec, mlp=None)], width=40, seed=3)
    model = build_zobasun(cfg, t, dtype, "cuda")
    lens = [37, 5, 1]
    sess, ctx = _mixer_ctx(model, lens)
    h = torch.randn(sum(lens), 40, generator=torch.Generator().manual_seed(4)) * 2
    got = model.layers[0]["mixer"].forward(h.cuda(), ctx)
    m, W, at = cfg["layers"][0]["mixer"], {k: v.double() for k, v in t.items()}, 0
    for n in lens:
        hs = h[at:at + n].double()
        c, kr = O.latent_cache_entries(hs, W["l0.mix.dkv"], W["l0.mix.dkv.norm"], m["kv_rank"], m["rot"]["dims"], m["rot"]["base"], 1e-5)
        want = O.latent_attention(hs, c, kr, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                                  rot_dims=m["rot"]["dims"], rot_base=m["rot"]["base"], scale=m["scale"], eps=1e-5,
                                  w_dq=W["l0.mix.dq"], w_dq_norm=W["l0.mix.dq.norm"], w_uq=W["l0.mix.uq"], w_uk=W["l0.mix.uk"],
                                  w_uv=W["l0.mix.uv"], w_o=W["l0.mix.o"])
        _close(got[at:at + n], want, dtype, f"latent attention, sequence of {n}")
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [REC, dict(REC, width=64, blocks=1, conv=1), dict(REC, width=40, blocks=5, conv=6)])
def test_gated_linear_recurrence_alone(dtype, spec):
    from trtllm_llama_b200.models.zobasun import build_zobasun
    cfg, t = O.random_zobasun([spec], width=40, seed=6)
    model = build_zobasun(cfg, t, dtype, "cuda")
    lens = [29, 2, 1]
    sess, ctx = _mixer_ctx(model, lens)
    for conv_state, rec_state in sess.states.values():      # whatever a slot held before must not matter at position 0
        conv_state.fill_(1e3)
        rec_state.fill_(-1e3)
    h = torch.randn(sum(lens), 40, generator=torch.Generator().manual_seed(7))
    got = model.layers[0]["mixer"].forward(h.cuda(), ctx)
    m, W, at = cfg["layers"][0]["mixer"], {k[len("l0.mix."):].replace(".", "_"): v.double() for k, v in t.items() if k.startswith("l0.mix.")}, 0
    for n in lens:
        want = O.gated_linear_recurrence(h[at:at + n].double(), channels=m["width"], blocks=m["blocks"], w_y=W["y"], b_y=W["y_b"],
                                         w_x=W["x"], b_x=W["x_b"], conv_w=W["conv"], conv_b=W["conv_b"], w_ra=W["ra"],
                                         b_ra=W["ra_b"], w_ri=W["ri"], b_ri=W["ri_b"], lam=W["lam"], w_o=W["o"])
        _close(got[at:at + n], want, dtype, f"recurrent block, sequence of {n}")
        at += n


@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_one_key_stands_out(dtype, where):
    """Cache entries are random except one, whose direction the query is made to match with a large score: the output
    must be that entry's latent — whether the entry is the first position, far back, the last of a page, the first of
    the next, or the row's own position.  A page read from the wrong block or a key lost at a border shows at once."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    lat, rot, H, page, L = 32, 16, 2, 16, 150
    D = lat + rot
    g = torch.Generator().manual_seed(8)
    blocks = torch.randperm(16, generator=g).tolist()[:-(-L // page)]
    kv = torch.randn(L, D, generator=g)
    pool = torch.full((16 * page, D), float("nan"), dtype=dtype, device="cuda")
    fill = RaggedBatch([([0] * L, 0, 0, blocks)], [], "cuda")
    ones = torch.ones(lat, dtype=dtype, device="cuda")
    table = ops.rope_table(fill.tok_pos, rot, 10000.0)
    ops.latent_kv_append(pool, kv.cuda(), ones, 1e-6, table, rot, fill, page, lat, rot)
    entries = torch.cat([O.rms_norm(kv[:, :lat].double(), None, 1e-6),
                         O.rotate_pairs(kv[:, lat:].double(), torch.arange(L), 10000.0, rot)], 1)
    for target in (0, 1, page - 1, page, page + 1, 5 * page - 1, 5 * page, L - 2, L - 1):
        if where == "decoded":
            rows, pos = [([0], L - 1, 0, blocks)], [L - 1]
        else:       # a portion of three rows ending at L - 1; the middle row cannot see L - 1
            rows, pos = [([0] * 3, L - 3, 0, blocks)], [L - 3, L - 2, L - 1]
        batch = RaggedBatch(rows, [], "cuda")
        qa = torch.randn(len(pos), H, D, generator=g) * 0.1
        qa[:, 1] += 6.0 * entries[target].float()
        got = ops.latent_attention(qa.to(dtype).cuda(), pool, batch, page, H, lat, rot, 1.0)
        for r, p in enumerate(pos):
            vis = entries[: p + 1].to(dtype).double()
            s = torch.softmax(qa[r].to(dtype).double() @ vis.T, -1)
            want = s @ vis[:, :lat]
            _close(got[r], want, dtype, f"key {target} seen from {p}", scale=2.0)
            if target <= p:
                assert s[1, target] > 0.9, "the test's spike is not sharp enough"
                _close(got[r, 1], entries[target, :lat], dtype, f"spike at {target} seen from {p}", scale=8.0)


@pytest.mark.parametrize("lat,rot,heads", [(32, 16, 1), (96, 32, 5), (128, 16, 20), (160, 16, 16), (192, 64, 3), (256, 16, 17),
                                          (384, 32, 2), (512, 64, 16), (512, 64, 33), (40, 6, 3), (64, 8, 4)])
def test_latent_attention_operator_sizes(lat, rot, heads):
    """Every latent width the tensor-core kernel is instantiated for (and two it is not), more heads than one CTA
    takes, a prompt portion and single rows whose keys are dealt to several CTAs, over shuffled pages."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    dtype, page, D = torch.bfloat16, 16, lat + rot
    g = torch.Generator().manual_seed(lat + heads)
    lens = [300, 70]
    nblk = [-(-n // page) for n in lens]
    perm = torch.randperm(sum(nblk) + 3, generator=g).tolist()
    blocks = [perm[:nblk[0]], perm[nblk[0]:nblk[0] + nblk[1]]]
    entries = [torch.randn(n, D, generator=g).to(dtype) for n in lens]
    pool = torch.full(((sum(nblk) + 3) * page, D), float("nan"), dtype=dtype)
    for e, b in zip(entries, blocks):
        for j in range(e.shape[0]):
            pool[b[j // page] * page + j % page] = e[j]
    pool = pool.cuda()

    def want(q, e, p):           # q [H, D] at position p of a sequence whose entries are e
        vis = e[: p + 1].double()
        return torch.softmax(q.double() @ vis.T * 0.3, -1) @ vis[:, :lat]

    # a portion of 40 rows at the end of the first sequence beside the whole second sequence
    rows = [([0] * 40, lens[0] - 40, 0, blocks[0]), ([0] * lens[1], 0, 1, blocks[1])]
    qa = (torch.randn(40 + lens[1], heads, D, generator=g) * 0.5).to(dtype)
    got = ops.latent_attention(qa.cuda(), pool, RaggedBatch(rows, [], "cuda"), page, heads, lat, rot, 0.3)
    ref = torch.stack([want(qa[r], entries[0], lens[0] - 40 + r) for r in range(40)] +
                      [want(qa[40 + r], entries[1], r) for r in range(lens[1])])
    _close(got, ref, dtype, f"prompt rows, latent {lat} rot {rot} heads {heads}")
    # the tensor-core kernel against the warp-per-head kernel on the same operands: only the bf16 rounding of the
    # probabilities and of the outputs may differ
    ops.FORCE_SIMT_ATTENTION = True
    try:
        plain = ops.latent_attention(qa.cuda(), pool, RaggedBatch(rows, [], "cuda"), page, heads, lat, rot, 0.3)
    finally:
        ops.FORCE_SIMT_ATTENTION = False
    assert (got.float() - plain.float()).abs().max() <= 1.2e-2 * ref.abs().max(), "the two attention kernels disagree"
    # single rows at the last positions: long enough for the keys to be split over CTAs
    rows = [([0], lens[0] - 1, 0, blocks[0]), ([0], lens[1] - 1, 1, blocks[1])]
    qd = (torch.randn(2, heads, D, generator=g) * 0.5).to(dtype)
    got = ops.latent_attention(qd.cuda(), pool, RaggedBatch(rows, [], "cuda"), page, heads, lat, rot, 0.3)
    ref = torch.stack([want(qd[0], entries[0], lens[0] - 1), want(qd[1], entries[1], lens[1] - 1)])
    _close(got, ref, dtype, f"single rows, latent {lat} rot {rot} heads {heads}")


# ---------------------------------------------------------------------------------------------------------------
# whole models through the session
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(STACKS))
def test_prefill_matches_oracle_and_decode(dtype, name):
    cfg, t, model = _model(name, dtype)
    toks = _tokens(83, cfg["vocab"], 9)
    want, want_layers = _oracle(name, 0, toks, layers=True)
    sess = _session(model, max_tokens=256, page=16)
    layers = []
    got = sess.step([("a", toks, list(range(len(toks))))], on_layer=lambda i, x: layers.append(x.clone()))
    for i, (g_, w_) in enumerate(zip(layers, want_layers)):
        _close(g_, w_, dtype, f"{name}: residual stream after layer {i}", scale=2.0)
    _close(got, want, dtype, f"{name}: whole prompt", scale=2.0)
    rows = [sess.step([("b", [tok], [0])])[0] for tok in toks]          # token by token from position 0
    _close(torch.stack(rows), want, dtype, f"{name}: token-by-token", scale=2.0)
    _close(torch.stack(rows), got, dtype, f"{name}: prefill against decoding", scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 77], [1, 15, 1, 16, 17, 33], [31, 2, 50], [64, 19], [3] * 27 + [2]])
def test_portions(dtype, cuts):
    cfg, t, model = _model("odd", dtype)
    toks = _tokens(sum(cuts), cfg["vocab"], 10)
    want = _oracle("odd", 0, toks)
    sess = _session(model, max_tokens=128, page=16)
    at, rows = 0, []
    for n in cuts:
        rows.append(sess.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    _close(torch.cat(rows), want, dtype, f"portions {cuts[:6]}", scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "tc", "tc8"])
def test_mixed_batches_and_reuse(dtype, name):
    """Five requests of unequal length through FOUR slots and a pool that cannot hold them all at once: portions beside
    single tokens, requests that sit a step out, pages and slots handed on — every logit equals the request run alone."""
    cfg, t, model = _model(name, dtype)
    lens = {"a": 70, "b": 33, "c": 5, "d": 90, "e": 41}
    toks = {k: _tokens(n, cfg["vocab"], 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: _oracle(name, 0, v) for k, v in toks.items()}
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
def test_long_decoding_across_pages(dtype, graph):
    """Generation steps are replayed CUDA graphs (re-captured when the block table outgrows its width); the eager
    launches of the same step must give the same answer."""
    cfg, t, model = _model("tc", dtype, seed=2)
    toks = _tokens(20 + 180, cfg["vocab"], 30)
    want = _oracle("tc", 2, toks)
    sess = _session(model, max_tokens=208, page=16)
    sess.use_cuda_graph = graph
    rows = [sess.step([("a", toks[:20], [19])])[0]]
    rows += [sess.step([("a", [tok], [0])])[0] for tok in toks[20:]]
    _close(torch.stack(rows), want[19:], dtype, "180 decoded tokens", scale=2.0)
    assert bool(sess._graphs) == graph


def test_pool_exhaustion_is_refused_cleanly():
    cfg, t, model = _model("odd", torch.float32)
    sess = _session(model, max_tokens=32, max_seqs=2, page=16)
    sess.step([("a", _tokens(20, cfg["vocab"], 1), [])])
    with pytest.raises(RuntimeError):
        sess.step([("b", _tokens(20, cfg["vocab"], 2), [])])
    assert "b" not in sess.live and len(sess.slot_manager.free) == 1
    sess.end("a")
    assert sess.step([("b", _tokens(20, cfg["vocab"], 2), [19])]).shape == (1, cfg["vocab"])


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_scheduler(dtype):
    """Six prompts through four slots with a small per-step budget (chunked prefill beside decodes); every generated
    id is the oracle's arg-max on the same history unless the oracle's two best logits are closer than the tolerance."""
    from trtllm_llama_b200.runtime import SamplingConfig
    cfg, t, model = _model("odd", dtype, seed=4)
    prompts = [_tokens(n, cfg["vocab"], 40 + n) for n in (1, 9, 40, 17, 3, 26)]
    sess = _session(model, max_tokens=16 * 12, max_seqs=4, page=16)
    new = 12
    outs = sess.generate(prompts, new, SamplingConfig(end_id=None), max_step_tokens=24)
    assert not sess.live and len(sess.kv_cache_manager.free_blocks) == 12
    for p, o in zip(prompts, outs):
        assert len(o) == new
        lg = O.zobasun_forward(cfg, t, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            best = lg[i].topk(2)
            if int(best.indices[0]) != tok:
                assert float(best.values[0] - lg[i][tok]) <= 2 * TOL[dtype] * float(lg.abs().max()), f"step {i}: id {tok} is not the arg-max"


def test_sampled_generation_uses_the_sampling_kernel():
    """top-k sampling through the scheduler: reproducible for a seed, different for another, and every id is one of the
    oracle's k best on the same history (or within tolerance of the k-th)."""
    from trtllm_llama_b200.runtime import SamplingConfig
    cfg, t, model = _model("odd", torch.float32, seed=5)
    prompts = [_tokens(n, cfg["vocab"], 60 + n) for n in (7, 21)]
    sess = _session(model, max_tokens=16 * 8, max_seqs=2, page=16)
    sc = SamplingConfig(end_id=None, top_k=4, top_p=0.0, temperature=0.8, random_seed=11)
    a = sess.generate(prompts, 10, sc, max_step_tokens=16)
    b = sess.generate(prompts, 10, sc, max_step_tokens=16)
    c = sess.generate(prompts, 10, SamplingConfig(end_id=None, top_k=4, top_p=0.0, temperature=0.8, random_seed=12), max_step_tokens=16)
    assert a == b and a != c
    for p, o in zip(prompts, a):
        lg = O.zobasun_forward(cfg, t, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            kth = lg[i].topk(4).values[-1]
            assert lg[i][tok] >= kth - 2 * TOL[torch.float32] * float(lg.abs().max()), f"step {i}: id {tok} is outside the top 4"


def test_registry_loads_a_checkpoint_folder(tmp_path):
    from trtllm_llama_b200 import models
    from trtllm_llama_b200.checkpoint import write_safetensors
    cfg, t = O.random_zobasun(**STACKS["odd"])
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    model = models.load_model(str(tmp_path), "float32")
    toks = _tokens(12, cfg["vocab"], 3)
    got = _session(model, 64, page=16).step([("a", toks, [11])])
    _close(got[0], O.zobasun_forward(cfg, t, toks)[-1], torch.float32, "model loaded through the registry", scale=2.0)


def test_trace_tool_end_to_end(tmp_path):
    """bin/trace_run as a user runs it: a folder, steps on standard input, logits files and 'done' lines out."""
    import subprocess
    import sys
    import numpy as np
    from trtllm_llama_b200.checkpoint import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, t = O.random_zobasun(**STACKS["odd"])
    os.makedirs(tmp_path / "m")
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    a, b = _tokens(30, cfg["vocab"], 5), _tokens(7, cfg["vocab"], 6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [19]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [4]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[20:], "want": [0, 9]}], "end": ["a"]}]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = O.zobasun_forward(cfg, t, a), O.zobasun_forward(cfg, t, b)
    rd = lambda n: torch.from_numpy(np.fromfile(tmp_path / "o" / f"{n}.f32", dtype="<f4")).view(-1, cfg["vocab"])  # noqa: E731
    _close(rd(0), wa[19:20], torch.float32, "step 0", scale=2.0)
    _close(rd(1), wb[6:7], torch.float32, "step 1", scale=2.0)
    _close(rd(2), wa[[20, 29]], torch.float32, "step 2", scale=2.0)
