"""Host-side parts of the Nililix design: the configuration reader and what it asks of the session (one cache pool and
one convolution state per layer RUN of a looped block), configuration errors, and properties of the plain oracle that
the GPU tests lean on (causality, the window's reach, the sink, the group restriction of the router)."""
import math

import pytest
import torch

from oracle import nililix_plain as O

ATT = dict(heads=4, kv_heads=2, dim=8, vdim=6, conv=3, window=5, rot_dims=4, scaling=(4.0, 1.0, 4.0, 64))


def _build(layers, **kw):
    from trtllm_llama_b200.models.nililix import build_nililix
    cfg, t = O.random_nililix(layers, width=24, vocab=30, **kw)
    return cfg, t, build_nililix(cfg, t, "float32", "cpu")


def test_layer_runs_pools_and_states_of_a_looped_block():
    layers = [dict(ATT, mlp=("dense", 16)), dict(ATT, kv_heads=4, conv=1, mlp=None), dict(ATT, mlp=("moe", 8, 6, 2, 3, 2))]
    cfg, t, model = _build(layers, loop=(1, 3, 2))
    assert model.runs == [(0, 0, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False)]
    assert model.runs == O.layer_runs(cfg)
    pools, states = model.cache_layers(), model.state_layers()
    assert set(pools) == {(0, 0), (1, 0), (2, 0), (1, 1), (2, 1)}
    assert pools[(0, 0)] == 2 * (8 + 6) and pools[(1, 1)] == 4 * (8 + 6)
    assert states[(2, 1)] == (3, 4 * 8 + 2 * (8 + 6), False) and states[(1, 0)][0] == 1
    assert model.residual_mult == cfg["residual_mult"] and model.logit_cap == cfg["logit_softcap"]
    mlp = model.layers[2]["mlp"]
    assert (mlp.experts, mlp.top, mlp.groups, mlp.keep) == (6, 2, 3, 2) and tuple(mlp.w_gate_up.shape) == (6, 16, 24)


def test_no_loop_no_cap_no_feed_forward():
    cfg, t, model = _build([dict(ATT, mlp=None, sink=False, gate=False)], loop=None, logit_softcap=None)
    assert model.runs == [(0, 0, False)] and model.logit_cap == 0.0 and model.loop_step is None
    assert model.layers[0]["mixer"].sink is None and not model.layers[0]["mixer"].gated


def test_configuration_errors():
    from trtllm_llama_b200.models.nililix import build_nililix
    cfg, t = O.random_nililix([dict(ATT, mlp=None)], width=24, vocab=30)
    bad = dict(cfg, layers=[dict(cfg["layers"][0], type="recurrent")])
    with pytest.raises(ValueError):
        build_nililix(bad, t, "float32", "cpu")
    bad = dict(cfg, layers=[dict(cfg["layers"][0], mixer=dict(cfg["layers"][0]["mixer"], kv_heads=3))])
    with pytest.raises(ValueError):
        build_nililix(bad, t, "float32", "cpu")
    with pytest.raises(KeyError):
        build_nililix(cfg, {k: v for k, v in t.items() if k != "l0.mix.o"}, "float32", "cpu")
    with pytest.raises(ValueError):
        build_nililix(dict(cfg, loop={"start": 0, "stop": 2, "times": 2}), t, "float32", "cpu")


def test_oracle_reach_of_the_window():
    """One layer with window w: position i depends on tokens i - (w - 1) - (taps - 1) .. i and on nothing else."""
    cfg, t = O.random_nililix([dict(ATT, mlp=("dense", 16))], width=24, vocab=30, seed=1)
    w, taps = 5, 3
    toks = list(range(20))
    base = O.nililix_forward(cfg, t, toks)
    for j in (2, 9):
        other = list(toks)
        other[j] = 29
        z = O.nililix_forward(cfg, t, other)
        changed = [(z[i] - base[i]).abs().max().item() > 1e-9 for i in range(20)]
        reach = (w - 1) + (taps - 1)
        assert changed == [j <= i <= j + reach for i in range(20)]


def test_oracle_sink_only_shrinks():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(6, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    free = O.windowed_sink_attention(q, k, v, 0.5, 0, None)
    low = O.windowed_sink_attention(q, k, v, 0.5, 0, torch.tensor([-50.0, -50.0], dtype=torch.float64))
    high = O.windowed_sink_attention(q, k, v, 0.5, 0, torch.tensor([50.0, 50.0], dtype=torch.float64))
    assert (free - low).abs().max() < 1e-12 and high.abs().max() < 1e-12
    one = O.windowed_sink_attention(q[:1], k[:1], v[:1], 0.5, 0, torch.zeros(2, dtype=torch.float64))
    s = (q[0] * k[0]).sum(-1) * 0.5                       # a single key against a sink of 0: weight e^s / (e^s + 1)
    assert (one[0] - torch.sigmoid(s)[:, None] * v[0]).abs().max() < 1e-12


def test_oracle_router_groups():
    P = {"router": torch.eye(6, dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 0.3, 0.0, -5.0, 0.95], dtype=torch.float64)}
    h = torch.tensor([[3.0, 2.5, 0.0, 0.1, 4.0, -4.0]], dtype=torch.float64)
    rc = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    (ids, ws), = O.route(h, P, "", rc)
    assert sorted(ids) == [0, 1]                            # group 0 has the best pair although expert 5 is the best single choice
    assert abs(ws[ids.index(0)] - 1 / (1 + math.exp(-3.0))) < 1e-12
    (ids, _), = O.route(h, P, "", dict(rc, groups={"count": 1, "keep": 1}))
    assert sorted(ids) == [0, 5]                            # without groups expert 5 (0.018 + 0.95) is taken
