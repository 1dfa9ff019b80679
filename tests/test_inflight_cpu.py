"""Host-side logic of the in-flight runtime (no GPU): page and slot bookkeeping, the scheduler's plans, the checkpoint
reader, the model registry, and the oracle's own consistency (whole sequence against a prefix)."""
import json

import pytest
import torch

from oracle import seq_mixers as O


def test_kv_manager_reserve_release_reuse():
    from trtllm_llama_b200.runtime import GenerationSequence, KVCacheManager
    m = KVCacheManager(blocks=6, tokens_per_block=16, max_blocks_per_seq=6)
    a, b = GenerationSequence(0, 0), GenerationSequence(1, 1)
    assert m.reserve(a, 17) and len(m.blocks_of(a)) == 2
    assert not m.reserve(a, 32) and m.reserve(a, 33) and len(m.blocks_of(a)) == 3
    m.reserve(b, 48)
    assert not m.has_free_block()
    with pytest.raises(RuntimeError):
        m.reserve(a, 49)
    assert len(m.blocks_of(a)) == 3, "a refused reservation must not change the sequence"
    held = set(m.blocks_of(b))
    m.release(b)
    c = GenerationSequence(2, 1)
    m.reserve(c, 40)
    assert set(m.blocks_of(c)) <= held and set(m.blocks_of(c)).isdisjoint(m.blocks_of(a))


def test_slot_manager():
    from trtllm_llama_b200.inflight import StateSlotManager
    s = StateSlotManager(2)
    x, y = s.acquire(), s.acquire()
    with pytest.raises(RuntimeError):
        s.acquire()
    s.release(x)
    assert s.acquire() == x and {x, y} == {0, 1}


class _FakeSession:
    def __init__(self, blocks, slots, page=16):
        from trtllm_llama_b200.inflight import StateSlotManager
        from trtllm_llama_b200.runtime import KVCacheManager
        self.kv_cache_manager = KVCacheManager(blocks, page, blocks)
        self.slot_manager = StateSlotManager(slots)
        self.ended = []

    def end(self, seq_id):
        self.ended.append(seq_id)


def test_scheduler_budget_admission_and_order():
    from trtllm_llama_b200.inflight import InflightScheduler
    s = _FakeSession(blocks=8, slots=2)
    sch = InflightScheduler(s, max_step_tokens=10)
    sch.add("a", list(range(25)), 4)       # 2 pages
    sch.add("b", list(range(3)), 4)        # 1 page
    sch.add("c", list(range(90)), 6)       # 6 pages: has to wait for a slot, then fits beside what is left
    fed = {"a": 0, "b": 0, "c": 0}
    seen_c_before_a_done = False
    for _ in range(200):
        if not sch.busy():
            break
        entries, sampled = sch.schedule()
        assert sum(len(e[1]) for e in entries) <= 10 and len(entries) <= 2
        for sid, toks, want in entries:
            fed[sid] += len(toks)
            assert want in ([], [len(toks) - 1])
        if any(e[0] == "c" for e in entries) and "a" not in s.ended and "b" not in s.ended:
            seen_c_before_a_done = True
        assert [r.seq_id for r in sampled] == [e[0] for e in entries if e[2]]
        sch.accept(sampled, [1] * len(sampled))
    assert not sch.busy() and not seen_c_before_a_done
    assert set(s.ended) == {"a", "b", "c"} and sch.promised == 0
    assert [len(sch.finished[k]) for k in "abc"] == [4, 4, 6]
    assert fed == {"a": 25 + 3, "b": 3 + 3, "c": 90 + 5}


def test_scheduler_stops_at_end_id_and_rejects_oversized():
    from trtllm_llama_b200.inflight import InflightScheduler
    s = _FakeSession(blocks=2, slots=2)
    sch = InflightScheduler(s, 64)
    sch.add("a", [1, 2, 3], 10)
    entries, sampled = sch.schedule()
    sch.accept(sampled, [9], end_id=9)
    assert sch.finished["a"] == [9] and not sch.busy()
    sch.add("big", list(range(40)), 10)
    with pytest.raises(RuntimeError):
        sch.schedule()


def test_checkpoint_roundtrip_and_registry(tmp_path):
    from trtllm_llama_b200 import models
    from trtllm_llama_b200.checkpoint import read_safetensors, write_safetensors
    t = {"a.b": torch.randn(3, 5).to(torch.bfloat16), "c": torch.arange(7, dtype=torch.int32), "d": torch.randn(2, 2, 2)}
    write_safetensors(str(tmp_path / "x.safetensors"), t)
    back = read_safetensors(str(tmp_path / "x.safetensors"))
    assert set(back) == set(t) and all(back[k].dtype == t[k].dtype and torch.equal(back[k], t[k]) for k in t)
    assert "zobasun" in models.registered_models() and "llama" in models.registered_models()
    assert models.architecture_of({"architecture": "Zobasun"}) == "Zobasun"
    assert models.architecture_of({"builder_config": {}}) == "llama"
    with open(tmp_path / "config.json", "w") as f:
        json.dump({"architecture": "NoSuchModel"}, f)
    with pytest.raises(ValueError):
        models.load_model(str(tmp_path))


def test_model_definition_checks_its_config():
    from trtllm_llama_b200.models.zobasun import build_zobasun
    att = dict(type="latent_attention", heads=2, dim=4, rot_dim=4, vdim=4, kv_rank=8, q_rank=8, mlp=None)
    cfg, t = O.random_zobasun([att, dict(att, kv_from=0)], width=16, vocab=20)
    cfg["layers"][1]["mixer"]["kv_rank"] = 12          # a reader of another layer's cache must have its geometry
    with pytest.raises(ValueError):
        build_zobasun(cfg, t, torch.float32, "cpu")
    cfg, t = O.random_zobasun([att], width=16, vocab=20)
    del t["l0.mix.uk"]
    with pytest.raises(KeyError):
        build_zobasun(cfg, t, torch.float32, "cpu")


def test_oracle_is_causal_and_stateless():
    """The oracle on a prefix equals the oracle on the whole sequence, cut: nothing leaks backwards."""
    att = dict(type="latent_attention", heads=2, dim=6, rot_dim=4, vdim=5, kv_rank=12, q_rank=8, mlp=(20, 1.0))
    rec = dict(type="rglru", width=12, blocks=2, conv=3, mlp=None)
    cfg, t = O.random_zobasun([rec, att, dict(att, kv_from=1)], width=16, vocab=23, seed=1)
    toks = list(range(1, 20))
    full, part = O.zobasun_forward(cfg, t, toks), O.zobasun_forward(cfg, t, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-12)
    # the recurrence's first step starts from zero: output at position 0 does not depend on anything else
    one = O.zobasun_forward(cfg, t, toks[:1])
    assert torch.allclose(full[:1], one, atol=1e-12)
