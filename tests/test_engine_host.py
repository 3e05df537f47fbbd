"""Host side of the step engine without a GPU: the state-slot pool (C++), the scheduler's plan under token, slot and
page limits, the registry's choice by config.json, and the Nisasun configuration reader."""
import json

import numpy as np
import pytest

from mistralrs_b200 import engine, kilizen, nisasun, registry


def test_state_slots_lowest_free_first_and_reuse():
    s = engine.StateSlots(3)
    assert [s.acquire(r) for r in (10, 11, 12)] == [0, 1, 2]
    assert s.acquire(13) == -1 and s.num_free() == 0
    assert s.acquire(11) == 1                       # a known request keeps its slot
    assert s.release(11) and not s.release(11)
    assert s.slot_of(11) == -1 and s.acquire(13) == 1
    s.release(10), s.release(12)
    assert s.acquire(14) == 0 and s.num_free() == 1 and s.capacity() == 3
    with pytest.raises(ValueError):
        engine.StateSlots(0)


class _FakeEngine:
    def __init__(self, slots, pages, page=16):
        self.slots, self.pages, self.page = slots, pages, page

    def pages_needed(self, r, n):
        return -(-(r.n_computed + n) // self.page) - -(-r.n_computed // self.page)

    def free_pages(self):
        return self.pages

    def free_slots(self):
        return self.slots


def _req(rid, n):
    return engine.Request(rid, list(range(n)), n)


def test_scheduler_budget_portions_and_admission():
    sch = engine.Scheduler(max_step_tokens=40)
    a, b, c = _req(1, 100), _req(2, 10), _req(3, 5)
    for r in (a, b, c):
        sch.add(r)
    eng = _FakeEngine(slots=3, pages=100)
    plan = sch.plan(eng)
    assert [(r.rid, n) for r, n in plan] == [(1, 40)]              # the budget cuts the first prompt into portions
    a.n_computed = 40
    plan = sch.plan(eng)
    assert [(r.rid, n) for r, n in plan] == [(1, 40)] and list(sch.waiting) == [b, c]
    a.n_computed = 80
    plan = sch.plan(eng)
    assert [(r.rid, n) for r, n in plan] == [(1, 20), (2, 10), (3, 5)]   # running first, then admissions while the budget lasts
    sch3 = engine.Scheduler(max_step_tokens=100)
    for i in range(4):
        sch3.add(_req(20 + i, 20))
    assert [r.rid for r, _ in sch3.plan(_FakeEngine(slots=2, pages=100))] == [20, 21]   # one plan never promises a slot twice
    assert [r.rid for r, _ in sch3.plan(_FakeEngine(slots=2, pages=1))] == []           # ... nor a page (running ones need none here)
    eng.slots = 0
    sch2 = engine.Scheduler(max_step_tokens=40)
    sch2.add(_req(4, 3))
    assert sch2.plan(eng) == []                                     # no state slot: nothing is admitted
    eng.slots, eng.pages = 1, 0
    assert sch2.plan(eng) == []                                     # no page either
    a.n_computed, a.tokens = 100, a.tokens + [7]
    eng.pages = 1
    assert [(r.rid, n) for r, n in sch.plan(eng)][0] == (1, 1)      # a decoded token is a portion of one


def test_registry_picks_by_config(tmp_path):
    assert "Nisasun" in registry.registered() and "Kilizen" in registry.registered() and "LlamaForCausalLM" in registry.registered()
    assert registry.architecture_of({"architecture": "Nisasun"}) == "Nisasun"
    assert registry.architecture_of({"architectures": ["LlamaForCausalLM"], "model_type": "llama"}) == "LlamaForCausalLM"
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Unheard"}))
    with pytest.raises(NotImplementedError):
        registry.load_model(str(tmp_path), "cpu", None)


def test_config_reader_shapes_and_branches():
    cj = {"architecture": "Nisasun", "vocab": 50, "width": 24, "streams": 2, "norm": {"eps": 1e-6}, "layers": [
        {"type": "lightning", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.5, 0.9]}, "mlp": None},
        {"type": "parallel", "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 3, "top": 1, "groups": {"count": 1, "keep": 1}}},
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 4, "mask": {"size": 5}, "scale": 0.4},
                   "right": {"heads": 2, "vdim": 8, "state": 4, "groups": 1, "norm_groups": 2, "conv": 3}, "left_scale": 1.0, "right_scale": 1.0}}]}
    cfg = nisasun.NisasunConfig(cj)
    sh = cfg.tensor_shapes()
    assert "l0.norm2" not in sh and "l0.hc2.mix" not in sh and sh["l0.hc1.mix"] == (2, 2)
    assert sh["l0.mix.q"] == (8, 24) and sh["l0.mix.v"] == (12, 24) and sh["l0.mix.o"] == (24, 12)
    assert sh["l1.mix.left.k"] == (12, 24) and sh["l1.mix.left.v"] == (8, 24) and sh["l1.mix.left.o"] == (24, 16)
    assert sh["l1.mix.right.in"] == (2 * 16 + 2 * 4 + 2, 24) and sh["l1.mix.right.conv"] == (24, 3)
    assert sh["l1.mlp.e2.down"] == (24, 10) and sh["l1.mlp.router"] == (3, 24) and sh["l1.mlp.correction"] == (3,)
    t = nisasun.random_tensors(cfg, 0)
    assert set(t) == set(sh) and all(tuple(t[k].shape) == tuple(v) for k, v in sh.items())
    for bad in ({"type": "other"}, {"mlp": {"kind": "sparse"}}):
        c2 = json.loads(json.dumps(cj))
        c2["layers"][0].update(bad)
        with pytest.raises(NotImplementedError):
            nisasun.NisasunConfig(c2)


def test_kilizen_config_reader_shapes_order_and_branches():
    cj = {"architecture": "Kilizen", "vocab": 50, "width": 24, "norm": {"eps": 1e-6}, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
        {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4, "rot": {"base": 100.0, "dims": 4}}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "dim": 8, "vdim": 8, "scale": 0.3, "mask": {"size": 5, "keep_first": 2}},
         "mlp": {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 3, "top": 1}, "shared": {"ff": 7}}},
        {"type": "mlstm", "mixer": {"heads": 3, "dim": 4, "vdim": 6, "gate_cap": 9.0}, "mlp": {"kind": "dense", "ff": 30}}]}
    cfg = kilizen.KilizenConfig(cj)
    assert cfg.runs() == [(0, False), (1, False), (2, False), (1, True), (2, False)]
    sh = cfg.tensor_shapes()
    assert "l0.norm2" not in sh and sh["l0.norm1b.alpha"] == () and sh["final.norm.b"] == (24,)
    assert sh["l0.mix.q"] == (24, 24) and sh["l0.mix.k.b"] == (12,) and sh["l0.mix.v"] == (20, 24) and sh["l0.mix.q.norm"] == (24,) and sh["l0.mix.o"] == (24, 40)
    assert sh["l1.mix.k"] == (16, 24) and sh["l1.mix.k.norm"] == (8,) and "l1.mix.v" not in sh and sh["l1.mix.sink"] == (2,)   # no kv_heads entry: one per head
    assert sh["l1.mlp.e2.down"] == (24, 10) and sh["l1.mlp.shared.up"] == (7, 24) and sh["l1.mlp.router"] == (3, 24)
    assert sh["l2.mix.i"] == (3, 24) and sh["l2.mix.f.b"] == (3,) and sh["l2.mix.norm"] == (18,) and sh["l2.mlp.up"] == (30, 24)
    t = kilizen.random_tensors(cfg, 0)
    assert set(t) == set(sh) and all(tuple(t[k].shape) == tuple(v) for k, v in sh.items())
    for bad in ({"type": "other"}, {"mlp": {"kind": "sparse"}}):
        c2 = json.loads(json.dumps(cj))
        c2["layers"][0].update(bad)
        with pytest.raises(NotImplementedError):
            kilizen.KilizenConfig(c2)
    c2 = json.loads(json.dumps(cj))
    c2["loop"] = {"start": 2, "stop": 5, "times": 2}
    with pytest.raises(ValueError):
        kilizen.KilizenConfig(c2)


def test_step_batch_layout_cpu():
    b = engine.StepBatch("cpu", [5, 6, 7, 8], [3, 1], [0, 9], [1, 0], [[2], [4, 5]], np.array([32, 33, 34, 89], dtype=np.int64), [2, 3])
    assert b.cu_tok.tolist() == [0, 3, 4] and b.seq_of_tok.tolist() == [0, 0, 0, 1] and b.pos_of_tok.tolist() == [0, 1, 2, 9]
    assert b.pages.tolist() == [[2, 0], [4, 5]] and b.slot_of_tok.tolist() == [32, 33, 34, 89] and b.rows.tolist() == [2, 3]
    assert b.past.tolist() == [0, 9] and b.slot.tolist() == [1, 0] and b.ids.tolist() == [5, 6, 7, 8]
    many = engine.StepBatch("cpu", [0] * 76, [40, 1, 35], [0, 9, 0], [1, 0, 2], [[2, 3, 6], [4], [7, 8, 9]], np.arange(76, dtype=np.int64), [])
    assert many.fresh == [(0, 40), (41, 35)] and many.paged_tok.tolist() == [40]
    assert many.long == [(0, 40, 0, 0), (41, 35, 0, 2)] and many.long_rows.tolist() == [0, 40, 0, 0, 41, 35, 0, 2] and many.short_tok.tolist() == [40]
    cont = engine.StepBatch("cpu", [0] * 36, [33, 3], [20, 0], [1, 0], [[2, 3, 6, 7], [4]], np.arange(36, dtype=np.int64), [])
    assert cont.fresh == [] and cont.long == [(0, 33, 20, 0)] and cont.short_tok.tolist() == [33, 34, 35] and cont.paged_tok.numel() == 36
