"""Kuzupel without a GPU: the configuration reader, the model spec, the cache manager's groups with kept first
pages, the launch plan's chunk counts, and the plain implementation's own mechanisms on cases worked by hand."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import kuzupel_cases as cases
import plain_kuzupel as plain
from snowllm_b200.cache import CacheManager
from snowllm_b200.config.registry import resolve
from snowllm_b200.errors import ConfigError
from snowllm_b200.loader import build_model
from snowllm_b200.parts.spec import PagedKVSpec, SlotStateSpec


def test_config_reads_back_and_builds_the_parts():
    model = build_model(cases.MIXED, "float32")
    cfg = model.config
    assert resolve(["Kuzupel"]).read_config(cfg.to_json_dict()) == cfg
    kinds = [(type(b.mixer).__name__, type(b.ffn).__name__ if b.ffn is not None else None) for b in model.blocks]
    assert kinds == [("ConvGateAttention", "GatedFFN"), ("SlopeAttention", "SigmoidMoE"), ("ConvGateAttention", "SigmoidMoE"),
                     ("SlopeAttention", None), ("ConvGateAttention", "SigmoidMoE")]
    assert all(b.residual_scale == 0.6 for b in model.blocks)
    specs = model.cache_specs()
    assert specs[model.EMBEDDING_CACHE] == SlotStateSpec(((),), ("i32",))
    pages, state = specs[0]
    assert pages == PagedKVSpec(1, 16, 13, 8, separate=True, keep_first=3) and pages.reach == (13, 3)
    assert state == SlotStateSpec(((2, 3 * 16 + 16 + 8),), ("compute",))
    assert specs[1].reach == 21 and specs[4][0].reach == (19, 1)
    names = {spec.name for _, spec in model.declare(lambda n: False)}
    assert {"embed", "bigram", "l0.mix.q.conv", "l0.mix.g", "l1.mix.q.norm", "l1.mlp.router.b", "l1.mlp.shared.sg",
            "l1.mlp.e4.down", "l0.mlp.gate", "final.norm", "head"} <= names
    assert "l3.norm2" not in names and "l2.mlp.shared.sg" not in names
    shapes = {spec.name: spec.shape for _, spec in model.declare(lambda n: False)}
    assert shapes["l1.mix.q.norm"] == (4 * 12,) and shapes["l1.mix.k.norm"] == (2 * 12,)     # over the whole projection
    assert shapes["l0.mix.q.norm"] == (16,) and shapes["bigram"] == (54, 40) and shapes["l0.mix.g"] == (3, 40)


def test_what_a_file_leaves_out_is_off():
    cfg = cases.config([cases.conv_layer(window=None, keep_first=None, conv=None, rot_dims=0, mlp=None)], mult=None,
                       cap=None, pair=None)
    del cfg["embedding"]
    model = build_model(cfg, "float32")
    c = model.config
    assert (c.residual_mult, c.logit_softcap, c.embedding_scale, c.pair_table) == (1.0, None, 1.0, None)
    assert type(model.embedding).__name__ == "Embedding" and model.head.softcap is None
    mixer = model.blocks[0].mixer
    assert mixer.window is None and mixer.keep_first == 0 and mixer.conv_taps == 0
    assert model.cache_specs() == {0: PagedKVSpec(1, 16, None, 8, separate=True)}


def test_config_errors_name_every_key():
    cfg = copy.deepcopy(cases.MIXED)
    del cfg["vocab"]
    cfg["layers"][0]["mixer"]["rot"]["dims"] = 7
    cfg["layers"][1]["mlp"]["router"]["top"] = 9
    cfg["layers"][2]["mixer"]["conv"] = 40
    cfg["layers"][3]["type"] = "attention_3"
    cfg["embedding"]["bigram"].pop("mul_cur")
    with pytest.raises(ConfigError) as e:
        build_model(cfg, "float32")
    for part in ("vocab", "rot.dims=7", "top=9", "conv=40", "attention_3", "embedding.bigram.mul_cur"):
        assert part in str(e.value), part
    bad = cases.config([cases.conv_layer(window=None, keep_first=4)])
    bad["layers"][0]["mixer"]["mask"] = {"keep_first": 4}
    with pytest.raises(ConfigError):
        build_model(bad, "float32")


def test_cache_manager_keeps_the_first_pages_and_gives_back_the_rest():
    specs = {0: PagedKVSpec(1, 8, 10, 8, separate=True, keep_first=9), 1: PagedKVSpec(1, 8, 10, 8, separate=True)}
    cache = CacheManager(specs, 4, 12, 2, torch.float32, device=None)
    kept, plain_window = ("paged", (10, 9)), ("paged", 10)
    assert set(cache.groups) == {kept, plain_window}
    rc = cache.admit()
    assert cache.ensure(rc, 30)
    cache.commit(rc, 30)
    # a query at 30 or later reaches positions 21..: entries 0..4 are behind the window, 0..2 hold kept positions
    assert [p >= 0 for p in rc.tables[kept]] == [True, True, True, False, False, True, True, True]
    assert [p >= 0 for p in rc.tables[plain_window]] == [False] * 5 + [True] * 3
    assert cache.groups[kept].held() == 6 and cache.groups[plain_window].held() == 3
    assert cache.missing_pages(rc, 34) == {kept: 1, plain_window: 1}
    assert cache.ensure(rc, 47)
    cache.commit(rc, 47)
    assert [p >= 0 for p in rc.tables[kept]] == [True] * 3 + [False] * 6 + [True] * 3
    cache.free(rc)
    assert all(pool.held() == 0 for pool in cache.groups.values())
    # a request that comes back after a preemption with many tokens at once: the kept entries and the window's
    rc = cache.admit()
    cache.commit(rc, 0)
    assert cache.ensure(rc, 3) and cache.missing_pages(rc, 3) == {kept: 0, plain_window: 0}
    cache.commit(rc, 3)
    assert cache.missing_pages(rc, 40) == {kept: 9, plain_window: 9}
    # the pool cannot hold more than it has: nothing is taken
    other = cache.admit()
    assert cache.ensure(other, 40) and not cache.ensure(rc, 40)
    assert len(rc.tables[kept]) == 1


def test_chunk_plan_counts_kept_chunks():
    import numpy as np
    from snowllm_b200.parts import attention_plan as plan

    class Ctx:
        capture_max_len = None
        memo = {}

        def __init__(self, positions):
            self.host_positions = np.asarray(positions, dtype=np.int64)

    def by_hand(pos, window, keep, chunk):
        lo = max(0, pos - window + 1)
        return -(-min(keep, lo) // chunk) + pos // chunk - lo // chunk + 1
    for window, keep, chunk in ((40, 6, 128), (21, 150, 128), (300, 700, 256), (5, 0, 128)):
        for positions in ([0], [5, 127, 128, 129], [1000, 3], [149, 150, 170, 171, 299]):
            want = max(by_hand(p, window, keep, chunk) for p in positions)
            assert plan.chunks(Ctx(positions), window, None, chunk, keep=keep) == want
    captured = Ctx([0])
    captured.capture_max_len = 1024
    assert plan.chunks(captured, 21, None, 128, keep=150) == 8 + 2


# --- the plain implementation's own mechanisms ------------------------------------------------------

def test_plain_mask_and_softmax_by_hand():
    m = plain.window_mask(8, 3, 2)
    assert m[7].tolist() == [True, True, False, False, False, True, True, True]
    assert m[2].tolist() == [True, True, True, False, False, False, False, False]
    assert plain.window_mask(8, 3)[7].tolist() == [False] * 5 + [True] * 3
    s = torch.tensor([[0.0, 1.0, 2.0]], dtype=torch.float64)
    p = plain.masked_softmax(s, torch.tensor([[True, True, False]]), one_more=True)
    assert torch.allclose(p, torch.tensor([[1.0, math.e, 0.0]], dtype=torch.float64) / (2 + math.e))
    p = plain.masked_softmax(s - 50, torch.tensor([[True, True, True]]), one_more=True)
    assert float(p.sum()) < 1e-20 * 1e3 or float(p.sum()) < 1e-15              # the extra term takes everything


def test_plain_conv_hash_and_cap_by_hand():
    u = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 10.0, 100.0]], dtype=torch.float64)
    assert plain.causal_taps(u, w).flatten().tolist() == [100.0, 210.0, 320.5, 431.0]
    assert plain.hashed_pair_rows([3, 4, 4], 7, 5, 2).tolist() == [7, (15 + 8) % 7, (20 + 8) % 7]
    assert plain.hashed_pair_rows([9], 7, 5, 2).tolist() == [7]
    z = torch.tensor([0.0, 1.0, -1000.0], dtype=torch.float64)
    assert torch.allclose(plain.soft_cap(z, 4.0), torch.tensor([0.0, 4 * math.tanh(0.25), -4.0], dtype=torch.float64))
    assert plain.soft_cap(z, None) is z


def test_plain_router_weights_and_shared_gate():
    t = {"r.router": torch.tensor([[1.0], [2.0], [0.5]], dtype=torch.float64),
         "r.router.b": torch.tensor([0.0, -3.0, 0.2], dtype=torch.float64)}
    for e in range(3):
        t[f"r.e{e}.gate"] = torch.full((2, 1), 1.0 + e, dtype=torch.float64)
        t[f"r.e{e}.up"] = torch.full((2, 1), 0.5, dtype=torch.float64)
        t[f"r.e{e}.down"] = torch.ones(1, 2, dtype=torch.float64)
    mlp = {"router": {"experts": 3, "top": 2}, "expert": {"limit": 10.0}}
    h = torch.tensor([[1.0]], dtype=torch.float64)
    out, picks = plain.picked_softmax_experts(h, t, mlp, "r.")
    assert picks.tolist() == [[0, 2]]                                # logits 1.0, -1.0, 0.7: the bias changed the choice
    w = torch.softmax(torch.tensor([1.0, 0.7], dtype=torch.float64), -1)
    each = [2 * (g * torch.sigmoid(torch.tensor(1.702 * g, dtype=torch.float64)) * 1.5) for g in (1.0, 3.0)]
    assert torch.allclose(out, (w[0] * each[0] + w[1] * each[1]).view(1, 1))
