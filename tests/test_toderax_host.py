"""Toderax on the host: configuration, model spec, declared tensors, the cache book-keeping of its block-local
groups and state slots, and the plain implementation's own properties.  No GPU."""
from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import plain_toderax as plain
import toderax_cases as cases
from snowllm_b200.cache import CacheManager
from snowllm_b200.config.registry import architectures, read_config_json
from snowllm_b200.config.toderax import read_toderax_config
from snowllm_b200.errors import ConfigError, WeightError
from snowllm_b200.loader import build_model
from snowllm_b200.parts.spec import PagedKVSpec, SlotStateSpec, first_reachable
from snowllm_b200.weights.loader import load_tensors


def test_architecture_is_registered_and_read_by_its_single_name(tmp_path):
    assert "Toderax" in architectures()
    (tmp_path / "config.json").write_text(json.dumps(cases.MIXED))
    arch, cfg, _ = read_config_json(tmp_path)
    assert arch.name == "Toderax" and cfg.width == cases.MIXED["width"] and len(cfg.layers) == 5
    assert read_toderax_config(cfg.to_json_dict()) == cfg           # the written form reads back
    assert cfg.streams == 3 and cfg.norm_groups == 5 and cfg.embedding_scale == 3.0
    assert cfg.layers[0].mlp == {"ff": 24, "limit": 1.2, "experts": 5, "top": 2, "shared": {"ff": 16, "limit": 0.8}}
    assert cfg.layers[2].mlp["shared"] is None and cfg.layers[3].mlp is None
    assert cfg.layers[0].mixer["left"]["block"] == 21 and cfg.layers[4].mixer["right"]["decay"] == [1.0, 0.5]


def test_what_a_configuration_leaves_out_is_off():
    cfg = cases.config([cases.pair_layer(chunk=None, rot_dims=0), cases.memory_layer(mlp=None)], streams=None)
    del cfg["norm"]["groups"]
    del cfg["embedding"]
    c = read_toderax_config(cfg)
    assert c.streams is None and c.norm_groups == 1 and c.embedding_scale == 1.0
    assert c.layers[0].mixer["left"]["block"] is None and c.layers[0].mixer["right"]["rot"] is None
    assert read_toderax_config(c.to_json_dict()) == c
    model = build_model(cfg, "float32")
    assert model.blocks[0].streams == 1 and model.blocks[0].hc is None
    assert model.blocks[0].mixer.left.block is None
    assert type(model.blocks[0].mixer.right.position).__name__ != "RotaryPosition"
    assert not any(".hc" in s.name for _, s in model.declare(lambda n: False))


def test_every_problem_of_a_configuration_is_listed_at_once():
    bad = copy.deepcopy(cases.MIXED)
    del bad["width"]
    bad["streams"] = 9
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3               # 4 heads over 3 kv heads
    bad["layers"][0]["mixer"]["right"]["decay"] = [0.5]             # three heads
    bad["layers"][1]["mixer"].pop("vdim")
    bad["layers"][2]["mlp"]["router"]["top"] = 9                    # more picks than experts
    bad["layers"][3]["type"] = "conv"
    bad["layers"][4]["mixer"]["right"]["rot"]["dims"] = 7
    with pytest.raises(ConfigError) as e:
        read_toderax_config(bad)
    text = str(e.value)
    for piece in ("width", "streams=9", "kv_heads=3", "decay=[0.5]", "vdim", "top=9", "'conv'", "rot.dims=7"):
        assert piece in text, (piece, text)
    bad = copy.deepcopy(cases.MIXED)
    bad["norm"]["groups"] = 3                                       # does not divide the width
    bad["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(ConfigError) as e:
        read_toderax_config(bad)
    assert "groups=3" in str(e.value) and "'dense'" in str(e.value)


def test_model_spec_names_the_parts_and_their_caches():
    model = build_model(cases.MIXED, "float32")
    assert all(layer.block == "hyper" for layer in model.spec.layers)
    assert [type(b.mixer).__name__ for b in model.blocks] == ["SideBySide", "Hgrn2", "SideBySide", "Hgrn2", "SideBySide"]
    specs = model.cache_specs()
    # a pair keeps pages for its attention (the current block of positions only) and a float state for its memory
    assert specs[0] == (PagedKVSpec(2, 12, None, 20, separate=True, block=21), SlotStateSpec(((3, 16, 8),), ("f32",)))
    assert specs[0][0].reach == -21 and specs[1] == SlotStateSpec(((3, 8, 12),), ("f32",))
    assert specs[4][1] == SlotStateSpec(((2, 12, 12),), ("f32",))
    pair = model.blocks[2].mixer
    assert pair.left.block == 33 and pair.left.num_heads == pair.left.num_kv_heads == 3 and pair.left.scale == 0.7
    assert pair.right.decay_values == [0.97] and pair.mix == (0.5, 0.5)
    assert model.blocks[4].mixer.right.position.rot_dim == 4 and model.blocks[4].mixer.right.head_dim == 12
    ffn = model.blocks[0].ffn
    assert (ffn.scoring, ffn.activation, ffn.limit, ffn.top_k, ffn.num_experts) == ("softmax", "swish_clamp", 1.2, 2, 5)
    assert not ffn.norm_topk_prob and ffn.shared == {"intermediate_size": 16, "limit": 0.8}
    assert model.blocks[2].ffn.shared is None and model.blocks[3].ffn is None
    assert len(model.blocks[0].hc) == 2 and len(model.blocks[3].hc) == 1 and model.blocks[0].streams == 3
    assert model.blocks[0].mixer_norm.groups == 5 and model.final_norm.groups == 5
    assert model.embedding.scale == 3.0


def test_declared_tensors_and_their_names():
    model = build_model(cases.MIXED, "float32")
    names = {s.name: s for _, s in model.declare(lambda n: False)}
    assert names["l0.mix.left.q"].shape == (4 * 12, 40) and names["l0.mix.left.k"].shape == (2 * 12, 40)
    assert names["l0.mix.left.v.b"].shape == (2 * 20,) and names["l0.mix.left.o"].shape == (40, 4 * 20)
    assert names["l0.mix.left.temp"].shape == names["l0.mix.left.sink"].shape == (4,)
    assert names["l0.mix.right.q"].shape == (3 * 16, 40) and names["l0.mix.right.g"].shape == (3 * 8, 40)
    assert names["l0.mix.left.out"].shape == names["l0.mix.right.out"].shape == (40,)
    assert "l0.mix.right.q.b" not in names and "l0.mix.left.q_norm" not in names
    assert names["l1.mix.f"].shape == (3 * 8, 40) and names["l1.mix.lower"].shape == names["l1.mix.f.b"].shape == (24,)
    assert names["l1.mix.norm"].shape == (12,) and names["l1.mix.v"].shape == (36, 40)
    assert names["l0.hc1.mix"].shape == (3, 3) and names["l0.hc2.in"].shape == (3,) and "l3.hc2.in" not in names
    assert {"l0.mlp.router", "l0.mlp.e4.gate", "l0.mlp.shared.down", "l2.mlp.e2.up"} <= set(names)
    assert "l0.mlp.e5.gate" not in names and "l2.mlp.shared.gate" not in names and "l3.norm2" not in names
    assert names["l2.mlp.e0.down"].shape == (40, 16) and names["final.norm"].shape == (40,)
    assert names["head"].shape == (96, 40) and names["embed"].shape == (96, 40)


def test_missing_and_unexpected_tensors_are_listed():
    tensors = cases.draw_weights(cases.MIXED, dtype=torch.float32)
    del tensors["l2.mix.left.sink"]
    tensors["l1.mix.k"] = torch.zeros(24, 40)
    with pytest.raises(WeightError) as e:
        load_tensors(build_model(cases.MIXED, "float32"), tensors, "cpu")
    assert "l2.mix.left.sink" in str(e.value) and "l1.mix.k" in str(e.value)


def test_first_reachable_position_under_a_window_a_block_and_neither():
    assert [first_reachable(None, p) for p in (0, 5, 500)] == [0, 0, 0]
    assert [first_reachable(7, p) for p in (0, 6, 7, 20)] == [0, 0, 1, 14]
    assert [first_reachable(-7, p) for p in (0, 6, 7, 13, 14, 20)] == [0, 0, 7, 7, 14, 14]
    with pytest.raises(ValueError):
        PagedKVSpec(1, 8, 5, 8, block=4).reach


def test_block_local_groups_give_pages_back_and_slots_are_used_again():
    model = build_model(cases.MIXED, "float32")
    cache = CacheManager(model.cache_specs(), 8, 12, 2, torch.float32, device=None)
    assert set(cache.groups) == {("paged", -21), ("paged", -33), ("paged", -19)}
    a = cache.admit()
    assert cache.ensure(a, 50)
    cache.commit(a, 50)
    for (_, reach), table in a.tables.items():
        first = (50 - 50 % -reach) // 8                             # the page of the current block's first position
        assert all(p < 0 for p in table[:first]) and all(p >= 0 for p in table[first:7]), (reach, table)
    held = {k: p.held() for k, p in cache.groups.items()}
    assert held[("paged", -21)] == 7 - 42 // 8 and held[("paged", -33)] == 7 - 33 // 8
    b = cache.admit()
    assert cache.ensure(b, 40)
    cache.commit(b, 40)
    assert cache.admit() is None                                   # two slots
    cache.free(a)
    c = cache.admit()
    assert c is not None and c.slot == a.slot                      # the slot is used again
    assert cache.ensure(c, 30)
    cache.free(b)
    cache.free(c)
    assert all(p.held() == 0 for p in cache.groups.values())
    # a long request never holds more pages than one block spans (plus the page it shares with the next)
    d = cache.admit()
    for total in range(16, 400, 16):
        assert cache.ensure(d, total)
        cache.commit(d, total)
        assert cache.groups[("paged", -19)].held() <= 19 // 8 + 3
    cache.free(d)


def test_plain_mask_softmax_and_rotation():
    m = plain.same_chunk_causal(12, 5)
    assert bool(m[4, 0]) and not bool(m[5, 4]) and bool(m[9, 5]) and not bool(m[9, 4]) and not bool(m[3, 4])
    assert bool(plain.same_chunk_causal(12, None)[11, 0])
    # the sink: with one visible key of score s the weight is e^s / (e^s + e^sink), counted once
    p = plain.softmax_with_sink(torch.tensor([[0.7, 5.0]], dtype=torch.float64), torch.tensor([[True, False]]),
                                torch.tensor(-0.2, dtype=torch.float64))
    assert float(p[0, 0]) == pytest.approx(math.exp(0.7) / (math.exp(0.7) + math.exp(-0.2)), rel=1e-12)
    assert float(p[0, 1]) == 0.0
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 10, generator=g).double(), torch.randn(1, 1, 10, generator=g).double()

    def at(x, pos):
        return plain.rotate_halves(x, torch.tensor([pos]), 300.0, 6)
    assert torch.equal(at(q, 7)[..., 6:], q[..., 6:])                           # the rest passes unchanged
    assert float(((at(q, 40) * at(k, 33)).sum() - (at(q, 107) * at(k, 100)).sum()).abs()) < 1e-12
    e0 = torch.zeros(1, 1, 6).double()
    e0[..., 0] = 1                                                              # element 0 turns with element 3
    got = at(e0, 1)[0, 0]
    assert float(got[0]) == pytest.approx(math.cos(1.0)) and float(got[3]) == pytest.approx(math.sin(1.0))
    assert float(got[1]) == 0.0


def test_plain_memories_streams_and_experts():
    g = torch.Generator().manual_seed(2)
    T, d, dv = 9, 4, 3
    q, k, v = (torch.randn(T, n, generator=g).double() for n in (d, d, dv))
    # a fixed decay: o_t = sum_j decay^(t - j) (q_t . k_j) v_j
    out = plain.decayed_memory(q, k, v, torch.full((T, d), 0.8, dtype=torch.float64))
    want = sum(0.8 ** (8 - j) * (q[8] @ k[j]) * v[j] for j in range(T))
    assert torch.allclose(out[8], want, atol=1e-12)
    # a gate of one keeps the state, a gate of zero forgets it
    a = torch.ones(T, d, dtype=torch.float64)
    a[5] = 0
    out = plain.decayed_memory(q, k, v, a)
    assert torch.allclose(out[8], sum((q[8] @ k[j]) * v[j] for j in range(5, T)), atol=1e-12)
    # streams: identity mix, ones in and out, one stream: the plain residual sum
    x = torch.randn(T, 6, generator=g).double()
    t = {"in": torch.ones(1).double(), "out": torch.ones(1).double(), "mix": torch.ones(1, 1).double()}
    assert torch.allclose(plain.hyper_step([x], t, "", lambda u: 2 * u)[0], 3 * x)
    # the update reads the old streams only: [from, to]
    t = {"in": torch.tensor([1.0, 0.0]).double(), "out": torch.tensor([0.0, 1.0]).double(),
         "mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]]).double()}
    a, b = plain.hyper_step([x, 5 * x], t, "", lambda u: u + 1)
    assert torch.equal(a, torch.zeros_like(x)) and torch.allclose(b, x + (x + 1))
    # norm in groups: one group is the plain norm; each group has a unit mean square of its own
    w = torch.ones(6).double()
    assert torch.allclose(plain.group_rms_norm(x, w, 1, 0.0), plain.rms(x, 0.0))
    parts = plain.group_rms_norm(x * torch.tensor([1, 1, 50, 50, 0.1, 0.1]).double(), w, 3, 0.0).view(T, 3, 2)
    assert torch.allclose((parts ** 2).mean(-1), torch.ones(T, 3).double())
    # experts: softmax over all, the largest picked, their scores as they are; the activation's clamps
    h = torch.randn(4, 6, generator=g).double()
    tt = {"router": torch.randn(3, 6, generator=g).double() * 2}
    for e in ("e0.", "e1.", "e2.", "shared."):
        tt.update({e + "gate": torch.randn(5, 6, generator=g).double() * 2, e + "up": torch.randn(5, 6, generator=g).double() * 2,
                   e + "down": torch.randn(6, 5, generator=g).double()})
    mlp = {"expert": {"limit": 0.9}, "router": {"experts": 3, "top": 2}, "shared": {"limit": 0.4}}
    out, picks = plain.routed_experts(h, tt, mlp, "")
    s = torch.softmax(h @ tt["router"].T, -1)
    assert torch.equal(picks, s.topk(2).indices.sort(-1).values)
    row = sum(s[0, e] * plain.clamped_expert(h[:1], tt, f"e{int(e)}.", 0.9)[0] for e in picks[0])
    assert torch.allclose(out[0], row + plain.clamped_expert(h[:1], tt, "shared.", 0.4)[0], atol=1e-12)
    one = {"gate": torch.tensor([[3.0], [-3.0]]).double(), "up": torch.tensor([[-7.0], [0.5]]).double(),
           "down": torch.eye(2).double()}
    y = plain.clamped_expert(torch.ones(1, 1).double(), one, "", 2.0)[0]
    assert float(y[0]) == pytest.approx(2.0 / (1 + math.exp(-1.702 * 2.0)) * (-2.0 + 1))
    assert float(y[1]) == pytest.approx(-3.0 / (1 + math.exp(1.702 * 3.0)) * 1.5)


def test_plain_implementation_is_causal_and_its_chunks_start_at_position_zero():
    cfg = cases.config([cases.pair_layer(chunk=9, mlp=None)])
    tensors = {k: v.double() for k, v in cases.draw_weights(cfg, dtype=torch.float32).items()}
    for name in list(tensors):                    # silence the memory: only the attention passes tokens on
        if name.endswith("right.out"):
            tensors[name] = torch.zeros_like(tensors[name])
    toks = cases.tokens_for(cfg, 40)
    base = cases.plain_logits(cfg, tensors, toks)
    assert torch.equal(cases.plain_logits(cfg, tensors, toks[:25]), base[:25])      # causal
    other = list(toks)
    other[35] = (other[35] + 1) % cfg["vocab"]                     # the last position of the chunk before 36..44
    assert torch.equal(cases.plain_logits(cfg, tensors, other)[36:], base[36:])
    other = list(toks)
    other[36] = (other[36] + 1) % cfg["vocab"]                     # the first position of the last row's chunk
    assert not torch.equal(cases.plain_logits(cfg, tensors, other)[-1], base[-1])


def test_command_line_writes_a_model_folder_that_the_loader_accepts(tmp_path):
    from snowllm_b200 import cli
    from snowllm_b200.weights.loader import check_against
    from snowllm_b200.weights.safetensors_io import Checkpoint
    src = tmp_path / "config.json"
    src.write_text(json.dumps(cases.MIXED))
    out = tmp_path / "model"
    assert cli.main(["random-weights", str(src), str(out), "--seed", "3"]) == 0
    arch, cfg, _ = read_config_json(out)
    assert arch.name == "Toderax" and cfg == read_toderax_config(cases.MIXED)
    model = build_model(out, "bfloat16")
    ck = Checkpoint(out)
    try:
        check_against([s for _, s in model.declare(ck.has)], ck.names(), ck.meta)
        assert tuple(ck.meta("l0.hc1.mix")[1]) == (3, 3) and tuple(ck.meta("l2.mix.left.sink")[1]) == (3,)
    finally:
        ck.close()


def test_bench_design_option_builds_both_models_at_equal_size():
    import bench
    name, ours_of, (other, theirs_of), _ = bench.DESIGNS["toderax"]
    assert name == "Toderax" and other == "lfm2_moe_hybrid"
    for width, layers, ff in bench.DESIGN_SIZES.values():
        ours = build_model(ours_of(width, layers, ff), "bfloat16")
        theirs = build_model(theirs_of(width, layers, ff), "bfloat16")
        assert len(ours.run) == len(theirs.run) == layers
        assert ours.spec.hidden_size == theirs.spec.hidden_size == width
        for mine, other_block in zip(ours.blocks, theirs.blocks):
            pair = type(mine.mixer).__name__ == "SideBySide"
            assert pair == (type(other_block.mixer).__name__ == "Attention")
            if pair:
                assert mine.mixer.left.num_heads == other_block.mixer.num_heads
                assert mine.mixer.left.num_kv_heads == other_block.mixer.num_kv_heads
                assert all(0 < d < 1 for d in mine.mixer.right.decay_values)
        routed, theirs_routed = ours.blocks[1].ffn, theirs.blocks[1].ffn
        assert (routed.num_experts, routed.top_k, routed.intermediate_size) == \
               (theirs_routed.num_experts, theirs_routed.top_k, theirs_routed.intermediate_size)
        assert routed.shared is not None and ours.blocks[0].streams == 4


def test_piece_size_fills_the_rounds_of_blocks():
    from snowllm_b200.parts.decay_memory import PIECE_CHOICES, PIECE_ROWS, piece_rows_for
    # 16 blocks a piece on 296 places: 37 pieces of 56 rows fill two rounds, 32 of 64 leave the second a quarter empty
    assert piece_rows_for([2048], 16, 148) == 56
    # equal cost: the standing size
    assert piece_rows_for([8192], 16, 148) == PIECE_ROWS
    # room for every block at any size: the smallest pieces are through soonest
    assert piece_rows_for([200, 130], 4, 148) == min(PIECE_CHOICES)
    # whatever the segments, a size of the list
    for lens in ([1], [97, 3, 4000], [129] * 7):
        assert piece_rows_for(lens, 3, 20) in PIECE_CHOICES
