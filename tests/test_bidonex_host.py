"""Bidonex on the host: configuration, registry, tensor list, cache plan, kept first pages."""

import json

import pytest
import torch

import bidonex_helpers as bh
from paged_attention_engine_b200.cache import BlockAllocator, CacheManager, HOLE, plan_cache
from paged_attention_engine_b200.config import BidonexConfig, ConfigError, resolve
from paged_attention_engine_b200.weights import WeightsError, check_against_specs, collect_tensor_specs, write_random_model
from plain import bidonex_plain as plain


def test_configuration_round_trip_and_registry():
    for raw, _page, _seed in bh.SMALL.values():
        cfg, spec = resolve(raw)
        assert isinstance(cfg, BidonexConfig)
        assert BidonexConfig.from_dict(cfg.to_dict()) == cfg
        assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"]
        assert len(spec.layers) == len(raw["layers"])
        for layer, entry in zip(spec.layers, raw["layers"]):
            assert layer.block == ("parallel_residual" if entry["mlp"] else "mixer_residual")
            assert layer.mixer.kind == ("general_delta" if entry["type"] == "general_delta" else "scored_window_attention")


def test_absent_keys_mean_absent_mechanisms():
    cfg = BidonexConfig.from_dict(bh.SMALL_A)
    last = cfg.layers[4].mixer
    assert (last.conv, last.window, last.keep_first) == (0, 0, 0) and last.softcap == 30.0
    assert cfg.layers[3].mixer.softcap == 0.0 and cfg.layers[2].ff == 0
    names = collect_tensor_specs(resolve(bh.SMALL_A)[1])
    assert "l4.mix.q.conv" not in names and "l3.mix.q.conv" in names and "l2.mlp.up" not in names
    assert names["l1.mix.v"].shape == (2 * 24, 64) and names["l1.mix.o"].shape == (64, 4 * 24)


@pytest.mark.parametrize("damage, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0].update(type="mamba"), "layers[0].type"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "layers[1].mixer.vdim"),
    (lambda c: c["layers"][1]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "layers[1].mlp.kind"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(damage, text):
    raw = json.loads(json.dumps(bh.SMALL_A))
    damage(raw)
    with pytest.raises(ConfigError, match=text.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
        BidonexConfig.from_dict(raw)


def test_decay_rank_is_read_from_the_tensors():
    raw = json.loads(json.dumps(bh.ONLY_DELTA))
    for layer in raw["layers"]:
        layer["mixer"].pop("rank")
    specs = collect_tensor_specs(resolve(raw)[1])
    present = {n: s.drawn_shape() for n, s in specs.items()}
    present["l0.mix.w1"], present["l0.mix.w2"] = (5, 48), (48, 5)
    check_against_specs(specs, present, "test")
    present["l0.mix.w1"] = (5, 47)
    with pytest.raises(WeightsError, match="l0.mix.w1"):
        check_against_specs(specs, present, "test")


def test_cache_plan_groups_by_every_size():
    plan = plan_cache(resolve(bh.SMALL_A)[1])
    assert [(g.num_kv_heads, g.head_dim, g.value_head_dim, g.window, g.keep_first) for g in plan.groups] == [
        (2, 16, 24, 12, 3), (3, 20, 12, 7, 0), (1, 8, 8, 0, 0)]
    assert plan.state_needs[0].shape == (2, 16, 16) and plan.state_needs[2].shape == (1, 40, 40)
    assert plan.state_needs[1].shape == (2, (4 + 2) * 16 + 2 * 24) and plan.state_needs[3].shape == (1, 6 * 20 + 3 * 12)
    assert 4 not in plan.state_needs                     # no convolution, no state
    assert plan.bytes_per_block(4, 2) == 2 * 4 * (2 * (16 + 24) + 3 * (20 + 12) + 1 * (8 + 8))


def test_release_passes_over_the_kept_first_blocks():
    a = BlockAllocator(16, 4)
    a.create_sequence("s")
    assert a.append_tokens("s", 40).ok
    first = a.block_table("s")
    freed = a.release_before("s", 22, keep_blocks=2)           # blocks 0, 1 kept; 2..4 lie before position 22
    assert freed == first[2:5] and a.block_table("s")[:2] == first[:2]
    assert a.block_table("s")[2:5] == (HOLE,) * 3 and a.num_held("s") == 7
    assert a.release_before("s", 30, keep_blocks=2) == first[5:7] and a.num_allocated == 5
    with pytest.raises(ValueError):
        a.release_before("s", 36, keep_blocks=1)
    assert sorted(a.free_sequence("s")) == sorted(first[:2] + first[7:])
    assert a.num_free == 16


def test_manager_keeps_the_pages_of_the_first_keys():
    plan = plan_cache(resolve(bh.SMALL_B)[1])            # group 0: window 5, 9 kept keys; group 1: window 33, 1 kept
    manager = CacheManager(plan.groups, 32, 4, 4)
    assert manager.create_request("r") == 0
    assert manager.reserve("r", 60).ok
    manager.advance("r", 60)
    table0 = manager.block_table("r", 0)
    assert all(b != HOLE for b in table0[:3])            # 9 keys: three pages of 4 stay
    assert all(b == HOLE for b in table0[3:14]) and table0[14] != HOLE      # next query at 60 reads keys from 56 on
    rows = manager.table_rows(0, [0], 15)
    assert (rows[0, 3:14] == HOLE).all() and (rows[0, :3] >= 0).all()
    table1 = manager.block_table("r", 1)
    assert table1[0] != HOLE and all(b == HOLE for b in table1[1:7]) and table1[7] != HOLE
    manager.free_request("r")
    assert manager.num_free == 32


def test_random_folder_runs_through_the_plain_model(tmp_path):
    folder = write_random_model(tmp_path / "m", bh.ONLY_ATTENTION, 3, torch.bfloat16)
    raw, tensors = bh.read_model(folder)
    assert raw["architecture"] == "Bidonex" and tensors["l0.mix.q.conv"].shape == (48, 3)
    assert float(tensors["l0.mix.r2"].min()) > 0.0
    logits = plain.forward(raw, tensors, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 97) and torch.isfinite(logits).all()


def test_plain_mechanisms_on_known_values():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    y = plain.layer_norm(x, torch.ones(4), torch.zeros(4), 0.0)
    assert torch.allclose(y.mean(), torch.tensor(0.0, dtype=torch.float64)) and torch.allclose((y * y).mean(), torch.tensor(1.0, dtype=torch.float64))
    u = torch.arange(8, dtype=torch.float64).reshape(4, 2)
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    assert plain.causal_conv(u, w)[:, 0].tolist() == [0.0, 200.0, 420.0, 642.0] and plain.causal_conv(u, w)[:, 1].tolist() == [1.0, 3.0, 5.0, 7.0]
    # One key, no sink: the output is its value. With a sink of equal logit: half of it.
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[4.0, 8.0]]], dtype=torch.float64)
    assert plain.scored_attention(q, q, v, 1.0)[0, 0].tolist() == [4.0, 8.0]
    assert plain.scored_attention(q, q, v, 1.0, sink=torch.zeros(1))[0, 0].tolist() == [2.0, 4.0]


def test_command_line_writes_a_random_model(tmp_path):
    from paged_attention_engine_b200 import cli

    config = tmp_path / "config.json"
    config.write_text(json.dumps(bh.SMALL_B))
    assert cli.main(["random-model", "--config", str(config), "--seed", "3", "--dtype", "bfloat16", "--out", str(tmp_path / "m")]) == 0
    raw, tensors = bh.read_model(tmp_path / "m")
    assert BidonexConfig.from_dict(raw) == BidonexConfig.from_dict(bh.SMALL_B)
    assert tensors["l1.mix.w1"].shape == (16, 96) and tensors["pos"].shape == (512, 96)
