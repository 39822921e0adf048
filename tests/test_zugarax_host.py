"""Zugarax on the host: configuration, registry, tensor list, cache plan, rotation frequencies."""

import json
import math

import pytest
import torch

import zugarax_helpers as zh
from paged_attention_engine_b200.cache import plan_cache
from paged_attention_engine_b200.config import ConfigError, ZugaraxConfig, resolve
from paged_attention_engine_b200.parts.rotary import banded_frequencies, ramped_frequencies
from paged_attention_engine_b200.weights import collect_tensor_specs
from plain import zugarax_plain as plain


def test_configuration_round_trip_and_registry():
    for raw, _page, _seed in zh.SMALL.values():
        cfg, spec = resolve(raw)
        assert isinstance(cfg, ZugaraxConfig)
        assert ZugaraxConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.to_dict() == raw
        assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"]
        kinds = {"attention": "gated_window_attention", "latent_attention": "latent_attention", "mlstm": "matrix_memory"}
        for layer, entry in zip(spec.layers, raw["layers"]):
            assert layer.block == ("pre_norm_residual" if entry["mlp"] else "mixer_residual")
            assert layer.mixer.kind == kinds[entry["type"]]


def test_absent_keys_mean_absent_mechanisms():
    cfg = ZugaraxConfig.from_dict(zh.SMALL_A)
    assert cfg.layers[3].mixer.window == 0 and cfg.layers[3].mixer.rot.scaling is None
    assert cfg.layers[0].mixer.window == 12 and dict(cfg.layers[0].mixer.rot.scaling)["low"] == 0.5
    assert cfg.layers[2].ff == 0 and cfg.layers[4].mixer.kv_from == 1
    assert ZugaraxConfig.from_dict(zh.SMALL_C).logit_softcap == 0.0
    bare = json.loads(json.dumps(zh.ONLY_ATTENTION))
    bare["layers"][0]["mixer"].pop("rot")
    cfg_bare, spec_bare = resolve(bare)
    assert cfg_bare.layers[0].mixer.rot is None and spec_bare.layers[0].mixer.params["position_encoding"] is None
    assert cfg_bare.to_dict() == bare
    names = collect_tensor_specs(resolve(zh.SMALL_A)[1])
    assert "l4.mix.dkv" not in names and "l4.mix.dkv.norm" not in names and "l1.mix.dkv" in names
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names
    assert names["l1.mix.q"].shape == (3 * (8 + 4), 64) and names["l1.mix.dkv"].shape == (20 + 4, 64)
    assert names["l1.mix.uk"].shape == (3 * 8, 20) and names["l4.mix.uv"].shape == (2 * 6, 20)
    assert names["l0.mix.g"].shape == (4 * 24, 64) and names["l0.mix.q.norm"].shape == (16,)
    assert names["l2.mix.i"].shape == (2, 64) and names["l2.mix.norm"].shape == (2 * 20,)
    assert names["l0.mlp.gate.b"].shape == (96,) and names["l0.mlp.down.b"].shape == (64,)


@pytest.mark.parametrize("damage, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.pop("embedding"), "embedding.scale"),
    (lambda c: c["layers"][0].update(type="mamba"), "layers[0].type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "layers[0].mixer.vdim"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("high"), "rot.scaling.high"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "rot_dim"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][4]["mixer"].update(kv_rank=24), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"].pop("gate_cap"), "layers[2].mixer.gate_cap"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "layers[1].mlp.kind"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "layers[1].mlp.limit"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_the_key(damage, text):
    raw = json.loads(json.dumps(zh.SMALL_A))
    damage(raw)
    with pytest.raises(ConfigError, match=text.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
        ZugaraxConfig.from_dict(raw)


def test_cache_plan_groups_windows_latents_and_states():
    plan = plan_cache(resolve(zh.SMALL_A)[1])
    by_entry = {pos: plan.groups[g] for pos, (g, _i) in plan.entry_group.items()}
    assert (by_entry[0].num_kv_heads, by_entry[0].head_dim, by_entry[0].value_dim, by_entry[0].window) == (2, 16, 24, 12)
    assert (by_entry[3].window, by_entry[3].value_dim) == (0, 12)
    latent = by_entry[1]
    assert (latent.num_kv_heads, latent.head_dim, latent.value_dim, latent.values_in_keys) == (1, 24, 20, True)
    assert latent.stored_per_token == 24            # the latent and the shared rotated part, nothing else
    assert plan.entry_group[4] == plan.entry_group[1] and plan.entry_writes[1] and not plan.entry_writes[4]
    assert plan.state_needs[2].shape == (2, 12 * 21 + 1) and plan.state_needs[5].shape == (1, 24 * 9 + 1)
    # two latents of different sizes are two groups; the reader shares its source's
    plan = plan_cache(resolve(zh.SMALL_C)[1])
    assert plan.entry_group[0] == plan.entry_group[3] and plan.entry_group[2][0] != plan.entry_group[0][0]
    assert plan.bytes_per_block(8, 2) == (304 + 32) * 8 * 2


def test_scaled_frequencies_against_the_plain_formulas():
    for dims, base, factor, low, high, original in [(8, 10000.0, 4.0, 0.5, 3.0, 24), (64, 500000.0, 8.0, 1.0, 4.0, 8192),
                                                    (32, 100.0, 2.0, 2.0, 16.0, 40)]:
        freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        got = banded_frequencies(freqs, factor, low, high, original)
        want = plain.banded_frequencies(dims, base, factor, low, high, original)
        assert got == pytest.approx(want, rel=1e-12)
        kinds = {"kept": sum(g == f for g, f in zip(got, freqs)), "slowed": sum(abs(g - f / factor) < 1e-15 for g, f in zip(got, freqs))}
        assert kinds["kept"] + kinds["slowed"] <= len(freqs)
    for dims, base, factor, original, fast, slow in [(4, 50000.0, 6.0, 16, 8.0, 2.0), (64, 10000.0, 40.0, 4096, 32.0, 1.0),
                                                     (32, 500.0, 8.0, 32, 16.0, 1.0)]:
        freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        got, amplitude = ramped_frequencies(freqs, dims, base, factor, original, fast, slow)
        want, want_amplitude = plain.ramped_frequencies(dims, base, factor, original, fast, slow)
        assert got == pytest.approx(want, rel=1e-12) and amplitude == pytest.approx(want_amplitude, rel=1e-12)
    # the three bands are all met by the first attention layer of the small configuration
    rot = zh.SMALL_A["layers"][0]["mixer"]["rot"]
    s = rot["scaling"]
    freqs = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)]
    got = banded_frequencies(freqs, s["factor"], s["low"], s["high"], s["original"])
    ratios = [g / f for g, f in zip(got, freqs)]
    assert ratios[0] == 1.0 and ratios[-1] == pytest.approx(1 / s["factor"]) and any(1 / s["factor"] < r < 1.0 for r in ratios)


def test_plain_mechanisms_on_cases_worked_by_hand():
    # one key, score 0: the sink halves the weight
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[2.0, 4.0]]], dtype=torch.float64)
    assert torch.allclose(plain.softmax_attention(q, q, v, 1.0, extra_one=True), v / 2)
    assert torch.allclose(plain.softmax_attention(q, q, v, 1.0), v)
    # the matrix memory's first token: m = max(f, i), S = e^(i - m) k v^T
    k = torch.tensor([[[1.0, 2.0]]], dtype=torch.float64)
    o, state = plain.matrix_memory_scan(k, k, v, torch.tensor([[0.3]]), torch.tensor([[-0.2]]), 15.0)
    S, n, m = state[0]
    assert m == pytest.approx(15.0 * math.tanh(0.3 / 15.0), abs=1e-7)            # the capped input gate; log sigmoid(.) < 0 is below it
    assert torch.allclose(S, torch.outer(k[0, 0], v[0, 0]), atol=1e-6) and torch.allclose(n, k[0, 0], atol=1e-6)
    assert torch.allclose(o[0, 0], v[0, 0] * 5.0 / (5.0 + 1e-6), atol=1e-9)
    # a pair at position 1 with frequency pi / 2 turns by a quarter
    x = torch.tensor([[[1.0, 0.0, 7.0]], [[1.0, 0.0, 7.0]]], dtype=torch.float64)
    turned = plain.rotate(x, [0, 1], [torch.pi / 2], "half")
    assert torch.allclose(turned[1, 0], torch.tensor([0.0, 1.0, 7.0], dtype=torch.float64), atol=1e-12)
    assert torch.allclose(turned[0, 0], x[0, 0])
