"""Pabelix on the CPU: its configuration, the run order and tensor list that follow from it, and the plain
implementation's own mechanisms on inputs made so that a fault would show."""
import copy
import math

import pytest
import torch

import pabelix_tiny as pt
from plain import pabelix_plain as plain
from prelude_b200.cache.manager import CacheManager
from prelude_b200.config import ConfigError, load_model_config, resolve_architecture
from prelude_b200.config.spec import ClampedGluSpec, DiffAttentionSpec, RoutedExpertsSpec
from prelude_b200.parts.model import DecoderModel


def test_the_architecture_key_resolves_and_layers_are_read_one_by_one():
    assert resolve_architecture(pt.PABELIX_P).name == "Pabelix"
    spec = load_model_config(pt.PABELIX_P).to_model_spec()
    assert (spec.vocab_size, spec.hidden_size, spec.final_norm.eps, spec.final_norm.offset) == (97, 40, 1e-5, 1.0)
    assert spec.embedding.kind == "token_embedding_sinusoid" and spec.tie_embeddings
    m0, m4 = spec.blocks[0].mixer, spec.blocks[4].mixer
    assert isinstance(m0, DiffAttentionSpec)
    assert (m0.num_heads, m0.num_kv_heads, m0.head_dim, m0.value_dim, m0.softmax_scale, m0.lambda_init) == (4, 2, 12, 20, 0.3, 0.4)
    assert (m0.query_temperature.coef, m0.query_temperature.every) == (0.7, 4)
    assert (m4.num_heads, m4.head_dim, m4.value_dim) == (3, 7, 33)
    f0, f1, f3, f4 = (spec.blocks[i].feed_forward for i in (0, 1, 3, 4))
    assert isinstance(f0, ClampedGluSpec) and (f0.intermediate_size, f0.limit, f0.alpha) == (56, 0.8, 1.702)
    assert isinstance(f1, RoutedExpertsSpec) and (f1.n_experts, f1.expert_size, f1.top_k, f1.n_groups, f1.keep_groups) == (6, 24, 2, 3, 2)
    assert (f3.n_experts, f3.top_k, f3.n_groups, f3.keep_groups) == (4, 1, 1, 1)
    assert (f4.n_groups, f4.keep_groups, f4.group_score_top) == (1, 1, 2)
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].ff_norm is None


def test_a_layer_that_reads_another_layers_keys_owns_no_cache_and_no_key_value_tensors():
    spec = load_model_config(pt.PABELIX_P).to_model_spec()
    order = spec.resolved_order()
    assert [(c.cache, c.writes_cache) for c in order] == [(0, True), (1, True), (0, False), (1, False), (4, True)]
    model = DecoderModel(spec)
    req, _ = model.tensors()
    assert "l0.mix.k" in req and "l0.mix.v" in req and "l2.mix.q" in req and "l2.mix.g" in req
    assert "l2.mix.k" not in req and "l2.mix.v" not in req and "l3.mix.k" not in req
    assert "l2.norm1b" in req and "l2.norm2" not in req and "l2.norm2b" not in req and not any(n.startswith("l2.mlp") for n in req)
    assert req["l1.mlp.e5.down"].shape == (40, 24) and req["l1.mlp.router"].shape == (6, 40)
    assert req["l4.mix.q"].shape == (3 * 2 * 7, 40) and req["l4.mix.v"].shape == (3 * 33, 40) and req["l4.mix.lq2"].shape == (7,)
    assert req["embed"].shape == (97, 40) and "final.norm" in req
    needs = model.cache_needs()
    assert needs[2] is None and needs[3] is None
    assert (needs[0].n_kv_heads, needs[0].head_dim, needs[0].value_heads, needs[0].value_dim) == (4, 12, 2, 20)
    # keys and values of different sizes: a page costs their sum, and layers of equal need share a group
    cache = CacheManager(needs, page_size=4, num_pages=8, max_slots=2)
    assert len(cache.groups) == 3
    assert CacheManager.bytes_per_page(needs, 4, 2) == 4 * 2 * ((4 * 12 + 2 * 20) + (2 * 16 + 1 * 8) + (6 * 7 + 3 * 33))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="recurrent"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "without keys and values of its own"),
    (lambda c: c["layers"][2]["mixer"].update(dim=10), "sizes differ"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][3]["mlp"]["router"].update(top=5), "cannot come from"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "missing field `vdim`"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "not a multiple"),
    (lambda c: c.pop("norm"), "missing field `norm`"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_a_bad_configuration_is_refused_with_its_reason(change, message):
    cfg = copy.deepcopy(pt.PABELIX_P)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        load_model_config(cfg)


def test_random_weights_store_norm_scales_around_zero():
    t = pt.random_tensors(pt.PABELIX_P, seed=3, std=0.1, norm_jitter=0.2)
    assert float(t["l0.norm1"].abs().max()) <= 0.2 and float(t["final.norm"].abs().max()) <= 0.2
    assert t["l4.mix.lk1"].shape == (7,)


# -- the plain implementation's mechanisms, on inputs where the answer is known ------------------------------------
def test_plain_position_vector_and_temperature():
    s = plain.sinusoid(6, 8)
    assert torch.allclose(s[0], torch.tensor([0.0, 1.0] * 4, dtype=torch.float64))
    for i in range(4):
        ang = 5 * 10000.0 ** (-2 * i / 8)
        assert abs(float(s[5, 2 * i]) - math.sin(ang)) < 1e-12 and abs(float(s[5, 2 * i + 1]) - math.cos(ang)) < 1e-12
    tau = plain.query_temperature(9, 0.5, 4, torch.float64)
    assert torch.allclose(tau[:3], torch.ones(3, dtype=torch.float64))             # (p + 1) // 4 == 0 for p < 3
    assert abs(float(tau[3]) - (1 + 0.5 * math.log(2))) < 1e-12 and abs(float(tau[6]) - (1 + 0.5 * math.log(2))) < 1e-12
    assert abs(float(tau[7]) - (1 + 0.5 * math.log(3))) < 1e-12


def test_plain_route_keeps_to_the_best_groups():
    # three groups of two; group scores (sum of the two largest): 1.2, 1.5, 0.95 -> groups 1 and 0 are kept;
    # the single largest score sits in group 2 and must not be chosen
    s = torch.tensor([[0.7, 0.5, 0.8, 0.7, 0.9, 0.05]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    idx, w = plain.route(z, top=3, groups=3, keep=2)
    assert sorted(idx[0].tolist()) == [0, 2, 3]
    assert torch.allclose(w[0].sort().values, torch.tensor([0.7, 0.7, 0.8], dtype=torch.float64))
    idx, w = plain.route(z, top=2, groups=1, keep=1)
    assert sorted(idx[0].tolist()) == [2, 4] and abs(float(w.sum()) - 1.7) < 1e-12       # not renormalised


def test_plain_clamped_unit_clamps_gate_from_above_and_up_on_both_sides():
    w = {"gate": torch.eye(3, dtype=torch.float64), "up": torch.eye(3, dtype=torch.float64), "down": torch.eye(3, dtype=torch.float64)}
    y = plain.clamped_glu(torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64), w, limit=1.0)
    sg = lambda a: a / (1 + math.exp(-1.702 * a))
    assert torch.allclose(y[0], torch.tensor([sg(1.0) * 2.0, sg(-5.0) * 0.0, sg(0.5) * 1.5], dtype=torch.float64))
