"""Kolisun without a GPU: configuration, run order, tensor list, refusals, cache needs of mixers made of several,
and the oracle's mechanisms on inputs with known answers."""
import copy
import math

import pytest
import torch

import kolisun_tiny as kt
from plain import kolisun_plain as plain
from prelude_b200.cache.manager import CacheManager
from prelude_b200.config import ConfigError, load_model_config
from prelude_b200.config.spec import (GqaSpec, LatentAttentionSpec, ParallelMixerSpec, RotaryBandScaling, RotaryRampScaling,
                                      RotaryRatesSpec, StateSpaceSpec)
from prelude_b200.parts.model import DecoderModel
from prelude_b200.parts.registry import CombinedNeed, KvPagesNeed, StateNeed, leaf_needs
from prelude_b200.parts.rope import rotary_rates


def test_every_layer_is_parsed_on_its_own():
    cfg = load_model_config(kt.KOLISUN_K)
    spec = cfg.to_model_spec()
    assert spec.architecture == "Kolisun" and spec.vocab_size == 97 and spec.hidden_size == 40 and not spec.tie_embeddings
    kinds = [type(b.mixer) for b in spec.blocks]
    assert kinds == [LatentAttentionSpec, ParallelMixerSpec, ParallelMixerSpec, LatentAttentionSpec]
    assert all(b.kind == "postnorm_residual" and b.mixer_norm is None for b in spec.blocks)
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].ff_post_norm is None
    par = spec.blocks[1].mixer
    assert isinstance(par.mixers[0], GqaSpec) and isinstance(par.mixers[1], StateSpaceSpec) and par.scales == (0.7, 1.3)
    att = par.mixers[0]
    assert (att.num_heads, att.num_kv_heads, att.head_dim, att.value_dim, att.window) == (4, 2, 12, 20, 7)
    assert att.qkv_bias and att.whole_qk_norm_eps == 1e-5 and att.position.adjacent and att.position.dims == 8
    assert isinstance(att.position.scaling, RotaryBandScaling) and spec.blocks[2].mixer.mixers[0].position.scaling is None
    lat = spec.blocks[0].mixer
    assert (lat.kv_rank, lat.q_rank, lat.rot_dim, lat.value_dim) == (10, 14, 6, 20) and lat.sink and not lat.position.adjacent
    assert isinstance(lat.position.scaling, RotaryRampScaling) and spec.blocks[3].mixer.position.scaling is None


def test_tensor_list_has_the_designs_names_and_shapes():
    req, _ = DecoderModel(load_model_config(kt.KOLISUN_K).to_model_spec()).tensors()
    want = {"embed": (97, 40), "head": (97, 40), "final.norm": (40,), "l0.norm1": (40,), "l0.norm2": (40,), "l0.mix.dq": (14, 40),
            "l0.mix.dq.norm": (14,), "l0.mix.uq": (3 * 18, 14), "l0.mix.dkv": (16, 40), "l0.mix.dkv.norm": (10,), "l0.mix.uk": (36, 10),
            "l0.mix.uv": (60, 10), "l0.mix.sink": (3,), "l0.mix.o": (40, 60), "l0.mlp.gate": (56, 40), "l0.mlp.down": (40, 56),
            "l1.mix.left.q": (48, 40), "l1.mix.left.q.b": (48,), "l1.mix.left.k": (24, 40), "l1.mix.left.v": (40, 40),
            "l1.mix.left.v.b": (40,), "l1.mix.left.q.norm": (48,), "l1.mix.left.k.norm": (24,), "l1.mix.left.o": (40, 80),
            "l1.mix.right.in": (24 + 24 + 10 + 4, 40), "l1.mix.right.conv": (34, 3), "l1.mix.right.conv.b": (34,),
            "l1.mix.right.dt_bias": (4,), "l1.mix.right.A_log": (4,), "l1.mix.right.D": (4,), "l1.mix.right.norm": (24,),
            "l1.mix.right.o": (40, 24)}
    for name, shape in want.items():
        assert tuple(req[name].shape) == shape, name
    assert "l2.norm2" not in req and not any(n.startswith("l2.mlp") for n in req)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1].update(type="window"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(groups=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=5), "equal parts"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8), "at most the 6 elements"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "unknown kind"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused_with_the_reason(change, word):
    cfg = copy.deepcopy(kt.KOLISUN_K)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        load_model_config(cfg)
    assert word in str(e.value)


def test_cache_needs_of_mixers_made_of_several():
    model = DecoderModel(load_model_config(kt.KOLISUN_K).to_model_spec())
    needs = model.cache_needs()
    assert needs[0] == KvPagesNeed(1, 16, None, v_heads=0, v_head_dim=0) and needs[0].elements_per_token == 16
    assert isinstance(needs[1], CombinedNeed)
    leaves = [leaf for _, leaf in leaf_needs(needs[1])]
    assert leaves == [KvPagesNeed(2, 12, 7, v_heads=2, v_head_dim=20), StateNeed((4, 5, 6), torch.float32), StateNeed((2, 34), None)]
    caps = model.runtime_caps()
    assert caps.kv_cache and caps.state_slots and caps.cuda_graph
    cache = CacheManager(needs, 4, 10, 3, device=None)
    assert len(cache.groups) == 4                      # two latent rows of different sizes, two windows
    lc = cache.layer_cache(1)
    assert lc.kind == "combined" and lc.children[0].kind == "kv" and lc.children[1].kind == "combined"
    assert [c.kind for c in lc.children[1].children] == ["state", "state"]
    assert CacheManager.bytes_per_page(needs, 4, 2) == 4 * 2 * (16 + (24 + 40) + (10 + 6) + 17)
    # pages of the window's group come back as the window passes them; the latent's stay
    cache.add_request("a")
    cache.grow("a", 30)
    cache.trim("a")
    window_group = cache.group_of[(1, 0)]
    assert cache.requests["a"].tables[window_group][:5] == [-1] * 5 and cache.requests["a"].tables[cache.group_of[0]][0] >= 0
    cache.release("a")
    cache.check()


def test_band_scaled_rates_with_known_answers():
    # base 4096, 4 rates: 1, 1/8, 1/64, 1/512 -> wavelengths 6.28, 50.3, 402, 3217; original 64, low 1, high 4: kept below
    # 16, divided above 64, blended between
    r, amp = rotary_rates(RotaryRatesSpec(8, 4096.0, True, RotaryBandScaling(8.0, 1.0, 4.0, 64.0)))
    assert amp == 1.0 and r[0] == 1.0 and r[2] == pytest.approx(1 / 64 / 8) and r[3] == pytest.approx(1 / 512 / 8)
    s = (64.0 / (2 * math.pi / 0.125) - 1.0) / 3.0
    assert 0 < s < 1 and r[1] == pytest.approx((1 - s) * 0.125 / 8 + s * 0.125)
    assert r == pytest.approx(plain.banded_rates(8, 4096.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}))
    assert rotary_rates(RotaryRatesSpec(8, 16.0, True, None))[0] == pytest.approx(plain.plain_rates(8, 16.0))


def test_ramp_scaled_rates_with_known_answers():
    sc = {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}
    r, amp = rotary_rates(RotaryRatesSpec(16, 500000.0, False, RotaryRampScaling(4.0, 2048, 32.0, 1.0)))
    want, want_amp = plain.ramped_rates(16, 500000.0, sc)
    assert r == pytest.approx(want) and amp == pytest.approx(want_amp) == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert r[0] == pytest.approx(1.0)                                      # before the ramp: kept
    assert r[7] == pytest.approx(500000.0 ** (-14 / 16) / 4.0)              # past it: divided
    # a ramp of no width (both ends at one index) still divides by at least 0.001
    r2, _ = rotary_rates(RotaryRatesSpec(4, 10.0, False, RotaryRampScaling(2.0, 8, 1.0, 1.0)))
    assert r2 == pytest.approx(plain.ramped_rates(4, 10.0, {"factor": 2.0, "original": 8, "fast": 1.0, "slow": 1.0})[0])


def test_oracle_rotation_pairs_and_window_and_sink():
    x = torch.arange(1, 9, dtype=torch.float64).reshape(1, 1, 8)
    pos = torch.tensor([1])
    a = plain.rotate(x, pos, [math.pi / 2], 1.0, True)                      # elements 0, 1 turn by a quarter
    assert torch.allclose(a[0, 0], torch.tensor([-2.0, 1.0, 3, 4, 5, 6, 7, 8], dtype=torch.float64), atol=1e-12)
    b = plain.rotate(x, pos, [math.pi / 2, math.pi], 2.0, False)            # (0, 2) by a quarter, (1, 3) by a half, doubled
    assert torch.allclose(b[0, 0], torch.tensor([-6.0, -4.0, 2.0, -8.0, 5, 6, 7, 8], dtype=torch.float64), atol=1e-12)
    # window of 2: position 2 sees 1 and 2 only; equal scores -> the mean of their values
    q = torch.zeros(3, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[10.0]], [[100.0]]], dtype=torch.float64)
    o = plain.masked_softmax_attention(q, q, v, 1.0, 2)
    assert o[2, 0, 0] == pytest.approx(55.0) and o[0, 0, 0] == pytest.approx(1.0)
    # a sink of the same score as the one key halves the weight
    o = plain.masked_softmax_attention(q[:1], q[:1], v[:1], 1.0, None, torch.zeros(1, dtype=torch.float64))
    assert o[0, 0, 0] == pytest.approx(0.5)


def test_oracle_state_space_and_convolution_by_hand():
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    out = plain.causal_conv(u, torch.tensor([[0.5, 2.0]], dtype=torch.float64), torch.tensor([0.1], dtype=torch.float64))
    assert out.flatten().tolist() == pytest.approx([2.1, 4.6, 7.1])       # last tap on the current token, zeros before the start
    x = torch.ones(2, 1, 1, dtype=torch.float64)
    B = C = torch.ones(2, 1, 1, dtype=torch.float64)
    dt = torch.full((2, 1), 0.5, dtype=torch.float64)
    y = plain.state_space(x, B, C, dt, torch.zeros(1, dtype=torch.float64), torch.tensor([2.0], dtype=torch.float64))
    d = math.exp(-0.5)
    assert y.flatten().tolist() == pytest.approx([0.5 + 2.0, d * 0.5 + 0.5 + 2.0])
