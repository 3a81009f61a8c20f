"""Kolisun on the GPU against the plain implementation: every mechanism alone, then whole models through every way
of cutting requests into steps, in 32-bit and in bfloat16, with pools so small that pages and slots are used again."""
import copy
import json
import math
import os

import pytest
import torch

import harness
import kolisun_tiny as kt
import tiny
from plain import kolisun_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: (2e-4, 0.0), torch.bfloat16: (0.0, 4e-2)}


def _weights(folder):
    return {k: v for k, v in tiny.read_weights(folder).items()}


def _cfg(folder):
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def _reference(folder, reqs):
    cfg, w = _cfg(folder), _weights(folder)
    return {rid: plain.forward(cfg, w, toks, torch.float64) for rid, toks in reqs.items()}


def _compare(got, ref, dtype, loosen=1.0):
    """Every position within the bound in 32-bit; in bfloat16 the median well within it and no more than a tenth of
    the positions off (a fault of a mechanism puts every position after it off)."""
    atol, rel = TOL[dtype]
    off, ratios = [], []
    for (rid, pos), row in got.items():
        want = ref[rid][pos]
        bound = loosen * (atol * max(1.0, float(want.abs().max())) + rel * float(want.abs().max()))
        diff = float((row.double() - want).abs().max())
        ratios.append(diff / bound)
        if diff > bound:
            off.append(f"request {rid} position {pos}: max diff {diff:.3e} > {bound:.3e}")
    allowed = len(got) // 10 if dtype == torch.bfloat16 else 0
    assert sorted(ratios)[len(ratios) // 2] <= 0.5, f"the median position is at {sorted(ratios)[len(ratios) // 2]:.2f} of the bound"
    assert len(off) <= allowed, f"{len(off)} of {len(got)} positions off: " + "; ".join(off[:5])


def _runner(folder, dtype, page_size, num_pages, max_slots=4, graphs=False):
    from prelude_b200.engine.loading import load_model, make_runner
    model = load_model(folder, dtype, DEV)
    runner = make_runner(model, page_size=page_size, num_pages=num_pages, max_slots=max_slots,
                         max_request_tokens=num_pages * page_size if graphs else None)
    if graphs:
        runner.enable_step_graphs()
    return runner


def _steps_through_a_mixer(part, x, cuts, page, dtype, slots=2, use_slot=0):
    """x [T, width] through a mixer alone, cut into the steps ``cuts``; returns the outputs one below the other."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    dev = torch.device(DEV)
    T = x.shape[0]
    cache = CacheManager([part.cache_need()], page, -(-T // page) + 1, slots, dev, dtype)
    for i in range(use_slot):                      # the request does not get slot 0
        cache.add_request(f"other{i}")
    cache.add_request("a")
    got, at = [], 0
    for n in cuts:
        cache.grow("a", at + n)
        batch = build_step_batch([StepItem("a", [0] * n, at, [])], cache.block_tables(["a"]), [cache.slot_of("a")], dev, 10, 1 << 20)
        cache.zero_fresh_state()
        got.append(part.forward(x[at:at + n].to(DEV).contiguous(), batch, cache.layer_cache(0), True).float().cpu())
        assert int(batch.status.item()) == 0
        cache.trim("a")
        at += n
    assert at == T
    return torch.cat(got).double()


def _cuts(T, head):
    return [head] + [1] * (T - head)


# -- mechanisms alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("adjacent,dims,off,head,amp", [(True, 8, 0, 12, 1.0), (False, 6, 10, 16, 1.3), (True, 16, 0, 16, 1.0), (False, 4, 3, 9, 0.7)])
def test_norm_over_whole_projections_and_rotation_by_rates(dtype, adjacent, dims, off, head, amp):
    """The kernel between projection and attention, alone: a norm over all heads at once, a rotation of part of a
    head from an offset in either pairing at positions up to thousands, and the second part of the queries written
    elsewhere."""
    from prelude_b200.ops import kernels as K
    H, T = 3, 50
    g = torch.Generator().manual_seed(dims * 7 + head)
    q = torch.randn(T, H * head, generator=g).to(dtype)
    wq = (1.0 + 0.3 * torch.randn(H * head, generator=g)).to(dtype).float()
    rates = [0.9 ** i * 0.7 for i in range(dims // 2)]
    pos = torch.randint(0, 5000, (T,), generator=g).to(torch.int32)
    want = plain.rms_norm(q.double(), wq.double(), 1e-5).reshape(T, H, head)
    want[..., off:off + dims] = plain.rotate(want[..., off:off + dims], pos.long(), [float(torch.tensor(r, dtype=torch.float32)) for r in rates],
                                            amp, adjacent)
    split = off if off else head
    out1 = torch.zeros(T, H, split, dtype=dtype, device=DEV)
    out2 = torch.zeros(T, H, head + 5, dtype=dtype, device=DEV) if split < head else None
    K.qkv_prepare(q.to(DEV), None, None, n_heads=H, q_dim=head, q_weight=wq.to(DEV), eps=1e-5,
                  rates=torch.tensor(rates, dtype=torch.float32, device=DEV), rot_dims=dims, adjacent=adjacent, amplitude=amp,
                  q_rot_off=off, positions=pos.to(DEV), table_row=torch.zeros(T, dtype=torch.int32, device=DEV), q_out=out1,
                  q_split=split, q_out2=out2, q2_off=5)
    got = out1.float().cpu().double() if out2 is None else torch.cat([out1.float().cpu(), out2[:, :, 5:5 + head - split].float().cpu()], -1).double()
    # a 32-bit angle at position 5,000 is off by 3e-4: that much of a rotated element may move
    tol = 1e-3 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol * float(want.abs().max())
    if out2 is not None:
        assert float(out2[:, :, :5].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot,window,page", [(4, 2, 12, 20, 8, 7, 4), (8, 2, 64, 64, 64, 50, 16), (2, 1, 10, 6, 10, 19, 8),
                                                              (4, 4, 32, 32, 16, 33, 16), (6, 3, 16, 48, 16, None, 8), (4, 1, 128, 128, 64, 16, 16)])
def test_window_attention_mixer_equals_the_plain_one(dtype, heads, kv, dim, vdim, rot, window, page):
    """The attention of the parallel mixer alone over a prompt and then token by token.  One key is made to stand out:
    queries find it while it is inside the window and must lose it at the very token it leaves; a window that is one
    token off, a lost bias, a norm per head instead of over all heads or a wrong pairing changes the output at once."""
    from prelude_b200.config.spec import GqaSpec, RotaryBandScaling, RotaryRatesSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T, head_tokens = 48, 100, 61
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    m = kt.left(heads, kv, dim, vdim, 1.0 / math.sqrt(dim), window, rot, base=200.0, scaling=kt.bands(4.0, 1.0, 4.0, 32))
    w = {"q": torch.randn(heads * dim, width, generator=g) * 0.3, "k": torch.randn(kv * dim, width, generator=g) * 0.3,
         "v": torch.randn(kv * vdim, width, generator=g) * 0.3, "o": torch.randn(width, heads * vdim, generator=g) * 0.2,
         "q.b": torch.randn(heads * dim, generator=g) * 0.5, "k.b": torch.randn(kv * dim, generator=g) * 0.5,
         "v.b": torch.randn(kv * vdim, generator=g) * 0.5, "q.norm": 1.0 + 0.4 * torch.randn(heads * dim, generator=g),
         "k.norm": 1.0 + 0.4 * torch.randn(kv * dim, generator=g)}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g)
    x[58] *= 3.0                                      # its value stands out for as long as it is seen
    x = x.to(dtype)
    scale = 4.0 / math.sqrt(dim) if dtype == torch.float32 else 1.5 / math.sqrt(dim)     # sharp softmax
    m["scale"] = scale
    want = plain.window_attention(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-5)
    spec = GqaSpec(width, heads, kv, dim, vdim, scale, RotaryRatesSpec(rot, 200.0, True, RotaryBandScaling(4.0, 1.0, 4.0, 32.0)), qkv_bias=True,
                   whole_qk_norm_eps=1e-5, window=window)
    part = make_part("mixer", spec, "mix")
    part.load(lambda name: w[name[len("mix."):]], RunContext(torch.device(DEV), dtype))
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts in (_cuts(T, head_tokens), [T], [2, 30, 3, 26, 2, 37]):
        got = _steps_through_a_mixer(part, x, cuts, page, dtype)
        assert float((got - want).abs().max()) < tol * float(want.abs().max()), cuts[:3]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,dim,rot,vdim,kv_rank,q_rank,page,turned", [(3, 12, 6, 20, 10, 14, 4, 6), (4, 32, 16, 48, 64, 40, 16, 16), (1, 16, 16, 16, 16, 16, 8, 16),
                                                                           (8, 16, 32, 16, 32, 64, 16, 32), (2, 7, 4, 9, 13, 5, 8, 4), (4, 32, 16, 32, 64, 24, 16, 8)])
def test_latent_attention_mixer_equals_the_plain_one(dtype, heads, dim, rot, vdim, kv_rank, q_rank, page, turned):
    """The latent attention alone over a prompt and token by token, with sinks large enough to take a good share of
    every softmax (one left out shows at once) and an early token that later queries find among a hundred."""
    from prelude_b200.config.spec import LatentAttentionSpec, RotaryRampScaling, RotaryRatesSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T, head_tokens = 40, 120, 83
    g = torch.Generator().manual_seed(heads * 100 + kv_rank)
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": 2.0 / math.sqrt(dim + rot),
         "rot": {"dims": turned, "base": 300.0, "scaling": kt.ramp(3.0, 24, 6.0, 1.0)}}
    w = {"dq": torch.randn(q_rank, width, generator=g) * 0.3, "dq.norm": 1.0 + 0.3 * torch.randn(q_rank, generator=g),
         "uq": torch.randn(heads * (dim + rot), q_rank, generator=g) * 0.4, "dkv": torch.randn(kv_rank + rot, width, generator=g) * 0.3,
         "dkv.norm": 1.0 + 0.3 * torch.randn(kv_rank, generator=g), "uk": torch.randn(heads * dim, kv_rank, generator=g) * 0.4,
         "uv": torch.randn(heads * vdim, kv_rank, generator=g) * 0.3, "o": torch.randn(width, heads * vdim, generator=g) * 0.2,
         "sink": torch.linspace(3.0, 6.0, heads)}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g)
    x[3] *= 2.5
    x = x.to(dtype)
    want = plain.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-5)
    no_sink = plain.latent_attention(x.double(), {k: (v.double() if k != "sink" else v.double() - 50.0) for k, v in w.items()}, m, 1e-5)
    assert float((want - no_sink).abs().max()) > 0.02 * float(want.abs().max())          # the sinks matter here
    spec = LatentAttentionSpec(width, heads, dim, rot, vdim, kv_rank, q_rank, m["scale"], 1e-5,
                               RotaryRatesSpec(turned, 300.0, False, RotaryRampScaling(3.0, 24, 6.0, 1.0)), sink=True)
    part = make_part("mixer", spec, "mix")
    part.load(lambda name: w[name[len("mix."):]], RunContext(torch.device(DEV), dtype))
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts in (_cuts(T, head_tokens), [T], [2, 45, 3, 33, 2, 35]):
        got = _steps_through_a_mixer(part, x, cuts, page, dtype)
        assert float((got - want).abs().max()) < tol * float(want.abs().max()), cuts[:3]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,vdim,state,groups,taps,parts", [(4, 6, 5, 1, 3, 1), (4, 32, 64, 2, 4, 4), (3, 11, 9, 3, 5, 3), (1, 16, 16, 1, 2, 1),
                                                              (8, 16, 130, 4, 4, 2), (2, 40, 24, 2, 1, 1)])
def test_state_space_mixer_equals_the_plain_one(dtype, heads, vdim, state, groups, taps, parts):
    """The state-space mixer alone: a whole sequence at once, token by token, and in portions shorter than the
    convolution is long; in a state slot other than the first; decays between slow and fast, so that a state that is
    lost, carried in fewer bits or started from another sequence's shows."""
    from prelude_b200.config.spec import StateSpaceSpec
    from prelude_b200.parts.registry import RunContext, make_part
    width, T = 40, 90
    g = torch.Generator().manual_seed(heads * 10 + state)
    inner, gn = heads * vdim, groups * state
    m = kt.right(heads, vdim, state, groups, taps, parts)
    w = {"in": torch.randn(2 * inner + 2 * gn + heads, width, generator=g) * 0.3, "conv": torch.randn(inner + 2 * gn, taps, generator=g) * 0.5,
         "conv.b": torch.randn(inner + 2 * gn, generator=g) * 0.2, "dt_bias": torch.randn(heads, generator=g), "A_log": torch.linspace(-3.0, 1.0, heads),
         "D": torch.randn(heads, generator=g), "norm": 1.0 + 0.3 * torch.randn(inner, generator=g), "o": torch.randn(width, inner, generator=g) * 0.2}
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g).to(dtype)
    want = plain.mamba2(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-5)
    part = make_part("mixer", StateSpaceSpec(width, heads, vdim, state, groups, taps, parts, 1e-5), "mix")
    part.load(lambda name: w[name[len("mix."):]], RunContext(torch.device(DEV), dtype))
    tol = 5e-5 if dtype == torch.float32 else 4e-2
    for cuts, slot in (([T], 0), (_cuts(T, 40), 1), ([2, 1, 1, 2, 3, 1, 30, 2, 48], 2), ([1] * T, 0)):
        got = _steps_through_a_mixer(part, x, cuts, 16, dtype, slots=3, use_slot=slot)
        assert float((got - want).abs().max()) < tol * float(want.abs().max()), cuts[:3]


def test_mixers_side_by_side_are_added_with_their_scales():
    from prelude_b200.ops import kernels as K
    a = torch.randn(37, 50, device=DEV)
    b = torch.randn(37, 50, device=DEV)
    assert float((K.scaled_sum(a, 0.7, b, -1.3, torch.float32) - (0.7 * a + (-1.3) * b)).abs().max()) < 1e-6
    got = K.scaled_sum(a.bfloat16(), 0.7, b.bfloat16(), 1.3, torch.bfloat16).float()
    assert float((got - (0.7 * a.bfloat16().float() + 1.3 * b.bfloat16().float())).abs().max()) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("width", [40, 130, 4096])
def test_norm_of_a_sublayers_output_added_to_the_stream_it_is_read_from(dtype, width):
    from prelude_b200.ops import kernels as K
    g = torch.Generator().manual_seed(width)
    x = torch.randn(9, width, generator=g).to(dtype).to(DEV)
    w = (1.0 + 0.2 * torch.randn(width, generator=g)).to(DEV)
    res = torch.randn(9, width, generator=g).to(DEV)
    want = res.double() + plain.rms_norm(x.double(), w.double(), 1e-5)
    out = K.normed_add_rmsnorm(K.Normed(x, w, 1e-5), res, None, 0.0, dtype, sum_out=True)
    assert float((res.double() - want).abs().max()) < 1e-5
    assert out.dtype == dtype and torch.equal(out, res.to(dtype))


def test_products_head_by_head_on_the_32_bit_units():
    from prelude_b200.ops.linear import batched_linear
    g = torch.Generator().manual_seed(5)
    a = torch.randn(70, 3, 13, generator=g).to(DEV)
    w = torch.randn(3, 9, 13, generator=g).to(DEV)
    out = torch.zeros(70, 3, 12, device=DEV)
    batched_linear(a.transpose(0, 1), w, out.transpose(0, 1)[:, :, :9])
    want = torch.einsum("thk,hnk->thn", a.double(), w.double())
    assert float((out[:, :, :9].double() - want).abs().max()) < 1e-5 and float(out[:, :, 9:].abs().max()) == 0.0
    ab, wb, ob = a.bfloat16(), w.bfloat16(), torch.zeros(70, 3, 12, device=DEV, dtype=torch.bfloat16)
    batched_linear(ab.transpose(0, 1), wb, ob.transpose(0, 1)[:, :, :9])
    assert float((ob[:, :, :9].double() - want).abs().max()) < 0.1 and float(ob[:, :, 9:].abs().max()) == 0.0


# -- whole models ----------------------------------------------------------------------------------------------------
REQUESTS = {"K": {"k1": 1, "k2": 2, "k19": 19, "k70": 70, "k33": 33}, "L": {"l3": 3, "l150": 150, "l64": 64, "l41": 41, "l97": 97},
            "M": {"m1": 1, "m9": 9, "m40": 40, "m17": 17}}


def _requests(which):
    v = kt.PARAMS[which][0]["vocab"]
    return {rid: tiny.random_ids(n, v, sum(map(ord, rid))) for rid, n in REQUESTS[which].items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("kolisun")
    return {(w, d): kt.make_folder(root, w, d) for w in "KLM" for d in (torch.float32, torch.bfloat16)}


@pytest.fixture(scope="module")
def references(folders):
    return {w: _reference(folders[(w, torch.bfloat16)], _requests(w)) for w in "KLM"}, \
           {w: _reference(folders[(w, torch.float32)], _requests(w)) for w in "KLM"}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["K", "L", "M"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed", "mixed_graphs"])
def test_cuts_match_plain(folders, references, which, dtype, cut):
    """Whole prompts, a decoded tail that crosses windows and page borders, portions down to two tokens, and mixed
    batches in a pool that holds less than all requests (pages and slots used again), launched and captured."""
    reqs = _requests(which)
    ref = references[0 if dtype == torch.bfloat16 else 1][which]
    page = kt.PARAMS[which][2]
    make = {"whole": harness.whole, "tail_decode": lambda r: harness.tail_decode(r, 40), "portions": harness.portions,
            "mixed": lambda r: harness.mixed(r, max_live=3), "mixed_graphs": lambda r: harness.mixed(r, max_live=3, seed=5)}[cut]
    schedule = make(reqs)
    num_pages = harness.peak_tokens(schedule, page) // page
    if cut.startswith("mixed"):
        assert num_pages < sum(-(-len(t) // page) for t in reqs.values())
    runner = _runner(folders[(which, dtype)], dtype, page, num_pages, max_slots=3 if cut.startswith("mixed") else 1,
                     graphs=cut == "mixed_graphs")
    got = harness.run_schedule(runner, schedule)
    assert len(got) == sum(len(t) for t in reqs.values())
    _compare(got, ref, dtype)
    runner.cache.check()
    assert runner.cache.used_pages() == 0
    if cut == "mixed_graphs":
        assert runner.graph_steps_run > 0


@pytest.mark.parametrize("which", ["K", "L"])
def test_batched_requests_equal_each_alone_in_32_bit(folders, which):
    reqs = _requests(which)
    page = kt.PARAMS[which][2]
    folder = folders[(which, torch.float32)]
    alone = harness.run_schedule(_runner(folder, torch.float32, page, 64), harness.whole(reqs))
    together = harness.run_schedule(_runner(folder, torch.float32, page, 64, max_slots=5),
                                    [([(rid, toks, list(range(len(toks)))) for rid, toks in reqs.items()], list(reqs))])
    for key, row in alone.items():
        assert float((row - together[key]).abs().max()) <= 2e-5 * float(row.abs().max()), key


def test_cuts_agree_bitwise_in_32_bit(folders):
    """The order of every sum depends on a token's position only: however a request is cut, its logits have the same bits."""
    reqs = {"k70": _requests("K")["k70"]}
    folder = folders[("K", torch.float32)]
    a = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.whole(reqs))
    b = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.portions(reqs))
    c = harness.run_schedule(_runner(folder, torch.float32, 4, 20), harness.tail_decode(reqs, 50))
    for key, row in a.items():
        assert torch.equal(row, b[key]) and torch.equal(row, c[key]), key


def test_sharp_attention_finds_keys_far_back_and_at_window_and_page_borders(tmp_path):
    """Query and key matrices scaled up make every softmax pick few keys, wherever they lie: among hundreds of keys,
    at the first positions, on either side of a page border, just inside the window and just outside (where it must
    not be found).  32-bit, prompt in one step, in portions, and with a decoded tail longer than the windows."""
    cfg = copy.deepcopy(kt.KOLISUN_K)
    tensors = kt.random_tensors(cfg, seed=21, std=0.25, norm_jitter=0.3)
    for name in list(tensors):
        if name.endswith((".left.q.norm", ".left.k.norm", ".mix.uq", ".mix.uk")):
            tensors[name] = tensors[name] * 2.0
        if name.endswith(".mix.sink"):
            tensors[name] = tensors[name] + 2.0
    folder = kt.make_folder_from_tensors(tmp_path, "sharp", cfg, tensors)
    reqs = {"s": tiny.random_ids(300, cfg["vocab"], 77)}
    ref = _reference(folder, reqs)
    for schedule in (harness.whole(reqs), harness.portions(reqs, (37, 2, 64, 3, 29)), harness.tail_decode(reqs, 70)):
        got = harness.run_schedule(_runner(folder, torch.float32, 16, 19), schedule)
        _compare(got, ref, torch.float32, loosen=5.0)        # scores of tens: their 32-bit rounding shows in the weights


def test_long_decoding_through_freed_and_reused_slots(folders):
    """Two requests decoded token by token for 120 steps side by side after short prompts, then a third takes the
    slot (its state, its convolution inputs) and the pages that the first gave back."""
    cfg = kt.KOLISUN_K
    reqs = {"a": tiny.random_ids(130, cfg["vocab"], 1), "b": tiny.random_ids(127, cfg["vocab"], 2), "c": tiny.random_ids(60, cfg["vocab"], 3)}
    ref = _reference(folders[("K", torch.float32)], reqs)
    steps = [([("a", reqs["a"][:10], list(range(10))), ("b", reqs["b"][:7], list(range(7)))], [])]
    for i in range(120):
        steps.append(([("a", reqs["a"][10 + i:11 + i], [0]), ("b", reqs["b"][7 + i:8 + i], [0])], ["a", "b"] if i == 119 else []))
    steps.append(([("c", reqs["c"], list(range(60)))], ["c"]))
    runner = _runner(folders[("K", torch.float32)], torch.float32, 4, 66, max_slots=2)
    _compare(harness.run_schedule(runner, steps), ref, torch.float32)
    runner.cache.check()


@pytest.mark.parametrize("which,lens,new", [("K", [1, 5, 17], 20), ("L", [9, 64, 2, 31], 12)])
def test_greedy_generation_through_the_engine_equals_the_plain_one(folders, which, lens, new):
    from prelude_b200 import Engine
    folder = folders[(which, torch.float32)]
    cfg, w = _cfg(folder), _weights(folder)
    prompts = [tiny.random_ids(n, cfg["vocab"], 50 + n) for n in lens]
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(new):
            seq.append(int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax()))
        want.append(seq[len(p):])
    eng = Engine(folder, dtype="f32", page_size=kt.PARAMS[which][2], num_pages=64, max_running_requests=4)
    assert eng.caps.cuda_graph and eng.caps.state_slots
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
    assert [r.token_ids for r in got] == want
    # portions of a few tokens beside decoding requests, launched kernel by kernel: the same tokens
    eng2 = Engine(folder, dtype="f32", page_size=kt.PARAMS[which][2], num_pages=64, max_running_requests=4,
                  max_num_batched_tokens=7, long_prefill_token_threshold=3, cuda_graph=False)
    assert [r.token_ids for r in eng2.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)] == want
    assert eng.cache.used_pages() == 0 and eng2.cache.used_pages() == 0


def test_generation_in_bfloat16_runs_captured_steps(folders):
    from prelude_b200 import Engine
    folder = folders[("L", torch.bfloat16)]
    prompts = [tiny.random_ids(n, kt.KOLISUN_L["vocab"], 50 + n) for n in (40, 7, 90)]
    eng = Engine(folder, dtype="bf16", page_size=16, num_pages=64, max_running_requests=4)
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=16, ignore_eos=True)
    eng2 = Engine(folder, dtype="bf16", page_size=16, num_pages=64, max_running_requests=4, cuda_graph=False)
    got2 = eng2.generate(prompts, temperature=0.0, max_new_tokens=16, ignore_eos=True)
    assert all(len(r.token_ids) == 16 for r in got)
    # captured and launched steps run the same kernels on the same numbers
    assert [r.token_ids for r in got] == [r.token_ids for r in got2]


def test_trace_replay_of_a_kolisun_folder(folders, tmp_path):
    import subprocess
    import sys
    import numpy as np
    folder = folders[("K", torch.float32)]
    cfg = _cfg(folder)
    toks = tiny.random_ids(30, cfg["vocab"], 9)
    ref = plain.forward(cfg, _weights(folder), toks, torch.float64)
    lines = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:11], "want": [0, 10]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[11:13], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[13:], "want": [16]}], "end": ["x"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(x) + "\n" for x in lines), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [x for x in r.stdout.split("\n") if x.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    a = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    b = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)
    for row, pos in ((a[0], 0), (a[1], 10), (b[0], 29)):
        assert float(np.abs(row - ref[pos].numpy()).max()) < 2e-4 * float(ref[pos].abs().max())


def test_command_line_generates_from_a_kolisun_folder(folders):
    import subprocess
    import sys
    folder = folders[("L", torch.float32)]
    cfg, w = _cfg(folder), _weights(folder)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "prelude"), "--model", folder, "--dtype", "f32", "--prompt-ids", "5,17,3,200",
                          "--max-new-tokens", "5", "--temperature", "0", "--num-pages", "16", "--page-size", "16", "--ignore-eos"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    seq = [5, 17, 3, 200]
    for _ in range(5):
        seq.append(int(plain.forward(cfg, w, seq, torch.float64)[-1].argmax()))
    assert json.loads(out.stdout.strip().splitlines()[0])["token_ids"] == seq[4:]


# -- the tensor-core general attention kernel against the plain kernel ----------------------------------------------------
@pytest.mark.parametrize("heads,kv,kd,vd,shared,page,window,sink", [
    (16, 1, 576, 512, True, 16, None, True), (6, 1, 112, 96, True, 16, None, True), (8, 2, 64, 128, False, 16, 100, False),
    (4, 4, 48, 96, False, 8, None, True), (128, 1, 96, 64, True, 32, None, False), (5, 1, 32, 32, True, 16, 33, True),
    (4, 2, 128, 64, False, 64, 700, False), (64, 2, 160, 160, True, 16, None, True)])
def test_tensor_core_general_attention_equals_the_plain_kernel(heads, kv, kd, vd, shared, page, window, sink):
    """Random keys and values in scattered pages; requests of unequal length: long portions, a portion of two tokens,
    single tokens far into a long context (their keys dealt to several blocks), with and without a window and a sink;
    then a step of single tokens only.  Both kernels read the same pages."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import kernels as K
    from prelude_b200.ops import paged_general as G
    from prelude_b200.parts.registry import KvPagesNeed
    dev = torch.device(DEV)
    g = torch.Generator().manual_seed(heads * 31 + kd)
    need = KvPagesNeed(kv, kd, window, v_heads=0, v_head_dim=0) if shared else KvPagesNeed(kv, kd, window, v_heads=kv, v_head_dim=vd)
    sinks = torch.linspace(-1.0, 3.0, heads).to(dev) if sink else None
    mixed = [(0, 150), (700, 2), (1500, 1), (130, 70), (63, 1)]
    decode = [(1900, 1), (5, 1), (640, 1)]
    for shape in (mixed, decode):
        cache = CacheManager([need], page, sum(-(-(a + b) // page) for a, b in shape) + 3, 8, dev, torch.bfloat16)
        items, slots = [], []
        for i, (have, new) in enumerate(shape):
            cache.add_request(i)
            cache.grow(i, have + new)
            items.append(StepItem(i, [0] * new, have, []))
            slots.append(cache.slot_of(i))
        lc = cache.layer_cache(0)
        lc.k_pages.copy_(torch.randn(lc.k_pages.shape, generator=g).to(dev, torch.bfloat16))
        v_pages = None
        if not shared:
            lc.v_pages.copy_(torch.randn(lc.v_pages.shape, generator=g).to(dev, torch.bfloat16))
            v_pages = lc.v_pages
        batch = build_step_batch(items, cache.block_tables(list(range(len(shape)))), slots, dev, 10, 1 << 20)
        q = (torch.randn(batch.n_tokens, heads, kd, generator=g) * 1.5).to(dev, torch.bfloat16)
        scale = 1.0 / math.sqrt(kd)
        assert G.tc_takes(q, lc.k_pages, v_pages, vd)
        got = G.attention_general(q, lc.k_pages, v_pages, vd, batch, 0, scale, window, sinks).float()
        want = K.attention_paged(q, lc.k_pages, v_pages, vd, batch.positions, batch.table_row_of_token, batch.block_tables[0], scale,
                                 window, sinks, status=batch.status).float()
        assert int(batch.status.item()) == 0
        err = (got - want).abs()
        assert float(err.max()) < 4e-2 * float(want.abs().max()) and float(err.mean()) < 4e-3 * float(want.abs().max()), \
            (float(err.max()), float(err.mean()), float(want.abs().max()))
