"""Pabelix on the GPU against the plain implementation: every mechanism alone, then whole models through every way
of cutting requests into steps, in 32-bit and in bfloat16, with pools so small that pages and slots are used again."""
import copy
import math

import pytest
import torch

import harness
import pabelix_tiny as pt
import tiny
from plain import pabelix_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: (2e-4, 0.0), torch.bfloat16: (0.0, 3e-2)}


def _weights(folder):
    return {k: v for k, v in tiny.read_weights(folder).items()}


def _cfg(folder):
    import json
    import os
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def _reference(folder, reqs):
    cfg, w = _cfg(folder), _weights(folder)
    return {rid: plain.forward(cfg, w, toks, torch.float64) for rid, toks in reqs.items()}


def _compare(got, ref, dtype, loosen=1.0):
    """Every position within the bound in 32-bit.  In bfloat16 the rounding of a router's input can turn a close call
    between two experts, and a head whose two maps nearly cancel is divided by a small root mean square, which
    multiplies the rounding of its scores: either changes a position's logits outright.  There the test asks that
    the typical position is well within the bound and no more than a quarter of them are off; a fault of the
    mechanism puts every position off, and the 32-bit runs of the same schedules are held to every position."""
    atol, rel = TOL[dtype]
    off, ratios = [], []
    for (rid, pos), row in got.items():
        want = ref[rid][pos]
        bound = loosen * (atol * max(1.0, float(want.abs().max())) + rel * float(want.abs().max()))
        diff = float((row.double() - want).abs().max())
        ratios.append(diff / bound)
        if diff > bound:
            off.append(f"request {rid} position {pos}: max diff {diff:.3e} > {bound:.3e}")
    allowed = len(got) // 4 if dtype == torch.bfloat16 else 0
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


# -- mechanisms alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("width", [40, 129, 256])
def test_embedding_adds_the_position_vector(dtype, width):
    from prelude_b200.ops import kernels as K
    g = torch.Generator().manual_seed(width)
    table = (torch.randn(50, width, generator=g) * 0.5).to(dtype)
    ids = torch.randint(0, 50, (9,), generator=g, dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 3, 1000, 4095, 70000, 17, 5], dtype=torch.int32)
    rate = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -torch.arange(0, width, 2, dtype=torch.float64) / width)
    out = K.embed_sinusoid(ids.to(DEV), pos.to(DEV), table.to(DEV), rate.to(DEV)).cpu()
    for r in range(9):
        want = table[ids[r]].double() + plain.sinusoid(1, width, start=int(pos[r]))[0]
        assert float((out[r].double() - want).abs().max()) < 2e-7 * (1 + float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("width", [40, 130, 12000])
def test_norm_of_a_sublayers_output_fused_with_the_add_and_the_next_norm(dtype, width):
    from prelude_b200.ops import kernels as K
    g = torch.Generator().manual_seed(1 + width)
    rows = 7
    x = (torch.randn(rows, width, generator=g) * 3).to(dtype)
    res = torch.randn(rows, width, generator=g)
    wx, w = torch.rand(width, generator=g) + 0.5, torch.rand(width, generator=g) + 0.5
    eps_x, eps = 1e-3, 1e-5
    normed = plain.unit_offset_norm(x.double(), wx.double() - 1.0, eps_x)
    want_res = res.double() + normed
    want_y = plain.unit_offset_norm(want_res, w.double() - 1.0, eps)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    res_d = res.to(DEV)
    pick = torch.tensor([5, 0, 5, 3], dtype=torch.int32, device=DEV)
    picked = K.normed_add_rmsnorm(K.Normed(x.to(DEV), wx.to(DEV), eps_x), res_d, w.to(DEV), eps, dtype, rows=pick)
    assert torch.equal(res_d.cpu(), res)                                             # the gather form leaves the stream alone
    assert float((picked.cpu().double() - want_y[pick.cpu().long()]).abs().max()) < tol * float(want_y.abs().max())
    y = K.normed_add_rmsnorm(K.Normed(x.to(DEV), wx.to(DEV), eps_x), res_d, w.to(DEV), eps, dtype)
    assert float((res_d.cpu().double() - want_res).abs().max()) < 1e-5 * float(want_res.abs().max())   # the sum is 32-bit in both modes
    assert float((y.cpu().double() - want_y).abs().max()) < tol * float(want_y.abs().max())
    res_d = res.to(DEV)
    assert K.normed_add_rmsnorm(K.Normed(x.to(DEV), wx.to(DEV), eps_x), res_d, None, eps, dtype) is None
    assert float((res_d.cpu().double() - want_res).abs().max()) < 1e-5 * float(want_res.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_clamped_gated_unit(dtype):
    from prelude_b200.ops import kernels as K
    g = torch.Generator().manual_seed(5)
    inter = 37
    gu = (torch.randn(11, 2 * inter, generator=g) * 2).to(dtype)
    a = gu[:, :inter].double().clamp(max=0.9)
    b = gu[:, inter:].double().clamp(-0.9, 0.9)
    want = a * torch.sigmoid(1.702 * a) * (b + 1)
    assert float(a.max()) == 0.9 and float(b.min()) == -0.9                          # the limits bind
    got = K.clamped_glu(gu.to(DEV), 0.9, 1.702).cpu().double()
    assert float((got - want).abs().max()) < (1e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("rows,width,inter", [(1, 64, 48), (7, 128, 256), (100, 64, 48), (900, 256, 384), (5, 40, 56)])
def test_clamped_unit_feed_forward_on_every_product_kernel(rows, width, inter):
    """Few rows: the streaming product with the unit in its epilogue; hundreds: the paired-block product with it; between
    them, and for widths that neither takes: the library product and the activation kernel.  All against the plain one."""
    from prelude_b200.config.spec import ClampedGluSpec
    from prelude_b200.parts.registry import RunContext, make_part
    g = torch.Generator().manual_seed(rows + inter)
    w = {"gate": (torch.randn(inter, width, generator=g) * 0.3).bfloat16(), "up": (torch.randn(inter, width, generator=g) * 0.3).bfloat16(),
         "down": (torch.randn(width, inter, generator=g) * 0.1).bfloat16()}
    x = torch.randn(rows, width, generator=g).bfloat16()
    want = plain.clamped_glu(x.double(), {k: v.double() for k, v in w.items()}, 0.7)
    part = make_part("feed_forward", ClampedGluSpec(width, inter, 0.7), "ff")
    part.load(lambda name: w[name[len("ff."):]], RunContext(torch.device(DEV), torch.bfloat16))
    got = part.forward(x.to(DEV))
    got = got.materialize(torch.bfloat16) if hasattr(got, "materialize") else got
    assert float((got.cpu().double() - want).abs().max()) < 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("experts,top,groups,keep", [(12, 3, 3, 2), (8, 1, 1, 1), (6, 2, 6, 3), (16, 4, 2, 1), (5, 5, 1, 1), (64, 6, 8, 3)])
def test_router_choice_equals_the_plain_one(experts, top, groups, keep):
    from prelude_b200.ops import kernels as K
    g = torch.Generator().manual_seed(experts * 100 + top)
    z = torch.randn(300, experts, generator=g) * 2
    ids, w = K.moe_route(z.to(DEV), top, groups, keep, 2, False)
    want_ids, want_w = plain.route(z.double(), top, groups, keep)
    ids, w = ids.cpu().long(), w.cpu().double()
    order, want_order = ids.sort(dim=1), want_ids.sort(dim=1)
    assert torch.equal(order.values, want_order.values)
    assert float((w.gather(1, order.indices) - want_w.gather(1, want_order.indices)).abs().max()) < 1e-6
    # a largest score outside the kept groups is never chosen
    if keep < groups:
        per = experts // groups
        s = torch.sigmoid(z.double()).reshape(300, groups, per)
        gscore = s.topk(min(2, per), dim=-1).values.sum(-1)
        kept = gscore.topk(keep, dim=-1).indices
        assert all(int(e) // per in kept[t].tolist() for t in range(300) for e in ids[t])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("tokens,width,ff,experts,top", [(1, 40, 24, 6, 2), (150, 72, 10, 5, 1), (333, 64, 64, 8, 3), (70, 128, 40, 4, 4),
                                                         (1200, 64, 64, 4, 2), (700, 128, 40, 3, 1), (2100, 256, 320, 6, 3)])
def test_routed_experts_equal_the_plain_mixture(dtype, tokens, width, ff, experts, top):
    from prelude_b200.config.spec import RoutedExpertsSpec
    from prelude_b200.parts.registry import RunContext, make_part
    g = torch.Generator().manual_seed(tokens + width)
    w = {"router": torch.randn(experts, width, generator=g) * 0.3}
    for e in range(experts):
        w[f"e{e}.gate"] = torch.randn(ff, width, generator=g) * 0.2
        w[f"e{e}.up"] = torch.randn(ff, width, generator=g) * 0.2
        w[f"e{e}.down"] = torch.randn(width, ff, generator=g) * 0.2
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(tokens, width, generator=g).to(dtype)
    r = {"top": top, "groups": {"count": 1, "keep": 1}}
    want = plain.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, r)
    part = make_part("feed_forward", RoutedExpertsSpec(width, ff, experts, top), "ff")
    part.load(lambda name: w[name[len("ff."):]], RunContext(torch.device(DEV), dtype))
    got = part.forward(x.to(DEV)).cpu().double()
    # many rows per expert in bfloat16: the paired-block tcgen05 product; fewer: the 128-row or the 64-row tiles
    assert part.pair_takes(x.to(DEV)) == (dtype == torch.bfloat16 and tokens * top >= 192 * experts and ff >= 64)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol * float(want.abs().max())
    # a token's result does not depend on who else is in the step
    alone = part.forward(x[:1].to(DEV).contiguous()).cpu().double()
    assert float((alone - got[:1]).abs().max()) < (1e-6 if dtype == torch.float32 else 2e-2) * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("heads,kv,dim,vdim,page", [(4, 2, 12, 20, 4), (2, 1, 64, 64, 16), (3, 3, 7, 33, 8), (8, 2, 32, 128, 16), (4, 4, 128, 96, 32)])
def test_differential_attention_mixer_equals_the_plain_one(dtype, heads, kv, dim, vdim, page):
    """The mixer alone over a prompt of 75 tokens and then token by token, with one query and key scaled so that a
    key far back carries one map: a lost far key, a wrong key head or a swapped map changes the output at once."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.config.spec import DiffAttentionSpec, QueryTemperatureSpec
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.parts.registry import RunContext, make_part
    width, T, head_tokens = 48, 90, 75
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 1.0 / math.sqrt(dim), "diff": 0.35,
         "q_temp": {"coef": 0.6, "every": 8}}
    w = {"q": torch.randn(heads * 2 * dim, width, generator=g) * 0.3, "k": torch.randn(kv * 2 * dim, width, generator=g) * 0.3,
         "v": torch.randn(kv * vdim, width, generator=g) * 0.3, "g": torch.randn(heads * vdim, width, generator=g) * 0.2,
         "o": torch.randn(width, heads * vdim, generator=g) * 0.2}
    for n in ("lq1", "lk1", "lq2", "lk2"):
        w[n] = torch.randn(dim, generator=g) * 0.4
    w = {k: v.to(dtype) for k, v in w.items()}
    x = torch.randn(T, width, generator=g)
    # position 2: a key that later queries find far back (in bfloat16 less so: scores of tens round by tenths)
    x[2] *= 6.0 if dtype == torch.float32 else 2.0
    x = x.to(dtype)
    want, _ = plain.diff_attention(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-5)
    spec = DiffAttentionSpec(width, heads, kv, dim, vdim, m["scale"], 0.35, 1e-5, QueryTemperatureSpec(0.6, 8))
    part = make_part("mixer", spec, "mix")
    ctx = RunContext(torch.device(DEV), dtype)
    part.load(lambda name: w[name[len("mix."):]], ctx)
    cache = CacheManager([part.cache_need()], page, -(-T // page), 2, ctx.device, dtype)
    cache.add_request("a")
    got = []
    at = 0
    for n in [head_tokens] + [1] * (T - head_tokens):
        cache.grow("a", at + n)
        batch = build_step_batch([StepItem("a", [0] * n, at, [])], cache.block_tables(["a"]), [cache.slot_of("a")], ctx.device, 10, 1 << 20)
        got.append(part.forward(x[at:at + n].to(DEV).contiguous(), batch, cache.layer_cache(0), True).float().cpu())
        assert int(batch.status.item()) == 0
        at += n
    got = torch.cat(got).double()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert float((got - want).abs().max()) < tol * float(want.abs().max())


# -- whole models ----------------------------------------------------------------------------------------------------
REQUESTS = {"P": {"p1": 1, "p2": 2, "p19": 19, "p70": 70, "p33": 33}, "Q": {"q3": 3, "q150": 150, "q64": 64, "q41": 41, "q97": 97}}


def _requests(which):
    v = pt.PARAMS[which][0]["vocab"]
    return {rid: tiny.random_ids(n, v, sum(map(ord, rid))) for rid, n in REQUESTS[which].items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("pabelix")
    return {(w, d): pt.make_folder(root, w, d) for w in "PQ" for d in (torch.float32, torch.bfloat16)}


@pytest.fixture(scope="module")
def references(folders):
    return {w: _reference(folders[(w, torch.bfloat16)], _requests(w)) for w in "PQ"}, \
           {w: _reference(folders[(w, torch.float32)], _requests(w)) for w in "PQ"}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["P", "Q"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed", "mixed_graphs"])
def test_cuts_match_plain(folders, references, which, dtype, cut):
    """Whole prompts, a decoded tail that crosses temperature steps and page borders, portions down to two tokens, and
    mixed batches in a pool that holds less than all requests (pages and slots used again), launched and captured."""
    reqs = _requests(which)
    ref = references[0 if dtype == torch.bfloat16 else 1][which]
    page = pt.PARAMS[which][2]
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


def test_batched_requests_equal_each_alone_in_32_bit(folders):
    reqs = _requests("P")
    page = 4
    alone = harness.run_schedule(_runner(folders[("P", torch.float32)], torch.float32, page, 64), harness.whole(reqs))
    together = harness.run_schedule(_runner(folders[("P", torch.float32)], torch.float32, page, 64, max_slots=5),
                                    [([(rid, toks, list(range(len(toks)))) for rid, toks in reqs.items()], list(reqs))])
    for key, row in alone.items():
        assert float((row - together[key]).abs().max()) <= 2e-5 * float(row.abs().max()), key


def test_sharp_attention_finds_keys_far_back_and_at_page_borders(tmp_path):
    """Query and key matrices scaled up make every softmax pick few keys, wherever they lie: among hundreds of keys,
    at the first positions, on either side of a page border.  32-bit, prompt in one step and in portions with a decoded tail."""
    cfg = copy.deepcopy(pt.PABELIX_P)
    tensors = pt.random_tensors(cfg, seed=21, std=0.25, norm_jitter=0.3)
    for name in list(tensors):
        if name.endswith(".mix.q") or name.endswith(".mix.k"):
            tensors[name] = tensors[name] * 2.0
    folder = pt.make_folder_from_tensors(tmp_path, "sharp", cfg, tensors)
    reqs = {"s": tiny.random_ids(300, cfg["vocab"], 77)}
    ref = _reference(folder, reqs)
    for schedule in (harness.whole(reqs), harness.portions(reqs, (37, 2, 64, 3, 29)), harness.tail_decode(reqs, 70)):
        got = harness.run_schedule(_runner(folder, torch.float32, 16, 19), schedule)
        _compare(got, ref, torch.float32, loosen=5.0)        # scores of tens: their 32-bit rounding shows in the weights


def test_long_decoding_through_freed_and_reused_slots(folders):
    """Two requests decoded token by token for 120 steps side by side after short prompts, then a third takes the
    slot and pages that the first gave back."""
    cfg = pt.PABELIX_P
    reqs = {"a": tiny.random_ids(130, cfg["vocab"], 1), "b": tiny.random_ids(127, cfg["vocab"], 2), "c": tiny.random_ids(60, cfg["vocab"], 3)}
    ref = _reference(folders[("P", torch.float32)], reqs)
    steps = [([("a", reqs["a"][:10], list(range(10))), ("b", reqs["b"][:7], list(range(7)))], [])]
    for i in range(120):
        steps.append(([("a", reqs["a"][10 + i:11 + i], [0]), ("b", reqs["b"][7 + i:8 + i], [0])], ["a", "b"] if i == 119 else []))
    steps.append(([("c", reqs["c"], list(range(60)))], ["c"]))
    runner = _runner(folders[("P", torch.float32)], torch.float32, 4, 66, max_slots=2)
    _compare(harness.run_schedule(runner, steps), ref, torch.float32)
    runner.cache.check()


@pytest.mark.parametrize("which,lens,new", [("P", [1, 5, 17], 20), ("Q", [9, 64, 2, 31], 12)])
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
    eng = Engine(folder, dtype="f32", page_size=pt.PARAMS[which][2], num_pages=64, max_running_requests=4)
    got = eng.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)
    assert [r.token_ids for r in got] == want
    # portions of a few tokens beside decoding requests, launched kernel by kernel: the same tokens
    eng2 = Engine(folder, dtype="f32", page_size=pt.PARAMS[which][2], num_pages=64, max_running_requests=4,
                  max_num_batched_tokens=7, long_prefill_token_threshold=3, cuda_graph=False)
    assert [r.token_ids for r in eng2.generate(prompts, temperature=0.0, max_new_tokens=new, ignore_eos=True)] == want
    assert eng.cache.used_pages() == 0 and eng2.cache.used_pages() == 0


def test_trace_replay_of_a_pabelix_folder(folders, tmp_path):
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    folder = folders[("P", torch.float32)]
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


# -- the tensor-core attention kernel against the plain kernel -----------------------------------------------------------
@pytest.mark.parametrize("heads,kv,dim,vdim,page,window", [(8, 2, 64, 128, 16, None), (4, 4, 48, 80, 16, None), (16, 2, 128, 64, 32, None),
                                                        (6, 2, 32, 32, 8, 100), (2, 1, 256, 256, 64, None), (4, 1, 16, 240, 16, 33), (32, 1, 32, 64, 16, None)])
def test_tensor_core_attention_equals_the_plain_kernel(heads, kv, dim, vdim, page, window):
    """Random keys and values in scattered pages; requests of unequal length: long portions, a portion of two tokens,
    single tokens far into a long context (their keys cut into ranges), with and without a window; then a step of
    single tokens only.  Both kernels read the same pages."""
    from prelude_b200.cache.manager import CacheManager
    from prelude_b200.config.spec import DiffAttentionSpec, QueryTemperatureSpec
    from prelude_b200.engine.batch import StepItem, build_step_batch
    from prelude_b200.ops import diff_attention as D
    from prelude_b200.ops import kernels as K
    from prelude_b200.parts.registry import KvPagesNeed
    dev = torch.device(DEV)
    g = torch.Generator().manual_seed(heads * 31 + dim)
    spec = DiffAttentionSpec(64, heads, kv, dim, vdim, 1.0 / math.sqrt(dim), 0.3, 1e-6, QueryTemperatureSpec(0.4, 64), window=window)
    # (tokens already in the cache, tokens of this step)
    mixed = [(0, 150), (700, 2), (1500, 1), (130, 70), (63, 1)]
    decode = [(1900, 1), (5, 1), (640, 1)]
    for shape in (mixed, decode):
        total = sum(a + b for a, b in shape)
        cache = CacheManager([KvPagesNeed(2 * kv, dim, None, kv, vdim)], page, sum(-(-(a + b) // page) for a, b in shape) + 3, 8, dev, torch.bfloat16)
        items, slots = [], []
        for i, (have, new) in enumerate(shape):
            cache.add_request(i)
            cache.grow(i, have + new)
            items.append(StepItem(i, [0] * new, have, []))
            slots.append(cache.slot_of(i))
            # what earlier steps left: keys and values of the first `have` positions
            if have:
                fill = build_step_batch([StepItem(i, [0] * have, 0, [])], cache.block_tables([i]), [slots[-1]], dev, 10, 1 << 20)
                K.kv_write_pages((torch.randn(have, 2 * kv * dim, generator=g)).to(dev, torch.bfloat16),
                                 torch.randn(have, kv * vdim, generator=g).to(dev, torch.bfloat16), cache.layer_cache(0).k_pages,
                                 cache.layer_cache(0).v_pages, fill.positions, fill.table_row_of_token, fill.block_tables[0])
        batch = build_step_batch(items, cache.block_tables(list(range(len(shape)))), slots, dev, 10, 1 << 20)
        T = batch.n_tokens
        lc = cache.layer_cache(0)
        K.kv_write_pages(torch.randn(T, 2 * kv * dim, generator=g).to(dev, torch.bfloat16), torch.randn(T, kv * vdim, generator=g).to(dev, torch.bfloat16),
                         lc.k_pages, lc.v_pages, batch.positions, batch.table_row_of_token, batch.block_tables[0])
        proj = torch.randn(T, heads * 2 * dim + heads * vdim, generator=g).to(dev, torch.bfloat16)
        q, gate = proj[:, :heads * 2 * dim], proj[:, heads * 2 * dim:]
        got = D.diff_attention(q, gate, lc.k_pages, lc.v_pages, batch, 0, spec, 0.8).float()
        want = K.diff_attention_ref(q, gate, lc.k_pages, lc.v_pages, batch.positions, batch.table_row_of_token, batch.block_tables[0], heads,
                                    spec.softmax_scale, 0.4, 64, 0.8, 1e-6, 0.7, window, batch.status).float()
        assert int(batch.status.item()) == 0
        assert bool(D._l.library().pb_diff_attention_tc_supported(heads, kv, dim, vdim, q.stride(0)))
        err = (got - want).abs()
        assert float(err.max()) < 4e-2 * float(want.abs().max()) and float(err.mean()) < 4e-3 * float(want.abs().max()), \
            (float(err.max()), float(err.mean()), float(want.abs().max()))


def test_command_line_generates_from_a_pabelix_folder(folders):
    import json
    import os
    import subprocess
    import sys
    folder = folders[("Q", torch.float32)]
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
