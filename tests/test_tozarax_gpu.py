"""The Tozarax decoder on the GPU against the plain numpy restatement in oracle/tozarax.py.

Small random configurations of the tests' own; the product runs through the C ABI (models.TozaraxWithConfig /
DeviceCache.forward_ragged), the oracle token by token in float64.  Two precisions: "f32" (every product and the cache in 32-bit)
against the exact oracle; "bf16" (the serving precision: tensor-core GEMMs over hi | lo activation halves, bf16 key / value cache)
against the oracle that rounds the keys and values it caches to bf16.
"""
import copy
import json
import os
import subprocess

import numpy as np
import pytest

from fastllm_b200 import models
from fastllm_b200._lib import FastllmError
from oracle import tozarax as O

pytestmark = pytest.mark.gpu

TOL = {"f32": 4e-5, "bf16": 1e-2}


# ---- configurations ---------------------------------------------------------------------------------------------------------
def left(heads=4, kv_heads=2, dim=8, vdim=12, window=9, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale if scale is not None else dim ** -0.5}


def right(heads=4, kv_heads=2, dim=6, vdim=10, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def moe(experts=8, top=2, ff=12, groups=4, keep=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def layer(a=None, b=None, mlp="default"):
    return {"type": "parallel", "mixer": {"left": a or left(), "right": b or right()}, "mlp": moe() if mlp == "default" else mlp}


def config(layers, vocab=48, width=32, eps=1e-5, taps=3, max_positions=512):
    return {"architecture": "Tozarax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "max_positions": max_positions,
            "layers": layers}


def deep_cfg(**kw):
    """four unequal layers: with and without experts, other head counts and windows, groups of one expert, every expert eligible"""
    return config([layer(),
                   layer(left(heads=2, kv_heads=2, dim=10, vdim=6, window=70), right(heads=3, kv_heads=3, dim=4, vdim=12, conv=2), mlp=None),
                   layer(left(heads=6, kv_heads=1, dim=4, vdim=8, window=3, scale=0.7), right(heads=6, kv_heads=2, dim=8, vdim=4, conv=4),
                         mlp=moe(experts=6, top=3, ff=10, groups=6, keep=4)),
                   layer(left(heads=1, kv_heads=1, dim=16, vdim=16, window=200), right(heads=2, kv_heads=1, dim=12, vdim=20, conv=3),
                         mlp=moe(experts=4, top=1, ff=20, groups=1, keep=1))], **kw)


# ---- helpers ----------------------------------------------------------------------------------------------------------------
def to_bits(a):
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


_built = {}


def build(cfg, seed=0, dtype="f32", tweak=None):
    """-> (oracle, product adapter); weights are bf16-representable, handed over as bf16 bit patterns"""
    key = (repr(cfg), seed, dtype, tweak.__name__ if tweak else None)
    if key not in _built:
        w = O.random_weights(cfg, seed)
        if tweak:
            tweak(w)
        model, _ = models.TozaraxWithConfig.initialize_model(cfg, {k: to_bits(v) for k, v in w.items()}, dtype)
        _built[key] = (O.Tozarax(cfg, w, cache_round=O.to_bf16 if dtype == "bf16" else None), model)
    return _built[key]


def relerr(got, ref, allow=0.0):
    """worst position's error: rms over the vocabulary of the logits' difference (means taken off) relative to the rms of the
    logits.  allow: share of positions left out, worst first (long serving-precision runs only: a 1e-3 change upstream of a random
    router can flip a near-tied expert pick; the exact mode never needs it)."""
    d = np.asarray(got, dtype=np.float64) - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    e = np.sort(np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1)))
    return float(e[len(e) - 1 - int(allow * len(e))])


def tokens(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def run_whole(model, toks, slot=0, cache=None):
    cache = cache or model.new_device_cache(max_batch=4, max_seq=max(64, len(toks)))
    return cache.forward_ragged([slot], [toks], [list(range(len(toks)))])


def run_cut(model, toks, cuts, slot=0, cache=None):
    """feed the tokens in portions of the given sizes (the rest one by one) and collect every position's logits"""
    cache = cache or model.new_device_cache(max_batch=4, max_seq=max(64, len(toks)))
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = min(sizes.pop(0) if sizes else 1, len(toks) - at)
        out.append(cache.forward_ragged([slot], [toks[at:at + n]], [list(range(n))]))
        at += n
    return np.concatenate(out)


# ---- each mechanism alone ---------------------------------------------------------------------------------------------------
MECHANISMS = {
    "plain": config([layer()]),
    "no_experts": config([layer(mlp=None)]),
    "window_of_one": config([layer(left(window=1), mlp=None)]),
    "window_of_two_one_kv_head": config([layer(left(heads=6, kv_heads=1, dim=12, vdim=20, window=2, scale=1.5), mlp=None)]),
    "attention_equal_heads": config([layer(left(heads=3, kv_heads=3, dim=6, vdim=4, window=30), mlp=None)]),
    "delta_shared_keys": config([layer(b=right(heads=6, kv_heads=1, dim=12, vdim=40, conv=5), mlp=None)], width=40),
    "delta_equal_heads_one_tap": config([layer(b=right(heads=2, kv_heads=2, dim=16, vdim=8, conv=1), mlp=None)]),
    "input_conv_one_tap": config([layer()], taps=1),
    "input_conv_two_taps": config([layer()], taps=2),
    "input_conv_six_taps": config([layer(), layer()], taps=6),
    "router_one_group": config([layer(mlp=moe(experts=6, top=2, ff=16, groups=1, keep=1))]),
    "router_groups_of_one": config([layer(mlp=moe(experts=5, top=2, ff=16, groups=5, keep=3))]),
    "router_all_groups_kept_top_one": config([layer(mlp=moe(experts=8, top=1, ff=7, groups=2, keep=2))]),
    "router_takes_all_eligible": config([layer(mlp=moe(experts=9, top=6, ff=9, groups=3, keep=2))]),
    "one_expert": config([layer(mlp=moe(experts=1, top=1, ff=24, groups=1, keep=1))]),
    "one_head": config([layer(left(heads=1, kv_heads=1, dim=16, vdim=8, window=5), right(heads=1, kv_heads=1, dim=16, vdim=16))]),
    "three_layers_depth_average": config([layer(), layer(mlp=None), layer()]),
}


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_mechanism_alone(name, dtype):
    cfg = MECHANISMS[name]
    oracle, model = build(cfg, seed=3, dtype=dtype)
    toks = tokens(cfg, 37)
    assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL[dtype]


def test_odd_sizes_every_mechanism():
    """sizes that are no multiple of 4 / 8 / 32 anywhere, more than 32 value columns, 70 tokens across a page border"""
    cfg = config([layer(left(heads=6, kv_heads=3, dim=10, vdim=14, window=66), right(heads=5, kv_heads=5, dim=9, vdim=35, conv=4),
                        mlp=moe(experts=15, top=4, ff=11, groups=5, keep=3)),
                  layer(left(heads=3, kv_heads=1, dim=7, vdim=34, window=13), right(heads=3, kv_heads=1, dim=11, vdim=5, conv=2),
                        mlp=moe(experts=7, top=3, ff=22, groups=1, keep=1))], vocab=37, width=50, taps=5)
    oracle, model = build(cfg, seed=5)
    toks = tokens(cfg, 70)
    assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL["f32"]


def tc_cfg():
    """widths in whole 64-column blocks: in the serving precision the projections, the gates and the experts (grouped GEMM pair
    for few rows, every expert over all rows for many) run on the tensor-core GEMM; the delta rule's rows of the stacked input
    matrix start behind the attention's and end in a few per-head rows (padded to a multiple of 8)"""
    return config([layer(left(heads=4, kv_heads=2, dim=32, vdim=16, window=50), right(heads=4, kv_heads=2, dim=16, vdim=32, conv=4),
                         mlp=moe(experts=8, top=2, ff=64, groups=4, keep=2)),
                   layer(left(heads=8, kv_heads=2, dim=16, vdim=16, window=150), right(heads=2, kv_heads=2, dim=32, vdim=64, conv=3),
                         mlp=moe(experts=4, top=3, ff=128, groups=2, keep=2))], vocab=96, width=128, taps=4)


def tc_cfg_partial_tiles():
    """320-wide: five 64-column k blocks, matrices that end inside a 128-row tile; the first layer's experts lie outside the tiles
    (ff = 100) and run on the plain kernel beside tensor-core projections"""
    return config([layer(left(heads=3, kv_heads=1, dim=48, vdim=64, window=90), right(heads=3, kv_heads=3, dim=64, vdim=64, conv=4),
                         mlp=moe(experts=6, top=2, ff=100, groups=3, keep=2)),
                   layer(left(heads=6, kv_heads=3, dim=32, vdim=24, window=64), right(heads=3, kv_heads=1, dim=24, vdim=40, conv=2),
                         mlp=moe(experts=6, top=2, ff=320, groups=2, keep=1))], vocab=200, width=320)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("make", [tc_cfg, tc_cfg_partial_tiles])
def test_tensor_core_projections(make, dtype):
    """1 row, a few rows, up to 128 rows (weights as the 128-row operand, split-K) and more (tokens as rows) through the same layers;
    portions of 64 tokens and more also take the attention through the tensor-core GEMMs, with the window cutting into them"""
    cfg = make()
    oracle, model = build(cfg, seed=21, dtype=dtype)
    toks = tokens(cfg, 333, seed=9)
    ref = oracle.run(toks)
    allow = 0.02 if dtype == "bf16" else 0.0
    assert relerr(run_whole(model, toks, cache=model.new_device_cache(4, 384)), ref, allow) < TOL[dtype]
    assert relerr(run_cut(model, toks, [5, 128, 129, 2, 60], cache=model.new_device_cache(4, 384)), ref, allow) < TOL[dtype]


# ---- schedules: whole prompt, token by token, portions, batches ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_prefill_equals_token_by_token(dtype):
    cfg = deep_cfg()
    oracle, model = build(cfg, seed=7, dtype=dtype)
    toks = tokens(cfg, 90)
    ref = oracle.run(toks)
    whole, single = run_whole(model, toks), run_cut(model, toks, [])
    assert relerr(whole, ref) < TOL[dtype] and relerr(single, ref) < TOL[dtype]
    assert relerr(single, np.asarray(whole, dtype=np.float64)) < TOL[dtype]


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 2], [5, 64, 2, 17], [63, 2, 64], [1, 66, 2, 2, 2, 40], [3, 1, 1, 2, 1, 3, 1, 1, 1, 4]])
def test_portions(cuts):
    """a prompt cut into portions (down to two tokens and single ones: shorter than the convolutions reach back, so a row's taps
    come from this step, from the slot's carried inputs and from before the start at once), across page borders, the rest decoded"""
    cfg = deep_cfg(taps=4)
    oracle, model = build(cfg, seed=8)
    toks = tokens(cfg, 150, seed=4)
    assert relerr(run_cut(model, toks, cuts), oracle.run(toks)) < TOL["f32"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mixed_batch_equals_each_alone(dtype):
    """three requests of unequal length advance together: portions of one beside single tokens of another"""
    cfg = deep_cfg()
    oracle, model = build(cfg, seed=9, dtype=dtype)
    reqs = [tokens(cfg, n, seed=s) for n, s in ((75, 1), (9, 2), (40, 3))]
    cache = model.new_device_cache(max_batch=4, max_seq=128, pool_tokens=4 * 64)
    plan = [[(0, 3), (1, 1)], [(0, 30), (1, 1), (2, 2)], [(2, 38), (1, 7), (0, 1)], [(0, 41)]]
    at, got = [0, 0, 0], [[], [], []]
    slot = {0: 2, 1: 0, 2: 3}
    for step in plan:
        parts = [reqs[r][at[r]:at[r] + n] for r, n in step]
        lg = cache.forward_ragged([slot[r] for r, _ in step], parts, [list(range(len(p))) for p in parts])
        row = 0
        for (r, n), p in zip(step, parts):
            got[r].append(lg[row:row + len(p)])
            row += len(p)
            at[r] += len(p)
    for r in range(3):
        assert at[r] == len(reqs[r])
        alone = run_whole(model, reqs[r])
        together = np.concatenate(got[r])
        assert relerr(together, oracle.run(reqs[r])) < TOL[dtype]
        assert relerr(together, np.asarray(alone, dtype=np.float64)) < TOL[dtype]


def test_pages_and_slots_reused():
    """a pool of three pages and two slots serves seven requests one after another and two at a time; what a finished request left
    in its pages, its state slot and its carried convolution inputs (the mixers' and both sublayers' input convolutions) must not
    leak into the next one"""
    cfg = deep_cfg()
    oracle, model = build(cfg, seed=10)
    cache = model.new_device_cache(max_batch=2, max_seq=192, pool_tokens=192)
    assert cache.pool_stats() == (3, 3)
    for i, n in enumerate((130, 100, 64, 65, 3, 1, 2)):
        toks = tokens(cfg, n, seed=20 + i)
        slot = i % 2
        assert relerr(run_whole(model, toks, slot=slot, cache=cache), oracle.run(toks)) < TOL["f32"]
        assert cache.slot_len(slot) == n and cache.pool_stats()[1] == 3 - (n + 63) // 64
        cache.slot_reset(slot)
        assert cache.pool_stats() == (3, 3)
    a, b = tokens(cfg, 100, seed=31), tokens(cfg, 60, seed=32)
    lg = cache.forward_ragged([1, 0], [a, b], [list(range(100)), list(range(60))])
    assert cache.pool_stats()[1] == 0
    assert relerr(lg[:100], oracle.run(a)) < TOL["f32"] and relerr(lg[100:], oracle.run(b)) < TOL["f32"]
    with pytest.raises(FastllmError):          # b would need a second page: the pool is empty, nothing is changed
        cache.forward_ragged([0], [tokens(cfg, 10)], None)
    assert cache.slot_len(0) == 60
    cache.slot_reset(1)
    more = tokens(cfg, 10, seed=33)
    lg = cache.forward_ragged([0], [more], [list(range(10))])
    assert relerr(lg, oracle.run(b + more)[60:]) < TOL["f32"]
    # a request decoded token by token in a slot whose previous owner left a long state behind
    cache.slot_reset(0)
    short = tokens(cfg, 6, seed=34)
    assert relerr(run_cut(model, short, [], slot=0, cache=cache), oracle.run(short)) < TOL["f32"]


# ---- the window's edge, far tokens, every stack option: made to stand out -----------------------------------------------------
def _sharp(w):
    """query and key projections of the attention scaled up: the softmax is nearly one-hot, so a key that is wrongly dropped,
    wrongly admitted or taken from a wrong page moves the logits"""
    for k in w:
        if k.endswith("left.q") or k.endswith("left.k"):
            w[k] = O.to_bf16(w[k] * 4.0)


def _other_window(cfg, delta):
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        l["mixer"]["left"]["mask"]["size"] += delta
    return c


@pytest.mark.parametrize("window", [1, 2, 5, 63, 64, 65, 130])
def test_window_edges_in_prompts_and_decoding(window):
    """windows of one key, within a page, of exactly a page, just over it and over two pages: a whole prompt, portions that cut the
    window, and single tokens; the oracle itself with a window one key wider or narrower is far outside the bar"""
    cfg = config([layer(left(window=window, scale=1.0), mlp=None), layer(left(heads=2, kv_heads=1, window=window, scale=1.0))])
    oracle, model = build(cfg, seed=11, tweak=_sharp)
    toks = tokens(cfg, 210, seed=5)
    ref = oracle.run(toks)
    for d in (-1, 1):
        if window + d >= 1:
            assert relerr(O.Tozarax(_other_window(cfg, d), oracle.w).run(toks), ref) > 100 * TOL["f32"]
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [window, 2, 61, 66]), ref) < TOL["f32"]
    _, served = build(cfg, seed=11, dtype="bf16", tweak=_sharp)
    ref16 = O.Tozarax(cfg, oracle.w, cache_round=O.to_bf16).run(toks)
    assert relerr(run_whole(served, toks), ref16, 0.02) < TOL["bf16"]                   # long portions: attention on the tensor-core GEMMs
    assert relerr(run_cut(served, toks, [70, 2, 100]), ref16, 0.02) < TOL["bf16"]


def _long_memory(w):
    """slow decays: the delta rule's state forgets slowly, tokens hundreds of positions back still count"""
    for k in w:
        if k.endswith("A_log"):
            w[k] = O.to_bf16(np.full_like(w[k], -6.0))
        if k.endswith("dt_bias"):
            w[k] = O.to_bf16(np.full_like(w[k], -1.0))


def test_far_tokens_reach_through_the_state():
    """windows of four keys: only the recurrent state carries the first token to position 400"""
    lay = layer(left(window=4), right(dim=64), mlp=None)
    cfg = config([lay, copy.deepcopy(lay)])
    oracle, model = build(cfg, seed=12, tweak=_long_memory)
    toks = tokens(cfg, 400, seed=6)
    ref = oracle.run(toks)
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert relerr(oracle.run(other)[-1:], ref[-1:]) > 100 * TOL["f32"]
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [2, 300, 2]), ref) < TOL["f32"]


def test_every_stack_option_would_show():
    """the oracle itself with one piece taken out is far outside the bar the product is held to: positions, input convolutions,
    contribution gates, depth average, the choice correction, the group limit, the per-mixer output norms"""
    cfg = config([layer(), layer(mlp=moe(experts=8, top=2, ff=12, groups=4, keep=1)), layer()])
    w = O.random_weights(cfg, 13)
    toks = tokens(cfg, 40, seed=5)
    ref = O.Tozarax(cfg, w).run(toks)
    _, model = build(cfg, seed=13)
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]

    def without(change):
        v = {k: np.array(a, copy=True) for k, a in w.items()}
        change(v)
        return relerr(O.Tozarax(cfg, v).run(toks), ref)

    def zero(pattern):
        def f(v):
            for k in v:
                if pattern in k:
                    v[k][...] = 0.0
        return f

    def newest_only(v):
        for k in v:
            if k.endswith(".dwa"):
                v[k][...] = 0.0
                v[k][-1] = 1.0
    assert without(zero("pos")) > 100 * TOL["f32"]
    assert without(zero(".canon")) > 100 * TOL["f32"]
    assert without(zero(".rg")) > 100 * TOL["f32"]              # every gate becomes one half
    assert without(newest_only) > 100 * TOL["f32"]
    assert without(zero("correction")) > 100 * TOL["f32"]
    assert without(lambda v: v.__setitem__("l0.mix.left.out", np.ones_like(v["l0.mix.left.out"]))) > 100 * TOL["f32"]
    loose = copy.deepcopy(cfg)
    loose["layers"][1]["mlp"]["router"]["groups"]["keep"] = 4
    assert relerr(O.Tozarax(loose, w).run(toks), ref) > 100 * TOL["f32"]


def test_router_choice_in_closed_form():
    """the expert with the largest choice score of all sits in a group whose second expert drags the group's mark down: it is
    never chosen; a negative choice score still counts inside a kept group; weights are the uncorrected scores"""
    s = np.array([0.9, 0.5, 0.1, 0.1, 0.3, 0.2])
    z = np.log(s / (1.0 - s))
    corr = np.array([0.0, -2.5, 0.0, 0.0, 0.0, 0.0])            # choice scores 0.9, -2.0 | 0.1, 0.1 | 0.3, 0.2 -> marks -1.1, 0.2, 0.5
    chosen, wts = O.route(z, corr, top=3, n_groups=3, keep=2)
    assert chosen.tolist() == [4, 5, 2] and np.allclose(wts, [0.3, 0.2, 0.1])
    chosen, wts = O.route(z, corr, top=2, n_groups=3, keep=3)
    assert chosen.tolist() == [0, 4] and np.allclose(wts, [0.9, 0.3])
    chosen, wts = O.route(z, corr, top=2, n_groups=3, keep=1)
    assert chosen.tolist() == [4, 5]
    chosen, wts = O.route(z, corr - 5.0, top=1, n_groups=1, keep=1)             # all choice scores negative
    assert chosen.tolist() == [0] and np.allclose(wts, [0.9])


def test_first_tokens():
    cfg = deep_cfg(taps=5)
    oracle, model = build(cfg, seed=13)
    for n in (1, 2, 3, 5):
        toks = tokens(cfg, n, seed=n)
        assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL["f32"]
        assert relerr(run_cut(model, toks, []), oracle.run(toks)) < TOL["f32"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_long_decoding(dtype):
    cfg = deep_cfg()
    oracle, model = build(cfg, seed=14, dtype=dtype)
    toks = tokens(cfg, 330, seed=7)
    assert relerr(run_cut(model, toks, [10]), oracle.run(toks), 0.02 if dtype == "bf16" else 0.0) < TOL[dtype]


def test_steps_of_more_than_a_thousand_rows():
    """long steps take the input convolution through blocks that walk several rows: two requests in one step, the border between
    them inside a block of rows, then portions that start in the middle of such a block"""
    cfg = config([layer(left(window=100)), layer(left(heads=2, kv_heads=1, window=7), mlp=None)], width=40, taps=4, max_positions=1200)
    oracle, model = build(cfg, seed=19)
    a, b = tokens(cfg, 1100, seed=1), tokens(cfg, 75, seed=2)
    ra, rb = oracle.run(a), oracle.run(b)
    cache = model.new_device_cache(max_batch=2, max_seq=1152, pool_tokens=1152 + 128)
    lg = cache.forward_ragged([1, 0], [b[:3], a[:1027]], [list(range(3)), list(range(1027))])
    assert relerr(lg[:3], rb[:3]) < TOL["f32"] and relerr(lg[3:], ra[:1027]) < TOL["f32"]
    lg = cache.forward_ragged([0, 1], [a[1027:], b[3:]], [list(range(73)), list(range(72))])
    assert relerr(lg[:73], ra[1027:]) < TOL["f32"] and relerr(lg[73:], rb[3:]) < TOL["f32"]
    cache.slot_reset(0)
    lg = cache.forward_ragged([0], [a], [list(range(1100))])
    assert relerr(lg, ra) < TOL["f32"]


def test_position_table_bounds_a_sequence():
    cfg = config([layer()], max_positions=70)
    oracle, model = build(cfg, seed=18)
    toks = tokens(cfg, 70)
    cache = model.new_device_cache(max_batch=1, max_seq=128)
    assert relerr(run_whole(model, toks, cache=cache), oracle.run(toks)) < TOL["f32"]
    with pytest.raises(FastllmError):
        cache.forward_ragged([0], [[1]], None)


# ---- the framework's own entry points -------------------------------------------------------------------------------------------
def oracle_greedy(oracle, prompt, n):
    st = oracle.new_state()
    logits = oracle.run(prompt, st)[-1]
    out = []
    for _ in range(n):
        tok = int(np.flatnonzero(logits == logits.max())[-1])       # last index among equal maxima, as the sampler does
        out.append(tok)
        logits = oracle.step(tok, st)
    return out


def test_greedy_generation_through_model_and_batcher():
    cfg = deep_cfg()
    oracle, model = build(cfg, seed=15)
    prompts = [tokens(cfg, n, seed=40 + n) for n in (5, 70, 23, 9, 31)]
    want = [oracle_greedy(oracle, p, 12) for p in prompts]
    assert models.Model(model, None, eos_token_id=None).generate(prompts[0], 12) == want[0]
    assert models.ContinuousBatcher(model, max_batch=3, eos_token_id=None).generate(prompts, 12) == want
    b = models.ContinuousBatcher(model, max_batch=2, eos_token_id=None, prefill_chunk=16)
    assert b.generate(prompts, 12) == want
    assert b.cache.pool_stats()[0] == b.cache.pool_stats()[1]


def test_uniform_entry_points_and_errors():
    cfg = deep_cfg()
    oracle, model = build(cfg, seed=16)
    toks = tokens(cfg, 20)
    cache = model.new_device_cache(max_batch=2, max_seq=64)
    ref = oracle.run(toks)
    both = cache.forward(np.asarray([toks[:12], toks[:12]], dtype=np.uint32), 0)
    assert relerr(both, np.stack([ref[11], ref[11]])) < TOL["f32"]
    nxt = cache.forward_slots([1], np.asarray([toks[12:]], dtype=np.uint32), [12])
    assert relerr(nxt, ref[19:20]) < TOL["f32"]
    bad = config([layer(mlp=moe(experts=8, top=5, ff=8, groups=4, keep=2))])       # the kept groups hold four experts
    with pytest.raises(FastllmError):
        models.TozaraxWithConfig.initialize_model(bad, {k: to_bits(v) for k, v in O.random_weights(bad).items()}, "f32")
    missing = {k: to_bits(v) for k, v in O.random_weights(cfg).items() if k != "l2.mlp.correction"}
    with pytest.raises(FastllmError):
        models.TozaraxWithConfig.initialize_model(cfg, missing, "f32")
    clone = model.clone()
    assert relerr(run_whole(clone, toks), ref) < TOL["f32"]


def test_random_init_runs_both_precisions():
    """synthetic weights (the benchmark's way in): finite logits, whole prompt = token by token"""
    cfg = tc_cfg()
    for dtype in ("bf16", "f32"):
        model, _ = models.TozaraxWithConfig.initialize_model(cfg, None, dtype, random_seed=3)
        toks = tokens(cfg, 80)
        whole, single = run_whole(model, toks, cache=model.new_device_cache(2, 128)), run_cut(model, toks, [], cache=model.new_device_cache(2, 128))
        assert np.isfinite(whole).all() and relerr(single, np.asarray(whole, dtype=np.float64), 0.02) < TOL[dtype]


def _write_checkpoint(folder, cfg, w):
    from fastllm_b200 import safetensors_io
    folder.mkdir(exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    safetensors_io.write_safetensors(str(folder / "model.safetensors"), {k: to_bits(v) for k, v in w.items()})


def test_checkpoint_folder_through_the_registry(tmp_path):
    cfg = deep_cfg()
    w = O.random_weights(cfg, 17)
    _write_checkpoint(tmp_path / "m", cfg, w)
    model, _ = models.load_model(str(tmp_path / "m"), "f32")
    assert isinstance(model, models.TozaraxWithConfig)
    toks = tokens(cfg, 30)
    assert relerr(run_whole(model, toks), O.Tozarax(cfg, w).run(toks)) < TOL["f32"]


def test_command_line_generate(tmp_path):
    """python -m fastllm_b200 generate: registry, loader, continuous batcher with prompt portions, greedy sampling -- ids in, ids out"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = deep_cfg()
    w = O.random_weights(cfg, 29)
    _write_checkpoint(tmp_path / "m", cfg, w)
    prompts = [tokens(cfg, n, seed=60 + n) for n in (3, 40, 17)]
    cmd = ["python3", "-m", "fastllm_b200", "generate", "--model", str(tmp_path / "m"), "--dtype", "f32", "--max-tokens", "6", "--max-batch", "2",
           "--prefill-chunk", "16"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root, env=dict(os.environ, PYTHONPATH=root))
    assert r.returncode == 0, r.stderr[-2000:]
    got = [json.loads(l)["generated"] for l in r.stdout.splitlines() if l.startswith("{")]
    oracle = O.Tozarax(cfg, w)
    assert got == [oracle_greedy(oracle, p, 6) for p in prompts]


def test_trace_runner_end_to_end(tmp_path):
    """bin/trace_run as a process: steps on standard input (portions beside single tokens, a request that sits out a step, one that
    wants nothing, a fifth request that takes over a finished one's slot and pages), logits files out"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = deep_cfg()
    w = O.random_weights(cfg, 23)
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    _write_checkpoint(model_dir, cfg, w)
    reqs = {name: tokens(cfg, n, seed=50 + i) for i, (name, n) in enumerate((("a", 70), ("b", 5), ("c", 33), ("d", 64), ("e", 40)))}
    refs = {"float32": {k: O.Tozarax(cfg, w).run(v) for k, v in reqs.items()},
            "bfloat16": {k: O.Tozarax(cfg, w, cache_round=O.to_bf16).run(v) for k, v in reqs.items()}}
    plan = [[("a", 3, [0, 2]), ("b", 1, [0])],
            [("a", 60, [59]), ("c", 33, []), ("d", 2, [1])],
            [("b", 4, [0, 3]), ("d", 62, [0, 61])],
            [("a", 1, [0]), ("e", 40, [39])],
            [("a", 6, [0, 5])]]
    at = {k: 0 for k in reqs}
    lines, places = [], {}
    for n, step in enumerate(plan):
        entries, rows, end = [], [], []
        for rid, cnt, want in step:
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + cnt], "want": want})
            rows += [(rid, at[rid] + p) for p in want]
            at[rid] += cnt
            if at[rid] == len(reqs[rid]):
                end.append(rid)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
        places[n] = rows
    assert all(at[k] == len(reqs[k]) for k in reqs)
    for dtype, tol in (("float32", TOL["f32"]), ("bfloat16", TOL["bf16"])):
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "256"],
                           input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == ["done %d" % n for n in range(len(plan))]
        for n, rows in places.items():
            want = np.stack([refs[dtype][rid][p] for rid, p in rows])
            f = out_dir / ("%d.f32" % n)
            got = np.fromfile(f, dtype="<f4").reshape(-1, cfg["vocab"])
            assert got.shape == want.shape and relerr(got, want) < tol
            f.unlink()
