"""The Medulorn decoder on the GPU against the plain numpy restatement in oracle/medulorn.py.

Small random configurations of the tests' own; the product runs through the C ABI (models.MedulornWithConfig /
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
from oracle import medulorn as O

pytestmark = pytest.mark.gpu

TOL = {"f32": 4e-5, "bf16": 1e-2}


# ---- configurations ---------------------------------------------------------------------------------------------------------
def rot(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def chunked(heads=4, kv_heads=2, dim=8, vdim=12, chunk=11, scale=None, rot_=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "scale": scale if scale is not None else dim ** -0.5,
            "rot": rot_ if rot_ is not None else rot(dim - 2 if dim > 2 else 0)}


def windowed(heads=4, kv_heads=2, dim=8, vdim=12, window=9, keep=2, scale=None, rot_=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window, "keep_first": keep},
            "scale": scale if scale is not None else dim ** -0.5, "rot": rot_ if rot_ is not None else rot(dim, 50.0, (8.0, 1.0, 4.0, 32))}


def lightning(heads=3, dim=6, vdim=10, decay=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay if decay is not None else [0.5 + 0.45 * (h + 1) / heads for h in range(heads)]}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=12, limit=1.0, shared=10, shared_limit=2.0):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared, "limit": shared_limit}
    return m


def attn_layer(m=None, mlp="default"):
    return {"type": "attention", "mixer": m or chunked(), "mlp": moe() if mlp == "default" else mlp}


def par_layer(a=None, b=None, ls=0.7, rs=0.4, mlp="default"):
    return {"type": "parallel", "mixer": {"left": a or windowed(), "right": b or lightning(), "left_scale": ls, "right_scale": rs},
            "mlp": dense() if mlp == "default" else mlp}


def config(layers, vocab=48, width=32, eps=1e-5, alpha=1.5, escale=4.0, cap=20.0):
    return {"architecture": "Medulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha, "embedding": {"scale": escale},
            "logit_softcap": cap, "layers": layers}


def deep_cfg(**kw):
    """five unequal layers in an order of their own: with dense / expert / no feed-forward, other head counts, windows and chunks"""
    return config([attn_layer(),
                   par_layer(),
                   par_layer(windowed(heads=2, kv_heads=2, dim=10, vdim=6, window=70, keep=5), lightning(heads=2, dim=12, vdim=4), ls=1.0, rs=1.0, mlp=None),
                   attn_layer(chunked(heads=6, kv_heads=1, dim=4, vdim=8, chunk=64, scale=0.7), mlp=dense(40)),
                   par_layer(windowed(heads=1, kv_heads=1, dim=16, vdim=16, window=3, keep=0), lightning(heads=1, dim=20, vdim=36, decay=[0.99]),
                             mlp=moe(experts=4, top=1, ff=20, shared=0))], **kw)


# ---- helpers ----------------------------------------------------------------------------------------------------------------
def to_bits(a):
    return (np.ascontiguousarray(a, dtype=np.float32).reshape(-1).view(np.uint32) >> 16).astype(np.uint16).reshape(np.shape(a))


_built = {}


def build(cfg, seed=0, dtype="f32", tweak=None):
    """-> (oracle, product adapter); weights are bf16-representable, handed over as bf16 bit patterns"""
    key = (repr(cfg), seed, dtype, tweak.__name__ if tweak else None)
    if key not in _built:
        w = O.random_weights(cfg, seed)
        if tweak:
            tweak(w)
        model, _ = models.MedulornWithConfig.initialize_model(cfg, {k: to_bits(v) for k, v in w.items()}, dtype)
        _built[key] = (O.Medulorn(cfg, w, cache_round=O.to_bf16 if dtype == "bf16" else None), model)
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
    "chunked_attention_no_ff": config([attn_layer(mlp=None)]),
    "chunk_of_one": config([attn_layer(chunked(chunk=1), mlp=None)]),
    "chunk_of_two_one_kv_head": config([attn_layer(chunked(heads=6, kv_heads=1, dim=12, vdim=20, chunk=2, scale=1.5), mlp=None)]),
    "chunked_equal_heads_full_rotation": config([attn_layer(chunked(heads=3, kv_heads=3, dim=6, vdim=4, chunk=30, rot_=rot(6, 100.0)), mlp=None)]),
    "chunked_no_rotation": config([attn_layer(chunked(rot_={}), mlp=None)]),
    "chunked_scaled_rotation": config([attn_layer(chunked(dim=16, rot_=rot(12, 30.0, (3.0, 2.0, 6.0, 40))), mlp=None)]),
    "windowed_beside_lightning_no_ff": config([par_layer(mlp=None)]),
    "window_of_one_nothing_kept": config([par_layer(windowed(window=1, keep=0), mlp=None)]),
    "window_of_two_three_kept": config([par_layer(windowed(heads=6, kv_heads=1, dim=12, vdim=20, window=2, keep=3, scale=1.2), mlp=None)]),
    "kept_more_than_window": config([par_layer(windowed(window=3, keep=7), mlp=None)]),
    "windowed_plain_rotation_partial": config([par_layer(windowed(dim=12, rot_=rot(8, 1000.0)), mlp=None)]),
    "lightning_one_head_wide_values": config([par_layer(b=lightning(heads=1, dim=16, vdim=40, decay=[0.9]), ls=0.25, rs=2.0, mlp=None)], width=40),
    "lightning_decay_one_and_small": config([par_layer(b=lightning(heads=2, dim=5, vdim=7, decay=[1.0, 0.125]), mlp=None)]),
    "dense_relu_glu": config([attn_layer(mlp=dense(20))]),
    "experts_with_shared": config([par_layer(mlp=moe())]),
    "experts_without_shared_top_one": config([attn_layer(mlp=moe(experts=5, top=1, ff=16, shared=0))]),
    "experts_all_chosen": config([attn_layer(mlp=moe(experts=3, top=3, ff=9, limit=0.5, shared=7, shared_limit=0.25))]),
    "one_expert": config([attn_layer(mlp=moe(experts=1, top=1, ff=24))]),
    "alpha_one_no_scale_no_cap": config([attn_layer(), par_layer()], alpha=1.0, escale=1.0, cap=0.0),
    "three_layers": config([par_layer(), attn_layer(), par_layer(mlp=moe())], alpha=3.0),
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
    cfg = config([par_layer(windowed(heads=6, kv_heads=3, dim=10, vdim=14, window=66, keep=3), lightning(heads=5, dim=9, vdim=35),
                            mlp=moe(experts=15, top=4, ff=11, shared=13)),
                  attn_layer(chunked(heads=3, kv_heads=1, dim=7, vdim=34, chunk=13, rot_=rot(6)), mlp=dense(22))], vocab=37, width=50)
    oracle, model = build(cfg, seed=5)
    toks = tokens(cfg, 70)
    assert relerr(run_whole(model, toks), oracle.run(toks)) < TOL["f32"]


def tc_cfg():
    """widths in whole 64-column blocks: in the serving precision the projections, the feed-forwards and the experts (grouped GEMM
    pair for few rows, every expert over all rows for many) run on the tensor-core GEMM; masks wide enough that long portions take
    the attention through the tensor-core GEMMs too (kept first keys gathered in front of a block's keys, chunk borders inside a
    block of rows)"""
    return config([par_layer(windowed(heads=4, kv_heads=2, dim=32, vdim=16, window=290, keep=6), lightning(heads=4, dim=16, vdim=32),
                             mlp=moe(experts=8, top=2, ff=64, shared=64)),
                   attn_layer(chunked(heads=8, kv_heads=2, dim=16, vdim=16, chunk=300), mlp=dense(128)),
                   par_layer(windowed(heads=2, kv_heads=1, dim=64, vdim=64, window=50, keep=2), lightning(heads=2, dim=32, vdim=64), mlp=None)],
                  vocab=96, width=128)


def tc_cfg_partial_tiles():
    """320-wide: five 64-column k blocks, matrices that end inside a 128-row tile; the first layer's experts lie outside the tiles
    (ff = 100) and run on the plain kernel beside tensor-core projections"""
    return config([attn_layer(chunked(heads=3, kv_heads=1, dim=48, vdim=64, chunk=257), mlp=moe(experts=6, top=2, ff=100, shared=100)),
                   par_layer(windowed(heads=6, kv_heads=3, dim=32, vdim=24, window=260, keep=300), lightning(heads=3, dim=24, vdim=40),
                             mlp=moe(experts=6, top=2, ff=320, shared=64))], vocab=200, width=320)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("make", [tc_cfg, tc_cfg_partial_tiles])
def test_tensor_core_projections_and_attention(make, dtype):
    """1 row, a few rows, up to 128 rows (weights as the 128-row operand, split-K) and more (tokens as rows) through the same layers"""
    cfg = make()
    oracle, model = build(cfg, seed=21, dtype=dtype)
    toks = tokens(cfg, 700, seed=9)
    ref = oracle.run(toks)
    allow = 0.02 if dtype == "bf16" else 0.0
    assert relerr(run_whole(model, toks, cache=model.new_device_cache(4, 768)), ref, allow) < TOL[dtype]
    assert relerr(run_cut(model, toks, [5, 128, 129, 2, 330, 64, 40], cache=model.new_device_cache(4, 768)), ref, allow) < TOL[dtype]


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
    """a prompt cut into portions (down to two tokens and single ones: the token shift's previous row comes from this step, from the
    slot's carried row or from before the start), across page, window and chunk borders, the rest decoded"""
    cfg = deep_cfg()
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
    in its pages, its recurrent state and its carried token-shift rows must not leak into the next one"""
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


# ---- the masks' edges, far tokens, every piece: made to stand out ---------------------------------------------------------------
def _other_mask(cfg, key, delta):
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        m = l["mixer"]["left"] if l["type"] == "parallel" else l["mixer"]
        if key in m["mask"]:
            m["mask"][key] += delta
    return c


@pytest.mark.parametrize("window,keep", [(1, 0), (2, 1), (5, 3), (63, 2), (64, 64), (65, 1), (130, 7)])
def test_window_and_kept_first_edges(window, keep):
    """windows of one key, within a page, of exactly a page, just over it and over two pages, with none to a page of kept first keys;
    scores sharp enough that one key more or less moves the logits: the oracle itself with a window (or a kept count) one off is far
    outside the bar.  A whole prompt, portions that cut the window, single tokens, and the serving precision."""
    sharp = 3.0
    cfg = config([par_layer(windowed(window=window, keep=keep, scale=sharp), mlp=None),
                  par_layer(windowed(heads=2, kv_heads=1, window=window, keep=keep, scale=sharp), lightning(heads=2, decay=[0.3, 0.6]))])
    oracle, model = build(cfg, seed=11)
    toks = tokens(cfg, 210, seed=5)
    ref = oracle.run(toks)
    for key, d in (("size", -1), ("size", 1), ("keep_first", -1), ("keep_first", 1)):
        c = _other_mask(cfg, key, d)
        if c["layers"][0]["mixer"]["left"]["mask"][key] >= (1 if key == "size" else 0):
            assert relerr(O.Medulorn(c, oracle.w).run(toks), ref) > 100 * TOL["f32"]
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [window, 2, 61, 66]), ref) < TOL["f32"]
    _, served = build(cfg, seed=11, dtype="bf16")
    ref16 = O.Medulorn(cfg, oracle.w, cache_round=O.to_bf16).run(toks)
    assert relerr(run_whole(served, toks), ref16, 0.02) < TOL["bf16"]
    assert relerr(run_cut(served, toks, [70, 2, 100]), ref16, 0.02) < TOL["bf16"]


@pytest.mark.parametrize("chunk", [1, 2, 7, 63, 64, 65, 100])
def test_chunk_edges(chunk):
    """chunks of one position, inside a page, a page, just over it: the first position of a chunk sees itself alone (and the sink),
    the last sees the whole chunk; portions that start and end inside chunks"""
    sharp = 3.0
    cfg = config([attn_layer(chunked(chunk=chunk, scale=sharp), mlp=None), attn_layer(chunked(heads=2, kv_heads=1, chunk=chunk, scale=sharp))])
    oracle, model = build(cfg, seed=12)
    toks = tokens(cfg, 210, seed=6)
    ref = oracle.run(toks)
    for d in (-1, 1):
        if chunk + d >= 1:
            assert relerr(O.Medulorn(_other_mask(cfg, "size", d), oracle.w).run(toks), ref) > 100 * TOL["f32"]
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [chunk, 2, 61, 66]), ref) < TOL["f32"]
    _, served = build(cfg, seed=12, dtype="bf16")
    ref16 = O.Medulorn(cfg, oracle.w, cache_round=O.to_bf16).run(toks)
    assert relerr(run_whole(served, toks), ref16, 0.02) < TOL["bf16"]
    assert relerr(run_cut(served, toks, [70, 2, 100]), ref16, 0.02) < TOL["bf16"]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_wide_masks_on_the_gemm_attention(dtype):
    """masks that leave a row hundreds of keys: long portions of the serving precision run scores and weighted sums as GEMMs; kept
    first keys sit in front of a block's gathered keys, a chunk border and a window's start fall inside blocks of rows; sharp scores"""
    cfg = config([par_layer(windowed(heads=4, kv_heads=2, dim=16, vdim=16, window=300, keep=9, scale=1.5), mlp=None),
                  attn_layer(chunked(heads=4, kv_heads=1, dim=16, vdim=24, chunk=410, scale=1.5), mlp=None)], width=64)
    oracle, model = build(cfg, seed=22, dtype=dtype)
    toks = tokens(cfg, 1300, seed=3)
    ref = oracle.run(toks)
    if dtype == "f32":
        for key, d in (("size", -1), ("keep_first", -1)):
            assert relerr(O.Medulorn(_other_mask(cfg, key, d), oracle.w).run(toks), ref) > 100 * TOL["f32"]
    allow = 0.02 if dtype == "bf16" else 0.0
    assert relerr(run_whole(model, toks, cache=model.new_device_cache(2, 1344)), ref, allow) < TOL[dtype]
    assert relerr(run_cut(model, toks, [290, 330, 2, 600, 70], cache=model.new_device_cache(2, 1344)), ref, allow) < TOL[dtype]


def test_far_tokens_reach_through_the_state():
    """windows of four keys and nothing kept: only the lightning state (decay 0.999) carries the first token to position 400"""
    lay = par_layer(windowed(window=4, keep=0), lightning(heads=2, dim=64, vdim=10, decay=[0.999, 0.998]), ls=0.3, rs=1.0, mlp=None)
    cfg = config([lay, copy.deepcopy(lay)])
    oracle, model = build(cfg, seed=12)
    toks = tokens(cfg, 400, seed=6)
    ref = oracle.run(toks)
    other = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert relerr(oracle.run(other)[-1:], ref[-1:]) > 100 * TOL["f32"]
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [2, 300, 2]), ref) < TOL["f32"]


def test_kept_first_keys_reach_far():
    """a window of three keys and two kept first keys, no recurrent help (the lightning share is zero): the first token still moves
    position 300, the third does not"""
    lay = par_layer(windowed(window=3, keep=2, scale=2.0), ls=1.0, rs=0.0, mlp=None)
    cfg = config([lay])
    oracle, model = build(cfg, seed=14)
    toks = tokens(cfg, 300, seed=8)
    ref = oracle.run(toks)
    first = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    third = toks[:2] + [(toks[2] + 1) % cfg["vocab"]] + toks[3:]
    assert relerr(oracle.run(first)[-1:], ref[-1:]) > 100 * TOL["f32"]
    assert relerr(oracle.run(third)[-1:], ref[-1:]) < 1e-12
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]
    assert relerr(run_cut(model, toks, [1, 1, 1, 200]), ref) < TOL["f32"]


def test_every_piece_would_show():
    """the oracle itself with one piece taken out or changed is far outside the bar the product is held to"""
    cfg = config([par_layer(mlp=moe()), attn_layer(mlp=dense()), par_layer()])
    w = O.random_weights(cfg, 13)
    toks = tokens(cfg, 40, seed=5)
    ref = O.Medulorn(cfg, w).run(toks)
    _, model = build(cfg, seed=13)
    assert relerr(run_whole(model, toks), ref) < TOL["f32"]

    def changed(change=None, cfg_change=None):
        v = {k: np.array(a, copy=True) for k, a in w.items()}
        c = copy.deepcopy(cfg)
        if change:
            change(v)
        if cfg_change:
            cfg_change(c)
        return relerr(O.Medulorn(c, v).run(toks), ref)

    def zero(pattern):
        def f(v):
            for k in v:
                if k.endswith(pattern):
                    v[k] = np.zeros_like(v[k])
        return f
    assert changed(zero(".shift")) > 100 * TOL["f32"]
    assert changed(zero(".sink")) > 100 * TOL["f32"]
    assert changed(zero("q.b")) > 100 * TOL["f32"]
    assert changed(zero("router.b")) > 100 * TOL["f32"]
    assert changed(lambda v: v.__setitem__("l0.norm1", np.asarray(1.0))) > 100 * TOL["f32"]
    assert changed(lambda v: v.__setitem__("l0.mix.left.q.norm", np.ones_like(v["l0.mix.left.q.norm"]))) > 100 * TOL["f32"]
    assert changed(cfg_change=lambda c: c.__setitem__("postln_alpha", 1.0)) > 100 * TOL["f32"]
    assert changed(cfg_change=lambda c: c["embedding"].__setitem__("scale", 1.0)) > 100 * TOL["f32"]
    assert changed(cfg_change=lambda c: c.__setitem__("logit_softcap", 0.0)) > 100 * TOL["f32"]
    assert changed(cfg_change=lambda c: c["layers"][0]["mixer"].__setitem__("right_scale", 0.0)) > 100 * TOL["f32"]
    assert changed(cfg_change=lambda c: c["layers"][0]["mixer"]["right"].__setitem__("decay", [0.9, 0.9, 0.9])) > 100 * TOL["f32"]
    assert changed(cfg_change=lambda c: c["layers"][0]["mixer"]["left"]["rot"].pop("scaling")) > 100 * TOL["f32"]
    assert changed(cfg_change=lambda c: c["layers"][0]["mlp"]["shared"].__setitem__("limit", 0.1)) > 100 * TOL["f32"]


def test_first_tokens():
    cfg = deep_cfg()
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
    """two requests in one long step, then portions that go on from it"""
    cfg = config([par_layer(windowed(window=100, keep=3)), attn_layer(chunked(heads=2, kv_heads=1, chunk=7), mlp=None)], width=40)
    oracle, model = build(cfg, seed=19)
    a, b = tokens(cfg, 1100, seed=1), tokens(cfg, 75, seed=2)
    ra, rb = oracle.run(a), oracle.run(b)
    cache = model.new_device_cache(max_batch=2, max_seq=1152, pool_tokens=1152 + 128)
    lg = cache.forward_ragged([1, 0], [b[:3], a[:1027]], [list(range(3)), list(range(1027))])
    assert relerr(lg[:3], rb[:3]) < TOL["f32"] and relerr(lg[3:], ra[:1027]) < TOL["f32"]
    lg = cache.forward_ragged([0, 1], [a[1027:], b[3:]], [list(range(73)), list(range(72))])
    assert relerr(lg[:73], ra[1027:]) < TOL["f32"] and relerr(lg[73:], rb[3:]) < TOL["f32"]


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
    bad = config([par_layer(b=lightning(heads=3, decay=[0.5, 0.5]))])              # one decay too few
    with pytest.raises(FastllmError):
        models.MedulornWithConfig.initialize_model(bad, None, "f32")
    missing = {k: to_bits(v) for k, v in O.random_weights(cfg).items() if k != "l1.mix.left.sink"}
    with pytest.raises(FastllmError):
        models.MedulornWithConfig.initialize_model(cfg, missing, "f32")
    clone = model.clone()
    assert relerr(run_whole(clone, toks), ref) < TOL["f32"]


def test_random_init_runs_both_precisions():
    """synthetic weights (the benchmark's way in): finite logits, whole prompt = token by token; the decays are the configuration's"""
    cfg = tc_cfg()
    for dtype in ("bf16", "f32"):
        model, _ = models.MedulornWithConfig.initialize_model(cfg, None, dtype, random_seed=3)
        toks = tokens(cfg, 80)
        whole, single = run_whole(model, toks, cache=model.new_device_cache(2, 128)), run_cut(model, toks, [], cache=model.new_device_cache(2, 128))
        assert np.isfinite(whole).all() and relerr(single, np.asarray(whole, dtype=np.float64), 0.02) < TOL[dtype]


def _write_checkpoint(folder, cfg, w):
    from fastllm_b200 import safetensors_io
    folder.mkdir(exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    safetensors_io.write_safetensors(str(folder / "model.safetensors"), {k: to_bits(v) for k, v in w.items()})


def test_checkpoint_folder_through_the_registry(tmp_path):
    """norm weights of one number are stored as tensors without a shape"""
    cfg = deep_cfg()
    w = O.random_weights(cfg, 17)
    assert w["final.norm"].shape == () and w["l0.norm1"].shape == ()
    _write_checkpoint(tmp_path / "m", cfg, w)
    model, _ = models.load_model(str(tmp_path / "m"), "f32")
    assert isinstance(model, models.MedulornWithConfig)
    toks = tokens(cfg, 30)
    assert relerr(run_whole(model, toks), O.Medulorn(cfg, w).run(toks)) < TOL["f32"]


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
    oracle = O.Medulorn(cfg, w)
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
    refs = {"float32": {k: O.Medulorn(cfg, w).run(v) for k, v in reqs.items()},
            "bfloat16": {k: O.Medulorn(cfg, w, cache_round=O.to_bf16).run(v) for k, v in reqs.items()}}
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
