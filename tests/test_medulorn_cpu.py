"""Host-side pieces of the Medulorn decoder that need no GPU: config.json -> layer descriptors, stack options and configuration
tensors, the registry, and closed-form checks of the plain restatement (oracle/medulorn.py) that the GPU tests lean on."""
import ctypes
import math

import numpy as np
import pytest

from fastllm_b200 import _lib, models
from oracle import medulorn as O


def _cfg():
    return {"architecture": "Medulorn", "vocab": 40, "width": 24, "norm": {"eps": 1e-6}, "postln_alpha": 1.25, "embedding": {"scale": 3.0},
            "logit_softcap": 12.0, "layers": [
        {"type": "attention",
         "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 10, "scale": 0.3, "mask": {"size": 17}, "rot": {"dims": 6, "base": 777.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 14, "limit": 0.75}, "router": {"experts": 10, "top": 3}, "shared": {"ff": 9, "limit": 2.5}}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "mask": {"size": 3, "keep_first": 2},
                            "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 2.0, "low": 1.0, "high": 8.0, "original": 64}}},
                   "right": {"heads": 3, "dim": 5, "vdim": 7, "decay": [0.5, 0.75, 0.999]}, "left_scale": 0.8, "right_scale": 0.3},
         "mlp": {"kind": "dense", "ff": 20}},
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "mask": {"size": 5}, "rot": {"dims": 2, "base": 10.0}},
         "mlp": None}]}


def test_config_to_layer_descs_and_stack_options():
    d = models.medulorn_layer_descs(_cfg())
    assert len(d) == 4
    a, b, r, c = d[0], d[1], d[2], d[3]
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.kv_from, a.beside) == (_lib.FL_MIXER["attention"], 6, 3, 8, 10, -1, 0)
    assert (a.mask_chunk, a.window, a.keep_first, a.qkv_bias, a.qk_norm_whole, a.sink, a.no_qk_norm) == (17, 0, 0, 1, 0, 1, 0)
    assert (a.rot_dims, a.rot_base, a.rot_halves, a.yarn_factor) == (6, 777.0, 1, 0.0) and abs(a.scale - 0.3) < 1e-7
    assert (a.ffn, a.ffn_act, a.ff, a.experts, a.top, a.router, a.router_bias, a.shared_ff, a.shared_plain) == \
        (_lib.FL_FFN["moe"], _lib.FL_ACT["swish_clamp"], 14, 10, 3, _lib.FL_ROUTER["softmax"], 1, 9, 1)
    assert (a.limit, a.shared_limit) == (0.75, 2.5)
    assert (b.mixer, b.window, b.keep_first, b.mask_chunk, b.qkv_bias, b.qk_norm_whole, b.sink, b.beside, b.pair_sum) == \
        (_lib.FL_MIXER["attention"], 3, 2, 0, 0, 1, 2, 1, 1)
    assert (b.rot_scaling, b.yarn_factor, b.yarn_original, b.yarn_fast, b.yarn_slow) == (_lib.FL_ROT_SCALE["bands"], 2.0, 64.0, 8.0, 1.0)
    assert abs(b.out_scale - 0.8) < 1e-7 and abs(r.out_scale - 0.3) < 1e-7
    assert (b.ffn, b.ffn_act, b.ff) == (_lib.FL_FFN["dense"], _lib.FL_ACT["relu"], 20)
    assert (r.mixer, r.heads, r.dim, r.vdim, r.beside) == (_lib.FL_MIXER["lightning"], 3, 5, 7, 0)
    assert (c.ffn, c.mask_chunk, c.beside) == (_lib.FL_FFN["none"], 5, 0)
    sc = _lib.FlStackConfig()
    models.MedulornWithConfig.stack_options(_cfg(), sc)
    assert (sc.post_sum_norm, sc.norm_scalar, sc.token_shift) == (1, 1, 1)
    assert (sc.residual_alpha, sc.embed_scale, sc.logit_softcap) == (1.25, 3.0, 12.0)
    extra = dict(models.MedulornWithConfig.config_tensors(_cfg()))
    assert list(extra) == ["l1.mix.right.decay"] and extra["l1.mix.right.decay"].dtype == np.float32
    assert extra["l1.mix.right.decay"].tolist() == [np.float32(0.5), np.float32(0.75), np.float32(0.999)]     # not rounded to bf16
    bad = _cfg()
    bad["layers"][0]["type"] = "delta"
    with pytest.raises(models.FastllmError):
        models.medulorn_layer_descs(bad)
    bad = _cfg()
    bad["layers"][1]["mixer"]["right"]["decay"] = [0.5]
    with pytest.raises(models.FastllmError):
        models.medulorn_layer_descs(bad)


def test_descriptor_layout_matches_header():
    """the newer fields sit where the header puts them: behind route_keep in the layer descriptor, behind depth_avg in the stack's"""
    assert _lib.FlLayerDesc.qkv_bias.offset == 104 + 15 * 4 and _lib.FlLayerDesc.shared_plain.offset == 104 + 23 * 4
    assert _lib.FlLayerDesc.out_scale.offset == 104 + 20 * 4
    assert _lib.FlStackConfig.post_sum_norm.offset == 13 * 4 and _lib.FlStackConfig.token_shift.offset == 18 * 4
    assert ctypes.sizeof(_lib.FlLayerDesc) == 208 and ctypes.sizeof(_lib.FlStackConfig) == 88


def test_registry_picks_by_architecture():
    assert models.model_class_for({"architecture": "Medulorn"}) is models.MedulornWithConfig
    assert models.model_class_for({"architecture": "Tozarax"}) is models.TozaraxWithConfig
    assert models.MedulornWithConfig in models.registered_models()
    assert models.MedulornWithConfig.get_family() == "Medulorn" and not models.MedulornWithConfig.supports_architecture("Rofetar")
    assert models.MedulornWithConfig.no_pre_norm and models.MedulornWithConfig.norm_plain and not models.MedulornWithConfig.no_post_norm


# ---- closed forms of the restatement ------------------------------------------------------------------------------------------
def test_token_shift_ends():
    h, prev = np.array([1.0, 2.0, 3.0]), np.array([5.0, 6.0, 7.0])
    assert np.allclose(O.token_shift(h, prev, np.array([0.0, 1.0, 0.5])), [1.0, 6.0, 5.0])


def test_banded_frequency_scaling():
    """base 100 over 8 channels: wavelengths 2 pi (1, 3.16, 10, 31.6) = 6.3, 19.9, 62.8, 198.7; with original 64, high 8, low 1 the
    first stays (below 8), the last is divided by the factor (above 64), the two between are blended"""
    f = O.rotary_freqs(8, 100.0)
    g = O.rotary_freqs(8, 100.0, {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 64})
    assert np.allclose(f, [1.0, 100 ** -0.25, 0.1, 100 ** -0.75])
    assert g[0] == f[0] and np.isclose(g[3], f[3] / 4.0)
    for i in (1, 2):
        s = (64 * f[i] / (2 * math.pi) - 1.0) / 7.0
        assert 0.0 < s < 1.0 and np.isclose(g[i], (1 - s) * f[i] / 4.0 + s * f[i])
    assert O.rotary_freqs(0, 100.0).size == 0


def test_rotation_is_relative_and_partial():
    rng = np.random.default_rng(1)
    q, k = rng.normal(size=(1, 6)), rng.normal(size=(1, 6))
    f = O.rotary_freqs(4, 50.0)
    a = O.rotate_halves(q, 9, f)[0] @ O.rotate_halves(k, 4, f)[0]
    b = O.rotate_halves(q, 25, f)[0] @ O.rotate_halves(k, 20, f)[0]
    assert np.isclose(a, b)
    assert np.allclose(O.rotate_halves(q, 9, f)[0, 4:], q[0, 4:])               # channels behind the rotated ones pass
    assert np.allclose(O.rotate_halves(q, 0, f), q)
    one = O.rotate_halves(np.array([[1.0, 0.0, 0.0, 0.0]]), 1, np.array([math.pi / 2, 0.0]))
    assert np.allclose(one, [[0.0, 0.0, 1.0, 0.0]])                             # channel 0 turns into channel 2 (its partner dims/2 away)


def test_masks():
    assert [j for j in range(12) if O.visible(11, j, window=3, keep_first=2)] == [0, 1, 9, 10, 11]
    assert [j for j in range(3) if O.visible(2, j, window=3, keep_first=2)] == [0, 1, 2]
    assert [j for j in range(12) if O.visible(11, j, chunk=5)] == [10, 11]
    assert [j for j in range(12) if O.visible(10, j, chunk=5)] == [10] and [j for j in range(12) if O.visible(9, j, chunk=5)] == [5, 6, 7, 8, 9]
    assert not O.visible(3, 4) and O.visible(3, 0)


def test_sink_softmax():
    K, V = np.zeros((3, 1, 2)), np.array([[[1.0]], [[2.0]], [[6.0]]])
    q = np.ones((1, 2))
    out = O.sink_softmax_attention(q, K, V, [0, 1, 2], 1.0, np.array([0.0]))      # three scores of zero and a sink of zero
    assert np.allclose(out, [[9.0 / 4.0]])
    out = O.sink_softmax_attention(q, K, V, [0, 1, 2], 1.0, np.array([math.log(5.0)]))
    assert np.allclose(out, [[9.0 / 8.0]])
    out = O.sink_softmax_attention(q, K, V, [2], 1.0, None)
    assert np.allclose(out, [[6.0]])


def test_lightning_state_is_a_decayed_sum():
    rng = np.random.default_rng(2)
    k, v, q = rng.normal(size=(7, 3)), rng.normal(size=(7, 2)), rng.normal(size=3)
    S = np.zeros((3, 2))
    for t in range(7):
        S, o = O.lightning_step(S, q, k[t], v[t], 0.8)
    want = sum(0.8 ** (6 - t) * (k[t] @ q) * v[t] for t in range(7))
    assert np.allclose(o, want)


def test_router_and_experts():
    chosen, wts = O.route_top(np.array([0.1, 2.0, -1.0, 2.0, 1.0]), 3)
    e = np.exp(np.array([0.0, 0.0, -1.0]))
    assert chosen == [1, 3, 4] and np.allclose(wts, e / e.sum())                # lower index first among equals; softmax over the chosen only
    x = np.array([1.0, -2.0])
    gate, up, down = np.array([[3.0, 0.0], [0.0, 1.0]]), np.array([[0.0, 1.0], [5.0, 0.0]]), np.array([[1.0, 1.0]])
    g, u = np.array([1.5, -2.0]), np.array([-1.5, 1.5])                         # min(3, 1.5), -2 | clip(-2), clip(5)
    assert np.allclose(O.clamped_swish_expert(x, gate, up, down, 1.5), [np.sum(g / (1 + np.exp(-1.702 * g)) * (u + 1))])
    assert np.allclose(O.relu_glu(x, gate, up, down), [3.0 * -2.0 + 0.0])


def test_model_shape_and_the_norm_of_the_sum():
    cfg = _cfg()
    w = O.random_weights(cfg, 3)
    assert set(w) == set(O.tensor_shapes(cfg)) and "l2.norm2" not in w and "l1.mix.right.decay" not in w and "l0.mlp.e9.down" in w
    assert w["l0.norm1"].shape == () and w["l1.mix.left.q.norm"].shape == (8,) and w["l0.mix.q.norm"].shape == (8,) and w["l1.mix.left.sink"].shape == (2,)
    m = O.Medulorn(cfg, w)
    lg, tr = m.run([1, 2, 3, 4, 5, 6], layer_trace=True)
    assert lg.shape == (6, 40) and tr.shape == (3, 6, 24) and np.abs(lg).max() < 12.0
    # after every layer the stream is a unit-rms row times the layer's last norm weight
    for i, name in enumerate(("l0.norm2", "l1.norm2", "l2.norm1")):
        assert np.allclose(np.sqrt((tr[i] ** 2).mean(-1)), abs(float(w[name])), rtol=1e-4)
