"""Host-side pieces of the Tozarax decoder that need no GPU: config.json -> layer descriptors and stack options, the registry, and
closed-form checks of the plain restatement (oracle/tozarax.py) that the GPU tests lean on."""
import ctypes
import math

import numpy as np
import pytest

from fastllm_b200 import _lib, models
from oracle import tozarax as O


def _cfg():
    return {"architecture": "Tozarax", "vocab": 40, "width": 24, "norm": {"eps": 1e-6}, "canon": {"taps": 5}, "max_positions": 96, "layers": [
        {"type": "parallel",
         "mixer": {"left": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 10, "scale": 0.3, "mask": {"size": 17}},
                   "right": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 9, "conv": 2}},
         "mlp": {"kind": "moe", "expert": {"ff": 14}, "router": {"experts": 12, "top": 3, "groups": {"count": 4, "keep": 2}}}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 3}},
                   "right": {"heads": 3, "kv_heads": 3, "dim": 5, "vdim": 7, "conv": 4}},
         "mlp": None}]}


def test_config_to_layer_descs_and_stack_options():
    d = models.tozarax_layer_descs(_cfg())
    assert len(d) == 4
    a, b, c, e = d[0], d[1], d[2], d[3]
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.kv_from, a.beside) == (_lib.FL_MIXER["attention"], 6, 3, 8, 10, 17, -1, 1)
    assert (a.no_qk_norm, a.rot_dims, a.sink, a.softcap) == (1, 0, 0, 0.0) and abs(a.scale - 0.3) < 1e-7
    assert (a.ffn, a.ffn_act, a.ff, a.experts, a.top, a.router, a.route_groups, a.route_keep, a.shared_ff) == \
        (_lib.FL_FFN["moe"], _lib.FL_ACT["relu2"], 14, 12, 3, _lib.FL_ROUTER["sigmoid_groups"], 4, 2, 0)
    assert (b.mixer, b.heads, b.kv_heads, b.dim, b.vdim, b.conv, b.beside) == (_lib.FL_MIXER["delta"], 4, 2, 6, 9, 2, 0)
    assert (c.window, c.ffn, c.beside) == (3, _lib.FL_FFN["none"], 1) and (e.heads, e.conv) == (3, 4)
    sc = _lib.FlStackConfig()
    models.TozaraxWithConfig.stack_options(_cfg(), sc)
    assert (sc.max_positions, sc.canon_taps, sc.gated_residual, sc.depth_avg) == (96, 5, 1, 1)
    bad = _cfg()
    bad["layers"][0]["type"] = "attention"
    with pytest.raises(models.FastllmError):
        models.tozarax_layer_descs(bad)
    bad = _cfg()
    bad["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(models.FastllmError):
        models.tozarax_layer_descs(bad)


def test_descriptor_layout_matches_header():
    """the new fields sit where the header puts them (4-byte fields behind ffn_bias; the stack options behind no_pre_norm)"""
    assert _lib.FlLayerDesc.no_qk_norm.offset == 104 + 10 * 4 and _lib.FlLayerDesc.route_keep.offset == 104 + 14 * 4
    assert ctypes.sizeof(_lib.FlLayerDesc) == 104 + 26 * 4
    assert _lib.FlStackConfig.no_post_norm.offset == 8 * 4 and _lib.FlStackConfig.depth_avg.offset == 12 * 4
    assert ctypes.sizeof(_lib.FlStackConfig) == 22 * 4


def test_registry_picks_by_architecture():
    assert models.model_class_for({"architecture": "Tozarax"}) is models.TozaraxWithConfig
    assert models.model_class_for({"architecture": "Rofetar"}) is models.RofetarWithConfig
    assert models.TozaraxWithConfig in models.registered_models()
    assert models.TozaraxWithConfig.get_family() == "Tozarax" and not models.TozaraxWithConfig.supports_architecture("Nifunex")
    assert models.TozaraxWithConfig.no_post_norm and not models.TozaraxWithConfig.no_pre_norm and not models.TozaraxWithConfig.norm_plain
    assert not models.NifunexWithConfig.no_post_norm and not models.RofetarWithConfig.no_post_norm


# ---- closed forms of the restatement ------------------------------------------------------------------------------------------
def test_input_conv_is_identity_plus_causal_convolution():
    rng = np.random.default_rng(1)
    x, w = rng.normal(size=(9, 3)), rng.normal(size=(3, 4))
    hist, got = np.zeros((3, 3)), []
    for t in range(9):
        y, hist = O.input_conv(hist, x[t], w)
        got.append(y)
    for c in range(3):
        want = x[:, c] + np.convolve(x[:, c], w[c, ::-1])[:9]     # the last column of w meets the current input
        assert np.allclose(np.asarray(got)[:, c], want)


def test_window_attention_sees_exactly_the_window():
    rng = np.random.default_rng(2)
    K, V, q = rng.normal(size=(10, 1, 4)), rng.normal(size=(10, 1, 3)), rng.normal(size=(2, 4))
    full = O.window_softmax_attention(q, K, V, 9, 100, 0.5, 1)
    s = (K[:, 0] @ q[1]) * 0.5
    assert np.allclose(full[1], (np.exp(s) / np.exp(s).sum()) @ V[:, 0])
    assert np.allclose(O.window_softmax_attention(q, K, V, 9, 1, 0.5, 1), np.stack([V[9, 0], V[9, 0]]))       # itself only
    three = O.window_softmax_attention(q, K, V, 9, 3, 0.5, 1)
    Kh, Vh = K.copy(), V.copy()
    Kh[:7], Vh[:7] = 99.0, 99.0                                   # what lies outside the window does not matter
    assert np.allclose(O.window_softmax_attention(q, Kh, Vh, 9, 3, 0.5, 1), three)
    Kh[7] += 1.0
    assert not np.allclose(O.window_softmax_attention(q, Kh, Vh, 9, 3, 0.5, 1), three)


def test_delta_rule_stores_and_overwrites():
    """with no decay and full write strength, writing v at a unit key and then v' at the same key leaves exactly v' there, and the
    read-out of the same step already sees it"""
    S = np.zeros((3, 2))
    k = np.array([0.6, 0.8, 0.0])
    S, o = O.delta_rule_step(S, k, k, np.array([1.0, -2.0]), 1.0, 1.0)
    assert np.allclose(o, [1.0, -2.0])
    S, o = O.delta_rule_step(S, k, k, np.array([5.0, 7.0]), 1.0, 1.0)
    assert np.allclose(o, [5.0, 7.0]) and np.allclose(S.T @ k, [5.0, 7.0])
    S, o = O.delta_rule_step(S, k, k, np.array([5.0, 7.0]), 0.0, 0.5)          # no write: the state only fades
    assert np.allclose(o, [2.5, 3.5])


def test_router_groups_and_weights():
    s = np.array([0.9, 0.5, 0.1, 0.1, 0.3, 0.2])
    z = np.log(s / (1.0 - s))
    corr = np.array([0.0, -2.5, 0.0, 0.0, 0.0, 0.0])
    chosen, wts = O.route(z, corr, top=3, n_groups=3, keep=2)
    assert chosen.tolist() == [4, 5, 2] and np.allclose(wts, [0.3, 0.2, 0.1])   # expert 0's group is dropped; weights are not renormalised
    chosen, _ = O.route(z, np.zeros(6), top=2, n_groups=6, keep=6)              # groups of one: plain top-k
    assert chosen.tolist() == [0, 1]


def test_expert_and_layer_shape():
    x = np.array([1.0, -2.0])
    up, down = np.array([[1.0, 0.0], [0.0, 1.0], [2.0, 1.0]]), np.array([[1.0, 1.0, 1.0]])
    assert np.allclose(O.relu2_expert(x, up, down), [1.0])                      # relu(1, -2, 0)^2 summed
    cfg = _cfg()
    w = O.random_weights(cfg, 3)
    assert set(w) == set(O.tensor_shapes(cfg)) and "l1.norm2" not in w and "l1.rg2" not in w and "l0.mlp.e11.down" in w
    assert w["l0.dwa"].shape == (2,) and w["l1.dwa"].shape == (3,) and w["pos"].shape == (96, 24)
    lg, tr = O.Tozarax(cfg, w).run([1, 2, 3, 4, 5, 6], layer_trace=True)
    assert lg.shape == (6, 40) and tr.shape == (2, 6, 24)
    # the depth average of the last layer: with its weights set to "the embedding output only", the logits are those of the embedding
    v = dict(w)
    v["l1.dwa"] = np.array([1.0, 0.0, 0.0], dtype=np.float32)
    m = O.Tozarax(cfg, v)
    x0 = m.w["embed"][3] + m.w["pos"][0]
    assert np.allclose(m.run([3])[0], m.w["head"] @ O.norm_one_plus(x0, m.w["final.norm"], 1e-6))
