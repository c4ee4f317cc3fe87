"""Host-side pieces of the Rofetar decoder that need no GPU: config.json -> layer descriptors, the registry, and closed-form checks
of the plain restatement (oracle/rofetar.py) that the GPU tests lean on."""
import ctypes
import math

import numpy as np
import pytest

from fastllm_b200 import _lib, models
from oracle import rofetar as O


def _cfg():
    rot = {"base": 777.0, "dims": 4, "scaling": {"factor": 2.0, "original": 64, "fast": 8.0, "slow": 2.0}}
    return {"architecture": "Rofetar", "vocab": 40, "width": 24, "norm": {"eps": 1e-6}, "layers": [
        {"type": "mamba2", "mixer": {"heads": 6, "vdim": 5, "state": 7, "groups": 3, "norm_groups": 2, "conv": 3}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 10, "scale": 0.3, "softcap": 12.5, "rot": rot},
         "mlp": {"kind": "dense", "ff": 20}},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 9, "conv": 5}, "mlp": {"kind": "dense", "ff": 12}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 10, "scale": 0.5, "kv_from": 1, "rot": {"base": 100.0, "dims": 8}},
         "mlp": None}]}


def test_config_to_layer_descs():
    d = models.rofetar_layer_descs(_cfg())
    s, a, r, b = d[0], d[1], d[2], d[3]
    assert (s.mixer, s.heads, s.vdim, s.state, s.groups, s.norm_groups, s.conv, s.ffn) == (_lib.FL_MIXER["mamba2"], 6, 5, 7, 3, 2, 3, _lib.FL_FFN["none"])
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.kv_from, a.sink, a.rot_halves) == (_lib.FL_MIXER["attention"], 6, 3, 8, 10, -1, 1, 1)
    assert (a.rot_dims, a.rot_base, a.yarn_factor, a.yarn_original, a.yarn_fast, a.yarn_slow) == (4, 777.0, 2.0, 64.0, 8.0, 2.0)
    assert abs(a.scale - 0.3) < 1e-7 and a.softcap == 12.5
    assert (a.ffn, a.ff, a.ffn_act, a.ffn_bias) == (_lib.FL_FFN["dense"], 20, _lib.FL_ACT["gelu_tanh"], 1)
    assert (r.mixer, r.heads, r.kv_heads, r.dim, r.vdim, r.conv, r.ff) == (_lib.FL_MIXER["delta"], 4, 2, 6, 9, 5, 12)
    assert (b.kv_from, b.softcap, b.yarn_factor, b.rot_dims, b.ffn) == (1, 0.0, 0.0, 8, _lib.FL_FFN["none"])
    bad = _cfg()
    bad["layers"][0]["type"] = "gla"
    with pytest.raises(models.FastllmError):
        models.rofetar_layer_descs(bad)


def test_descriptor_layout_matches_header():
    """the two structs as the header lays them out (4-byte fields, one double aligned to 8)"""
    assert ctypes.sizeof(_lib.FlStackConfig) == 22 * 4
    assert _lib.FlLayerDesc.rot_base.offset == 48 and _lib.FlLayerDesc.kv_heads.offset == 104
    assert ctypes.sizeof(_lib.FlLayerDesc) == 104 + 26 * 4


def test_registry_picks_by_architecture():
    assert models.model_class_for({"architecture": "Rofetar"}) is models.RofetarWithConfig
    assert models.model_class_for({"architecture": "Nifunex"}) is models.NifunexWithConfig
    assert models.RofetarWithConfig.get_family() == "Rofetar" and not models.RofetarWithConfig.supports_architecture("Nifunex")
    assert models.RofetarWithConfig.norm_plain and models.RofetarWithConfig.no_pre_norm and not models.NifunexWithConfig.no_pre_norm


# ---- closed forms of the restatement ------------------------------------------------------------------------------------------
def test_rotation_by_halves_is_relative_and_partial():
    rng = np.random.default_rng(0)
    f, mult = O.rotary_freqs(6, 50.0, None)
    assert mult == 1.0 and np.allclose(f, 50.0 ** (-np.arange(3) / 3.0))
    q, k = rng.normal(size=10), rng.normal(size=10)
    a = O.rotate_halves(q, 9, f, 1.0, 6) @ O.rotate_halves(k, 4, f, 1.0, 6)
    b = O.rotate_halves(q, 25, f, 1.0, 6) @ O.rotate_halves(k, 20, f, 1.0, 6)
    assert abs(a - b) < 1e-9                                    # scores depend on the distance alone
    r = O.rotate_halves(q, 7, f, 1.0, 6)
    assert np.array_equal(r[6:], q[6:])                         # channels past `dims` pass
    assert np.isclose(r[0], q[0] * math.cos(7 * f[0]) - q[3] * math.sin(7 * f[0]))      # entry i turns with entry i + dims / 2
    assert np.isclose(r[3], q[3] * math.cos(7 * f[0]) + q[0] * math.sin(7 * f[0]))


def test_yarn_ramp_ends():
    f0, _ = O.rotary_freqs(16, 10000.0, None)
    f, mult = O.rotary_freqs(16, 10000.0, {"factor": 4.0, "original": 32, "fast": 16.0, "slow": 0.25})
    assert np.isclose(mult, 0.1 * math.log(4.0) + 1.0)
    assert np.isclose(f[0], f0[0]) and np.isclose(f[-1], f0[-1] / 4.0)      # fast pairs keep their frequency, slow ones are stretched
    assert np.all(np.diff(f / f0) <= 1e-12)


def test_sink_softmax():
    s = np.array([0.3, -1.0, 2.0])
    p = O.sink_softmax(s)
    assert np.allclose(p, np.exp(s) / (1.0 + np.exp(s).sum())) and p.sum() < 1.0
    assert np.allclose(O.sink_softmax(np.array([-800.0])), 0.0) and np.isclose(O.sink_softmax(np.array([800.0]))[0], 1.0)


def test_conv_step_is_a_causal_convolution():
    rng = np.random.default_rng(1)
    x, w, b = rng.normal(size=(9, 3)), rng.normal(size=(3, 4)), rng.normal(size=3)
    hist, got = np.zeros((3, 3)), []
    for t in range(9):
        y, hist = O.conv_step(hist, x[t], w, b)
        got.append(y)
    for c in range(3):
        want = np.convolve(x[:, c], w[c, ::-1])[:9] + b[c]       # the last column of w meets the current input
        assert np.allclose(np.asarray(got)[:, c], want)


def test_delta_rule_stores_and_overwrites():
    """with no decay and full write strength, writing value v at key k and then v' at the same unit key leaves exactly v' there"""
    cfg = {"vocab": 4, "width": 4, "norm": {"eps": 1e-6}, "layers": [{"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 3, "vdim": 2, "conv": 1}, "mlp": None}]}
    S = np.zeros((3, 2))
    k = np.array([0.6, 0.8, 0.0])
    for v in (np.array([1.0, -2.0]), np.array([5.0, 7.0])):
        u = 1.0 * (v - S.T @ k)
        S = S + np.outer(k, u)
    assert np.allclose(S.T @ k, [5.0, 7.0])
    # and the model's own step does the same arithmetic: one layer, hand-made weights
    w = O.random_weights(cfg, 0)
    m = O.Rofetar(cfg, w)
    st = m.new_state()
    x = m.w["embed"][1]
    m.delta(0, x, st)
    p = "l0.mix."
    q = O.silu(m.w[p + "q"] @ x * m.w[p + "q.conv"][:, -1])
    kk = O.silu(m.w[p + "k"] @ x * m.w[p + "k.conv"][:, -1])
    vv = O.silu(m.w[p + "v"] @ x * m.w[p + "v.conv"][:, -1])
    kk = kk / math.sqrt(kk @ kk + 1e-6)
    beta = O.sigmoid(m.w[p + "b"] @ x)[0]
    assert np.allclose(st["S"][0][0], np.outer(kk, beta * vv))
    assert q.shape == (3,)


def test_mamba_state_is_a_decayed_sum():
    cfg = {"vocab": 6, "width": 8, "norm": {"eps": 1e-6}, "layers": [{"type": "mamba2", "mixer": {"heads": 2, "vdim": 3, "state": 4, "groups": 1, "norm_groups": 1, "conv": 1}, "mlp": None}]}
    w = O.random_weights(cfg, 2)
    m = O.Rofetar(cfg, w)
    st = m.new_state()
    toks, want = [1, 4, 2, 5], np.zeros((2, 4, 3))
    p = "l0.mix."
    for t in toks:
        x = m.w["embed"][t]
        m.mamba2(0, x, st)
        u = m.w[p + "in"] @ x
        xbc = O.silu(u[6:20] * m.w[p + "conv"][:, -1] + m.w[p + "conv.b"])
        dt = O.softplus(u[20:] + m.w[p + "dt_bias"])
        for h in range(2):
            want[h] = math.exp(-math.exp(m.w[p + "A_log"][h]) * dt[h]) * want[h] + dt[h] * np.outer(xbc[6:10], xbc[3 * h:3 * h + 3])
    assert np.allclose(st["S"][0], want)


def test_gelu_glu_and_layer_shape():
    z = np.array([-3.0, -0.5, 0.0, 0.7, 4.0])
    assert np.allclose(O.gelu_tanh(z), 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))
    assert O.gelu_tanh(np.array([0.0]))[0] == 0.0 and abs(O.gelu_tanh(np.array([10.0]))[0] - 10.0) < 1e-9
    cfg = _cfg()
    w = O.random_weights(cfg, 3)
    assert set(w) == set(O.tensor_shapes(cfg)) and "l3.mix.k" not in w and "l0.norm2" not in w and "l1.mlp.down.b" in w
    lg, tr = O.Rofetar(cfg, w).run([1, 2, 3], layer_trace=True)
    assert lg.shape == (3, 40) and tr.shape == (4, 3, 24)
