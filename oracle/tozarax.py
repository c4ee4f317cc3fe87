"""Plain, slow restatement of the Tozarax decoder: learned positions, pre-normed sublayers that read their input through a short
causal "input convolution", a mixer made of two mixers side by side (sliding-window softmax attention without rotation beside a
gated delta rule), a sigmoid-routed mixture of small squared-relu experts with group-limited choice, a learned gate on every
sublayer's contribution and a learned average over the outputs of all earlier layers.  Test infrastructure only: numpy, one
function per mechanism, token by token, float64.  Nothing of the product imports this file and this file imports nothing of the
product.

Notation: n = norm(x) is what a sublayer is handed, W matrices are [out, in] and applied as W @ n.
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces ----------------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """the layer norms and the final norm: the stored weight sits around zero"""
    return unit_rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def causal_taps(hist, x, w):
    """per-channel causal convolution of one new input: hist [taps-1, channels] are the inputs before it (oldest first, zeros
    before the sequence's start), w [channels, taps] with the last column on the new input.  -> (output, new hist)"""
    full = np.concatenate([hist, x[None, :]], axis=0)
    return np.einsum("tc,ct->c", full, w), full[1:]


def input_conv(hist, n, w):
    """what a sublayer reads: n + conv(n)"""
    y, hist = causal_taps(hist, n, w)
    return n + y, hist


def window_softmax_attention(q, K, V, pos, window, scale, groups):
    """q [H, D]; K [n, G, D], V [n, G, Dv] hold positions 0..pos; position pos sees j with 0 <= pos - j < window"""
    H = q.shape[0]
    lo = max(0, pos - window + 1)
    out = np.zeros((H, V.shape[-1]))
    for h in range(H):
        g = h // (H // groups)
        s = (K[lo:pos + 1, g, :] @ q[h]) * scale
        e = np.exp(s - s.max())
        out[h] = (e / e.sum()) @ V[lo:pos + 1, g, :]
    return out


def delta_rule_step(S, q, k, v, beta, decay):
    """one head, one token: S [D, Dv] forgets, is corrected towards v along k, then is read by q (which sees the correction)"""
    S = decay * S
    u = beta * (v - S.T @ k)
    S = S + np.outer(k, u)
    return S, S.T @ q


def route(z, correction, top, n_groups, keep):
    """z: router logits.  -> (chosen experts, their weights).  Choice by sigmoid(z) + correction inside the `keep` best groups
    (a group's mark: the sum of its two largest choice scores); weights are sigmoid(z) of the chosen, as they are."""
    s = sigmoid(z)
    c = s + correction
    E = len(z)
    per = E // n_groups
    marks = np.array([np.sort(c[g * per:(g + 1) * per])[-2:].sum() for g in range(n_groups)])
    kept = np.argsort(-marks, kind="stable")[:keep]
    masked = np.full(E, -np.inf)
    for g in kept:
        masked[g * per:(g + 1) * per] = c[g * per:(g + 1) * per]
    chosen = np.argsort(-masked, kind="stable")[:top]
    return chosen, s[chosen]


def relu2_expert(x, up, down):
    a = np.maximum(up @ x, 0.0)
    return down @ (a * a)


# ---- the model -------------------------------------------------------------------------------------------------------
class Tozarax:
    """weights: dict name -> float array holding the values the product sees (bf16-representable).
    cache_round: optional function applied to the keys and values the attention caches."""

    def __init__(self, config: dict, weights: dict, cache_round=None):
        self.cfg = config
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.layers = config["layers"]
        self.taps = int(config["canon"]["taps"])
        self.W = int(config["width"])
        self.cache_round = cache_round

    def new_state(self):
        st = {"pos": 0, "kv": {}, "S": {}, "conv": {}, "canon": {}}
        for i, l in enumerate(self.layers):
            if l["type"] != "parallel":
                raise ValueError(l["type"])
            a, r = l["mixer"]["left"], l["mixer"]["right"]
            st["kv"][i] = ([], [])
            st["S"][i] = np.zeros((r["heads"], r["dim"], r["vdim"]))
            st["conv"][i] = {"q": np.zeros((r["conv"] - 1, r["kv_heads"] * r["dim"])),
                             "k": np.zeros((r["conv"] - 1, r["kv_heads"] * r["dim"])),
                             "v": np.zeros((r["conv"] - 1, r["heads"] * r["vdim"]))}
            st["canon"][i] = [np.zeros((self.taps - 1, self.W)), np.zeros((self.taps - 1, self.W))]
        return st

    # -- the two mixers of a layer --
    def left(self, i, h, st):
        m, w, p = self.layers[i]["mixer"]["left"], self.w, f"l{i}.mix.left."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q = (w[p + "q"] @ h).reshape(H, D)
        k = (w[p + "k"] @ h).reshape(G, D)
        v = (w[p + "v"] @ h).reshape(G, Dv)
        if self.cache_round is not None:
            k, v = np.asarray(self.cache_round(k), dtype=np.float64), np.asarray(self.cache_round(v), dtype=np.float64)
        st["kv"][i][0].append(k)
        st["kv"][i][1].append(v)
        o = window_softmax_attention(q, np.stack(st["kv"][i][0]), np.stack(st["kv"][i][1]), st["pos"], int(m["mask"]["size"]),
                                     float(m["scale"]), G)
        return w[p + "o"] @ o.reshape(-1)

    def right(self, i, h, st):
        m, w, p = self.layers[i]["mixer"]["right"], self.w, f"l{i}.mix.right."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        cs = st["conv"][i]
        q, cs["q"] = causal_taps(cs["q"], w[p + "q"] @ h, w[p + "q.conv"])
        k, cs["k"] = causal_taps(cs["k"], w[p + "k"] @ h, w[p + "k.conv"])
        v, cs["v"] = causal_taps(cs["v"], w[p + "v"] @ h, w[p + "v.conv"])
        q, k, v = silu(q).reshape(G, D), silu(k).reshape(G, D), silu(v).reshape(H, Dv)
        q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * D ** -0.5
        k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
        beta = sigmoid(w[p + "b"] @ h)
        decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(w[p + "a"] @ h + w[p + "dt_bias"]))
        o = np.zeros((H, Dv))
        for hd in range(H):
            g = hd // (H // G)
            st["S"][i][hd], o[hd] = delta_rule_step(st["S"][i][hd], q[g], k[g], v[hd], beta[hd], decay[hd])
        o = (unit_rms(o, self.eps) * w[p + "norm"]).reshape(-1) * silu(w[p + "g"] @ h)
        return w[p + "o"] @ o

    def mixer(self, i, h, st):
        w, p = self.w, f"l{i}.mix."
        a = unit_rms(self.left(i, h, st), self.eps) * w[p + "left.out"]
        b = unit_rms(self.right(i, h, st), self.eps) * w[p + "right.out"]
        return 0.5 * (a + b)

    def experts(self, i, h):
        c, w, p = self.layers[i]["mlp"], self.w, f"l{i}.mlp."
        r = c["router"]
        chosen, wts = route(w[p + "router"] @ h, w[p + "correction"], int(r["top"]), int(r["groups"]["count"]), int(r["groups"]["keep"]))
        y = np.zeros(self.W)
        for e, g in zip(chosen, wts):
            y = y + g * relu2_expert(h, w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
        return y

    # -- one token through every layer --
    def step(self, token, st, layer_trace=None):
        w, eps = self.w, self.eps
        x = w["embed"][int(token)] + w["pos"][st["pos"]]
        outs = [x.copy()]                        # X_0, X_1, ...: the embedding output and every layer's own result
        for i, l in enumerate(self.layers):
            n = norm_one_plus(x, w[f"l{i}.norm1"], eps)
            gate = sigmoid(w[f"l{i}.rg1"] @ n + w[f"l{i}.rg1.b"])
            h, st["canon"][i][0] = input_conv(st["canon"][i][0], n, w[f"l{i}.canon1"])
            x = x + gate * self.mixer(i, h, st)
            if l.get("mlp"):
                n = norm_one_plus(x, w[f"l{i}.norm2"], eps)
                gate = sigmoid(w[f"l{i}.rg2"] @ n + w[f"l{i}.rg2.b"])
                h, st["canon"][i][1] = input_conv(st["canon"][i][1], n, w[f"l{i}.canon2"])
                x = x + gate * self.experts(i, h)
            outs.append(x.copy())
            x = np.tensordot(w[f"l{i}.dwa"], np.stack(outs), axes=1)
            if layer_trace is not None:
                layer_trace.append(x.copy())
        st["pos"] += 1
        return w["head"] @ norm_one_plus(x, w["final.norm"], eps)

    def run(self, tokens, st=None, layer_trace=False):
        """-> logits [len(tokens), vocab] (and the residual stream after every layer [layers, tokens, width] if asked)"""
        st = st if st is not None else self.new_state()
        out, tr = [], []
        for t in tokens:
            lt = [] if layer_trace else None
            out.append(self.step(t, st, lt))
            if layer_trace:
                tr.append(lt)
        logits = np.stack(out)
        if layer_trace:
            return logits, np.transpose(np.asarray(tr), (1, 0, 2))
        return logits


# ---- random models for tests -----------------------------------------------------------------------------------------
def to_bf16(a):
    """round-to-nearest-even to bfloat16, returned as float32"""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.view(np.float32)


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor the configuration asks for"""
    W, V, T, out = cfg["width"], cfg["vocab"], cfg["canon"]["taps"], {}
    out["embed"], out["pos"], out["head"], out["final.norm"] = (V, W), (cfg["max_positions"], W), (V, W), (W,)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        a, r = l["mixer"]["left"], l["mixer"]["right"]
        out[p + "norm1"], out[p + "canon1"], out[p + "rg1"], out[p + "rg1.b"] = (W,), (W, T), (W, W), (W,)
        out[p + "dwa"] = (i + 2,)
        H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        q = p + "mix.left."
        out[q + "q"], out[q + "k"], out[q + "v"], out[q + "o"] = (H * D, W), (G * D, W), (G * Dv, W), (W, H * Dv)
        H, G, D, Dv = r["heads"], r["kv_heads"], r["dim"], r["vdim"]
        q = p + "mix.right."
        for n, rows in (("q", G * D), ("k", G * D), ("v", H * Dv)):
            out[q + n], out[q + n + ".conv"] = (rows, W), (rows, r["conv"])
        out[q + "b"], out[q + "a"], out[q + "A_log"], out[q + "dt_bias"], out[q + "norm"] = (H, W), (H, W), (H,), (H,), (Dv,)
        out[q + "g"], out[q + "o"] = (H * Dv, W), (W, H * Dv)
        out[p + "mix.left.out"], out[p + "mix.right.out"] = (W,), (W,)
        c = l.get("mlp")
        if not c:
            continue
        out[p + "norm2"], out[p + "canon2"], out[p + "rg2"], out[p + "rg2.b"] = (W,), (W, T), (W, W), (W,)
        E, F = c["router"]["experts"], c["expert"]["ff"]
        out[p + "mlp.router"], out[p + "mlp.correction"] = (E, W), (E,)
        for e in range(E):
            out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = (F, W), (W, F)
    return out


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """bf16-representable random weights: matrices N(0, 1/in); plain norm weights around 1, one-plus weights around 0; decays
    spread over fast and slow heads; every layer's depth average near "mostly the newest output"."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shp in tensor_shapes(cfg).items():
        if name.endswith("A_log"):
            a = rng.uniform(-3.0, 1.0, shp)
        elif name.endswith("dt_bias"):
            a = rng.uniform(-3.0, 0.5, shp)
        elif name.endswith(".conv") or ".canon" in name:
            a = rng.normal(0.0, 0.5, shp)
        elif name.endswith(".dwa"):
            a = rng.normal(0.0, 0.25, shp)
            a[-1] += 1.0
        elif name.endswith("correction"):
            a = rng.normal(0.0, 0.3, shp)
        elif name.endswith("router"):
            a = rng.normal(0.0, 2.0, shp) / math.sqrt(shp[1])
        elif len(shp) == 1:
            a = rng.normal(0.0, 0.2, shp)
            if name.endswith(("mix.right.norm", "left.out", "right.out")):
                a = 1.0 + a
        elif name == "embed":
            a = rng.normal(0.0, 1.0, shp)
        elif name == "pos":
            a = rng.normal(0.0, 0.5, shp)
        else:
            a = rng.normal(0.0, 1.0, shp) / math.sqrt(shp[1])
        w[name] = to_bf16(a)
    return w
