"""Plain, slow restatement of the Medulorn decoder: a post-norm stack (the norm follows the sum of the scaled stream and the
sublayer's result, with one number as its weight) whose mixers read their input through a token shift; layers of grouped-query
softmax attention (biased projections, per-head q/k norm, partial half-split rotation, chunk mask, a sink of score zero) and
layers that run a sliding-window attention (q/k norm over the whole projection, Llama-3.1 frequency scaling, kept first tokens, a
learned sink per head) beside lightning attention (a linear recurrence with one fixed decay per head); dense relu-gated or
mixture-of-experts feed-forward (clamped swish experts, biased router, softmax over the chosen logits, an always-on shared
expert); scaled embedding and capped logits.  Test infrastructure only: numpy, one function per mechanism, token by token,
float64.  Nothing of the product imports this file and this file imports nothing of the product.

Notation: x = the residual row, h = what a mixer reads, W matrices are [out, in] and applied as W @ h.
"""
from __future__ import annotations

import math

import numpy as np


# ---- small pieces ----------------------------------------------------------------------------------------------------
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def token_shift(h, prev, mu):
    """the mixer's input: every channel moves from this token's value towards the previous token's by its own share mu"""
    return h + (prev - h) * mu


def rotary_freqs(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with Llama-3.1 scaling, slow pairs (wavelength above original/low) are divided by the
    factor, fast ones (below original/high) stay, the band between is blended linearly in original/wavelength"""
    f = np.array([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)])
    if scaling:
        fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f:
            wl = 2.0 * math.pi / fi
            if wl < orig / hi:
                out.append(fi)
            elif wl > orig / lo:
                out.append(fi / fac)
            else:
                s = (orig / wl - lo) / (hi - lo)
                out.append((1.0 - s) * fi / fac + s * fi)
        f = np.array(out)
    return f


def rotate_halves(v, pos, freqs):
    """v [heads, dim]: channel i turns with channel i + n/2 by the angle pos * f_i, n = 2 len(freqs) leading channels"""
    n = 2 * len(freqs)
    if n == 0:
        return v
    a = pos * freqs
    c, s = np.cos(a), np.sin(a)
    u, w = v[:, :n // 2], v[:, n // 2:n]
    return np.concatenate([u * c - w * s, w * c + u * s, v[:, n:]], axis=1)


def visible(i, j, window=0, keep_first=0, chunk=0):
    """may position i read position j?"""
    if j > i:
        return False
    if chunk and i // chunk != j // chunk:
        return False
    if window and not (i - j < window or j < keep_first):
        return False
    return True


def sink_softmax_attention(q, K, V, keys, scale, sinks):
    """q [H, D]; K [n, G, D], V [n, G, Dv]; keys: the positions this query may read; sinks [H]: a score per head that joins the
    denominator without a value (None: a plain softmax)"""
    H, G = q.shape[0], K.shape[1]
    out = np.zeros((H, V.shape[-1]))
    for h in range(H):
        g = h // (H // G)
        s = (K[keys, g, :] @ q[h]) * scale
        m = max(s.max(), sinks[h]) if sinks is not None else s.max()
        e = np.exp(s - m)
        den = e.sum() + (np.exp(sinks[h] - m) if sinks is not None else 0.0)
        out[h] = (e / den) @ V[keys, g, :]
    return out


def lightning_step(S, q, k, v, decay):
    """one head, one token: S [D, Dv] fades by a fixed factor, takes k v^T, and is read by q"""
    S = decay * S + np.outer(k, v)
    return S, S.T @ q


def clamped_swish_expert(h, gate, up, down, limit):
    g = np.minimum(gate @ h, limit)
    u = np.clip(up @ h, -limit, limit)
    return down @ (g * sigmoid(1.702 * g) * (u + 1.0))


def relu_glu(h, gate, up, down):
    return down @ (np.maximum(gate @ h, 0.0) * (up @ h))


def route_top(z, top):
    """the `top` largest logits (lower index first among equals) and the softmax over just those"""
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    zz = np.array([z[e] for e in order])
    e = np.exp(zz - zz.max())
    return order, e / e.sum()


# ---- the model -------------------------------------------------------------------------------------------------------
class Medulorn:
    """weights: dict name -> float array holding the values the product sees (bf16-representable; norm weights of one number may
    come as 0-d or 1-element arrays).  cache_round: optional function applied to the keys and values the attentions cache."""

    def __init__(self, config: dict, weights: dict, cache_round=None):
        self.cfg = config
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.eps = float(config["norm"]["eps"])
        self.alpha = float(config["postln_alpha"])
        self.layers = config["layers"]
        self.W = int(config["width"])
        self.cache_round = cache_round
        self.freqs = {}

    def new_state(self):
        st = {"pos": 0, "kv": {}, "S": {}, "prev": {}}
        for i, l in enumerate(self.layers):
            st["prev"][i] = np.zeros(self.W)
            if l["type"] == "attention":
                st["kv"][i] = ([], [])
            elif l["type"] == "parallel":
                st["kv"][i] = ([], [])
                r = l["mixer"]["right"]
                st["S"][i] = np.zeros((r["heads"], r["dim"], r["vdim"]))
            else:
                raise ValueError(l["type"])
        return st

    def scalar_norm(self, x, name):
        return unit_rms(x, self.eps) * float(np.asarray(self.w[name]).reshape(-1)[0])

    def _freqs(self, key, rot):
        if key not in self.freqs:
            self.freqs[key] = rotary_freqs(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot and rot.get("dims") else np.zeros(0)
        return self.freqs[key]

    def softmax_attention(self, i, m, p, h, st, whole_norm, bias, learned_sink):
        w = self.w
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q, k, v = w[p + "q"] @ h, w[p + "k"] @ h, w[p + "v"] @ h
        if bias:
            q, k, v = q + w[p + "q.b"], k + w[p + "k.b"], v + w[p + "v.b"]
        if whole_norm:
            q = (unit_rms(q, self.eps) * w[p + "q.norm"]).reshape(H, D)
            k = (unit_rms(k, self.eps) * w[p + "k.norm"]).reshape(G, D)
        else:
            q = unit_rms(q.reshape(H, D), self.eps) * w[p + "q.norm"]
            k = unit_rms(k.reshape(G, D), self.eps) * w[p + "k.norm"]
        f = self._freqs(p, m.get("rot"))
        pos = st["pos"]
        q, k = rotate_halves(q, pos, f), rotate_halves(k, pos, f)
        v = v.reshape(G, Dv)
        if self.cache_round is not None:
            k, v = np.asarray(self.cache_round(k), dtype=np.float64), np.asarray(self.cache_round(v), dtype=np.float64)
        st["kv"][i][0].append(k)
        st["kv"][i][1].append(v)
        mask = m.get("mask") or {}
        if whole_norm:      # the windowed kind
            keys = [j for j in range(pos + 1) if visible(pos, j, window=int(mask.get("size") or 0), keep_first=int(mask.get("keep_first") or 0))]
        else:
            keys = [j for j in range(pos + 1) if visible(pos, j, chunk=int(mask.get("size") or 0))]
        sinks = w[p + "sink"] if learned_sink else np.zeros(H)
        o = sink_softmax_attention(q, np.stack(st["kv"][i][0]), np.stack(st["kv"][i][1]), keys, float(m["scale"]), sinks)
        return w[p + "o"] @ o.reshape(-1)

    def lightning(self, i, m, p, h, st):
        w = self.w
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        q, k, v = silu(w[p + "q"] @ h).reshape(H, D), silu(w[p + "k"] @ h).reshape(H, D), silu(w[p + "v"] @ h).reshape(H, Dv)
        o = np.zeros((H, Dv))
        for hd in range(H):
            st["S"][i][hd], o[hd] = lightning_step(st["S"][i][hd], q[hd], k[hd], v[hd], float(m["decay"][hd]))
        o = unit_rms(o.reshape(-1), self.eps) * w[p + "norm"] * sigmoid(w[p + "g"] @ h)
        return w[p + "o"] @ o

    def mixer(self, i, h, st):
        l = self.layers[i]
        m = l["mixer"]
        if l["type"] == "attention":
            return self.softmax_attention(i, m, f"l{i}.mix.", h, st, whole_norm=False, bias=True, learned_sink=False)
        a = self.softmax_attention(i, m["left"], f"l{i}.mix.left.", h, st, whole_norm=True, bias=False, learned_sink=True)
        b = self.lightning(i, m["right"], f"l{i}.mix.right.", h, st)
        return float(m["left_scale"]) * a + float(m["right_scale"]) * b

    def feed_forward(self, i, x):
        c, w, p = self.layers[i]["mlp"], self.w, f"l{i}.mlp."
        if c["kind"] == "dense":
            return relu_glu(x, w[p + "gate"], w[p + "up"], w[p + "down"])
        chosen, wts = route_top(w[p + "router"] @ x + w[p + "router.b"], int(c["router"]["top"]))
        y = np.zeros(self.W)
        lim = float(c["expert"]["limit"])
        for e, g in zip(chosen, wts):
            y = y + g * clamped_swish_expert(x, w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], lim)
        if c.get("shared"):
            y = y + clamped_swish_expert(x, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], float(c["shared"]["limit"]))
        return y

    # -- one token through every layer --
    def step(self, token, st, layer_trace=None):
        w = self.w
        x = w["embed"][int(token)] * float(self.cfg["embedding"]["scale"])
        for i, l in enumerate(self.layers):
            h = token_shift(x, st["prev"][i], w[f"l{i}.shift"])
            st["prev"][i] = x.copy()
            x = self.scalar_norm(self.alpha * x + self.mixer(i, h, st), f"l{i}.norm1")
            if l.get("mlp"):
                x = self.scalar_norm(self.alpha * x + self.feed_forward(i, x), f"l{i}.norm2")
            if layer_trace is not None:
                layer_trace.append(x.copy())
        st["pos"] += 1
        z = w["head"] @ self.scalar_norm(x, "final.norm")
        cap = float(self.cfg.get("logit_softcap") or 0.0)
        return cap * np.tanh(z / cap) if cap else z

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
    shape = np.shape(a)
    b = np.ascontiguousarray(a, dtype=np.float32).reshape(-1).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.view(np.float32).reshape(shape)


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor the configuration asks for"""
    W, V, out = cfg["width"], cfg["vocab"], {}
    out["embed"], out["head"], out["final.norm"] = (V, W), (V, W), ()

    def softmax_mixer(q, m, bias, whole, sink):
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[q + "q"], out[q + "k"], out[q + "v"], out[q + "o"] = (H * D, W), (G * D, W), (G * Dv, W), (W, H * Dv)
        if bias:
            out[q + "q.b"], out[q + "k.b"], out[q + "v.b"] = (H * D,), (G * D,), (G * Dv,)
        out[q + "q.norm"], out[q + "k.norm"] = ((H * D,), (G * D,)) if whole else ((D,), (D,))
        if sink:
            out[q + "sink"] = (H,)

    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        out[p + "norm1"], out[p + "shift"] = (), (W,)
        if l["type"] == "attention":
            softmax_mixer(p + "mix.", l["mixer"], True, False, False)
        else:
            softmax_mixer(p + "mix.left.", l["mixer"]["left"], False, True, True)
            r, q = l["mixer"]["right"], p + "mix.right."
            H, D, Dv = r["heads"], r["dim"], r["vdim"]
            out[q + "q"], out[q + "k"], out[q + "v"], out[q + "g"] = (H * D, W), (H * D, W), (H * Dv, W), (H * Dv, W)
            out[q + "norm"], out[q + "o"] = (H * Dv,), (W, H * Dv)
        c = l.get("mlp")
        if not c:
            continue
        out[p + "norm2"] = ()
        if c["kind"] == "dense":
            F = c["ff"]
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (F, W), (F, W), (W, F)
            continue
        E, F = c["router"]["experts"], c["expert"]["ff"]
        out[p + "mlp.router"], out[p + "mlp.router.b"] = (E, W), (E,)
        for e in range(E):
            out[f"{p}mlp.e{e}.gate"], out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = (F, W), (F, W), (W, F)
        if c.get("shared"):
            Fs = c["shared"]["ff"]
            out[p + "mlp.shared.gate"], out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = (Fs, W), (Fs, W), (W, Fs)
    return out


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """bf16-representable random weights: matrices N(0, 1/in); norm weights around 1; shifts in (0, 1); sinks and biases of
    order one; router rows wide enough that the choice is rarely a near-tie"""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shp in tensor_shapes(cfg).items():
        if name.endswith(".shift"):
            a = rng.uniform(0.05, 0.95, shp)
        elif name.endswith(("norm1", "norm2")) or name == "final.norm":
            a = np.asarray(rng.uniform(0.7, 1.6))
        elif name.endswith(".norm"):
            a = 1.0 + rng.normal(0.0, 0.2, shp)
        elif name.endswith(".sink"):
            a = rng.normal(0.0, 1.0, shp)
        elif name.endswith("router"):
            a = rng.normal(0.0, 2.0, shp) / math.sqrt(shp[1])
        elif name.endswith(".b"):
            a = rng.normal(0.0, 0.5, shp)
        elif name == "embed":
            a = rng.normal(0.0, 1.0, shp) / float(cfg["embedding"]["scale"])
        else:
            a = rng.normal(0.0, 1.0, shp) / math.sqrt(shp[1])
        w[name] = to_bf16(a)
    return w
