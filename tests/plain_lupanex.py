"""A plain, slow statement of the Lupanex decoder in NumPy: whole sequences, no cache, one function per mechanism.

It shares nothing with the engine: its own reader of config.json and model.safetensors, its own arithmetic
(float64 unless told otherwise, so that it is the sharper side of every comparison).

Notation.  T tokens of one sequence at positions 0..T-1; W the width; a layer has a mixer and, unless its
configuration says null, a feed-forward; s residual streams.

  embedding        x_t = scale * E[id_t] + P[t]
  rms(x, w)        x / sqrt(mean(x^2) + eps) * w
  streams          X = [x, x, .., x] (s copies).  For a sublayer f with weights (a [s], M [s, s], b [s], w):
                   u = sum_i a_i X_i;  y = f(rms(u, w));  X_j <- sum_i M[i, j] X_i + b_j y.  At the end x = sum_j X_j.
  attention        q, k unit-RMS per head; q_t *= 1 + c ln(floor((t + 1) / e) + 1);
                   score(t, j) = scale (q_t . k_j) + R[bucket(t - j), head], j <= t; softmax; heads joined; W_o.
  delta            causal short convolution and silu on q, k, v; q, k unit length per head, q / sqrt(dim);
                   per head: S <- g S;  S <- S + k (beta (v - S^T k))^T;  o = S^T q;  then rms over vdim, a shared
                   weight, a silu gate, W_o.
  feed-forward     W_down act(W_up h), act the erf form of gelu.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ----------------------------------------------------------------------------------------------------------------
# reading a model folder
# ----------------------------------------------------------------------------------------------------------------

def read_tensors(path):
    """name -> array (float64 for floating tensors, int64 for integer ones)."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    directory = json.loads(raw[8:8 + n].decode("utf-8"))
    out = {}
    for name, d in directory.items():
        if name == "__metadata__":
            continue
        lo, hi = d["data_offsets"]
        blob = raw[8 + n + lo:8 + n + hi]
        if d["dtype"] == "BF16":
            a = (np.frombuffer(blob, "<u2").astype(np.uint32) << 16).view("<f4").astype(np.float64)
        elif d["dtype"] == "F32":
            a = np.frombuffer(blob, "<f4").astype(np.float64)
        elif d["dtype"] == "I32":
            a = np.frombuffer(blob, "<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {d['dtype']}")
        out[name] = a.reshape(d["shape"])
    return out


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_tensors(os.path.join(model_dir, "model.safetensors"))


# ----------------------------------------------------------------------------------------------------------------
# small pieces
# ----------------------------------------------------------------------------------------------------------------

def rms(x, eps, w=None):
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def silu(x):
    return x / (1.0 + np.exp(-x))


_erf = np.vectorize(math.erf, otypes=[np.float64])


def gelu_erf(x):
    return 0.5 * x * (1.0 + _erf(x / math.sqrt(2.0)))


def gelu_tanh(x):
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def softplus(x):
    return np.log1p(np.exp(-np.abs(x))) + np.maximum(x, 0.0)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def distance_bucket(n, rows, far):
    """Row of the distance table for the distance n >= 0: one row per distance below rows/2, then rows that widen
    geometrically up to the distance `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def embed(E, P, ids, scale, first=0):
    ids = np.asarray(ids)
    return E[ids] * scale + P[first:first + len(ids)]


# ----------------------------------------------------------------------------------------------------------------
# mixers
# ----------------------------------------------------------------------------------------------------------------

def attention(h, W, p, m, eps):
    """h [T, width] -> [T, width].  W: tensors, p: the layer's prefix, m: the mixer's configuration."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "mix.q"].T).reshape(T, H, dk)
    k = (h @ W[p + "mix.k"].T).reshape(T, G, dk)
    v = (h @ W[p + "mix.v"].T).reshape(T, G, dv)
    q, k = rms(q, eps), rms(k, eps)
    qt = m.get("q_temp")
    if qt is not None:
        t = np.arange(T)
        q = q * (1.0 + qt["coef"] * np.log(np.floor((t + 1) / qt["every"]) + 1.0))[:, None, None]
    rel = W.get(p + "mix.rel")
    out = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, hd]) * m["scale"]
            if rel is not None:
                s = s + np.array([rel[distance_bucket(t - j, rel.shape[0], m["bias_max"]), hd] for j in range(t + 1)])
            e = np.exp(s - s.max())
            out[t, hd] = (e / e.sum()) @ v[:t + 1, g]
    return out.reshape(T, H * dv) @ W[p + "mix.o"].T


def short_conv(x, w):
    """x [T, C], w [C, taps]; y_t = sum_i w[:, taps-1-i] x_{t-i}, zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = np.zeros_like(x)
    for i in range(taps):
        y[i:] += x[:T - i] * w[:, taps - 1 - i] if i else x * w[:, taps - 1]
    return y


def delta(h, W, p, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "mix.q"].T, W[p + "mix.q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "mix.k"].T, W[p + "mix.k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "mix.v"].T, W[p + "mix.v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, -1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt(np.sum(k * k, -1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[p + "mix.b"].T)                                                  # [T, H]
    decay = np.exp(-np.exp(W[p + "mix.A_log"]) * softplus(h @ W[p + "mix.a"].T + W[p + "mix.dt_bias"]))
    gate = silu(h @ W[p + "mix.g"].T).reshape(T, H, dv)
    o = np.zeros((T, H, dv))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = rms(o, eps, W[p + "mix.norm"]) * gate
    return o.reshape(T, H * dv) @ W[p + "mix.o"].T


def feed_forward(h, W, p, mlp):
    if mlp.get("kind", "dense") != "dense":
        raise ValueError(f"feed-forward kind {mlp.get('kind')}")
    return gelu_erf(h @ W[p + "mlp.up"].T) @ W[p + "mlp.down"].T


MIXERS = {"attention": attention, "delta": delta}


# ----------------------------------------------------------------------------------------------------------------
# the whole model
# ----------------------------------------------------------------------------------------------------------------

def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def forward(cfg, W, ids, want_layers=False):
    """Logits [T, vocab] of one whole sequence (and, if asked, the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = embed(W["embed"], W["pos"], ids, cfg["embedding"]["scale"])
    s = cfg.get("streams")
    X = None if s is None else [x.copy() for _ in range(s)]
    after = []
    for l in order_with_names(cfg):
        spec, p = cfg["layers"][l], f"l{l}."
        subs = [(1, lambda h: MIXERS[spec["type"]](h, W, p, spec["mixer"], eps))]
        if spec.get("mlp") is not None:
            subs.append((2, lambda h: feed_forward(h, W, p, spec["mlp"])))
        for qn, f in subs:
            w = W[p + f"norm{qn}"]
            if X is None:
                x = x + f(rms(x, eps, w))
            else:
                a, M, b = W[p + f"hc{qn}.in"], W[p + f"hc{qn}.mix"], W[p + f"hc{qn}.out"]
                y = f(rms(sum(a[i] * X[i] for i in range(s)), eps, w))
                X = [sum(M[i, j] * X[i] for i in range(s)) + b[j] * y for j in range(s)]
        after.append(x.copy() if X is None else sum(X))
    if X is not None:
        x = sum(X)
    logits = rms(x, eps, W["final.norm"]) @ W["head"].T
    return (logits, np.stack(after)) if want_layers else logits


def order_with_names(cfg):
    return layer_order(cfg)
