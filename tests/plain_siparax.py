"""A plain, slow statement of the Siparax decoder in NumPy: whole sequences, no cache, one function per mechanism.

It shares nothing with the engine: its own reader of config.json and model.safetensors, its own arithmetic
(float64, so that it is the sharper side of every comparison).

Notation.  T tokens of one sequence at positions 0..T-1; W the width; every layer is  x += mixer(ln(x)), and, unless its
configuration says null,  x += ff(ln(x)),  ln the layer norm with weight and bias.

  embedding        x_t = ln(E[id_t])
  latent attention cq = rms(W_dq h) w;  q = W_uq cq, per head [dim plain | rot rotated];  W_dkv h = [c_raw | kr];
                   c = rms(c_raw) w;  per head k = W_uk c, v = W_uv c;  score(t, j) = scale (q_plain . k_j + rot(q_rot, t) . rot(kr_j, j)),
                   j <= t;  softmax;  (second form: head h times sigmoid(W_g h)_h; a layer may take c and kr of another layer);  W_o.
  rotation         pair (u, v) at position p -> (u cos a - v sin a, v cos a + u sin a), a = p f_i; pairs (2i, 2i+1) or (i, i + n/2);
                   f_i blended between base^(-2i/n) and that over `factor` by a ramp over i; cos and sin times 0.1 ln(factor) + 1.
  channel delta    causal short convolution and silu on q, k, v; q, k unit length per head, q / sqrt(dim); beta = sigmoid(W_b h);
                   g = exp(-exp(A_h) softplus(W_a2 W_a1 h + dt)) per head and key channel;
                   per head: S <- diag(g) S;  S <- S + k (beta (v - S^T k))^T;  o = S^T q;  then rms over vdim, a shared
                   weight, sigmoid(W_g2 W_g1 h), W_o.
  feed-forward     W_down (gelu_tanh(W_gate h) * (W_up h)).
  output           cap * tanh(head ln(x) / cap)
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


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


def layer_norm(x, w, b, eps):
    mu = np.mean(x, axis=-1, keepdims=True)
    var = np.mean((x - mu) ** 2, axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def silu(x):
    return x / (1.0 + np.exp(-x))


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def softplus(x):
    return np.maximum(x, 0.0) + np.log1p(np.exp(-np.abs(x)))


def gelu_tanh(x):
    return 0.5 * x * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


# ----------------------------------------------------------------------------------------------------------------
# rotation
# ----------------------------------------------------------------------------------------------------------------

def rotation_frequencies(rot):
    """(f [dims/2], factor on cos and sin) of a rotation {base, dims, scaling {factor, original, fast, slow} or absent}."""
    n, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / n) for i in range(n // 2)])
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def at(turns):
        return n * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(float(sc["fast"]))), 0)
    hi = min(math.ceil(at(float(sc["slow"]))), n - 1)
    ramp = np.clip((np.arange(n // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, first, rot, pairing):
    """x [T, ..., n] at positions first..first+T-1; only the first rot.dims entries of the last axis turn."""
    n = int(rot["dims"])
    f, mag = rotation_frequencies(rot)
    pos = np.arange(first, first + x.shape[0], dtype=np.float64)
    a = pos[:, None] * f[None, :]
    a = a.reshape((x.shape[0],) + (1,) * (x.ndim - 2) + (n // 2,))
    cos, sin = np.cos(a) * mag, np.sin(a) * mag
    out = x.copy()
    if pairing == "interleaved":
        u, v = x[..., 0:n:2], x[..., 1:n:2]
        out[..., 0:n:2] = u * cos - v * sin
        out[..., 1:n:2] = v * cos + u * sin
    else:
        u, v = x[..., :n // 2], x[..., n // 2:n]
        out[..., :n // 2] = u * cos - v * sin
        out[..., n // 2:n] = v * cos + u * sin
    return out


# ----------------------------------------------------------------------------------------------------------------
# mixers
# ----------------------------------------------------------------------------------------------------------------

def latent_kv(h, W, p, m, eps, pairing):
    """What a latent attention layer keeps of every token: (c [T, kv_rank], rotated shared key part [T, rot_dim])."""
    r = int(m["kv_rank"])
    ckv = h @ W[p + "dkv"].T
    c = rms(ckv[:, :r], eps, W[p + "dkv.norm"])
    return c, rotate(ckv[:, r:], 0, m["rot"], pairing)


def latent_attention(h, W, p, m, eps, pairing, kv, gated):
    T = h.shape[0]
    H, dim, rd, vd, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms(h @ W[p + "dq"].T, eps, W[p + "dq.norm"])
    q = (cq @ W[p + "uq"].T).reshape(T, H, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], 0, m["rot"], pairing)
    c, kr = kv
    k = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vd)
    out = np.zeros((T, H, vd))
    for t in range(T):
        s = (np.einsum("hd,jhd->hj", q_plain[t], k[:t + 1]) + np.einsum("hd,jd->hj", q_rot[t], kr[:t + 1])) * float(m["scale"])
        s = s - s.max(axis=1, keepdims=True)
        w = np.exp(s)
        w /= w.sum(axis=1, keepdims=True)
        out[t] = np.einsum("hj,jhd->hd", w, v[:t + 1])
    if gated:
        out = out * sigmoid(h @ W[p + "g"].T)[:, :, None]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def short_conv(x, w):
    """x [T, C], w [C, taps], the last column the current token's; zeros before the start."""
    taps = w.shape[1]
    xp = np.concatenate([np.zeros((taps - 1, x.shape[1])), x], axis=0)
    return sum(xp[j:j + x.shape[0]] * w[:, j] for j in range(taps))


def channel_delta(h, W, p, m, eps):
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m.get("vdim") or m["dim"])
    G = int(m.get("kv_heads") or H)
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].T)
    a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, dk))
    gate = sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, dv)
    o = np.zeros((T, H, dv))
    for hh in range(H):
        kh = hh // (H // G)
        S = np.zeros((dk, dv))
        for t in range(T):
            S = g[t, hh][:, None] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, kh])
            S = S + np.outer(k[t, kh], u)
            o[t, hh] = S.T @ q[t, kh]
    o = rms(o, eps, W[p + "norm"]) * gate
    return o.reshape(T, H * dv) @ W[p + "o"].T


def feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ----------------------------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------------------------

PAIRING = {"latent_attention": "interleaved", "latent_attention_2": "half"}


def forward(cfg, W, ids, want_layers=False):
    """Logits [T, vocab] of one sequence from its first token (and the residual stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    x = layer_norm(W["embed"][np.asarray(ids)], W["embed.norm"], W["embed.norm.b"], eps)
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if kind == "channel_delta":
            y = channel_delta(h, W, p + "mix.", m, eps)
        elif kind in PAIRING:
            if m.get("kv_from") is not None:
                kv = kept[int(m["kv_from"])]
            else:
                kv = kept[i] = latent_kv(h, W, p + "mix.", m, eps, PAIRING[kind])
            y = latent_attention(h, W, p + "mix.", m, eps, PAIRING[kind], kv, gated=kind == "latent_attention_2")
        else:
            raise ValueError(f"layer {i}: type {kind!r}")
        x = x + y
        if layer.get("mlp") is not None:
            x = x + feed_forward(layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps), W, p + "mlp.")
        after.append(x.copy())
    z = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap is not None:
        z = float(cap) * np.tanh(z / float(cap))
    return (z, np.stack(after)) if want_layers else z
