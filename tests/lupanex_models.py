"""Small Lupanex models for the tests: configurations of the tests' own, random weights of the tests' own making.

None of the configurations is anybody's model.  Between them they vary what a single model would make equal: key
heads per value head (1:1, 2:1, 3:1), sizes of keys against values, taps of the short convolution (1, 2, 3, 4), residual
streams (none, 1, 2, 4), loops (none, once, three times, over one layer and over several), layers without a
feed-forward, attention with and without the distance bias and the query factor, widths that the tensor-core kernels
take and widths that they refuse.
"""
import json
import os

import numpy as np
import torch


def att(heads, kv, dim, vdim, scale, bias_max=None, q_temp=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale)
    if bias_max is not None:
        m["bias_max"] = bias_max
    if q_temp is not None:
        m["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    return m


def layer(kind, mixer, ff=None):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def delta(heads, kv, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)


def config(vocab, width, layers, *, max_positions=768, eps=1e-5, scale=1.5, streams=None, loop=None):
    c = dict(architecture="Lupanex", vocab=vocab, width=width, max_positions=max_positions, embedding=dict(scale=scale),
             norm=dict(eps=eps), layers=layers)
    if streams is not None:
        c["streams"] = streams
    if loop is not None:
        c["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return c


# two streams, a loop over both layers, tensor-core sizes, grouped heads, bias and query factor
CFG_LOOPED = config(97, 64, [layer("attention", att(4, 2, 32, 64, 0.35, bias_max=40, q_temp=(0.5, 16)), 96),
                             layer("delta", delta(4, 4, 32, 32, 4), 96)], streams=2, loop=(0, 2, 2))
# one plain residual stream, odd sizes that only the general kernels take, a layer without a feed-forward, no loop
CFG_PLAIN = config(61, 48, [layer("delta", delta(2, 1, 16, 24, 2)),
                            layer("attention", att(3, 1, 24, 16, 0.3), 80),
                            layer("attention", att(2, 2, 32, 32, 0.4, bias_max=24), 40),
                            layer("delta", delta(3, 1, 8, 40, 1), 56)], eps=1e-6, scale=0.7)
# four streams, a loop over the middle layer alone, three times; multi-query attention 3:1 with the query factor only
CFG_STREAMS = config(83, 96, [layer("delta", delta(6, 2, 32, 16, 3), 64),
                              layer("attention", att(3, 1, 64, 32, 0.25, q_temp=(0.2, 5)), 128),
                              layer("delta", delta(2, 2, 64, 64, 2))], streams=4, loop=(1, 2, 3), scale=2.5)
# a single stream that still goes through hyper-connections
CFG_ONE_STREAM = config(50, 32, [layer("attention", att(2, 1, 32, 32, 0.5, bias_max=10), 48), layer("delta", delta(1, 1, 32, 32, 2), 48)],
                        streams=1, loop=(1, 2, 1))

CONFIGS = {"looped": CFG_LOOPED, "plain": CFG_PLAIN, "streams": CFG_STREAMS, "one_stream": CFG_ONE_STREAM}
REL_ROWS = {"looped": 12, "plain": 8, "streams": 6, "one_stream": 6}


def make_tensors(cfg, seed, rel_rows=8, sharp=1.0):
    """name -> float32 array, drawn so that every mechanism matters: mixing matrices near the identity, decays spread
    between fast and slow, distance biases of order one, position rows as large as token rows."""
    rng = np.random.default_rng(seed)
    W, s = cfg["width"], cfg.get("streams")
    n = lambda *shape, std=1.0: (rng.standard_normal(shape) * std).astype(np.float32)
    t = {"embed": n(cfg["vocab"], W, std=0.5), "pos": n(cfg["max_positions"], W, std=0.3), "final.norm": 1 + n(W, std=0.1),
         "head": n(cfg["vocab"], W, std=W ** -0.5)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        t[p + "norm1"] = 1 + n(W, std=0.1)
        if l["type"] == "attention":
            t[p + "mix.q"] = n(m["heads"] * m["dim"], W, std=sharp * W ** -0.5)
            t[p + "mix.k"] = n(m["kv_heads"] * m["dim"], W, std=sharp * W ** -0.5)
            t[p + "mix.v"] = n(m["kv_heads"] * m["vdim"], W, std=W ** -0.5)
            t[p + "mix.o"] = n(W, m["heads"] * m["vdim"], std=(m["heads"] * m["vdim"]) ** -0.5)
            if "bias_max" in m:
                t[p + "mix.rel"] = n(rel_rows, m["heads"], std=1.5)
        else:
            qk, v = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for name, rows in (("q", qk), ("k", qk), ("v", v)):
                t[p + f"mix.{name}"] = n(rows, W, std=2 * W ** -0.5)
                t[p + f"mix.{name}.conv"] = n(rows, m["conv"], std=0.6)
            t[p + "mix.b"] = n(m["heads"], W, std=2 * W ** -0.5)
            t[p + "mix.a"] = n(m["heads"], W, std=2 * W ** -0.5)
            t[p + "mix.A_log"] = n(m["heads"], std=1.0) - 1.0
            t[p + "mix.dt_bias"] = n(m["heads"], std=1.0)
            t[p + "mix.norm"] = 1 + n(m["vdim"], std=0.1)
            t[p + "mix.g"] = n(v, W, std=2 * W ** -0.5)
            t[p + "mix.o"] = n(W, v, std=v ** -0.5)
        subs = [1]
        if l["mlp"] is not None:
            subs.append(2)
            t[p + "norm2"] = 1 + n(W, std=0.1)
            t[p + "mlp.up"] = n(l["mlp"]["ff"], W, std=1.5 * W ** -0.5)
            t[p + "mlp.down"] = n(W, l["mlp"]["ff"], std=l["mlp"]["ff"] ** -0.5)
        if s is not None:
            for q in subs:
                t[p + f"hc{q}.in"] = (np.full(s, 1.0 / s) + n(s, std=0.2)).astype(np.float32)
                t[p + f"hc{q}.out"] = 1 + n(s, std=0.3)
                t[p + f"hc{q}.mix"] = (np.eye(s) + n(s, s, std=0.15)).astype(np.float32)
    return t


def write_model(model_dir, cfg, tensors, dtype=torch.bfloat16):
    """config.json and model.safetensors; matrices are stored in `dtype` (the values a bfloat16 checkpoint holds are what
    both the engine and the plain implementation then read)."""
    from vitna_anchor_b200.weights import write_model_folder
    os.makedirs(model_dir, exist_ok=True)
    write_model_folder(model_dir, cfg, {k: torch.from_numpy(v).to(dtype) for k, v in tensors.items()})
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return str(model_dir)


def make_model(model_dir, name, seed=0, **kw):
    return write_model(model_dir, CONFIGS[name], make_tensors(CONFIGS[name], seed, REL_ROWS[name], **kw))
