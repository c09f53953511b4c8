"""Small Siparax models for the tests: configurations of the tests' own, random weights of the tests' own making.

None of the configurations is anybody's model.  Between them they vary what a single model would make equal: heads,
plain against rotated against value sizes, ranks of the two latents, rotations with and without rescaled frequencies
and with fewer turned values than the rotated part has, layers that read another layer's cached rows, key heads per value
head of the delta rule (1:1, 2:1, 3:1), key against value sizes, taps (1 to 4), ranks of the two low-rank projections,
layers without a feed-forward, logits with and without a cap, sizes the tensor-core kernels take and sizes they refuse.
"""
import json
import os

import numpy as np
import torch


def rot(base, dims, scaling=None):
    r = dict(base=base, dims=dims)
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rotation, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale, rot=rotation)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def cdelta(heads, kv, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)


def layer(kind, mixer, ff=None):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(kind="dense", ff=ff))


def config(vocab, width, layers, *, eps=1e-5, cap=None):
    c = dict(architecture="Siparax", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if cap is not None:
        c["logit_softcap"] = cap
    return c


ROT_A = rot(10000.0, 8, (4.0, 64, 8.0, 1.0))
ROT_B = rot(300.0, 16, (1.5, 40, 16.0, 2.0))
# both forms of the attention, a layer that reads rows of layer 0, tensor-core sizes, grouped delta heads
CFG_SHARED = config(97, 64, [layer("latent_attention_2", latent(4, 16, 8, 24, 24, 40, 0.3, ROT_A), 96),
                             layer("channel_delta", cdelta(4, 2, 32, 32, 4)),
                             layer("latent_attention", latent(2, 32, 16, 16, 48, 32, 0.2, ROT_B), 80),
                             layer("latent_attention_2", latent(3, 8, 8, 40, 24, 16, 0.5, ROT_A, kv_from=0), 48),
                             layer("channel_delta", cdelta(2, 2, 16, 48, 2), 64)], cap=9.0)
# odd sizes that only the general kernels take, no cap, no rescaling, fewer turned values than the rotated part has
CFG_ODD = config(61, 40, [layer("channel_delta", cdelta(3, 1, 12, 20, 3), 56),
                          layer("latent_attention", latent(3, 10, 6, 14, 20, 12, 0.4, rot(50.0, 4))),
                          layer("latent_attention_2", latent(1, 20, 10, 12, 18, 28, 0.3, rot(1000.0, 10, (2.0, 30, 4.0, 0.5))), 72),
                          layer("channel_delta", cdelta(1, 1, 24, 8, 1))], eps=1e-6)
# several layers reading one layer's rows, wide delta heads
CFG_WIDE = config(83, 96, [layer("latent_attention_2", latent(6, 16, 16, 16, 48, 64, 0.25, ROT_B), 128),
                           layer("latent_attention_2", latent(2, 32, 16, 48, 48, 24, 0.2, ROT_B, kv_from=0)),
                           layer("channel_delta", cdelta(2, 1, 64, 64, 2), 64),
                           layer("latent_attention_2", latent(4, 8, 16, 8, 48, 32, 0.35, ROT_B, kv_from=0), 64)], cap=30.0)

CONFIGS = {"shared": CFG_SHARED, "odd": CFG_ODD, "wide": CFG_WIDE}
RANKS = {"shared": (6, 10), "odd": (3, 5), "wide": (16, 4)}         # ranks of the decay's and the gate's low-rank projections


def make_tensors(cfg, seed, ranks=(6, 10), sharp=1.0):
    """name -> float32 array, drawn so that every mechanism matters: biases and norm weights away from 0 and 1, decays spread
    between fast and slow per channel, gates away from one half, scores of order one."""
    rng = np.random.default_rng(seed)
    W = cfg["width"]
    n = lambda *shape, std=1.0: (rng.standard_normal(shape) * std).astype(np.float32)
    t = {"embed": n(cfg["vocab"], W, std=0.7), "head": n(cfg["vocab"], W, std=1.5 * W ** -0.5)}

    def norm(name):
        t[name] = 1 + n(W, std=0.15)
        t[name + ".b"] = n(W, std=0.2)

    norm("embed.norm")
    norm("final.norm")
    ra, rg = ranks
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        norm(p + "norm1")
        if l["type"] == "channel_delta":
            qk, v = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            for name, rows in (("q", qk), ("k", qk), ("v", v)):
                t[p + f"mix.{name}"] = n(rows, W, std=2 * W ** -0.5)
                t[p + f"mix.{name}.conv"] = n(rows, m["conv"], std=0.6)
            t[p + "mix.b"] = n(m["heads"], W, std=2 * W ** -0.5)
            t[p + "mix.A_log"] = n(m["heads"], std=1.0) - 1.0
            t[p + "mix.a1"] = n(ra, W, std=W ** -0.5)
            t[p + "mix.a2"] = n(m["heads"] * m["dim"], ra, std=2 * ra ** -0.5)
            t[p + "mix.dt_bias"] = n(m["heads"] * m["dim"], std=1.0)
            t[p + "mix.g1"] = n(rg, W, std=W ** -0.5)
            t[p + "mix.g2"] = n(v, rg, std=2 * rg ** -0.5)
            t[p + "mix.norm"] = 1 + n(m["vdim"], std=0.1)
            t[p + "mix.o"] = n(W, v, std=v ** -0.5)
        else:
            H, qd = m["heads"], m["dim"] + m["rot_dim"]
            t[p + "mix.dq"] = n(m["q_rank"], W, std=W ** -0.5)
            t[p + "mix.dq.norm"] = 1 + n(m["q_rank"], std=0.1)
            t[p + "mix.uq"] = n(H * qd, m["q_rank"], std=sharp * 2.0 * m["q_rank"] ** -0.5)
            if "kv_from" not in m:
                t[p + "mix.dkv"] = n(m["kv_rank"] + m["rot_dim"], W, std=2.0 * W ** -0.5)
                t[p + "mix.dkv.norm"] = 1 + n(m["kv_rank"], std=0.1)
            t[p + "mix.uk"] = n(H * m["dim"], m["kv_rank"], std=sharp * 2.0 * m["kv_rank"] ** -0.5)
            t[p + "mix.uv"] = n(H * m["vdim"], m["kv_rank"], std=m["kv_rank"] ** -0.5)
            if l["type"] == "latent_attention_2":
                t[p + "mix.g"] = n(H, W, std=3 * W ** -0.5)
            t[p + "mix.o"] = n(W, H * m["vdim"], std=(H * m["vdim"]) ** -0.5)
        if l["mlp"] is not None:
            norm(p + "norm2")
            t[p + "mlp.gate"] = n(l["mlp"]["ff"], W, std=1.5 * W ** -0.5)
            t[p + "mlp.up"] = n(l["mlp"]["ff"], W, std=1.5 * W ** -0.5)
            t[p + "mlp.down"] = n(W, l["mlp"]["ff"], std=l["mlp"]["ff"] ** -0.5)
    return t


def write_model(model_dir, cfg, tensors, dtype=torch.bfloat16):
    """config.json and model.safetensors; tensors are stored in `dtype` (the values a bfloat16 checkpoint holds are what
    both the engine and the plain implementation then read)."""
    from vitna_anchor_b200.weights import write_model_folder
    os.makedirs(model_dir, exist_ok=True)
    write_model_folder(str(model_dir), cfg, {k: torch.from_numpy(v).to(dtype) for k, v in tensors.items()})
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return str(model_dir)


def make_model(model_dir, name, seed=0, **kw):
    return write_model(model_dir, CONFIGS[name], make_tensors(CONFIGS[name], seed, RANKS[name], **kw))
