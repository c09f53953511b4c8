"""Siparax on the CPU: the configuration reader, the manifest, the rotation's frequencies and the folding of the latent
attention's matrices, each against the plain statement."""
import copy

import numpy as np
import pytest
import torch

import plain_siparax as PS
import siparax_models as SM
from vitna_anchor_b200.config import ConfigError, resolve
from vitna_anchor_b200.config.siparax import SiparaxConfig
from vitna_anchor_b200.models.siparax import siparax_manifest
from vitna_anchor_b200.parts.rotary import blended_frequencies


@pytest.mark.parametrize("name", sorted(SM.CONFIGS))
def test_a_configuration_reads_and_writes_back(name):
    cfg = SiparaxConfig.from_dict(SM.CONFIGS[name])
    assert SiparaxConfig.from_dict(cfg.to_dict()) == cfg
    assert resolve(SM.CONFIGS[name]).name == "Siparax"
    names = {w.name for w in siparax_manifest(cfg)}
    assert names == set(SM.make_tensors(SM.CONFIGS[name], 0, SM.RANKS[name]))


def test_what_the_reader_does_not_know_is_refused():
    base = SM.CONFIGS["shared"]
    for change in (lambda c: c["layers"][0]["mixer"].update(window=8), lambda c: c["layers"][1]["mixer"].update(gate="x"),
                   lambda c: c["layers"][0].update(type="attention"), lambda c: c["layers"][3]["mixer"].update(kv_from=2),
                   lambda c: c["layers"][3]["mixer"].update(kv_rank=32), lambda c: c["layers"][3]["mixer"].update(kv_from=3),
                   lambda c: c["layers"][2]["mixer"].update(kv_from=0),          # the first form has no such key
                   lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10),
                   lambda c: c["layers"][4]["mlp"].update(kind="experts"), lambda c: c.update(logit_softcap=0.0),
                   lambda c: c["norm"].update(kind="rms")):
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError):
            SiparaxConfig.from_dict(c)


@pytest.mark.parametrize("r", [SM.ROT_A, SM.ROT_B, SM.rot(50.0, 4), SM.rot(1000000.0, 64, (16.0, 4096, 24.0, 2.0)), SM.rot(10000.0, 2, (3.0, 16, 1.0, 1.0))])
def test_the_rotation_frequencies(r):
    sc = r.get("scaling")
    f, mag = blended_frequencies(r["base"], r["dims"], None if sc is None else (sc["factor"], sc["original"], sc["fast"], sc["slow"]))
    pf, pmag = PS.rotation_frequencies(r)
    assert f.dtype == np.float32 and np.allclose(f, pf, rtol=1e-7, atol=0) and abs(mag - pmag) < 1e-12


@pytest.mark.parametrize("gated,shared", [(False, False), (True, False), (True, True)])
def test_the_folded_matrices_give_the_scores_and_outputs_of_the_unfolded_ones(gated, shared):
    """The part's folded query matrix against cached rows [c | kr], and its folded output matrix on weighted sums of c, equal
    the plain per-head keys, values and output projection."""
    from vitna_anchor_b200.parts.latent import LatentAttention
    rng = np.random.default_rng(3)
    W, H, dim, rd, vd, r, qr, T = 24, 3, 10, 6, 14, 16, 12, 9
    n = lambda *s: torch.from_numpy(rng.standard_normal(s))
    w = dict(w_dq=n(qr, W), q_norm=n(qr), w_uq=n(H * (dim + rd), qr), w_dkv=None if shared else n(r + rd, W),
             kv_norm=None if shared else n(r), w_uk=n(H * dim, r), w_uv=n(H * vd, r), w_o=n(W, H * vd), w_gate=n(H, W) if gated else None)
    part = LatentAttention.from_matrices(hidden=W, num_heads=H, dim=dim, rot_dim=rd, v_dim=vd, kv_rank=r, q_rank=qr, scale=0.3, eps=1e-5,
                                         freq=np.ones(rd // 2, np.float32), mag=1.0, rot_dims=rd, interleaved=True, dtype=torch.float64,
                                         device="cpu", **w)
    assert part.w_in.shape[0] == qr + (0 if shared else r + rd) + (H if gated else 0)
    assert part.kv_off == (-1 if shared else qr) and part.gate_off == (part.w_in.shape[0] - H if gated else -1)
    cq, c, kr = n(T, qr), n(T, r), n(T, rd)
    q = (cq @ w["w_uq"].T).reshape(T, H, dim + rd)
    k = (c @ w["w_uk"].T).reshape(T, H, dim)
    plain_scores = torch.einsum("thd,jhd->thj", q[..., :dim], k) + torch.einsum("thd,jd->thj", q[..., dim:], kr)
    folded_q = (cq @ part.w_q.T).reshape(T, H, r + rd)
    assert torch.allclose(torch.einsum("thd,jd->thj", folded_q, torch.cat([c, kr], 1)), plain_scores, rtol=1e-10, atol=1e-10)
    p = torch.softmax(plain_scores, -1)
    v = (c @ w["w_uv"].T).reshape(T, H, vd)
    plain_out = torch.einsum("thj,jhd->thd", p, v).reshape(T, H * vd) @ w["w_o"].T
    assert torch.allclose(torch.einsum("thj,jr->thr", p, c).reshape(T, H * r) @ part.w_out.T, plain_out, rtol=1e-10, atol=1e-10)
