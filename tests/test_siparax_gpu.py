"""Siparax through the engine against the plain implementation (tests/plain_siparax.py), on small models of the tests' own.

Every comparison is between the engine's step function (cache and state manager, kernels, CUDA graphs as in serving)
and plain_siparax.forward on whole sequences.  float32 is held to 3e-5 of the logits' scale; bfloat16 to what 8 bits of
mantissa cost on these sharp little models, and between ways of cutting the same request to less.
"""
import numpy as np
import pytest
import torch

import plain_siparax as PS
import replay_util as RU
import siparax_models as SM

pytestmark = pytest.mark.gpu

F32_TOL = 3e-5
BF16_TOL = 1e-1
BF16_CUT_TOL = 8e-2


def _runner(model_dir, dtype, *, tokens=1024, page=16, slots=4, graphs=True):
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner
    model = load_model(model_dir, dtype, "cuda")
    return ModelRunner(model, page_size=page, num_pages=-(-tokens // page), max_requests=slots, max_batch_tokens=tokens,
                       max_model_len=tokens, device="cuda", cuda_graphs=graphs)


def _play(runner, steps):
    """steps as replay_util makes them -> {(request, position): logits row}; requests are opened at their first entry
    and closed when a step ends them, as the replay program does."""
    from vitna_anchor_b200.engine.runner import StepEntry
    got, at = {}, {}
    for entries, end in steps:
        for rid, _, _ in entries:
            if not runner.cache.is_open(rid):
                runner.open(rid)
        logits = runner.step([StepEntry(rid, list(map(int, toks)), list(want)) for rid, toks, want in entries])
        host = None if logits is None else logits.cpu().numpy()
        runner.check(sync=True)
        r = 0
        for rid, toks, want in entries:
            base = at.get(rid, 0)
            for w in want:
                got[(rid, base + w)] = host[r].copy()
                r += 1
            at[rid] = base + len(toks)
        for rid in end:
            runner.close(rid)
            at.pop(rid, None)
        runner.cache.check()
    return got


def _plain(model_dir, ids):
    cfg, W = PS.read_model(model_dir)
    return PS.forward(cfg, W, ids)


def _worst(got, want_by_req, rms):
    """The worst row's difference between the engine and the plain logits.  float32 rows (rms False): the largest difference of
    one logit as a fraction of the request's largest logit.  bfloat16 rows differ by rounding noise in every logit, so there the
    measure is the root mean square of a row's differences over that of the request's logits."""
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = want_by_req[rid]
        if rms:
            worst = max(worst, float(np.sqrt(np.mean((row - ref[pos]) ** 2)) / np.sqrt(np.mean(ref ** 2))))
        else:
            worst = max(worst, float(np.abs(row - ref[pos]).max() / max(1.0, np.abs(ref).max())))
    return worst


def _ids(rng, vocab, n):
    return [int(t) for t in rng.integers(0, vocab, n)]


# ---------------------------------------------------------------------------------------------------------------
# each mechanism alone: models of one layer (two where a layer reads another layer's rows)
# ---------------------------------------------------------------------------------------------------------------

R1, R2 = SM.rot(10000.0, 8, (4.0, 16, 4.0, 0.5)), SM.rot(100.0, 16)
ALONE = {
    "latent_neighbours": SM.config(40, 32, [SM.layer("latent_attention", SM.latent(2, 16, 8, 8, 24, 16, 0.4, R1))]),
    "latent_halves_gated": SM.config(40, 32, [SM.layer("latent_attention_2", SM.latent(3, 8, 16, 24, 16, 20, 0.3, R2))]),
    "latent_part_turned": SM.config(40, 32, [SM.layer("latent_attention_2", SM.latent(2, 8, 16, 8, 16, 8, 0.3, SM.rot(30.0, 6)))]),
    "latent_tensor_core_sizes": SM.config(40, 64, [SM.layer("latent_attention_2", SM.latent(4, 16, 32, 16, 64, 32, 0.2, SM.rot(1000.0, 32, (2.0, 32, 8.0, 1.0))))]),
    "latent_odd": SM.config(40, 24, [SM.layer("latent_attention", SM.latent(1, 7, 2, 5, 9, 11, 0.5, SM.rot(20.0, 2, (2.0, 8, 2.0, 1.0))))]),
    "latent_shared_rows": SM.config(40, 32, [SM.layer("latent_attention_2", SM.latent(2, 8, 8, 8, 24, 16, 0.4, R1)),
                                             SM.layer("latent_attention_2", SM.latent(4, 16, 8, 4, 24, 8, 0.2, R1, kv_from=0))]),
    "delta": SM.config(40, 32, [SM.layer("channel_delta", SM.cdelta(2, 1, 16, 8, 3))]),
    "delta_no_conv": SM.config(40, 32, [SM.layer("channel_delta", SM.cdelta(2, 2, 32, 32, 1))]),
    "delta_odd": SM.config(40, 24, [SM.layer("channel_delta", SM.cdelta(3, 3, 10, 7, 2))]),
    "feed_forward": SM.config(40, 32, [SM.layer("channel_delta", SM.cdelta(1, 1, 8, 8, 2), 72)]),
    "cap": SM.config(40, 32, [SM.layer("channel_delta", SM.cdelta(1, 1, 8, 8, 2), 24)], cap=2.0),
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = ALONE[name]
    d = SM.write_model(tmp_path / name, cfg, SM.make_tensors(cfg, 5, ranks=(3, 7)))
    ids = _ids(np.random.default_rng(1), cfg["vocab"], 70)
    ref = _plain(d, ids)
    if name == "cap":
        assert np.abs(ref).max() > 1.5          # the cap bends these logits
    runner = _runner(d, dtype, tokens=128, page=8)
    whole = _play(runner, RU.whole("a", ids))
    one = _play(runner, RU.tail_one_by_one("b", ids, tail=69))        # the first token, then every token alone
    tol, rms = (F32_TOL, False) if dtype == "float32" else (BF16_TOL, True)
    assert _worst(whole, {"a": ref}, rms) < tol
    assert _worst(one, {"b": ref}, rms) < tol


# ---------------------------------------------------------------------------------------------------------------
# whole models: prompts, token by token, portions, mixed batches, pages and slots used again
# ---------------------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("siparax")
    out = {}
    for i, name in enumerate(sorted(SM.CONFIGS)):
        d = SM.make_model(root / name, name, seed=10 + i)
        rng = np.random.default_rng(100 + i)
        reqs = {f"r{k}": _ids(rng, SM.CONFIGS[name]["vocab"], n) for k, n in enumerate((150, 1, 37, 64, 91, 17))}
        out[name] = (d, reqs, {r: _plain(d, ids) for r, ids in reqs.items()})
    return out


@pytest.mark.parametrize("name", sorted(SM.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_decoding_portions_and_mixed_batches(models, name, dtype):
    d, reqs, ref = models[name]
    tol, rms = (F32_TOL, False) if dtype == "float32" else (BF16_TOL, True)
    cut_tol = 1e-5 if dtype == "float32" else BF16_CUT_TOL
    runner = _runner(d, dtype, tokens=384, page=8, slots=4)
    whole = {}
    for r, ids in reqs.items():
        whole.update(_play(runner, RU.whole(r, ids)))
    assert _worst(whole, ref, rms) < tol
    runs = {}
    runs["decode"] = {k: v for r, ids in reqs.items() for k, v in _play(runner, RU.tail_one_by_one(r, ids, tail=40)).items()}
    # portions of changing sizes down to two tokens, cut inside pages and inside the recurrence's groups of tokens
    runs["portions"] = {k: v for r, ids in reqs.items()
                        for k, v in _play(runner, RU.changing_portions(r, ids, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 8, 11))).items()}
    # up to four requests live, portions of some beside single tokens of others; six requests through four slots and a
    # pool that holds fewer positions than the requests have in all
    rng = np.random.default_rng(3)
    runs["mixed"] = _play(runner, RU.mixed(reqs, {r: max(1, len(ids) - 20) for r, ids in reqs.items()}, rng, live_max=4))
    rng = np.random.default_rng(4)
    runs["beside"] = _play(runner, RU.mixed(reqs, {r: len(ids) // 2 for r, ids in reqs.items()}, rng, live_max=3, portions=(2, 40),
                                           one_prompt_at_a_time=True))
    for how, got in runs.items():
        assert len(got) == sum(len(i) for i in reqs.values()), how
        assert _worst(got, ref, rms) < tol, how
        cut = _worst(got, {r: np.stack([whole[(r, p)] for p in range(len(ids))]) for r, ids in reqs.items()}, rms)
        assert cut < cut_tol, (how, cut)
    runner.cache.check()
    assert all(f == p.num_pages for f, p in zip(runner.cache.free_pages(), runner.cache.tables.pools))     # every page came back


def test_a_request_alone_and_beside_others_on_other_pages_and_slots(models):
    """The same request first alone in a fresh engine, then as the fourth of four whose neighbours took the low pages and slots."""
    d, reqs, ref = models["shared"]
    ids = reqs["r4"]
    alone = _play(_runner(d, "float32", tokens=512, page=8), RU.changing_portions("x", ids))
    runner = _runner(d, "float32", tokens=512, page=8)
    steps = [([("n0", reqs["r0"][:50], []), ("n1", reqs["r2"], []), ("n2", reqs["r3"][:9], [])], ["n1"])]      # n1's slot and pages come back
    steps += [([("n0", reqs["r0"][50:52], []), ("x", ids[:30], range(30)), ("n2", reqs["r3"][9:10], [])], [])]
    steps += [([("x", ids[30:31], [0]), ("n3", reqs["r5"], []), ("n0", reqs["r0"][52:53], [])], ["n3"])]
    steps += [([("x", ids[31:], range(len(ids) - 31)), ("n2", reqs["r3"][10:11], [])], ["x", "n0", "n2"])]
    beside = _play(runner, steps)
    for k, row in alone.items():
        assert np.abs(beside[k] - row).max() / np.abs(ref["r4"]).max() < 1e-5


def test_long_decoding(tmp_path):
    """300 tokens one by one after a short prompt: the recurrent state is carried 300 times, the convolution's memory moves 300
    times, the rotation passes hundreds of positions."""
    cfg = SM.CONFIGS["shared"]
    d = SM.make_model(tmp_path / "m", "shared", seed=77)
    ids = _ids(np.random.default_rng(8), cfg["vocab"], 310)
    ref = _plain(d, ids)
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        got = _play(_runner(d, dtype, tokens=320, page=16), RU.tail_one_by_one("a", ids, tail=300))
        assert _worst(got, {"a": ref}, dtype == "bfloat16") < tol


# ---------------------------------------------------------------------------------------------------------------
# one key that must be found: far back, at the first position, on either side of a page's border
# ---------------------------------------------------------------------------------------------------------------

def _needle_model(tmp_path, width=32, vocab=700):
    """One latent attention layer, one head, whose query and key are the normed input itself: both latents are the identity
    (ranks = width), the expansions too, nothing is rotated (the rotated parts are zero).  A token that comes twice scores
    width * scale against its first coming and about sqrt(width) * scale against all others, so the last token's output is the
    value of ONE far row of the cache.  A wrong page, slot or offset returns another token's value."""
    cfg = SM.config(vocab, width, [SM.layer("latent_attention", SM.latent(1, width, 4, width, width, width, 1.0, SM.rot(100.0, 4)))])
    t = SM.make_tensors(cfg, 3)
    eye = np.eye(width, dtype=np.float32)
    for name in ("embed.norm", "l0.norm1"):
        t[name][:] = 1.0
        t[name + ".b"][:] = 0.0
    t["l0.mix.dq"], t["l0.mix.dq.norm"][:] = eye.copy(), 1.0
    t["l0.mix.dkv"] = np.concatenate([eye, np.zeros((4, width), np.float32)])
    t["l0.mix.dkv.norm"][:] = 1.0
    t["l0.mix.uq"] = np.concatenate([eye, np.zeros((4, width), np.float32)])
    t["l0.mix.uk"] = eye.copy()
    t["l0.mix.uv"] *= 4.0
    return SM.write_model(tmp_path / "needle", cfg, t, dtype=torch.float32), cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_is_found_wherever_it_lies(tmp_path, dtype):
    d, cfg = _needle_model(tmp_path)
    rng = np.random.default_rng(0)
    n, page = 600, 16
    base = [int(t) for t in rng.permutation(cfg["vocab"])[:n]]            # all different
    c, W = PS.read_model(d)
    runner = _runner(d, dtype, tokens=640, page=page)
    for place in (0, 1, 3, page - 1, page, page + 1, 255, 256, 257, n - 3):
        ids = base[:n - 1] + [base[place]]                               # the last token repeats the one at `place`
        ref = PS.forward(c, W, ids)
        # the test is sharp: in the plain implementation the far key has nearly all of the last token's weight
        x = PS.layer_norm(W["embed"][np.asarray(ids)], 1.0, 0.0, c["norm"]["eps"])
        h = PS.rms(PS.layer_norm(x, 1.0, 0.0, c["norm"]["eps"]), c["norm"]["eps"])
        s = h @ h[-1]
        e = np.exp(s - s.max())
        assert e[place] / e.sum() > 0.45 and e[place] / e.sum() + e[-1] / e.sum() > 0.95
        tol = F32_TOL if dtype == "float32" else BF16_TOL
        for how, steps in (("prompt", RU.whole("a", ids)), ("decoded", RU.tail_one_by_one("a", ids, tail=2)),
                           ("portions", RU.changing_portions("a", ids, sizes=(250, 5, 2, 100)))):
            got = _play(runner, [(e_, end) for e_, end in steps])
            last = {k: v for k, v in got.items() if k[1] == n - 1}
            assert _worst(last, {"a": ref}, dtype == "bfloat16") < tol, (place, how)


def test_the_rotation_alone_decides_at_every_distance(tmp_path):
    """A model whose scores come from the rotated parts alone (the plain query part is zero): a position
    that is off by one, a wrong pairing or a frequency that is not rescaled changes every softmax weight."""
    cfg = SM.config(30, 32, [SM.layer("latent_attention_2", SM.latent(2, 8, 16, 8, 16, 8, 0.25, SM.rot(40.0, 16, (3.0, 24, 6.0, 1.0))))])
    t = SM.make_tensors(cfg, 9)
    uq = t["l0.mix.uq"].reshape(2, 24, 8)
    uq[:, :8] = 0.0
    d = SM.write_model(tmp_path / "rot", cfg, t)
    ids = _ids(np.random.default_rng(2), 30, 300)
    ref = _plain(d, ids)
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        runner = _runner(d, dtype, tokens=320, page=16)
        assert _worst(_play(runner, RU.whole("a", ids)), {"a": ref}, dtype == "bfloat16") < tol
        assert _worst(_play(runner, RU.tail_one_by_one("a", ids, tail=120)), {"a": ref}, dtype == "bfloat16") < tol


# ---------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("width", [24, 200, 1030])
def test_layer_norm_rows(width):
    from vitna_anchor_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(37, width, generator=g, device="cuda") * 3 + 1.5
    w, b = 1 + 0.2 * torch.randn(width, generator=g, device="cuda"), torch.randn(width, generator=g, device="cuda")
    want = PS.layer_norm(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy(), 1e-5)
    out = ops.layernorm_rows(x, w, b, 1e-5, torch.empty(37, width, device="cuda"))
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device="cuda")
    picked = ops.layernorm_rows(x, w, b, 1e-5, torch.empty(4, width, dtype=torch.bfloat16, device="cuda"), rows)
    assert np.abs(picked.float().cpu().numpy() - want[[5, 0, 36, 5]]).max() < 3e-2
    same = x.clone()
    ops.layernorm_rows(same, w, b, 1e-5, same)                          # where the rows lie
    assert torch.equal(same, out)


def test_soft_cap_and_the_gated_activations():
    from vitna_anchor_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(2)
    z = torch.randn(7, 50, generator=g, device="cuda") * 20
    want = 9.0 * np.tanh(z.double().cpu().numpy() / 9.0)
    assert np.abs(ops.softcap(z.clone(), 9.0).cpu().numpy() - want).max() < 1e-5
    gu = torch.randn(11, 2 * 36, generator=g, device="cuda") * 2
    a = gu.double().cpu().numpy()
    for kind, f in (("gelu_tanh", PS.gelu_tanh), ("silu", PS.silu)):
        want = f(a[:, :36]) * a[:, 36:]
        assert np.abs(ops.act_mul(gu, torch.empty(11, 36, device="cuda"), kind).cpu().numpy() - want).max() < 1e-5
        got = ops.act_mul(gu.bfloat16(), torch.empty(11, 36, dtype=torch.bfloat16, device="cuda"), kind).float().cpu().numpy()
        a16 = gu.bfloat16().double().cpu().numpy()
        want16 = f(a16[:, :36]) * a16[:, 36:]
        assert (np.abs(got - want16) <= 5e-3 * (1 + np.abs(want16))).all()         # one rounding to bfloat16


@pytest.mark.parametrize("interleaved", [True, False])
def test_latent_prepare_and_the_query_rotation(interleaved):
    """Both norms, the rotation at scattered positions (up to 100,000) and the cache write at scattered slots, against NumPy."""
    from vitna_anchor_b200 import ops
    rng = np.random.default_rng(6)
    T, qr, r, rd, dims, H, ps, pages = 9, 12, 20, 10, 6, 3, 4, 7
    N = qr + r + rd + H
    pairing = "interleaved" if interleaved else "half"
    rot = SM.rot(1000.0, dims, (2.0, 30, 4.0, 0.5))
    freq, mag = PS.rotation_frequencies(rot)
    proj = rng.standard_normal((T, N))
    qw, kw = 1 + 0.1 * rng.standard_normal(qr), 1 + 0.1 * rng.standard_normal(r)
    pos = np.array([0, 1, 2, 17, 300, 4095, 65536, 99999, 5])
    slots = np.array([3, 27, 0, 9, -1, 14, 1, 20, 26])
    f = lambda a, dt=torch.float32: torch.tensor(np.asarray(a), dtype=dt, device="cuda")
    cache = torch.zeros(pages, ps * (r + rd), device="cuda")
    cq = ops.latent_prepare(f(proj), qr, f(qw), torch.empty(T, qr, device="cuda"), 1e-5, f(pos, torch.int32), f(freq), mag, dims, interleaved,
                            kv_off=qr, kv_rank=r, rot_dim=rd, kv_norm_w=f(kw), slot_mapping=f(slots, torch.int32), cache_layer=cache, page_size=ps)
    assert np.abs(cq.cpu().numpy() - PS.rms(proj[:, :qr], 1e-5, qw)).max() < 1e-5
    c = PS.rms(proj[:, qr:qr + r], 1e-5, kw)
    host = cache.cpu().numpy()
    for t in range(T):
        if slots[t] < 0:
            continue
        kr = PS.rotate(proj[t:t + 1, qr + r:qr + r + rd], int(pos[t]), rot, pairing)[0]
        page, off = host[slots[t] // ps], slots[t] % ps
        krow = page[off * (r + rd):(off + 1) * (r + rd)]
        assert np.abs(krow[:r] - c[t]).max() < 1e-5
        assert np.abs(krow[r:] - kr).max() < 2e-2 * (1 + pos[t] * 1e-5)      # float32 angles: the error grows with the position
        if pos[t] < 5000:
            assert np.abs(krow[r:] - kr).max() < 5e-4
    untouched = np.ones(pages * ps, bool)
    untouched[slots[slots >= 0]] = False
    keys = host.reshape(pages * ps, r + rd)
    assert not keys[untouched].any()
    q = rng.standard_normal((T, H * (r + rd)))
    got = ops.latent_rotate_q(f(q), f(pos, torch.int32), f(freq), mag, H, r, rd, dims, interleaved).cpu().numpy().reshape(T, H, r + rd)
    want = q.reshape(T, H, r + rd).copy()
    for t in range(T):
        want[t, :, r:] = PS.rotate(want[t:t + 1, :, r:], int(pos[t]), rot, pairing)[0]
    small = pos < 5000
    assert np.abs(got[small] - want[small]).max() < 5e-4 and np.array_equal(got[:, :, :r], want[:, :, :r].astype(np.float32))
    gated = ops.head_gate(f(q[:, :H * r]), f(proj), qr + r + rd, H).cpu().numpy().reshape(T, H, r)
    assert np.abs(gated - q[:, :H * r].reshape(T, H, r) * PS.sigmoid(proj[:, qr + r + rd:])[:, :, None]).max() < 1e-5


@pytest.mark.parametrize("chunked", [False, True])
def test_the_channel_delta_kernels_against_the_recurrence_written_out(chunked):
    """Segments of unequal length on scattered slots, a second step that continues from the state of the first, a padding segment;
    key sizes from 10 to 256, sizes that are no multiples of four, and decays that differ widely between the channels of a head."""
    from vitna_anchor_b200 import ops
    rng = np.random.default_rng(5)
    sizes = ((1, 2, 16, 8, 3, 3, 5), (2, 2, 64, 128, 4, 8, 8), (1, 3, 40, 24, 1, 2, 9), (2, 4, 128, 64, 2, 16, 4), (1, 2, 10, 12, 2, 4, 4),
             (1, 1, 256, 32, 2, 5, 3), (3, 3, 7, 5, 2, 2, 2), (3, 9, 64, 64, 4, 16, 16))
    for (G, H, dk, dv, taps, ra, rg) in sizes:
        if chunked and not ops.delta_chunked_takes(G, H, dk, dv, taps):
            continue
        C = 2 * G * dk + H * dv
        N = C + H + ra + rg
        lens1, lens2, slots = ([70, 1, 128, 0], [1, 97, 64, 0], [3, 0, 2, -1]) if chunked else ([70, 1, 19, 0], [1, 97, 2, 0], [3, 0, 2, -1])
        conv = rng.standard_normal((C, taps)) * 0.6
        a_log, dt_bias, nw = rng.standard_normal(H) - 1, rng.standard_normal(H * dk) * 2, 1 + 0.1 * rng.standard_normal(dv)
        a2, g2 = rng.standard_normal((H * dk, ra)) * 2, rng.standard_normal((H * dv, rg))
        proj_all = [rng.standard_normal((l1 + l2, N)) for l1, l2 in zip(lens1[:3], lens2[:3])]
        state = torch.zeros(4, ops.delta_state_floats(G, H, dk, dv, taps), device="cuda")
        f = lambda a: torch.tensor(np.asarray(a), dtype=torch.float32, device="cuda")
        outs = [[] for _ in proj_all]
        for step, lens in enumerate((lens1, lens2)):
            T = sum(lens)
            rows = np.concatenate([p[(0 if step == 0 else lens1[i]):(lens1[i] if step == 0 else None)] for i, p in enumerate(proj_all)])
            seg_starts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
            token_seg = torch.tensor(np.repeat(np.arange(len(lens)), lens), dtype=torch.int32, device="cuda")
            out = torch.empty(T, H * dv, device="cuda")
            ops.channel_delta_rule(f(rows), f(conv), f(a_log), f(dt_bias), f(a2.T.copy()), f(g2.T.copy()), f(nw), 1e-5, token_seg, seg_starts,
                                   torch.tensor(slots, dtype=torch.int32, device="cuda"), state,
                                   torch.empty(T, ops.channel_delta_prep_width(G, H, dk, dv), device="cuda"),
                                   torch.empty(ops.channel_delta_group_floats(T, H, dk), device="cuda"), torch.empty(T, H * dv, device="cuda"),
                                   out, G, H, dk, dv, taps,
                                   chunk_scratch=torch.empty(ops.channel_delta_chunked_scratch_floats(T, len(lens), H, dk, dv), device="cuda") if chunked else None)
            o = out.cpu().numpy()
            at = 0
            for i, n in enumerate(lens[:3]):
                outs[i].append(o[at:at + n])
                at += n
        for i, p in enumerate(proj_all):                                  # the recurrence written out, whole sequence at once
            q = PS.silu(PS.short_conv(p[:, :G * dk], conv[:G * dk])).reshape(-1, G, dk)
            k = PS.silu(PS.short_conv(p[:, G * dk:2 * G * dk], conv[G * dk:2 * G * dk])).reshape(-1, G, dk)
            v = PS.silu(PS.short_conv(p[:, 2 * G * dk:C], conv[2 * G * dk:])).reshape(-1, H, dv)
            q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
            k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
            beta = PS.sigmoid(p[:, C:C + H])
            decay = np.exp(-np.exp(a_log)[None, :, None] * PS.softplus(p[:, C + H:C + H + ra] @ a2.T + dt_bias).reshape(-1, H, dk))
            gate = PS.sigmoid(p[:, C + H + ra:] @ g2.T).reshape(-1, H, dv)
            assert decay.min() < 0.3 and decay.max() > 0.9             # the channels of a head decay at widely different rates
            want = np.zeros((len(p), H, dv))
            for h in range(H):
                S = np.zeros((dk, dv))
                for t in range(len(p)):
                    S = decay[t, h][:, None] * S
                    S = S + np.outer(k[t, h // (H // G)], beta[t, h] * (v[t, h] - S.T @ k[t, h // (H // G)]))
                    want[t, h] = S.T @ q[t, h // (H // G)]
            want = (PS.rms(want, 1e-5, nw) * gate).reshape(len(p), H * dv)
            assert np.abs(np.concatenate(outs[i]) - want).max() < 2e-5 * max(1.0, np.abs(want).max()), (G, H, dk, dv, taps, i)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_values_inside_the_keys_give_what_values_beside_them_give(dtype):
    """The three attention kernels on a cache of keys alone whose first vd values are the values, against the same kernels on a
    cache that holds those values once more beside the keys: a prompt's portion far into its context and two decoded tokens."""
    from vitna_anchor_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    nh, hd, vd, ps, pages, scale = 4, 96, 64, 8, 40, 0.11
    keys = (torch.randn(pages, ps, hd, generator=g, device="cuda") * 1.5).to(dtype)
    inside = keys.reshape(pages, ps * hd).contiguous()
    beside = torch.cat([keys.reshape(pages, ps * hd), keys[..., :vd].reshape(pages, ps * vd)], dim=1).contiguous()
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    bt = torch.stack([perm[:20], perm[20:]]).contiguous().cuda()                  # two requests, 20 pages each
    pos = list(range(100, 130)) + [159, 77]                                       # a portion of 30 tokens, then two single tokens
    seg = [0] * 30 + [1, 0]
    T = len(pos)
    q = (torch.randn(T, nh * hd, generator=g, device="cuda")).to(dtype)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    positions, token_seg = i32(pos), i32(seg)
    outs = {}
    for name, cache, flag in (("inside", inside, True), ("beside", beside, False)):
        rows = ops.attention_rows_biased(q, cache, bt, token_seg, positions, torch.zeros(T, nh * vd, dtype=dtype, device="cuda"), nh, 1, hd, vd, ps,
                                         scale, v_in_key=flag)
        dec = torch.zeros(T, nh * vd, dtype=dtype, device="cuda")
        scratch = torch.zeros(ops.attention_decode_scratch_bytes(4, nh, 1, hd, 512), dtype=torch.uint8, device="cuda")
        ops.attention_decode_biased(q, cache, bt, token_seg, positions, dec, scratch, 4, nh, 1, hd, vd, ps, scale, 512, 160, tok_list=i32([30, 31]),
                                    v_in_key=flag)
        outs[name] = [rows, dec[30:]]
        if dtype == torch.bfloat16:
            pre = torch.zeros(T, nh * vd, dtype=dtype, device="cuda")
            ops.attention_prefill_biased(q, cache, bt, i32([[0, 30, 100, 0]]), pre, nh, 1, hd, vd, ps, scale, v_in_key=flag)
            outs[name].append(pre[:30])
    ops.check_device_errors()
    for a, b in zip(outs["inside"], outs["beside"]):
        assert torch.equal(a, b)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (outs["inside"][1].float() - outs["inside"][0][30:].float()).abs().max() < tol
    if dtype == torch.bfloat16:
        assert (outs["inside"][2].float() - outs["inside"][0][:30].float()).abs().max() < tol


def test_the_one_kernel_channel_delta_rule_for_single_tokens_gives_what_the_other_kernels_give():
    from vitna_anchor_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(4)
    r = lambda *s: torch.randn(*s, generator=g, device="cuda")
    for (G, H, dk, dv, taps, ra, rg) in ((1, 2, 16, 8, 3, 3, 5), (3, 9, 64, 64, 4, 16, 16), (4, 16, 128, 128, 4, 8, 24), (1, 3, 40, 7, 1, 2, 2),
                                         (2, 2, 256, 32, 2, 4, 4), (1, 1, 8, 300, 2, 5, 1)):
        assert ops.channel_delta_decode_takes(G, H, dk, dv, taps, ra, rg)
        C, S = 2 * G * dk + H * dv, 5
        N = C + H + ra + rg
        conv, a_log, dt, nw = r(C, taps) * 0.6, r(H) - 1, r(H * dk) * 2, 1 + 0.1 * r(dv)
        a2t, g2t = r(ra, H * dk) * 2, r(rg, H * dv)
        slots = torch.tensor([3, -1, 0, 6, 2], dtype=torch.int32, device="cuda")         # one padding segment
        seg_starts = torch.arange(S + 1, dtype=torch.int32, device="cuda")
        token_seg = torch.arange(S, dtype=torch.int32, device="cuda")
        states = [r(8, ops.delta_state_floats(G, H, dk, dv, taps)) * 0.3 for _ in range(2)]
        states[1].copy_(states[0])
        for step in range(3):                                # the state and the convolution's memory are carried
            proj = r(S, N)
            outs = []
            for single in (False, True):
                out = torch.zeros(S, H * dv, device="cuda")
                ops.channel_delta_rule(proj, conv, a_log, dt, a2t, g2t, nw, 1e-5, token_seg, seg_starts, slots, states[single],
                                       torch.empty(S, ops.channel_delta_prep_width(G, H, dk, dv), device="cuda"),
                                       torch.empty(ops.channel_delta_group_floats(S, H, dk), device="cuda"), torch.zeros(S, H * dv, device="cuda"),
                                       out, G, H, dk, dv, taps, single_tokens=single)
                outs.append(out)
            live = slots >= 0
            assert torch.allclose(outs[0][live], outs[1][live], rtol=1e-4, atol=1e-5), (G, H, dk, dv, taps, step)
            assert torch.allclose(states[0], states[1], rtol=1e-4, atol=1e-5)


# ---------------------------------------------------------------------------------------------------------------
# the engine's own entry point and scheduler, the command line, the replay program
# ---------------------------------------------------------------------------------------------------------------

def _plain_greedy(model_dir, ids, n):
    cfg, W = PS.read_model(model_dir)
    ids = list(ids)
    for _ in range(n):
        ids.append(int(np.argmax(PS.forward(cfg, W, ids)[-1])))
    return ids[-n:]


def test_greedy_generation_through_the_engine_and_its_scheduler(models):
    from vitna_anchor_b200.engine.engine import Engine
    d, reqs, _ = models["wide"]
    eng = Engine(d, dtype="float32", ctx=256, parallel=3, kv_block=8, max_batch_tokens=64, max_prompt_portion=24)
    prompts = [reqs["r2"], reqs["r5"], reqs["r1"], reqs["r3"][:30]]       # four requests through three slots
    handles = [eng.add_request(p, max_new=12) for p in prompts]
    while eng.scheduler.has_work():
        eng.step()
    eng.flush()
    for h, p in zip(handles, prompts):
        assert list(h.output) == _plain_greedy(d, p, 12)
    assert eng.generate(prompts[0], max_new=12) == _plain_greedy(d, prompts[0], 12)


def test_the_replay_program_and_the_command_line(models, tmp_path):
    import json
    import os
    import subprocess
    import sys
    d, reqs, ref = models["odd"]
    rp = RU.Replay(d, "float32", tmp_path / "out", max_tokens=256, kv_block=8)
    got = rp.run(RU.changing_portions("a", reqs["r4"]) + RU.tail_one_by_one("b", reqs["r2"], tail=10), SM.CONFIGS["odd"]["vocab"])
    rp.close()
    assert _worst(got, {"a": ref["r4"], "b": ref["r2"]}, False) < F32_TOL
    out = subprocess.run([sys.executable, os.path.join(RU.ROOT, "bin", "vitna-anchor"), "generate", "--model", d, "--ids",
                          ",".join(map(str, reqs["r5"])), "--max-new", "8", "--greedy", "--dtype", "float32"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert _plain_greedy(d, reqs["r5"], 8) == [int(t) for t in json.loads(out.stdout.strip().splitlines()[-1])["ids"]]
