"""Lupanex through the engine against the plain implementation (tests/plain_lupanex.py), on small models of the tests' own.

Every comparison is between the engine's step function (cache and state manager, kernels, CUDA graphs as in serving)
and plain_lupanex.forward on whole sequences.  float32 is held to 3e-5 of the logits' scale; bfloat16 to what 8 bits of
mantissa cost on these sharp little models, and between ways of cutting the same request to much less.
"""
import numpy as np
import pytest
import torch

import lupanex_models as LM
import plain_lupanex as PL
import replay_util as RU

pytestmark = pytest.mark.gpu

F32_TOL = 3e-5
BF16_TOL = 1e-1
BF16_CUT_TOL = 8e-2


def _runner(model_dir, dtype, *, tokens=1024, page=16, slots=4, graphs=True):
    from vitna_anchor_b200.engine.loading import load_model
    from vitna_anchor_b200.engine.runner import ModelRunner
    model = load_model(model_dir, dtype, "cuda")
    return ModelRunner(model, page_size=page, num_pages=-(-tokens // page), max_requests=slots, max_batch_tokens=tokens,
                       max_model_len=model.max_positions, device="cuda", cuda_graphs=graphs)


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
    cfg, W = PL.read_model(model_dir)
    return PL.forward(cfg, W, ids)


def _worst(got, want_by_req):
    """The worst row's difference between the engine and the plain logits.  float32 rows: the largest difference of one logit
    as a fraction of the request's largest logit.  bfloat16 rows differ by rounding noise in every logit, so there the measure is
    the root mean square of a row's differences over that of the request's logits."""
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = want_by_req[rid]
        if _worst.rms:
            worst = max(worst, float(np.sqrt(np.mean((row - ref[pos]) ** 2)) / np.sqrt(np.mean(ref ** 2))))
        else:
            worst = max(worst, float(np.abs(row - ref[pos]).max() / max(1.0, np.abs(ref).max())))
    return worst


_worst.rms = False


@pytest.fixture(autouse=True)
def _measure(request):
    """Tests parametrised by dtype measure bfloat16 rows by their root mean square."""
    callspec = getattr(request.node, "callspec", None)
    _worst.rms = bool(callspec and callspec.params.get("dtype") == "bfloat16")
    yield
    _worst.rms = False


def _ids(rng, vocab, n):
    return [int(t) for t in rng.integers(0, vocab, n)]


# ---------------------------------------------------------------------------------------------------------------
# each mechanism alone: models of one layer
# ---------------------------------------------------------------------------------------------------------------

ALONE = {
    "attention_plain": LM.config(40, 32, [LM.layer("attention", LM.att(2, 1, 16, 8, 0.4))]),
    "attention_bias": LM.config(40, 32, [LM.layer("attention", LM.att(2, 2, 32, 32, 0.3, bias_max=20))]),
    "attention_qtemp": LM.config(40, 32, [LM.layer("attention", LM.att(4, 2, 32, 64, 0.3, q_temp=(0.7, 3)))]),
    "delta": LM.config(40, 32, [LM.layer("delta", LM.delta(2, 1, 16, 8, 3))]),
    "delta_no_conv": LM.config(40, 32, [LM.layer("delta", LM.delta(2, 2, 32, 32, 1))]),
    "feed_forward": LM.config(40, 32, [LM.layer("attention", LM.att(1, 1, 8, 8, 0.3), 72)]),
    "hyper": LM.config(40, 32, [LM.layer("attention", LM.att(1, 1, 8, 8, 0.3), 24)] * 2, streams=3),
    "loop": LM.config(40, 64, [LM.layer("delta", LM.delta(2, 1, 16, 16, 2), 48)], loop=(0, 1, 3)),
}


@pytest.mark.parametrize("name", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = ALONE[name]
    d = LM.write_model(tmp_path / name, cfg, LM.make_tensors(cfg, 5, rel_rows=6))
    ids = _ids(np.random.default_rng(1), cfg["vocab"], 70)
    ref = _plain(d, ids)
    runner = _runner(d, dtype, tokens=128, page=8)
    whole = _play(runner, RU.whole("a", ids))
    one = _play(runner, RU.tail_one_by_one("b", ids, tail=69))        # the first token, then every token alone
    tol = F32_TOL if dtype == "float32" else BF16_TOL
    assert _worst(whole, {"a": ref}) < tol
    assert _worst(one, {"b": ref}) < tol


# ---------------------------------------------------------------------------------------------------------------
# whole models: prompts, token by token, portions, mixed batches, pages and slots used again
# ---------------------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("lupanex")
    out = {}
    for i, name in enumerate(sorted(LM.CONFIGS)):
        d = LM.make_model(root / name, name, seed=10 + i)
        rng = np.random.default_rng(100 + i)
        reqs = {f"r{k}": _ids(rng, LM.CONFIGS[name]["vocab"], n) for k, n in enumerate((150, 1, 37, 64, 91, 17))}
        out[name] = (d, reqs, {r: _plain(d, ids) for r, ids in reqs.items()})
    return out


@pytest.mark.parametrize("name", sorted(LM.CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_decoding_portions_and_mixed_batches(models, name, dtype):
    d, reqs, ref = models[name]
    tol = F32_TOL if dtype == "float32" else BF16_TOL
    cut_tol = 1e-5 if dtype == "float32" else BF16_CUT_TOL
    runner = _runner(d, dtype, tokens=384, page=8, slots=4)
    whole = {}
    for r, ids in reqs.items():
        whole.update(_play(runner, RU.whole(r, ids)))
    assert _worst(whole, ref) < tol
    runs = {}
    # the last 40 tokens one by one (the one-token request is a prompt of one token)
    runs["decode"] = {k: v for r, ids in reqs.items() for k, v in _play(runner, RU.tail_one_by_one(r, ids, tail=40)).items()}
    # portions of changing sizes down to two tokens, cut inside pages
    runs["portions"] = {k: v for r, ids in reqs.items()
                        for k, v in _play(runner, RU.changing_portions(r, ids, sizes=(7, 2, 13, 3, 2, 29, 5, 2, 8, 11))).items()}
    # up to four requests live, portions of some beside single tokens of others; six requests through four slots and a
    # pool that holds fewer positions than the requests have in all
    rng = np.random.default_rng(3)
    runs["mixed"] = _play(runner, RU.mixed(reqs, {r: max(1, len(ids) - 20) for r, ids in reqs.items()}, rng, live_max=4))
    # one prompt in portions beside decoding requests
    rng = np.random.default_rng(4)
    runs["beside"] = _play(runner, RU.mixed(reqs, {r: len(ids) // 2 for r, ids in reqs.items()}, rng, live_max=3, portions=(2, 40),
                                           one_prompt_at_a_time=True))
    for how, got in runs.items():
        assert len(got) == sum(len(i) for i in reqs.values()), how
        assert _worst(got, ref) < tol, how
        cut = _worst(got, {r: np.stack([whole[(r, p)] for p in range(len(ids))]) for r, ids in reqs.items()})
        assert cut < cut_tol, (how, cut)
    runner.cache.check()
    assert all(f == p.num_pages for f, p in zip(runner.cache.free_pages(), runner.cache.tables.pools))     # every page came back


def test_a_request_alone_and_beside_others_on_other_pages_and_slots(models):
    """The same request first alone in a fresh engine, then as the fourth of four whose neighbours took the low pages and slots."""
    d, reqs, ref = models["looped"]
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
    """300 tokens one by one after a short prompt: the recurrent state is carried 300 times, the window of the convolution moves
    300 times, the query factor passes its steps and the distances pass every bucket."""
    cfg = LM.CONFIGS["looped"]
    d = LM.make_model(tmp_path / "m", "looped", seed=77)
    ids = _ids(np.random.default_rng(8), cfg["vocab"], 310)
    ref = _plain(d, ids)
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        _worst.rms = dtype == "bfloat16"
        got = _play(_runner(d, dtype, tokens=320, page=16), RU.tail_one_by_one("a", ids, tail=300))
        assert _worst(got, {"a": ref}) < tol


# ---------------------------------------------------------------------------------------------------------------
# one key that must be found: far back, at the first position, on either side of a page's border
# ---------------------------------------------------------------------------------------------------------------

def _needle_model(tmp_path, width=32, vocab=700):
    """One attention layer whose query and key are the normed embedding itself (W_q = W_k = I, no position rows, one head):
    a token that comes twice scores dim * scale against its first coming and about sqrt(dim) * scale against all others, so
    the last token's output is the value of ONE far key.  A wrong page, slot or offset returns another token's value."""
    cfg = LM.config(vocab, width, [LM.layer("attention", LM.att(1, 1, width, width, 1.0))], max_positions=1024, scale=1.0)
    t = LM.make_tensors(cfg, 3)
    t["pos"][:] = 0.0
    t["l0.norm1"][:] = 1.0
    t["l0.mix.q"] = np.eye(width, dtype=np.float32)
    t["l0.mix.k"] = np.eye(width, dtype=np.float32)
    t["l0.mix.v"] *= 4.0
    return LM.write_model(tmp_path / "needle", cfg, t, dtype=torch.float32), cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_is_found_wherever_it_lies(tmp_path, dtype):
    d, cfg = _needle_model(tmp_path)
    rng = np.random.default_rng(0)
    n, page = 600, 16
    base = [int(t) for t in rng.permutation(cfg["vocab"])[:n]]            # all different
    c, W = PL.read_model(d)
    runner = _runner(d, dtype, tokens=640, page=page)
    for place in (0, 1, 3, page - 1, page, page + 1, 255, 256, 257, n - 3):
        ids = base[:n - 1] + [base[place]]                               # the last token repeats the one at `place`
        ref = PL.forward(c, W, ids)
        # the test is sharp: in the plain implementation the far key has nearly all of the last token's weight
        x = PL.rms(PL.embed(W["embed"], W["pos"], ids, 1.0), c["norm"]["eps"])
        s = (PL.rms(x, c["norm"]["eps"]) @ PL.rms(x[-1], c["norm"]["eps"])) * 1.0
        e = np.exp(s - s.max())
        assert e[place] / e.sum() > 0.45 and e[place] / e.sum() + e[-1] / e.sum() > 0.95
        tol = F32_TOL if dtype == "float32" else BF16_TOL
        for how, steps in (("prompt", RU.whole("a", ids)), ("decoded", RU.tail_one_by_one("a", ids, tail=2)),
                           ("portions", RU.changing_portions("a", ids, sizes=(250, 5, 2, 100)))):
            got = _play(runner, [(e_, end) for e_, end in steps])
            last = {k: v for k, v in got.items() if k[1] == n - 1}
            assert _worst(last, {"a": ref}) < tol, (place, how)


def test_distances_on_both_sides_of_every_bucket_edge(tmp_path):
    """A model whose only signal is the distance bias: keys and queries are zero, so the softmax weights are the biases alone.
    Every distance 0..299 is met by the last tokens, in prompts and decoded."""
    cfg = LM.config(30, 32, [LM.layer("attention", LM.att(2, 1, 32, 32, 1.0, bias_max=50))], max_positions=512)
    t = LM.make_tensors(cfg, 9, rel_rows=14)
    t["l0.mix.q"][:] = 0.0
    t["l0.mix.rel"] *= 3.0
    d = LM.write_model(tmp_path / "bias", cfg, t)
    ids = _ids(np.random.default_rng(2), 30, 300)
    ref = _plain(d, ids)
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        _worst.rms = dtype == "bfloat16"
        runner = _runner(d, dtype, tokens=320, page=16)
        assert _worst(_play(runner, RU.whole("a", ids)), {"a": ref}) < tol
        assert _worst(_play(runner, RU.tail_one_by_one("a", ids, tail=120)), {"a": ref}) < tol
    from vitna_anchor_b200.parts.attention import distance_bucket
    assert [distance_bucket(n, 14, 50) for n in range(400)] == [PL.distance_bucket(n, 14, 50) for n in range(400)]


# ---------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("streams,width", [(1, 24), (3, 200), (8, 64)])
def test_hyper_step_kernel(streams, width):
    from vitna_anchor_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(streams)
    r = lambda *s: torch.randn(*s, generator=g, device="cuda")
    T = 37
    xs, y, mix, out_w, in_w, nw = r(T, streams * width), r(T, width), r(streams, streams), r(streams), r(streams), r(width)
    X = xs.view(T, streams, width).double()
    new = torch.einsum("ij,tiw->tjw", mix.double(), X) + out_w.double()[None, :, None] * y.double()[:, None, :]
    u = torch.einsum("i,tiw->tw", in_w.double(), new)
    xn_ref = u / torch.sqrt((u * u).mean(-1, keepdim=True) + 1e-5) * nw.double()
    xn = torch.empty(T, width, device="cuda")
    total = torch.empty(T, width, device="cuda")
    ops.hyper_step(xs, y, streams, mix=mix, out_w=out_w, in_w=in_w, norm_w=nw, eps=1e-5, xn=xn, sum_out=total)
    torch.cuda.synchronize()
    assert torch.allclose(xs.view(T, streams, width).double(), new, atol=1e-5)
    assert torch.allclose(xn.double(), xn_ref, atol=2e-5) and torch.allclose(total.double(), u, atol=2e-5)
    assert float(y.abs().max()) == 0.0                                   # left zeroed for the next sublayer
    ops.hyper_step(xs, None, streams, sum_out=total)                      # the plain sum of the rows
    torch.cuda.synchronize()
    assert torch.allclose(total.double(), new.sum(1), atol=2e-5)


@pytest.mark.parametrize("kind", ["gelu", "gelu_tanh", "silu"])
def test_activation_alone_and_in_the_epilogues(kind):
    from vitna_anchor_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(1)
    ref = {"gelu": PL.gelu_erf, "gelu_tanh": PL.gelu_tanh, "silu": PL.silu}[kind]
    x = torch.randn(5, 333, generator=g, device="cuda") * 3
    got = ops.activation(x.clone(), kind)
    assert np.abs(got.cpu().numpy() - ref(x.double().cpu().numpy())).max() < 2e-6
    for M in (3, 40, 200):                                               # few-rows kernel, few-rows kernel, tcgen05 kernel
        a = (torch.randn(M, 128, generator=g, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(264, 128, generator=g, device="cuda") * 0.2).bfloat16()
        out = torch.empty(M, 264, dtype=torch.bfloat16, device="cuda")
        ops.linear_act(a, w, out, kind)
        ops.check_device_errors()
        want = ref(a.double().cpu().numpy() @ w.double().cpu().numpy().T)
        assert np.abs(out.float().cpu().numpy() - want).max() < 2e-2 * max(1.0, np.abs(want).max())


def test_the_one_kernel_delta_rule_for_single_tokens_gives_what_the_three_kernels_give():
    from vitna_anchor_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(4)
    r = lambda *s: torch.randn(*s, generator=g, device="cuda")
    for (G, H, dk, dv, taps) in ((1, 2, 16, 8, 3), (3, 9, 64, 64, 4), (4, 16, 128, 128, 4), (1, 3, 40, 24, 1), (2, 2, 256, 32, 2), (1, 1, 8, 300, 2)):
        assert ops.delta_decode_takes(G, H, dk, dv, taps)
        C, N, S = 2 * G * dk + H * dv, 2 * G * dk + 2 * H * dv + 2 * H, 5
        conv, a_log, dt, nw = r(C, taps) * 0.6, r(H) - 1, r(H), 1 + 0.1 * r(dv)
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
                ops.delta_rule(proj, conv, a_log, dt, nw, 1e-5, token_seg, seg_starts, slots, states[single],
                               torch.empty(S, ops.delta_prep_width(G, H, dk, dv), device="cuda"), torch.zeros(S, H * dv, device="cuda"), out,
                               G, H, dk, dv, taps, single_tokens=single)
                outs.append(out)
            live = slots >= 0
            assert torch.allclose(outs[0][live], outs[1][live], rtol=1e-4, atol=1e-5), (G, H, dk, dv, taps, step)
            assert torch.allclose(states[0], states[1], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("chunked", [False, True])
def test_the_delta_rule_kernels_against_the_recurrence_written_out(chunked):
    """Segments of unequal length on scattered slots, a second step that continues from the state of the first; token by token and
    in the chunked form (segments that end inside a chunk, exactly at its end, and single tokens beside them)."""
    from vitna_anchor_b200 import ops
    rng = np.random.default_rng(5)
    sizes = ((1, 2, 16, 8, 3), (2, 2, 64, 128, 4), (1, 3, 40, 24, 1), (2, 4, 128, 64, 2), (1, 2, 10, 12, 2), (1, 1, 256, 32, 2))
    for (G, H, dk, dv, taps) in sizes:
        if chunked and not ops.delta_chunked_takes(G, H, dk, dv, taps):
            continue
        C, N = 2 * G * dk + H * dv, 2 * G * dk + 2 * H * dv + 2 * H
        lens1, lens2, slots = ([70, 1, 128], [1, 97, 64], [3, 0, 2]) if chunked else ([5, 1, 19], [1, 7, 2], [3, 0, 2])
        conv = rng.standard_normal((C, taps)) * 0.6
        a_log, dt_bias, nw = rng.standard_normal(H) - 1, rng.standard_normal(H), 1 + 0.1 * rng.standard_normal(dv)
        proj_all = [rng.standard_normal((l1 + l2, N)) for l1, l2 in zip(lens1, lens2)]
        state = torch.zeros(4, ops.delta_state_floats(G, H, dk, dv, taps), device="cuda")
        f = lambda a: torch.tensor(np.asarray(a), dtype=torch.float32, device="cuda")
        outs = [[] for _ in lens1]
        for step, lens in enumerate((lens1, lens2)):
            T = sum(lens)
            rows = np.concatenate([p[(0 if step == 0 else lens1[i]):(lens1[i] if step == 0 else None)] for i, p in enumerate(proj_all)])
            seg_starts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
            token_seg = torch.tensor(np.repeat(np.arange(len(lens)), lens), dtype=torch.int32, device="cuda")
            out = torch.empty(T, H * dv, device="cuda")
            ops.delta_rule(f(rows), f(conv), f(a_log), f(dt_bias), f(nw), 1e-5, token_seg, seg_starts,
                           torch.tensor(slots, dtype=torch.int32, device="cuda"), state, torch.empty(T, ops.delta_prep_width(G, H, dk, dv), device="cuda"),
                           torch.empty(T, H * dv, device="cuda"), out, G, H, dk, dv, taps,
                           chunk_scratch=torch.empty(ops.delta_chunked_scratch_floats(T, len(lens), H, dk, dv), device="cuda") if chunked else None)
            o = out.cpu().numpy()
            at = 0
            for i, n in enumerate(lens):
                outs[i].append(o[at:at + n])
                at += n
        for i, p in enumerate(proj_all):                                  # the recurrence written out, whole sequence at once
            q = PL.silu(PL.short_conv(p[:, :G * dk], conv[:G * dk])).reshape(-1, G, dk)
            k = PL.silu(PL.short_conv(p[:, G * dk:2 * G * dk], conv[G * dk:2 * G * dk])).reshape(-1, G, dk)
            v = PL.silu(PL.short_conv(p[:, 2 * G * dk:C], conv[2 * G * dk:])).reshape(-1, H, dv)
            q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
            k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
            gate = PL.silu(p[:, C:C + H * dv]).reshape(-1, H, dv)
            beta, decay = PL.sigmoid(p[:, C + H * dv:C + H * dv + H]), np.exp(-np.exp(a_log) * PL.softplus(p[:, C + H * dv + H:] + dt_bias))
            want = np.zeros((len(p), H, dv))
            for h in range(H):
                S = np.zeros((dk, dv))
                for t in range(len(p)):
                    S = decay[t, h] * S
                    S = S + np.outer(k[t, h // (H // G)], beta[t, h] * (v[t, h] - S.T @ k[t, h // (H // G)]))
                    want[t, h] = S.T @ q[t, h // (H // G)]
            want = (PL.rms(want, 1e-5, nw) * gate).reshape(len(p), H * dv)
            assert np.abs(np.concatenate(outs[i]) - want).max() < 2e-5 * max(1.0, np.abs(want).max()), (G, H, dk, dv, taps, i)


# ---------------------------------------------------------------------------------------------------------------
# the engine's own entry point and scheduler, the command line, the replay program
# ---------------------------------------------------------------------------------------------------------------

def _plain_greedy(model_dir, ids, n):
    cfg, W = PL.read_model(model_dir)
    ids = list(ids)
    for _ in range(n):
        ids.append(int(np.argmax(PL.forward(cfg, W, ids)[-1])))
    return ids[-n:]


def test_greedy_generation_through_the_engine_and_its_scheduler(models):
    from vitna_anchor_b200.engine.engine import Engine
    d, reqs, _ = models["streams"]
    eng = Engine(d, dtype="float32", parallel=3, kv_block=8, max_batch_tokens=64, max_prompt_portion=24)
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
    import subprocess
    import sys
    d, reqs, ref = models["plain"]
    rp = RU.Replay(d, "float32", tmp_path / "out", max_tokens=256, kv_block=8)
    got = rp.run(RU.changing_portions("a", reqs["r4"]) + RU.tail_one_by_one("b", reqs["r2"], tail=10), LM.CONFIGS["plain"]["vocab"])
    rp.close()
    assert _worst(got, {"a": ref["r4"], "b": ref["r2"]}) < F32_TOL
    import os
    out = subprocess.run([sys.executable, os.path.join(RU.ROOT, "bin", "vitna-anchor"), "generate", "--model", d, "--ids",
                          ",".join(map(str, reqs["r5"])), "--max-new", "8", "--greedy", "--dtype", "float32"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert _plain_greedy(d, reqs["r5"], 8) == [int(t) for t in json.loads(out.stdout.strip().splitlines()[-1])["ids"]]
