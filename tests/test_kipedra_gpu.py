"""The Kipedra decoder in the engine against the plain implementation (tests/plain_kipedra.py): each mechanism alone
(models of one layer), whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with
so few pages and slots that both are used again, long decoding, and greedy generation through the engine's entry point.

Where random weights would hide a fault the inputs are made so that it shows: the score scale of an attention layer is
raised so that the softmax of every (position, head) rests on one or two keys (a key wrongly seen or hidden, one
position off at the window's edge or a page's border, then moves that position's logits by far more than rounding),
and the decays of a delta layer are brought close to one so that the first tokens of a long prompt still weigh in its
last positions (a state that is lost, or started from another request's, shows)."""
import pytest
import torch

import helpers
import kipedra_configs as kc
import kipedra_helpers as kh
import plain_kipedra

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


# ------------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("C, taps, act", [(10, 4, "silu"), (300, 1, None), (37, 5, None), (64, 2, "silu")])
def test_short_convolution_with_tails(C, taps, act):
    """Three requests, each in two steps cut at another place, beside the convolution over the whole sequences; the slots'
    tails carry what a portion needs of the one before; extra columns pass through."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(C + taps)
    lens, cuts, slots, extra = [9, 1, 6], [2, 1, 5], [3, 0, 1], 5
    w, bias = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    seqs = [torch.randn(2, n, C + extra, generator=g) for n in lens]          # two slices whose sum is the projection
    want = []
    for x in seqs:
        p = x.sum(0)[:, :C].double() + bias.double()
        y = plain_kipedra.causal_conv(p, w.double())
        want.append(plain_kipedra.silu(y) if act else y)
    tail = torch.zeros(5, max(taps - 1, 0), C).cuda()
    tail[4] = 7.0                                                             # a slot no request of the step owns stays as it is
    got = [[] for _ in lens]
    for part in (0, 1):
        rows = [x[:, :c] if part == 0 else x[:, c:] for x, c in zip(seqs, cuts)]
        live = [i for i, r in enumerate(rows) if r.shape[1]]
        ctx = helpers.make_context([rows[i].shape[1] for i in live], [0] * len(live), [[[0]] * len(live)])
        ctx.slot_ids = torch.tensor([slots[i] for i in live], dtype=torch.int32).cuda()
        x = torch.cat([rows[i] for i in live], dim=1).contiguous().cuda()
        out = ops.short_conv(x, C, w.cuda(), bias.cuda(), tail, ctx.req_of_token, ctx.q_start, ctx.slot_ids, ctx.R, act=act, copy_to=C + extra)
        assert (out[:, C:].double().cpu() - x.sum(0)[:, C:].double().cpu()).abs().max() < 1e-5
        at = 0
        for i in live:
            got[i].append(out[at:at + rows[i].shape[1], :C].double().cpu())
            at += rows[i].shape[1]
    for i in range(len(lens)):
        assert (torch.cat(got[i]) - want[i]).abs().max() < 2e-5, f"request {i}"
    assert bool((tail[4] == 7.0).all())


@pytest.mark.parametrize("H, G, dk, dv", [(4, 2, 24, 12), (3, 3, 100, 20), (2, 1, 136, 33), (5, 5, 7, 9), (2, 2, 256, 16)])
def test_gated_delta_kernel_in_portions(H, G, dk, dv):
    """The recurrence over a request, whole and cut into portions of changing size, with the per-token inputs made inside
    the kernel and by the kernel of their own, against loops in double precision; the state lives in the request's slot
    from step to step and is the same, up to FP32 rounding, however the prompt is cut."""
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(H * dk + dv)
    n, C = 75, 2 * G * dk + H * dv
    u = torch.randn(n, C, generator=g)
    p = torch.randn(n, 2 * H + 3, generator=g)
    A_log, dt_bias = torch.randn(H, generator=g) - 3.0, torch.randn(H, generator=g)
    ud, pd = u.double(), p.double()
    q = ud[:, :G * dk].view(n, G, dk)
    k = ud[:, G * dk:2 * G * dk].view(n, G, dk)
    v = ud[:, 2 * G * dk:].view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(pd[:, 1:1 + H])
    decay = torch.exp(-torch.exp(A_log.double()) * plain_kipedra.softplus(pd[:, 2 + H:2 + 2 * H] + dt_bias.double()))
    want = torch.zeros(n, H, dv, dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(dk, dv, dtype=torch.float64)
        for t in range(n):
            S = decay[t, h] * S
            S = S + torch.outer(k[t, h // (H // G)], beta[t, h] * (v[t, h] - S.T @ k[t, h // (H // G)]))
            want[t, h] = S.T @ q[t, h // (H // G)]
    results = []
    for cuts, prepare in (([n], True), ([n], False), ([1, 2, 30, 1, 17, 24], False), ([40, 3, 32], True)):
        state = torch.zeros(3, H, dv, dk).cuda()
        outs, at = [], 0
        for c in cuts:
            ctx = helpers.make_context([c], [at], [[[0]]])
            ctx.slot_ids = torch.tensor([2], dtype=torch.int32).cuda()
            outs.append(ops.gated_delta(u[at:at + c].contiguous().cuda(), p[at:at + c].contiguous().cuda(), 1, 2 + H, A_log.cuda(), dt_bias.cuda(),
                                        state, ctx.q_start, ctx.slot_ids, 1, H, G, dk, dv, prepare=prepare))
            at += c
        results.append((torch.cat(outs).cpu(), state.cpu()))
        err = (results[-1][0].double().view(n, H, dv) - want).abs().max() / want.abs().max()
        assert err < 2e-5, f"cuts {cuts}: {float(err):.3e}"
        assert bool((state[:2] == 0).all())
    for other in results[1:]:
        for a, b in zip(results[0], other):
            assert float((a - b).abs().max()) <= 2e-6 * float(a.abs().max())


@pytest.mark.parametrize("D", [50, 256, 1000])
def test_scaled_add_and_both_norms(D):
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(D)
    T, S = 6, 3
    h, a, b = torch.randn(T, D, generator=g), torch.randn(3, T, D, generator=g), torch.randn(T, D, generator=g)
    y, pw = torch.randn(T * S, D, generator=g), torch.rand(T, S, generator=g)
    rows = torch.randperm(T * S, generator=g).to(torch.int32)
    w1, w2 = torch.randn(D, generator=g), torch.randn(D, generator=g)
    picked = (pw.double()[:, :, None] * y.double()[rows.long()].view(T, S, D)).sum(1)
    want_h = h.double() + 0.3 * (a.double().sum(0) + b.double() + picked)
    norm = lambda x, w: x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w.double()
    hh = h.clone().cuda()
    o1, o2 = ops.scaled_add_norm(hh, a.cuda(), b.cuda(), (y.cuda(), rows.cuda(), pw.cuda()), 0.3, w1.cuda(), w2.cuda(), 1e-5, torch.float32)
    assert (hh.double().cpu() - want_h).abs().max() < 1e-5
    assert (o1.double().cpu() - norm(want_h, w1)).abs().max() < 3e-5 and (o2.double().cpu() - norm(want_h, w2)).abs().max() < 3e-5
    pick = torch.tensor([4, 0, 4], dtype=torch.int32).cuda()
    o1, o2 = ops.scaled_add_norm(hh, None, None, None, 0.0, w1.cuda(), None, 1e-5, torch.bfloat16, rows=pick)
    assert o2 is None and (o1.double().cpu() - norm(want_h[pick.long().cpu()], w1)).abs().max() < 0.05


@pytest.mark.parametrize("E, k", [(5, 2), (40, 40), (300, 33), (1500, 4)])
def test_router_with_a_correction(E, k):
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(E)
    T = 9
    z, bias = torch.randn(2, T, E, generator=g), torch.randn(E, generator=g)
    s = torch.sigmoid(z.sum(0).double())
    chosen = torch.topk(s + bias.double(), k, dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    want = picked / (picked.sum(-1, keepdim=True) + 1e-20) * 2.5
    sel_e, sel_w = ops.route_biased(z.cuda(), k, bias.cuda(), 2.5)
    assert torch.equal(sel_e.cpu().long().sort(-1).values, chosen.sort(-1).values)
    order = sel_e.cpu().long().argsort(-1)
    assert (torch.gather(sel_w.cpu().double(), 1, order) - torch.gather(want, 1, chosen.argsort(-1))).abs().max() < 1e-6


@pytest.mark.parametrize("act", ["silu", "gelu_tanh", "relu2"])
def test_activations(act):
    from quench6k_b200 import ops
    x = (torch.randn(7, 26, generator=torch.Generator().manual_seed(1)) * 3).cuda()
    f = {"silu": plain_kipedra.silu, "gelu_tanh": plain_kipedra.gelu_tanh, "relu2": lambda z: torch.relu(z) ** 2}[act]
    xd = x.double().cpu()
    assert (ops.activate(x, 13, True, act, torch.float32).double().cpu() - f(xd[:, :13]) * xd[:, 13:]).abs().max() < 1e-5
    assert (ops.activate(x, 26, False, act, torch.float32).double().cpu() - f(xd)).abs().max() < 1e-5


# ------------------------------------------------------------------------------------------------- one mechanism alone
ONE = {
    "delta": kc.delta(4, 2, 24, 12, 3),
    "delta_as_many_key_heads": kc.delta(3, 3, 100, 20, 4),
    "delta_one_tap_wide_keys": kc.delta(2, 1, 136, 33, 1),
    "window": kc.attention(4, 2, 8, 12, 3, 5, 4, 100.0, 3.0),
    "window_of_pages": kc.attention(3, 1, 16, 4, 2, 64, 16, 10000.0, 2.0),
    "window_of_one": kc.attention(2, 2, 16, 16, 4, 1, 8, 50.0, 1.0),
    "window_never_reached": kc.attention(2, 1, 40, 40, 1, 1000, 0, 10000.0, 1.0),
    "window_and_dense": kc.attention(4, 4, 16, 8, 2, 11, 6, 1000.0, 2.0, ff=("dense", 30)),
    "window_and_experts": kc.attention(2, 1, 8, 8, 3, 6, 8, 20.0, 2.0, ff=("moe", 6, 2, 20, 1.7)),
    "delta_and_one_expert": kc.delta(2, 2, 16, 8, 2, ff=("moe", 4, 1, 12, 0.6)),
}


def _slow_decays(weights):
    """Decays close to one: what the first tokens wrote is still in the state after hundreds of tokens."""
    for name, w in weights.items():
        if name.endswith(".A_log"):
            w.fill_(-5.0)


@pytest.fixture(scope="module", params=sorted(ONE))
def single(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    cfg, weights = kh.make_folder(folder, kc.one_layer(ONE[name]), seed=3, init_std=0.3, doctor=_slow_decays)
    reqs = {"long": helpers.random_tokens(330, cfg["vocab"], 1), "short": helpers.random_tokens(9, cfg["vocab"], 2),
            "one": helpers.random_tokens(1, cfg["vocab"], 3)}
    return name, folder, cfg, weights, reqs


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_whole_prompt(single, dtype):
    name, folder, cfg, weights, reqs = single
    steps, mt = helpers.schedule_whole(reqs)
    kh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_token_by_token(single, dtype):
    """Every token decoded alone from the first one on: each key is found through the cache, each state and tail through its slot."""
    name, folder, cfg, weights, reqs = single
    reqs = {"long": reqs["long"][:150], "short": reqs["short"]}
    steps, mt = helpers.schedule_tail(reqs, tail=10 ** 6)
    kh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_portions(single, dtype):
    name, folder, cfg, weights, reqs = single
    for seed in (0, 1):
        steps, mt = helpers.schedule_portions(reqs, seed=seed)
        kh.replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} portions")


def test_a_hidden_key_would_show(single):
    """The premise of the tests above: a key more or less in a window, or a state that forgot its first tokens, is far
    beyond the tolerance.  The plain implementation with the window one wider, or started in the middle, differs from itself."""
    name, folder, cfg, weights, reqs = single
    a = kh.plain(cfg, weights, reqs["long"])
    if name.startswith("window") and cfg["layers"][0]["mixer"]["mask"]["size"] < 32 and cfg["layers"][0]["mlp"] is None:
        other = kc.one_layer(ONE[name])
        other["layers"][0]["mixer"]["mask"]["size"] += 1
        b = kh.plain(other, weights, reqs["long"])
        moved = ((a - b).abs().max(-1).values / a.abs().max()) > 3 * kh.TOL["bfloat16"]
        assert moved.float().mean() > 0.15
    elif name.startswith("delta") and cfg["layers"][0]["mlp"] is None:
        b = kh.plain(cfg, weights, reqs["long"][150:])
        moved = (a[150:] - b).abs().max(-1).values / a.abs().max()
        assert (moved[:40] > 3 * kh.TOL["bfloat16"]).float().mean() > 0.5, "a lost state does not show in the next tokens"
        assert float(moved[100:].median()) > 100 * kh.TOL["float32"], "the state of the first 150 tokens no longer shows 100 tokens later"
    else:
        pytest.skip("written for the window and for the recurrent state")


# ------------------------------------------------------------------------------------------------- a key that stands out
BEACON, WINDOW = 17, 37


def _beacon_model(folder):
    """One attention layer whose every query looks, above all, for one token: entry 15 of every key (it does not rotate)
    is large for that token alone, and entry 15 of every query is a large bias.  A position that has the token inside
    its window gives it nearly all its weight; one position further it is gone."""
    cfg = kc.one_layer(kc.attention(4, 2, 16, 8, 1, WINDOW, 4, 100.0, 1.0), width=48, vocab=61, page=4)

    def doctor(w):
        x = w["embed"][BEACON].double()
        xn = x / torch.sqrt((x * x).mean() + 1e-5) * (1.0 + w["l0.norm1"].double())
        for name in ("l0.mix.q.conv", "l0.mix.k.conv", "l0.mix.v.conv"):
            w[name].fill_(1.0)
        for g in range(2):
            w["l0.mix.k"][g * 16 + 15] = (8.0 * xn / (xn * xn).sum()).to(torch.bfloat16)
            w["l0.mix.k.b"][g * 16 + 15] = 0.0
        for h in range(4):
            w["l0.mix.q"][h * 16 + 15] = 0.0
            w["l0.mix.q.b"][h * 16 + 15] = 20.0

    return kh.make_folder(folder, cfg, seed=11, init_std=0.3, doctor=doctor)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_at_the_window_edge(tmp_path, dtype):
    """The token every query looks for stands at a page's border and inside a page; the positions that see it last and
    the first that no longer see it lie in a prompt (whole and in portions) and among tokens decoded one by one."""
    cfg, weights = _beacon_model(str(tmp_path))
    toks = [t if t != BEACON else 3 for t in helpers.random_tokens(200, cfg["vocab"], 5)]
    for p in (8, 101):
        toks[p] = BEACON
    reqs = {"b": toks}
    want = kh.plain(cfg, weights, toks)
    narrower = kc.one_layer(cfg["layers"][0])
    narrower["layers"][0]["mixer"]["mask"]["size"] = WINDOW - 1
    other = kh.plain(narrower, weights, toks)
    for p in (8, 101):
        last, gone = p + WINDOW - 1, p + WINDOW
        scale = float(want.abs().max())
        assert float((want[last] - other[last]).abs().max()) > 0.1 * scale, "the last position that sees the token does not depend on it"
        assert float((want[gone] - other[gone]).abs().max()) < 1e-3 * scale, "the first position beyond the token still depends on it"
    for what, (steps, mt) in {"whole": helpers.schedule_whole(reqs), "decoded": helpers.schedule_tail(reqs, tail=70),
                              "from the start": helpers.schedule_tail(reqs, tail=10 ** 6), "portions": helpers.schedule_portions(reqs, seed=2),
                              "portions again": helpers.schedule_portions(reqs, seed=3)}.items():
        outputs, _ = helpers.run_replay(str(tmp_path), dtype, steps, mt, max_requests=2)
        got = helpers.collect(reqs, steps, outputs)["b"]
        kh.assert_close(got, want, dtype, f"window edge, {what}")
        for p in (8, 101):                       # the edge itself, held to the plain tolerance whatever the rest does
            for at in (p + WINDOW - 1, p + WINDOW):
                err = float((got[at].double() - want[at]).abs().max()) / float(want.abs().max())
                assert err <= (3 if dtype == "bfloat16" else 1) * kh.TOL[dtype], f"window edge, {what} {dtype}: position {at}: {err:.3e}"


# ------------------------------------------------------------------------------------------------- whole models
LENGTHS = {"K1": [71, 130, 45, 96, 64, 33, 1, 58, 77], "K2": [85, 140, 37, 101, 2, 50, 90, 125, 44], "K3": [90, 257, 129, 48, 75, 40, 310, 66, 83],
           "K4": [70, 33, 131, 20, 64, 3, 95, 41, 58]}


@pytest.fixture(scope="module", params=["K1", "K2", "K3", "K4"])
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    cfg, weights = kh.make_folder(folder, kc.get(name), seed=7, init_std=0.08)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(LENGTHS[name])}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs}


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_whole(model, dtype):
    steps, mt = helpers.schedule_whole(model["requests"])
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_prefill_then_decode(model, dtype):
    steps, mt = helpers.schedule_tail(model["requests"], tail=40)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " tail")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_portions(model, dtype):
    steps, mt = helpers.schedule_portions(model["requests"], seed=5)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_mixed_batches_reuse_pages_and_slots(model, dtype):
    """Up to four live requests, unequal portions beside single tokens, requests that sit steps out; nine requests go
    through four slots and a pool of the live requests' size, so every slot and most pages are used again."""
    page = model["cfg"]["kv_page_size"]
    for seed in (0, 1):
        steps, mt = helpers.schedule_mixed(model["requests"], page, seed=seed, max_live=4)
        got = kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype,
                                    model["name"] + " mixed", max_requests=4)
    if dtype == "float32":
        # and the same requests each alone: what else is in the batch, and which pages and slots are used, changes nothing
        steps, mt = helpers.schedule_whole(model["requests"])
        outputs, _ = helpers.run_replay(model["folder"], dtype, steps, mt)
        alone = helpers.collect(model["requests"], steps, outputs)
        for rid in model["requests"]:
            kh.assert_close(got[rid], alone[rid], dtype, f"{model['name']} {dtype} {rid} batched against alone", tol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_many_decoding_together(model, dtype):
    page = model["cfg"]["kv_page_size"]
    reqs = {rid: t for rid, t in model["requests"].items() if len(t) > 12}
    steps, mt = helpers.schedule_wide_decode(reqs, page)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " wide decode",
                          max_requests=len(reqs))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """A short prompt and hundreds of tokens decoded one by one: windows and pages pass over decoded tokens, the recurrent
    state runs long, the decode steps are replayed from a recorded graph."""
    reqs = {"d": helpers.random_tokens(420, model["cfg"]["vocab"], 9)}
    steps, mt = helpers.schedule_tail(reqs, tail=410)
    kh.replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " long decode")


def test_greedy_generation_through_the_engine(model):
    """Engine.generate (scheduler, continuous batching, device-side argmax, CUDA graphs) against greedy decoding with the
    plain implementation, float32; prompts of unequal length in one engine with few pages."""
    import quench6k_b200 as q
    cfg, weights = model["cfg"], model["weights"]
    prompts = [helpers.random_tokens(n, cfg["vocab"], 50 + n) for n in (5, 23, 1, 40, 12, 31)]
    page = cfg["kv_page_size"]
    eng = q.Engine.from_folder(model["folder"], dtype="float32", page_size=page, num_pages=4 * (64 // page + 2), max_requests=4,
                               max_batch_tokens=32)
    outs = eng.generate(prompts, q.SamplingParams(max_tokens=12, temperature=0))
    for prompt, out in zip(prompts, outs):
        toks = list(prompt)
        for i in range(12):
            logits = kh.plain(cfg, weights, toks)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < 1e-3 * float(logits.abs().max()):
                break                                  # a near-tie: float32 may pick either; the continuation is not comparable
            assert out.tokens[i] == int(logits.argmax()), f"{model['name']}: prompt of {len(prompt)}, generated token {i}"
            toks.append(out.tokens[i])
    eng.runner.manager.check()


def test_command_line_generates(model):
    """`generate` of the command line on a Kipedra model folder: the model class comes from config.json."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, weights = model["cfg"], model["weights"]
    prompt = helpers.random_tokens(11, cfg["vocab"], 77)
    r = subprocess.run([sys.executable, "-m", "quench6k_b200", "generate", "--model", model["folder"], "--prompt-ids", ",".join(map(str, prompt)),
                        "--n", "6", "--dtype", "float32", "--context", "128"], cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    toks = list(prompt)
    for _ in range(6):
        logits = kh.plain(cfg, weights, toks)[-1]
        top2 = logits.topk(2).values
        if float(top2[0] - top2[1]) < 1e-3 * float(logits.abs().max()):
            return
        toks.append(int(logits.argmax()))
    assert "prompt: 11 tokens" in r.stdout and f"ids: {toks[11:]}" in r.stdout
