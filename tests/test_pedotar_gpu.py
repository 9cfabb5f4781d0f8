"""The Pedotar decoder in the engine against the plain implementation (tests/plain_pedotar.py): each mechanism alone
(models of one layer), whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with
so few pages and slots that both are used again, long decoding, and greedy generation through the engine's entry point.

Where random weights would hide a fault the score scale of the configuration is raised so that the softmax of every
(position, head) rests on one or two keys: a key that is wrongly seen or wrongly hidden (one position off at a chunk's
start, a page's border, the far end of a long context) then moves that position's logits by far more than rounding."""
import pytest
import torch

import helpers
import pedotar_configs as pc
import pedotar_helpers as ph

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _replay_and_compare(folder, cfg, weights, requests, steps, max_tokens, dtype, what, page=None, max_requests=4):
    outputs, runner = helpers.run_replay(folder, dtype, steps, max_tokens, page_size=page, max_requests=max_requests)
    got = helpers.collect(requests, steps, outputs)
    worst = 0.0
    for rid, toks in requests.items():
        worst = max(worst, ph.assert_close(got[rid], ph.plain(cfg, weights, toks), dtype, f"{what} {dtype} {rid}"))
    print(f"{what} {dtype}: worst error {worst:.3e}")
    return got


# ------------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("D", [48, 256, 1000])
def test_layernorm_kernel_steps(D):
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(D)
    T = 7
    h = torch.randn(T, D, generator=g).cuda() * 3 + 1
    y = torch.randn(3, T, D, generator=g).cuda()
    extra = torch.randn(T, D, generator=g).cuda()
    wa, ba, w, b = (torch.randn(D, generator=g).cuda() for _ in range(4))
    eps = 1e-5

    def ln(x, ww, bb):
        x = x.double()
        mu = x.mean(-1, keepdim=True)
        return (x - mu) / torch.sqrt(((x - mu) ** 2).mean(-1, keepdim=True) + eps) * ww.double() + bb.double()

    want_h = h.double() + ln(y.double().sum(0), wa, ba) + extra.double()
    want_out = ln(want_h, w, b)
    hh = h.clone()
    out = ops.layernorm(hh, w, b, eps, torch.float32, after=(y, wa, ba), extra=extra)
    assert (hh.double() - want_h).abs().max() < 1e-5 and (out.double() - want_out).abs().max() < 2e-5
    # each step alone, and rows picked for the last norm
    hh = h.clone()
    assert ops.layernorm(hh, None, None, eps, torch.float32, after=(y[0], wa, ba)) is None
    assert (hh.double() - (h.double() + ln(y[0], wa, ba))).abs().max() < 1e-5
    rows = torch.tensor([5, 0, 5], dtype=torch.int32).cuda()
    out = ops.layernorm(h, w, b, eps, torch.bfloat16, rows=rows)
    assert out.dtype == torch.bfloat16 and (out.double() - ln(h[rows.long()], w, b)).abs().max() < 0.05


# ------------------------------------------------------------------------------------------------- one mechanism alone
ONE = {
    "scan": pc.scan(40, 6, 3, 2),
    "scan_wide_state": pc.scan(24, 70, 4, 5),
    "scan_one_tap": pc.scan(33, 3, 1, 1),
    "latent": pc.latent(3, 8, 6, 10, 12, 200.0, 2.0),
    "latent_part_turns": pc.latent(2, 16, 8, 4, 24, 10000.0, 1.0, dims=4),
    "latent_nothing_turns": pc.latent(2, 8, 0, 8, 16, 10000.0, 1.5),
    "chunked": pc.chunked(4, 2, 8, 12, 5, 3.0),
    "chunked_one_kv_head": pc.chunked(3, 1, 16, 4, 7, 2.0),
    "chunked_wide": pc.chunked(2, 2, 40, 40, 64, 1.0),
}


@pytest.fixture(scope="module", params=sorted(ONE))
def single(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    cfg, weights = ph.make_folder(folder, pc.one_layer(ONE[name]), seed=3, init_std=0.3)
    reqs = {"long": helpers.random_tokens(330, cfg["vocab"], 1), "short": helpers.random_tokens(9, cfg["vocab"], 2),
            "one": helpers.random_tokens(1, cfg["vocab"], 3)}
    return name, folder, cfg, weights, reqs


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_whole_prompt(single, dtype):
    name, folder, cfg, weights, reqs = single
    steps, mt = helpers.schedule_whole(reqs)
    _replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_token_by_token(single, dtype):
    """Every token decoded alone from the first one on: each key is found through the cache, each state through its slot."""
    name, folder, cfg, weights, reqs = single
    reqs = {"long": reqs["long"][:150], "short": reqs["short"]}
    steps, mt = helpers.schedule_tail(reqs, tail=10 ** 6)
    _replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mechanism_alone_portions(single, dtype):
    name, folder, cfg, weights, reqs = single
    for seed in (0, 1):
        steps, mt = helpers.schedule_portions(reqs, seed=seed)
        _replay_and_compare(folder, cfg, weights, reqs, steps, mt, dtype, f"{name} portions")


def test_a_hidden_key_would_show(single):
    """The premise of the tests above: in these models one key more or less in a softmax is far beyond the tolerance.
    The plain implementation with the chunk (or the causal edge) moved by one position differs from itself."""
    name, folder, cfg, weights, reqs = single
    if "chunked" not in name:
        pytest.skip("the check is written for the chunked mask")
    other = pc.one_layer(ONE[name])
    other["layers"][0]["mixer"]["mask"]["size"] += 1
    a, b = ph.plain(cfg, weights, reqs["long"]), ph.plain(other, weights, reqs["long"])
    moved = ((a - b).abs().max(-1).values / a.abs().max()) > 3 * ph.TOL["bfloat16"]
    assert moved.float().mean() > 0.15


# ------------------------------------------------------------------------------------------------- whole models
LENGTHS = {"P1": [71, 130, 45, 96, 64, 33, 1, 58, 77], "P2": [85, 140, 37, 101, 2, 50, 90, 125, 44], "P3": [90, 257, 129, 48, 75, 40, 310, 66, 83],
           "P4": [70, 33, 131, 20, 64, 3, 95, 41, 58]}


@pytest.fixture(scope="module", params=["P1", "P2", "P3", "P4"])
def model(request, tmp_path_factory):
    name = request.param
    folder = str(tmp_path_factory.mktemp(name))
    # matrices of a smaller spread than in the models of one layer: through seven and more layer runs a sharp softmax would
    # multiply bfloat16 rounding up to the size of the faults the tests look for
    cfg, weights = ph.make_folder(folder, pc.get(name), seed=7, init_std=0.06)
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(LENGTHS[name])}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs}


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_whole(model, dtype):
    steps, mt = helpers.schedule_whole(model["requests"])
    _replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_prefill_then_decode(model, dtype):
    steps, mt = helpers.schedule_tail(model["requests"], tail=40)
    _replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " tail")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_portions(model, dtype):
    steps, mt = helpers.schedule_portions(model["requests"], seed=5)
    _replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype, model["name"] + " portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_mixed_batches_reuse_pages_and_slots(model, dtype):
    """Up to four live requests, unequal portions beside single tokens, requests that sit steps out; nine requests go
    through four slots and a pool of the live requests' size, so every slot and most pages are used again."""
    page = model["cfg"]["kv_page_size"]
    for seed in (0, 1):
        steps, mt = helpers.schedule_mixed(model["requests"], page, seed=seed, max_live=4)
        got = _replay_and_compare(model["folder"], model["cfg"], model["weights"], model["requests"], steps, mt, dtype,
                                  model["name"] + " mixed", max_requests=4)
    # and the same requests each alone: what else is in the batch changes nothing beyond rounding
    steps, mt = helpers.schedule_whole(model["requests"])
    outputs, _ = helpers.run_replay(model["folder"], dtype, steps, mt)
    alone = helpers.collect(model["requests"], steps, outputs)
    for rid in model["requests"]:
        ph.assert_close(got[rid], alone[rid], dtype, f"{model['name']} {dtype} {rid} batched against alone", tol=2 * ph.TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_many_decoding_together(model, dtype):
    page = model["cfg"]["kv_page_size"]
    reqs = {rid: t for rid, t in model["requests"].items() if len(t) > 12}
    steps, mt = helpers.schedule_wide_decode(reqs, page)
    _replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " wide decode",
                        max_requests=len(reqs))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """A short prompt and hundreds of tokens decoded one by one: chunks and pages pass over decoded tokens, the recurrent
    state runs long, the decode steps are replayed from a recorded graph."""
    reqs = {"d": helpers.random_tokens(420, model["cfg"]["vocab"], 9)}
    steps, mt = helpers.schedule_tail(reqs, tail=410)
    _replay_and_compare(model["folder"], model["cfg"], model["weights"], reqs, steps, mt, dtype, model["name"] + " long decode")


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
            logits = ph.plain(cfg, weights, toks)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < 1e-3 * float(logits.abs().max()):
                break                                  # a near-tie: float32 may pick either; the continuation is not comparable
            assert out.tokens[i] == int(logits.argmax()), f"{model['name']}: prompt of {len(prompt)}, generated token {i}"
            toks.append(out.tokens[i])
    eng.runner.manager.check()


# ------------------------------------------------------------------------------------------------- the two attention kernels
@pytest.mark.parametrize("H, Hkv, dk, dv, chunk", [(8, 2, 64, 64, 100), (16, 4, 128, 128, 512), (6, 6, 32, 16, 37), (4, 1, 16, 8, 2000)])
def test_tensor_core_mixed_heads_against_the_plain_kernel(H, Hkv, dk, dv, chunk):
    from quench6k_b200 import ops
    g = torch.Generator().manual_seed(H + dk)
    page = 16
    q_lens, starts = [90, 1, 40, 1], [0, 1234, 500, 99]
    n_pages = sum((s + n + page - 1) // page for s, n in zip(starts, q_lens))
    order = torch.randperm(n_pages, generator=g).tolist()
    tables, at = [], 0
    for s, n in zip(starts, q_lens):
        k = (s + n + page - 1) // page
        tables.append(order[at:at + k])
        at += k
    ctx = helpers.make_context(q_lens, starts, [tables])
    k_pages = (torch.randn(Hkv, n_pages, page, dk, generator=g) * 0.5).to(torch.bfloat16).cuda()
    v_pages = torch.randn(Hkv, n_pages, page, dv, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(ctx.T * H, dk, generator=g).to(torch.bfloat16).cuda()
    talk = torch.randn(H, H, generator=g).cuda()
    args = (None, q, False, k_pages, v_pages, ctx.block_tables[0], ctx.req_of_token, ctx.positions, H, 0.3)
    want = ops.attention_flex(*args, chunk=chunk, talk=talk)
    before = ops.launch_count
    got = ops.attention_flex(*args, chunk=chunk, talk=talk, tiles=ctx.query_tiles(ops.attention_flex_tile_tokens(H, Hkv)), max_context=2000)
    assert ops.launch_count - before == 2, "the tensor-core kernel did not take the shape"
    err = (got.float() - want.float()).abs().max().item() / want.float().abs().max().item()
    assert err < 2e-2, f"{err:.3e}"


@pytest.mark.parametrize("H, Hkv, da, db, dv, shared, window, chunk", [
    (16, 1, 128, 16, 128, True, None, None),        # a cached latent: values inside the key rows, part of the query in FP32
    (8, 1, 512, 64, 512, True, None, None),         # the widest rows the kernel takes
    (6, 2, 0, 32, 24, False, None, 37),             # groups that do not divide a row tile, chunks
    (4, 4, 0, 64, 64, False, 50, None),             # one head per group, a window
    (5, 1, 16, 16, 8, False, 90, 64),               # window and chunks together
])
def test_tensor_core_flexible_attention_against_the_plain_kernel(H, Hkv, da, db, dv, shared, window, chunk):
    """bfloat16 pages: the mma kernel (row tiles, with and without key ranges) against the CUDA-core kernel on the same
    data, for prompt portions that start anywhere beside single tokens deep into a context, pages in shuffled order."""
    from quench6k_b200 import ops
    from quench6k_b200.engine.batch import StepContext
    g = torch.Generator().manual_seed(H * 1000 + da + dv)
    page, dk = 16, da + db
    q_lens, starts = [70, 1, 1, 9, 33], [0, 1500, 63, 700, 250]
    n_pages = sum((s + n + page - 1) // page for s, n in zip(starts, q_lens))
    order = torch.randperm(n_pages, generator=g).tolist()
    tables, at = [], 0
    for s, n in zip(starts, q_lens):
        k = (s + n + page - 1) // page
        tables.append(order[at:at + k])
        at += k
    ctx = helpers.make_context(q_lens, starts, [tables])
    T = ctx.T
    k_pages = (torch.randn(Hkv, n_pages, page, dk, generator=g) * 0.5).to(torch.bfloat16).cuda()
    v_pages = k_pages[..., :dv] if shared else (torch.randn(Hkv, n_pages, page, dv, generator=g)).to(torch.bfloat16).cuda()
    qa = torch.randn(H * T, da, generator=g).cuda() if da else None
    qb = torch.randn(H * T, db, generator=g).to(torch.bfloat16).cuda() if db else None
    common = dict(window=window, chunk=chunk, out_head_major=True)
    want = ops.attention_flex(qa, qb, True, k_pages, v_pages, ctx.block_tables[0], ctx.req_of_token, ctx.positions, H, 0.2, **common)
    tiles = ctx.query_tiles(ops.attention_flex_tile_tokens(H, Hkv))
    for max_context in (0, max(s + n for s, n in zip(starts, q_lens))):      # 0: one key range; else fixed ranges, merged
        before = ops.launch_count
        got = ops.attention_flex(qa, qb, True, k_pages, v_pages, ctx.block_tables[0], ctx.req_of_token, ctx.positions, H, 0.2,
                                 tiles=tiles, max_context=max_context, **common)
        assert ops.launch_count - before == 2, "the tensor-core kernel did not take the shape"
        err = (got.float() - want.float()).abs().max().item() / want.float().abs().max().item()
        assert err < 2e-2, f"max_context {max_context}: {err:.3e}"


def test_command_line_generates_and_scores(model, tmp_path):
    """`generate`, `bench` and `ppl` of the command line on a Pedotar model folder: the model class comes from config.json."""
    import json
    import math
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, weights = model["cfg"], model["weights"]
    run = lambda *args: subprocess.run([sys.executable, "-m", "quench6k_b200", *args], cwd=root, capture_output=True, text=True, timeout=600)
    prompt = helpers.random_tokens(11, cfg["vocab"], 77)
    r = run("generate", "--model", model["folder"], "--prompt-ids", ",".join(map(str, prompt)), "--n", "6", "--dtype", "float32", "--context", "128")
    assert r.returncode == 0, r.stderr[-2000:]
    toks = list(prompt)
    for _ in range(6):
        toks.append(int(ph.plain(cfg, weights, toks)[-1].argmax()))
    assert "prompt: 11 tokens" in r.stdout and f"ids: {toks[11:]}" in r.stdout
    ids = helpers.random_tokens(72, cfg["vocab"], 78)
    corpus = tmp_path / "ids.txt"
    corpus.write_text(" ".join(map(str, ids)))
    out = tmp_path / "bench.jsonl"
    r = run("bench", "--model", model["folder"], "--ids", str(corpus), "--ctx", "24", "--generate", "6", "--json", str(out), "--dtype", "float32",
            "--max-batch-tokens", "10")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "graph decoding matches eager decoding (6 tokens)" in r.stdout
    assert [x["ctx"] for x in map(json.loads, out.read_text().splitlines())] == [24]
    r = run("ppl", "--model", model["folder"], "--file", str(corpus), "--ctx", "24", "--chunks", "3", "--dtype", "float32", "--max-batch-tokens", "7")
    assert r.returncode == 0, r.stderr[-2000:]
    nll, count = 0.0, 0
    for c in range(3):
        part = ids[c * 24:(c + 1) * 24]
        logits = ph.plain(cfg, weights, part)
        for p in range(12, 23):
            nll += float(torch.logsumexp(logits[p], -1) - logits[p][part[p + 1]])
            count += 1
    got = float(r.stdout.strip().splitlines()[-1].split(":")[1].split("(")[0])
    assert abs(got - math.exp(nll / count)) <= 2e-4 * got, (got, math.exp(nll / count))
