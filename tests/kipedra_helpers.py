"""Helpers of the Kipedra tests: model folders with random weights and the comparison with the plain implementation."""
import json
import os

import torch

import helpers
import plain_kipedra

# Relative to the largest logit of the sequence.  float32: the engine against float64 arithmetic, every position.
# bfloat16: the engine (bfloat16 operands, FP32 accumulation, FP32 where the design asks for it) against the same float64
# arithmetic on the bfloat16 weights; 95% of the positions of a sequence must be within TOL and all within 3 TOL (the test
# models' softmaxes are sharp on purpose, which now and then amplifies the rounding of a score; a key wrongly seen or
# hidden moves a position by far more, see test_a_hidden_key_would_show).  Set when the kernels first passed; not to be widened.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def make_folder(folder, cfg_d, seed=0, init_std=0.15, doctor=None):
    """config.json + model.safetensors with random weights, the experts stored one by one; returns (config dict,
    {stored name: tensor}).  doctor(weights) may change tensors in place before they are written."""
    from quench6k_b200.config.kipedra import KipedraConfig
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.kipedra import build_spec
    from quench6k_b200.weights.random_init import make_tensor
    from quench6k_b200.weights.safetensors_io import write_safetensors

    cfg = KipedraConfig.from_dict(cfg_d)
    model = DecoderModel(build_spec(cfg, norm_init="random"))
    weights = {}
    for t in model.tensors():
        w = make_tensor(t, seed, init_std)
        w = w.to(torch.bfloat16) if w.dtype == torch.float32 else w                  # the files hold bfloat16 throughout
        if ".mlp.experts." in t.name:                                               # l<i>.mlp.experts.up -> l<i>.mlp.e<j>.up
            head, kind = t.name.split(".experts.")
            for j in range(w.shape[0]):
                weights[f"{head}.e{j}.{kind}"] = w[j].contiguous()
        else:
            weights[t.name] = w
    if doctor is not None:
        doctor(weights)
    os.makedirs(folder, exist_ok=True)
    cfg.save(folder)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights.items())
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f), weights


def plain(cfg_d, weights, tokens, forced=None):
    return plain_kipedra.forward(cfg_d, weights, tokens, forced=forced)


def assert_close(got, want, dtype, what, tol=None):
    want = want.to(torch.float64)
    got = got.to(device=want.device, dtype=torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: the engine produced non-finite logits"
    scale = float(want.abs().max())
    per_pos = (got - want).abs().reshape(want.shape[0], -1).max(dim=-1).values / scale
    worst = int(per_pos.argmax())
    limit = tol if tol is not None else TOL[dtype]
    if dtype == "bfloat16":
        over = int((per_pos > limit).sum())
        assert over <= 0.05 * len(per_pos) and float(per_pos[worst]) <= 3 * limit, (
            f"{what}: {over} of {len(per_pos)} positions beyond {limit:.1e}, the worst {float(per_pos[worst]):.3e} of scale {scale:.3f} at position {worst}")
        return float(per_pos[worst])
    assert float(per_pos[worst]) <= limit, (f"{what}: error {float(per_pos[worst]):.3e} of scale {scale:.3f} at position {worst} exceeds "
                                            f"{limit:.1e} ({int((per_pos > limit).sum())} of {len(per_pos)} positions do)")
    return float(per_pos[worst])


def replay_and_compare(folder, cfg, weights, requests, steps, max_tokens, dtype, what, page=None, max_requests=4):
    """Replays the steps through the engine and compares every request with the plain implementation.  A mixture of experts
    is discontinuous (a rounding that flips a near-tie of two choice scores moves a position by far more than rounding), so
    the engine reports the experts it chose and the plain implementation is run on those; how often its own choice would
    have differed is counted and must stay rare."""
    routed = any(L.get("mlp") and L["mlp"]["kind"] == "moe" for L in cfg["layers"])
    outputs, runner = helpers.run_replay(folder, dtype, steps, max_tokens, page_size=page, max_requests=max_requests, tap=routed)
    got = helpers.collect(requests, steps, outputs)
    worst, flips, positions = 0.0, 0, 0
    for rid, toks in requests.items():
        forced = runner.routing[rid]["experts"] if routed else None
        want = plain(cfg, weights, toks, forced)
        if routed:
            own = plain_kipedra.forward(cfg, weights, toks)
            del own
            for p, chosen in plain_kipedra.forward.chosen.items():
                flips += int((chosen.sort(-1).values != forced[p].sort(-1).values).any(-1).sum())
                positions += len(toks)
        worst = max(worst, assert_close(got[rid], want, dtype, f"{what} {dtype} {rid}"))
    assert flips <= (0.002 if dtype == "float32" else 0.05) * positions + 1, f"{what} {dtype}: {flips} of {positions} choices of experts differ"
    print(f"{what} {dtype}: worst error {worst:.3e}, {flips} of {positions} choices of experts differ")
    return got
