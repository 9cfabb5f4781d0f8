"""Helpers of the Pedotar tests: model folders with random weights and the comparison with the plain implementation."""
import json
import os

import torch

import plain_pedotar

# Relative to the largest logit of the sequence.  float32: the engine against float64 arithmetic, every position.
# bfloat16: the engine (bfloat16 operands, FP32 accumulation, FP32 where the design asks for it) against the same float64
# arithmetic on the bfloat16 weights; the test models' softmaxes are sharp on purpose, which also amplifies the rounding
# of a score now and then, so 95% of the positions of a sequence must be within TOL and all within 3 TOL (a key wrongly
# seen or hidden moves a position by 10 TOL and more, see test_a_hidden_key_would_show).  Set when the kernels first
# passed; not to be widened.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def make_folder(folder, cfg_d, seed=0, init_std=0.15, doctor=None):
    """config.json + model.safetensors with random weights; returns (config dict, {name: tensor}).  doctor(weights)
    may change tensors in place before they are written."""
    from quench6k_b200.config.pedotar import PedotarConfig
    from quench6k_b200.models.decoder import DecoderModel
    from quench6k_b200.models.pedotar import build_spec
    from quench6k_b200.weights.random_init import make_tensor
    from quench6k_b200.weights.safetensors_io import write_safetensors

    cfg = PedotarConfig.from_dict(cfg_d)
    model = DecoderModel(build_spec(cfg, norm_init="random"))
    weights = {}
    for t in model.tensors():
        w = make_tensor(t, seed, init_std)
        weights[t.name] = w.to(torch.bfloat16) if w.dtype == torch.float32 else w      # the files hold bfloat16 throughout
    if doctor is not None:
        doctor(weights)
    os.makedirs(folder, exist_ok=True)
    cfg.save(folder)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights.items())
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f), weights


def plain(cfg_d, weights, tokens):
    return plain_pedotar.forward(cfg_d, weights, tokens)


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
