"""Kipedra configurations drawn at random over everything config.json allows (any head counts and groups, key and value
widths that are equal or not, multiples of 16 or not, widths and vocabularies that are no multiple of 8, one to six taps,
windows from one position to longer than any prompt, rotations of none, part or all of a head, experts from two up,
every kind of feed-forward, any repeated span, pages of odd sizes), each replayed in mixed batches with reused pages and
slots in float32 and bfloat16 against the plain implementation: a size the kernels do not take must be handed to a kernel
that does, never computed wrongly."""
import random

import pytest

import helpers
import kipedra_helpers as kh

pytestmark = pytest.mark.gpu


def draw(seed, head_dim=None):
    rng = random.Random(seed)
    n_layers = rng.choice([1, 2, 3, 4])

    def feed_forward():
        kind = rng.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return {"kind": "dense", "ff": rng.choice([8, 20, 40, 72, 136])}
        experts = rng.choice([2, 3, 5, 9, 17, 40])
        return {"kind": "moe", "expert": {"ff": rng.choice([8, 12, 24, 40, 64])},
                "router": {"experts": experts, "top": rng.randint(1, min(experts, 5)), "scale": rng.choice([0.5, 1.0, 2.5])}}

    def layer():
        kv = rng.choice([1, 2, 3, 4])
        heads = kv * rng.choice([1, 2, 3, 4, 8])
        dim = head_dim or rng.choice([6, 8, 16, 24, 32, 40, 48, 64, 80, 128])
        vdim = dim if rng.random() < 0.5 else rng.choice([4, 8, 12, 16, 32, 48, 64, 128])
        while heads * max(dim, vdim) > 2048 and heads > kv:
            heads //= 2 if (heads // 2) % kv == 0 else heads // kv
            heads = max(heads, kv)
        conv = rng.choice([1, 2, 3, 4, 4, 6])
        if rng.random() < 0.45:
            return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": feed_forward()}
        dims = rng.choice([0, 2, dim // 2 // 2 * 2, dim // 2 * 2])
        return {"type": "attention",
                "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": rng.choice([0.05, 0.125, 0.3]),
                          "mask": {"size": rng.choice([1, 2, 7, 16, 30, 64, 500])}, "rot": {"base": rng.choice([50.0, 10000.0, 1e6]), "dims": dims}},
                "mlp": feed_forward()}

    cfg = {"architecture": "Kipedra", "vocab": rng.choice([17, 100, 257, 1001]), "width": rng.choice([24, 40, 72, 100, 136, 264]),
           "norm": {"eps": rng.choice([1e-6, 1e-5, 3e-4])}, "residual_mult": rng.choice([0.2, 0.5, 1.0]),
           "kv_page_size": rng.choice([1, 3, 4, 8, 16, 24, 32]), "layers": [layer() for _ in range(n_layers)]}
    if rng.random() < 0.6:
        a = rng.randint(0, n_layers - 1)
        cfg["loop"] = {"start": a, "stop": rng.randint(a, n_layers), "times": rng.choice([1, 2, 3])}
    return cfg


# the last six with the head sizes the tensor-core attention kernels take, whatever group and page sizes come with them
@pytest.mark.parametrize("seed,head_dim", [(s, None) for s in range(12)] + [(12, 64), (13, 128), (14, 64), (15, 128), (16, 128), (17, 64)])
def test_random_configuration(tmp_path, seed, head_dim):
    cfg = draw(seed, head_dim)
    cfg_d, weights = kh.make_folder(str(tmp_path), cfg, seed=seed, init_std=0.08)
    V, page = cfg["vocab"], cfg["kv_page_size"]
    rng = random.Random(100 + seed)
    reqs = {f"r{i}": helpers.random_tokens(rng.randint(3, 90), V, 7 * seed + i) for i in range(5)}
    steps, mt = helpers.schedule_mixed(reqs, page, seed=seed, max_live=3)
    for dtype in ("float32", "bfloat16"):
        kh.replay_and_compare(str(tmp_path), cfg_d, weights, reqs, steps, mt, dtype, f"configuration {seed}: {cfg}", max_requests=3)
    from quench6k_b200 import ops
    assert ops.tc_status() == 0
