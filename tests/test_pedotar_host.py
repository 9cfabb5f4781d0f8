"""Host-side tests of the Pedotar architecture: configuration, execution order, tensor declaration, the architecture
registry, and the cache group of a chunked mask in both cache managers.  No GPU."""
import json

import pytest
import torch

import pedotar_configs
import plain_pedotar
from quench6k_b200.cache.manager import CacheManager as PyCacheManager, GroupSpec, OutOfPages
from quench6k_b200.cache.native import NativeCacheManager
from quench6k_b200.config.pedotar import ConfigError, PedotarConfig
from quench6k_b200.config.registry import architecture_of, load_config
from quench6k_b200.models.decoder import DecoderModel
from quench6k_b200.models.pedotar import build_spec


@pytest.mark.parametrize("name", ["P1", "P2", "P3", "P4"])
def test_config_round_trip_and_order(name, tmp_path):
    d = pedotar_configs.get(name)
    cfg = PedotarConfig.from_dict(d)
    cfg.save(str(tmp_path))
    arch, again = load_config(str(tmp_path))
    assert arch.name == "Pedotar" and again.to_dict() == cfg.to_dict()
    order, readd = cfg.execution()
    plain = plain_pedotar.executed_layers(d)
    assert order == [i for i, _ in plain]
    assert readd == [p for p, (_, again_) in enumerate(plain) if again_]


def test_execution_order_cases():
    base = pedotar_configs.get("P1")
    for loop, order, readd in [({"start": 1, "stop": 3, "times": 3}, [0, 1, 2, 1, 2, 1, 2], [3, 5]),
                               ({"start": 0, "stop": 3, "times": 2}, [0, 1, 2, 0, 1, 2], [3]),
                               ({"start": 0, "stop": 1, "times": 1}, [0, 1, 2], []),
                               ({"start": 2, "stop": 2, "times": 4}, [0, 1, 2], []),
                               (None, [0, 1, 2], [])]:
        d = dict(base)
        if loop is None:
            d.pop("loop")
        else:
            d["loop"] = loop
        assert PedotarConfig.from_dict(d).execution() == (order, readd)


def test_registry_reads_either_key():
    assert architecture_of({"architecture": "Pedotar"}).name == "Pedotar"
    assert architecture_of({"architectures": ["Pedotar"]}).name == "Pedotar"
    assert architecture_of({"architectures": ["FlintForCausalLM"]}).name == "FlintForCausalLM"


@pytest.mark.parametrize("breakage, text", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["layers"][0].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda d: d["layers"][1].update(mlp={"kind": "moe", "ff": 8}), "mlp"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d["layers"][2]["mixer"]["rot"].update(dims=7), "rotating"),
])
def test_config_errors_name_the_key(breakage, text):
    d = pedotar_configs.get("P1")
    breakage(d)
    with pytest.raises(ConfigError, match=text):
        PedotarConfig.from_dict(d)


def test_declared_tensors():
    d = pedotar_configs.get("P1")
    model = DecoderModel(build_spec(PedotarConfig.from_dict(d)))
    names = {t.name: tuple(t.shape) for t in model.tensors()}
    assert names["embed"] == (211, 96) and names["final.norm"] == (96,) and names["final.norm.b"] == (96,)
    assert names["l0.mix.talk"] == (6, 6) and names["l0.mix.v"] == (2 * 24, 96) and names["l0.mix.o"] == (96, 6 * 24)
    assert names["l0.mix.q.norm"] == (16,) and "l0.norm2" not in names and "l0.mlp.gate" not in names
    assert names["l1.mix.in"] == (160, 96) and names["l1.mix.x"] == (3 + 2 * 5, 80) and names["l1.mix.conv"] == (80, 4)
    assert names["l1.mix.dt"] == (80, 3) and names["l1.mix.A_log"] == (80, 5) and names["l1.norm2b.b"] == (96,)
    assert names["l2.mix.q"] == (3 * 16, 96) and names["l2.mix.dkv"] == (28, 96) and names["l2.mix.dkv.norm"] == (20,)
    assert names["l2.mix.uk"] == (24, 20) and names["l2.mix.uv"] == (36, 20) and names["l2.mix.o"] == (96, 36)
    # every executed position has a cache or a state of its own
    assert len(model.cache_requests()) == 7 and len(model.state_shapes()) == 7
    assert [r.kind if r else None for r in model.cache_requests()] == ["chunked", None, "full", None, "full", None, "full"]
    assert model.state_shapes()[1] == {"ssm": ((80, 5), torch.float32), "conv": ((3, 80), torch.float32)}


# --------------------------------------------------------------------------------------------- the chunked cache group
@pytest.fixture(params=[PyCacheManager, NativeCacheManager], ids=["python", "native"])
def manager_cls(request):
    return request.param


def test_chunked_group_gives_back_what_a_chunk_start_hides(manager_cls):
    page, size = 4, 10
    m = manager_cls([GroupSpec("chunked", size), GroupSpec("full")], page, [8, 64], 2)
    m.add("a")
    length = 0
    for n in (3, 6, 1, 1, 9, 2, 17, 1, 30):
        m.reserve("a", n)
        m.commit("a")
        length += n
        m.check()
        table = m.table("a", 0)
        first_seen = length // size * size                 # the next query's first visible key
        for b, p in enumerate(table):
            wholly_hidden = (b + 1) * page <= first_seen
            assert (p < 0) == wholly_hidden, f"length {length}: block {b} page {p}"
        assert all(p >= 0 for p in m.table("a", 1))
    m.remove("a")
    assert m.pools[0].num_free == 8 and m.pools[1].num_free == 64


def test_chunked_group_pool_of_a_chunk_suffices_for_single_tokens(manager_cls):
    page, size = 4, 10
    m = manager_cls([GroupSpec("chunked", size)], page, [4], 1)       # ceil(10 / 4) + 1 pages
    m.add("a")
    for _ in range(200):
        m.reserve("a", 1)
        m.commit("a")
    m.check()
    with pytest.raises(OutOfPages):
        m.reserve("a", 40)                               # a portion that spans more chunks than the pool holds
    m.remove("a")


def test_group_spec_rejects_a_chunk_without_size():
    with pytest.raises(ValueError):
        GroupSpec("chunked")
    with pytest.raises(ValueError):
        GroupSpec("striped", 4)
