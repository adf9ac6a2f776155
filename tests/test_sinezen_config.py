"""Sinezen's configuration, its description as parts, the order of its layer runs, and the cache's
books for a block mask: what needs no GPU."""
import copy

import pytest
import torch

import plain_sinezen as P
import sinezen_helpers as Z


def describe(c, dtype="bfloat16"):
    from libllm_b200 import _lib
    return _lib.describe_model(c, dtype)


@pytest.mark.parametrize("name", sorted(Z.CONFIGS))
def test_tensors_asked_for_are_the_designs_names_and_shapes(name):
    c = Z.CONFIGS[name]
    d = describe(c)
    assert {t["name"]: t["shape"] for t in d["tensor_needs"]} == Z.tensor_shapes(c)
    roles = {t["name"]: t["role"] for t in d["tensor_needs"]}
    assert roles["l0.norm1"] == roles["l0.mix.q.norm"] == roles["final.norm"] == "vector"
    assert roles["l0.mix.g"] == roles["embed"] == "matrix"
    assert d["capturable"]


@pytest.mark.parametrize("name", sorted(Z.CONFIGS))
def test_order_of_runs_and_where_the_tokens_are_mixed_in_again(name):
    c = Z.CONFIGS[name]
    sched = describe(c)["spec"]["schedule"]
    assert [(e["layer"], e["input_mix"] == "loop.in") for e in sched] == P.layer_runs(c)
    assert all(e["cache_from"] is None for e in sched)


def test_loop_orders_by_hand():
    c = copy.deepcopy(Z.CONFIGS["Z2"])
    assert [e["layer"] for e in describe(c)["spec"]["schedule"]] == [0, 1, 1, 1, 2]
    c["loop"] = dict(start=0, stop=3, times=2)
    assert [e["layer"] for e in describe(c)["spec"]["schedule"]] == [0, 1, 2, 0, 1, 2]
    c["loop"] = dict(start=2, stop=3, times=1)
    s = describe(c)["spec"]["schedule"]
    assert [e["layer"] for e in s] == [0, 1, 2] and [e["input_mix"] for e in s] == [None, None, "loop.in"]
    del c["loop"]
    s = describe(c)
    assert [e["input_mix"] for e in s["spec"]["schedule"]] == [None] * 3
    assert "loop.in" not in {t["name"] for t in s["tensor_needs"]}


def test_every_constant_reaches_its_part():
    c = Z.CONFIGS["Z2"]
    layers = describe(c)["spec"]["layers"]
    a = layers[0]["mixer"]
    assert layers[0]["kind"] == "parallel" and layers[0]["ff"] is None and layers[0]["norm"]["eps"] == 1e-5
    assert (a["n_heads"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["block"], a["scale"]) == (3, 3, 24, 40, 50, 0.3)
    assert a["position"]["rotary_dim"] == 12 and a["position"]["theta"] == 5e5 and a["qk_norm"]["eps"] == 1e-5
    assert a["head_gate"] == "l0.mix.g" and a["window"] is None
    f = layers[1]["ff"]
    assert (f["kind"], f["experts"], f["top"], f["score"], f["renormalize"], f["weight_on"]) == ("moe", 5, 1, "sigmoid", False, "input")
    assert f["expert"] == dict(intermediate=24, activation="gelu", up="l1.mlp.e{}.up", down="l1.mlp.e{}.down") and f["shared"] is None
    assert layers[2]["ff"]["kind"] == "swiglu" and layers[2]["ff"]["intermediate"] == 80
    z4 = describe(Z.CONFIGS["Z4"])["spec"]["layers"][1]["mixer"]
    assert z4["position"] is None and z4["block"] is None
    shared = describe(Z.CONFIGS["Z3"])["spec"]["layers"][1]["ff"]["shared"]
    assert shared["kind"] == "mlp" and shared["intermediate"] == 64 and shared["activation"] == "gelu"


def test_the_architecture_key_picks_the_model_and_faults_are_named():
    from libllm_b200.config import parse_config
    from libllm_b200.errors import ConfigError
    c = Z.CONFIGS["Z1"]
    n = parse_config(c)
    assert n["architecture"] == "Sinezen" and n["layers"][1]["mlp"]["shared"] == dict(ff=48)
    assert parse_config(dict(c, model_type="Sinezen"))["width"] == 64
    with pytest.raises(ConfigError, match="unexpected model type 'Sinezan'"):
        parse_config(dict(c, architecture="Sinezan"))
    bad = copy.deepcopy(c)
    bad["loop"]["stop"] = 5
    with pytest.raises(ConfigError, match="loop"):
        parse_config(bad)
    bad = copy.deepcopy(c)
    bad["layers"][1]["mlp"]["router"]["top"] = 9
    with pytest.raises(ConfigError, match="'top' exceeds"):
        parse_config(bad)
    bad = copy.deepcopy(c)
    bad["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(ConfigError, match="'sparse' is not known"):
        parse_config(bad)
    bad = copy.deepcopy(c)
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="multiple of 'kv_heads'"):
        parse_config(bad)
    bad = copy.deepcopy(c)
    del bad["norm"]
    with pytest.raises(ConfigError, match="norm"):
        parse_config(bad)


def test_cache_books_give_pages_of_finished_blocks_back():
    """A block mask of 100 positions with pages of 64: when a sequence has grown to n tokens, every
    page that lies wholly before the block of position n is free again; a window group beside it
    follows its own rule; a full group keeps everything."""
    from libllm_b200.cache import CacheBook
    need = lambda **kw: dict(n_kv_heads=1, k_dim=8, v_dim=4, **kw)
    book = CacheBook([need(kind="block", block=100), need(kind="full"), need(kind="window", window=70),
                      need(kind="block", block=100)], capacity_tokens=64 * 14, page_size=64)
    info = book.info()
    assert [g["kind"] for g in info["groups"]] == ["block", "full", "window"]
    assert info["groups"][0]["runs"] == [0, 3] and info["groups"][0]["block"] == 100
    s = book.open()
    for n in (1, 63, 64, 99, 100, 101, 199, 200, 257, 300, 640):
        book.reserve({s: n})
        book.commit(s, n)
        pages = book.info()["sequences"][str(s)]["pages"]
        first_block_page = (n // 100 * 100) // 64
        assert [p >= 0 for p in pages[0]] == [j >= first_block_page for j in range((n + 63) // 64)], n
        assert all(p >= 0 for p in pages[1])
        assert [p >= 0 for p in pages[2]] == [j >= max(0, n - 70 + 1) // 64 for j in range((n + 63) // 64)], n
        book.check()
    t = book.open()
    book.reserve({t: 130})               # pages that the first sequence gave back are used again
    book.commit(t, 130)
    book.check()
    book.close(s)
    book.close(t)
    assert [g["pages_in_use"] for g in book.info()["groups"]] == [0, 0, 0]


def test_plain_mask_and_rotation_by_hand():
    m = P.chunk_mask(torch.arange(7), torch.arange(7), 3)
    assert m.int().tolist() == [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0],
                                [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1]]
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64)
    r = P.rotate(x, torch.tensor([1]), 4, 100.0)
    a0, a1 = 1.0, 100.0 ** (-0.5)
    want = [1 * torch.cos(torch.tensor(a0)) - 3 * torch.sin(torch.tensor(a0)), 2 * torch.cos(torch.tensor(a1)) - 4 * torch.sin(torch.tensor(a1)),
            3 * torch.cos(torch.tensor(a0)) + 1 * torch.sin(torch.tensor(a0)), 4 * torch.cos(torch.tensor(a1)) + 2 * torch.sin(torch.tensor(a1)), 5.0, 6.0]
    assert torch.allclose(r[0, 0], torch.tensor([float(v) for v in want], dtype=torch.float64))
    assert torch.equal(P.rotate(x, torch.tensor([0]), 6, 9.0), x)
