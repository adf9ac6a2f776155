"""Sesuzen's configuration, its description as parts, the order of its layer runs, the state each run keeps and
the cache's books for a window that keeps its first positions: what needs no GPU.  Also the plain
implementation's small functions by hand."""
import copy

import pytest
import torch

import plain_sesuzen as P
import sesuzen_helpers as S


def describe(c, dtype="bfloat16"):
    from libllm_b200 import _lib
    return _lib.describe_model(c, dtype)


@pytest.mark.parametrize("name", sorted(S.CONFIGS))
def test_tensors_asked_for_are_the_designs_names_and_shapes(name):
    c = S.CONFIGS[name]
    d = describe(c)
    want = S.tensor_shapes(c, -1)                    # a rank the configuration does not give is left open (-1)
    assert {t["name"]: t["shape"] for t in d["tensor_needs"]} == want
    roles = {t["name"]: t["role"] for t in d["tensor_needs"]}
    assert roles["l0.norm1"] == roles["l0.norm1.b"] == roles["final.norm.b"] == roles["l0.canon1"] == "vector"
    assert roles["embed"] == roles["pos"] == roles["l0.mix.k"] == "matrix"
    assert d["capturable"]
    assert "recurrent" in d["kernel_families"]


@pytest.mark.parametrize("name", sorted(S.CONFIGS))
def test_order_of_runs(name):
    c = S.CONFIGS[name]
    sched = describe(c)["spec"]["schedule"]
    assert [e["layer"] for e in sched] == P.layer_runs(c)
    assert all(e["cache_from"] is None and e["input_mix"] is None for e in sched)


def test_loop_orders_by_hand():
    c = copy.deepcopy(S.CONFIGS["S2"])
    order = lambda: [e["layer"] for e in describe(c)["spec"]["schedule"]]
    assert order() == [0, 1, 1, 1, 2]
    c["loop"] = dict(start=0, stop=3, times=2)
    assert order() == [0, 1, 2, 0, 1, 2]
    c["loop"] = dict(start=2, stop=3, times=1)
    assert order() == [0, 1, 2]
    c["loop"] = dict(start=1, stop=1, times=5)       # an empty run of layers
    assert order() == [0, 1, 2]
    del c["loop"]
    assert order() == [0, 1, 2]


def test_every_constant_reaches_its_part():
    c = S.CONFIGS["S2"]
    spec = describe(c)["spec"]
    assert spec["position_table"] == "pos" and spec["head"] in (None, "") and spec["logit_softcap"] == 30.0
    assert spec["final_norm"] == dict(kind="layernorm", size=72, eps=1e-5, weight="final.norm", bias="final.norm.b")
    layers = spec["layers"]
    a = layers[0]["mixer"]
    assert layers[0]["kind"] == "prenorm" and layers[0]["ff"] is None and layers[0]["ff_norm"] is None
    assert layers[0]["mixer_norm"]["kind"] == "layernorm" and layers[0]["mixer_norm"]["bias"] == "l0.norm1.b"
    assert layers[0]["mixer_conv"] == dict(taps=2, weight="l0.canon1", hidden=72)
    assert (a["n_heads"], a["n_kv_heads"], a["head_dim"], a["v_head_dim"], a["window"], a["sink"], a["scale"]) == (3, 3, 24, 40, 50, 1, 0.3)
    assert a["position"] is None and a["bias"] is True and a["q_bias"] == "l0.mix.q.b" and a["v_norm"] == dict(eps=1e-5)
    assert a["out_gate"] == "l0.mix.g"
    assert "sink" not in layers[2]["mixer"] and layers[2]["mixer"]["window"] == 7          # no kept first tokens
    g = layers[1]["mixer"]
    assert (g["kind"], g["n_heads"], g["head_dim"], g["decay_rank"], g["eps"], g["key_eps"]) == ("general_delta", 3, 24, None, 1e-5, 1e-6)
    assert abs(g["decay_scale"] - 0.6065306597126334) < 1e-15 and g["a_bias"] == "l1.mix.a.b" and g["norm"] == "l1.mix.norm"
    f = layers[1]["ff"]
    assert (f["kind"], f["experts"], f["top"], f["score"], f["renormalize"], f["weight_on"]) == ("moe", 5, 1, "softmax", True, "output")
    assert f["expert"] == dict(intermediate=24, activation="silu", gate="l1.mlp.e{}.gate", up="l1.mlp.e{}.up", down="l1.mlp.e{}.down")
    d = layers[2]["ff"]
    assert (d["kind"], d["intermediate"], d["activation"]) == ("mlp", 80, "relu2")
    assert describe(S.CONFIGS["S4"])["spec"]["layers"][1]["mixer"]["decay_rank"] == 24   # given by the configuration
    full = describe(S.CONFIGS["S5"])["spec"]["layers"][1]["mixer"]
    assert full["window"] is None and "sink" not in full
    one_tap = copy.deepcopy(S.CONFIGS["S4"])
    del one_tap["canon"]
    assert "mixer_conv" not in describe(one_tap)["spec"]["layers"][0]
    assert "l0.canon1" not in {t["name"] for t in describe(one_tap)["tensor_needs"]}


def test_the_architecture_key_picks_the_model_and_faults_are_named():
    from libllm_b200.config import parse_config
    from libllm_b200.errors import ConfigError
    c = S.CONFIGS["S1"]
    n = parse_config(c)
    assert n["architecture"] == "Sesuzen" and n["layers"][1]["mixer"]["mask"] == dict(size=24, keep_first=3)
    assert parse_config(dict(c, model_type="Sesuzen"))["width"] == 64
    for change, message in [(lambda b: b["loop"].update(stop=5), "loop"),
                            (lambda b: b["layers"][1]["mlp"]["router"].update(top=9), "'top' exceeds"),
                            (lambda b: b["layers"][0]["mlp"].update(kind="sparse"), "'sparse' is not known"),
                            (lambda b: b["layers"][1]["mixer"].update(kv_heads=3), "multiple of 'kv_heads'"),
                            (lambda b: b["layers"][0].update(type="delta"), "'delta' is not known"),
                            (lambda b: b.pop("norm"), "norm"), (lambda b: b.pop("max_positions"), "max_positions")]:
        bad = copy.deepcopy(c)
        change(bad)
        with pytest.raises(ConfigError, match=message):
            parse_config(bad)


def test_cache_books_keep_the_first_pages_of_a_window_with_kept_first_positions():
    """Windows of 70 positions with pages of 64: one keeps its first 3 positions (one page), one its first 65 (two
    pages), one none; when a sequence has grown to n tokens every page that lies wholly before position
    n - 70 + 1 is free again, but for the kept ones."""
    from libllm_b200.cache import CacheBook
    need = lambda **kw: dict(n_kv_heads=1, k_dim=8, v_dim=4, **kw)
    book = CacheBook([need(kind="window", window=70, sink=3), need(kind="window", window=70), need(kind="window", window=70, sink=65),
                      need(kind="window", window=70, sink=3)], capacity_tokens=64 * 14, page_size=64)
    info = book.info()
    assert [(g["kind"], g["sink"]) for g in info["groups"]] == [("window", 3), ("window", None), ("window", 65)]
    assert info["groups"][0]["runs"] == [0, 3]
    s = book.open()
    for n in (1, 63, 64, 70, 71, 133, 134, 135, 199, 257, 300, 640):
        book.reserve({s: n})
        book.commit(s, n)
        pages = book.info()["sequences"][str(s)]["pages"]
        first = max(0, n - 70 + 1) // 64
        for group, kept in ((0, 1), (1, 0), (2, 2)):
            assert [p >= 0 for p in pages[group]] == [j >= first or j < kept for j in range((n + 63) // 64)], (n, group)
        book.check()
    t = book.open()
    book.reserve({t: 130})               # pages that the first sequence gave back are used again
    book.commit(t, 130)
    book.check()
    book.close(s)
    book.close(t)
    assert [g["pages_in_use"] for g in book.info()["groups"]] == [0, 0, 0]


def test_plain_functions_by_hand():
    m = P.window_mask(6, 2, 1)
    assert m.int().tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0], [1, 0, 1, 1, 0, 0], [1, 0, 0, 1, 1, 0],
                                [1, 0, 0, 0, 1, 1]]
    assert P.window_mask(4, None, 0).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]]
    h = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, 0.25, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)        # taps: two back, one back, itself
    out = P.time_conv(h, w)
    assert out[:, 0].tolist() == [1 + 2 * 1, 2 + 0.25 * 1 + 2 * 2, 3 + 0.5 * 1 + 0.25 * 2 + 2 * 3, 4 + 0.5 * 2 + 0.25 * 3 + 2 * 4]
    assert out[:, 1].tolist() == [10.0, 20 + 10, 30 + 20, 40 + 30]
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    ln = P.layer_norm(x, torch.full((4,), 2.0, dtype=torch.float64), torch.ones(4, dtype=torch.float64), 0.0)
    assert torch.allclose(ln, 2 * (x - 3.0) / (14.0 / 4) ** 0.5 + 1)
    # one head, two channels: the state after two tokens by hand
    one = lambda *v: torch.tensor(v, dtype=torch.float64).view(1, 1, -1)
    r, k, v = torch.cat([one(1.0, 0.0), one(0.0, 1.0)]), torch.cat([one(2.0, 0.0), one(0.0, 3.0)]), torch.cat([one(1.0, 1.0), one(1.0, -1.0)])
    decay, rate, unit = torch.full((2, 1, 2), 0.5, dtype=torch.float64), torch.full((2, 1, 2), 1.0, dtype=torch.float64), torch.cat([one(1.0, 0.0), one(0.0, 1.0)])
    o, S2 = P.delta_scan(r, k, v, decay, rate, unit)
    # token 0: S = k v^T = [[2, 2], [0, 0]], o = S^T r = [2, 2]; token 1: decay halves it, removal along e2 takes nothing,
    # k v^T adds [[0, 0], [3, -3]]; o = S^T e2 = [3, -3]
    assert o[0, 0].tolist() == [2.0, 2.0] and o[1, 0].tolist() == [3.0, -3.0]
    assert S2[0].tolist() == [[1.0, 1.0], [3.0, -3.0]]
    chosen, weight = P.route(torch.tensor([[1.0, 3.0, 3.0, 0.0]], dtype=torch.float64), 2)
    assert chosen.tolist() == [[1, 2]] and weight.tolist() == [[0.5, 0.5]]
