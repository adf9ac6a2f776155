"""The Sinezen decoder through the engine (its step function, cache and scheduler) against the
plain implementation, in float32 and bfloat16, for every way of cutting the work: whole prompts,
prompts then single tokens, portions of prompts down to two tokens, unequal batches, pages and
slots used again, long decoding across block edges and page borders, the first tokens, other
sizes, and greedy generation."""
import pytest
import torch

import plain_sinezen as P
import sinezen_helpers as Z
from libllm_b200.engine import GREEDY, StepItem
from replay import replay_batch

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = sorted(Z.CONFIGS)
_engines, _refs = {}, {}


def setup(name, dtype, max_tokens=4096, **kw):
    from libllm_b200.engine import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        c = Z.CONFIGS[name]
        w = Z.random_weights(c, seed=len(name) + ord(name[-1]))
        _engines[key] = (Engine.from_tensors(c, w, dtype=dtype, max_tokens=max_tokens, **kw), c, w)
    return _engines[key]


def plain(name, c, w, toks):
    key = (name, tuple(toks))
    if key not in _refs:
        _refs[key] = P.forward(c, w, toks)
    return _refs[key]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(name, dtype):
    """Lengths around the masks' edges (7, 8, 24, 33, 50, 96, 100) and the page border (64)."""
    engine, c, w = setup(name, dtype)
    for i, n in enumerate([1, 2, 3, 8, 9, 25, 34, 51, 64, 65, 101, 130, 203]):
        toks = Z.tokens(c, n, i)
        got = replay_batch(engine, [("r", toks, n)])["r"]
        Z.check_rows(got, plain(name, c, w, toks), dtype, f"{name} whole {n}", routed=Z.is_routed(c))
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens_agrees_with_the_whole_prompt(name, dtype):
    """The same request as one prompt and as a prompt followed by 40 single tokens (the single
    tokens pass block edges and a page border); also from a one-token prompt on."""
    engine, c, w = setup(name, dtype)
    for i, (n, n_prompt) in enumerate([(140, 100), (75, 35), (48, 1)]):
        toks = Z.tokens(c, n, 20 + i)
        ref = plain(name, c, w, toks)
        got = replay_batch(engine, [("r", toks, n_prompt)])["r"]
        Z.check_rows(got, ref, dtype, f"{name} {n_prompt} + {n - n_prompt} single tokens", routed=Z.is_routed(c))
        if dtype == "float32":
            whole = replay_batch(engine, [("r", toks, n)])["r"]
            assert float(Z.row_errors(got, whole).max()) < Z.TOL[dtype], f"{name}: decoding differs from the whole prompt"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_a_prompt(name, dtype):
    """A prompt brought in portions of several sizes, down to two tokens and one: a portion starts
    inside a block, at a block's first position, and at a page's."""
    engine, c, w = setup(name, dtype)
    toks = Z.tokens(c, 212, 31)
    ref = plain(name, c, w, toks)
    for sizes in ([64, 64, 64, 20], [2] * 20 + [57, 3, 100, 12], [7, 1, 42, 50, 2, 26, 70, 14], [100, 28, 72, 12]):
        assert sum(sizes) == len(toks)
        slot = engine.open_sequence()
        rows, at = [], 0
        for n in sizes:
            rows.append(torch.from_numpy(engine.step([StepItem(slot, toks[at:at + n], list(range(n)))])))
            at += n
        engine.close_sequence(slot)
        Z.check_rows(torch.cat(rows), ref, dtype, f"{name} portions {sizes[:4]}...", routed=Z.is_routed(c))
    engine.cache_check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_against_each_request_alone(name, dtype):
    """Three batches of unequal requests on a cache that holds one batch at a time, so that pages and
    slots are used again; shorter requests end earlier; each request against the plain
    implementation and, in float32, against itself alone."""
    prompts, n_dec = [1, 70, 9, 131], 12
    cap = sum((p + n_dec + 4 + 63) // 64 * 64 for p in prompts)
    engine, c, w = setup(name, dtype, max_tokens=cap)
    alone, _, _ = setup(name, dtype)
    for b in range(3):
        reqs = []
        for j, p in enumerate(prompts):
            total = p + n_dec - (j if b % 2 == 0 else 3 - j)
            reqs.append((f"b{b}r{j}", Z.tokens(c, total, 100 * b + j), p))
        got = replay_batch(engine, reqs)
        for rid, toks, p in reqs:
            Z.check_rows(got[rid], plain(name, c, w, toks), dtype, f"{name} batch {b} {rid}", routed=Z.is_routed(c))
            if dtype == "float32" and b == 0:
                single = replay_batch(alone, [(rid, toks, p)])[rid]
                assert float(Z.row_errors(got[rid], single).max()) < Z.TOL[dtype], f"{name} {rid}: the batch changes the result"
    assert engine.pages_in_use() == [0] * len(engine.pages_in_use())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Z2", "Z3"])
def test_long_decoding(name, dtype):
    """One token a step for 330 steps: blocks end and begin, pages are given back and taken."""
    engine, c, w = setup(name, dtype)
    toks = Z.tokens(c, 330, 77)
    got = replay_batch(engine, [("r", toks, 2)])["r"]
    Z.check_rows(got, plain(name, c, w, toks), dtype, f"{name} long decoding", routed=Z.is_routed(c))


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_beside_a_long_neighbour(dtype):
    engine, c, w = setup("Z1", dtype)
    short, long_ = Z.tokens(c, 3, 5), Z.tokens(c, 90, 6)
    both = replay_batch(engine, [("l", long_, 60), ("s", short, 1)])
    Z.check_rows(both["s"], plain("Z1", c, w, short), dtype, "first tokens beside a long request", routed=Z.is_routed(c))
    Z.check_rows(both["l"], plain("Z1", c, w, long_), dtype, "long neighbour", routed=Z.is_routed(c))


@pytest.mark.parametrize("name", NAMES)
def test_pages_of_finished_blocks_come_back_while_a_sequence_grows(name):
    """The groups of a block mask hold no more pages than the block and the page in hand need."""
    engine, c, w = setup(name, "float32")
    slot = engine.open_sequence()
    engine.step([StepItem(slot, Z.tokens(c, 300, 3), [299])])
    for g in engine.cache_info()["groups"]:
        if g["kind"] == "block":
            assert g["pages_in_use"] <= (g["block"] + 63) // 64 + 1, g
        else:
            assert g["pages_in_use"] == (300 + 63) // 64
    engine.close_sequence(slot)
    engine.cache_check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_cut_into_launch_sequences(dtype):
    """max_step_tokens below the prompts' lengths: the engine itself cuts inside a prompt."""
    engine, c, w = setup("Z2", dtype, max_step_tokens=48)
    reqs = [("a", Z.tokens(c, 150, 1), 150), ("b", Z.tokens(c, 30, 2), 30)]
    got = replay_batch(engine, reqs)
    for rid, toks, _ in reqs:
        Z.check_rows(got[rid], plain("Z2", c, w, toks), dtype, f"cut {rid}", routed=Z.is_routed(c))


@pytest.mark.parametrize("name", NAMES)
def test_the_last_row_alone(name):
    """A prompt of which only the last place is wanted (the last layer then runs its feed-forward
    for that row alone), and a portion of which nothing is wanted."""
    engine, c, w = setup(name, "float32")
    toks = Z.tokens(c, 77, 9)
    ref = plain(name, c, w, toks)
    slot = engine.open_sequence()
    assert engine.step([StepItem(slot, toks[:40], [])]).shape[0] == 0
    got = torch.from_numpy(engine.step([StepItem(slot, toks[40:], [36, 0])]))
    engine.close_sequence(slot)
    Z.check_rows(got, ref[[76, 40]], "float32", f"{name} chosen rows")


@pytest.mark.parametrize("name", ["Z1", "Z3"])
def test_greedy_generation_through_the_generation_loop(name):
    """engine.generate (scheduler, sampling, stop rule) in float32 against the plain implementation's
    own greedy loop, for prompts of unequal lengths in one call."""
    engine, c, w = setup(name, "float32")
    prompts = [Z.tokens(c, n, 50 + n) for n in (5, 23, 1)]
    out = engine.generate(prompts, max_new_tokens=[10, 6, 12], sampling=GREEDY, stop_tokens=[])
    for p, got, n in zip(prompts, out, (10, 6, 12)):
        seq = list(p)
        for _ in range(n):
            logits = P.forward(c, w, seq)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) < 1e-3:        # a close call is no test of anything
                break
            seq.append(int(logits.argmax()))
        want = seq[len(p):]
        assert got[:len(want)] == want, f"{name}: generated {got}, the plain loop {want}"
        assert len(got) == n


def test_the_model_folder_route_and_the_command_line_description(tmp_path):
    """Weights written as a safetensors file and loaded by folder give the engine that tensors in
    memory give; an unexpected or missing tensor is named."""
    import json
    from helpers import write_safetensors
    from libllm_b200.engine import Engine
    from libllm_b200.errors import WeightsError
    c = Z.CONFIGS["Z4"]
    w = Z.random_weights(c, 3)
    (tmp_path / "config.json").write_text(json.dumps(c))
    write_safetensors(str(tmp_path / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    engine = Engine.from_folder(str(tmp_path), dtype="float32", max_tokens=256)
    toks = Z.tokens(c, 40, 1)
    Z.check_rows(replay_batch(engine, [("r", toks, 30)])["r"], P.forward(c, w, toks), "float32", "from a folder")
    del w["l1.mlp.e2.down"]
    w["l1.mlp.e7.up"] = torch.zeros(16, 48)
    with pytest.raises(WeightsError) as e:
        Engine.from_tensors(c, w, dtype="float32", max_tokens=256)
    assert e.value.missing == ["l1.mlp.e2.down"] and e.value.unexpected == ["l1.mlp.e7.up"]


def sinezen_folder(tmp_path, name, seed):
    import json
    from helpers import write_safetensors
    c = Z.CONFIGS[name]
    w = Z.random_weights(c, seed)
    (tmp_path / "config.json").write_text(json.dumps(c))
    write_safetensors(str(tmp_path / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    return str(tmp_path), c, w


def test_the_command_line_generates_from_a_sinezen_folder(tmp_path):
    """``bin/llm generate`` picks the model by config.json's ``architecture`` and builds what it needs."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder, c, w = sinezen_folder(tmp_path, "Z4", 8)
    prompt = Z.tokens(c, 7, 800)
    out = subprocess.run([os.path.join(root, "bin", "llm"), "generate", "-m", folder, "--prompt-ids", ",".join(map(str, prompt)),
                          "--max-new-tokens", "4", "--temperature", "0", "--dtype", "float32", "--no-stop"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    got = [int(t) for t in out.stdout.strip().splitlines()[-1].split(",")]
    seq = list(prompt)
    for tok in got:
        logits = P.forward(c, w, seq)[-1]
        top2 = logits.topk(2)
        assert tok == int(top2.indices[0]) or float(top2.values[0] - top2.values[1]) < 1e-3
        seq.append(tok)
    assert len(got) == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_of_a_sinezen_folder(dtype, tmp_path):
    """``bin/trace_run`` on a folder: two unequal requests that start together and go on by single
    tokens, then a third alone that uses their slots and pages again."""
    from test_entry_points_gpu import collect, run_trace, trace_of
    folder, c, w = sinezen_folder(tmp_path, "Z2", 9)
    first = [("a", Z.tokens(c, 120, 1), 101), ("b", Z.tokens(c, 40, 2), 7)]
    steps = trace_of(first)
    steps += trace_of([("c", Z.tokens(c, 70, 3), 66)], first_step=len(steps))
    out_dir = str(tmp_path / "out")
    run_trace(folder, dtype, steps, out_dir, max_tokens=256)
    got = collect(steps, out_dir, c["vocab"])
    for rid, toks, _ in first + [("c", Z.tokens(c, 70, 3), 66)]:
        Z.check_rows(got[rid], P.forward(c, w, toks), dtype, f"trace {rid}", routed=Z.is_routed(c))
