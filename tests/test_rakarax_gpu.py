"""Rakarax through the engine against the plain implementation: every mechanism alone and together, whole prompts,
decoding token by token, prompts in portions, batches of unequal requests with slots and pages used again, long
decoding past every window, states that last for hundreds of tokens, sharp softmaxes at the windows' edges, and greedy
generation through the library's entry points and programs."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import engine_replay as replay
import plain_rakarax as plain
import rakarax_configs as rc
from burn_transformers_b200 import (AutoCausalLm, AutoLoadOptions, CausalGenerationRequest, Engine, GenerationConfig,
                                    StepEntry, generate_causal)

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
# (16-bit: these models are a few dozen channels wide, so one rounding moves a logit by about a hundredth of the
# largest; the worst position may reach a tenth, the typical one stays far below)
TOL = {"float32": 1e-4, "bfloat16": 1e-1}
TYPICAL_16 = 2.5e-2
# lengths around the borders of a page (64), of the recurrences' staging (16) and chunks (64), and of the windows
LENGTHS = {"mixed": [1, 2, 7, 39, 41, 64, 65, 101, 129, 260], "odd": [1, 33, 34, 64, 130], "odder": [1, 2, 66, 150],
           "large": [1, 70, 71, 200], "only_left": [1, 5, 50, 51, 64, 140], "only_right": [1, 5, 64, 97, 200],
           "only_retention": [1, 5, 64, 65, 97, 200], "only_feed_forward": [1, 5, 70]}


def assert_close(got, ref, dtype, tol=None, note=""):
    tol = TOL[dtype] if tol is None else tol
    err, where = replay.worst_error(got, ref)
    assert err < tol, f"{note}{err:.3e} at {where}"
    if dtype == "bfloat16":
        each = [float(np.abs(row - ref[r][p]).max() / np.abs(ref[r]).max()) for (r, p), row in got.items()]
        assert np.median(each) < TYPICAL_16, f"{note}median {np.median(each):.3e}"


@pytest.fixture(scope="module", params=list(rc.CONFIGS))
def case(request, tmp_path_factory):
    name = request.param
    config = rc.CONFIGS[name]
    folder = rc.make_folder(tmp_path_factory.mktemp(name), config, seed=21)
    pcfg, pw = rc.load_plain(folder)
    seqs = rc.prompts(config, LENGTHS[name], seed=2)
    return name, folder, seqs, [plain.forward(pcfg, pw, s) for s in seqs]


def engine_for(folder, dtype, max_tokens=64 * 16, **kw):
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_request_whole(case, dtype):
    _, folder, seqs, ref = case
    got = replay.whole(engine_for(folder, dtype), seqs)
    assert len(got) == sum(len(s) for s in seqs)
    assert_close(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_tokens_one_by_one(case, dtype):
    _, folder, seqs, ref = case
    got = replay.tail_one_by_one(engine_for(folder, dtype), seqs, tail=45)
    assert_close(got, ref, dtype)


def in_portions(engine, seqs, size):
    """Each request alone, `size` tokens a step."""
    got = {}
    for r, seq in enumerate(seqs):
        slot = engine.new_sequence()
        for lo in range(0, len(seq), size):
            piece = seq[lo:lo + size]
            logits = engine.step([StepEntry(slot, piece, list(range(len(piece))))]).detach().cpu().double().numpy()
            for i, row in enumerate(logits):
                got[(r, lo + i)] = row
        engine.release(slot)
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [2, 3, 15, 25, 70])
def test_prompts_in_portions(case, dtype, size):
    """Portions as long as every window's ring of pages allows (a ring keeps one window and one run of new tokens);
    the convolutions' taps, the scans' states and the pages carry a sequence from one portion to the next."""
    name, folder, seqs, ref = case
    if name not in ("mixed", "only_right", "only_retention") and size in (3, 15, 70):
        pytest.skip("the full set of portion sizes runs on three configurations")
    engine = engine_for(folder, dtype)
    limit = engine.cache.max_continued_run
    if limit is not None and size > limit:
        pytest.skip(f"a window of this model lets a sequence go on by {limit} tokens a step")
    got = in_portions(engine, seqs, size)
    assert_close(got, ref, dtype, note=f"portions of {size}: ")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests_use_slots_and_pages_again(case, dtype):
    _, folder, seqs, ref = case
    n = len(seqs)
    groups = [list(range(0, n, 2)), list(range(1, n, 2)), list(range(n))[:3], list(range(n))[::-1][:3]]
    cut = [max(1, len(s) // 3) for s in seqs]
    cut[0] = 1
    need = max(sum(-(-len(seqs[r]) // 64) * 64 for r in g) for g in groups)
    engine = engine_for(folder, dtype, max_tokens=need, max_slots=max(len(g) for g in groups))
    got = replay.batches(engine, seqs, groups, cut)
    assert_close(got, ref, dtype)
    assert engine.cache.slots.held == 0 and all(g.pool.held == 0 for g in engine.cache.groups)
    if dtype == "float32":
        # a request's logits do not depend on what else is in the batch
        alone = replay.whole(engine, seqs)
        drift = max(float(np.abs(alone[k] - got[k]).max() / np.abs(ref[k[0]]).max()) for k in got)
        assert drift < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(case, dtype):
    """Every token decoded alone: the windows pass over decoded tokens, the rings of pages come round, the
    convolutions start from their zero state."""
    _, folder, seqs, ref = case
    long = max(range(len(seqs)), key=lambda r: len(seqs[r]))
    got = replay.tail_one_by_one(engine_for(folder, dtype), [seqs[long]], tail=10 ** 6)
    assert len(got) == len(seqs[long])
    assert_close({(long, p): row for (_, p), row in got.items()}, ref, dtype)


def test_a_released_slot_starts_from_an_empty_state(case):
    """A sequence that takes over a slot finds neither the old states, nor the old taps, nor the old keys."""
    _, folder, seqs, ref = case
    engine = engine_for(folder, "float32", max_tokens=64 * 5, max_slots=1)
    for r in (len(seqs) - 1, 1, len(seqs) - 2):
        slot = engine.new_sequence()
        assert slot == 0
        got = engine.step([StepEntry(slot, seqs[r], [len(seqs[r]) - 1])]).cpu().double().numpy()[0]
        engine.release(slot)
        assert np.abs(got - ref[r][-1]).max() / np.abs(ref[r]).max() < TOL["float32"], r


@pytest.mark.parametrize("name", ["mixed", "only_left", "odd"])
def test_sharp_softmaxes_at_the_windows_edges(name, tmp_path):
    """Scores scaled up eightfold: a row's weight sits on one or two keys anywhere in its window, the oldest one it may
    see as often as any other, so a window that is one token too short or too long, or a key lost where the ring of
    pages comes round, moves the logits visibly; in prompts, in decoding, and in a batch.  32-bit only."""
    config = rc.sharp(rc.CONFIGS[name])
    folder = rc.make_folder(tmp_path, config, seed=8)
    pcfg, pw = rc.load_plain(folder)
    seqs = rc.prompts(config, [290, 131], seed=6)
    ref = [plain.forward(pcfg, pw, s) for s in seqs]
    engine = engine_for(folder, "float32")
    for got in (replay.whole(engine, seqs), replay.tail_one_by_one(engine, seqs, tail=120),
                replay.batches(engine, seqs, [[0, 1]], [150, 3])):
        err, where = replay.worst_error(got, ref)
        assert err < 3e-4, f"{err:.3e} at {where}"


def test_the_window_is_exact(tmp_path):
    """One loud key: a token whose key every later query prefers by far, whatever the distance.  It carries the softmax
    exactly while it is among the last `window` tokens, the plain implementation says, and not one position longer."""
    config = rc.ONLY_LEFT
    window = config["layers"][0]["mixer"]["left"]["mask"]["size"]
    heads = config["layers"][0]["mixer"]["left"]["heads"]

    def loud(tensors):
        # channel 1 of the stream is the same large number for every token, and all queries read it, so every query
        # points the same way; keys read channel 0, which is zero for every token but token 7, so only that token's
        # key points the queries' way and all others point anywhere (a head's norm keeps directions only).  The
        # convolutions pass the current token only, the heads do not talk, and the scores (scaled up with their cap)
        # outweigh the distance's bias
        tensors["embed"][:, 1] = 5.0
        tensors["embed"][:, 0] = 0.0
        tensors["embed"][7] = 0.0
        tensors["embed"][7, 0], tensors["embed"][7, 1] = 30.0, 5.0
        tensors["pos"] = tensors["pos"] * 0.05
        tensors["pos"][:, 0] = 0.0
        tensors["l0.norm1"][:2] = 0.0
        tensors["l0.mix.left.q"] = tensors["l0.mix.left.q"] * 0.02
        tensors["l0.mix.left.k"] = tensors["l0.mix.left.k"] * 0.02
        tensors["l0.mix.left.q"][:, 1] = 4.0
        tensors["l0.mix.left.k"][:, 0] = 3.0
        for name in ("l0.mix.left.q.conv", "l0.mix.left.k.conv"):
            tensors[name][:, :-1] = 0.0
            tensors[name][:, -1] = 1.0
        tensors["l0.mix.left.talk"] = np.eye(heads)
        tensors["l0.mix.left.temp"][:] = 1.0
        return tensors

    config = rc.sharp(config, 20.0)
    folder = rc.make_folder(tmp_path, config, seed=5, edit=loud)
    pcfg, pw = rc.load_plain(folder)
    rng = np.random.default_rng(3)
    seq = rng.integers(8, config["vocab"], 3 * window + 20).tolist()
    seq[10] = 7
    seq[window + 30] = 7
    ref = plain.forward(pcfg, pw, seq)
    # the plain implementation itself sees the edge: the logits jump where the loud key leaves the window
    jump = np.abs(ref[10 + window] - ref[10 + window - 1]).max()
    assert jump > 100 * TOL["float32"] * np.abs(ref).max()
    engine = engine_for(folder, "float32")
    for got in (replay.whole(engine, [seq]), replay.tail_one_by_one(engine, [seq], tail=2 * window + 5),
                in_portions(engine, [seq], 9)):
        err, where = replay.worst_error(got, [ref])
        assert err < TOL["float32"], f"{err:.3e} at {where}"


@pytest.mark.parametrize("name", ["mixed", "only_right", "only_retention"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_states_that_last(name, dtype, tmp_path):
    """Small steps and slow decays: the first tokens still count after hundreds, through prompts, decoding, portions and
    batches; a state that is dropped or handed to another sequence shows everywhere after."""
    config = rc.CONFIGS[name]
    folder = rc.make_folder(tmp_path, config, seed=11, edit=rc.long_memory)
    pcfg, pw = rc.load_plain(folder)
    seqs = rc.prompts(config, [330, 70, 150], seed=4)
    ref = [plain.forward(pcfg, pw, s) for s in seqs]
    # the memory is long: the same tokens after another beginning give other logits at the end
    other = [(t + 1) % config["vocab"] for t in seqs[0][:20]] + seqs[0][20:]
    if name != "mixed":
        assert np.abs(plain.forward(pcfg, pw, other)[-1] - ref[0][-1]).max() > 20 * TOL["float32"] * np.abs(ref[0]).max()
    engine = engine_for(folder, dtype)
    for got in (replay.whole(engine, seqs), replay.tail_one_by_one(engine, seqs, tail=50), in_portions(engine, seqs, 2),
                replay.batches(engine, seqs, [[0, 1, 2], [2, 0]], [200, 5, 66])):
        assert_close(got, ref, dtype)


def plain_greedy(pcfg, pw, prompt, n):
    seq = list(prompt)
    margins = []
    for _ in range(n):
        row = plain.forward(pcfg, pw, seq)[-1]
        order = np.argsort(row)
        margins.append(float(row[order[-1]] - row[order[-2]]))
        seq.append(int(order[-1]))
    return seq[len(prompt):], margins


def test_greedy_generation_through_the_entry_point(tmp_path):
    """Three unequal prompts as one batch through load_local and generate_causal (the scheduler, the recorded decode
    steps, the device sampler): the plain implementation's tokens."""
    folder = rc.make_folder(tmp_path, rc.MIXED, seed=13)
    pcfg, pw = rc.load_plain(folder)
    prompts = rc.prompts(rc.MIXED, [3, 70, 18], seed=9)
    want = [plain_greedy(pcfg, pw, p, 12) for p in prompts]
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="float32", max_tokens=64 * 4))
    out = generate_causal(loaded.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=12)))
    for sequence, (tokens, margins) in zip(out.sequences, want):
        # (compared up to the first step the plain implementation itself decides by less than rounding can move)
        sure = next((i for i, m in enumerate(margins) if m < 1e-3), len(tokens))
        assert sequence.token_ids[:sure] == tokens[:sure] and sure >= 4
    bf16 = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="bfloat16", max_tokens=64 * 4))
    out16 = generate_causal(bf16.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=12)))
    assert all(len(s.token_ids) == 12 for s in out16.sequences)
    assert sum(a == b for s, (t, _) in zip(out16.sequences, want) for a, b in zip(s.token_ids, t)) >= 18


def test_the_programs_serve_the_model(tmp_path):
    """bin/random_model writes a folder from a configuration file, bin/generate decodes from it, bin/trace_run replays a
    batch of two unequal requests on it."""
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(rc.ODD))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, str(ROOT / "bin" / "random_model"), str(cfg_file), str(folder), "--seed", "4"],
                          capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr
    pcfg, pw = rc.load_plain(folder)
    done = subprocess.run([str(ROOT / "bin" / "generate"), str(folder), "5,6,7,8", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr
    ids = [int(x) for x in done.stdout.split()]
    tokens, margins = plain_greedy(pcfg, pw, [5, 6, 7, 8], 6)
    sure = next((i for i, m in enumerate(margins) if m < 1e-3), 6)
    assert ids[:4] == [5, 6, 7, 8] and ids[4:4 + sure] == tokens[:sure]
    a, b = rc.prompts(rc.ODD, [70, 9], seed=1)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:2], "want": []}],
              "end": []}]
    for i in range(7):
        live = [("a", a, 66 + i)] * (66 + i < len(a)) + [("b", b, 2 + i)]
        steps.append({"step": i + 1, "entries": [{"id": r, "tokens": [s[p]], "want": [0]} for r, s, p in live],
                      "end": [r for r, s, p in live if p + 1 == len(s)]})
    out = tmp_path / "out"
    run = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                          "--max-tokens", "79"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=900, env=dict(os.environ))
    assert run.returncode == 0, run.stderr
    assert run.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    ref = {"a": plain.forward(pcfg, pw, a), "b": plain.forward(pcfg, pw, b)}
    first = np.frombuffer((out / "0.f32").read_bytes(), dtype="<f4").reshape(2, -1)
    assert np.abs(first[1] - ref["a"][65]).max() / np.abs(ref["a"]).max() < 1e-4
    last = np.frombuffer((out / "7.f32").read_bytes(), dtype="<f4").reshape(1, -1)
    assert np.abs(last[0] - ref["b"][8]).max() / np.abs(ref["b"]).max() < 1e-4
