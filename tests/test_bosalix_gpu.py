"""Bosalix through the engine against the plain implementation: every mechanism alone and together, whole prompts,
decoding token by token, prompts in portions down to two tokens, batches of unequal requests with slots and pages used
again, long decoding past every window, sharp scores at the windows' edges and at the kept first positions, one loud key
that shows each edge exactly, and greedy generation through the library's entry points and programs."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import bosalix_configs as bc
import engine_replay as replay
import plain_bosalix as plain
from burn_transformers_b200 import (AutoCausalLm, AutoLoadOptions, CausalGenerationRequest, Engine, GenerationConfig,
                                    StepEntry, generate_causal)

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
# 32-bit: every position.  16-bit: these models are a few dozen channels wide, so one rounding moves a logit by about a
# hundredth of the largest; and where two experts' scores lie closer than rounding, the 16-bit model may choose the
# other one at that token, so the bound holds for all but a few positions in a hundred, the typical one stays far below
TOL = {"float32": 1e-4, "bfloat16": 1e-1}
TYPICAL_16 = 2.5e-2
# lengths around the borders of a page (64), of the attention kernels' tiles (32) and of the windows
LENGTHS = {"mixed": [1, 2, 7, 39, 41, 64, 65, 101, 129, 260], "odd": [1, 9, 33, 64, 130], "large": [1, 70, 71, 200],
           "only_sigmoid": [1, 5, 50, 51, 64, 140], "only_latent": [1, 5, 50, 51, 64, 140], "only_experts": [1, 5, 70],
           "value_mixing": [1, 31, 97]}


def assert_close(got, ref, dtype, tol=None, note=""):
    tol = TOL[dtype] if tol is None else tol
    each = [float(np.abs(row - ref[r][p]).max() / np.abs(ref[r]).max()) for (r, p), row in got.items()]
    if dtype == "float32":
        err, where = replay.worst_error(got, ref)
        assert err < tol, f"{note}{err:.3e} at {where}"
    else:
        assert np.quantile(each, 0.95) < tol, f"{note}95th percentile {np.quantile(each, 0.95):.3e}"
        assert np.median(each) < TYPICAL_16, f"{note}median {np.median(each):.3e}"


@pytest.fixture(scope="module", params=list(bc.CONFIGS))
def case(request, tmp_path_factory):
    name = request.param
    config = bc.CONFIGS[name]
    folder = bc.make_folder(tmp_path_factory.mktemp(name), config, seed=21)
    pcfg, pw = bc.load_plain(folder)
    seqs = bc.prompts(config, LENGTHS[name], seed=2)
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
    """The pages, the row a token shift keeps, and the positions carry a sequence from one portion to the next; the
    values a later layer blends in are those of the portion's own tokens."""
    name, folder, seqs, ref = case
    if name not in ("mixed", "value_mixing", "large") and size in (3, 15, 70):
        pytest.skip("the full set of portion sizes runs on three configurations")
    engine = engine_for(folder, dtype)
    assert engine.cache.max_continued_run is None
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
    """Every token decoded alone: the windows pass over decoded tokens, the kept first positions are decoded ones, the
    token shift starts from its zero state."""
    _, folder, seqs, ref = case
    long = max(range(len(seqs)), key=lambda r: len(seqs[r]))
    got = replay.tail_one_by_one(engine_for(folder, dtype), [seqs[long]], tail=10 ** 6)
    assert len(got) == len(seqs[long])
    assert_close({(long, p): row for (_, p), row in got.items()}, ref, dtype)


def test_a_released_slot_starts_from_an_empty_state(case):
    """A sequence that takes over a slot finds neither the row the token shift kept nor the old keys."""
    _, folder, seqs, ref = case
    engine = engine_for(folder, "float32", max_tokens=64 * 5, max_slots=1)
    for r in (len(seqs) - 1, 1, len(seqs) - 2):
        slot = engine.new_sequence()
        assert slot == 0
        got = engine.step([StepEntry(slot, seqs[r], [len(seqs[r]) - 1])]).cpu().double().numpy()[0]
        engine.release(slot)
        assert np.abs(got - ref[r][-1]).max() / np.abs(ref[r]).max() < TOL["float32"], r


def test_the_token_shift_reads_the_row_before(tmp_path):
    """With shift weights of one the mixer reads the token before only: the logits at a position then do not depend on
    that position's own token through the mixer, and the engine agrees with the plain implementation about it through
    prompts, single tokens and portions."""
    def all_shift(tensors):
        tensors["l0.shift"][:] = 1.0
        return tensors
    folder = bc.make_folder(tmp_path, bc.ONLY_SIGMOID, seed=4, edit=all_shift)
    pcfg, pw = bc.load_plain(folder)
    seq, = bc.prompts(bc.ONLY_SIGMOID, [70], seed=3)
    ref = plain.forward(pcfg, pw, seq)
    engine = engine_for(folder, "float32")
    for got in (replay.whole(engine, [seq]), replay.tail_one_by_one(engine, [seq], tail=69), in_portions(engine, [seq], 2)):
        err, where = replay.worst_error(got, [ref])
        assert err < TOL["float32"], f"{err:.3e} at {where}"


@pytest.mark.parametrize("name", ["mixed", "only_sigmoid", "only_latent", "odd"])
def test_sharp_scores_at_the_windows_edges(name, tmp_path):
    """Scores scaled up eightfold: a softmax row's weight sits on one or two keys anywhere in its window and a sigmoid is
    nearly a step, so a window that is one token too short or too long, a kept position too few or too many, or a key
    lost at a page's border moves the logits visibly; in prompts, in decoding, and in a batch.  32-bit only."""
    config = bc.sharp(bc.CONFIGS[name])
    folder = bc.make_folder(tmp_path, config, seed=8)
    pcfg, pw = bc.load_plain(folder)
    seqs = bc.prompts(config, [290, 131], seed=6)
    ref = [plain.forward(pcfg, pw, s) for s in seqs]
    engine = engine_for(folder, "float32")
    for got in (replay.whole(engine, seqs), replay.tail_one_by_one(engine, seqs, tail=120),
                replay.batches(engine, seqs, [[0, 1]], [150, 3]), in_portions(engine, seqs, 37)):
        err, where = replay.worst_error(got, ref)
        assert err < 3e-4, f"{err:.3e} at {where}"


def _loud_key(tensors, prefix, q_name, k_name, quiet):
    """Token 7's key stands out for every query: channel 1 of the stream is the same large number for every token and
    all queries read it; keys read channel 0, which is zero for every token but token 7."""
    tensors["embed"][:, 1] = 5.0
    tensors["embed"][:, 0] = 0.0
    tensors["embed"][7] = 0.0
    tensors["embed"][7, 0], tensors["embed"][7, 1] = 30.0, 5.0
    tensors["l0.shift"][:] = 0.0
    for name in quiet:
        tensors[prefix + name] = tensors[prefix + name] * 0.02
    tensors[prefix + q_name][:, 1] = 4.0
    tensors[prefix + k_name][:, 0] = 3.0
    return tensors


def _loud_latent(tensors):
    """The same for a latent attention: every query's latent points one way, so does token 7's key latent, and equal
    positive up-projections carry both into keys and queries that agree; the rotated key part stays an ordinary one."""
    tensors = _loud_key(tensors, "l0.mix.", "dq", "dkv", ("dq", "dkv"))
    rank = tensors["l0.mix.dkv.norm"].shape[0]
    tensors["l0.mix.dkv"][rank:, 0] = 0.0
    tensors["l0.mix.dq.norm"] = np.abs(tensors["l0.mix.dq.norm"]) + 0.5
    tensors["l0.mix.dkv.norm"] = np.abs(tensors["l0.mix.dkv.norm"]) + 0.5
    tensors["l0.mix.uq"][:] = 0.05
    tensors["l0.mix.uk"][:] = 0.1
    return tensors


@pytest.mark.parametrize("kind", ["sigmoid", "latent"])
def test_the_window_and_the_kept_positions_are_exact(kind, tmp_path):
    """One loud key, several times in a sequence: at the last kept first position of the sigmoid attention and at the first
    that is not kept, and at position `window` + 30.  The plain implementation says where its weight ends: `window`
    positions later and not one sooner or later (for the kept one: never).  Whole prompts, decoding and portions agree
    with it."""
    if kind == "sigmoid":
        config = bc.sharp(bc.ONLY_SIGMOID, 6.0)

        def edit(t):
            t = _loud_key(t, "l0.mix.", "q", "k", ("q", "k"))
            t["l0.mix.q.b"][:] = 0.0
            t["l0.mix.k.b"][:] = 0.0
            t["l0.mix.pb"][:] = -12.0        # (a key that does not stand out weighs next to nothing)
            return t
    else:
        config = bc.sharp(bc.ONLY_LATENT, 20.0)

        edit = _loud_latent
    window = config["layers"][0]["mixer"]["mask"]["size"]
    folder = bc.make_folder(tmp_path, config, seed=5, edit=edit)
    pcfg, pw = bc.load_plain(folder)
    rng = np.random.default_rng(3)
    seq = rng.integers(8, config["vocab"], 3 * window + 20).tolist()
    keep = config["layers"][0]["mixer"]["mask"].get("keep_first", 0)
    early = [keep - 1, keep] if kind == "sigmoid" else [2]      # the last kept position and the first that is not
    for at in early + [window + 30]:
        seq[at] = 7
    ref = plain.forward(pcfg, pw, seq)
    big = 100 * TOL["float32"] * np.abs(ref).max()

    def without(at):
        other = list(seq)
        other[at] = 9
        return plain.forward(pcfg, pw, other)
    # the plain implementation itself sees the edges: with another token in a loud one's place the logits differ up to
    # the last position of its window and not at the next; a kept position counts for ever
    alt = without(window + 30)
    edge = 2 * window + 30
    assert np.abs(alt[edge - 1] - ref[edge - 1]).max() > big and np.abs(alt[edge] - ref[edge]).max() < 1e-9
    alt = without(early[-1])
    edge = early[-1] + window
    assert np.abs(alt[edge - 1] - ref[edge - 1]).max() > big and np.abs(alt[edge] - ref[edge]).max() < 1e-9
    if kind == "sigmoid":
        alt = without(keep - 1)
        assert np.abs(alt[-1] - ref[-1]).max() > big and np.abs(alt[keep - 1 + window] - ref[keep - 1 + window]).max() > big
    engine = engine_for(folder, "float32")
    for got in (replay.whole(engine, [seq]), replay.tail_one_by_one(engine, [seq], tail=2 * window + 5),
                in_portions(engine, [seq], 9)):
        err, where = replay.worst_error(got, [ref])
        assert err < TOL["float32"], f"{err:.3e} at {where}"


def test_a_key_far_back_among_hundreds(tmp_path):
    """A layer without a window: the loud key at position 5 still carries the softmax 600 tokens later, across ten pages,
    in a prompt and in decoding."""
    config = bc.sharp(bc.model(120, 64, 1e-5, 1.0, 3.0, [bc.latent(4, 16, 8, 24, 32, 48, 0.25, 1000.0)]), 20.0)
    folder = bc.make_folder(tmp_path, config, seed=5, edit=_loud_latent)
    pcfg, pw = bc.load_plain(folder)
    rng = np.random.default_rng(4)
    seq = rng.integers(8, config["vocab"], 640).tolist()
    seq[5] = 7
    ref = plain.forward(pcfg, pw, seq)
    without = list(seq)
    without[5] = 9
    assert np.abs(plain.forward(pcfg, pw, without)[-1] - ref[-1]).max() > 100 * TOL["float32"] * np.abs(ref).max()
    engine = engine_for(folder, "float32")
    for got in (replay.whole(engine, [seq]), replay.tail_one_by_one(engine, [seq], tail=40)):
        err, where = replay.worst_error(got, [ref])
        assert err < TOL["float32"], f"{err:.3e} at {where}"


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
    steps, the device sampler), with and without prompts fed in portions: the plain implementation's tokens."""
    folder = bc.make_folder(tmp_path, bc.MIXED, seed=13)
    pcfg, pw = bc.load_plain(folder)
    prompts = bc.prompts(bc.MIXED, [3, 70, 18], seed=9)
    want = [plain_greedy(pcfg, pw, p, 12) for p in prompts]
    loaded = AutoCausalLm.load_local(folder, AutoLoadOptions(dtype="float32", max_tokens=64 * 4))
    for portion in (None, 16):
        out = generate_causal(loaded.model, CausalGenerationRequest(prompts, GenerationConfig(max_new_tokens=12),
                                                                    prefill_chunk_size=portion))
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
    cfg_file.write_text(json.dumps(bc.ODD))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, str(ROOT / "bin" / "random_model"), str(cfg_file), str(folder), "--seed", "4"],
                          capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr
    pcfg, pw = bc.load_plain(folder)
    done = subprocess.run([str(ROOT / "bin" / "generate"), str(folder), "5,6,7,8", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr
    ids = [int(x) for x in done.stdout.split()]
    tokens, margins = plain_greedy(pcfg, pw, [5, 6, 7, 8], 6)
    sure = next((i for i, m in enumerate(margins) if m < 1e-3), 6)
    assert ids[:4] == [5, 6, 7, 8] and ids[4:4 + sure] == tokens[:sure]
    a, b = bc.prompts(bc.ODD, [70, 9], seed=1)
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
