"""Bosalix's configuration, plan and weights on the CPU: the registry finds the design by its `architecture` key, every
broken field is named, the plan asks a checkpoint for exactly the stored tensors and lays projections of one input end
to end, the layers' cache needs follow the configuration, and the plain implementation agrees with itself where two of
its functions overlap."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import bosalix_configs as bc
import plain_bosalix as plain
from burn_transformers_b200 import models  # noqa: F401
from burn_transformers_b200.config.bosalix import BosalixConfig
from burn_transformers_b200.config.registry import architecture_for, config_from_folder
from burn_transformers_b200.errors import CheckpointError, ConfigError
from burn_transformers_b200.weights.loader import load_weights


def test_the_registry_knows_the_design(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(bc.MIXED))
    arch, config = config_from_folder(tmp_path)
    assert arch.name == "bosalix" and isinstance(config, BosalixConfig)
    assert architecture_for("Bosalix") is arch
    assert config.to_dict()["layers"] == bc.MIXED["layers"]
    assert config.eps == 1e-5 and config.embedding_scale == 9.0 and config.value_mixers() == [0, 2, 5]


def test_the_layers_cache_needs_follow_the_configuration():
    plan = architecture_for("Bosalix").build(BosalixConfig.from_dict(bc.MIXED))
    needs = plan.cache_needs()
    # one row [key | value] per position and key head; every position is kept (the first ones stay visible)
    assert (needs[0].kv.n_kv_heads, needs[0].kv.head_dim, needs[0].kv.window, needs[0].kv.has_values) == (2, 40, None, False)
    assert (needs[5].kv.n_kv_heads, needs[5].kv.head_dim) == (2, 56)
    # one row [latent | rotated key part] per position
    assert (needs[1].kv.n_kv_heads, needs[1].kv.head_dim, needs[1].kv.has_values) == (1, 56, False)
    # the row before a sequence's next token, in every layer
    assert all([(s.name, s.shape, s.dtype) for s in need.states] == [("shift_prev", (96,), torch.float32)] for need in needs)
    # the first value-mixing layer publishes, the later ones blend; a layer that says false, and a model with one such
    # layer only, do neither
    mixers = [b.mixer for b in plan.blocks]
    assert [(getattr(m, "values_as", None), getattr(m, "values_from", None)) for m in mixers] == [
        ("first_values", None), (None, None), (None, "first_values"), (None, None), (None, None), (None, "first_values")]
    assert plan.step_tensors == {"first_values": (32, torch.float32)}
    odd = architecture_for("Bosalix").build(BosalixConfig.from_dict(bc.ODD))
    assert odd.step_tensors == {} and odd.blocks[0].mixer.values_as is None
    assert odd.blocks[3].feed_forward is None and odd.blocks[3].norm2 is None
    # windows and kept positions reach the parts; what is not mentioned does not exist
    assert (mixers[0].window, mixers[0].keep_first, mixers[3].window, mixers[4].window) == (40, 5, None, None)
    assert mixers[0].positions.stretch == (4.0, 1.0, 4.0, 64.0) and mixers[2].positions.stretch is None
    ff = plan.blocks[5].feed_forward
    assert (ff.n_experts, ff.identity, ff.top, ff.gated, ff.router, ff.normalise) == (2, 0, 2, False, "softmax", False)


@pytest.mark.parametrize("path, value, named", [
    (("width",), 0, "width"),
    (("norm",), {}, "norm.eps"),
    (("embedding",), {}, "embedding.scale"),
    (("residual_mult",), "x", "residual_mult"),
    (("layers", 0, "type"), "serial", "layers[0].type"),
    (("layers", 0, "mixer", "kv_heads"), 4, "layers[0].mixer.kv_heads"),
    (("layers", 0, "mixer", "mask", "size"), 0, "layers[0].mixer.mask.size"),
    (("layers", 0, "mixer", "mask", "keep_first"), -1, "layers[0].mixer.mask.keep_first"),
    (("layers", 0, "mixer", "rot", "dims"), 26, "layers[0].mixer.rot.dims"),
    (("layers", 0, "mixer", "rot", "scaling", "high"), 0.5, "layers[0].mixer.rot.scaling.high"),
    (("layers", 0, "mixer", "v_mix"), 1, "layers[0].mixer.v_mix"),
    (("layers", 0, "mlp", "kind"), "dense", "layers[0].mlp.kind"),
    (("layers", 0, "mlp", "router", "top"), 9, "layers[0].mlp.router.top"),
    (("layers", 0, "mlp", "router", "identity"), -2, "layers[0].mlp.router.identity"),
    (("layers", 1, "mixer", "q_rank"), 0, "layers[1].mixer.q_rank"),
    (("layers", 1, "mixer", "rot", "dims"), 10, "layers[1].mixer.rot.dims"),
    (("layers", 1, "mixer", "mask", "keep_first"), 3, "layers[1].mixer.mask.keep_first"),
    (("layers", 2, "mixer", "vdim"), 24, "layers[2].mixer.v_mix"),
])
def test_a_broken_field_is_named(path, value, named):
    data = copy.deepcopy(bc.MIXED)
    at = data
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        BosalixConfig.from_dict(data)
    assert named in str(error.value)


def test_the_plan_reads_exactly_the_stored_tensors(tmp_path):
    folder = bc.make_folder(tmp_path, bc.MIXED, seed=5)
    config, weights = bc.load_plain(folder)
    plan = architecture_for("Bosalix").build(BosalixConfig.from_dict(config))
    assert set(plan.weights.stored()) == set(weights)
    assert "l0.mix.vmix" not in weights and "l3.mix.vmix" not in weights and weights["l2.mix.vmix"].shape == ()
    tensors, _ = load_weights(folder, plan.weights, "float32", torch.device("cpu"))
    # queries, keys and values of layer 0 as one matrix with one bias
    rows = tensors["l0.mix.in"].numpy()
    assert rows.shape == (6 * 24 + 2 * 24 + 2 * 16, 96)
    np.testing.assert_array_equal(rows[6 * 24:8 * 24], weights["l0.mix.k"].astype(np.float32))
    np.testing.assert_array_equal(tensors["l0.mix.in.b"].numpy()[8 * 24:], weights["l0.mix.v.b"].astype(np.float32))
    # the latent layer's two down-projections as one
    assert tensors["l1.mix.in"].shape == (40 + 48 + 8, 96)
    np.testing.assert_array_equal(tensors["l1.mix.in"].numpy()[40:], weights["l1.mix.dkv"].astype(np.float32))
    # all experts' matrices end to end; the router also has rows for the experts without tensors
    assert tensors["l0.mlp.experts.up"].shape == (6 * 40, 96) and tensors["l0.mlp.experts.down"].shape == (6 * 96, 40)
    np.testing.assert_array_equal(tensors["l0.mlp.experts.down"].numpy()[96:192], weights["l0.mlp.e1.down"].astype(np.float32))
    assert tensors["l0.mlp.router"].shape == (8, 96) and tensors["l0.mlp.correction"].shape == (8,)
    # a stored mixing number of a layer that does not use one is let pass; a missing tensor is named
    from burn_transformers_b200.weights.safetensors_io import write_file
    weights["l0.mix.vmix"] = np.array(0.5)
    (folder / "model.safetensors").unlink()
    write_file(folder / "model.safetensors", {k: torch.tensor(np.asarray(v)).to(torch.float32) for k, v in weights.items()})
    load_weights(folder, plan.weights, "float32", torch.device("cpu"))
    del weights["l2.mix.pb"]
    (folder / "model.safetensors").unlink()
    write_file(folder / "model.safetensors", {k: torch.tensor(np.asarray(v)).to(torch.float32) for k, v in weights.items()})
    with pytest.raises(CheckpointError) as error:
        load_weights(folder, plan.weights, "float32", torch.device("cpu"))
    assert "l2.mix.pb" in str(error.value)


def test_stretched_frequencies_of_the_part_and_of_the_plain_implementation():
    from burn_transformers_b200.parts import HalfSplitRotary
    part = HalfSplitRotary(16, 10000.0, (4.0, 1.0, 4.0, 64))
    want = plain.stretched_frequencies(16, 10000.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64})
    np.testing.assert_allclose(part.frequencies(), want, rtol=1e-14)
    bare = plain.plain_frequencies(16, 10000.0)
    # short waves stay, long waves slow down fourfold, and one in between is blended
    assert want[0] == bare[0] and want[-1] == bare[-1] / 4.0
    assert any(b / 4.0 < w < b for w, b in zip(want, bare))
    assert HalfSplitRotary(16, 10000.0).frequencies() == bare


def test_the_plain_rotations_keep_lengths_and_turn_by_position():
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((5, 2, 10)))
    freqs = plain.plain_frequencies(6, 100.0)
    for layout, partner in (("half", 3), ("interleaved", 1)):
        turned = plain.rotate_pairs(x, torch.arange(5), freqs, layout)
        assert torch.equal(turned[..., 6:], x[..., 6:]) and torch.equal(turned[0], x[0])
        np.testing.assert_allclose((turned ** 2).sum(-1), (x ** 2).sum(-1), rtol=1e-12)
        # channel 0's partner: at position 1 and frequency 1 the pair turns by one radian
        np.testing.assert_allclose(turned[1, 0, 0], x[1, 0, 0] * math.cos(1.0) - x[1, 0, partner] * math.sin(1.0), rtol=1e-12)


def test_the_plain_token_shift_goes_on_from_the_row_it_kept():
    rng = np.random.default_rng(2)
    h, shift = torch.from_numpy(rng.standard_normal((9, 4))), torch.from_numpy(rng.standard_normal(4))
    whole, last = plain.token_shift(h, shift)
    np.testing.assert_allclose(whole[0], h[0] * (1 - shift), rtol=1e-12)
    first, kept = plain.token_shift(h[:4], shift)
    second, _ = plain.token_shift(h[4:], shift, before=kept)
    np.testing.assert_allclose(torch.cat([first, second]), whole, rtol=1e-12)
    assert torch.equal(last, h[-1])


def test_the_plain_windows():
    seen = plain.visibility(12, 3, 2)
    assert seen[5].tolist() == [True, True, False, True, True, True] + [False] * 6
    assert plain.visibility(4, None, 0).tolist() == torch.ones(4, 4).tril().bool().tolist()
    assert plain.visibility(6, 1, 0).tolist() == torch.eye(6).bool().tolist()


def test_the_plain_router_weighs_by_the_bare_scores():
    """Two stored experts and one that hands its input on; the correction moves the choice, not the weights."""
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=torch.float64)
    w = {"router": torch.tensor([[2.0, 0.0], [0.0, 0.0], [0.0, 2.0]], dtype=torch.float64),
         "correction": torch.tensor([0.0, 5.0, 0.0], dtype=torch.float64),
         "e0.up": torch.eye(2, dtype=torch.float64), "e0.down": torch.eye(2, dtype=torch.float64),
         "e1.up": torch.eye(2, dtype=torch.float64), "e1.down": 3.0 * torch.eye(2, dtype=torch.float64)}
    mlp = {"router": {"experts": 2, "identity": 1, "top": 2}}
    out = plain.routed_experts(h, w, mlp)
    scores = torch.softmax(h @ w["router"].T, -1)
    g = plain.gelu_erf(torch.tensor(1.0, dtype=torch.float64))
    # token 0: expert 1 (by its correction) and expert 0; token 1: expert 1 and the one that hands its input on
    np.testing.assert_allclose(out[0], [scores[0, 1] * 3 * g + scores[0, 0] * g, 0.0], rtol=1e-12)
    np.testing.assert_allclose(out[1], [0.0, scores[1, 1] * 3 * g + scores[1, 2] * 1.0], rtol=1e-12)
