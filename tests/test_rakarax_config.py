"""Rakarax's configuration, plan and weights on the CPU: the registry finds the design by its `architecture` key, every
broken field is named, layers that run with another layer's tensors share a block and own a cache, the plan asks a
checkpoint for exactly the stored tensors, and the plain implementation agrees with itself where two of its functions
overlap."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_rakarax as plain
import rakarax_configs as rc
from burn_transformers_b200 import models  # noqa: F401
from burn_transformers_b200.config.rakarax import RakaraxConfig
from burn_transformers_b200.config.registry import architecture_for, config_from_folder
from burn_transformers_b200.errors import CheckpointError, ConfigError
from burn_transformers_b200.weights.loader import load_weights


def test_the_registry_knows_the_design(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(rc.MIXED))
    arch, config = config_from_folder(tmp_path)
    assert arch.name == "rakarax" and isinstance(config, RakaraxConfig)
    assert architecture_for("Rakarax") is arch
    assert config.to_dict()["layers"] == rc.MIXED["layers"]
    assert config.eps == 1e-5 and [config.owner(i) for i in range(6)] == [0, 1, 2, 1, 0, 5]


def test_layers_that_share_tensors_share_a_block_and_own_a_cache():
    plan = architecture_for("Rakarax").build(RakaraxConfig.from_dict(rc.MIXED))
    assert len(plan.blocks) == 4 and [c.block for c in plan.schedule] == [0, 1, 2, 1, 0, 3]
    assert all(c.cache is None for c in plan.schedule)
    needs = plan.cache_needs()
    assert needs[0] == needs[4] and needs[1] == needs[3]
    assert needs[0].kv.window == 40 and needs[0].kv.n_kv_heads == 2 and needs[0].kv.head_dim == 24
    assert [s.name for s in needs[0].states] == ["qk_taps", "scan", "x_taps"]
    assert needs[0].states[0].shape == (2, 8 * 24) and needs[0].states[1].shape == (80, 12)
    assert needs[1].kv is None and [s.shape for s in needs[1].states] == [(3, 16, 24)]
    # a convolution of one tap keeps nothing
    odd = architecture_for("Rakarax").build(RakaraxConfig.from_dict(rc.ODD)).cache_needs()
    assert [s.name for s in odd[0].states] == ["scan", "x_taps"] and [s.name for s in odd[2].states] == ["qk_taps", "scan"]
    assert not any(name.startswith(("l3.", "l4.")) for name in plan.weights.stored())


@pytest.mark.parametrize("path, value, named", [
    (("width",), 0, "width"),
    (("norm",), {}, "norm.eps"),
    (("layers", 0, "type"), "serial", "layers[0].type"),
    (("layers", 0, "mixer", "left", "kv_heads"), 4, "layers[0].mixer.left.kv_heads"),
    (("layers", 0, "mixer", "left", "mask"), None, "layers[0].mixer.left.mask"),
    (("layers", 0, "mixer", "left", "vdim"), 16, "layers[0].mixer.left.vdim"),
    (("layers", 0, "mixer", "left", "softcap"), 0.0, "layers[0].mixer.left.softcap"),
    (("layers", 2, "mixer", "right", "dt_rank"), 0, "layers[2].mixer.right.dt_rank"),
    (("layers", 0, "mixer", "right_scale"), "x", "layers[0].mixer.right_scale"),
    (("layers", 0, "mlp", "kind"), "sparse", "layers[0].mlp.kind"),
    (("layers", 1, "mixer", "decay"), [0.9, 0.8], "layers[1].mixer.decay"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "layers[1].mixer.rot.dims"),
    (("layers", 5, "mixer", "rot", "dims"), 42, "layers[5].mixer.rot.dims"),
    (("layers", 3, "weights_of"), 4, "layers[3].weights_of"),
    (("layers", 3, "weights_of"), 3, "layers[3].weights_of"),
    (("layers", 4, "weights_of"), 2, "layers[4].weights_of"),
])
def test_a_broken_field_is_named(path, value, named):
    data = copy.deepcopy(rc.MIXED)
    at = data
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        RakaraxConfig.from_dict(data)
    assert named in str(error.value)


def test_the_plan_reads_exactly_the_stored_tensors(tmp_path):
    folder = rc.make_folder(tmp_path, rc.MIXED, seed=5)
    config, weights = rc.load_plain(folder)
    plan = architecture_for("Rakarax").build(RakaraxConfig.from_dict(config))
    assert set(plan.weights.stored()) == set(weights)
    tensors, _ = load_weights(folder, plan.weights, "float32", torch.device("cpu"))
    # queries, keys and the gate of layer 0's attention as one matrix, the two convolutions as one
    rows = tensors["l0.mix.left.in"].numpy()
    assert rows.shape == ((6 + 2 + 6) * 24, 96)
    np.testing.assert_array_equal(rows[6 * 24:8 * 24], weights["l0.mix.left.k"].astype(np.float32))
    np.testing.assert_array_equal(rows[8 * 24:], weights["l0.mix.left.g"].astype(np.float32))
    taps = tensors["l0.mix.left.conv"].numpy()
    assert taps.shape == (8 * 24, 3) and taps.dtype == np.float32
    np.testing.assert_array_equal(taps[6 * 24:], weights["l0.mix.left.k.conv"].astype(np.float32))
    # the scan's low-rank rows filled up to a multiple of 8
    low = tensors["l0.mix.right.x.rows"].numpy()
    assert low.shape == (32, 80) and not low[29:].any()
    np.testing.assert_array_equal(low[:29], weights["l0.mix.right.x"].astype(np.float32))
    assert tensors["l2.mix.right.x.rows"].shape == (88, 64)
    # the retention's four projections as one
    assert tensors["l1.mix.in"].shape == (2 * 48 + 2 * 72, 96)
    np.testing.assert_array_equal(tensors["l1.mix.in"].numpy()[96:168], weights["l1.mix.v"].astype(np.float32))
    (folder / "model.safetensors").unlink()
    del weights["l2.mix.left.talk"]
    from burn_transformers_b200.weights.safetensors_io import write_file
    write_file(folder / "model.safetensors", {k: torch.from_numpy(v).to(torch.float32) for k, v in weights.items()})
    with pytest.raises(CheckpointError) as error:
        load_weights(folder, plan.weights, "float32", torch.device("cpu"))
    assert "l2.mix.left.talk" in str(error.value)


def test_a_norms_gain_is_one_plus_what_the_file_keeps():
    from burn_transformers_b200.parts import RmsNorm
    norm = RmsNorm(4, 1e-5, offset=1.0)
    norm.bind({"weight": torch.tensor([0.0, -0.25, 0.5, 1.0])})
    assert norm.t_weight.tolist() == [1.0, 0.75, 1.5, 2.0] and norm.t_weight.dtype == torch.float32
    plain_norm = RmsNorm(4, 1e-5)
    plain_norm.bind({"weight": torch.tensor([0.0, -0.25, 0.5, 1.0])})
    assert plain_norm.t_weight.tolist() == [0.0, -0.25, 0.5, 1.0]


def test_the_plain_convolution_is_causal_and_ends_on_the_current_token():
    rng = np.random.default_rng(0)
    u, w = rng.standard_normal((9, 3)), rng.standard_normal((3, 4))
    y = plain.causal_conv(u, w)
    np.testing.assert_allclose(y[0], w[:, 3] * u[0], rtol=1e-12)
    np.testing.assert_allclose(y[5], sum(w[:, j] * u[5 - 3 + j] for j in range(4)), rtol=1e-12)
    later = u.copy()
    later[6:] += 1.0
    np.testing.assert_array_equal(plain.causal_conv(later, w)[:6], y[:6])


def test_the_plain_rotation_keeps_lengths_and_turns_by_position():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((5, 2, 10))
    turned = plain.rotate_half(x, np.arange(5), 6, 100.0)
    np.testing.assert_array_equal(turned[..., 6:], x[..., 6:])
    np.testing.assert_array_equal(turned[0], x[0])
    np.testing.assert_allclose((turned ** 2).sum(-1), (x ** 2).sum(-1), rtol=1e-12)
    # channel 0 goes with channel 3: at position 1 and frequency 1 the pair turns by one radian
    np.testing.assert_allclose(turned[1, 0, 0], x[1, 0, 0] * np.cos(1.0) - x[1, 0, 3] * np.sin(1.0), rtol=1e-12)
    # the scores of rotated queries and keys depend on the distance only
    q, k = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    a = (plain.rotate_half(q, np.array([9]), 6, 50.0) * plain.rotate_half(k, np.array([4]), 6, 50.0)).sum()
    b = (plain.rotate_half(q, np.array([25]), 6, 50.0) * plain.rotate_half(k, np.array([20]), 6, 50.0)).sum()
    np.testing.assert_allclose(a, b, rtol=1e-10)


def test_the_plain_scan_forgets_at_the_rate_its_steps_say():
    """With B = C = 1, D = 0 and a constant input the state follows its closed form."""
    T, inner = 40, 2
    w = {"p.in": np.zeros((2 * inner, 1)), "p.conv": np.array([[0.0, 1.0]] * inner), "p.conv.b": np.zeros(inner),
         "p.x": np.zeros((1 + 2, inner)), "p.dt": np.zeros((inner, 1)), "p.dt.b": np.array([0.3, -1.0]),
         "p.A_log": np.log(np.array([[2.0], [0.5]])), "p.D": np.zeros(inner), "p.o": np.eye(inner)}
    # x = silu(2) for every token and channel, z = 1; B and C cannot come from zeros: give the rows of x a constant
    w["p.in"] = np.array([[2.0], [2.0], [1.0], [1.0]])
    w["p.x"] = np.array([[0.0, 0.0], [0.5 / plain.silu(2.0), 0.5 / plain.silu(2.0)], [0.5 / plain.silu(2.0)] * 2])
    y = plain.selective_scan(np.ones((T, 1)), w, "p.", {"inner": inner, "state": 1, "dt_rank": 1})
    dt = plain.softplus(np.array([0.3, -1.0]))
    decay = np.exp(-dt * np.array([2.0, 0.5]))
    state = dt * plain.silu(2.0) * (1 - decay ** T) / (1 - decay)
    np.testing.assert_allclose(y[-1], state * plain.silu(1.0), rtol=1e-10)
