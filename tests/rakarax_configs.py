"""Small Rakarax configurations for the tests, and helpers to write model folders (with tensors edited where random
weights would hide a fault) and to read them for the plain implementation.  The configurations differ from one another
in every size, in the order of their layers, in which layers run with another's tensors, and in which sizes happen to
be equal or one."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np
import torch

import burn_transformers_b200 as bt
import plain_gpt2
from burn_transformers_b200.weights.safetensors_io import write_file


def left(heads, kv_heads, dim, taps, window, scale, softcap):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": taps, "scale": scale,
            "softcap": softcap, "mask": {"size": window}}


def right(inner, state, dt_rank, taps):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": taps}


def parallel(left_part, right_part, left_scale, right_scale, ff=None, **more):
    return {"type": "parallel", "mixer": {"left": left_part, "left_scale": left_scale, "right": right_part,
                                          "right_scale": right_scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}, **more}


def retention(heads, dim, vdim, decay, rot_dims, base, ff=None, **more):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                                           "rot": {"dims": rot_dims, "base": base}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}, **more}


def again(config_layers, j):
    """An entry that runs with layer j's tensors."""
    entry = copy.deepcopy(config_layers[j])
    entry["weights_of"] = j
    return entry


def _mixed_layers():
    layers = [parallel(left(6, 2, 24, 3, 40, 0.2, 15.0), right(80, 12, 5, 4), 0.8, 1.3, ff=160),
              retention(3, 16, 24, (0.9, 0.97, 0.995), 8, 10000.0, ff=120),
              parallel(left(4, 4, 32, 2, 100, 0.18, 30.0), right(64, 40, 8, 2), 1.5, 0.6),
              None, None,
              retention(2, 40, 20, (0.999, 0.5), 40, 500.0)]
    layers[3] = again(layers, 1)
    layers[4] = again(layers, 0)
    return layers


# A: layers that all differ; 3 and 1 query heads a key head; windows of 40 and 100; convolutions of 3, 4 and 2 taps; a
# rotation of a part of the head and of all of it; layers without a feed-forward; two layers that run with earlier
# layers' tensors (one of each kind), each with a cache of its own.
MIXED = {"architecture": "Rakarax", "vocab": 310, "width": 96, "max_positions": 700, "norm": {"eps": 1e-5},
         "layers": _mixed_layers()}

# B: sizes that are no multiples of 8 (the kernels' element-by-element branches), an odd vocabulary, a convolution of one
# tap (no state) and one of five, one key head for five query heads, one retention head, no rotation at all.
ODD = {"architecture": "Rakarax", "vocab": 257, "width": 72, "max_positions": 300, "norm": {"eps": 1e-6},
       "layers": [parallel(left(5, 1, 12, 1, 33, 0.22, 8.0), right(36, 5, 3, 5), 1.1, 0.9, ff=100),
                  retention(1, 10, 6, (0.98,), 0, 100.0, ff=52),
                  parallel(left(2, 2, 20, 5, 300, 0.3, 50.0), right(44, 17, 1, 1), 0.7, -1.2, ff=36)]}

# C: a width and sizes that are no whole 16-byte pieces anywhere, a window of one token and one longer than any sequence,
# a single head, a state of one index.
ODDER = {"architecture": "Rakarax", "vocab": 131, "width": 52, "max_positions": 200, "norm": {"eps": 1e-5},
         "layers": [parallel(left(3, 1, 6, 2, 1, 0.4, 5.0), right(30, 1, 2, 3), 1.0, 1.0, ff=30),
                    parallel(left(1, 1, 14, 4, 1000, 0.25, 12.0), right(18, 3, 7, 2), -0.5, 0.8),
                    retention(3, 6, 10, (1.0, 0.75, 0.99), 2, 7.0, ff=22)]}

# D: larger heads and states (other branches of the kernels' size tables): 128 and 72 key channels a head, 70 and 130 state
# indices, a retention with 130 key channels.
LARGE = {"architecture": "Rakarax", "vocab": 150, "width": 80, "max_positions": 300, "norm": {"eps": 1e-5},
         "layers": [parallel(left(2, 1, 128, 4, 70, 0.09, 20.0), right(24, 70, 4, 4), 1.0, 0.5),
                    retention(1, 130, 20, (0.99,), 64, 1e6, ff=64),
                    parallel(left(4, 2, 72, 3, 130, 0.12, 25.0), right(16, 130, 6, 3), 1.0, 0.5, ff=40)]}

# One mechanism at a time (a scale of zero silences the other mixer; the stream still passes the layer).
ONLY_LEFT = {"architecture": "Rakarax", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
             "layers": [parallel(left(4, 2, 16, 3, 50, 0.3, 10.0), right(8, 2, 2, 2), 1.0, 0.0)]}
ONLY_RIGHT = {"architecture": "Rakarax", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
              "layers": [parallel(left(1, 1, 8, 2, 4, 0.3, 10.0), right(48, 20, 6, 4), 0.0, 1.0)]}
ONLY_RETENTION = {"architecture": "Rakarax", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
                  "layers": [retention(2, 24, 40, (0.96, 0.999), 12, 3000.0)]}
ONLY_FEED_FORWARD = {"architecture": "Rakarax", "vocab": 120, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
                     "layers": [parallel(left(1, 1, 8, 2, 4, 0.3, 10.0), right(8, 2, 2, 2), 0.0, 0.0, ff=88)]}

CONFIGS = {"mixed": MIXED, "odd": ODD, "odder": ODDER, "large": LARGE, "only_left": ONLY_LEFT, "only_right": ONLY_RIGHT,
           "only_retention": ONLY_RETENTION, "only_feed_forward": ONLY_FEED_FORWARD}


def sharp(config: dict, factor: float = 8.0) -> dict:
    """The same model with every attention score scaled up (and the cap lifted with it): softmaxes close to one-hot, so
    that a key that is lost at a page's border, doubled, or seen one position outside the window moves the logits by far
    more than rounding does."""
    out = copy.deepcopy(config)
    for entry in out["layers"]:
        if entry["type"] == "parallel":
            entry["mixer"]["left"]["scale"] *= factor
            entry["mixer"]["left"]["softcap"] *= factor
    return out


def long_memory(tensors: dict) -> dict:
    """Small steps and slow decays in the scans: the state still holds the first tokens after hundreds, so a state that
    is lost, zeroed or carried over to the wrong sequence shows at every later position."""
    for name in tensors:
        if name.endswith(".right.dt.b"):
            tensors[name] = tensors[name] * 0.2 - 4.0
        if name.endswith(".right.A_log"):
            tensors[name] = tensors[name] * 0.2 - 1.0
    return tensors


def make_folder(path, config: dict, *, seed=3, storage="bfloat16", edit=None) -> Path:
    """A folder with random weights.  Gains and biases, which a random model has as ones and zeros, are spread out (a
    gain read at another head's place, or a bias that is left out, would not show otherwise); `edit` then changes
    tensors by name."""
    folder = bt.write_random_model(path, config, seed=seed, storage=storage)
    stored = plain_gpt2.read_safetensors(folder / "model.safetensors")
    rng = np.random.default_rng(seed + 1000)
    tensors = {}
    for name, value in stored.items():
        value = np.array(value)
        if value.ndim == 1:
            value = value + rng.standard_normal(value.shape) * 0.2
        tensors[name] = value
    if edit is not None:
        tensors = edit(tensors)
    as_matrix = {"bfloat16": torch.bfloat16, "float32": torch.float32}[storage]
    write_file(folder / "model.safetensors",
               {k: torch.from_numpy(np.ascontiguousarray(v)).to(as_matrix if v.ndim == 2 else torch.float32)
                for k, v in tensors.items()})
    return folder


def load_plain(folder):
    """(configuration as a dictionary, float64 weights by checkpoint name) for plain_rakarax."""
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), plain_gpt2.read_safetensors(folder / "model.safetensors")


def prompts(config: dict, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, config["vocab"], n).tolist() for n in lengths]
