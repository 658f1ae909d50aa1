"""Small Bosalix configurations for the tests, and helpers to write model folders (with tensors edited where random
weights would hide a fault) and to read them for the plain implementation.  The configurations differ from one another
in every size, in the order of their layers, in which layers mix values, and in which sizes happen to be equal or one."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np
import torch

import burn_transformers_b200 as bt
import plain_gpt2
from burn_transformers_b200.weights.safetensors_io import write_file


def moe(experts, identity, top, ff):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base, *, window=None, keep_first=None, scaling=None,
              v_mix=None, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "rot": {"dims": rot_dims, "base": base}}
    if scaling is not None:
        mixer["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if window is not None:
        mixer["mask"] = {"size": window}
        if keep_first is not None:
            mixer["mask"]["keep_first"] = keep_first
    if v_mix is not None:
        mixer["v_mix"] = v_mix
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, *, window=None, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": scale, "rot": {"dims": rot_dim, "base": base}}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, eps, mult, embed_scale, layers):
    return {"architecture": "Bosalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": embed_scale}, "layers": layers}


# A: layers that all differ.  Three value-mixing layers (the first publishes) around one that mixes nothing; 3, 2 and 1
# query heads a key head; windows of 40, 70 and 100 with 5, 0 and 90 kept first positions, and one layer that sees
# everything; rotations of a part of the head and of all of it, with and without stretched frequencies; latent layers
# with and without a window; layers without a feed-forward; experts with and without ones that hand their input on.
MIXED = model(310, 96, 1e-5, 0.6, 9.0, [
    attention(6, 2, 24, 16, 0.2, 16, 10000.0, window=40, keep_first=5, scaling=(4.0, 1.0, 4.0, 64), v_mix=True,
              mlp=moe(6, 2, 2, 40)),
    latent(3, 16, 8, 24, 48, 40, 0.2, 5000.0, window=33, mlp=moe(4, 0, 1, 56)),
    attention(4, 2, 32, 16, 0.15, 32, 500.0, window=70, keep_first=0, v_mix=True),
    attention(2, 2, 16, 24, 0.25, 8, 100.0, v_mix=False, mlp=moe(3, 3, 3, 24)),
    latent(2, 24, 16, 16, 32, 64, 0.18, 20000.0, mlp=moe(5, 1, 2, 32)),
    attention(2, 2, 40, 16, 0.1, 20, 3000.0, window=100, keep_first=90, scaling=(8.0, 0.5, 2.0, 32), v_mix=True,
              mlp=moe(2, None, 2, 48)),
])

# B: sizes that are no multiples of 8 (the kernels' element-by-element branches), an odd vocabulary, one key head for
# five query heads, a window of one token and one longer than any sequence, more kept positions than the window is long,
# a latent attention with a single head, one expert a token out of one.
ODD = model(257, 72, 1e-6, 1.3, 1.0, [
    attention(5, 1, 12, 10, 0.3, 6, 50.0, window=1, keep_first=3, v_mix=True, mlp=moe(1, 2, 1, 20)),
    latent(1, 10, 6, 14, 20, 12, 0.3, 300.0, window=1000, mlp=moe(3, 0, 3, 36)),
    attention(3, 3, 20, 10, 0.22, 0, 10.0, window=7, keep_first=20, mlp=moe(7, 5, 4, 12)),
    latent(5, 6, 2, 6, 12, 30, 0.4, 7.0, window=2),
])

# C: larger heads (other branches of the kernels' size tables): 128 and 72 key channels a head, values of 96 and 130 channels, a
# latent of 160 channels, sixteen query heads a key head; two layers whose keys and values have 64 and 128 channels (the
# tcgen05 kernel for prompts and their portions).
LARGE = model(150, 80, 1e-5, 0.7, 4.0, [
    attention(16, 1, 128, 96, 0.09, 48, 1e6, window=70, keep_first=16, v_mix=True, mlp=moe(10, 3, 2, 88)),
    latent(6, 32, 16, 32, 160, 96, 0.14, 50000.0, window=50, mlp=moe(4, 4, 2, 64)),
    attention(4, 2, 72, 130, 0.12, 72, 10000.0, window=130, keep_first=1),
    attention(8, 2, 64, 64, 0.12, 32, 10000.0, window=90, keep_first=3, mlp=moe(3, 1, 2, 48)),
    attention(4, 1, 64, 128, 0.12, 64, 10000.0, window=40, keep_first=40),
])

# One mechanism at a time.
ONLY_SIGMOID = model(120, 64, 1e-5, 1.0, 3.0, [attention(4, 2, 16, 24, 0.3, 8, 1000.0, window=50, keep_first=4)])
ONLY_LATENT = model(120, 64, 1e-5, 1.0, 3.0, [latent(4, 16, 8, 24, 32, 48, 0.25, 1000.0, window=50)])
ONLY_EXPERTS = model(120, 64, 1e-5, 0.8, 3.0, [attention(1, 1, 8, 8, 0.3, 4, 100.0, window=2, mlp=moe(6, 3, 2, 88))])
VALUE_MIXING = model(120, 64, 1e-5, 1.0, 3.0, [attention(2, 1, 16, 40, 0.3, 16, 1000.0, v_mix=True),
                                              attention(4, 1, 8, 40, 0.3, 8, 1000.0, window=30, keep_first=2, v_mix=True)])

CONFIGS = {"mixed": MIXED, "odd": ODD, "large": LARGE, "only_sigmoid": ONLY_SIGMOID, "only_latent": ONLY_LATENT,
           "only_experts": ONLY_EXPERTS, "value_mixing": VALUE_MIXING}


def sharp(config: dict, factor: float = 8.0) -> dict:
    """The same model with every attention score scaled up: softmaxes close to one-hot and sigmoids close to steps, so
    that a key that is lost at a page's border, doubled, or seen one position outside a window moves the logits by far
    more than rounding does."""
    out = copy.deepcopy(config)
    for entry in out["layers"]:
        entry["mixer"]["scale"] *= factor
    return out


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
               {k: torch.tensor(v).to(as_matrix if v.ndim == 2 else torch.float32)
                for k, v in tensors.items()})
    return folder


def load_plain(folder):
    """(configuration as a dictionary, float64 weights by checkpoint name) for plain_bosalix."""
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), plain_gpt2.read_safetensors(folder / "model.safetensors")


def prompts(config: dict, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, config["vocab"], n).tolist() for n in lengths]
