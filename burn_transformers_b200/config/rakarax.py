"""Rakarax's configuration: a list of layers, each with one of two mixers; a layer may run with another layer's weights.

config.json gives every size and constant:

    {"architecture": "Rakarax", "vocab": V, "width": D, "max_positions": P, "norm": {"eps": e},
     "layers": [{"type": "retention",
                 "mixer": {"heads", "dim", "vdim", "decay": [one per head], "rot": {"dims", "base"}},
                 "mlp": null | {"kind": "dense", "ff": F}},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "conv", "scale", "softcap", "mask": {"size": W}},
                           "left_scale": a,
                           "right": {"inner", "state", "dt_rank", "conv"}, "right_scale": b},
                 "mlp": ...},
                {..., "weights_of": j}]}

Sizes have no defaults: one that is missing is an error that names it.  A layer with `weights_of`: j owns no tensors; it
runs with layer j's (which must own its tensors and have an equal entry) and keeps a cache and states of its own.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import I32_MAX, ModelConfig
from .sovozen import _is_int, _is_number

LAYER_TYPES = ("retention", "parallel")
FEED_FORWARD_KINDS = ("dense",)


@dataclasses.dataclass
class RakaraxConfig(ModelConfig):
    FAMILY: ClassVar[str] = "rakarax"
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("Rakarax", "rakarax")

    architecture: str = dataclasses.field(default="Rakarax", metadata={"aliases": ("model_type",)})
    vocab: int = dataclasses.field(default=0, metadata={"aliases": ()})
    width: int = dataclasses.field(default=0, metadata={"aliases": ()})
    max_positions: int = dataclasses.field(default=0, metadata={"aliases": ()})
    norm: dict = dataclasses.field(default_factory=dict, metadata={"aliases": ()})
    layers: list = dataclasses.field(default_factory=list, metadata={"aliases": ()})

    @property
    def model_type(self) -> str:
        return self.MODEL_TYPES[0]

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs with (itself unless it names another)."""
        return self.layers[i].get("weights_of", i)

    # ---- checks --------------------------------------------------------------------------------------------
    def _table(self, where: str, parent: dict, name: str) -> dict:
        value = parent.get(name) if isinstance(parent, dict) else None
        if not isinstance(value, dict):
            self._fail(f"{where}.{name}" if where else name, "is missing")
        return value

    def _ints(self, where: str, table: dict, names, *, minimum: int = 1):
        for name in names:
            if name not in table:
                self._fail(f"{where}.{name}", "is missing")
            value = table[name]
            if not _is_int(value) or value < minimum or value > I32_MAX:
                self._fail(f"{where}.{name}", f"expected an integer of at least {minimum}, found {value!r}")

    def _number(self, where: str, table: dict, name: str, *, positive: bool = False):
        if name not in table:
            self._fail(f"{where}.{name}", "is missing")
        value = table[name]
        if not _is_number(value) or (positive and value <= 0):
            self._fail(f"{where}.{name}", f"expected a finite {'positive ' if positive else ''}number, found {value!r}")

    def _check_retention(self, where: str, mixer: dict) -> None:
        self._ints(where, mixer, ("heads", "dim", "vdim"))
        decay = mixer.get("decay")
        if not isinstance(decay, list) or len(decay) != mixer["heads"] or not all(_is_number(d) for d in decay):
            self._fail(f"{where}.decay", f"expected one number per head ({mixer['heads']})")
        rot = self._table(where, mixer, "rot")
        self._ints(f"{where}.rot", rot, ("dims",), minimum=0)
        self._number(f"{where}.rot", rot, "base", positive=True)
        if rot["dims"] % 2 or rot["dims"] > mixer["dim"]:
            self._fail(f"{where}.rot.dims", f"expected an even number of at most dim = {mixer['dim']} channels, found "
                                            f"{rot['dims']}")

    def _check_parallel(self, where: str, mixer: dict) -> None:
        left = self._table(where, mixer, "left")
        lw = f"{where}.left"
        self._ints(lw, left, ("heads", "kv_heads", "dim", "vdim", "conv"))
        self._number(lw, left, "scale")
        self._number(lw, left, "softcap", positive=True)
        self._ints(f"{lw}.mask", self._table(lw, left, "mask"), ("size",))
        if left["heads"] % left["kv_heads"]:
            self._fail(f"{lw}.kv_heads", f"{left['heads']} query heads cannot share {left['kv_heads']} key heads")
        if left["vdim"] != left["dim"]:
            self._fail(f"{lw}.vdim", f"the values are the keys, so vdim must equal dim = {left['dim']}, found {left['vdim']}")
        right = self._table(where, mixer, "right")
        self._ints(f"{where}.right", right, ("inner", "state", "dt_rank", "conv"))
        self._number(where, mixer, "left_scale")
        self._number(where, mixer, "right_scale")

    def validate(self) -> None:
        self._check_model_type(self.architecture)
        self._check_extents(("vocab", "width", "max_positions"))
        if not isinstance(self.norm, dict):
            self._fail("norm", "must be an object")
        self._number("norm", self.norm, "eps", positive=True)
        if not isinstance(self.layers, list) or not self.layers:
            self._fail("layers", "must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                self._fail(f"{where}.type", f"expected one of {list(LAYER_TYPES)}, found "
                                            f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            mixer = self._table(where, layer, "mixer")
            if layer["type"] == "retention":
                self._check_retention(f"{where}.mixer", mixer)
            else:
                self._check_parallel(f"{where}.mixer", mixer)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in FEED_FORWARD_KINDS:
                    self._fail(f"{where}.mlp.kind", f"expected one of {list(FEED_FORWARD_KINDS)}")
                self._ints(f"{where}.mlp", mlp, ("ff",))
            if "weights_of" in layer:
                j = layer["weights_of"]
                if not _is_int(j) or not 0 <= j < len(self.layers) or j == i or "weights_of" in self.layers[j]:
                    self._fail(f"{where}.weights_of", f"expected another layer that owns its tensors, found {j!r}")
                mine = {k: v for k, v in layer.items() if k != "weights_of"}
                if mine != self.layers[j]:
                    self._fail(f"{where}.weights_of", f"the entry differs from layer {j}'s, whose tensors it uses")
