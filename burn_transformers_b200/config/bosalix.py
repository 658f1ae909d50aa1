"""Bosalix's configuration: a list of layers, each with one of two attention mixers and an optional feed-forward of
routed experts.

config.json gives every size and constant:

    {"architecture": "Bosalix", "vocab": V, "width": D, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"scale": s},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix": true | false,
                           "rot": {"dims", "base", "scaling": {"factor", "low", "high", "original"}},
                           "mask": {"size": W, "keep_first": F}},
                 "mlp": null | {"kind": "moe", "expert": {"ff": F}, "router": {"experts", "identity", "top"}}},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale",
                           "rot": {"dims", "base"}, "mask": {"size": W}},
                 "mlp": ...}]}

Sizes have no defaults: one that is missing is an error that names it.  What a configuration does not mention does not
exist: no `mask` is plain causal attention, no `keep_first` keeps nothing, no `scaling` leaves the frequencies as they
are, no `v_mix` mixes no values, no `identity` adds no experts without tensors, no `mlp` is a layer without a
feed-forward.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar

from .base import I32_MAX, ModelConfig
from .sovozen import _is_int, _is_number

LAYER_TYPES = ("attention", "latent_attention")
FEED_FORWARD_KINDS = ("moe",)


@dataclasses.dataclass
class BosalixConfig(ModelConfig):
    FAMILY: ClassVar[str] = "bosalix"
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("Bosalix", "bosalix")

    architecture: str = dataclasses.field(default="Bosalix", metadata={"aliases": ("model_type",)})
    vocab: int = dataclasses.field(default=0, metadata={"aliases": ()})
    width: int = dataclasses.field(default=0, metadata={"aliases": ()})
    residual_mult: float = dataclasses.field(default=1.0, metadata={"aliases": ()})
    norm: dict = dataclasses.field(default_factory=dict, metadata={"aliases": ()})
    embedding: dict = dataclasses.field(default_factory=dict, metadata={"aliases": ()})
    layers: list = dataclasses.field(default_factory=list, metadata={"aliases": ()})

    @property
    def model_type(self) -> str:
        return self.MODEL_TYPES[0]

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"])

    def value_mixers(self) -> list[int]:
        """The layers whose values are mixed, in order: the first one publishes its values, the others blend them in."""
        return [i for i, layer in enumerate(self.layers)
                if layer["type"] == "attention" and layer["mixer"].get("v_mix")]

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

    def _check_rotation(self, where: str, mixer: dict, most: int, scaling_allowed: bool) -> None:
        rot = self._table(where, mixer, "rot")
        self._ints(f"{where}.rot", rot, ("dims",), minimum=0)
        self._number(f"{where}.rot", rot, "base", positive=True)
        if rot["dims"] % 2 or rot["dims"] > most:
            self._fail(f"{where}.rot.dims", f"expected an even number of at most {most} channels, found {rot['dims']}")
        if rot.get("scaling") is not None:
            if not scaling_allowed:
                self._fail(f"{where}.rot.scaling", "this mixer's frequencies are not scaled")
            scaling = self._table(f"{where}.rot", rot, "scaling")
            for name in ("factor", "low", "high", "original"):
                self._number(f"{where}.rot.scaling", scaling, name, positive=name in ("factor", "original"))
            if scaling["high"] <= scaling["low"]:
                self._fail(f"{where}.rot.scaling.high", "must exceed low")

    def _check_mask(self, where: str, mixer: dict, keep_allowed: bool) -> None:
        if mixer.get("mask") is None:
            return
        mask = self._table(where, mixer, "mask")
        self._ints(f"{where}.mask", mask, ("size",))
        if "keep_first" in mask:
            if not keep_allowed:
                self._fail(f"{where}.mask.keep_first", "this mixer keeps no first positions")
            self._ints(f"{where}.mask", mask, ("keep_first",), minimum=0)

    def _check_attention(self, where: str, mixer: dict) -> None:
        self._ints(where, mixer, ("heads", "kv_heads", "dim", "vdim"))
        self._number(where, mixer, "scale")
        if mixer["heads"] % mixer["kv_heads"]:
            self._fail(f"{where}.kv_heads", f"{mixer['heads']} query heads cannot share {mixer['kv_heads']} key heads")
        self._check_rotation(where, mixer, mixer["dim"], True)
        self._check_mask(where, mixer, True)
        if "v_mix" in mixer and not isinstance(mixer["v_mix"], bool):
            self._fail(f"{where}.v_mix", f"expected true or false, found {mixer['v_mix']!r}")

    def _check_latent(self, where: str, mixer: dict) -> None:
        self._ints(where, mixer, ("heads", "dim", "vdim", "kv_rank", "q_rank"))
        self._ints(where, mixer, ("rot_dim",), minimum=0)
        self._number(where, mixer, "scale")
        self._check_rotation(where, mixer, mixer["rot_dim"], False)
        self._check_mask(where, mixer, False)

    def _check_mlp(self, where: str, mlp: dict) -> None:
        if not isinstance(mlp, dict) or mlp.get("kind") not in FEED_FORWARD_KINDS:
            self._fail(f"{where}.kind", f"expected one of {list(FEED_FORWARD_KINDS)}")
        self._ints(f"{where}.expert", self._table(where, mlp, "expert"), ("ff",))
        router = self._table(where, mlp, "router")
        self._ints(f"{where}.router", router, ("experts", "top"))
        if "identity" in router:
            self._ints(f"{where}.router", router, ("identity",), minimum=0)
        if router["top"] > router["experts"] + router.get("identity", 0):
            self._fail(f"{where}.router.top", f"{router['top']} choices among {router['experts']} + "
                                              f"{router.get('identity', 0)} experts")

    def validate(self) -> None:
        self._check_model_type(self.architecture)
        self._check_extents(("vocab", "width"))
        for name, table, key in (("norm", self.norm, "eps"), ("embedding", self.embedding, "scale")):
            if not isinstance(table, dict):
                self._fail(name, "must be an object")
            self._number(name, table, key, positive=name == "norm")
        if not _is_number(self.residual_mult):
            self._fail("residual_mult", f"expected a finite number, found {self.residual_mult!r}")
        if not isinstance(self.layers, list) or not self.layers:
            self._fail("layers", "must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
                self._fail(f"{where}.type", f"expected one of {list(LAYER_TYPES)}, found "
                                            f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            mixer = self._table(where, layer, "mixer")
            if layer["type"] == "attention":
                self._check_attention(f"{where}.mixer", mixer)
            else:
                self._check_latent(f"{where}.mixer", mixer)
            if layer.get("mlp") is not None:
                self._check_mlp(f"{where}.mlp", layer["mlp"])
        mixers = self.value_mixers()
        for i in mixers[1:]:
            a, b = self.layers[mixers[0]]["mixer"], self.layers[i]["mixer"]
            if (a["kv_heads"], a["vdim"]) != (b["kv_heads"], b["vdim"]):
                self._fail(f"layers[{i}].mixer.v_mix", f"values of {b['kv_heads']} x {b['vdim']} cannot be mixed with layer "
                                                      f"{mixers[0]}'s of {a['kv_heads']} x {a['vdim']}")
