"""Bosalix as a plan of parts: a scaled token embedding; layers whose norm stands on the sublayers' outputs, x + m *
norm(sublayer(x)), and whose mixer reads every row blended with the row before it (a learned token shift); the mixer is
either a sigmoid attention (grouped heads, normed and rotated queries and keys, normed values that later layers blend
with the first such layer's, a window with kept first positions) or a windowed latent attention whose queries come
through a latent of their own; a feed-forward of routed experts with a softmax router, a correction added for the choice
only, and experts without tensors that hand their input on; a final norm and an untied readout.

Checkpoint names: `embed`, `l<i>.shift`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.{q,k,v,o}` with `.b`, `l<i>.mix.{q,k}.norm`,
`l<i>.mix.{pb,vmix}` (sigmoid attention), `l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}` (latent attention),
`l<i>.mlp.{router,correction,e<j>.up,e<j>.down}`, `final.norm`, `head`; matrices are stored [out, in].  Projections that
read the same input are one product here: their rows are laid end to end when the weights are loaded.
"""
from __future__ import annotations

import torch

from ..config.bosalix import BosalixConfig
from ..config.registry import Architecture, register_architecture
from ..engine.model import UNBOUNDED_CONTEXT, LayerCall, ModelPlan
from ..parts import (HalfSplitRotary, InterleavedRotary, LatentAttention, LinearReadout, NoPositions, OutputNormBlock,
                     RmsNorm, RoutedFeedForward, SigmoidAttention, TokenEmbedding, TokenShift)
from ..weights.spec import Concat, Stored

FIRST_VALUES = "first_values"      # the step tensor in which the first value-mixing layer leaves its values


def _norm(names, name, width, eps):
    norm = RmsNorm(width, eps, offset=1.0)
    names[name] = (norm, "weight")
    return norm


def _sigmoid_attention(names, sources, p, width, m, eps, std, role):
    rot, mask = m["rot"], m.get("mask") or {}
    scaling = rot.get("scaling")
    stretch = None if scaling is None else (scaling["factor"], scaling["low"], scaling["high"], scaling["original"])
    mixer = SigmoidAttention(width, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], eps,
                             HalfSplitRotary(rot["dims"], rot["base"], stretch), window=mask.get("size"),
                             keep_first=mask.get("keep_first", 0), values_as=FIRST_VALUES if role == "first" else None,
                             values_from=FIRST_VALUES if role == "later" else None, init_std=std,
                             out_init_std=(m["heads"] * m["vdim"]) ** -0.5)
    names.update({p + "in": (mixer, "in.weight"), p + "in.b": (mixer, "in.bias"), p + "q.norm": (mixer, "q_norm.weight"),
                  p + "k.norm": (mixer, "k_norm.weight"), p + "pb": (mixer, "bias"), p + "o": (mixer, "out.weight"),
                  p + "o.b": (mixer, "out.bias")})
    sizes = (mixer.q_width, mixer.k_width, mixer.v_width)
    sources[p + "in"] = Concat((Stored(p + "q"), Stored(p + "k"), Stored(p + "v")), 0, sizes)
    sources[p + "in.b"] = Concat((Stored(p + "q.b"), Stored(p + "k.b"), Stored(p + "v.b")), 0, sizes)
    if role == "later":
        names[p + "vmix"] = (mixer, "mix")
    return mixer


def _latent_attention(names, sources, p, width, m, eps, std):
    rot, mask = m["rot"], m.get("mask") or {}
    mixer = LatentAttention(width, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"], eps,
                            InterleavedRotary(rot["dims"], rot["base"]), sink=False, gate=False, window=mask.get("size"),
                            q_rank=m["q_rank"], init_std=std, out_init_std=(m["heads"] * m["vdim"]) ** -0.5)
    names.update({p + "in": (mixer, "in.weight"), p + "dq.norm": (mixer, "q_norm.weight"), p + "uq": (mixer, "uq.weight"),
                  p + "dkv.norm": (mixer, "latent_norm.weight"), p + "uk": (mixer, "uk.weight"),
                  p + "uv": (mixer, "uv.weight"), p + "o": (mixer, "out.weight")})
    sources[p + "in"] = Concat((Stored(p + "dq"), Stored(p + "dkv")), 0, (m["q_rank"], mixer.latent_width))
    return mixer


def _routed(names, sources, p, width, mlp, std):
    router, inner = mlp["router"], mlp["expert"]["ff"]
    n_experts, identity = router["experts"], router.get("identity", 0)
    part = RoutedFeedForward(width, n_experts, router["top"], inner, activation="gelu_erf", gated=False, router="softmax",
                             choice_bias=True, normalise=False, identity=identity, init_std=std)
    names.update({p + "router": (part, "router.weight"), p + "correction": (part, "router.correction"),
                  p + "experts.up": (part, "in.weight"), p + "experts.down": (part, "out.weight")})
    sources[p + "experts.up"] = Concat(tuple(Stored(f"{p}e{j}.up") for j in range(n_experts)), 0, (inner,) * n_experts)
    sources[p + "experts.down"] = Concat(tuple(Stored(f"{p}e{j}.down") for j in range(n_experts)), 0,
                                         (width,) * n_experts)
    return part


def build_bosalix(config: BosalixConfig) -> ModelPlan:
    config.validate()
    width, eps = config.width, config.eps
    std = width ** -0.5
    embedding = TokenEmbedding(config.vocab, width, 1.0, scale=config.embedding_scale)
    readout = LinearReadout(config.vocab, width, 1.0, init_std=std)
    names = {"embed": (embedding, "weight"), "head": (readout, "weight")}
    final_norm = _norm(names, "final.norm", width, eps)
    sources = {}
    mixers = config.value_mixers()
    step_tensors = {}
    if len(mixers) > 1:
        first = config.layers[mixers[0]]["mixer"]
        step_tensors[FIRST_VALUES] = (first["kv_heads"] * first["vdim"], torch.float32)
    blocks = []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            role = None
            if i in mixers and len(mixers) > 1:
                role = "first" if i == mixers[0] else "later"
            mixer = _sigmoid_attention(names, sources, p + "mix.", width, m, eps, std, role)
        else:
            mixer = _latent_attention(names, sources, p + "mix.", width, m, eps, std)
        shift = TokenShift(width)
        names[p + "shift"] = (shift, "weight")
        norm1 = _norm(names, p + "norm1", width, eps)
        feed_forward = norm2 = None
        if layer.get("mlp") is not None:
            feed_forward = _routed(names, sources, p + "mlp.", width, layer["mlp"], std)
            norm2 = _norm(names, p + "norm2", width, eps)
        blocks.append(OutputNormBlock(mixer, norm1, feed_forward, norm2, scale=config.residual_mult, shift=shift))
    # a mixing number is stored for layers that do not use one too (the first value-mixing layer only publishes)
    unused = [i for i, layer in enumerate(config.layers) if layer["type"] == "attention" and i not in mixers[1:]]
    ignored = frozenset(f"l{i}.mix.vmix" for i in unused)
    return ModelPlan(config=config, embedding=embedding, positions=NoPositions(), blocks=blocks,
                     schedule=[LayerCall(i) for i in range(len(blocks))], final_norm=final_norm, readout=readout,
                     names=names, vocab=config.vocab, width=width, max_context=UNBOUNDED_CONTEXT, sources=sources,
                     step_tensors=step_tensors, ignored=ignored)


BOSALIX = register_architecture(Architecture("bosalix", BosalixConfig.MODEL_TYPES, BosalixConfig, build_bosalix),
                                replace=True)
