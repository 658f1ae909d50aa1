"""Rakarax as a plan of parts: token embedding plus a learned position vector; layers with an RMS norm (the gain kept
minus one) before and after each sublayer; the mixer is either a retention (rotated queries and keys, one decay per
head, a 32-bit state) or two side by side, each with a scale: a windowed softmax attention behind a short convolution
whose heads talk before the softmax and whose values are its keys, and a selective state-space scan; a dense
feed-forward with a polynomial activation; a layer may run with another layer's tensors and a cache of its own; a final
norm and an untied readout.

Checkpoint names: `embed`, `pos`, `l<i>.norm1`, `.norm1b`, `.norm2`, `.norm2b`, `l<i>.mix.{q,k,v,g,o}` (retention),
`l<i>.mix.left.{q,k,q.conv,k.conv,temp,talk,g,o}`, `l<i>.mix.right.{in,conv,conv.b,x,dt,dt.b,A_log,D,o}`,
`l<i>.mlp.{up,act,down}`, `final.norm`, `head`; matrices are stored [out, in].  Projections that read the same input
are one product here: their rows are laid end to end when the weights are loaded.
"""
from __future__ import annotations

from ..config.rakarax import RakaraxConfig
from ..config.registry import Architecture, register_architecture
from ..engine.model import LayerCall, ModelPlan
from ..parts import (HalfSplitRotary, LearnedPositions, LinearReadout, PolyNormFeedForward, Retention, RmsNorm,
                     SandwichBlock, SelectiveScan, SideBySideMixers, TalkingConvAttention, TokenEmbedding)
from ..weights.spec import Concat, PadBlocks, Stored


def _norm(names, name, width, eps):
    norm = RmsNorm(width, eps, offset=1.0)
    names[name] = (norm, "weight")
    return norm


def _retention(names, sources, p, width, m, eps, std):
    mixer = Retention(width, m["heads"], m["dim"], m["vdim"], m["decay"], eps,
                      HalfSplitRotary(m["rot"]["dims"], m["rot"]["base"]), init_std=std,
                      out_init_std=(m["heads"] * m["vdim"]) ** -0.5)
    names[p + "in"] = (mixer, "in.weight")
    names[p + "o"] = (mixer, "out.weight")
    sources[p + "in"] = Concat((Stored(p + "q"), Stored(p + "k"), Stored(p + "v"), Stored(p + "g")), 0,
                               (mixer.qk_width, mixer.qk_width, mixer.v_width, mixer.v_width))
    return mixer


def _side_by_side(names, sources, p, width, m, eps, std):
    c = m["left"]
    left = TalkingConvAttention(width, c["heads"], c["kv_heads"], c["dim"], c["conv"], c["scale"], c["softcap"], eps,
                                window=c["mask"]["size"], out_scale=m["left_scale"], init_std=std,
                                out_init_std=(c["heads"] * c["dim"]) ** -0.5)
    a = p + "left."
    names.update({a + "in": (left, "in.weight"), a + "conv": (left, "conv.weight"), a + "temp": (left, "temp"),
                  a + "talk": (left, "talk"), a + "o": (left, "out.weight")})
    sources[a + "in"] = Concat((Stored(a + "q"), Stored(a + "k"), Stored(a + "g")), 0,
                               (left.q_width, left.kv_width, left.q_width))
    sources[a + "conv"] = Concat((Stored(a + "q.conv"), Stored(a + "k.conv")), 0, (left.q_width, left.kv_width))
    c = m["right"]
    right = SelectiveScan(width, c["inner"], c["state"], c["dt_rank"], c["conv"], out_scale=m["right_scale"],
                          init_std=std, out_init_std=c["inner"] ** -0.5)
    b = p + "right."
    names.update({b + "in": (right, "in.weight"), b + "conv": (right, "conv.weight"), b + "conv.b": (right, "conv.bias"),
                  b + "x.rows": (right, "x.weight"), b + "dt": (right, "dt.weight"), b + "dt.b": (right, "dt.bias"),
                  b + "A_log": (right, "A_log"), b + "D": (right, "D"), b + "o": (right, "out.weight")})
    low = c["dt_rank"] + 2 * c["state"]
    sources[b + "x.rows"] = Stored(b + "x") if low == right.low_width else PadBlocks(Stored(b + "x"), 0, low,
                                                                                     right.low_width)
    return SideBySideMixers(left, right)


def build_rakarax(config: RakaraxConfig) -> ModelPlan:
    config.validate()
    width, eps = config.width, config.eps
    std = width ** -0.5
    embedding = TokenEmbedding(config.vocab, width, 1.0)
    positions = LearnedPositions(config.max_positions, width, 0.1)
    readout = LinearReadout(config.vocab, width, 1.0, init_std=std)
    names = {"embed": (embedding, "weight"), "pos": (positions, "weight"), "head": (readout, "weight")}
    final_norm = _norm(names, "final.norm", width, eps)
    sources = {}
    blocks, block_of = [], {}
    for i, layer in enumerate(config.layers):
        if config.owner(i) != i:
            continue
        p = f"l{i}."
        m = layer["mixer"]
        norm1, norm1b = _norm(names, p + "norm1", width, eps), _norm(names, p + "norm1b", width, eps)
        if layer["type"] == "retention":
            mixer = _retention(names, sources, p + "mix.", width, m, eps, std)
        else:
            mixer = _side_by_side(names, sources, p + "mix.", width, m, eps, std)
        norm2 = feed_forward = norm2b = None
        if layer.get("mlp") is not None:
            inner = layer["mlp"]["ff"]
            norm2, norm2b = _norm(names, p + "norm2", width, eps), _norm(names, p + "norm2b", width, eps)
            feed_forward = PolyNormFeedForward(width, inner, eps, init_std=std, down_init_std=inner ** -0.5)
            names.update({p + "mlp.up": (feed_forward, "up.weight"), p + "mlp.act": (feed_forward, "act"),
                          p + "mlp.down": (feed_forward, "down.weight")})
        block_of[i] = len(blocks)
        blocks.append(SandwichBlock(norm1, mixer, norm1b, norm2, feed_forward, norm2b))
    # the run order is the configuration's; a layer that names another's tensors runs that block with a cache of its own
    schedule = [LayerCall(block_of[config.owner(i)]) for i in range(len(config.layers))]
    return ModelPlan(config=config, embedding=embedding, positions=positions, blocks=blocks, schedule=schedule,
                     final_norm=final_norm, readout=readout, names=names, vocab=config.vocab, width=width,
                     max_context=config.max_positions, sources=sources)


RAKARAX = register_architecture(Architecture("rakarax", RakaraxConfig.MODEL_TYPES, RakaraxConfig, build_rakarax),
                                replace=True)
