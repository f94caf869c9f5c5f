"""Pezarax as data for the engine: tensor names and shapes, random initialisation, named
sizes, registration.  The model is put together by
:func:`pretrained_rstr_b200.models.assembly.build_model` from the parts that
``PezaraxConfig.layer_specs()`` names, in the order ``run_order()`` gives.

Tensor names: ``embed`` and ``head`` [vocab, width], ``final.norm`` [width] and per layer i
``l<i>.norm1``, ``l<i>.norm2`` [width] (the second only with a feed-forward), the mixer's
``l<i>.mix.*`` and the feed-forward's ``l<i>.mlp.*``; matrices are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..config.pezarax import PezaraxConfig
from ..config.registry import Architecture, register_architecture
from ..weights.loader import TensorExpectation, normal


def expected_tensors(cfg: PezaraxConfig) -> Dict[str, TensorExpectation]:
    d = cfg.width
    exp: Dict[str, TensorExpectation] = {
        "embed": TensorExpectation((cfg.vocab, d)),
        "head": TensorExpectation((cfg.vocab, d)),
        "final.norm": TensorExpectation((d,)),
    }
    for i, entry in enumerate(cfg.layers):
        p = f"l{i}."
        mx, mlp = entry["mixer"], entry.get("mlp")
        h, dim, vd = mx["heads"], mx["dim"], mx["vdim"]
        exp[p + "norm1"] = TensorExpectation((d,))
        if entry["type"] == "attention":
            g = mx["kv_heads"]
            exp.update({
                p + "mix.q": TensorExpectation((h * 2 * dim, d)),
                p + "mix.k": TensorExpectation((g * 2 * dim, d)),
                p + "mix.v": TensorExpectation((g * vd, d)),
                p + "mix.lq1": TensorExpectation((dim,)), p + "mix.lk1": TensorExpectation((dim,)),
                p + "mix.lq2": TensorExpectation((dim,)), p + "mix.lk2": TensorExpectation((dim,)),
                p + "mix.o": TensorExpectation((d, h * vd))})
        else:
            exp.update({
                p + "mix.q": TensorExpectation((h * dim, d)),
                p + "mix.k": TensorExpectation((h * dim, d)),
                p + "mix.v": TensorExpectation((h * vd, d)),
                p + "mix.g": TensorExpectation((h * vd, d)),
                p + "mix.o": TensorExpectation((d, h * vd))})
        if mlp is None:
            continue
        exp[p + "norm2"] = TensorExpectation((d,))
        n, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        for e in range(n):
            exp[f"{p}mlp.e{e}.up"] = TensorExpectation((ff, d))
            exp[f"{p}mlp.e{e}.down"] = TensorExpectation((d, ff))
        exp[p + "mlp.router"] = TensorExpectation((n, d))
    return exp


def random_tensors(cfg: PezaraxConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Seeded initialisation: matrices N(0, 1/in), the token table N(0, 1) / embedding scale
    (so that the stream starts near unit size), norm weights 1 + N(0, 0.1), the lambda vectors
    N(0, 0.3 / dim^(1/4)) (their dot products stay small), routers N(0, 4/in) (scores that spread); every tensor from a generator
    of its own."""
    out: Dict[str, torch.Tensor] = {}
    for name, exp in expected_tensors(cfg).items():
        if name == "embed":
            out[name] = normal(seed, name, exp.shape, 1.0 / max(abs(cfg.embedding_scale), 1e-6))
        elif name.endswith(("norm", "norm1", "norm2")):
            out[name] = normal(seed, name, exp.shape, 0.1, mean=1.0)
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            out[name] = normal(seed, name, exp.shape, 0.3 * exp.shape[0] ** -0.25)
        elif name.endswith(".router"):
            out[name] = normal(seed, name, exp.shape, 2.0 / math.sqrt(exp.shape[-1]))
        else:
            out[name] = normal(seed, name, exp.shape, 1.0 / math.sqrt(exp.shape[-1]))
    return out


def _retention(heads, dim, vdim, mlp, rot_dims=None, base=10000.0):
    # decays 1 - 2^-(5 + j): short memories on the first heads, long ones on the last
    return {"type": "retention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                      "decay": [1.0 - 2.0 ** (-5.0 - 3.0 * j / max(1, heads - 1)) for j in range(heads)],
                      "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}},
            "mlp": mlp}


def _attention(heads, kv_heads, dim, vdim, block, mlp, rot_dims=None, base=10000.0, diff=0.2):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                      "scale": 1.0 / math.sqrt(dim), "diff": diff, "mask": {"size": block},
                      "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}},
            "mlp": mlp}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _sized(vocab, width, layers, loop=None, scale=8.0, logit_scale=1.0):
    out = {"architecture": "Pezarax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
           "embedding": {"scale": scale}, "logit_scale": logit_scale, "layers": layers}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


#: Sizes a random-weight model can be asked for by name.  ``pezarax-small`` has the width, depth
#: (12 layer runs: 8 layers of which 2 run three times), head count and vocabulary of GPT-2
#: small, three retention layers to one attention layer, and 8 experts of 1,536 of which 2 run
#: (as many numbers at work per token as GPT-2's feed-forward of 3,072).  ``pezarax-wide`` has
#: GPT-2 XL's width with heads of 128.
NAMED_SIZES = {
    "pezarax-tiny": _sized(384, 64, [
        _retention(2, 16, 24, _moe(4, 2, 24), rot_dims=8),
        _attention(4, 2, 16, 24, 20, _moe(3, 1, 40), rot_dims=12, diff=0.25),
        _retention(4, 8, 16, None),
        _attention(2, 2, 24, 8, 48, _moe(4, 2, 24))], loop=(1, 3, 2), scale=6.0, logit_scale=0.7),
    "pezarax-small": _sized(50257, 768, [
        (_attention(12, 4, 32, 64, 512, _moe(8, 2, 1536)) if i % 4 == 2
         else _retention(12, 64, 64, _moe(8, 2, 1536))) for i in range(8)], loop=(2, 4, 3)),
    "pezarax-wide": _sized(50257, 1600, [
        (_attention(25, 5, 64, 128, 1024, _moe(8, 2, 3200)) if i % 4 == 2
         else _retention(25, 128, 128, _moe(8, 2, 3200))) for i in range(8)], loop=(2, 4, 3)),
}


def build(cfg: PezaraxConfig, store, runtime):
    from .assembly import build_model
    return build_model(cfg, store, runtime)


ARCHITECTURE = Architecture(
    name="Pezarax",
    config_class=PezaraxConfig,
    build=build,
    expected_tensors=expected_tensors,
    random_tensors=random_tensors,
    named_sizes=NAMED_SIZES,
)
register_architecture(PezaraxConfig.identifiers, ARCHITECTURE)
