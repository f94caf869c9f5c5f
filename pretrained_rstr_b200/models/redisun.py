"""Redisun as data for the engine: tensor names and shapes, random initialisation, named
sizes, registration.  The model is put together by
:func:`pretrained_rstr_b200.models.assembly.build_model` from the parts that
``RedisunConfig.layer_specs()`` names.

Tensor names: ``embed`` [vocab, width], ``bigram`` [buckets + 1, width], ``head`` [vocab,
width], ``final.norm`` [] and per layer i ``l<i>.norm1``, ``l<i>.norm2`` [], ``l<i>.rg1``,
``l<i>.rg2`` [width, width] with ``.b`` [width], the mixer's ``l<i>.mix.*`` and the
feed-forward's ``l<i>.mlp.*``; matrices are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..config.redisun import RedisunConfig
from ..config.registry import Architecture, register_architecture
from ..weights.loader import TensorExpectation, normal


def _gated(prefix: str, width: int, inner: int) -> Dict[str, TensorExpectation]:
    return {prefix + "gate": TensorExpectation((inner, width)),
            prefix + "up": TensorExpectation((inner, width)),
            prefix + "down": TensorExpectation((width, inner))}


def expected_tensors(cfg: RedisunConfig) -> Dict[str, TensorExpectation]:
    d = cfg.width
    exp: Dict[str, TensorExpectation] = {
        "embed": TensorExpectation((cfg.vocab, d)),
        "head": TensorExpectation((cfg.vocab, d)),
        "final.norm": TensorExpectation(()),
    }
    if cfg.bigram is not None:
        exp["bigram"] = TensorExpectation((cfg.bigram["buckets"] + 1, d))
    for i, entry in enumerate(cfg.layers):
        p = f"l{i}."
        mx, mlp = entry["mixer"], entry.get("mlp")
        h, dim, rot, vd = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"]
        rank, qr = mx["kv_rank"], mx["q_rank"]
        exp.update({
            p + "norm1": TensorExpectation(()),
            p + "rg1": TensorExpectation((d, d)), p + "rg1.b": TensorExpectation((d,)),
            p + "mix.dq": TensorExpectation((qr, d)), p + "mix.dq.norm": TensorExpectation((qr,)),
            p + "mix.uq": TensorExpectation((h * (dim + rot), qr)),
            p + "mix.dkv": TensorExpectation((rank + rot, d)),
            p + "mix.dkv.norm": TensorExpectation((rank,)),
            p + "mix.uk": TensorExpectation((h * dim, rank)),
            p + "mix.uv": TensorExpectation((h * vd, rank)),
            p + "mix.sink": TensorExpectation((h,)),
            p + "mix.g": TensorExpectation((h, d)),
            p + "mix.o": TensorExpectation((d, h * vd)),
        })
        if mlp is None:
            # (a file may still carry the second norm of a layer without a feed-forward; it is
            # then applied to the scaled stream alone)
            exp[p + "norm2"] = TensorExpectation((), optional=True)
            continue
        exp.update({p + "norm2": TensorExpectation(()),
                    p + "rg2": TensorExpectation((d, d)), p + "rg2.b": TensorExpectation((d,))})
        if mlp["kind"] == "dense":
            exp.update(_gated(p + "mlp.", d, mlp["ff"]))
        else:
            n = mlp["router"]["experts"]
            for e in range(n):
                exp.update(_gated(f"{p}mlp.e{e}.", d, mlp["expert"]["ff"]))
            exp[p + "mlp.router"] = TensorExpectation((n, d))
            exp[p + "mlp.router.b"] = TensorExpectation((n,))
            if mlp.get("shared"):
                exp.update(_gated(p + "mlp.shared.", d, mlp["shared"]["ff"]))
    return exp


def random_tensors(cfg: RedisunConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Seeded initialisation: matrices N(0, 1/in), tables N(0, 1), norm weights and gains
    1 + N(0, 0.1), sinks and biases N(0, 0.5); every tensor from a generator of its own."""
    out: Dict[str, torch.Tensor] = {}
    for name, exp in expected_tensors(cfg).items():
        if exp.optional:
            continue
        if name in ("embed", "bigram"):
            out[name] = normal(seed, name, exp.shape, 1.0)
        elif name.endswith(("norm", "norm1", "norm2")):
            out[name] = normal(seed, name, exp.shape, 0.1, mean=1.0)
        elif name.endswith((".b", ".sink")):
            out[name] = normal(seed, name, exp.shape, 0.5)
        else:
            out[name] = normal(seed, name, exp.shape, 1.0 / math.sqrt(exp.shape[-1]))
    return out


def _layer(heads, dim, rot_dim, vdim, kv_rank, q_rank, mlp, rot_dims=None, base=10000.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                      "kv_rank": kv_rank, "q_rank": q_rank,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
                      "scale": 1.0 / math.sqrt(dim + rot_dim)},
            "mlp": mlp}


def _moe(experts, top, ff, shared_ff, limit=7.0):
    return {"kind": "moe", "router": {"experts": experts, "top": top},
            "expert": {"ff": ff, "limit": limit},
            "shared": {"ff": shared_ff, "limit": limit} if shared_ff else None}


def _sized(vocab, width, layers, buckets):
    return {"architecture": "Redisun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "postln_alpha": 2.0, "layers": layers,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": 31, "mul_cur": 5}}}


#: Sizes a random-weight model can be asked for by name.  ``redisun-small`` has the width,
#: depth, head count and vocabulary of GPT-2 small (its gated feed-forward of 2,048 holds as
#: many numbers as GPT-2's of 3,072); ``redisun-small-moe`` swaps every second feed-forward
#: for eight experts of which two run, plus a shared one; ``redisun-wide`` has GPT-2 XL's width
#: and head count with heads of 128 + 64 dimensions over a latent of 256 (the most the
#: tensor-core attention kernel takes; a wider latent runs on the 32-bit-arithmetic kernel).
NAMED_SIZES = {
    "redisun-tiny": _sized(384, 48, [
        _layer(3, 16, 8, 16, 24, 16, {"kind": "dense", "ff": 64}),
        _layer(3, 16, 8, 16, 24, 16, _moe(6, 2, 16, 32, limit=1.5)),
        _layer(2, 24, 16, 8, 40, 32, None, rot_dims=8)], 211),
    "redisun-small": _sized(50257, 768, [
        _layer(12, 64, 32, 64, 256, 384, {"kind": "dense", "ff": 2048}) for _ in range(12)], 65521),
    "redisun-small-moe": _sized(50257, 768, [
        _layer(12, 64, 32, 64, 256, 384,
               {"kind": "dense", "ff": 2048} if i % 2 == 0 else _moe(8, 2, 512, 1024))
        for i in range(12)], 65521),
    "redisun-wide": _sized(50257, 1600, [
        _layer(25, 128, 64, 128, 256, 768, {"kind": "dense", "ff": 4096}) for _ in range(12)], 65521),
}


def build(cfg: RedisunConfig, store, runtime):
    from .assembly import build_model
    return build_model(cfg, store, runtime)


ARCHITECTURE = Architecture(
    name="Redisun",
    config_class=RedisunConfig,
    build=build,
    expected_tensors=expected_tensors,
    random_tensors=random_tensors,
    named_sizes=NAMED_SIZES,
)
register_architecture(RedisunConfig.identifiers, ARCHITECTURE)
