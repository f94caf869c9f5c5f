"""Pezarax configuration: a decoder whose layers are listed one by one in ``config.json``,
some of which may run several times in a row.

Keys read (nothing else exists in the design):

``vocab``, ``width``       sizes of the token table / head and of the residual stream
``embedding.scale``        constant the token rows are multiplied by
``norm.eps``               epsilon of every root-mean-square norm
``logit_scale``            constant the logits are multiplied by
``layers[i]``              ``type`` (the mixer: ``attention`` or ``retention``), ``mixer`` (its
                           sizes and constants) and ``mlp`` (``kind`` moe with its sizes, or
                           null for a layer without a feed-forward)
``loop``                   optional ``start``, ``stop``, ``times``: layers start .. stop - 1 run
                           ``times`` times in a row with the same weights; every pass has a
                           cache and state of its own, and before every pass but the first the
                           embedding's output is added to the stream

Every layer is a ``pre_norm`` block.  The design names no position limit; a loaded model's
limit is what its page pool holds (``position_limit`` caps it).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, RunEntry

_MIXERS = ("attention", "retention")


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class PezaraxConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple                           # the raw layer entries, validated
    loop: Optional[Dict[str, int]] = None
    position_limit: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    identifiers = ("Pezarax",)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PezaraxConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        loop = raw.get("loop")
        if loop is not None:
            loop = {"start": _int(loop, "start", "loop", 0), "stop": _int(loop, "stop", "loop", 0),
                    "times": _int(loop, "times", "loop", 1)}
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  eps=_num(raw.get("norm"), "eps", "norm"),
                  embedding_scale=_num(raw.get("embedding"), "scale", "embedding"),
                  logit_scale=_num(raw, "logit_scale", "config"),
                  layers=tuple(copy.deepcopy(layers)), loop=loop,
                  position_limit=int(raw.get("position_limit", 1 << 20)),
                  raw=copy.deepcopy(raw))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.eps < 0.0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if self.loop is not None and not 0 <= self.loop["start"] <= self.loop["stop"] <= len(self.layers):
            raise ConfigError(f"config.json: loop {self.loop} does not lie within the "
                              f"{len(self.layers)} layers")
        for i, entry in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or entry.get("type") not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type must be one of {list(_MIXERS)}")
            mx = entry.get("mixer")
            if not isinstance(mx, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            for key in ("heads", "dim", "vdim"):
                _int(mx, key, where + ".mixer")
            rot = mx.get("rot")
            dims = _int(rot, "dims", where + ".mixer.rot", 0)
            _num(rot, "base", where + ".mixer.rot")
            if dims % 2 or dims > mx["dim"]:
                raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most "
                                  f"dim, got {dims}")
            if entry["type"] == "attention":
                kv = _int(mx, "kv_heads", where + ".mixer")
                if mx["heads"] % kv:
                    raise ConfigError(f"config.json: {where}.mixer.heads is no multiple of kv_heads")
                _num(mx, "scale", where + ".mixer")
                _num(mx, "diff", where + ".mixer")
                if mx.get("mask") is not None:
                    _int(mx["mask"], "size", where + ".mixer.mask")
            else:
                decay = mx.get("decay")
                if not isinstance(decay, list) or len(decay) != mx["heads"] or \
                        any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                    raise ConfigError(f"config.json: {where}.mixer.decay must list one number per head")
            mlp = entry.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"config.json: {where}.mlp.kind must be 'moe' (or mlp null)")
            _int(mlp.get("expert"), "ff", where + ".mlp.expert")
            experts = _int(mlp.get("router"), "experts", where + ".mlp.router")
            if _int(mlp.get("router"), "top", where + ".mlp.router") > experts:
                raise ConfigError(f"config.json: {where}.mlp.router.top exceeds experts")

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": "Pezarax", "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
            "logit_scale": self.logit_scale, "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.position_limit != 1 << 20:
            out["position_limit"] = self.position_limit
        return out

    # ---------------------------------------------------------------- structure
    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        for i, entry in enumerate(self.layers):
            p = f"l{i}."
            mx, mlp = entry["mixer"], entry.get("mlp")
            common = {"width": self.width, "heads": mx["heads"], "dim": mx["dim"],
                      "vdim": mx["vdim"], "eps": self.eps, "rot_base": float(mx["rot"]["base"]),
                      "rot_dims": mx["rot"]["dims"]}
            if entry["type"] == "attention":
                diff = float(mx["diff"])
                mixer = PartSpec("differential_attention", {
                    **common, "kv_heads": mx["kv_heads"], "scale": float(mx["scale"]),
                    "block": (mx.get("mask") or {}).get("size"),
                    "lambda_init": diff, "out_scale": 1.0 - diff,
                    "weights": {"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v",
                                "out": p + "mix.o", "lambda_q1": p + "mix.lq1",
                                "lambda_k1": p + "mix.lk1", "lambda_q2": p + "mix.lq2",
                                "lambda_k2": p + "mix.lk2"}})
            else:
                mixer = PartSpec("retention", {
                    **common, "decay": [float(d) for d in mx["decay"]],
                    "k_scale": float(mx["dim"]) ** -0.5,
                    "weights": {"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v",
                                "gate": p + "mix.g", "out": p + "mix.o"}})
            norms = {"mixer": PartSpec("rms_norm", {"weight": p + "norm1", "eps": self.eps,
                                                    "size": self.width})}
            if mlp is None:
                ff = PartSpec("none", {})
            else:
                norms["feed_forward"] = PartSpec("rms_norm", {"weight": p + "norm2", "eps": self.eps,
                                                              "size": self.width})
                ff = PartSpec("routed_experts", {
                    "prefix": p + "mlp.", "width": self.width,
                    "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                    "inner": mlp["expert"]["ff"], "activation": "relu_squared",
                    "score": "sigmoid", "renormalize": False, "weight_on": "input"})
            specs.append(LayerSpec(prefix=p, arrangement="pre_norm", mixer=mixer, feed_forward=ff,
                                   norms=norms, width=self.width))
        return specs

    def run_order(self) -> List[RunEntry]:
        """Layers in order; the looped span ``times`` times in a row.  The first pass uses the
        layers' own caches, every further pass caches numbered after the last layer, and its
        first entry has the embedding's output added before it."""
        n = len(self.layers)
        if self.loop is None:
            return [RunEntry(i, i) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [RunEntry(i, i) for i in range(a)]
        for rep in range(times):
            for i in range(a, b):
                cache = i if rep == 0 else n + (rep - 1) * (b - a) + (i - a)
                order.append(RunEntry(i, cache, True, add_embedding=rep > 0 and i == a))
        return order + [RunEntry(i, i) for i in range(b, n)]

    def embedding_spec(self) -> PartSpec:
        return PartSpec("scaled_token_embedding", {"weights": "embed", "vocab": self.vocab,
                                                   "width": self.width,
                                                   "scale": self.embedding_scale})

    def final_norm_spec(self) -> PartSpec:
        # (the logits' constant rides in the norm's 32-bit weight: no pass over the logits)
        return PartSpec("rms_norm", {"weight": "final.norm", "eps": self.eps, "size": self.width,
                                     "scale": self.logit_scale})

    def head_spec(self) -> PartSpec:
        return PartSpec("linear_head", {"weights": "head", "vocab": self.vocab,
                                        "width": self.width})

    @property
    def max_positions(self) -> int:
        return self.position_limit
