"""Redisun configuration: a decoder whose layers are listed one by one in ``config.json``.

Keys read (nothing else exists in the design):

``vocab``, ``width``            sizes of the token table / head and of the residual stream
``embedding.bigram``            ``buckets``, ``mul_prev``, ``mul_cur`` of the hashed table of
                                (previous token, token) pairs; absent: token rows alone
``norm.eps``                    epsilon of every root-mean-square norm
``postln_alpha``                scale of the stream where a branch joins it
``layers[i]``                   ``type`` (the mixer), ``mixer`` (its sizes and constants) and
                                ``mlp`` (``kind`` dense or moe with its sizes, or null)

Every layer is a ``post_norm_gated`` block: x <- norm(alpha x + sigmoid(W x + b) * branch(x)),
for the mixer and then for the feed-forward.  The design names no position limit; a loaded
model's limit is what its page pool holds (``position_limit`` caps it).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec

_MIXERS = ("latent_attention",)
_MLP_KINDS = ("dense", "moe")


def _int(d: Dict[str, Any], key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d: Dict[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class RedisunConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    postln_alpha: float
    layers: tuple                           # the raw layer entries, validated
    bigram: Optional[Dict[str, int]] = None
    position_limit: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    identifiers = ("Redisun",)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "RedisunConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        bigram = (raw.get("embedding") or {}).get("bigram")
        if bigram is not None:
            bigram = {"buckets": _int(bigram, "buckets", "embedding.bigram"),
                      "mul_prev": _int(bigram, "mul_prev", "embedding.bigram", 0),
                      "mul_cur": _int(bigram, "mul_cur", "embedding.bigram", 0)}
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  eps=_num(norm, "eps", "norm"), postln_alpha=_num(raw, "postln_alpha", "config"),
                  layers=tuple(copy.deepcopy(layers)), bigram=bigram,
                  position_limit=int(raw.get("position_limit", 1 << 20)),
                  raw=copy.deepcopy(raw))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.eps < 0.0:
            raise ConfigError("config.json: norm.eps must not be negative")
        for i, entry in enumerate(self.layers):
            where = f"layers[{i}]"
            if entry.get("type") not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type {entry.get('type')!r} is not one of "
                                  f"{list(_MIXERS)}")
            mx = entry.get("mixer")
            if not isinstance(mx, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                _int(mx, key, where + ".mixer")
            _int(mx, "rot_dim", where + ".mixer", 0)
            _num(mx, "scale", where + ".mixer")
            rot = mx.get("rot") or {}
            dims = _int(rot, "dims", where + ".mixer.rot", 0)
            _num(rot, "base", where + ".mixer.rot")
            if dims % 2 or dims > mx["rot_dim"]:
                raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most "
                                  f"rot_dim, got {dims}")
            mlp = entry.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") not in _MLP_KINDS:
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not one of "
                                  f"{list(_MLP_KINDS)}")
            if mlp["kind"] == "dense":
                _int(mlp, "ff", where + ".mlp")
            else:
                _int(mlp.get("expert") or {}, "ff", where + ".mlp.expert")
                _num(mlp.get("expert") or {}, "limit", where + ".mlp.expert")
                experts = _int(mlp.get("router") or {}, "experts", where + ".mlp.router")
                top = _int(mlp.get("router") or {}, "top", where + ".mlp.router")
                if top > experts:
                    raise ConfigError(f"config.json: {where}.mlp.router.top exceeds experts")
                if mlp.get("shared") is not None:
                    _int(mlp["shared"], "ff", where + ".mlp.shared")
                    _num(mlp["shared"], "limit", where + ".mlp.shared")

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": "Redisun", "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.eps}, "postln_alpha": self.postln_alpha,
            "layers": copy.deepcopy(list(self.layers))}
        if self.bigram is not None:
            out["embedding"] = {"bigram": dict(self.bigram)}
        if self.position_limit != 1 << 20:
            out["position_limit"] = self.position_limit
        return out

    # ---------------------------------------------------------------- structure
    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        for i, entry in enumerate(self.layers):
            p = f"l{i}."
            mx, mlp = entry["mixer"], entry.get("mlp")
            mixer = PartSpec("latent_attention", {
                "weights": {"q_down": p + "mix.dq", "q_norm": p + "mix.dq.norm",
                            "q_up": p + "mix.uq", "kv_down": p + "mix.dkv",
                            "kv_norm": p + "mix.dkv.norm", "k_up": p + "mix.uk",
                            "v_up": p + "mix.uv", "sink": p + "mix.sink", "gate": p + "mix.g",
                            "out": p + "mix.o"},
                "width": self.width, "heads": mx["heads"], "dim": mx["dim"],
                "rot_dim": mx["rot_dim"], "vdim": mx["vdim"], "kv_rank": mx["kv_rank"],
                "q_rank": mx["q_rank"], "scale": float(mx["scale"]), "eps": self.eps,
                "rot_base": float(mx["rot"]["base"]), "rot_dims": mx["rot"]["dims"],
                "sink": True, "head_gate": True, "window": None})
            norms = {"mixer": PartSpec("rms_norm", {"gain": p + "norm1", "eps": self.eps,
                                                    "size": self.width})}
            if mlp is None:
                ff = PartSpec("none", {})
            else:
                norms["feed_forward"] = PartSpec("rms_norm", {"gain": p + "norm2", "eps": self.eps,
                                                              "size": self.width})
                if mlp["kind"] == "dense":
                    ff = PartSpec("gated_mlp", {
                        "weights": {"gate": p + "mlp.gate", "up": p + "mlp.up",
                                    "down": p + "mlp.down"},
                        "width": self.width, "inner": mlp["ff"], "limit": 0.0, "act_alpha": 1.0,
                        "up_shift": 0.0})
                else:
                    shared = mlp.get("shared")
                    ff = PartSpec("gated_moe", {
                        "prefix": p + "mlp.", "width": self.width,
                        "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                        "inner": mlp["expert"]["ff"], "limit": float(mlp["expert"]["limit"]),
                        "shared_inner": shared["ff"] if shared else 0,
                        "shared_limit": float(shared["limit"]) if shared else 0.0,
                        "act_alpha": 1.702, "up_shift": 1.0})
            gates = {"mixer": p + "rg1"}
            if mlp is not None:
                gates["feed_forward"] = p + "rg2"
            params = {"alpha": self.postln_alpha, "gates": gates}
            if mlp is None:
                params["norm_alone"] = {"gain": p + "norm2", "eps": self.eps}
            specs.append(LayerSpec(prefix=p, arrangement="post_norm_gated", mixer=mixer,
                                   feed_forward=ff, norms=norms, width=self.width,
                                   arrangement_params=params))
        return specs

    def embedding_spec(self) -> PartSpec:
        if self.bigram is None:
            return PartSpec("token_embedding", {"weights": "embed", "suffix": "",
                                                "vocab": self.vocab, "width": self.width})
        return PartSpec("token_pair_embedding", {
            "table": "embed", "pairs": "bigram", "vocab": self.vocab, "width": self.width,
            **self.bigram})

    def final_norm_spec(self) -> PartSpec:
        return PartSpec("rms_norm", {"gain": "final.norm", "eps": self.eps, "size": self.width})

    def head_spec(self) -> PartSpec:
        return PartSpec("linear_head", {"weights": "head", "vocab": self.vocab,
                                        "width": self.width})

    @property
    def max_positions(self) -> int:
        return self.position_limit
