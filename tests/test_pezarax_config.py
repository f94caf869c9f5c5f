"""Pezarax without a GPU: the configuration reader, the run order with its caches, expected
tensors, random models on disk, and the plain implementation's own consistency."""
import copy

import pytest
import torch

import plain_pezarax as P
from pretrained_rstr_b200.config.base import ConfigError
from pretrained_rstr_b200.config.registry import lookup, named_size, read_config
from pretrained_rstr_b200.weights import make_random_model

RAW = {"architecture": "Pezarax", "vocab": 90, "width": 32, "norm": {"eps": 1e-6},
       "embedding": {"scale": 4.0}, "logit_scale": 0.5,
       "loop": {"start": 1, "stop": 3, "times": 3},
       "layers": [
           {"type": "retention", "mlp": None,
            "mixer": {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.9, 0.99], "rot": {"base": 100.0, "dims": 4}}},
           {"type": "attention", "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 10}},
            "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4, "diff": 0.3,
                      "mask": {"size": 7}, "rot": {"base": 50.0, "dims": 6}}},
           {"type": "retention", "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 6}},
            "mixer": {"heads": 1, "dim": 16, "vdim": 8, "decay": [0.95], "rot": {"base": 100.0, "dims": 16}}},
           {"type": "attention", "mlp": None,
            "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "diff": 0.1,
                      "mask": {"size": 5}, "rot": {"base": 50.0, "dims": 0}}}]}


def test_registry_and_structure():
    arch = lookup(RAW)
    cfg = arch.config_class.from_dict(RAW)
    assert arch.name == "Pezarax" and cfg.to_dict()["loop"] == RAW["loop"]
    order = cfg.run_order()
    assert [e.layer for e in order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.cache_layer for e in order] == [0, 1, 2, 4, 5, 6, 7, 3]         # a cache per pass
    assert [e.add_embedding for e in order] == [False, False, False, True, False, True, False, False]
    assert [(a, b) for a, b in P.run_order(RAW)] == [(e.layer, e.add_embedding) for e in order]
    specs = cfg.layer_specs()
    assert [s.mixer.kind for s in specs] == ["retention", "differential_attention"] * 2
    assert [s.feed_forward.kind for s in specs] == ["none", "routed_experts", "routed_experts", "none"]
    assert specs[1].mixer.params["block"] == 7 and specs[1].mixer.params["out_scale"] == pytest.approx(0.7)
    assert set(specs[0].norms) == {"mixer"} and set(specs[1].norms) == {"mixer", "feed_forward"}
    exp = arch.expected_tensors(cfg)
    assert exp["l1.mix.q"].shape == (4 * 2 * 6, 32) and exp["l1.mix.k"].shape == (2 * 2 * 6, 32)
    assert exp["l1.mix.v"].shape == (2 * 10, 32) and exp["l2.mix.g"].shape == (8, 32)
    assert "l0.norm2" not in exp and "l1.mlp.e2.down" in exp and "l2.mlp.e2.up" not in exp
    no_loop = copy.deepcopy(RAW)
    del no_loop["loop"]
    assert [e.cache_layer for e in arch.config_class.from_dict(no_loop).run_order()] == [0, 1, 2, 3]


@pytest.mark.parametrize("change", [
    lambda r: r["layers"][0].__setitem__("type", "convolution"),
    lambda r: r["layers"][0]["mixer"].__setitem__("decay", [0.9]),
    lambda r: r["layers"][1]["mixer"].__setitem__("kv_heads", 3),
    lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 5),
    lambda r: r["layers"][1]["mlp"]["router"].__setitem__("top", 4),
    lambda r: r["loop"].__setitem__("stop", 9),
    lambda r: r.__delitem__("logit_scale"),
    lambda r: r["embedding"].__delitem__("scale")])
def test_bad_configurations_are_refused(change):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError):
        lookup(raw).config_class.from_dict(raw)


def test_random_folder_round_trip_and_plain_consistency(tmp_path):
    """A random model written by the package is read by the plain implementation's own reader;
    the plain model is causal, its blocks hide what they should, and its state carries."""
    arch = lookup(RAW)
    cfg = arch.config_class.from_dict(RAW)
    folder = str(tmp_path / "m")
    make_random_model(folder, cfg, 3, torch.float32)
    assert read_config(folder)[1].to_dict() == cfg.to_dict()
    raw, tensors = P.read_folder(folder)
    assert set(tensors) == set(arch.expected_tensors(cfg))
    ids = [5, 17, 3, 80, 41, 2, 2, 9, 63, 30, 11, 7, 55]
    taps = []
    full = P.forward(ids, tensors, raw, taps=taps)
    assert full.shape == (len(ids), 90) and len(taps) == 8
    assert torch.allclose(P.forward(ids[:6], tensors, raw), full[:6], atol=1e-10)       # causal
    mask = P.chunk_mask(12, 5)
    assert bool(mask[5, 5]) and not bool(mask[5, 4]) and bool(mask[9, 5]) and not bool(mask[10, 9])
    q, k, v = torch.randn(6, 1, 4).double(), torch.randn(6, 1, 4).double(), torch.randn(6, 1, 3).double()
    whole, _ = P.decayed_states(q, k, v, [0.9])
    _, mid = P.decayed_states(q[:4], k[:4], v[:4], [0.9])
    rest, _ = P.decayed_states(q[4:], k[4:], v[4:], [0.9], state=mid)
    assert torch.allclose(rest, whole[4:], atol=1e-12)
    # the expert's weight acts on its input: relu(w u)^2 = w^2 relu(u)^2
    h = torch.randn(3, 32).double()
    out = P.routed_experts(h, tensors, "l2.", RAW["layers"][2]["mlp"])
    s = torch.sigmoid(h @ tensors["l2.mlp.router"].double().T)
    for i in range(3):
        e = int(s[i].argmax())
        u = torch.relu(h[i] @ tensors[f"l2.mlp.e{e}.up"].double().T) ** 2
        assert torch.allclose(out[i], s[i, e] ** 2 * (u @ tensors[f"l2.mlp.e{e}.down"].double().T), atol=1e-10)


def test_named_sizes():
    for name in ("pezarax-tiny", "pezarax-small", "pezarax-wide"):
        arch, cfg = named_size(name)
        assert arch.name == "Pezarax" and len(cfg.run_order()) >= len(cfg.layers)
