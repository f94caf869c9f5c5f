"""Redisun's configuration, tensor list and cache layout (no GPU)."""
import copy

import pytest
import torch

import plain_redisun as P


def _raw():
    from pretrained_rstr_b200.config.registry import named_sizes
    return copy.deepcopy(named_sizes()["redisun-tiny"])


def test_registry_finds_the_design_by_its_architecture_key():
    from pretrained_rstr_b200.config.registry import lookup, registered
    raw = _raw()
    assert "Redisun" in registered()
    arch = lookup(raw)
    cfg = arch.config_class.from_dict(raw)
    assert cfg.to_dict()["layers"] == raw["layers"]
    assert arch.config_class.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_layer_specs_follow_the_layer_list():
    from pretrained_rstr_b200.config.registry import lookup
    raw = _raw()
    cfg = lookup(raw).config_class.from_dict(raw)
    specs = cfg.layer_specs()
    assert [s.feed_forward.kind for s in specs] == ["gated_mlp", "gated_moe", "none"]
    assert all(s.arrangement == "post_norm_gated" for s in specs)
    assert set(specs[2].norms) == {"mixer"} and set(specs[0].norms) == {"mixer", "feed_forward"}
    assert specs[2].mixer.params["rot_dims"] == 8 and specs[2].mixer.params["rot_dim"] == 16
    assert specs[1].arrangement_params["alpha"] == raw["postln_alpha"]
    raw["layers"].reverse()                                   # another order is another model
    other = lookup(raw).config_class.from_dict(raw).layer_specs()
    assert [s.feed_forward.kind for s in other] == ["none", "gated_moe", "gated_mlp"]
    assert other[0].prefix == "l0."
    del raw["embedding"]
    assert lookup(raw).config_class.from_dict(raw).embedding_spec().kind == "token_embedding"


@pytest.mark.parametrize("change,match", [
    (lambda r: r["layers"][0].update(type="ring"), "type"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda r: r["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.update(width=0), "width"),
])
def test_bad_configurations_are_refused(change, match):
    from pretrained_rstr_b200.config.base import ConfigError
    from pretrained_rstr_b200.config.registry import lookup
    raw = _raw()
    change(raw)
    with pytest.raises(ConfigError, match=match):
        lookup(raw).config_class.from_dict(raw)


def test_random_folder_has_exactly_the_expected_tensors(tmp_path):
    from pretrained_rstr_b200.config.registry import lookup
    from pretrained_rstr_b200.weights import make_random_model
    from pretrained_rstr_b200.weights.loader import WeightError, load_weights
    raw = _raw()
    arch = lookup(raw)
    cfg = arch.config_class.from_dict(raw)
    make_random_model(str(tmp_path), cfg, 4, torch.bfloat16)
    got_cfg, tensors = P.read_folder(str(tmp_path))
    exp = arch.expected_tensors(cfg)
    assert set(tensors) == {n for n, e in exp.items() if not e.optional}
    assert [n for n, e in exp.items() if e.optional] == ["l2.norm2"]
    assert all(tuple(tensors[n].shape) == tuple(exp[n].shape) for n in tensors)
    assert tensors["final.norm"].shape == () and "l2.norm2" not in tensors and "l2.rg2" not in tensors
    assert tensors["bigram"].shape[0] == raw["embedding"]["bigram"]["buckets"] + 1
    store = load_weights(str(tmp_path), exp, "cpu")
    assert store.get("l1.mlp.router.b").dtype == torch.bfloat16
    raw["layers"][0]["mixer"]["kv_rank"] += 8                 # the file no longer fits
    other = arch.config_class.from_dict(raw)
    with pytest.raises(WeightError, match="l0.mix.dkv"):
        load_weights(str(tmp_path), arch.expected_tensors(other), "cpu")
    # the plain implementation runs the folder it read
    logits = P.forward([3, 1, 4, 1, 5], tensors, got_cfg)
    assert logits.shape == (5, raw["vocab"]) and bool(torch.isfinite(logits).all())


def test_one_pool_per_layer_for_a_mixer_without_separate_values():
    from pretrained_rstr_b200.cache.manager import GroupSpec
    from pretrained_rstr_b200.cache.storage import CacheStorage
    groups = [GroupSpec("full.0", (0, 2), 1, 48, None, 1), GroupSpec("full.1", (1,), 2, 16, None)]
    st = CacheStorage(groups, [5, 3], 16, torch.float32, "cpu", {(-1, "previous_token"): type(
        "S", (), {"shape": (), "dtype": torch.int32})()}, 4)
    assert st.kv[0].shape == (2, 5, 1, 16, 48) and st.kv[1].shape == (2, 3, 2, 16, 16)
    k, v = st.layer_pages(0, 1)
    assert v is None and k.data_ptr() == st.kv[0][1].data_ptr()
    assert st.state[(-1, "previous_token")].shape == (4,)
    st.state[(-1, "previous_token")][1] = 9
    st.copy_state(1, 3)
    assert int(st.state[(-1, "previous_token")][3]) == 9


def test_plain_sink_softmax_and_rotation():
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=torch.float64)
    w = P.sink_softmax(s, torch.tensor([0.5], dtype=torch.float64))
    e = torch.exp(s)
    assert torch.allclose(w, e / (e.sum() + torch.exp(torch.tensor(0.5, dtype=torch.float64))))
    assert float(w.sum()) < 1.0
    v = torch.arange(12, dtype=torch.float64).reshape(2, 6) + 1
    r = P.rotate(v, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(r[0], v[0]) and torch.equal(r[1, 4:], v[1, 4:])       # position 0; unrotated rest
    assert torch.allclose((r[1, :4] ** 2).sum(), (v[1, :4] ** 2).sum())
    a = 3.0 * 100.0 ** (-2.0 / 4)
    assert abs(float(r[1, 1]) - (float(v[1, 1]) * torch.cos(torch.tensor(a)) -
                                 float(v[1, 3]) * torch.sin(torch.tensor(a)))) < 1e-9
