"""The Guronex configuration: config.json -> spec -> parts, without a GPU."""

import copy
import json

import pytest
import torch

from tests.guronex_util import CONFIGS, tensor_shapes


@pytest.mark.parametrize("tag", sorted(CONFIGS))
def test_the_parts_ask_for_exactly_the_designs_tensors(tag):
    from jax_vllm_b200 import registry
    from jax_vllm_b200.parts import BuildContext, Model
    c = CONFIGS[tag]
    cfg = registry.config_from_dict(copy.deepcopy(c))
    assert type(cfg).__name__ == "GuronexConfig"
    model = Model(cfg.to_spec(), BuildContext(dtype=torch.float32, device=torch.device("cpu")))
    specs = model.tensor_specs()
    assert {k: tuple(v.shape) for k, v in specs.items()} == tensor_shapes(c)
    assert json.loads(json.dumps(cfg.to_dict())) == c                       # what was read is what is written


def test_layers_are_read_one_by_one():
    from jax_vllm_b200 import registry
    spec = registry.config_from_dict(copy.deepcopy(CONFIGS["gc"])).to_spec()
    assert [ly.cache_from for ly in spec.layers] == [None, None, 0, 1]
    assert [ly.mixer.num_heads for ly in spec.layers] == [8, 8, 8, 4]
    assert [ly.mixer.position.theta for ly in spec.layers] == [1e4, 1e6, 1e4, 1e6]
    assert [(ly.feed_forward.n_groups, ly.feed_forward.keep_groups) for ly in spec.layers] == [(2, 1), (1, 1), (4, 3), (2, 1)]
    assert [ly.token_input.offset for ly in spec.layers] == [0, 12, 24, 36]
    assert all(ly.residual_scale == 0.25 and ly.kind == "branch_norm" for ly in spec.layers)
    ga = registry.config_from_dict(copy.deepcopy(CONFIGS["ga"])).to_spec()
    assert ga.layers[2].feed_forward is None and ga.layers[2].ffn_norm is None
    gb = registry.config_from_dict(copy.deepcopy(CONFIGS["gb"])).to_spec()
    assert all(ly.token_input is None for ly in gb.layers)


def test_cache_groups_follow_the_row_size_and_readers_keep_none():
    from jax_vllm_b200 import registry
    from jax_vllm_b200.cache import CacheManager
    from jax_vllm_b200.parts import BuildContext, Model
    for tag, groups in (("gb", [[0], [1]]), ("gc", [[0, 1]]), ("ga", [[0, 2]])):
        model = Model(registry.config_from_dict(copy.deepcopy(CONFIGS[tag])).to_spec(),
                      BuildContext(dtype=torch.float32, device=torch.device("cpu")))
        cache = CacheManager(model.cache_needs(), 16, 8, 4)
        assert [g.layers for g in cache.groups] == groups
        assert all(g.need.shared_kv and g.need.num_kv_heads == 1 for g in cache.groups)
        views = cache.allocate_storage(torch.float32, "cpu")
        assert all(v.k.data_ptr() == v.v.data_ptr() for v in views.values())                       # keys and values are one tensor
    assert model.place_cache == [0, 0, 2]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0]["mixer"].update(kv_from=0), "earlier layer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=32), "must equal those of layer 0"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8), "rot.dims must equal rot_dim"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router sizes do not fit"),
    (lambda c: c["layers"][0].update(type="other"), "not part of this design"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not part of this design"),
    (lambda c: c.pop("residual_mult"), "lacks"),
])
def test_what_does_not_fit_is_refused(change, message):
    from jax_vllm_b200 import registry
    c = copy.deepcopy(CONFIGS["ga"])
    change(c)
    with pytest.raises((ValueError, KeyError), match=message):
        registry.config_from_dict(c)


def test_the_oracle_route_keeps_to_the_best_groups():
    """The plain implementation itself, on a case worked by hand: 8 experts in 4 groups, 2 groups kept."""
    from tests.plain.guronex_plain import route
    z = torch.log(torch.tensor([[0.05, 0.30, 0.02, 0.03, 0.25, 0.01, 0.20, 0.14]], dtype=torch.float64))
    w = torch.eye(8, dtype=torch.float64)
    # groups (0,1) (2,3) (4,5) (6,7) score 0.30, 0.03, 0.25, 0.20: groups 0 and 2 stay; expert 6 (0.20) may not be chosen
    chosen, weight = route(z, w, {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}})
    assert chosen.tolist() == [[1, 4, 0]]
    assert torch.allclose(weight, torch.tensor([[0.30, 0.25, 0.05]], dtype=torch.float64))
    chosen, _ = route(z, w, {"experts": 8, "top": 3})
    assert chosen.tolist() == [[1, 4, 6]]
