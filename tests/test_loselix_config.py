"""Loselix: config.json -> configuration -> ModelSpec, on the CPU."""

from __future__ import annotations

import copy

import pytest
import torch

from jax_vllm_b200 import registry
from jax_vllm_b200.models.loselix import LoselixConfig
from jax_vllm_b200.parts import BuildContext, Model
from tests.loselix_util import CONFIGS, config, layer, sig, soft, tensor_shapes, twin
from tests.plain import loselix_plain as lp


@pytest.mark.parametrize("tag", sorted(CONFIGS))
def test_tensor_names_shapes_and_round_trip(tag):
    c = CONFIGS[tag]
    cfg = registry.config_from_dict(c)
    assert isinstance(cfg, LoselixConfig)
    assert LoselixConfig.from_dict(cfg.to_dict()) == cfg
    model = Model(cfg.to_spec(), BuildContext(dtype=torch.float32, device=torch.device("cpu")))
    assert {k: tuple(v.shape) for k, v in model.tensor_specs().items()} == tensor_shapes(c)


def test_run_order_and_where_the_embedding_is_added_again():
    five = [layer(soft(2, 1, 16, 16, rot=4), 8) for _ in range(5)]
    for loop, order, again in ((None, (0, 1, 2, 3, 4), ()),
                               ((0, 5, 2), (0, 1, 2, 3, 4, 0, 1, 2, 3, 4), (5,)),
                               ((1, 3, 3), (0, 1, 2, 1, 2, 1, 2, 3, 4), (3, 5)),
                               ((4, 5, 2), (0, 1, 2, 3, 4, 4), (5,)),
                               ((2, 4, 1), (0, 1, 2, 3, 4), ())):
        c = config(50, 32, copy.deepcopy(five), loop=loop)
        spec = registry.config_from_dict(c).to_spec()
        assert tuple(spec.run_order()) == order and tuple(spec.reinject) == again
        # the plain implementation reads the same order from the same keys
        plain = lp.run_order(c)
        assert tuple(i for i, _ in plain) == order
        assert tuple(k for k, (_, add) in enumerate(plain) if add) == again
        # every place of the order keeps keys and values of its own
        model = Model(spec, BuildContext(dtype=torch.float32, device=torch.device("cpu")))
        assert len(model.cache_needs()) == len(order) and all(n is not None for n in model.cache_needs())


def test_mixers_become_options_of_one_attention_part():
    c = config(64, 48, [layer(twin(4, 2, 16, 24, rot=8, softcap=7.0, diff=0.2), 16), layer(soft(4, 4, 8, 12, rot=8), None),
                        layer(sig(3, 1, 16, coef=0.7, every=9), 16)], eps=2e-6)
    a, b, s = (ly.mixer for ly in registry.config_from_dict(c).to_spec().layers)
    assert a.kind == b.kind == s.kind == "general_attention"
    assert (a.twin.offset, a.twin.eps, a.score_cap, a.gate, a.weights) == (0.2, 2e-6, 7.0, None, "softmax")
    assert (a.key_dim, a.value_dim, a.position.dim) == (16, 24, 8)
    assert (b.gate, b.twin, b.score_cap, b.num_kv_heads, b.position.dim) == ("head", None, None, 4, 8)
    assert (s.weights, s.score_bias, s.gate, s.values_from_keys, s.whole_norm_eps) == ("sigmoid", True, "element", True, 2e-6)
    assert s.query_temperature == (0.7, 9) and s.position is None
    spec = registry.config_from_dict(c).to_spec()
    assert [ly.kind for ly in spec.layers] == ["parallel"] * 3 and spec.layers[1].feed_forward is None
    assert spec.layers[0].feed_forward.activation == "relu2"


def test_what_the_design_does_not_have_is_refused():
    good = config(64, 48, [layer(soft(4, 2, 16, 16, rot=8), 16)])
    for change, err in ((lambda c: c["layers"][0].update(type="attention_9"), ValueError),
                        (lambda c: c["layers"][0]["mixer"].update(heads=3), ValueError),
                        (lambda c: c["layers"][0]["mixer"].pop("scale"), KeyError),
                        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), ValueError),
                        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), ValueError),
                        (lambda c: c["layers"][0]["mlp"].update(kind="moe"), ValueError),
                        (lambda c: c.update(loop={"start": 0, "stop": 2, "times": 2}), ValueError),
                        (lambda c: c.update(loop={"start": 0, "stop": 1}), KeyError),
                        (lambda c: c.pop("norm"), KeyError)):
        c = copy.deepcopy(good)
        change(c)
        with pytest.raises(err):
            registry.config_from_dict(c)
    with pytest.raises(ValueError):
        registry.config_from_dict(config(64, 48, [{"type": "attention_3", "mlp": None,
                                                   "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 16, "scale": 1.0}}]))
    with pytest.raises(KeyError):
        registry.config_from_dict(config(64, 48, [layer({"type": "attention", "mixer": soft(2, 1, 8, 8)["mixer"]}, 8)]))


def test_plain_implementation_mechanisms():
    """The oracle's own parts against numbers worked out by hand."""
    y = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(lp.unit_rms(y, 0.0), y / (12.5 ** 0.5))
    # rotation by a quarter turn of the first pair (dims 2: one frequency of 1), the rest untouched
    pos = torch.tensor([0, 1])
    z = torch.tensor([[[1.0, 0.0, 5.0]], [[1.0, 0.0, 5.0]]], dtype=torch.float64)
    r = lp.rotate_first(z, pos, 2, 123.0)
    assert torch.allclose(r[0], z[0]) and torch.allclose(r[1, 0], torch.tensor([0.5403023, 0.8414710, 5.0], dtype=torch.float64), atol=1e-6)
    assert lp.query_temperature(torch.tensor([0, 6, 7, 15, 16]), 0.5, 8).tolist() == \
        pytest.approx([1.0, 1.0, 1 + 0.5 * 0.6931472, 1 + 0.5 * 1.0986123, 1 + 0.5 * 1.0986123], abs=1e-6)
    assert lp.tanh_cap(torch.tensor([1e6, 0.1], dtype=torch.float64), 5.0).tolist() == pytest.approx([5.0, 0.09998667], abs=1e-6)
    s = torch.zeros((1, 2, 2), dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[3.0]]], dtype=torch.float64)
    assert lp.softmax_attend(s, v).flatten().tolist() == [1.0, 2.0]                     # causal mean
    assert lp.sigmoid_attend(s, torch.zeros(1, dtype=torch.float64), v).flatten().tolist() == [0.5, 2.0]   # 0.5 * (1 + 3), not a mean
