"""Nipurax's configuration, run order, tensor names and cache needs, and its plain implementation's
mechanisms against hand-made cases. No GPU."""

import json
import math

import pytest
import torch

import plain_nipurax as plain
from atomserve_b200.config.model_config import ModelConfigError
from atomserve_b200.config.registry import config_from_dict
from atomserve_b200.parts.model import build_model
from tiny_nipurax import NIPURAX


@pytest.mark.parametrize("name", list(NIPURAX))
def test_configuration_round_trips_and_names_the_plain_tensors(name):
    cfg, _ = NIPURAX[name]
    arch, config = config_from_dict(json.loads(json.dumps(cfg)))
    assert arch.name == "Nipurax" and config.to_dict() == cfg
    model = build_model(arch.build_spec(config))
    have = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert have == plain.tensor_shapes(cfg)


def test_run_order_and_what_each_entry_keeps():
    cfg, _ = NIPURAX["a"]
    arch, config = config_from_dict(cfg)
    assert config.run_order() == plain.run_order(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    spec = arch.build_spec(config)
    assert [c.layer for c in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [c.before for c in spec.schedule] == [None, (0, 0), None, (0, 1), None, (0, 2), None, None]
    needs = build_model(spec).cache_requirements()
    assert len(needs) == 9  # every run of a layer keeps pages of its own; the embedding keeps the last token
    assert all(pages is not None for pages, _ in needs[:8]) and needs[8][0] is None
    assert needs[8][1][0].dtype == torch.int32
    # a head of two maps of 12 under values of 40 runs at 40; of two maps of 20 over values of 24 at 40 too
    assert needs[1][0].tensors[0].width == 40 and needs[7][0].tensors[0].width == 40 and needs[0][0].tensors[0].width == 24
    assert needs[1][0].tensors[0].heads == 2  # the two maps of a kv head share one key head
    assert needs[1][0].chunk == 10 and needs[7][0].chunk == 33 and needs[0][0].chunk is None  # pages of passed chunks go back
    no_loop, _ = NIPURAX["b"]
    arch, config = config_from_dict(no_loop)
    spec = arch.build_spec(config)
    assert spec.stream_steps == () and all(c.before is None for c in spec.schedule)


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].__setitem__("type", "attention_3"), "mixer type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "positive"),
    (lambda c: c["loop"].__setitem__("stop", 9), "does not fit"),
    (lambda c: c["loop"].__setitem__("times", 0), "does not fit"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 7), "cannot choose"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "moe"),
    (lambda c: c["embedding"]["bigram"].__setitem__("buckets", 0), "buckets"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].__setitem__("every", 0), "every"),
])  # fmt: skip
def test_rejections(change, words):
    cfg = json.loads(json.dumps(NIPURAX["a"][0]))
    change(cfg)
    with pytest.raises(ModelConfigError, match=words):
        config_from_dict(cfg)


def test_pair_rows_by_hand():
    assert plain.pair_rows([5, 9, 9, 0], 7, 3, 2) == [7, (15 + 18) % 7, (27 + 18) % 7, 27 % 7]
    assert plain.pair_rows([4], 11, 1, 1) == [11]


def test_stretched_frequencies_by_hand():
    """dims 4, base 100: f = (1, 0.1), wavelengths 6.28 and 62.8. original 64: 64 / high and 64 / low
    bound the band."""
    rot = dict(base=100.0, dims=4)
    plainf = plain.rotary_frequencies(rot)
    assert torch.allclose(plainf, torch.tensor([1.0, 0.1], dtype=torch.float64))
    # both waves shorter than 64 / 4 = 16? the first is, the second is longer than 64 / 2 = 32: divided
    f = plain.rotary_frequencies(dict(rot, scaling=dict(factor=8.0, low=2.0, high=4.0, original=64)))
    assert torch.allclose(f, torch.tensor([1.0, 0.1 / 8], dtype=torch.float64))
    # the second wave inside the band 64 / 4 .. 64 / 0.5 = 16 .. 128
    f = plain.rotary_frequencies(dict(rot, scaling=dict(factor=8.0, low=0.5, high=4.0, original=64)))
    s = (64 / (2 * math.pi / 0.1) - 0.5) / 3.5
    assert abs(float(f[1]) - ((1 - s) * 0.1 / 8 + s * 0.1)) < 1e-15 and float(f[0]) == 1.0


def test_the_package_makes_the_same_frequencies():
    from atomserve_b200.parts.base import build_part
    from atomserve_b200.parts.spec import PartSpec

    for base, dims, scaling in [(100.0, 8, (4.0, 1.0, 4.0, 64)), (50.0, 4, (16.0, 2.0, 3.0, 8)), (1000.0, 12, (2.0, 100.0, 400.0, 64)),
                                (400000.0, 32, (2.0, 0.001, 0.01, 4096)), (10000.0, 32, (6.0, 1.0, 3.0, 128))]:  # fmt: skip
        rot = dict(base=base, dims=dims, scaling=dict(zip(("factor", "low", "high", "original"), scaling)))
        part = build_part("position", PartSpec("band_scaled_rotary", dict(head_dim=dims, theta=base, rotary_dim=dims, factor=scaling[0],
                                                                          low=scaling[1], high=scaling[2], original=scaling[3])), 8)  # fmt: skip
        part.prepare(torch.device("cpu"))
        assert torch.allclose(part.inv_freq.double(), plain.rotary_frequencies(rot), rtol=1e-6, atol=0)


def test_visibility_in_chunks():
    ok = plain.visible(7, 3)
    assert ok[2, 0] and ok[2, 2] and not ok[3, 2] and ok[5, 3] and not ok[6, 5] and ok[6, 6] and not ok[1, 2]
    assert plain.visible(4, None).sum() == 10


def test_a_sink_takes_weight_and_gives_nothing():
    scores = torch.zeros(1, 1, 3, dtype=torch.float64)
    p = plain.softmax_with_sink(scores, torch.ones(1, 3, dtype=torch.bool), torch.tensor([math.log(3.0)]))
    assert torch.allclose(p, torch.full((1, 1, 3), 1 / 6, dtype=torch.float64))


def test_identity_experts_and_offsets_by_hand():
    """Two experts and one identity expert, top 2. The offsets change the choice, not the weights."""
    h = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    router = torch.tensor([[0.0, 0.0], [1.0, 0.0], [2.0, 0.0]])
    zero, away = torch.zeros(3), torch.tensor([10.0, 0.0, 0.0])
    s = torch.softmax(torch.tensor([0.0, 1.0, 2.0], dtype=torch.float64), 0)
    chosen, weights = plain.route(h, router, zero, 2, 2.0)
    assert chosen.tolist() == [[2, 1]] and torch.allclose(weights, 2.0 * s[[2, 1]][None])
    chosen, weights = plain.route(h, router, away, 2, 1.0)
    assert chosen.tolist() == [[0, 2]] and torch.allclose(weights, s[[0, 2]][None])
    w = {"router": router, "correction": away, "e0.gate": torch.tensor([[3.0, 0.0]]), "e0.up": torch.tensor([[-9.0, 0.0]]),
         "e0.down": torch.tensor([[1.0], [1.0]]), "e1.gate": torch.zeros(1, 2), "e1.up": torch.zeros(1, 2), "e1.down": torch.zeros(2, 1)}  # fmt: skip
    mlp = dict(expert=dict(ff=1, limit=2.0), router=dict(experts=2, identity=1, top=2, scale=1.0))
    # expert 0: g = min(3, 2) = 2, u = clamp(-9) = -2: 2 sigmoid(3.404) (-1); the identity expert gives h back
    e0 = 2.0 / (1.0 + math.exp(-3.404)) * -1.0
    out = plain.routed_experts(h, w, mlp)
    assert torch.allclose(out, s[0] * e0 * torch.ones(1, 2, dtype=torch.float64) + s[2] * h)
