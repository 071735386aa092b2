"""The Tigesun configuration and model description on the CPU: keys, rejections, the round trip
through config.json, tensor names and shapes, the run order of layers that share tensors, what
each layer keeps between steps, and the stretched rotary encoding's frequencies."""

import copy
import math

import pytest
import torch

import plain_tigesun as plain
from tiny_tigesun import TIGESUN


def parse(raw):
    from atomserve_b200.config.registry import config_from_dict

    return config_from_dict(raw)


@pytest.mark.parametrize("name", list(TIGESUN))
def test_round_trip_and_tensor_list(name):
    from atomserve_b200.parts.model import build_model

    raw = TIGESUN[name][0]
    arch, config = parse(raw)
    assert arch.name == "Tigesun"
    assert parse(config.to_dict())[1] == config
    assert ("logit_softcap" in config.to_dict()) == ("logit_softcap" in raw)
    model = build_model(arch.build_spec(config))
    got = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert got == plain.tensor_shapes(raw)
    kinds = {s.name: s.kind for s in model.tensor_specs()}
    assert all(kinds[n] == ("matrix" if len(shape) == 2 and not n.endswith(".conv") else "gain") for n, shape in got.items())


def test_layers_that_run_anothers_tensors_keep_a_cache_of_their_own():
    from atomserve_b200.parts.model import build_model

    raw = TIGESUN["a"][0]
    arch, config = parse(raw)
    spec = arch.build_spec(config)
    assert len(spec.layers) == 3 and [c.layer for c in spec.schedule] == [0, 1, 2, 2, 0, 1, 2]
    assert all(c.cache_from is None for c in spec.schedule)
    needs = build_model(spec).cache_requirements()
    assert len(needs) == 7
    pages, state = needs[0]
    assert pages is None and [(s.name, tuple(s.shape)) for s in state] == [("s", (4, 24, 16)), ("conv", (3, 64 + 2 * 2 * 24))]
    assert needs[4][0] is None and [tuple(s.shape) for s in needs[4][1]] == [(4, 24, 16), (3, 160)]
    pages, state = needs[1]  # keys of 24 and values of 40 entries: pages at the larger of the two
    assert pages.window is None and [(t.name, t.heads, t.width) for t in pages.tensors] == [("k", 2, 40), ("v", 2, 40)] and not state
    for i in (2, 3, 6):
        pages, state = needs[i]
        assert pages.window == 20 and [(t.name, t.heads, t.width) for t in pages.tensors] == [("latent", 1, 40)] and not state


def test_a_layer_without_feed_forward_has_no_second_norms():
    raw = TIGESUN["a"][0]
    names = set(plain.tensor_shapes(raw))
    assert "l0.norm2b" in names and "l1.norm1b" in names and "l1.norm2" not in names and "l1.norm2b" not in names
    assert not any(n.startswith("l3.") for n in names)


@pytest.mark.parametrize("dims,base,scaling", [(16, 100.0, (4.0, 64, 8.0, 1.0)), (12, 1000.0, (16.0, 32, 64.0, 32.0)),
                                               (64, 500000.0, (2.0, 4096, 1.0, 0.01)), (8, 30.0, (32.0, 16, 2.0, 0.5)),
                                               (64, 10000.0, (8.0, 128, 16.0, 2.0)), (6, 7.0, (1.0, 10, 3.0, 1.0))])  # fmt: skip
def test_stretched_frequencies(dims, base, scaling):
    """The encoding's frequency table against the plain implementation's angles at position 1, also
    where the ramp's ends fall outside the head's frequencies or on one another."""
    from atomserve_b200.parts import PartSpec, build_part

    factor, original, fast, slow = scaling
    part = build_part("position", PartSpec("scaled_rotary", dict(head_dim=dims + 8, theta=base, rotary_dim=dims, factor=factor,
                                                                 original=original, fast=fast, slow=slow)), 32)  # fmt: skip
    part.prepare(torch.device("cpu"))
    rot = dict(base=base, dims=dims, scaling=dict(factor=factor, original=original, fast=fast, slow=slow))
    cos, sin = plain.scaled_rotary_tables(torch.tensor([1]), rot)
    mag = 0.1 * math.log(factor) + 1.0
    assert part.magnitude == pytest.approx(mag)
    angle = torch.atan2(sin[0] / mag, cos[0] / mag)
    assert torch.allclose(part.inv_freq.double(), angle, rtol=1e-6, atol=1e-9)
    fused = part.fused_rotary()
    assert fused.rotary_dim == dims and fused.pairing == "half" and fused.magnitude == pytest.approx(mag)


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "not one of"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 4), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 26), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "dense"),
    (lambda c: c["layers"][3].__setitem__("weights_of", 9), "weights_of"),
    (lambda c: c["layers"][4].__setitem__("weights_of", 4), "weights_of"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 6), "circle"),
    (lambda c: c["layers"][4].__setitem__("weights_of", 3), "sizes"),
    (lambda c: c["layers"][3].__setitem__("mixer", dict(c["layers"][3]["mixer"], heads=4)), "sizes"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("logit_softcap", -1.0), "logit_softcap"),
])  # fmt: skip
def test_rejections(change, text):
    from atomserve_b200.config.model_config import ModelConfigError

    raw = copy.deepcopy(TIGESUN["a"][0])
    change(raw)
    with pytest.raises(ModelConfigError, match=text):
        parse(raw)


def test_a_chain_of_layers_that_run_anothers_tensors():
    raw = copy.deepcopy(TIGESUN["a"][0])
    raw["layers"][6]["weights_of"] = 3  # 6 -> 3 -> 2
    arch, config = parse(raw)
    assert [config.source_of(i) for i in range(7)] == [0, 1, 2, 2, 0, 1, 2]
    assert [call.layer for call in arch.build_spec(config).schedule] == [0, 1, 2, 2, 0, 1, 2]
