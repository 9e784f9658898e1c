"""The Mizupel design without a GPU: configuration and its refusals, the spec (tensor names, run order of layers that run
another layer's tensors, cache and state needs), rescaled rotation frequencies, a size that only the weight file knows."""
import copy
import math

import pytest
import torch

import plain_mizupel as pm
from mizupel_configs import MIZ_A, MIZ_B, MIZ_D, ALL

from tiny_transformer_inference_engine_b200 import ModelConfig
from tiny_transformer_inference_engine_b200.config import ConfigError, MizupelConfig
from tiny_transformer_inference_engine_b200.models.model import Model
from tiny_transformer_inference_engine_b200.parts.base import PagedKVNeed, FixedStateNeed, PartSpec
from tiny_transformer_inference_engine_b200.registry import model_spec, build_part
from tiny_transformer_inference_engine_b200.weights import random_tensors
from tiny_transformer_inference_engine_b200.weights.loader import place, WeightError


def test_config_is_picked_by_architecture_and_round_trips(tmp_path):
    cfg = ModelConfig.from_dict(MIZ_A)
    assert isinstance(cfg, MizupelConfig) and cfg.vocab_size == 131 and cfg.d_model == 64 and cfg.logit_softcap == 10.0
    cfg.save(str(tmp_path))
    again = ModelConfig.from_json(str(tmp_path))
    assert again == cfg and ModelConfig.from_dict(MIZ_B).logit_softcap is None


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][3].update(weights_of=3), "another layer"),
    (lambda c: c["layers"][4].update(weights_of=3), "owns no tensors"),
    (lambda c: c["layers"][3].update(weights_of=2), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "unknown"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refusals(change, message):
    raw = copy.deepcopy(MIZ_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        ModelConfig.from_dict(raw)


def test_tensor_names_run_order_and_needs():
    model = Model(model_spec(ModelConfig.from_dict(MIZ_A)))
    names = set(model.param_specs())
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.conv", "l0.mix.g", "l0.mix.o",
            "l0.mlp.up", "l0.mlp.down", "l1.mix.i.b", "l1.mix.f", "l1.mix.norm", "l2.mix.mu.w", "l2.mix.w1", "l2.mix.w0", "l2.mix.u"} <= names
    assert not any(n.startswith(("l3.", "l4.")) for n in names)       # entries with weights_of own nothing
    assert "l1.norm2" not in names                                   # no feed-forward, no second norm
    assert [e.layer for e in model.run_order] == [0, 1, 2, 0, 2] and all(e.cache_from is None for e in model.run_order)
    needs = model.cache_needs()
    a = MIZ_A["layers"][0]["mixer"]
    channels = (a["heads"] + a["kv_heads"]) * a["dim"] + a["kv_heads"] * a["vdim"]
    assert needs[0] == needs[3] == [PagedKVNeed(2, 32, 11, None), FixedStateNeed((2, channels), "float32")]     # rows padded to 32 values
    assert needs[1] == [FixedStateNeed((2, 24, 16)), FixedStateNeed((2, 16)), FixedStateNeed((2,))]
    assert needs[2] == needs[4] == [FixedStateNeed((2, 32, 32)), FixedStateNeed((64,))]
    shapes = {n: s[2].shape for n, s in model.param_specs().items()}
    assert shapes["l0.mix.v"] == (48, 64) and shapes["l0.mix.o"] == (64, 96) and shapes["l0.mix.q.conv"] == (64, 3)
    assert shapes["l2.mix.w1"] == (8, 64) and shapes["l2.mix.w2"] == (64, 8) and shapes["l1.mix.g"] == (48, 64)


def test_one_tap_keeps_no_state_and_no_convolution_has_no_tensor():
    model = Model(model_spec(ModelConfig.from_dict(MIZ_B)))
    needs, names = model.cache_needs(), set(model.param_specs())
    assert needs[1] == [PagedKVNeed(3, 16, None, None)] and "l1.mix.q.conv" in names
    assert needs[3] == [PagedKVNeed(1, 16, 200, None)] and "l3.mix.q.conv" not in names
    assert needs[0][0] == FixedStateNeed((3, 12, 16)) and needs[2][0] == FixedStateNeed((1, 20, 64))   # key channels padded per slice


def test_rescaled_frequencies_cover_the_three_bands():
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    part = build_part("position", PartSpec("rope", "", {"dim": 8, "base": 100.0, "style": "half", "scaling": rot["scaling"]}))
    got = part.frequencies().double()
    plain = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    want = torch.tensor(pm.rotary_frequencies(rot), dtype=torch.float64)
    assert torch.allclose(got, want, rtol=1e-6)
    kinds = []
    for f, g in zip(plain, want.tolist()):
        kinds.append("kept" if math.isclose(f, g) else "divided" if math.isclose(f / 8.0, g) else "blended")
    assert set(kinds) == {"kept", "divided", "blended"}, kinds
    unscaled = build_part("position", PartSpec("rope", "", {"dim": 8, "base": 100.0, "style": "half"})).frequencies().double()
    assert torch.allclose(unscaled, torch.tensor(plain, dtype=torch.float64), rtol=1e-6)


def test_the_decay_rank_may_be_left_to_the_weight_file():
    raw = copy.deepcopy(MIZ_D)
    w = random_tensors(ModelConfig.from_dict(raw), 0)
    for L in raw["layers"]:
        L["mixer"].pop("decay_rank", None)
    cfg = ModelConfig.from_dict(raw)
    model = Model(model_spec(cfg))
    assert model.param_specs()["l0.mix.w1"][2].shape == (-1, 40)
    placed = place(w, model.param_specs(), torch.float32, "cpu")
    assert placed["l0.mix.w1"].shape == (3, 40)
    with pytest.raises(ValueError, match="leaves a size"):
        random_tensors(cfg, 0)
    w["l0.mix.w2"] = torch.zeros(48, 4)
    placed = place(w, model.param_specs(), torch.float32, "cpu")
    with pytest.raises(ValueError, match="disagree"):
        model.blocks[0].mixer.load({k[len("l0.mix."):]: v for k, v in placed.items() if k.startswith("l0.mix.")})
    w["l0.mix.r"] = torch.zeros(47, 40)
    with pytest.raises(WeightError, match="wrong shape"):
        place(w, model.param_specs(), torch.float32, "cpu")


def test_plain_model_prefix_property():
    """The plain model is causal: logits of a prefix equal the prefix of the logits (every mixer, both feed-forward cases)."""
    for cfg in ALL.values():
        if cfg["width"] > 64:
            continue
        w = random_tensors(ModelConfig.from_dict(cfg), 1, std=0.1, perturb_norms=True)
        toks = torch.randint(0, cfg["vocab"], (14,), generator=torch.Generator().manual_seed(2)).tolist()
        full, part = pm.forward(cfg, w, toks), pm.forward(cfg, w, toks[:9])
        assert torch.allclose(full[:9], part, rtol=1e-9, atol=1e-9)
