"""The Munevik configuration, its model as data, and what its layers ask of the cache manager (no GPU)."""
import copy

import pytest
import torch

from munevik_configs import MUN_A, MUN_B, MUN_C, attention_layer, dense_mlp

from tiny_transformer_inference_engine_b200 import ModelConfig
from tiny_transformer_inference_engine_b200.cache import CacheManager
from tiny_transformer_inference_engine_b200.config import ConfigError, MunevikConfig
from tiny_transformer_inference_engine_b200.models.model import Model
from tiny_transformer_inference_engine_b200.parts.base import PagedKVNeed, FixedStateNeed
from tiny_transformer_inference_engine_b200.registry import model_spec
from tiny_transformer_inference_engine_b200.weights import random_tensors, write_random_model, read_safetensors


def test_architecture_picks_the_config_class_and_round_trips(tmp_path):
    cfg = ModelConfig.from_dict(MUN_B)
    assert isinstance(cfg, MunevikConfig)
    assert (cfg.vocab_size, cfg.d_model, cfg.postln_alpha, cfg.norm_eps) == (131, 48, 1.0, 1e-5)
    write_random_model(cfg, 3, str(tmp_path))
    again = ModelConfig.from_json(str(tmp_path))
    assert again == cfg and again.to_dict() == cfg.to_dict()
    stored = read_safetensors(str(tmp_path))
    assert set(stored) == set(Model(model_spec(cfg)).param_specs())


def test_tensor_names_and_shapes():
    specs = {k: tuple(v[2].shape) for k, v in Model(model_spec(ModelConfig.from_dict(MUN_B))).param_specs().items()}
    assert specs["embed"] == (131, 48) and specs["final.norm"] == (48,) and specs["final.norm.b"] == (48,)
    assert specs["l0.mix.conv"] == (72, 2) and specs["l0.mix.ra"] == (3, 24, 24) and specs["l0.mix.ri.b"] == (3, 24)
    assert "l0.norm2" not in specs and "l0.mlp.gate" not in specs               # a layer without a feed-forward
    assert specs["l1.mix.dkv"] == (24, 48) and specs["l1.mix.dkv.norm"] == (20,) and specs["l1.mix.q"] == (48, 48)
    assert specs["l1.mix.uk"] == (36, 20) and specs["l1.mix.uv"] == (24, 20) and specs["l1.mix.g"] == (3, 48)
    assert "l2.mix.dkv" not in specs and specs["l2.mix.uk"] == (20, 20)           # reads layer 1's cache
    assert specs["l1.mlp.router"] == (6, 48) and specs["l1.mlp.e5.down"] == (48, 24) and "l1.mlp.shared.gate" not in specs
    assert specs["l3.mlp.gate"] == (56, 48) and specs["l3.mix.lam"] == (48,)
    assert "head" not in " ".join(specs)                                          # the logits come from the embedding table


def test_cache_needs_and_the_widest_window_of_a_shared_cache():
    model = Model(model_spec(ModelConfig.from_dict(MUN_B)))
    needs = model.cache_needs()
    assert needs[0] == [FixedStateNeed((2, 72), "float32")] and needs[3] == [FixedStateNeed((1, 48), "float32")]
    assert needs[1] == [PagedKVNeed(1, 32, 19, None, planes=1)] and needs[2] == []      # layer 2 (window 19) reads layer 1's (window 5)
    assert model.run_order[2].cache_from == 1
    mgr = CacheManager(needs, model.run_order, 8, 6, 2, "float32", "cpu")
    assert mgr.groups[0].kv.shape == (1, 1, 6, 1, 8, 32)                                  # one plane: keys and values are one array
    views = mgr.views({0: torch.zeros(1, 4, dtype=torch.int32)})
    assert views[1][0].k_pages.data_ptr() == views[1][0].v_pages.data_ptr()
    assert views[2][0].k_pages.data_ptr() == views[1][0].k_pages.data_ptr() and not views[2][0].writable
    # pages leave only when the widest window has passed them
    mgr.admit("r")
    mgr.extend("r", 0, 40)
    mgr.extend("r", 40, 41)
    assert [p != 0 for p in mgr.table(0, "r")] == [False, False, True, True, True, True]   # key 22 is the oldest that token 40 sees
    mgr.release("r")
    mgr.check()


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "earlier"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "no latent cache"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=24), "must equal"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=2), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(blocks=5), "multiple"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][1].update(type="conv"), "unknown"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c["layers"][3]["mlp"].pop("limit"), "limit"),
])
def test_bad_configs_are_refused(edit, text):
    cfg = copy.deepcopy(MUN_B)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        ModelConfig.from_dict(cfg)


def test_random_weights_are_reproducible():
    cfg = ModelConfig.from_dict(MUN_A)
    a, b = random_tensors(cfg, 5), random_tensors(cfg, 5)
    assert all(torch.equal(a[k], b[k]) for k in a)
