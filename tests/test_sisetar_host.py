"""Sisetar on the CPU: the configuration, the model's structure, and the engine's host side (cache slots, state rows,
batching, scheduler) over the torch stand-ins of the kernels."""
import copy
import json
import os

import pytest
import torch

import helpers
import sisetar_cases as cases


@pytest.fixture(scope="module")
def sisetar_folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = cases.make_folder(name, str(tmp_path_factory.mktemp(f"sisetar_{name}")))
        return made[name]
    return get


def test_configuration_reads_every_size_and_round_trips():
    from vt_transformer_b200.config import ConfigError, SisetarConfig, config_from_dict
    cfg = config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    assert isinstance(cfg, SisetarConfig) and cfg.vocab == 300 and cfg.width == 64 and len(cfg.layers) == 4
    left = cfg.layers[3].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.rot_dims, left.chunk) == (4, 1, 40, 16, 8, 33)
    assert cfg.layers[1].ff == 72 and cfg.layers[2].ff is None and cfg.layers[3].ff == 50 and cfg.layers[1].mixer.tau == 4.0
    assert config_from_dict(cfg.to_dict()) == cfg
    bad = copy.deepcopy(cases.CONFIGS["mix"])
    bad["layers"][0]["type"] = "other"
    with pytest.raises(ConfigError, match="layers\\[0\\].*'other'"):
        config_from_dict(bad)
    bad = copy.deepcopy(cases.CONFIGS["mix"])
    del bad["layers"][1]["mixer"]["tau"]
    with pytest.raises(ConfigError, match="layers\\[1\\].mixer.*'tau'"):
        config_from_dict(bad)
    bad = copy.deepcopy(cases.CONFIGS["mix"])
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 33
    with pytest.raises(ConfigError, match="rot.dims"):
        config_from_dict(bad)


def test_the_model_declares_pages_and_states_for_what_its_layers_keep():
    from vt_transformer_b200.config import config_from_dict, get_architecture
    from vt_transformer_b200.models.base import DecoderModel
    from vt_transformer_b200.parts import KVCacheSpec, Runtime, StateSpec
    cfg = config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    model = DecoderModel(get_architecture(cfg.architecture).model_spec(cfg), Runtime(torch.device("cpu"), torch.float32, None))
    slots = model.cache_slots()
    assert [type(slots[i]) for i in sorted(slots)] == [KVCacheSpec, StateSpec, StateSpec, StateSpec, KVCacheSpec, StateSpec]
    assert slots[0] == KVCacheSpec(4, 32, None, v_dim=48) and slots[1].shape == (2, 40, 40) and slots[2].shape == (3, 24, 40)
    names = set(model.param_specs())
    assert {"embed", "final.norm", "l0.norm2", "l0.mix.left.q", "l0.mix.right.w0", "l1.mix.a2.b", "l1.mlp.act"} <= names
    assert "l2.norm2" not in names and "l2.mlp.up" not in names and "l2.mlp.act" not in names
    assert model.graph_safe()


@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(fake_backend, sisetar_folders, family):
    cases.replay(sisetar_folders("mix"), cases.prompts_for("mix"), family, "cpu", "float32")


def test_a_model_without_attention_has_no_pages_and_still_steps(fake_backend, sisetar_folders):
    folder = sisetar_folders("gla_only")
    assert cases.runner_for(folder, "cpu", "float32", num_pages=1).cache.groups == []
    cases.replay(folder, cases.prompts_for("gla_only"), "mixed", "cpu", "float32")


def test_greedy_generation_through_the_entry_point(fake_backend, sisetar_folders):
    cases.greedy_generation(sisetar_folders("mix"), "mix", "cpu", "float32", n_new=6)


def test_the_rank_of_the_low_rank_gates_comes_from_the_weights(fake_backend, sisetar_folders, tmp_path):
    def change(t):
        g = torch.Generator().manual_seed(1)
        for n in list(t):
            if n.endswith(".a1") or n.endswith(".w1"):
                t[n] = (torch.randn((5, t[n].shape[1]), generator=g) * 0.2).to(torch.bfloat16)
            if n.endswith(".a2") or n.endswith(".w2"):
                t[n] = (torch.randn((t[n].shape[0], 5), generator=g) * 0.3).to(torch.bfloat16)
    folder = cases.rewritten(sisetar_folders("mix"), str(tmp_path / "rank5"), change)
    cases.replay(folder, cases.prompts_for("mix")[:3], "portions", "cpu", "float32")
    from vt_transformer_b200.weights import WeightError

    def spoil(t):
        t["l1.mix.a2"] = t["l1.mix.a2"][:-1]
    with pytest.raises(WeightError):
        cases.runner_for(cases.rewritten(folder, str(tmp_path / "bad"), spoil), "cpu", "float32", num_pages=4)
