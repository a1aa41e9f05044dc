"""Vegilix on the CPU: the configuration, the model's structure, and the engine's host side (cache slots of a repeated
span, state rows, kept first pages, batching, scheduler) over the torch stand-ins of the kernels."""
import copy

import pytest
import torch

import helpers
import vegilix_cases as cases


@pytest.fixture(scope="module")
def vegilix_folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = cases.make_folder(name, str(tmp_path_factory.mktemp(f"vegilix_{name}")))
        return made[name]
    return get


def test_configuration_reads_every_size_and_round_trips():
    from vt_transformer_b200.config import ConfigError, VegilixConfig, config_from_dict
    cfg = config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    assert isinstance(cfg, VegilixConfig) and cfg.vocab == 300 and cfg.width == 64 and len(cfg.layers) == 4
    att = cfg.layers[1].mixer
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.rot.dims, att.window, att.keep_first) == (4, 2, 24, 40, 12, 21, 3)
    assert att.rot.scaling.factor == 4.0 and att.rot.scaling.original == 64 and att.diff == 0.25 and att.scale == 0.21
    assert cfg.layers[0].mixer.decay == (0.9, 0.97, 1.0) and cfg.layers[2].mlp is None
    assert (cfg.layers[0].mlp.experts, cfg.layers[0].mlp.top, cfg.layers[0].mlp.ff, cfg.layers[0].mlp.shared_ff) == (5, 2, 20, 36)
    assert cfg.layers[1].mlp.shared_ff is None and cfg.residual_mult == 0.6
    assert cfg.run_order() == (0, 1, 2, 1, 2, 3)
    assert config_from_dict(cfg.to_dict()) == cfg
    for spoil, match in ((lambda c: c["layers"][0].__setitem__("type", "other"), "layers\\[0\\].*'other'"),
                         (lambda c: c["layers"][1]["mixer"].pop("diff"), "layers\\[1\\].mixer.*'diff'"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 26), "rot.dims"),
                         (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5]), "decay"),
                         (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6), "top"),
                         (lambda c: c["loop"].__setitem__("stop", 9), "loop")):
        bad = copy.deepcopy(cases.CONFIGS["mix"])
        spoil(bad)
        with pytest.raises(ConfigError, match=match):
            config_from_dict(bad)


def test_every_pass_of_a_repeated_layer_has_a_cache_of_its_own():
    from vt_transformer_b200.config import config_from_dict, get_architecture
    from vt_transformer_b200.models.base import DecoderModel
    from vt_transformer_b200.parts import KVCacheSpec, Runtime, StateSpec
    cfg = config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    model = DecoderModel(get_architecture(cfg.architecture).model_spec(cfg), Runtime(torch.device("cpu"), torch.float32, None))
    assert [r.block for r in model.spec.order] == [0, 1, 2, 1, 2, 3] and [r.cache for r in model.spec.order] == [0, 1, 2, 3, 4, 5]
    slots = model.cache_slots()
    assert [type(slots[i]) for i in sorted(slots)] == [StateSpec, KVCacheSpec, KVCacheSpec, KVCacheSpec, KVCacheSpec, StateSpec]
    assert slots[1] == slots[3] == KVCacheSpec(2, 24, 21, v_dim=40, k_maps=2, keep_first=3) and slots[0].shape == (3, 24, 40)
    names = set(model.param_specs())
    assert {"embed", "head", "final.norm", "l0.norm1b", "l0.norm2b", "l1.mix.q.norm", "l1.mix.lk2", "l0.mix.g", "l0.mlp.router",
            "l0.mlp.e4.down", "l0.mlp.shared.up", "l3.mlp.e2.gate"} <= names
    assert "l2.norm2" not in names and "l2.norm2b" not in names and "l1.mlp.shared.up" not in names and "l0.mlp.e5.up" not in names
    assert model.graph_safe()


def test_scaled_frequencies_keep_slow_and_blend_between():
    import math
    from plain import vegilix_plain as plain
    from vt_transformer_b200.parts.rope import rotation_frequencies
    rot = {"dims": 24, "base": 3000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}}
    got = rotation_frequencies(24, 3000.0, (4.0, 1.0, 3.0, 64)).double()
    want = torch.tensor(plain.frequencies(rot), dtype=torch.float64)
    assert float((got / want - 1).abs().max()) < 1e-6
    plainf = torch.tensor([3000.0 ** (-2.0 * i / 24) for i in range(12)], dtype=torch.float64)
    ratio = want / plainf
    wavelengths = 2 * math.pi / plainf
    assert bool((ratio[wavelengths < 64 / 3] == 1).all()) and bool(((ratio[wavelengths > 64] - 0.25).abs() < 1e-12).all())
    between = (wavelengths >= 64 / 3) & (wavelengths <= 64)
    assert int(between.sum()) >= 1 and bool(((ratio[between] > 0.25) & (ratio[between] < 1)).all())      # every branch is hit


def test_a_window_gives_pages_back_except_those_of_the_kept_first_tokens():
    from vt_transformer_b200.cache.manager import CacheManager
    from vt_transformer_b200.parts import KVCacheSpec
    cache = CacheManager({0: KVCacheSpec(1, 8, window=20, v_dim=8, k_maps=2, keep_first=17), 1: KVCacheSpec(1, 8, window=20)},
                         page_size=16, num_pages=12, max_requests=2, max_seq_len=192, dtype=torch.float32, device="cpu", allocate=False)
    kept, plainw = (0, 1) if cache.groups[0].layout.keep_first else (1, 0)
    row = cache.admit()
    for n in (10, 40, 100, 101, 150):
        cache.extend([(row, n)])
        cache.commit(row, n)
        cache.check()
    first_needed = (150 - 20 + 1) // 16
    held = lambda g: [i for i, p in enumerate(cache.groups[g].table[row]) if p >= 0]
    assert held(plainw) == list(range(first_needed, 10))
    assert held(kept) == [0, 1] + list(range(first_needed, 10))          # 17 kept tokens lie in pages 0 and 1
    cache.release(row)
    assert cache.free_pages() == [12, 12]


@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(fake_backend, vegilix_folders, family):
    cases.replay(vegilix_folders("mix"), cases.prompts_for("mix"), family, "cpu", "float32")


def test_tokens_grouped_by_expert_equal_the_plain_implementation(fake_backend, vegilix_folders, monkeypatch):
    from vt_transformer_b200 import ops
    monkeypatch.setattr(ops, "EXPERTS_GROUPED_MIN_PICKS", 1)
    for name in ("mix", "experts_alone"):
        cases.replay(vegilix_folders(name), cases.prompts_for(name), "portions", "cpu", "float32")
        cases.replay(vegilix_folders(name), cases.prompts_for(name), "mixed", "cpu", "float32")


def test_long_retention_walks_cut_into_segments(fake_backend, vegilix_folders, monkeypatch):
    """Sequences of 16 tokens and more in a step have their walk cut into up to 3 segments (states carried between them,
    the later segments' outputs completed): whole prompts, portions and mixed batches still equal the plain walk."""
    from vt_transformer_b200 import ops
    monkeypatch.setattr(ops, "RETENTION_SEGMENT_MIN", 8)
    monkeypatch.setattr(ops, "RETENTION_SEGMENTS", 3)
    for name in ("retention_alone", "mix"):
        for family in ("whole", "portions", "mixed"):
            cases.replay(vegilix_folders(name), cases.prompts_for(name), family, "cpu", "float32", sizes=(40, 3, 17, 2, 64))


def test_a_span_repeated_from_the_first_layer(fake_backend, vegilix_folders):
    cases.replay(vegilix_folders("looped_start"), cases.prompts_for("looped_start"), "mixed", "cpu", "float32")


def test_greedy_generation_through_the_entry_point(fake_backend, vegilix_folders):
    cases.greedy_generation(vegilix_folders("mix"), "mix", "cpu", "float32", n_new=6)


def test_a_tensor_of_the_wrong_shape_is_refused(fake_backend, vegilix_folders, tmp_path):
    from vt_transformer_b200.weights import WeightError

    def spoil(t):
        t["l1.mix.k"] = t["l1.mix.k"][:-1]
    with pytest.raises(WeightError):
        cases.runner_for(cases.rewritten(vegilix_folders("mix"), str(tmp_path / "bad"), spoil), "cpu", "float32", num_pages=4)


def test_random_weights_mode_of_the_command_line_writes_a_folder_that_loads(tmp_path):
    import json
    import os
    import subprocess
    import sys
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(cases.CONFIGS["mix"]))
    out = tmp_path / "model"
    res = subprocess.run([sys.executable, "-m", "vt_transformer_b200", "random-weights", "--config", str(cfg), "--out", str(out),
                          "--seed", "5", "--sigma", "0.05"], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, PYTHONPATH=helpers.ROOT), cwd=helpers.ROOT)
    assert res.returncode == 0, res.stderr
    from vt_transformer_b200.config import config_from_dict, load_config
    from vt_transformer_b200.weights import SafetensorsSource, check_against
    from vt_transformer_b200.weights.random_init import parameter_table
    config = load_config(str(out))
    assert config == config_from_dict(copy.deepcopy(cases.CONFIGS["mix"]))
    check_against(SafetensorsSource(str(out)), parameter_table(config))
