"""Baporax without a GPU: its configuration, run order, tensor names, cache plan, and the plain oracle."""

import json

import pytest
import torch

import baporax_cases as C
import plain_baporax as P


def test_config_round_trip_and_registry(tmp_path):
    from turboserve_b200.config import BaporaxConfig, config_from_dict, config_from_dir, registered_architectures

    assert "Baporax" in registered_architectures()
    for name, (raw, _) in C.CASES.items():
        config = config_from_dict(raw)
        assert isinstance(config, BaporaxConfig) and config.architecture == "Baporax"
        assert config_from_dict(config.to_dict()) == config
        assert config.vocab_size == raw["vocab"] and config.hidden_size == raw["width"]
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(raw))
        assert config_from_dir(tmp_path / name) == config


def test_bad_configurations_are_refused():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.baporax import BaporaxConfigError

    raw = json.loads(json.dumps(C.CASE_Y))
    raw["layers"][0]["type"] = "convolution"
    with pytest.raises(BaporaxConfigError):
        config_from_dict(raw)
    raw = json.loads(json.dumps(C.CASE_Y))
    raw["layers"][1]["mlp"] = {"kind": "experts", "ff": 8}
    with pytest.raises(BaporaxConfigError):
        config_from_dict(raw)
    raw = json.loads(json.dumps(C.CASE_X))
    raw["loop"]["stop"] = 9
    with pytest.raises(BaporaxConfigError):
        config_from_dict(raw)
    raw = json.loads(json.dumps(C.CASE_Y))
    del raw["layers"][0]["mixer"]["diff"]
    with pytest.raises(BaporaxConfigError):
        config_from_dict(raw)


def test_run_order_repeats_the_looped_stretch_and_names_a_shift_per_pass():
    from turboserve_b200.config import config_from_dict

    spec = config_from_dict(C.CASE_X).to_model_spec()
    assert [(run.layer, run.shift) for run in spec.order] == [
        (0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert [(i, s) for i, s in P.run_order(C.CASE_X)] == [(run.layer, run.shift) for run in spec.order]
    assert all(run.cache_from is None for run in spec.order)  # every pass keeps a cache of its own
    plain = config_from_dict(C.CASE_Y).to_model_spec()
    assert plain.stream_shifts is None and [run.layer for run in plain.order] == [0, 1]
    once = config_from_dict(C.CASE_Z).to_model_spec()
    assert [(run.layer, run.shift) for run in once.order] == [(0, 0), (1, None)]


def test_tensor_names_and_shapes():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.registry import lookup

    config = config_from_dict(C.CASE_X)
    model = lookup("Baporax").build_model(config, torch.float32, "cpu")
    shapes = {p.name: tuple(p.spec.shape) for p in model.named_params()}
    assert shapes["embed"] == (200, 96) and shapes["loop.step"] == (3, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.in"] == (2 * 96 + 2 * 16 + 4, 96) and shapes["l0.mix.conv"] == (96 + 32, 3)
    assert shapes["l0.mix.conv.b"] == (128,) and shapes["l0.mix.norm"] == (96,) and shapes["l0.mix.o"] == (96, 96)
    assert shapes["l0.mix.A_log"] == shapes["l0.mix.D"] == shapes["l0.mix.dt_bias"] == (4,)
    assert shapes["l1.mix.q"] == (6 * 2 * 16, 96) and shapes["l1.mix.k"] == (2 * 2 * 16, 96) and shapes["l1.mix.v"] == (80, 96)
    assert shapes["l1.mix.q.conv"] == (192, 2) and shapes["l1.mix.lk2"] == (16,) and shapes["l1.mix.o"] == (96, 240)
    assert shapes["l1.mlp.up"] == (160, 96) and shapes["l1.mlp.down"] == (96, 160) and shapes["l1.norm2"] == (96,)
    assert "l2.norm2" not in shapes and "l2.mlp.up" not in shapes  # the layer without a feed-forward
    assert not any(name.startswith("head.") for name in shapes)   # the head is the embedding table


def test_cache_plan_pages_states_and_bytes():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.registry import lookup
    from turboserve_b200.parts import PagedKVNeed, StateNeed

    model = lookup("Baporax").build_model(config_from_dict(C.CASE_X), torch.float32, "cpu")
    plan = model.cache_plan()
    assert plan.windows == [24, None]
    kinds = [run.kind for run in plan.runs]
    assert kinds == ["state", "paged", "paged", "paged", "paged", "paged", "paged", "state"]
    first = plan.runs[1]
    assert first.need == PagedKVNeed(2, 32, 24, value_dim=40) and first.states == (StateNeed((1, 192 + 64 + 80), None),)
    assert plan.runs[0].states == (StateNeed((4, 24, 16), torch.float32), StateNeed((2, 128), None))
    # a page id of the windowed group stands for the three runs of layer 1: keys of 2 x 32, values of 2 x 40
    assert plan.bytes_per_page(16, 2) == [3 * 16 * 2 * (32 + 40) * 2, 3 * 16 * 2 * (48 + 32) * 2]
    assert plan.state_bytes_per_slot() > 0
    no_taps = lookup("Baporax").build_model(config_from_dict(C.CASE_Y), torch.float32, "cpu").cache_plan()
    assert no_taps.runs[0].states == ()  # one tap: nothing to remember


def test_random_model_folder_and_checkpoint_check(tmp_path):
    from safetensors.torch import load_file, save_file

    from turboserve_b200.config import config_from_dir
    from turboserve_b200.config.registry import lookup
    from turboserve_b200.weights.loader import WeightLoadError, check_checkpoint, checkpoint_index

    folder = C.write_case("Y", tmp_path / "y")
    config = config_from_dir(folder)
    model = lookup(config.architecture).build_model(config, torch.float32, "cpu")
    check_checkpoint(model, checkpoint_index(folder))
    tensors = load_file(str(folder / "model.safetensors"))
    assert tensors["l0.norm1"].abs().max() < 0.5  # norm weights are stored around zero
    tensors["l1.norm2"] = torch.zeros(64)  # a second norm of the layer without a feed-forward is let through
    save_file(tensors, str(folder / "model.safetensors"))
    check_checkpoint(model, checkpoint_index(folder))
    del tensors["l1.mix.dt_bias"]
    tensors["l1.mix.extra"] = torch.zeros(3)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightLoadError) as error:
        check_checkpoint(model, checkpoint_index(folder))
    assert "l1.mix.dt_bias" in str(error.value) and "l1.mix.extra" in str(error.value)


def test_plain_oracle_is_causal_and_its_window_ends_where_it_should(tmp_path):
    """The oracle's own sanity: a prefix's logits do not depend on what follows, and with sharp scores
    a change of one token moves a later position's logits only while the token is within reach of
    something (the windowed model without recurrence forgets it)."""
    folder = C.write_case("Y", tmp_path / "y", sharp=True)
    config, weights = P.read_model_folder(folder)
    tokens = torch.randint(0, config["vocab"], (60,), generator=torch.Generator().manual_seed(0)).tolist()
    full = P.forward(config, weights, tokens)
    assert torch.allclose(P.forward(config, weights, tokens[:25]), full[:25], atol=1e-12)
    attention_only = dict(config, layers=config["layers"][:1])
    base = P.forward(attention_only, weights, tokens)
    other = list(tokens)
    other[10] = (tokens[10] + 1) % config["vocab"]
    moved = (P.forward(attention_only, weights, other) - base).abs().amax(-1)
    assert moved[10] > 0 and moved[26] > 0 and moved[27:].max() == 0  # a window of 17: positions 10 .. 26


def test_command_line_writes_a_model_folder_and_sizes_its_cache(tmp_path):
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    (tmp_path / "config.json").write_text(json.dumps(C.CASE_X))

    def cli(*args):
        return subprocess.run([sys.executable, "-m", "turboserve_b200.cli", *args], capture_output=True, text=True, cwd=root,
                              env={**os.environ, "PYTHONDONTWRITEBYTECODE": "1"})

    out = cli("engine", "random-weights", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "m"), "--seed", "3")
    assert out.returncode == 0, out.stderr
    config, weights = P.read_model_folder(tmp_path / "m")
    assert config["architecture"] == "Baporax" and weights["loop.step"].shape == (3, 96)
    assert torch.isfinite(P.forward(config, weights, [1, 2, 3, 4])).all()
    out = cli("engine", "kv-size", "-m", str(tmp_path / "m"), "--total-memory-gib", "8", "--max-num-seqs", "4")
    assert out.returncode == 0, out.stderr
    sizing = json.loads(out.stdout)
    # per page id: three runs of layer 1 (keys 2 x 32, values 2 x 40) and three of layer 2 (keys 2 x 48, values 2 x 32), 16 slots, 2 bytes
    assert sizing["num_groups"] == 2 and sizing["bytes_per_block"] == 3 * 16 * 2 * (72 + 80) * 2 and sizing["state_bytes"] > 0
