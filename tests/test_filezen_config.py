"""Filezen without a GPU: its configuration, run order, tensor names, cache plan, and the plain oracle."""

import json

import pytest
import torch

import filezen_cases as C
import plain_filezen as P


def test_config_round_trip_and_registry(tmp_path):
    from turboserve_b200.config import FilezenConfig, config_from_dict, config_from_dir, registered_architectures

    assert "Filezen" in registered_architectures()
    for name, (raw, _) in C.CASES.items():
        config = config_from_dict(raw)
        assert isinstance(config, FilezenConfig) and config.architecture == "Filezen"
        assert config_from_dict(config.to_dict()) == config
        assert config.vocab_size == raw["vocab"] and config.hidden_size == raw["width"]
        assert config.embedding_scale == raw["embedding"]["scale"] and config.residual_mult == raw["residual_mult"]
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(raw))
        assert config_from_dir(tmp_path / name) == config


def test_bad_configurations_are_refused():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.filezen import FilezenConfigError

    def broken(change):
        raw = json.loads(json.dumps(C.CASE_A))
        change(raw)
        with pytest.raises(FilezenConfigError):
            config_from_dict(raw)

    broken(lambda raw: raw["layers"][0].update(type="convolution"))
    broken(lambda raw: raw["layers"][1].update(mlp={"kind": "sparse", "ff": 8}))
    broken(lambda raw: raw["layers"][0]["mixer"].pop("kv_rank"))
    broken(lambda raw: raw["layers"][1]["mixer"].update(decay=[0.5]))            # one decay for three heads
    broken(lambda raw: raw["layers"][2]["mixer"].update(kv_from=3))              # a later layer
    broken(lambda raw: raw["layers"][2]["mixer"].update(kv_from=1))              # not a latent attention layer
    broken(lambda raw: raw["layers"][2]["mixer"].update(kv_rank=48))             # another latent size than its source
    broken(lambda raw: raw["layers"][0]["mlp"]["router"].pop("top"))
    broken(lambda raw: raw.pop("norm"))


def test_run_order_shares_the_rows_of_the_named_layer():
    from turboserve_b200.config import config_from_dict

    spec = config_from_dict(C.CASE_A).to_model_spec()
    assert [(run.layer, run.cache_from) for run in spec.order] == [(0, None), (1, None), (2, 0), (3, None)]
    assert all(layer.block == "output_norm" and layer.block_params["residual_mult"] == 0.5 for layer in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    assert spec.tie_word_embeddings and spec.embedding["scale"] == 3.0
    # rows are kept for the largest window of the layers that read them
    assert spec.layers[0].mixer["window"] == 24 and spec.layers[2].mixer["window"] == 40
    assert spec.layers[0].mixer["cache_window"] == spec.layers[2].mixer["cache_window"] == 40
    b = config_from_dict(C.CASE_B).to_model_spec()
    assert b.layers[1].mixer["cache_window"] is None and b.layers[2].mixer["cache_window"] is None and b.layers[2].mixer["window"] == 17
    c = config_from_dict(C.CASE_C).to_model_spec()
    assert c.layers[0].mixer["cache_window"] == 64 and c.layers[4].mixer["window"] == 20


def test_tensor_names_shapes_and_cache_plan():
    from turboserve_b200.config import config_from_dict
    from turboserve_b200.config.registry import lookup

    config = config_from_dict(C.CASE_A)
    model = lookup("Filezen").build_model(config, torch.float32, "cpu")
    shapes = {p.name: tuple(p.spec.shape) for p in model.named_params()}
    assert shapes["embed"] == (190, 96) and shapes["final.norm"] == (96,)
    assert shapes["l0.mix.q"] == (4 * 32, 96) and shapes["l0.mix.dkv"] == (48, 96) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (4 * 24, 40) and shapes["l0.mix.uv"] == (4 * 20, 40) and shapes["l0.mix.o"] == (96, 80)
    assert "l2.mix.dkv" not in shapes and "l2.mix.dkv.norm" not in shapes and shapes["l2.mix.uk"] == (32, 40)
    assert shapes["l1.mix.q"] == shapes["l1.mix.k"] == (48, 96) and shapes["l1.mix.v"] == shapes["l1.mix.g"] == (72, 96)
    assert shapes["l1.mlp.gate"] == (112, 96) and shapes["l1.mlp.down"] == (96, 112)
    assert shapes["l0.mlp.router"] == (8, 96) and shapes["l0.mlp.e7.up"] == (48, 96) and shapes["l0.mlp.e0.down"] == (96, 48)
    assert shapes["l0.mlp.shared.gate"] == (32, 96) and "l3.mlp.shared.gate" not in shapes and "l3.mlp.e5.gate" in shapes
    assert "l2.norm2" not in shapes and "l2.norm2" in model.optional_names() and "l2.norm1" in shapes
    plan = model.cache_plan()
    assert [(run.kind, run.owner) for run in plan.runs] == [("paged", 0), ("state", 1), ("paged", 0), ("state", 3)]
    assert plan.windows == [40]
    assert plan.runs[0].need.head_dim == 48 and plan.runs[0].need.v_dim == 0 and plan.runs[0].need.num_kv_heads == 1
    assert plan.runs[1].states[0].shape == (3, 24, 16) and plan.runs[1].states[0].dtype == torch.float32
    assert model.graph_safe


def test_frequencies_with_and_without_scaling_agree_with_the_plain_ones():
    from turboserve_b200.parts.rope import scaled_rotary_frequencies

    for spec in (C.rot(10000.0, 16), C.rot(5000.0, 8, (4.0, 64, 16.0, 2.0)), C.rot(20000.0, 8, (16.0, 40, 4.0, 0.5)),
                 C.rot(10000.0, 32, (6.0, 128, 24.0, 1.5))):
        freq, amplitude = scaled_rotary_frequencies(spec["dims"], spec["base"], spec.get("scaling"))
        want, factor = P.rotary_constants(spec)
        assert torch.allclose(freq.double(), want, rtol=1e-7, atol=0) and abs(amplitude - factor) < 1e-12
    scaled, _ = scaled_rotary_frequencies(32, 10000.0, dict(factor=6.0, original=128, fast=24.0, slow=1.5))
    plain, _ = scaled_rotary_frequencies(32, 10000.0)
    assert scaled[0] == plain[0] and torch.isclose(scaled[-1], plain[-1] / 6.0)  # fast pairs kept, slow pairs stretched


def test_the_oracle_is_causal_keeps_its_windows_and_routes_inside_the_kept_groups(tmp_path):
    folder = C.write_case("A", tmp_path / "a")
    config, weights = P.read_model_folder(folder)
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, config["vocab"], (50,), generator=g).tolist()
    logits, layers = P.forward(config, weights, tokens)
    shorter, _ = P.forward(config, weights, tokens[:31])
    assert torch.allclose(logits[:31], shorter, atol=1e-9)
    assert layers.shape == (4, 50, 96)
    h = torch.randn(40, 96, generator=g, dtype=torch.float64)
    router = torch.randn(8, 96, generator=g, dtype=torch.float64)
    chosen, weights_ = P.route(h, router, {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 1}})
    assert ((chosen[:, 0] // 2) == (chosen[:, 1] // 2)).all()  # one group kept: both experts are neighbours
    assert torch.allclose(weights_.sum(-1), torch.ones(40, dtype=torch.float64))
    q = torch.zeros(6, 6, dtype=torch.float64)
    seen = P.window_softmax(q, 3)
    assert torch.allclose(seen[5], torch.tensor([0, 0, 0, 1 / 3, 1 / 3, 1 / 3], dtype=torch.float64))
    assert torch.allclose(seen[1], torch.tensor([0.5, 0.5, 0, 0, 0, 0], dtype=torch.float64))
