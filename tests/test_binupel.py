"""Binupel without a GPU: its configuration, what the model asks of the weights and of the cache, and the plain
implementation against itself (a prompt whole and token by token through the explicit states)."""

import copy

import pytest
import torch

import plain_binupel as plain
from binupel_models import BINUPEL_P, BINUPEL_Q, CONFIGS, make_folder, tensor_shapes


def model_of(config):
    from qwen3_from_scratch_b200.engine.model import Model
    from qwen3_from_scratch_b200.registry import build_model_spec, config_from_dict
    return Model(build_model_spec(config_from_dict(config)))


@pytest.mark.parametrize("key", list(CONFIGS))
def test_the_model_asks_for_the_tensors_the_design_names(key):
    config = CONFIGS[key][0]
    asked = {s.name: tuple(s.shape) for s in model_of(config).weight_specs()}
    assert asked == tensor_shapes(config)


def test_configuration_round_trip_and_registry_by_single_name():
    from qwen3_from_scratch_b200.registry import config_from_dict
    cfg = config_from_dict(BINUPEL_P)
    assert cfg.architecture == "Binupel" and len(cfg.layers) == 6 and cfg.layers[4].weights_of == 0
    assert config_from_dict(cfg.to_dict()) == cfg
    assert cfg.layers[0].sizes()["q_temp_every"] == 7 and "q_temp_every" not in config_from_dict(BINUPEL_Q).layers[1].sizes()


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0]["mixer"].update(vdim=32), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(blocks=5), "multiple"),
    (lambda c: c["layers"][0].update(type="hyena"), "not built"),
    (lambda c: c["layers"][0].update(mlp={"kind": "moe", "ff": 8}), "dense"),
    (lambda c: c["layers"][3].update(weights_of=9), "weights_of"),
    (lambda c: c["layers"][3].update(weights_of=3), "weights_of"),
    (lambda c: c["layers"][3].update(type="attention"), "of its type"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][2]["mixer"].pop("dt_rank"), "dt_rank"),
])
def test_configuration_errors_name_the_key(change, message):
    from qwen3_from_scratch_b200.config.model_config import ConfigError
    from qwen3_from_scratch_b200.registry import config_from_dict
    config = copy.deepcopy(BINUPEL_P)
    change(config)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_weights_of_may_lead_on_and_point_ahead():
    """An entry's tensors are those of the entry its `weights_of` leads to, through another sharing entry or to a
    later one; its own sizes are not read; `vdim` may be left out (the values are the keys)."""
    from qwen3_from_scratch_b200.registry import config_from_dict
    config = copy.deepcopy(BINUPEL_P)
    config["layers"][0] = {"type": "rglru", "weights_of": 3}          # ahead, and 3 leads on to 1
    del config["layers"][4]["mixer"]                                    # a sharing entry needs no sizes
    config["layers"][4]["weights_of"] = 5
    config["layers"][5] = {"type": "attention", "mlp": {"kind": "dense", "ff": 72},
                           "mixer": {"heads": 4, "kv_heads": 2, "dim": 48, "scale": 0.21}}
    cfg = config_from_dict(config)
    assert [l.weights_of for l in cfg.layers] == [1, None, None, 1, 5, None]
    assert cfg.layers[0].sizes() == cfg.layers[1].sizes() and cfg.layers[4].sizes()["vdim"] == 48
    model = model_of(config)
    assert [(c.layer, c.cache) for c in model.spec.order] == [(0, 0), (0, 1), (1, 2), (0, 3), (2, 4), (2, 5)]
    assert config_from_dict(cfg.to_dict()) == cfg


def test_run_order_and_cache_needs():
    """Shared weights: one layer, two entries of the run order, each with pages or state of its own; every entry
    keeps the last input of its shift; the recurrences keep a state and the tail of their convolution."""
    model = model_of(BINUPEL_P)
    assert len(model.layers) == 3
    assert [(c.layer, c.cache) for c in model.spec.order] == [(0, 0), (1, 1), (2, 2), (1, 3), (0, 4), (2, 5)]
    layout = model.cache_layout()
    assert [g.cache_ids for g in layout.groups] == [[0, 4]]
    assert [p.name for p in layout.groups[0].spec.planes] == ["k", "v"]
    states = {k: v.shape for k, v in layout.states.items()}
    assert states[(1, "state")] == (96,) and states[(3, "conv")] == (3, 96) and states[(3, "state")] == (96,)
    assert states[(2, "state")] == (8, 80) and states[(5, "conv")] == (1, 80)
    assert all(states[(i, "shift")] == (64,) for i in range(6))
    assert all(v.dtype == "float32" for v in layout.states.values())


def test_cache_manager_files_named_needs():
    from qwen3_from_scratch_b200.cache import cache_key, layout_of
    from qwen3_from_scratch_b200.parts.base import KVCacheSpec, StateSpec
    layout = layout_of({0: {"": KVCacheSpec(2, 16), "shift": StateSpec((8,))}, 1: StateSpec((4,)),
                        2: {"state": StateSpec((3, 5)), "conv": StateSpec((2, 5))}})
    assert [g.cache_ids for g in layout.groups] == [[0]]
    assert set(layout.states) == {(0, "shift"), 1, (2, "state"), (2, "conv")}
    assert cache_key(3) == 3 and cache_key(3, "conv") == (3, "conv")


def test_random_model_folder_through_the_framework_writer(tmp_path):
    from qwen3_from_scratch_b200.registry import config_from_dict, load_config
    from qwen3_from_scratch_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), config_from_dict(BINUPEL_Q), seed=1)
    assert load_config(folder) == config_from_dict(BINUPEL_Q)
    _, w = plain.read_model_folder(folder)
    assert {k: tuple(v.shape) for k, v in w.items()} == tensor_shapes(BINUPEL_Q)


@pytest.mark.parametrize("key", ["p", "q"])
def test_plain_whole_prompt_equals_plain_token_by_token(tmp_path, key):
    """The plain implementation agrees with itself however the prompt is cut: the states it hands on are the
    whole of what a later token needs."""
    config, seed = CONFIGS[key]
    cfg, w = plain.read_model_folder(make_folder(str(tmp_path / key), config, seed))
    ids = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(7)).tolist()
    whole = plain.forward_logits(cfg, w, ids)
    rows, states = [], None
    for cut in ([5, 1, 2, 9, 1, 1, 4] if key == "p" else [1] * 23):
        at = sum(r.shape[0] for r in rows)
        logits, states = plain.forward(cfg, w, ids[at:at + cut], states)
        rows.append(logits)
    assert float((torch.cat(rows) - whole).abs().max()) < 1e-9 * float(whole.abs().max())


def test_plain_mechanisms_on_values_worked_by_hand():
    one = torch.ones(1, dtype=plain.F64)
    # shift: the first token is pulled towards zero, the second towards the first
    h, last = plain.token_shift(torch.tensor([[2.0], [6.0]], dtype=plain.F64), 0.25 * one, None)
    assert h.flatten().tolist() == [1.5, 5.0] and last.tolist() == [6.0]
    # convolution: the last tap meets the current token, zeros come before the start
    out, tail = plain.causal_conv(torch.tensor([[1.0], [2.0], [3.0]], dtype=plain.F64),
                                  torch.tensor([[100.0, 10.0, 1.0]], dtype=plain.F64), 0.5 * one, None)
    assert out.flatten().tolist() == [1.5, 12.5, 123.5] and tail.flatten().tolist() == [2.0, 3.0]
    # temperature: floor((p + 1) / every) changes at p = every - 1
    tau = plain.query_temperature(torch.tensor([0, 5, 6, 13]), 1.0, 7)
    assert torch.allclose(tau, 1 + torch.log(torch.tensor([1.0, 1.0, 2.0, 3.0], dtype=plain.F64)))
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=plain.F64))) - 0.8411919906082768) < 1e-12
