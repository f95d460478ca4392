"""Bikadra without a GPU: its configuration, what the model asks of the weights and of the cache, and the plain
implementation against itself (a prompt whole and token by token through the explicit caches and states) and on
values worked by hand."""

import copy
import math

import pytest
import torch

import plain_bikadra as plain
from bikadra_models import BIKADRA_X, BIKADRA_Y, CONFIGS, make_folder, tensor_shapes


def model_of(config):
    from qwen3_from_scratch_b200.engine.model import Model
    from qwen3_from_scratch_b200.registry import build_model_spec, config_from_dict
    return Model(build_model_spec(config_from_dict(config)))


@pytest.mark.parametrize("key", list(CONFIGS))
def test_the_model_asks_for_the_tensors_the_design_names(key):
    config = CONFIGS[key][0]
    asked = {s.name: tuple(s.shape) for s in model_of(config).weight_specs()}
    assert asked == tensor_shapes(config)


def test_configuration_round_trip():
    from qwen3_from_scratch_b200.registry import config_from_dict
    cfg = config_from_dict(BIKADRA_X)
    assert cfg.architecture == "Bikadra" and cfg.streams == 3 and cfg.loop == (1, 3, 3)
    assert cfg.layers[0].rot_scaling.factor == 4.0 and cfg.layers[2].rot_scaling is None
    assert config_from_dict(cfg.to_dict()) == cfg
    y = config_from_dict(BIKADRA_Y)
    assert y.loop is None and y.logit_softcap is None and config_from_dict(y.to_dict()) == y


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"].update(groups=4), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "multiple"),
    (lambda c: c["layers"][0].update(type="hyena"), "not built"),
    (lambda c: c["layers"][0].update(mlp={"kind": "moe", "ff": 8}), "dense"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c.pop("streams"), "streams"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_configuration_errors_name_the_key(change, message):
    from qwen3_from_scratch_b200.config.model_config import ConfigError
    from qwen3_from_scratch_b200.registry import config_from_dict
    config = copy.deepcopy(BIKADRA_X)
    change(config)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_run_order_and_cache_needs():
    """The looped span becomes further runs of the same layers, each with a cache id of its own; attention runs
    keep pages with a latent plane and a rotated-key plane, state-space runs a state and a convolution tail."""
    from qwen3_from_scratch_b200.parts.base import PagedCacheSpec, StateSpec
    model = model_of(BIKADRA_X)
    assert [c.layer for c in model.spec.order] == [0, 1, 2, 1, 2, 1, 2, 3] == plain.run_order(BIKADRA_X)
    assert [c.cache for c in model.spec.order] == list(range(8))
    layout = model.cache_layout()
    groups = {tuple((p.name, p.heads, p.width) for p in g.spec.planes): g.cache_ids for g in layout.groups}
    assert groups == {(("c", 1, 40), ("r", 1, 16)): [0], (("c", 1, 48), ("r", 1, 8)): [2, 4, 6]}
    assert layout.states[(1, "state")] == StateSpec((6, 24, 16), "float32") == layout.states[(5, "state")]
    assert layout.states[(3, "conv")] == StateSpec((3, 6 * 16 + 2 * 3 * 24), "float32")
    assert layout.states[(7, "conv")] == StateSpec((1, 4 * 8 + 2 * 40), "float32")
    assert all(isinstance(g.spec, PagedCacheSpec) and g.spec.window is None for g in layout.groups)
    assert len(model.layers) == 4


def test_random_model_folder_through_the_framework_writer(tmp_path):
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), config_from_dict(BIKADRA_Y), seed=1)
    cfg, w = plain.read_model_folder(folder)
    assert {k: tuple(v.shape) for k, v in w.items()} == tensor_shapes(BIKADRA_Y)
    assert torch.isfinite(plain.forward_logits(cfg, w, [3, 1, 4, 1, 5])).all()


@pytest.mark.parametrize("key", ["x", "y"])
def test_plain_whole_prompt_equals_plain_token_by_token(tmp_path, key):
    config, seed = CONFIGS[key]
    cfg, w = plain.read_model_folder(make_folder(str(tmp_path / key), config, seed))
    ids = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(5)).tolist()
    whole = plain.forward_logits(cfg, w, ids)
    rows, states = [], None
    for cut in ([ids[:9], ids[9:11]] + [[t] for t in ids[11:]]):
        logits, states = plain.forward(cfg, w, cut, states)
        rows.append(logits)
    assert float((torch.cat(rows) - whole).abs().max()) < 1e-9 * float(whole.abs().max())


def test_plain_mechanisms_on_values_worked_by_hand():
    # the streams: read, then write from the old streams with mix indexed [from, to]
    xs = torch.tensor([[[1.0, 2.0]], [[10.0, 20.0]]], dtype=plain.F64)  # two streams, one token, width 2
    assert plain.streams_read(xs, torch.tensor([0.5, 2.0], dtype=plain.F64)).tolist() == [[20.5, 41.0]]
    mix = torch.tensor([[1.0, 3.0], [0.0, 2.0]], dtype=plain.F64)  # stream 0 goes to both, stream 1 only to itself
    new = plain.streams_write(xs, torch.tensor([[1.0, 1.0]], dtype=plain.F64), mix, torch.tensor([100.0, 0.0], dtype=plain.F64))
    assert new.tolist() == [[[101.0, 102.0]], [[23.0, 46.0]]]
    # stretched frequencies: no scaling gives the plain ones; with scaling the slow pairs are divided by the factor
    f, mag = plain.yarn_frequencies(8, 100.0, None)
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=plain.F64))
    f2, mag2 = plain.yarn_frequencies(8, 100.0, {"factor": 4.0, "original": 2 * math.pi * 10, "fast": 10.0, "slow": 1.0})
    # pair(10) = 0, pair(1) = 8 ln 10 / (2 ln 100) = 2: ramp 0, 0.5, 1, 1
    assert abs(mag2 - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    assert torch.allclose(f2, f * torch.tensor([1.0, 0.625, 0.25, 0.25], dtype=plain.F64))
    # rotation of the pair (i, i + dims / 2) by position * f, the rest passing
    x = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 7.0]]], dtype=plain.F64)
    out = plain.rotate_half(x, torch.tensor([3]), torch.tensor([math.pi / 6, 0.0], dtype=plain.F64), 2.0)
    assert torch.allclose(out, torch.tensor([[[0.0, 0.0, 2.0, 2.0, 7.0]]], dtype=plain.F64), atol=1e-12)
    # the convolution: the last column multiplies the current token, zeros before the start, the tail carried on
    y, tail = plain.causal_conv(torch.tensor([[1.0], [2.0], [3.0]], dtype=plain.F64),
                                torch.tensor([[100.0, 10.0, 1.0]], dtype=plain.F64), torch.tensor([0.5], dtype=plain.F64), None)
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5] and tail[:, 0].tolist() == [2.0, 3.0]
    y2, _ = plain.causal_conv(torch.tensor([[4.0]], dtype=plain.F64), torch.tensor([[100.0, 10.0, 1.0]], dtype=plain.F64),
                              torch.tensor([0.5], dtype=plain.F64), tail)
    assert y2[0, 0].item() == 234.5
