"""The Gupizen configuration on the host: what config.json gives, what is refused, the order of runs that a loop makes,
and the parts and tensors the specification asks for."""
import copy

import pytest

import gupizen_models as gm
from mynah_slm_b200.config.keys import ConfigError
from mynah_slm_b200.engine.model import Model
from mynah_slm_b200.registry import known_architectures, parse_config


def test_registered_and_round_trips():
    assert "Gupizen" in known_architectures()
    for cfg in gm.CONFIGS.values():
        typed = parse_config(cfg)
        assert parse_config(typed.to_dict()).to_dict() == typed.to_dict()
        back = typed.to_dict()
        assert back["layers"] == cfg["layers"] and back.get("loop") == cfg.get("loop") and back["canon"] == cfg["canon"]


@pytest.mark.parametrize("name,runs", [
    ("hybrid", [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False), (4, False)]),
    ("odd", [(0, False), (1, False), (0, True), (1, False), (2, False)]),
    ("once", [(0, False), (1, False), (2, False)]),
    ("parallel", [(0, False)])])
def test_order_of_runs(name, runs):
    spec = parse_config(gm.CONFIGS[name]).model_spec()
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == runs
    assert all(e.cache_from is None for e in spec.schedule)          # every pass has cache and state of its own


def test_tensors_and_cache_groups():
    for name, cfg in gm.CONFIGS.items():
        model = Model(parse_config(cfg).model_spec())
        want = gm.tensor_shapes(cfg)
        got = {ts.name: ts.shape for _, ts in model.tensor_specs() if not ts.ignorable}
        assert set(got) == set(want), name
        for n, shape in got.items():
            assert len(shape) == len(want[n]) and all(a in (-1, b) for a, b in zip(shape, want[n])), (name, n)
    model = Model(parse_config(gm.HYBRID).model_spec())
    plan = model.cache_plan()
    # layer 2 runs three times: three entries in its group; windows and head sizes set the groups apart
    groups = {(g.kv_heads, g.head_dim, g.window, g.v_head_dim): len(g.entries) for g in plan.groups}
    assert groups == {(2, 16, 40, 24): 1, (3, 8, 70, 16): 3, (1, 32, 130, 8): 1}
    assert all(e.block_state is not None for e in plan.entries)      # the input convolutions' last rows
    assert sorted(plan.entries[0].state) == ["1"] and sorted(plan.entries[0].state["1"]) == ["S", "conv"]
    assert sorted(plan.entries[1].state) == ["S", "conv"]


def test_narrow_sizes_come_from_the_file_or_the_tensors():
    spec = parse_config(gm.HYBRID).model_spec()
    shapes = {ts.name: ts.shape for _, ts in Model(spec).tensor_specs()}
    assert shapes["l1.mix.a1"] == (-1, 64) and shapes["l1.mix.g2"] == (4 * 8, -1)
    assert shapes["l3.mix.a1"] == (8, 64) and shapes["l3.mix.g2"] == (2 * 12, 16)


def _broken(path, value, base=gm.HYBRID):
    cfg = copy.deepcopy(base)
    at = cfg
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value", [
    (("vocab",), None), (("norm",), None), (("canon", "taps"), None), (("embedding",), None), (("layers",), []),
    (("layers", 0, "type"), "other"), (("layers", 0, "mixer", "left", "heads"), 3), (("layers", 0, "mixer", "left", "vdim"), 7),
    (("layers", 0, "mixer", "left", "rot", "dims"), 18), (("layers", 0, "mixer", "left", "rot", "dims"), 7),
    (("layers", 0, "mixer", "left", "mask"), None), (("layers", 0, "mixer", "right", "blocks"), 5),
    (("layers", 0, "mixer", "left", "rot", "scaling", "high"), 1.0), (("layers", 1, "mixer", "kv_heads"), 3),
    (("layers", 0, "mlp", "kind"), "dense"), (("layers", 0, "mlp", "router", "top"), 9), (("loop", "stop"), 9), (("loop", "start"), 3),
    (("norm", "eps"), 0.0)])
def test_refused(path, value):
    with pytest.raises(ConfigError):
        parse_config(_broken(path, value)).model_spec()


def test_a_wrong_tensor_shape_is_named(tmp_path):
    import torch
    from mynah_slm_b200.weights.loader import WeightError, check
    from mynah_slm_b200.weights.safetensors_io import Checkpoint
    W = gm.make_weights(gm.RAGGED, 1)
    W["l1.mix.a2"] = torch.zeros((3, 12), dtype=torch.bfloat16)
    folder = gm.write_model(str(tmp_path / "m"), gm.RAGGED, W)
    model = Model(parse_config(gm.RAGGED).model_spec())
    with pytest.raises(WeightError) as e:
        check(model.tensor_specs(), Checkpoint(folder))
    assert [n for n, _, _ in e.value.wrong_shape] == ["l1.mix.a2"]
