"""The Gomuzen configuration on the host: what config.json gives, what is refused, the order of runs that a loop makes
with the vector each pass adds, the parts, tensors and cache groups the specification asks for, and controls that the
plain implementation would notice a wrong reading."""
import copy
import zlib

import numpy as np
import pytest

import gomuzen_models as gm
from helpers import rel_err
from mynah_slm_b200.config.keys import ConfigError
from mynah_slm_b200.engine.model import Model
from mynah_slm_b200.registry import known_architectures, parse_config
from plain import gomuzen as plain


def test_registered_and_round_trips():
    assert "Gomuzen" in known_architectures()
    for cfg in gm.CONFIGS.values():
        typed = parse_config(cfg)
        assert parse_config(typed.to_dict()).to_dict() == typed.to_dict()
        back = typed.to_dict()
        assert back["layers"] == cfg["layers"] and back.get("loop") == cfg.get("loop")


@pytest.mark.parametrize("name,runs", [
    ("hybrid", [(0, None), (1, 0), (2, None), (3, None), (1, 1), (2, None), (3, None), (1, 2), (2, None), (3, None), (4, None),
                (5, None), (6, None)]),
    ("odd", [(0, 0), (1, None), (2, None), (3, None), (4, None)]),
    ("plain", [(0, None), (1, None)])])
def test_order_of_runs_and_their_vectors(name, runs):
    spec = parse_config(gm.CONFIGS[name]).model_spec()
    assert [(e.layer, e.add_vector) for e in spec.schedule] == runs
    assert all(e.cache_from is None and not e.add_embedding for e in spec.schedule)      # every pass has a cache of its own
    assert (spec.stream_vectors is None) == ("loop" not in gm.CONFIGS[name])
    assert plain.layer_runs(gm.CONFIGS[name]) == runs


def test_tensors_and_cache_groups():
    for name, cfg in gm.CONFIGS.items():
        model = Model(parse_config(cfg).model_spec())
        want = gm.tensor_shapes(cfg)
        got = {ts.name: tuple(ts.shape) for _, ts in model.tensor_specs() if not ts.ignorable}
        assert got == want, name
    plan = Model(parse_config(gm.HYBRID).model_spec()).cache_plan()
    # (key heads, stored key width, window that frees pages, stored value width, value heads) -> runs kept there
    groups = {(g.kv_heads, g.head_dim, g.window, g.v_head_dim, g.v_heads): len(g.entries) for g in plan.groups}
    assert groups == {(1, 48, None, 0, 1): 1,        # the latent of 40 + 8
                      (4, 16, None, 24, 2): 3,       # two maps on each of two kv heads, three passes
                      (2, 16, None, 8, 2): 3,        # a window that keeps first tokens gives no page back
                      (1, 24, None, 16, 1): 3,
                      (1, 40, None, 0, 1): 1,
                      (6, 8, None, 16, 3): 1,
                      (4, 8, 70, 8, 4): 1}           # a window alone does
    assert all(e.state is None and e.block_state is None for e in plan.entries)


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


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "mamba", "type"), (("layers", 1, "mixer", "softcap"), None, "softcap"),
    (("layers", 1, "mixer", "diff"), None, "diff"), (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "rot.dims"), (("layers", 2, "mixer", "rot", "dims"), 18, "rot.dims"),
    (("layers", 2, "mixer", "mask", "size"), None, "size"), (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 0, "mlp", "router", "top"), 5, "top"), (("layers", 0, "mlp", "router", "scale"), None, "scale"),
    (("layers", 0, "mlp", "expert", "limit"), None, "limit"), (("loop", "stop"), 9, "loop"), (("norm",), None, "norm"),
    (("layers", 3, "mixer", "scale"), 0.0, "scale"), (("vocab",), 2.5, "vocab")])
def test_refusals_name_the_key(path, value, word):
    with pytest.raises(ConfigError) as e:
        parse_config(_broken(path, value))
    assert word in str(e.value)


def test_what_may_be_absent():
    cfg = _broken(("layers", 2, "mixer", "mask", "keep_first"), None)
    assert parse_config(cfg).model_spec().layers[2].mixer["keep_first"] == 0
    cfg = _broken(("layers", 0, "mlp", "router", "groups"), None)
    ffn = parse_config(cfg).model_spec().layers[0].ffn
    assert (ffn["groups"], ffn["keep"]) == (1, 1)
    spec = parse_config(gm.HYBRID).model_spec()
    assert spec.layers[3].mixer["window"] is None and spec.layers[3].ffn is None and "ffn" not in spec.layers[3].norms


# ------------------------------------------------------------------ controls on the plain implementation
def _logits(cfg, W, n=90, seed=3):
    toks = np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()
    return plain.forward(cfg, W, toks)


def test_the_plain_implementation_notices_a_wrong_reading():
    cfg = gm.HYBRID
    W = gm.as_numpy(gm.make_weights(cfg, zlib.crc32(b"hybrid") % 1000))
    ref = _logits(cfg, W)
    for path, value in ((("layers", 1, "mixer", "diff"), 0.31), (("layers", 1, "mixer", "softcap"), 3.0),
                        (("layers", 2, "mixer", "mask", "size"), 39), (("layers", 2, "mixer", "mask", "keep_first"), 4),
                        (("layers", 0, "mlp", "router", "scale"), 1.6), (("layers", 0, "mlp", "expert", "limit"), 1.4),
                        (("layers", 0, "mixer", "scale"), 0.31), (("loop", "times"), 2),
                        (("layers", 2, "mixer", "rot", "scaling", "factor"), 3.9)):
        other = _broken(path, value)
        Wo = W if path != ("loop", "times") else {**W, "loop.step": W["loop.step"][:2]}
        assert rel_err(ref, _logits(other, Wo)) > 1e-3, path
    for name in ("loop.step", "l0.mix.g", "l1.mix.lq1", "l1.mix.k.norm", "l2.mix.k.b", "l0.mlp.correction", "l0.mix.dkv.norm"):
        Wo = dict(W)
        Wo[name] = W[name] * 1.5 + 0.05
        assert rel_err(ref, _logits(cfg, Wo)) > 1e-4, name
    # the pairing of rotated dimensions: the windowed mixer with the latent mixer's pairing gives other logits
    swapped = dict(plain.MIXERS)
    before = plain.turn

    def other_pairing(x, positions, rot, pairing):
        return before(x, positions, rot, "half" if pairing == "interleaved" else "interleaved")
    plain.turn = other_pairing
    try:
        assert rel_err(ref, _logits(cfg, W)) > 1e-3
    finally:
        plain.turn = before
    assert swapped == plain.MIXERS


def test_groups_leave_better_experts_out():
    """The best single expert sits in a group whose two largest sum to less than another group's, so it is NOT chosen;
    the weights carry the score without the correction; with two groups kept it comes back."""
    W = {"router": np.zeros((6, 4)), "correction": np.array([0.9, -2.0, 0.3, 0.35, -3.0, -3.1])}
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    picked, weights = plain.pick_experts(np.zeros((1, 4)), W, "", router)
    assert sorted(picked[0].tolist()) == [2, 3] and np.allclose(weights, 0.5 * 2.0)
    router["groups"]["keep"] = 2
    picked, _ = plain.pick_experts(np.zeros((1, 4)), W, "", router)
    assert sorted(picked[0].tolist()) == [0, 3]


def test_the_window_keeps_first_tokens_at_their_places():
    vis = plain.visible(np.arange(12), window=4, keep_first=2)
    assert vis[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert vis[3].tolist() == [True] * 4 + [False] * 8 and vis[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert plain.visible(np.arange(5)).sum() == 15
