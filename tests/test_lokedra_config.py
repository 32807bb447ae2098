"""Lokedra without a GPU: the configuration and its errors, the model as data (the loop's schedule, the states a layer's
parts keep under their names, tensor names), and the plain rules on hand cases."""
import copy

import numpy as np
import pytest

import plain_lokedra as PL
from kapel_b200.cache import CacheManager, CacheNeeds, PagedKV, StateSpec
from kapel_b200.config import ConfigError, config_from_json

MOE = {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 12, "limit": 1.5}}
RAW = {"architecture": "Lokedra", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
       "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
    {"type": "general_delta", "mixer": {"heads": 2, "dim": 8, "lora": 5}, "mlp": MOE},
    {"type": "parallel", "mlp": None, "mixer": {
        "left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "conv": 3, "scale": 0.3, "mask": {"size": 9}},
        "right": {"heads": 2, "dim": 6, "vdim": 10}, "left_scale": 0.5, "right_scale": 2.0}},
    {"type": "latent_attention", "mlp": MOE, "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 8, "q_rank": 10, "kv_rank": 12, "scale": 0.25,
                                                      "rot": {"base": 50.0, "dims": 4, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}}},
]}


def test_round_trip_and_schedule():
    c = config_from_json(RAW)
    assert type(c).__name__ == "LokedraConfig" and config_from_json(c.to_json()) == c
    spec = c.to_spec()
    # the embedding's output is added ahead of every pass of the loop but the first
    assert [(e.layer, e.replica, e.before is not None) for e in spec.schedule] == \
        [(0, 0, False), (1, 0, False), (2, 0, False), (1, 1, True), (2, 1, False), (1, 2, True), (2, 2, False)]
    assert all(l.kind == "parallel" and set(l.norms) == {"pre"} and l.norms["pre"].offset == 1.0 for l in spec.layers)
    assert spec.layers[1].ffn is None and spec.layers[1].scales == ("l1.ls1", None) and spec.layers[0].scales == ("l0.ls1", "l0.ls2")
    assert spec.head.weight == "embed" and spec.embed.scale == 3.0 and spec.final_norm.offset == 1.0
    left = spec.layers[1].mixer.left
    assert left.values_are_keys and left.conv == 3 and left.block_mask == 9 and left.unit_sink and left.out_bias and left.position.kind == "none"
    lat = spec.layers[2].mixer
    assert lat.position.pairing == "neighbours" and lat.position.scaling.factor == 4.0 and not lat.sink and not lat.gated
    moe = spec.layers[0].ffn
    assert moe.scoring == "softmax" and not moe.renormalize and moe.gated and moe.limit == 1.5 and moe.activation == "clamped_swish"
    assert abs(spec.layers[0].mixer.decay_scale - np.exp(-0.5)) < 1e-12
    no_loop = copy.deepcopy(RAW)
    del no_loop["loop"]
    assert [(e.layer, e.replica, e.before) for e in config_from_json(no_loop).to_spec().schedule] == [(0, 0, None), (1, 0, None), (2, 0, None)]
    once = dict(copy.deepcopy(RAW), loop={"start": 0, "stop": 3, "times": 1})
    assert [e.before for e in config_from_json(once).to_spec().schedule] == [None, None, None]
    empty = dict(copy.deepcopy(RAW), loop={"start": 2, "stop": 2, "times": 5})
    assert len(config_from_json(empty).to_spec().schedule) == 3


def test_tensor_names_shapes_and_the_size_only_a_tensor_gives():
    from kapel_b200.parts import expected_tensors

    t = expected_tensors(config_from_json(RAW).to_spec())
    assert t["embed"] == (50, 24) and "head" not in t and t["final.norm"] == (24,)
    assert t["l0.mix.r"] == (16, 24) and t["l0.mix.w1"] == (5, 24) and t["l0.mix.w2"] == (16, 5) and t["l0.mix.a.b"] == (16,) and t["l0.mix.norm"] == (16,)
    assert t["l0.mlp.e3.gate"] == (12, 24) and t["l0.mlp.e0.down"] == (24, 12) and t["l0.mlp.correction"] == (4,) and t["l0.shift"] == (24,)
    assert t["l1.mix.left.q"] == (32, 24) and t["l1.mix.left.k.conv"] == (16, 3) and t["l1.mix.left.o.b"] == (24,) and "l1.mix.left.v" not in t
    assert t["l1.mix.right.lower"] == (12,) and t["l1.mix.right.norm"] == (10,) and t["l1.mix.right.o"] == (24, 20) and "l1.ls2" not in t
    assert t["l2.mix.dkv"] == (16, 24) and t["l2.mix.uq"] == (20, 10) and "l2.mix.sink" not in t and "l2.mix.g" not in t
    bare = copy.deepcopy(RAW)
    del bare["layers"][0]["mixer"]["lora"]
    c = config_from_json(bare)
    with pytest.raises(ConfigError, match="tensors"):
        c.to_spec()
    shapes = {"l0.mix.w1": (7, 24)}
    assert c.with_shapes(lambda n: shapes[n]).layers[0].mixer.lora == 7
    with pytest.raises(ConfigError, match="missing"):
        c.with_shapes(lambda n: {}[n])


@pytest.mark.parametrize("edit,words", [
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][1]["mixer"]["left"].update(vdim=6), "no value projection"),
    (lambda r: r["layers"][1]["mixer"]["left"].pop("mask"), "mask"),
    (lambda r: r["layers"][1]["mixer"]["left"].update(conv=0), "conv"),
    (lambda r: r["layers"][1]["mixer"].pop("right"), "right"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=2), "rot_dim"),
    (lambda r: r["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda r: r["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda r: r["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda r: r["loop"].update(stop=4), "loop.stop"),
    (lambda r: r["loop"].update(times=0), "loop.times"),
    (lambda r: r.pop("width"), "width"),
])
def test_what_the_file_cannot_say(edit, words):
    raw = copy.deepcopy(RAW)
    edit(raw)
    with pytest.raises(ConfigError, match=words):
        config_from_json(raw)


def test_a_layers_parts_keep_their_states_under_their_names():
    a = CacheNeeds(paged=PagedKV(2, 8, None, 0, None, shared_values=True), states=(("conv", StateSpec((5,))),))
    b = CacheNeeds(state=StateSpec((7,)))
    both = a.named("left").merged(b.named("right")).named("mixer").merged(CacheNeeds(states=(("shift", StateSpec((3,))),)))
    assert both.paged == a.paged and both.state is None
    assert dict(both.states) == {"mixer.left.conv": StateSpec((5,)), "mixer.right": StateSpec((7,)), "shift": StateSpec((3,))}
    with pytest.raises(ValueError, match="pages"):
        a.merged(a.named("x"))
    with pytest.raises(ValueError, match="same name"):
        b.named("x").merged(b.named("x"))
    made = []
    m = CacheManager({0: both, 1: b}, 16, 4, 3, allocate=lambda shape, dtype: made.append(shape) or np.zeros(shape), dtype="float32")
    assert set(m.states) == {(0, "mixer.left.conv"), (0, "mixer.right"), (0, "shift"), 1}
    assert m.states[(0, "shift")].shape == (4, 3) and m.states[1].shape == (4, 7)


# -------------------------------------------------------------------------------------- the plain rules on hand cases
def test_generalized_delta_rule_by_hand():
    """Without decay and with a removal rate of one, a unit key's old value is removed before the new one is written
    (the delta rule); with a removal rate of zero values under one key add up; the decay fades a channel's row."""
    d = 4
    one, zero = np.ones((4, d)), np.zeros((4, d))
    k = np.eye(d)[[0, 1, 0, 2]].astype(np.float64)
    v = np.arange(16, dtype=np.float64).reshape(4, d) + 1
    r = np.eye(d)[[0, 0, 0, 0]].astype(np.float64)
    out = PL.general_delta_recurrence(r, k, v, one, one)
    assert np.allclose(out[0], v[0], atol=1e-5) and np.allclose(out[1], v[0], atol=1e-5) and np.allclose(out[2], v[2], atol=1e-4)
    out = PL.general_delta_recurrence(r, k, v, one, zero)
    assert np.allclose(out[2], v[0] + v[2]) and np.allclose(out[3], v[0] + v[2])
    out = PL.general_delta_recurrence(r, k, v, one * 0.5, zero)
    assert np.allclose(out[1], 0.5 * v[0]) and np.allclose(out[2], 0.25 * v[0] + v[2])


def test_forget_gate_memory_by_hand():
    """A gate of 1 keeps the memory and writes nothing; a gate of 0 replaces the channel's row by the value."""
    q = np.array([[1.0, 0.0], [1.0, 0.0], [1.0, 1.0]])
    v = np.array([[2.0], [5.0], [7.0]])
    f = np.array([[0.0, 0.0], [1.0, 1.0], [0.5, 0.0]])
    out = PL.forget_gate_recurrence(q, f, v)
    assert np.allclose(out[:, 0], [2.0, 2.0, 0.5 * 2.0 + 0.5 * 7.0 + 7.0])


def test_shift_convolution_chunks_and_rotation_by_hand():
    h = np.array([[1.0, 2.0], [3.0, 6.0], [5.0, 5.0]])
    assert np.allclose(PL.token_shift(h, np.array([0.0, 1.0])), [[1.0, 0.0], [3.0, 2.0], [5.0, 6.0]])
    x = np.array([[1.0], [2.0], [4.0]])
    assert np.allclose(PL.short_conv(x, np.array([[10.0, 1.0]])), [[1.0], [12.0], [24.0]])           # the last weight is the row's own
    s = np.zeros((5, 5))
    i, j = np.arange(5)[:, None], np.arange(5)[None, :]
    w = PL.masked_softmax(s, (j <= i) & (i // 2 == j // 2), one_more=True)
    assert np.allclose(w[1], [1 / 3, 1 / 3, 0, 0, 0]) and np.allclose(w[2], [0, 0, 0.5, 0, 0]) and np.allclose(w[4], [0, 0, 0, 0, 0.5])
    # neighbouring components turn together; a pair that turns fast is left alone by the stretching, a slow one is slowed
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0}}
    f, mag = PL.stretched_frequencies(rot)
    assert np.isclose(f[0], 1.0) and np.isclose(f[1], 0.1 / 4.0) and np.isclose(mag, 0.1 * np.log(4.0) + 1.0)
    x = np.array([[[1.0, 0.0, 0.0, 1.0]]])
    y = PL.rotate_pairs(x, [3], rot)[0, 0]
    assert np.allclose(y, mag * np.array([np.cos(3.0), np.sin(3.0), -np.sin(0.075), np.cos(0.075)]))


def test_experts_by_hand():
    t = {"m.router": np.array([[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]]), "m.correction": np.array([0.0, 0.0, 10.0])}
    chosen, weights = PL.route(np.array([[2.0, 0.0]]), t, "m", {"router": {"top": 2}})
    s = np.exp([2.0, 0.0, 0.0]) / np.exp([2.0, 0.0, 0.0]).sum()
    assert list(chosen[0]) == [2, 0] and np.allclose(weights[0], [s[2], s[0]])                  # the correction chooses, the score weighs
    t = {"e.gate": np.array([[1.0]]), "e.up": np.array([[1.0]]), "e.down": np.array([[1.0]])}
    y = PL.expert(np.array([[5.0], [-5.0]]), t, "e", 2.0)
    assert np.allclose(y[:, 0], [2.0 * PL.sigmoid(1.702 * 2.0) * 3.0, -5.0 * PL.sigmoid(1.702 * -5.0) * -1.0])
