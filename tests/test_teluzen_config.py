"""Teluzen without a GPU: the configuration and its errors, the model as data (tensor names, cache
needs, which layer keeps values for the others), the scaled rotation's frequencies, the cutting of
keys into slices, and the plain rules on hand cases."""
import copy
import math

import numpy as np
import pytest

import plain_teluzen as PT
from kapel_b200.config import ConfigError, config_from_json


def layer(heads, kv_heads, dim, vdim, scale, size, pool, rot, v_mix, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size, "pool": pool}, "v_mix": v_mix}
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def moe(ff, experts, top, shared_ff=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        out["shared"] = {"ff": shared_ff}
    return out


RAW = {"architecture": "Teluzen", "vocab": 50, "width": 24, "max_positions": 96, "norm": {"eps": 1e-5}, "layers": [
    layer(4, 2, 8, 6, 0.3, 12, 4, {"base": 100.0, "dims": 4}, False, {"kind": "dense", "ff": 16}),
    layer(2, 1, 8, 12, 0.25, 7, 3, {"base": 1000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}, True, moe(8, 5, 2, 16)),
    layer(3, 1, 6, 12, 0.4, 9, 2, None, True, None),
    layer(2, 1, 8, 12, 0.2, 5, 5, {"base": 50.0, "dims": 8}, True, moe(8, 3, 1)),
]}


def test_round_trip_and_the_model_as_data():
    c = config_from_json(RAW)
    assert type(c).__name__ == "TeluzenConfig" and config_from_json(c.to_json()) == c
    spec = c.to_spec()
    assert [l.mixer.value_mix for l in spec.layers] == [None, "source", "mix", "mix"]
    assert [l.mixer.pool for l in spec.layers] == [4, 3, 2, 5] and [l.mixer.window for l in spec.layers] == [12, 7, 9, 5]
    assert [l.mixer.pool_blocks for l in spec.layers] == [24, 32, 48, 19]
    assert spec.layers[2].ffn is None and set(spec.layers[2].norms) == {"pre_mixer", "post_mixer"}
    assert spec.layers[0].ffn.kind == "mlp" and spec.layers[0].ffn.activation == "relu2"
    m = spec.layers[1].ffn
    assert m.kind == "moe" and m.gated and m.scoring == "softmax_chosen" and m.shared.intermediate == 16 and m.top == 2
    assert spec.layers[3].ffn.shared is None and spec.layers[3].ffn.top == 1
    assert spec.layers[2].mixer.position.kind == "none" and spec.layers[1].mixer.position.pairing == "neighbours"
    assert spec.layers[1].mixer.position.scaling.factor == 4.0 and spec.layers[0].mixer.position.scaling is None
    assert spec.embed.positions == "pos" and spec.embed.max_positions == 96 and spec.embed.scale == 1.0
    assert all(n.kind == "rms" and n.offset == 0.0 for l in spec.layers for n in l.norms.values())


def test_tensor_names_and_shapes():
    from kapel_b200.parts import expected_tensors

    t = expected_tensors(config_from_json(RAW).to_spec())
    assert t["embed"] == (50, 24) and t["pos"] == (96, 24) and t["head"] == (50, 24) and t["final.norm"] == (24,)
    assert t["l0.mix.q"] == (32, 24) and t["l0.mix.k"] == (16, 24) and t["l0.mix.v"] == (12, 24) and t["l0.mix.o"] == (24, 24)
    assert t["l0.mix.q.b"] == (32,) and t["l0.mix.k.b"] == (16,) and t["l0.mix.v.b"] == (12,)
    assert t["l0.mix.q.norm"] == (32,) and t["l0.mix.k.norm"] == (16,) and t["l0.mix.talk"] == (4, 4) and t["l0.mix.temp"] == (4,)
    assert "l0.mix.vmix" not in t and "l1.mix.vmix" not in t and t["l2.mix.vmix"] == () and t["l3.mix.vmix"] == ()
    assert t["l0.mlp.up"] == (16, 24) and t["l0.mlp.down"] == (24, 16) and "l0.mlp.gate" not in t
    assert t["l1.mlp.router"] == (5, 24) and t["l1.mlp.e4.gate"] == (8, 24) and t["l1.mlp.e0.down"] == (24, 8) and "l1.mlp.e5.up" not in t
    assert t["l1.mlp.shared.gate"] == (16, 24) and t["l1.mlp.shared.down"] == (24, 16) and "l3.mlp.shared.up" not in t
    assert "l2.norm2" not in t and "l2.mlp.up" not in t and t["l2.norm1b"] == (24,) and t["l3.norm2b"] == (24,)


@pytest.mark.parametrize("edit,words", [
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=3), "even"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda r: r["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda r: r["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].update(v_mix=1), "v_mix"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=10), "v_mix"),
    (lambda r: r["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda r: r["layers"][0]["mlp"].update(kind="gated"), "kind"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda r: r["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r.pop("max_positions"), "max_positions"),
    (lambda r: r.update(layers=[]), "layers"),
])
def test_errors_name_the_key(edit, words):
    raw = copy.deepcopy(RAW)
    edit(raw)
    with pytest.raises(ConfigError, match=words):
        config_from_json(raw)


def test_cache_needs_pages_for_the_window_and_a_slot_of_block_means():
    import torch

    from kapel_b200.engine.model import ModelParts
    from kapel_b200.parts import BuildContext

    spec = config_from_json(RAW).to_spec()
    model = ModelParts(spec, BuildContext(dtype=torch.float32, device=torch.device("cpu")))
    needs = model.cache_needs()
    assert sorted(needs) == [0, 1, 2, 3]
    assert [needs[i].paged.window for i in range(4)] == [12, 7, 9, 5]                      # at least a block's tokens stay until it is whole
    assert needs[0].state.shape == (24, 2, 8 + 6) and needs[1].state.shape == (32, 1, 8 + 12) and needs[3].state.shape == (19, 1, 8 + 12)
    wide = copy.deepcopy(RAW)
    wide["layers"][0]["mixer"]["mask"] = {"size": 3, "pool": 8}                            # a block longer than the window
    needs = ModelParts(config_from_json(wide).to_spec(), BuildContext(dtype=torch.float32, device=torch.device("cpu"))).cache_needs()
    assert needs[0].paged.window == 8


def test_scaled_frequencies_follow_the_plain_rule():
    from kapel_b200.config import RopeScaling
    from kapel_b200.parts.position import scaled_frequencies

    for dims, base, sc in ((8, 1000.0, (4.0, 64.0, 8.0, 1.0)), (32, 10000.0, (16.0, 512.0, 32.0, 2.0)), (6, 50.0, (2.0, 4096.0, 1.0, 1.0)),
                           (64, 500000.0, (8.0, 8192.0, 4.0, 0.5))):
        rot = {"dims": dims, "base": base, "scaling": dict(zip(("factor", "original", "fast", "slow"), sc))}
        want, factor = PT.rotary_frequencies(rot)
        got, got_factor = scaled_frequencies(dims, base, RopeScaling(*sc))
        assert np.allclose(got, want, rtol=1e-14, atol=0) and math.isclose(got_factor, factor, rel_tol=1e-14)
    plain, one = scaled_frequencies(8, 100.0, None)
    assert one == 1.0 and np.allclose(plain, [100.0 ** (-2 * i / 8) for i in range(4)])
    # the ends of the ramp: a pair that turns often keeps its frequency, a slow one is divided by the factor
    f, _ = PT.rotary_frequencies({"dims": 64, "base": 10000.0, "scaling": {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}})
    assert math.isclose(f[0], 1.0) and math.isclose(f[31], 10000.0 ** (-62 / 64) / 8.0)


def test_who_sees_whom_on_hand_cases():
    # window 4, blocks of 3: position 9 sees tokens 6..9; block 0 (0..2) ends at 2 <= 5, block 1 (3..5) ends at 5 <= 5
    assert list(PT.seen_tokens(9, 4)) == [6, 7, 8, 9] and list(PT.seen_blocks(9, 4, 3)) == [0, 1]
    assert list(PT.seen_blocks(8, 4, 3)) == [0]                                            # 5 > 8 - 4: token 4 has left the window and is not seen at all
    assert list(PT.seen_tokens(2, 4)) == [0, 1, 2] and list(PT.seen_blocks(3, 4, 3)) == [] and list(PT.seen_blocks(5, 4, 3)) == []
    assert list(PT.seen_blocks(6, 4, 3)) == [0]
    assert list(PT.seen_blocks(7, 1, 1)) == list(range(7)) and list(PT.seen_tokens(7, 1)) == [7]
    assert list(PT.seen_blocks(20, 2, 8)) == [0, 1] and list(PT.seen_blocks(17, 2, 8)) == [0, 1] and list(PT.seen_blocks(16, 2, 8)) == [0]


def test_slices_of_the_keys_cover_them_in_multiples_of_the_chunk():
    from kapel_b200.engine.batch import pooled_slices

    for rows, longest, window, pool in ((1, 5000, 1024, 16), (3, 130, 64, 8), (1, 64, None, 0), (300, 100000, 512, 4), (2, 3000, None, 0), (1, 1 << 20, 4096, 64)):
        slices, keys = pooled_slices(rows, longest, window, pool, 148, 64)
        tokens = min(longest, window) if window else longest
        seen = tokens + (max(0, longest - window) // pool if (window and pool) else 0)
        if slices == 1:
            assert keys == 0
        else:
            assert keys % 64 == 0 and (slices - 1) * keys < seen <= slices * keys and slices * rows <= 2 * 148 + rows
