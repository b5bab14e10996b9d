"""Host-side tests of the Damadra architecture: configuration parsing and its errors, the model description's
tensor names, the unrolled distance-bias rows against the plain bucket function, and what the output-norm block
hands between its parts."""
from __future__ import annotations

import copy

import pytest

import damadra_tiny as dt
import plain_damadra as plain
from reinfer_b200.config.damadra import DamadraConfig
from reinfer_b200.config.errors import InvalidValue, MissingKey
from reinfer_b200.config.registry import resolve_architecture


def test_round_trip_and_registry():
    for cfg in (dt.TINY_A, dt.TINY_B, dt.TINY_C, dt.TINY_D):
        c = DamadraConfig.from_dict(cfg)
        assert DamadraConfig.from_dict(c.to_dict()) == c
        assert resolve_architecture(c.to_dict()).config_cls is DamadraConfig
        assert c.vocab_size == cfg["vocab"] and c.hidden_size == cfg["width"]
        assert c.residual_mult == cfg["residual_mult"] and c.embedding_scale == cfg["embedding"]["scale"]


def test_bias_rows_come_from_the_checkpoint_shapes():
    raw = copy.deepcopy(dt.TINY_A)
    rows = [l["mixer"].pop("bias_rows") for l in raw["layers"]]
    with pytest.raises(MissingKey):
        DamadraConfig.from_dict(raw)
    shapes = {f"l{i}.mix.rel": (r, raw["layers"][i]["mixer"]["heads"]) for i, r in enumerate(rows)}
    c = DamadraConfig.from_dict(raw, shapes)
    assert [l.mixer["bias_rows"] for l in c.layers] == rows


@pytest.mark.parametrize("change, error", [
    (lambda c: c.pop("residual_mult"), MissingKey),
    (lambda c: c.pop("embedding"), MissingKey),
    (lambda c: c["layers"][0].update(type="attention_3"), InvalidValue),
    (lambda c: c["layers"][1]["mixer"].pop("mask"), MissingKey),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), InvalidValue),          # 6 heads over 4
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), InvalidValue),           # not an earlier layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), InvalidValue),           # another kind of layer
    (lambda c: c["layers"][2]["mixer"].update(vdim=16), InvalidValue),             # differs from its source
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), InvalidValue),
    (lambda c: c["layers"][1]["mixer"].update(bias_max=4), InvalidValue),          # no distance beyond the exact rows
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), InvalidValue),              # the values are the keys
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), InvalidValue),
])
def test_refusals(change, error):
    raw = copy.deepcopy(dt.TINY_A)
    change(raw)
    with pytest.raises(error):
        DamadraConfig.from_dict(raw)


def test_tensor_names_and_shapes():
    from reinfer_b200.models.damadra import build_spec
    from reinfer_b200.parts.model import expected_params
    exp = expected_params(build_spec(DamadraConfig.from_dict(dt.TINY_A)))
    assert tuple(exp["embed"].shape) == (211, 64) and tuple(exp["head"].shape) == (211, 64) and tuple(exp["final.norm"].shape) == (64,)
    assert tuple(exp["l0.mix.q"].shape) == (96, 64) and tuple(exp["l0.mix.k"].shape) == (48, 64) and tuple(exp["l0.mix.v"].shape) == (72, 64)
    assert tuple(exp["l0.mix.q.norm"].shape) == (16,) and tuple(exp["l0.mix.o"].shape) == (64, 144) and tuple(exp["l0.mix.rel"].shape) == (8, 6)
    # the windowed mixer: norms over the whole projection, no value matrix
    assert tuple(exp["l1.mix.q.norm"].shape) == (64,) and tuple(exp["l1.mix.k.norm"].shape) == (32,) and "l1.mix.v" not in exp
    # a layer that reads another's keys and values has none of their tensors
    assert not any(n in exp for n in ("l2.mix.k", "l2.mix.v", "l2.mix.k.norm")) and "l2.mix.q.norm" in exp
    assert tuple(exp["l1.mlp.router"].shape) == (7, 64) and tuple(exp["l1.mlp.correction"].shape) == (7,)
    assert "l1.mlp.e4.up" in exp and "l1.mlp.e5.up" not in exp and tuple(exp["l1.mlp.e0.down"].shape) == (64, 24)
    assert tuple(exp["l0.mlp.gate"].shape) == (72, 64) and tuple(exp["l0.norm1"].shape) == (64,) and "l0.norm2" in exp


def test_a_layer_without_feed_forward_ignores_its_second_norm():
    from reinfer_b200.models.damadra import build_spec
    spec = build_spec(DamadraConfig.from_dict(dt.TINY_B))
    assert "l1.norm2" in spec.ignorable_tensors
    assert spec.layers[3].cache_from == "l1" and spec.layers[0].cache_from is None


@pytest.mark.parametrize("rows, far", [(8, 30), (10, 30), (6, 25), (4, 9), (16, 50), (32, 300), (16, 128), (2, 5), (20, 300)])
def test_unrolled_bias_rows_are_the_bucket_function(rows, far):
    from reinfer_b200.parts.biased_attention import distance_rows
    got = distance_rows(rows, far)
    assert len(got) == far + 1
    assert got == [plain.distance_bucket(n, rows, far) for n in range(far + 1)]
    assert got[-1] == rows - 1 and all(plain.distance_bucket(n, rows, far) == rows - 1 for n in range(far, far + 500, 7))
    assert got[:rows // 2] == list(range(rows // 2)) and all(a <= b for a, b in zip(got, got[1:]))


def test_cache_groups_by_need():
    """Windowed layers of different windows and the causal layers each get pages of their own; a reading layer owns none."""
    from reinfer_b200.models.damadra import build_spec
    from reinfer_b200.parts.model import Model
    from reinfer_b200.cache.manager import group_layers
    m = Model(build_spec(DamadraConfig.from_dict(dt.TINY_A)))
    paged, states = m.cache_layout()
    assert set(paged) == {"l0", "l1", "l3"} and not states
    groups = group_layers(paged)
    assert sorted(g[0].window or 0 for g in groups) == [0, 11, 19]
    assert [b for b in m.cache_bindings() if b[0] == "l2"] == [("l2", "l0", False)]
    assert paged["l0"].value_dim == 24 and paged["l0"].head_dim == 16
