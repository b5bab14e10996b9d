"""Host-side pieces of the Silutar architecture: the configuration (sizes from config.json, inner
widths from tensor shapes), the model description's tensor names, the states and pages it asks of
the cache manager, and the release of pages behind a chunk."""
from __future__ import annotations

import json
import os

import pytest
import torch

import silutar_tiny as st


def test_inner_widths_come_from_tensor_shapes_when_the_file_leaves_them_out(tmp_path):
    from reinfer_b200.config import load_config
    from reinfer_b200.config.silutar import SilutarConfig
    d = st.make_model_dir(str(tmp_path / "m"), "A", torch.bfloat16)
    raw = json.load(open(os.path.join(d, "config.json")))
    assert "decay_rank" not in json.dumps(raw)
    arch, cfg = load_config(d)
    assert arch.name == "Silutar" and isinstance(cfg, SilutarConfig)
    assert cfg.layers[0].mixer["right"]["decay_rank"] == 8 and cfg.layers[1].mixer["decay_rank"] == 8
    assert cfg.layers[2].mixer["decay_rank"] == 8 and cfg.layers[2].mixer["gate_rank"] == 16
    assert cfg.layers[1].ff is None and cfg.layers[0].ff == 96
    again = SilutarConfig.from_dict(cfg.to_dict())              # a written configuration states them itself
    assert again == cfg


def test_bad_configurations_are_refused():
    from reinfer_b200.config import InvalidValue, MissingKey
    from reinfer_b200.config.silutar import SilutarConfig
    good = json.loads(json.dumps(st.TINY_A))
    SilutarConfig.from_dict(good)
    for path, value, err in ((("layers", 0, "type"), "conv", InvalidValue), (("layers", 1, "mlp"), {"kind": "routed", "ff": 8}, InvalidValue),
                             (("layers", 2, "mixer", "kv_heads"), 3, InvalidValue), (("norm",), None, MissingKey),
                             (("layers", 1, "mixer", "tau"), 0.0, InvalidValue), (("layers", 0, "mixer", "left", "mask"), None, MissingKey)):
        bad = json.loads(json.dumps(good))
        node = bad
        for p in path[:-1]:
            node = node[p]
        node[path[-1]] = value
        with pytest.raises(err):
            SilutarConfig.from_dict(bad)
    bad = json.loads(json.dumps(good))
    del bad["layers"][1]["mixer"]["decay_rank"]                 # neither stated nor readable from a shape
    with pytest.raises(MissingKey):
        SilutarConfig.from_dict(bad)


def test_tensor_names_states_and_pages_of_the_description():
    from reinfer_b200.config.silutar import SilutarConfig
    from reinfer_b200.models.silutar import build_spec
    from reinfer_b200.parts.base import PagedKVSpec
    from reinfer_b200.parts.model import Model
    m = Model(build_spec(SilutarConfig.from_dict(st.TINY_A)))
    names = m.param_specs()
    for n, shape in (("embed", (211, 64)), ("pos", (400, 64)), ("l0.norm1", (64,)), ("l0.norm1.b", (64,)), ("l0.norm1.alpha", ()),
                     ("l0.mix.left.q", (64, 64)), ("l0.mix.left.v", (48, 64)), ("l0.mix.left.q.conv", (64, 4)), ("l0.mix.left.r1", (4,)),
                     ("l0.mix.left.o", (64, 96)), ("l0.mix.right.w1", (8, 64)), ("l0.mix.right.a.b", (32,)), ("l0.mix.right.norm", (32,)),
                     ("l1.mix.a2.b", (32,)), ("l1.mix.norm", (24,)), ("l2.mix.b", (4, 64)), ("l2.mix.q", (32, 64)), ("l2.mix.v", (32, 64)),
                     ("l2.mix.g2", (32, 16)), ("l2.mix.A_log", (4,)), ("l2.mlp.down", (64, 80)), ("final.norm.alpha", ())):
        assert tuple(names[n].shape) == shape, n
    assert "l1.norm2" not in names and "l1.mlp.gate" not in names         # the layer without a feed-forward
    paged, states = m.cache_layout()
    assert paged == {"l0": PagedKVSpec(2, 16, None, 24, 24)}
    assert set(states) == {"l0", "l1", "l2"}
    assert tuple(states["l0"]["left"]["conv"].shape) == (3, 64 + 32 + 48) and tuple(states["l0"]["right"].shape) == (2, 16, 16)
    assert tuple(states["l1"].shape) == (2, 16, 24)
    assert tuple(states["l2"]["S"].shape) == (4, 16, 8) and tuple(states["l2"]["conv"].shape) == (1, 96)


def test_pages_behind_a_chunk_go_back_to_the_pool():
    from reinfer_b200.cache import CacheManager
    from reinfer_b200.parts.base import PagedKVSpec
    cm = CacheManager({"a": PagedKVSpec(1, 8, None, None, 24)}, {}, page_size=8, num_pages=6, max_seqs=2)
    cm.admit("x")
    held = lambda: [p for p in cm.table("x", 0) if p >= 0]
    for new_len in (5, 23, 24, 25, 40, 47, 48, 70, 85, 100):
        # after `new_len` tokens the next token is at position new_len: it reads keys from its chunk's start on
        if cm.pages_needed("x", new_len) > cm.free_pages():
            pytest.fail("the pool of six pages must do")
        cm.reserve("x", new_len)
        cm.commit("x", new_len)
        first = (new_len // 24 * 24) // 8
        assert len(held()) == -(-new_len // 8) - first, new_len
        cm.check()
    cm.release("x")
    assert cm.free_pages() == 6


def test_scalar_tensors_pass_through_the_file_format(tmp_path):
    from reinfer_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    p = str(tmp_path / "s.safetensors")
    write_safetensors(p, {"alpha": torch.tensor(0.75, dtype=torch.bfloat16), "v": torch.arange(3, dtype=torch.float32)})
    f = SafetensorsFile(p)
    assert f.shape("alpha") == () and float(f.tensor("alpha")) == 0.75
