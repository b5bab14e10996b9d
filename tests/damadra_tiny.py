"""Small Damadra configurations for the tests - they differ from one another in every size and option - and
weights of the tests' own making: large enough that every mechanism moves the logits (distance biases of order
one, routers that decide clearly, norm weights around one)."""
from __future__ import annotations

import json
import math
import os
import random
from typing import Dict, List

import torch


def _win(heads, kv, dim, scale, window, far, rows):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
                                           "bias_max": far, "bias_rows": rows, "mask": {"size": window}}}


def _cau(heads, kv, dim, vdim, scale, far, rows, temp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far, "bias_rows": rows}
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, identity, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def _layer(mix, mlp):
    return dict(mix, mlp=mlp)


# A: value heads wider than the keys', a window that is no multiple of a page, warm-up every 5 positions, a layer
#    that reads an earlier layer's keys and values, identity experts, biases that reach beyond the window
TINY_A = {"architecture": "Damadra", "vocab": 211, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
          "residual_mult": 0.7,
          "layers": [_layer(_cau(6, 3, 16, 24, 0.3, 30, 8, temp=(0.4, 5)), _dense(72)),
                     _layer(_win(4, 2, 16, 0.25, 11, 30, 10), _moe(5, 2, 3, 24)),
                     _layer(_cau(6, 3, 16, 24, 0.3, 40, 12, temp=(0.2, 7), kv_from=0), _moe(3, 1, 2, 40)),
                     _layer(_win(2, 2, 24, 0.2, 19, 25, 6), _dense(48))]}
# B: nothing is a multiple of 8 (the aligned products and the tensor-core attention must find their plain forms by
#    themselves), key/value heads = query heads, a window of ONE position, no warm-up, no identity experts, top 1,
#    a layer without feed-forward, multiplier and embedding scale of 1
TINY_B = {"architecture": "Damadra", "vocab": 97, "width": 52, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
          "residual_mult": 1.0,
          "layers": [_layer(_win(3, 3, 12, 0.3, 1, 9, 4), _moe(3, 0, 1, 18)),
                     _layer(_cau(2, 2, 10, 6, 0.35, 21, 6), None),
                     _layer(_win(2, 1, 20, 0.22, 5, 50, 16), _dense(36)),
                     _layer(_cau(2, 2, 10, 6, 0.35, 33, 14, kv_from=1), _moe(2, 0, 2, 10))]}
# C: one key/value head for all eight query heads, keys wider than the values, a window of whole pages, warm-up at
#    every position, every expert chosen every time (top = all), two layers reading the same earlier layer, a bias
#    table that reaches beyond every request
TINY_C = {"architecture": "Damadra", "vocab": 130, "width": 96, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-6},
          "residual_mult": 0.4,
          "layers": [_layer(_win(4, 1, 32, 0.18, 16, 300, 32), _dense(128)),
                     _layer(_cau(8, 1, 32, 16, 0.2, 300, 20, temp=(0.6, 1)), _moe(2, 2, 4, 32)),
                     _layer(_cau(8, 1, 32, 16, 0.2, 120, 8, temp=(0.1, 64), kv_from=1), _dense(64)),
                     _layer(_cau(8, 1, 32, 16, 0.15, 90, 16, kv_from=1), _moe(6, 3, 2, 16))]}
# D: heads of 128 and 64 at a width of 256 with pages of 64: what a small real model looks like (not in TINY: its
#    tests name it)
TINY_D = {"architecture": "Damadra", "vocab": 500, "width": 256, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
          "residual_mult": 0.5,
          "layers": [_layer(_cau(4, 2, 128, 128, 0.09, 200, 32, temp=(0.3, 32)), _moe(4, 2, 2, 128)),
                     _layer(_win(4, 4, 64, 0.12, 100, 150, 16), _dense(512)),
                     _layer(_cau(4, 2, 128, 128, 0.09, 200, 32, temp=(0.3, 32), kv_from=0), _dense(384))]}
TINY = {"A": (TINY_A, 31, 8), "B": (TINY_B, 32, 4), "C": (TINY_C, 33, 16)}      # config, weight seed, page size


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """float32 tensors for every name the model declares, drawn by the tensor's role (read off its name)."""
    from reinfer_b200.config.damadra import DamadraConfig
    from reinfer_b200.models.damadra import build_spec
    from reinfer_b200.parts.model import expected_params
    expected = expected_params(build_spec(DamadraConfig.from_dict(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, ps in expected.items():
        shape = tuple(ps.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        last = name.split(".")[-1]
        if name == "embed":
            t = n(0.8)
        elif last == "rel":
            t = n(1.0)
        elif last == "router":
            t = n(3.0 / math.sqrt(shape[1]))
        elif last == "correction":
            t = n(0.15)
        elif len(shape) == 1:
            t = n(0.1, 1.0)                 # norm weights
        else:
            t = n(1.4 / math.sqrt(shape[1]))
        out[name] = t.float()
    return out


def make_model_dir(path: str, which: str, store_dtype=torch.float32, cfg=None, seed=None) -> str:
    from reinfer_b200.weights.safetensors_io import write_safetensors
    base, s, _ = TINY[which] if which in TINY else (cfg, seed, None)
    cfg = cfg or base
    seed = s if seed is None else seed
    os.makedirs(path, exist_ok=True)
    raw = json.loads(json.dumps(cfg))
    for l in raw["layers"]:                 # a checkpoint's config.json leaves the bias tables' rows to the tensors' shapes
        l["mixer"].pop("bias_rows", None)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.to(store_dtype) for k, v in make_weights(cfg, seed).items()})
    return path


def sequences(which: str, lengths=None, seed=7) -> Dict[str, List[int]]:
    cfg = TINY[which][0]
    rnd = random.Random(seed)
    lengths = lengths or {"A": [5, 17, 33, 70, 40, 26, 51], "B": [1, 9, 24, 50, 90, 37, 64, 12], "C": [3, 44, 21, 60, 30]}[which]
    return {f"r{i}": [rnd.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: three to six layers in any order, head counts, head sizes (also ones the
    tensor-core kernels pad or refuse), windows from one position to beyond the requests, bias tables of few and many
    rows, readers of earlier layers, dense and mixture feed-forwards or none."""
    rnd = random.Random(seed)
    width = rnd.choice([48, 64, 128, 192])
    layers, own = [], {}
    for i in range(rnd.randint(3, 6)):
        kind = rnd.choice(["attention", "attention_2", "attention_2"])
        kv = rnd.choice([1, 2, 4])
        heads = kv * rnd.choice([1, 2, 3])
        dim = rnd.choice([8, 12, 16, 32, 48, 64, 128])
        rows = rnd.choice([4, 8, 16, 32])
        far = max(rnd.choice([5, 20, 100, 128, 400]), rows // 2 + 1)
        if kind == "attention":
            layer = _win(heads, kv, dim, rnd.choice([dim ** -0.5, 0.2]), rnd.choice([1, 7, 16, 40, 100, 500]), far, rows)
        else:
            vdim = rnd.choice([8, 16, 20, 64, 128, dim])
            temp = (rnd.choice([0.1, 0.5]), rnd.choice([1, 16, 64])) if rnd.random() < 0.7 else None
            sig = (heads, kv, dim, vdim)
            src = own.get(sig) if rnd.random() < 0.5 else None
            if src is None and own and rnd.random() < 0.4:
                sig = rnd.choice(sorted(own))
                heads, kv, dim, vdim = sig
                src = own[sig]
            layer = _cau(heads, kv, dim, vdim, rnd.choice([dim ** -0.5, 0.15]), far, rows, temp=temp, kv_from=src)
            if src is None:
                own.setdefault(sig, i)
        r = rnd.random()
        if r < 0.15:
            mlp = None
        elif r < 0.5:
            mlp = _dense(rnd.choice([40, 64, 96]))
        else:
            e, idn = rnd.choice([2, 3, 8]), rnd.choice([0, 1, 3])
            mlp = _moe(e, idn, rnd.randint(1, min(4, e + idn)), rnd.choice([12, 32, 64]))
        layers.append(_layer(layer, mlp))
    return {"architecture": "Damadra", "vocab": rnd.choice([97, 300, 500]), "width": width,
            "embedding": {"scale": rnd.choice([1.0, 2.5, 12.0])}, "norm": {"eps": rnd.choice([1e-5, 1e-6])},
            "residual_mult": rnd.choice([0.3, 0.6, 1.0]), "layers": layers}
