"""Small Silutar configurations for the tests - they differ from one another in every size and
option - and weights of the tests' own making: large enough that every mechanism moves the logits
(a statistics-free norm does not rescale small activations), decays spread between fast and slow."""
from __future__ import annotations

import json
import math
import os
import random
from typing import Dict, List

import torch


def _gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}}


def _cd(heads, kv, dim, vdim, conv, ra, rg):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": ra, "gate_rank": rg}}


def _par(heads, kv, dim, vdim, conv, chunk, scale, rheads, rdim, rrank, ls, rs):
    return {"type": "parallel", "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                                                    "mask": {"size": chunk}, "scale": scale},
                                          "right": {"heads": rheads, "dim": rdim, "decay_rank": rrank},
                                          "left_scale": ls, "right_scale": rs}}


def _layer(mix, ff):
    return dict(mix, mlp=None if ff is None else {"kind": "dense", "ff": ff})


# A: value heads of another size than the keys', a chunk that is no multiple of a page, four taps, a layer without
#    feed-forward, grouped key heads in the delta rule, a soft cap
TINY_A = {"architecture": "Silutar", "vocab": 211, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
          "logit_softcap": 12.0,
          "layers": [_layer(_par(4, 2, 16, 24, 4, 24, 0.3, 2, 16, 8, 0.7, 1.1), 96),
                     _layer(_gla(2, 16, 24, 8.0, 8), None),
                     _layer(_cd(4, 2, 16, 8, 2, 8, 16), 80)]}
# B: one tap (no convolution state), key/value heads = query heads, chunk = page, key size that fills no register
#    slice (40), scales of 1, no soft cap, the same mixer twice
TINY_B = {"architecture": "Silutar", "vocab": 97, "width": 48, "max_positions": 300, "norm": {"eps": 1e-6},
          "layers": [_layer(_cd(3, 3, 40, 24, 1, 16, 8), 64),
                     _layer(_par(2, 2, 8, 8, 1, 16, 0.5, 3, 24, 16, 1.0, 1.0), 64),
                     _layer(_gla(3, 40, 8, 2.0, 16), 64),
                     _layer(_gla(1, 8, 72, 32.0, 8), None)]}
# C: wide heads (every register-slice size of the recurrence kernel), one key/value head for all query heads,
#    a chunk of a few positions, five taps
TINY_C = {"architecture": "Silutar", "vocab": 130, "width": 96, "max_positions": 256, "norm": {"eps": 1e-6},
          "logit_softcap": 30.0,
          "layers": [_layer(_gla(2, 72, 40, 16.0, 8), 128),
                     _layer(_cd(2, 1, 136, 32, 5, 8, 8), None),
                     _layer(_par(4, 1, 32, 16, 5, 5, 0.2, 1, 136, 8, 0.5, 2.0), 128)]}
# D: nothing is a multiple of 8 - width, feed-forward, vocabulary, head sizes, inner widths: the products and the
#    attention that want aligned operands must find their plain forms by themselves
TINY_D = {"architecture": "Silutar", "vocab": 77, "width": 52, "max_positions": 200, "norm": {"eps": 1e-5},
          "logit_softcap": 25.0,
          "layers": [_layer(_par(3, 3, 12, 12, 3, 7, 0.25, 2, 6, 5, 0.9, 0.4), 36),
                     _layer(_gla(2, 6, 10, 4.0, 5), 50),
                     _layer(_cd(2, 2, 10, 6, 3, 3, 7), 36)]}
# E: a width in tiles of 128, attention heads of 128 and a chunk of one key tile: the sizes at which a decode step's
#    products do the next norm's work and the chunk attention runs on the tensor cores - prompt portions on the
#    tcgen05 kernel, single tokens on the flash-decoding kernel (not in TINY: its tests name it)
TINY_E = {"architecture": "Silutar", "vocab": 300, "width": 128, "max_positions": 256, "norm": {"eps": 1e-6},
          "logit_softcap": 30.0,
          "layers": [_layer(_par(2, 1, 128, 128, 3, 64, 0.09, 2, 32, 8, 0.6, 0.9), 256),
                     _layer(_cd(2, 1, 32, 64, 4, 8, 8), 256),
                     _layer(_gla(2, 32, 64, 8.0, 8), 256)]}
# F: two attention layers with different needs (two cache groups, each with block tables and a chunk of its own: 16
#    positions = one page, and 40 positions over pages of 16), every mixer twice or in another order
TINY_F = {"architecture": "Silutar", "vocab": 150, "width": 64, "max_positions": 300, "norm": {"eps": 1e-6},
          "logit_softcap": 20.0,
          "layers": [_layer(_gla(2, 16, 16, 4.0, 8), 96),
                     _layer(_par(4, 1, 16, 16, 2, 16, 0.25, 2, 16, 8, 1.2, 0.3), None),
                     _layer(_cd(2, 2, 16, 16, 3, 8, 8), 96),
                     _layer(_par(2, 2, 8, 24, 4, 40, 0.35, 4, 8, 8, 0.5, 0.5), 96)]}
# G: no attention at all: the model owns no pages, only states in the request slots
TINY_G = {"architecture": "Silutar", "vocab": 120, "width": 48, "max_positions": 300, "norm": {"eps": 1e-6},
          "layers": [_layer(_cd(2, 1, 24, 16, 2, 8, 8), 64),
                     _layer(_gla(3, 8, 16, 6.0, 8), 64)]}
# H: a width of 256 with attention heads of 128 and recurrence heads of 64: what a small real model looks like, and where
#    every tensor-core and fused form applies at once (not in TINY: its test names it)
TINY_H = {"architecture": "Silutar", "vocab": 500, "width": 256, "max_positions": 512, "norm": {"eps": 1e-6},
          "logit_softcap": 30.0,
          "layers": [_layer(_par(4, 2, 128, 128, 3, 128, 0.09, 4, 64, 16, 0.6, 0.9), 512),
                     _layer(_cd(4, 2, 64, 128, 4, 16, 16), 512),
                     _layer(_gla(4, 64, 64, 16.0, 16), 512)]}
TINY = {"A": (TINY_A, 11, 16), "B": (TINY_B, 12, 16), "C": (TINY_C, 13, 8), "D": (TINY_D, 14, 4), "F": (TINY_F, 16, 16),
        "G": (TINY_G, 17, 16)}      # config, weight seed, page size


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """float32 tensors for every name the model declares, drawn by the tensor's role (read off its name)."""
    from reinfer_b200.config.silutar import SilutarConfig
    from reinfer_b200.models.silutar import build_spec
    from reinfer_b200.parts.model import expected_params
    expected = expected_params(build_spec(SilutarConfig.from_dict(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, ps in expected.items():
        shape = tuple(ps.shape)
        n = lambda std=1.0, mean=0.0: torch.randn(shape, generator=g) * std + mean
        u = lambda lo, hi: torch.rand(shape, generator=g) * (hi - lo) + lo
        last = name.split(".")[-1]
        if name in ("embed", "pos"):
            t = n(0.8)
        elif last == "alpha":
            t = u(0.4, 0.9)
        elif last == "conv":
            t = n(0.6)
        elif last in ("r1", "r2"):
            t = u(0.2, 1.5)
        elif last == "A_log":
            t = n(0.7, -1.0)
        elif name.endswith("a2.b"):
            t = n(1.5, 2.0)                 # decays between fast and very slow
        elif last in ("dt_bias", "w0"):
            t = n(1.5, -1.0)
        elif name.endswith(".b") and len(shape) == 1 and ("norm" in name):
            t = n(0.1)                      # a Dynamic Tanh bias
        elif last == "b" and len(shape) == 1:
            t = n(1.0)                      # the removal rate's bias
        elif len(shape) == 1:
            t = n(0.1, 1.0)                 # norm weights
        elif len(shape) == 2:
            t = n(1.4 / math.sqrt(shape[1]))
        else:
            t = n(1.0)
        out[name] = t.float()
    return out


def make_model_dir(path: str, which: str, store_dtype=torch.float32, cfg=None, seed=None) -> str:
    from reinfer_b200.weights.safetensors_io import write_safetensors
    base, s, _ = TINY[which] if which in TINY else (cfg, seed, None)
    cfg = cfg or base
    seed = s if seed is None else seed
    os.makedirs(path, exist_ok=True)
    raw = json.loads(json.dumps(cfg))
    for l in raw["layers"]:                 # a checkpoint's config.json leaves the inner widths to the tensors' shapes
        for m in (l["mixer"], l["mixer"].get("right", {})):
            m.pop("decay_rank", None)
            m.pop("gate_rank", None)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.to(store_dtype) for k, v in make_weights(cfg, seed).items()})
    return path


def sequences(which: str, lengths=None, seed=7) -> Dict[str, List[int]]:
    cfg = TINY[which][0]
    rnd = random.Random(seed)
    lengths = lengths or {"A": [5, 17, 33, 70, 40, 26, 51], "B": [1, 9, 24, 50, 90, 37, 64, 12], "C": [3, 44, 21, 60, 30],
                          "D": [2, 31, 18, 45, 9], "F": [4, 50, 23, 81, 36], "G": [6, 40, 17, 29]}[which]
    return {f"r{i}": [rnd.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}
